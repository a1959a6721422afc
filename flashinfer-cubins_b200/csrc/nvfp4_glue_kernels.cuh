// The two small kernels around the NVFP4 dual GEMM: the scale relayout into the
// blocked 128x4 layout and the silu gate over FP32 intermediates. Both are plain
// bandwidth kernels: 16-byte accesses, grid-stride loops.
#pragma once

#include <cstdint>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace nvfp4 {

// scales: [batches][rows][cols] bytes. packed: [batches][rb][cb][32][4][4] bytes with
// rb = ceil(rows/128), cb = ceil(cols/4); scale (r, c) goes to
// [r/128][c/4][r%32][(r/32)%4][c%4]; padding is zero. One thread writes one 16-byte
// line (fixed r%32 of one atom): four source rows x four source columns.
__global__ void pack_scales_kernel(const uint8_t* __restrict__ scales,
                                   uint8_t* __restrict__ packed, int rows, int cols,
                                   int batches) {
  const int rb = (rows + 127) / 128;
  const int cb = (cols + 3) / 4;
  const long long lines = static_cast<long long>(batches) * rb * cb * 32;
  const bool fast_cols = (cols % 4 == 0) && (reinterpret_cast<uintptr_t>(scales) % 4 == 0);
  for (long long line = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
       line < lines; line += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r32 = static_cast<int>(line % 32);
    long long rest = line / 32;
    const int c_blk = static_cast<int>(rest % cb);
    rest /= cb;
    const int r_blk = static_cast<int>(rest % rb);
    const int batch = static_cast<int>(rest / rb);
    const uint8_t* src = scales + static_cast<long long>(batch) * rows * cols;
    uint32_t words[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int r = r_blk * 128 + q * 32 + r32;
      uint32_t w = 0;
      if (r < rows) {
        const uint8_t* row_ptr = src + static_cast<long long>(r) * cols + c_blk * 4;
        if (fast_cols) {
          w = *reinterpret_cast<const uint32_t*>(row_ptr);
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (c_blk * 4 + c < cols) w |= static_cast<uint32_t>(row_ptr[c]) << (8 * c);
          }
        }
      }
      words[q] = w;
    }
    *reinterpret_cast<uint4*>(packed + line * 16) =
        make_uint4(words[0], words[1], words[2], words[3]);
  }
}

__device__ __forceinline__ float silu_gate(float a, float b) {
  return a / (1.0f + expf(-a)) * b;
}

// out[i] = half(silu(h1[i]) * h2[i]); eight elements per thread when the arrays are
// 16-byte aligned, scalar tail otherwise.
__global__ void silu_product_kernel(const float* __restrict__ h1, const float* __restrict__ h2,
                                    __half* __restrict__ out, long long size, int vector_ok) {
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long groups = vector_ok ? size / 8 : 0;
  for (long long g = tid; g < groups; g += nthreads) {
    const float4 a0 = reinterpret_cast<const float4*>(h1)[2 * g];
    const float4 a1 = reinterpret_cast<const float4*>(h1)[2 * g + 1];
    const float4 b0 = reinterpret_cast<const float4*>(h2)[2 * g];
    const float4 b1 = reinterpret_cast<const float4*>(h2)[2 * g + 1];
    __half2 r0 = __floats2half2_rn(silu_gate(a0.x, b0.x), silu_gate(a0.y, b0.y));
    __half2 r1 = __floats2half2_rn(silu_gate(a0.z, b0.z), silu_gate(a0.w, b0.w));
    __half2 r2 = __floats2half2_rn(silu_gate(a1.x, b1.x), silu_gate(a1.y, b1.y));
    __half2 r3 = __floats2half2_rn(silu_gate(a1.z, b1.z), silu_gate(a1.w, b1.w));
    uint4 q;
    q.x = *reinterpret_cast<uint32_t*>(&r0);
    q.y = *reinterpret_cast<uint32_t*>(&r1);
    q.z = *reinterpret_cast<uint32_t*>(&r2);
    q.w = *reinterpret_cast<uint32_t*>(&r3);
    reinterpret_cast<uint4*>(out)[g] = q;
  }
  for (long long i = groups * 8 + tid; i < size; i += nthreads) {
    out[i] = __float2half_rn(silu_gate(h1[i], h2[i]));
  }
}

}  // namespace nvfp4
