// The small bandwidth kernels around the NVFP4 GEMMs: the scale relayout into the blocked
// 128x4 layout, the FP32/BF16 -> NVFP4 quantiser that writes blocked scales directly, and the
// silu gate over FP32 intermediates. 16-byte accesses, grid-stride loops.
#pragma once

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "sm100_ptx.cuh"

namespace nvfp4 {

// A few KB of host data delivered to device memory *as a kernel parameter*: the runtime
// copies parameters when the launch is enqueued, so the host buffer they came from may be
// freed or reused as soon as the launch call returns, on every system (an asynchronous copy
// from pageable host memory has no such guarantee where the GPU can read pageable memory
// directly), and the launch can be captured in a graph. `bytes` is a multiple of 16.
struct alignas(16) ParamBlob {
  static constexpr int kBytes = 3584;
  uint8_t data[kBytes];
};

__global__ void write_blob_kernel(uint8_t* __restrict__ dst, const __grid_constant__ ParamBlob blob,
                                  int bytes) {
  const uint4* src = reinterpret_cast<const uint4*>(blob.data);
  uint4* out = reinterpret_cast<uint4*>(dst);
  for (int i = threadIdx.x; i < bytes / 16; i += blockDim.x) out[i] = src[i];
}

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

// UE4M3 bits of the scale of a 16-element block with the given absolute maximum:
// amax / 6 rounded to nearest even, saturating at 448.
__device__ __forceinline__ uint32_t nvfp4_scale_bits(float amax) {
  // amax / 6 correctly rounded without the division: q = amax y with y = RN(1/6), then
  // q + (amax - 6 q) y (see quantize_nvfp4_kernel). Infinity: the residual would be NaN, and
  // the result saturates anyway.
  constexpr float kSixth = 1.0f / 6.0f;
  const float q = amax * kSixth;
  const float sixth = amax <= 3.0e38f ? __fmaf_rn(__fmaf_rn(-6.0f, q, amax), kSixth, q) : amax;
  return static_cast<uint32_t>(
      __nv_cvt_float_to_fp8(fminf(sixth, 448.0f), __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ float nvfp4_scale_value(uint32_t bits) {
  return __half2float(
      __half(__nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(bits), __NV_E4M3)));
}

// The sixteen E2M1 codes of a block with absolute maximum `amax` and scale `scale` > 0
// (x = low word: elements 0-7, y = elements 8-15; element i in nibble i % 8): the correctly
// rounded quotient x / scale goes through the hardware conversion (round to nearest even,
// saturating at +-6). (A bare reciprocal multiply would break exact ties such as
// x / scale == 0.75.) With finite inputs the quotient comes from the correctly rounded
// reciprocal and two fused multiply-adds, q = x y, q' = q + (x - scale q) y, which is the
// correctly rounded quotient whenever the divisor's significand is not all ones (a scale has
// four significant bits): three instructions (packed, for two quotients at a time) in place
// of an IEEE division. Blocks with an infinity take the division itself. A negative value that rounds to zero gets code 0, not -0.
// Used by the quantiser kernel and by the GEMM epilogues that write NVFP4, so that both produce
// the same bytes from the same FP32 values.
__device__ __forceinline__ uint2 nvfp4_block_codes(const float (&v)[16], float amax, float scale) {
  float2 quotient[8];
  if (amax <= 3.0e38f) {
    // Two quotients per instruction (packed FP32 multiply and fused multiply-add).
    const float y = __frcp_rn(scale);
    const float2 y2 = make_float2(y, y);
    const float2 minus_scale = make_float2(-scale, -scale);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float2 x = make_float2(v[2 * j], v[2 * j + 1]);
      const float2 q = __fmul2_rn(x, y2);
      quotient[j] = __ffma2_rn(__ffma2_rn(minus_scale, q, x), y2, q);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      quotient[j] = make_float2(__fdiv_rn(v[2 * j], scale), __fdiv_rn(v[2 * j + 1], scale));
    }
  }
  uint32_t words[2] = {0u, 0u};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t pair = __nv_cvt_float2_to_fp4x2(quotient[j], __NV_E2M1, cudaRoundNearest);
    words[j / 4] |= pair << (8 * (j % 4));
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    // A nibble's magnitude m is 0..7: m + 7 sets bit 3 exactly when m is not zero, without a
    // carry into the next nibble.
    const uint32_t magnitude = words[h] & 0x77777777u;
    const uint32_t nonzero = (magnitude + 0x77777777u) & 0x88888888u;
    words[h] = magnitude | (words[h] & nonzero);
  }
  return make_uint2(words[0], words[1]);
}

// FP32/BF16 [batches][rows][k] -> packed E2M1 [batches][rows][k/2] and UE4M3 scales in the
// blocked layout [batches][rb][cb][32][4][4] (zero padded): scale = e4m3(amax / 6) (round to
// nearest even, saturating), element = E2M1 rounding of x / scale, zero scale -> zero codes.
//
// One thread per 16-element block of the padded scale grid and four rows, placed by the
// launch geometry instead of by divisions: a CTA is 64 blocks of sixteen rows (threadIdx.x the
// block, threadIdx.y + 4 i the row for i = 0..3), blockIdx.x the group of sixteen rows,
// blockIdx.y the group of 64 blocks, blockIdx.z the batch. A thread issues the loads of its
// four rows before it works on the first, so that enough bytes are in flight. A warp is 32
// consecutive blocks of one row: it reads 1 KB (BF16) or 2 KB (FP32) and writes 256 B of
// codes in a row, and the scale bytes of four neighbouring blocks, which are neighbours in
// the blocked layout too, leave as one 32-bit word.
constexpr int kQuantBlocksX = 64;
constexpr int kQuantRowsY = 4;
constexpr int kQuantRowsPerThread = 4;
constexpr int kQuantRowsPerCta = kQuantRowsY * kQuantRowsPerThread;

// MODE 0: every row of x[batches][rows][k]. MODE 1 (one batch): rows come in 128-row blocks of
// which only the first info[b] rows hold data. MODE 2 (one batch): output row r is input row
// info[r] of x, or nothing if info[r] < 0 (a gather: the permuted rows of a mixture-of-experts
// layer straight from the token activations). In modes 1 and 2 the rows without data are
// neither read nor written: their codes and scales keep what the buffers held.
constexpr int kQuantDense = 0, kQuantBlocks = 1, kQuantGather = 2;

template <typename In, int MODE>
__global__ void __launch_bounds__(kQuantBlocksX* kQuantRowsY)
quantize_nvfp4_kernel(const In* __restrict__ x, uint8_t* __restrict__ packed,
                      uint8_t* __restrict__ scales, int rows, int k, int batches,
                      const int* __restrict__ info) {
  constexpr int kVectors = sizeof(In) == 4 ? 4 : 2;  // 16-byte loads per block
  const int cols = k / 16;
  const int rb = (rows + 127) / 128;
  const int cb = (cols + 3) / 4;
  const int c = blockIdx.y * kQuantBlocksX + threadIdx.x;
  const int r0 = blockIdx.x * kQuantRowsPerCta + threadIdx.y;
  int live_rows = rows;
  if constexpr (MODE == kQuantBlocks) {
    // A CTA's sixteen rows lie in one block.
    live_rows = min(rows, (r0 / 128) * 128 + __ldg(info + r0 / 128));
    if (static_cast<int>(blockIdx.x) * kQuantRowsPerCta >= live_rows) return;
  }
  // The input row of each of this thread's rows, or -1.
  int source[kQuantRowsPerThread];
#pragma unroll
  for (int i = 0; i < kQuantRowsPerThread; ++i) {
    const int r = r0 + kQuantRowsY * i;
    if constexpr (MODE == kQuantGather) {
      source[i] = r < rows ? __ldg(info + r) : -1;
    } else {
      source[i] = r < live_rows ? r : -1;
    }
  }
  for (int batch = blockIdx.z; batch < batches; batch += gridDim.z) {
    uint4 raw[kQuantRowsPerThread][kVectors];
#pragma unroll
    for (int i = 0; i < kQuantRowsPerThread; ++i) {
      if (source[i] >= 0 && c < cols) {
        const long long element =
            (static_cast<long long>(batch) * rows + source[i]) * k + c * 16;
        const uint4* src = reinterpret_cast<const uint4*>(x + element);
#pragma unroll
        for (int q = 0; q < kVectors; ++q) raw[i][q] = src[q];
      }
    }
#pragma unroll
    for (int i = 0; i < kQuantRowsPerThread; ++i) {
      const int r = r0 + kQuantRowsY * i;
      uint32_t scale_bits = 0;
      if (source[i] >= 0 && c < cols) {
        const long long element = (static_cast<long long>(batch) * rows + r) * k + c * 16;
        float v[16];
#pragma unroll
        for (int q = 0; q < kVectors; ++q) {
          const uint32_t w[4] = {raw[i][q].x, raw[i][q].y, raw[i][q].z, raw[i][q].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if constexpr (sizeof(In) == 4) {
              v[4 * q + j] = __uint_as_float(w[j]);
            } else {
              v[8 * q + 2 * j] = __uint_as_float(w[j] << 16);
              v[8 * q + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
            }
          }
        }
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
        scale_bits = nvfp4_scale_bits(amax);
        const float scale = nvfp4_scale_value(scale_bits);
        const uint2 codes = scale > 0.0f ? nvfp4_block_codes(v, amax, scale) : make_uint2(0u, 0u);
        *reinterpret_cast<uint2*>(packed + element / 2) = codes;
      }
      // Scale bytes of blocks c..c+3 (c a multiple of four) of row r are one aligned word of
      // the atom; in mode 0 padding rows and columns of the grid get zeros.
      uint32_t word = scale_bits << (8 * (threadIdx.x & 3));
      word |= __shfl_xor_sync(0xFFFFFFFFu, word, 1);
      word |= __shfl_xor_sync(0xFFFFFFFFu, word, 2);
      if ((threadIdx.x & 3) == 0 && c < cb * 4 && (MODE == kQuantDense || source[i] >= 0)) {
        const long long atom = (static_cast<long long>(batch) * rb + r / 128) * cb + c / 4;
        *reinterpret_cast<uint32_t*>(scales + atom * 512 + (r % 32) * 16 + ((r / 32) % 4) * 4) =
            word;
      }
    }
  }
}

// Routing of a mixture-of-experts layer, in two launches around the one host read that the
// grouped plans need (the row count per expert):
//   moe_count_kernel: counts[e] = number of (token, choice) pairs whose expert is e;
//   moe_place_kernel: every pair gets a row in its expert's block (first row starts[e], the
//     host's prefix over the counts padded to whole 128-row blocks) - row_of_pair[i] for the
//     combine, token_of_row[row] = i / choices for the gathering quantiser. Rows inside a
//     block are handed out by an atomic counter: which pair gets which row differs from run
//     to run, the result of the layer does not (every row is computed on its own).
// Ids outside [0, experts) get no row (row_of_pair = -1).
constexpr int kMoeMaxExperts = 512;

struct MoeStarts {
  int first_row[kMoeMaxExperts];
};

template <typename Id>
__global__ void moe_count_kernel(const Id* __restrict__ ids, long long pairs, int experts,
                                 int* __restrict__ counts) {
  __shared__ int local[kMoeMaxExperts];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) local[e] = 0;
  __syncthreads();
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < pairs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = static_cast<long long>(ids[i]);
    if (e >= 0 && e < experts) atomicAdd(&local[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    if (local[e] != 0) atomicAdd(&counts[e], local[e]);
  }
}

template <typename Id>
__global__ void moe_place_kernel(const Id* __restrict__ ids, long long pairs, int choices,
                                 int experts, const __grid_constant__ MoeStarts starts,
                                 const int* __restrict__ device_starts,
                                 int* __restrict__ cursors, int* __restrict__ row_of_pair,
                                 int* __restrict__ token_of_row) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < pairs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = static_cast<long long>(ids[i]);
    int row = -1;
    if (e >= 0 && e < experts) {
      // The blocks' first rows come from the host (a kernel parameter) or, when the layout
      // was made on the device, from device memory.
      const int first = device_starts != nullptr ? __ldg(device_starts + e) : starts.first_row[e];
      row = first + atomicAdd(&cursors[e], 1);
      token_of_row[row] = static_cast<int>(i / choices);
    }
    row_of_pair[i] = row;
  }
}

// The combine of a mixture-of-experts layer: out[t][:] = sum_j weights[t][j] * y[row(t, j)][:]
// in FP32, y FP16 rows picked by row_of_pair[t * choices + j] (a negative row contributes
// nothing). One thread per token and eight columns: `choices` 16-byte loads, two 16-byte
// stores; every row of y is read once.
__global__ void moe_combine_kernel(const __half* __restrict__ y, const int* __restrict__ row_of_pair,
                                   const float* __restrict__ weights, float* __restrict__ out,
                                   int tokens, int choices, int hidden) {
  const int chunks = hidden / 8;
  const long long total = static_cast<long long>(tokens) * chunks;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / chunks);
    const int c = static_cast<int>(i % chunks);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < choices; ++j) {
      const int row = __ldg(row_of_pair + static_cast<long long>(t) * choices + j);
      if (row < 0) continue;
      const float w = __ldg(weights + static_cast<long long>(t) * choices + j);
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(y + static_cast<long long>(row) * hidden) + c);
      const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&words[q]));
        acc[2 * q] = fmaf(w, f.x, acc[2 * q]);
        acc[2 * q + 1] = fmaf(w, f.y, acc[2 * q + 1]);
      }
    }
    float4* dst = reinterpret_cast<float4*>(out + static_cast<long long>(t) * hidden) + 2 * c;
    dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
}

// silu(a) * b with ex2.approx and rcp.approx (no slow path when exp(-a) overflows).
__device__ __forceinline__ float silu_gate(float a, float b) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(a * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return a * r * b;
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

// Issue rate of the block-scaled FP4 MMA with nothing else going on: every CTA issues
// `iters` x 4 tcgen05.mma (128 x 256 x 64, operands wherever shared memory happens to be
// zero-filled, scales and accumulator in tensor memory) back to back and waits for the last.
// The host divides the FLOPs by the elapsed time: the tensor pipe's rate at the clocks the
// GPU really runs at, which is the denominator the GEMM kernels are compared with besides
// the nominal figure. `status` gets 1 if the final wait was abandoned.
__global__ void __launch_bounds__(128, 1) mma_issue_peak_kernel(int iters, int* status) {
  extern __shared__ uint8_t peak_smem[];
  __shared__ alignas(8) uint64_t done_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const uint32_t base = (smem_u32(peak_smem) + 1023u) & ~1023u;
  for (uint32_t i = threadIdx.x; i < (48u * 1024u) / 16u; i += blockDim.x) {
    st_shared_v4(base + i * 16u, 0u, 0u, 0u, 0u);
  }
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&done_bar), 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  if (threadIdx.x < 32) tmem_alloc(smem_u32(&tmem_slot), 512);
  fence_proxy_async_shared();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (threadIdx.x < 32) {
    constexpr uint32_t idesc = nvf4_instr_desc(128, 256);
    constexpr uint32_t kHi = (1024u >> 4) | (1u << 14) | (2u << 29);
    const uint32_t lo_a = ((base >> 4) & 0x3FFFu) | (1u << 16);
    const uint32_t lo_b = lo_a + (16384u >> 4);
    if (elect_one()) {
      for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          tc_mma_nvf4(tmem, pack_desc(lo_a + 2 * j, kHi), pack_desc(lo_b + 2 * j, kHi), idesc,
                      tmem + 256 + 4 * j, tmem + 272 + 8 * j, 1u);
        }
      }
      tc_commit(smem_u32(&done_bar));
    }
    __syncwarp();
    if (!mbar_wait(smem_u32(&done_bar), 0, &abort_flag)) atomicExch(status, 1);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace nvfp4
