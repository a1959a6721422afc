// The NVFP4 block-scaled GEMM kernel for sm_100a: one persistent, warp-specialised
// kernel template that serves the dense/batched GEMM, the fused dual GEMM and the
// ragged grouped GEMM.
//
//   D[m, n] = alpha * sum_k (A[m, k] * SFA[m, k/16]) * (B[n, k] * SFB[n, k/16])
//
// A and B are packed E2M1 (two values per byte, low nibble = even k, K contiguous),
// SFA/SFB are UE4M3 bytes in the blocked 128x4 layout: scale (r, c) of a batch lives
// at byte ((r/128) * kb + c/4) * 512 + (r%32) * 16 + ((r/32)%4) * 4 + c%4, kb =
// ceil(k/64) (the layout of harness/workloads/quantization.py:90-102 in the reference).
//
// Roles (320 threads): warp 0 issues TMA loads into a ring of shared-memory stages;
// warps 6-9 move each stage's scale atoms from shared memory into that stage's columns of
// tensor memory (one warp per 32-lane quarter: a 512-byte atom is 32 rows of 16 bytes, i.e.
// ld.shared.v4 per atom and tcgen05.st.32x32b.x16 per sixteen columns, no reshuffle) and
// arrive on the stage's full barrier next to the producer; warp 1 issues tcgen05.mma
// kind::mxf4nvf4 (128 x BN x 64 per instruction, accumulators in tensor memory); warps 2-5
// read finished accumulators (tcgen05.ld), apply the epilogue and store through a small
// swizzled staging buffer so that global stores are coalesced. Warps 0 and 1 run their
// loops with all lanes and elect one lane for the issuing instructions. Keeping the scale
// copies off the MMA issue queue matters: tcgen05.cp there cost about as much queue time
// as the MMAs themselves.
//
// Work is a list of (tile, k-tile range) segments that every role derives from the
// same counters: in data-parallel mode CTA c takes tiles c, c + grid, ...; in stream-K
// mode the (tile, k-tile) units of all tiles are cut into `grid` equal contiguous
// ranges. A segment that does not cover its tile's whole K writes an FP32 partial to
// the workspace; the last CTA to arrive at the tile (one atomic counter per tile, reset
// by that CTA) adds the partials in segment order and finishes the tile, so results do
// not depend on arrival order, and no CTA waits on another. With `split` > 1 the CTAs of a
// thread-block cluster share one tile's K and exchange partial columns through shared
// memory instead (cluster_reduce): there each CTA waits, bounded, for its cluster peers,
// which the hardware schedules together.
//
// Every mbarrier wait is bounded; a role that gives up records a code in the status
// word, raises the shared abort flag and falls through to the common exit where tensor
// memory is freed.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "nvfp4_glue_kernels.cuh"
#include "sm100_ptx.cuh"

namespace nvfp4 {

// One GEMM problem: the dense (batched) problem, or one group of a grouped GEMM.
struct alignas(16) ProblemDesc {
  const uint8_t* sfa;
  const uint8_t* sfb;
  const uint8_t* sfb2;  // dual GEMM: scales of the second B
  void* d;
  int m, n, k, batches;
  int tiles_m, tiles_n;  // output tiles per batch
  int k_tiles;           // ceil(k / 256)
  int sf_kb;             // scale atoms along K: ceil(k / 64)
  int sf_mb, sf_nb;      // scale atom rows: ceil(m / 128), ceil(n / 128)
  uint8_t* sfd;          // NVFP4 output: blocked UE4M3 scales of D (rows m, one per 16 columns)
  long long tile_begin;  // first global tile index of this problem
  long long unit_begin;  // first global (tile, k-tile) unit of this problem
  int a_row0;            // routed groups: the group's first row in the A buffer all groups share
  int reserved;
};

enum : int { kModeDataParallel = 0, kModeStreamK = 1 };

// Routed groups: what the device needs to lay the groups out once the row count of every
// group is known (it lives in the plan's workspace, written by the bind).
struct alignas(16) RoutedHeader {
  long long total_tiles;        // written by moe_layout_kernel, read by the GEMM kernel
  const uint8_t* sfa_base;      // scales of the shared A buffer (blocked, 128-row atom rows)
  uint8_t* d_base;              // output buffer all groups share
  uint8_t* sfd_base;            // its scales (NVFP4 output) or null
  long long d_row_bytes;        // bytes of one output row
  long long sfa_block_bytes;    // bytes of one 128-row atom row of A's scales
  long long sfd_block_bytes;    // the same for D's scales
  int max_rows;                 // rows of the shared buffers (a multiple of 128)
  int overflow;                 // set (and left set) if some layout's padded rows did not fit
  int first_rows[kMoeMaxExperts];  // written by moe_layout_kernel: first row of every group
};

// Fills in what depends on the groups' row counts: every group's m, tile counts, first row
// in the shared buffers (blocks padded to 128 rows), operand addresses, and the totals; the
// rest of the table was written by the bind. One CTA of kMoeMaxExperts threads, one group per
// thread, two prefix sums in shared memory (blocks before a group; blocks that fit).
__global__ void __launch_bounds__(kMoeMaxExperts)
moe_layout_kernel(ProblemDesc* __restrict__ table, RoutedHeader* __restrict__ header,
                  const int* __restrict__ counts, int groups) {
  __shared__ int scan[kMoeMaxExperts];
  const int g = threadIdx.x;
  const int max_blocks = header->max_rows / 128;
  auto exclusive_prefix = [&](int value) {
    // Inclusive Hillis-Steele scan, then shifted by the own value.
    scan[g] = value;
    __syncthreads();
    for (int step = 1; step < kMoeMaxExperts; step *= 2) {
      const int other = g >= step ? scan[g - step] : 0;
      __syncthreads();
      scan[g] += other;
      __syncthreads();
    }
    const int before = scan[g] - value;
    __syncthreads();
    return before;
  };
  int m = g < groups ? max(counts[g], 0) : 0;
  int blocks = (m + 127) / 128;
  const int first_block = exclusive_prefix(blocks);
  // Groups that do not fit in the shared buffers are cut (the caller sized them too small).
  const int fits = min(blocks, max(max_blocks - first_block, 0));
  const bool cut = fits < blocks;
  blocks = fits;
  m = min(m, blocks * 128);
  const int tiles_before = exclusive_prefix(blocks);  // in units of one row of tiles
  if (g < groups) {
    ProblemDesc* pd = table + g;
    const int row = first_block * 128;
    const long long tile_begin = static_cast<long long>(tiles_before) * pd->tiles_n;
    pd->m = m;
    pd->tiles_m = blocks;
    pd->sf_mb = blocks;
    pd->a_row0 = row;
    pd->sfa = header->sfa_base + static_cast<long long>(first_block) * header->sfa_block_bytes;
    pd->d = header->d_base + static_cast<long long>(row) * header->d_row_bytes;
    pd->sfd = header->sfd_base != nullptr
                  ? header->sfd_base + static_cast<long long>(first_block) * header->sfd_block_bytes
                  : nullptr;
    pd->tile_begin = tile_begin;
    pd->unit_begin = tile_begin * pd->k_tiles;
    header->first_rows[g] = row;
    if (cut) header->overflow = 1;
    if (g == groups - 1) {
      header->total_tiles = tile_begin + static_cast<long long>(blocks) * pd->tiles_n;
    }
  }
}

enum : int {
  kStatusOk = 0,
  kStatusProducerTimeout = 1,
  kStatusMmaInputTimeout = 2,
  kStatusMmaAccumTimeout = 3,
  kStatusEpilogueTimeout = 4,
  kStatusScaleTimeout = 5,
  kStatusClusterTimeout = 6,
};

struct alignas(64) KernelParams {
  CUtensorMap map_a, map_b, map_b2;  // dense / dual: by value
  CUtensorMap map_d;  // 2-CTA kernel, 16-bit output: D as [l][m][n], box 64 columns x 128 rows
  ProblemDesc dense;
  const ProblemDesc* problems;  // grouped: one per group, device memory
  const CUtensorMap* maps;      // grouped: maps[s g] = A_g, maps[s g + 1] = B_g (dual: B1_g and
                                // maps[s g + 2] = B2_g), s = maps_per_group
  const float* alpha;           // device scalar, may be null (= 1)
  float* partials;              // stream-K: 2 * grid slots of slot_floats FP32 each
  unsigned int* counters;       // stream-K: one per tile, zero between launches
  int* status;                  // one word, 0 unless a wait was abandoned
  long long total_tiles, total_units;
  long long slot_floats;
  int num_problems;
  int mode;
  int b_streams;  // B is read once: mark its loads evict-first in L2
  int b_shuffle;  // 0, or 16 / 32: rows of B (and of its scales) are stored in FlashInfer's
                  // epilogue-shuffled order inside blocks of that many rows
  int split;      // > 1: CTAs of a cluster of this size split each tile's K (stream-K mode
                  // with grid = tiles * split) and reduce through peer shared memory
  int ring_stages;   // pipeline stages in use (fewer than the kernel's when the top of the
                     // pipeline memory is set aside as the cluster inbox)
  int inbox_offset;  // byte offset of that inbox from the pipeline base, or -1: peers may then
                     // write only after this CTA has told them its pipeline memory is free
  int maps_per_group;  // grouped: 2, or 3 for the grouped dual GEMM
  // Routed groups (a mixture-of-experts layer whose rows per expert are decided on the
  // device): the number of tiles is read from here, the group table was filled in by
  // moe_layout_kernel, and all groups share one A buffer described by maps[0]. Null otherwise.
  const long long* routed_tiles;
};

struct Segment {
  int prob;
  int m_tile, n_tile, batch;
  int k0, k1;              // k-tile range [k0, k1)
  long long tile_global;   // index into counters
  long long tile_unit0;    // first global unit of this tile
};

template <bool GROUPED>
struct WorkIter {
  const KernelParams& p;
  ProblemDesc pd;
  long long cur, end, step;
  int prob;

  __device__ __forceinline__ explicit WorkIter(const KernelParams& params) : p(params) {
    const long long cta = blockIdx.x, grid = gridDim.x;
    if (p.mode == kModeDataParallel) {
      cur = cta;
      end = p.total_tiles;
      if constexpr (GROUPED) {
        if (p.routed_tiles != nullptr) end = *p.routed_tiles;
      }
      step = grid;
    } else {
      cur = p.total_units * cta / grid;
      end = p.total_units * (cta + 1) / grid;
      step = 0;
    }
    prob = 0;
    load(0);
  }

  __device__ __forceinline__ void load(int g) {
    if constexpr (GROUPED) {
      pd = p.problems[g];
    } else {
      pd = p.dense;
    }
  }

  __device__ __forceinline__ long long tiles_of() const {
    return static_cast<long long>(pd.tiles_m) * pd.tiles_n * pd.batches;
  }

  // Tile index inside the current problem -> (batch, m_tile, n_tile). Tiles are
  // numbered down bands of eight tile rows so that tiles running at the same time
  // share rows of A and B in L2.
  __device__ __forceinline__ void decode(long long t, Segment& s) const {
    const int per_batch = pd.tiles_m * pd.tiles_n;
    s.batch = static_cast<int>(t / per_batch);
    const int r = static_cast<int>(t % per_batch);
    const int band_tiles = 8 * pd.tiles_n;
    const int band = r / band_tiles;
    const int in_band = r % band_tiles;
    const int height = min(8, pd.tiles_m - band * 8);
    s.m_tile = band * 8 + in_band % height;
    s.n_tile = in_band / height;
  }

  __device__ __forceinline__ bool next(Segment& s) {
    if (cur >= end) return false;
    if (p.mode == kModeDataParallel) {
      while (cur >= pd.tile_begin + tiles_of()) load(++prob);
      const long long t = cur - pd.tile_begin;
      decode(t, s);
      s.k0 = 0;
      s.k1 = pd.k_tiles;
      s.tile_global = cur;
      s.tile_unit0 = pd.unit_begin + t * pd.k_tiles;
      cur += step;
    } else {
      while (cur >= pd.unit_begin + tiles_of() * pd.k_tiles) load(++prob);
      const long long local = cur - pd.unit_begin;
      const long long t = local / pd.k_tiles;
      decode(t, s);
      s.k0 = static_cast<int>(local % pd.k_tiles);
      const long long len = min(static_cast<long long>(pd.k_tiles - s.k0), end - cur);
      s.k1 = s.k0 + static_cast<int>(len);
      s.tile_global = pd.tile_begin + t;
      s.tile_unit0 = pd.unit_begin + t * pd.k_tiles;
      cur += len;
    }
    s.prob = prob;
    return true;
  }
};

constexpr int const_min(int a, int b) { return a < b ? a : b; }
constexpr int const_max(int a, int b) { return a > b ? a : b; }
constexpr int const_pow2_at_least(int v) {
  int r = 32;
  while (r < v) r *= 2;
  return r;
}

template <typename T>
inline constexpr bool kIsBf16 = false;
template <>
inline constexpr bool kIsBf16<__nv_bfloat16> = true;

// Output type tag: D quantised to NVFP4 in the epilogue (packed E2M1 + blocked UE4M3 scales,
// one scale per 16 consecutive columns of a row), ready to be the A operand of the next GEMM.
struct Fp4Out {};

template <int BN_, bool DUAL_, typename OutT_, bool GROUPED_>
struct GemmConfig {
  static constexpr int BN = BN_;  // MMA N; for the dual GEMM both B tiles side by side
  static constexpr bool DUAL = DUAL_;
  static constexpr bool GROUPED = GROUPED_;
  using OutT = OutT_;
  static constexpr bool FP4_OUT = sizeof(OutT_) == 1;  // Fp4Out is the only one-byte tag
  static constexpr int BM = 128;
  static constexpr int OUT_BN = DUAL ? BN / 2 : BN;  // output columns per tile
  static constexpr int A_BYTES = BM * 128;           // 128 rows x 256 E2M1
  static constexpr int B_BYTES = BN * 128;
  // 128-row scale atoms per k-block: the dual GEMM always reads one atom of each B (a
  // 64-row tile uses half of it).
  static constexpr int SFB_BLOCKS = DUAL ? 2 : (BN + 127) / 128;
  // Dual GEMM on 64-column output tiles: the MMA's 128 scale columns are the tile's half
  // of B1's atom followed by the same half of B2's atom.
  static constexpr bool NARROW_DUAL = DUAL && BN == 128;
  static constexpr int SFA_BYTES = 4 * 512;
  static constexpr int SFB_BYTES = 4 * 512 * SFB_BLOCKS;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  // 227 KiB per CTA less 1 KiB alignment slack, the barriers, and the epilogue warps'
  // 8 KiB of staging for coalesced stores (both static).
  static constexpr int SMEM_BUDGET = 227 * 1024 - 2048 - 8192;
  static constexpr int STAGES = const_min(8, SMEM_BUDGET / STAGE_BYTES);
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
  static constexpr int ACC_BUFS = BN <= 128 ? 2 : 1;
  static constexpr int SFB_COLS = const_max(4, BN / 32);  // columns per k-block
  // Scale columns of one stage: SFA (4 k-blocks x 4) then SFB (4 k-blocks x SFB_COLS).
  static constexpr int SF_STAGE_COLS = 16 + 4 * SFB_COLS;
  static constexpr int SF_COL = ACC_BUFS * BN;  // first scale column
  static constexpr int TMEM_COLS = const_pow2_at_least(SF_COL + STAGES * SF_STAGE_COLS);
  static constexpr int THREADS = 320;
  static_assert(BN == 64 || BN == 128 || BN == 256, "unsupported tile width");
  static_assert(!DUAL || BN == 256 || BN == 128, "dual GEMM uses two 128- or 64-column B tiles");
  static_assert(TMEM_COLS <= 512, "tensor memory exceeded");
  static_assert(STAGES >= 2, "pipeline too shallow");
};

__device__ __forceinline__ void report_failure(const KernelParams& p, volatile int* abort_flag,
                                               int code) {
  *abort_flag = 1;
  atomicCAS(p.status, 0, code);
}

// x * sigmoid(x) on the special-function unit alone: ex2.approx and rcp.approx, about
// 2 ulp of FP32, far inside one FP16 rounding of the result. Neither has a slow path:
// the IEEE division and the correctly rounded reciprocal both branch to a subroutine
// when exp(-x) overflows to infinity, which cost ~20 us per 128x128 tile here.
// x -> -inf gives x * rcp(inf) = -0.
__device__ __forceinline__ float silu_f32(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return x * r;
}

// Two FP32 values rounded to nearest even into one 32-bit word of the 16-bit output type.
template <typename OutT>
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi) {
  if constexpr (sizeof(OutT) == 2 && !kIsBf16<OutT>) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

// Stores 32 consecutive output columns of one row in 16-byte pieces (8-byte pieces of
// FP16 when n is only a multiple of 4, whose rows are 8-byte aligned), dropping the
// pieces that start at or beyond column n (n is a multiple of the piece width).
template <typename OutT>
__device__ __forceinline__ void store_row_chunk(OutT* row_ptr, int col0, int n,
                                                const float (&v)[32]) {
  if constexpr (sizeof(OutT) == 2) {
    if ((n & 7) == 0) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        if (col0 + 8 * g < n) {
          uint4 q;
          q.x = pack_pair<OutT>(v[8 * g + 0], v[8 * g + 1]);
          q.y = pack_pair<OutT>(v[8 * g + 2], v[8 * g + 3]);
          q.z = pack_pair<OutT>(v[8 * g + 4], v[8 * g + 5]);
          q.w = pack_pair<OutT>(v[8 * g + 6], v[8 * g + 7]);
          *reinterpret_cast<uint4*>(row_ptr + col0 + 8 * g) = q;
        }
      }
    } else {
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        if (col0 + 4 * g < n) {
          uint2 q;
          q.x = pack_pair<OutT>(v[4 * g + 0], v[4 * g + 1]);
          q.y = pack_pair<OutT>(v[4 * g + 2], v[4 * g + 3]);
          *reinterpret_cast<uint2*>(row_ptr + col0 + 4 * g) = q;
        }
      }
    }
  } else {
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      if (col0 + 4 * g < n) {
        float4 q = make_float4(v[4 * g + 0], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
        *reinterpret_cast<float4*>(row_ptr + col0 + 4 * g) = q;
      }
    }
  }
}

// Coalesced form of the same store for a whole warp. Each lane holds 64 bytes of its own
// row (words w); stored directly, one warp instruction would touch 32 different rows, and
// the load/store unit handles one row per clock. The warp instead passes the 32 x 64-byte
// block through 2 KiB of shared memory (16-byte pieces XOR-swizzled by row pair, so both
// the row-wise writes and the 8-row reads are free of bank conflicts) and writes it out
// eight rows per instruction, four lanes per 64-byte run. `block` points at the block's
// first row at column 0; `col` is the first of its columns; rows at or beyond
// `rows_valid` and pieces at or beyond column `n` are dropped. Needs rows of D 16-byte
// aligned (n a multiple of 16 / sizeof(OutT)).
template <typename OutT>
__device__ __forceinline__ void store_block_coalesced(uint32_t stage, const uint32_t (&w)[16],
                                                      OutT* block, int col, int n,
                                                      int rows_valid, int lane) {
  constexpr int kPieceElems = 16 / static_cast<int>(sizeof(OutT));
  const uint32_t own = stage + static_cast<uint32_t>(lane) * 64u;
  const uint32_t own_swizzle = (static_cast<uint32_t>(lane) >> 1) & 3u;
#pragma unroll
  for (uint32_t q = 0; q < 4; ++q) {
    st_shared_v4(own + ((q ^ own_swizzle) << 4), w[4 * q], w[4 * q + 1], w[4 * q + 2],
                 w[4 * q + 3]);
  }
  __syncwarp();
  const int sub = lane >> 2;
  const uint32_t piece = static_cast<uint32_t>(lane) & 3u;
  const uint32_t src = stage + static_cast<uint32_t>(sub) * 64u +
                       ((piece ^ ((static_cast<uint32_t>(sub) >> 1) & 3u)) << 4);
  const int piece_col = col + static_cast<int>(piece) * kPieceElems;
  OutT* dst = block + static_cast<long long>(sub) * n + piece_col;
  const long long step = 8ll * n;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 v = ld_shared_v4(src + static_cast<uint32_t>(j) * 512u);
    if (8 * j + sub < rows_valid && piece_col < n) *reinterpret_cast<uint4*>(dst + j * step) = v;
  }
  __syncwarp();
}

// Weights prepared for FlashInfer's trtllm-gen kernels have their rows permuted inside blocks
// of 16 or 32 rows (physical row base + map[o] holds logical row base + o, with
// map[o] = (o % 4) * 8 + o / 4 for blocks of 32 and (o % 2) * 8 + o / 2 for blocks of 16:
// harness/workloads/batched_gemm/formats.py:143-161 in the reference). A GEMM on such a B
// produces the columns of D in the physical order; this puts the 32 columns a thread holds
// (one or two whole blocks) back in logical order. A register renaming: no data moves.
__device__ __forceinline__ void unshuffle_columns(float (&v)[32], int block) {
  if (block == 0) return;
  float u[32];
  if (block == 32) {
#pragma unroll
    for (int o = 0; o < 32; ++o) u[o] = v[(o % 4) * 8 + o / 4];
  } else {
#pragma unroll
    for (int o = 0; o < 32; ++o) u[o] = v[(o / 16) * 16 + ((o % 16) % 2) * 8 + (o % 16) / 2];
  }
#pragma unroll
  for (int o = 0; o < 32; ++o) v[o] = u[o];
}

// 32 output columns of the warp's 32 rows: coalesced when the rows of D are 16-byte
// aligned, row by row otherwise. `v` is this lane's row; `block` as above; `row_ptr`
// this lane's own row at column 0; `row_ok` whether that row exists.
template <typename OutT>
__device__ __forceinline__ void store_warp_chunk(uint32_t stage, OutT* block, OutT* row_ptr,
                                                 bool row_ok, int col0, int n, int rows_valid,
                                                 int lane, const float (&v)[32]) {
  constexpr int kPieceElems = 16 / static_cast<int>(sizeof(OutT));
  if (n % kPieceElems != 0) {
    if (row_ok) store_row_chunk<OutT>(row_ptr, col0, n, v);
    return;
  }
  if constexpr (sizeof(OutT) == 2) {
    uint32_t w[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      w[i] = pack_pair<OutT>(v[2 * i], v[2 * i + 1]);
    }
    store_block_coalesced<OutT>(stage, w, block, col0, n, rows_valid, lane);
  } else {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) w[i] = __float_as_uint(v[16 * half + i]);
      store_block_coalesced<OutT>(stage, w, block, col0 + 16 * half, n, rows_valid, lane);
    }
  }
}

// Adds to s1 (and s2 for the dual GEMM) the 32-column chunk `c` of row `row` of the
// partial tiles that CTAs [first, last] left in the workspace for the tile whose first
// unit is `tile_unit0`, in CTA order; loads of two partials are in flight together.
template <class Cfg>
__device__ __forceinline__ void add_partials(const KernelParams& p, float (&s1)[32],
                                             float (&s2)[32], long long first, long long last,
                                             long long tile_unit0, long long grid, int c, int row) {
  constexpr int GROUP = 1;
#pragma unroll 1
  for (long long b0 = first; b0 <= last; b0 += GROUP) {
    float4 t1[GROUP][8];
    float4 t2[GROUP][8];
#pragma unroll
    for (int u = 0; u < GROUP; ++u) {
      const long long b = b0 + u;
      if (b <= last) {
        const long long b_start = p.total_units * b / grid;
        const long long slot = 2 * b + (b_start < tile_unit0 ? 1 : 0);
        const float4* src = reinterpret_cast<const float4*>(p.partials + slot * p.slot_floats);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          t1[u][q] = __ldcg(src + (c * 8 + q) * 128 + row);
          if constexpr (Cfg::DUAL) {
            t2[u][q] = __ldcg(src + (Cfg::OUT_BN / 4 + c * 8 + q) * 128 + row);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < GROUP; ++u) {
      if (b0 + u <= last) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          s1[4 * q + 0] += t1[u][q].x;
          s1[4 * q + 1] += t1[u][q].y;
          s1[4 * q + 2] += t1[u][q].z;
          s1[4 * q + 3] += t1[u][q].w;
          if constexpr (Cfg::DUAL) {
            s2[4 * q + 0] += t2[u][q].x;
            s2[4 * q + 1] += t2[u][q].y;
            s2[4 * q + 2] += t2[u][q].z;
            s2[4 * q + 3] += t2[u][q].w;
          }
        }
      }
    }
  }
}

// Split-K inside a cluster: the `split` CTAs of a cluster hold partial sums of the same
// tile (one K slice each) in tensor memory. CTA r owns output columns
// [r * W, (r + 1) * W), W = tile width / split. Every CTA sends the columns it does not
// own to their owners' shared memory (the pipeline stages, free once the mainloop is
// done: each CTA first tells its peers so), then adds what it received to its own
// columns in rank order and stores them. No global workspace, no atomics; the result
// does not depend on timing. Called by the 128 epilogue threads.
template <class Cfg>
__device__ __forceinline__ void cluster_reduce(const KernelParams& p, const ProblemDesc& pd,
                                               const Segment& s, uint32_t taddr,
                                               uint32_t staging, uint32_t bar_ready,
                                               uint32_t bar_data, volatile int* abort_ptr,
                                               float alpha, int row, int epi_tid, int grow,
                                               typename Cfg::OutT* out_row,
                                               typename Cfg::OutT* out_block, int rows_valid,
                                               uint32_t store_stage) {
  using OutT = typename Cfg::OutT;
  // The dual GEMM keeps two accumulators side by side (h1 in columns [0, OUT_BN), h2 in
  // [OUT_BN, 2 * OUT_BN)); an owner of output columns needs both halves of them.
  constexpr int HALVES = Cfg::DUAL ? 2 : 1;
  const int split = p.split;
  const int rank = static_cast<int>(cluster_cta_rank());
  const int width = Cfg::OUT_BN / split;  // output columns per owner, a multiple of 32
  const int chunks = width / 32;
  const int lane = row & 31;
  // Bytes one CTA sends to one peer: the peer's columns of both accumulator halves, as
  // float4 [chunk][half][column / 4][row].
  const uint32_t portion = static_cast<uint32_t>(chunks * HALVES) * 16384u;
  uint32_t inbox = staging;  // where peers' columns arrive
  if (p.inbox_offset >= 0) {
    // Inbox path: the top of the pipeline memory was never used by this launch's pipeline, so
    // peers need no permission to write there. Every CTA puts the columns of each peer
    // into its own (now idle) pipeline memory with plain stores and sends them with one
    // bulk copy per peer, which counts its bytes on the peer's barrier: no remote store per
    // thread, no cluster-scope fence, no round trip to ask whether the peer is ready.
    inbox = staging + static_cast<uint32_t>(p.inbox_offset);
    if (epi_tid == 0) mbar_expect_tx(bar_data, static_cast<uint32_t>(split - 1) * portion);
    for (int peer = 0; peer < split; ++peer) {
      if (peer == rank) continue;
      const int out_slot = peer < rank ? peer : peer - 1;
      const uint32_t outbox = staging + static_cast<uint32_t>(out_slot) * portion;
#pragma unroll 1
      for (int c = 0; c < chunks; ++c) {
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {
          uint32_t r1[32];
          tmem_load_32(taddr + h * Cfg::OUT_BN + peer * width + c * 32, r1);
          tmem_load_wait();
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint32_t index = ((c * HALVES + h) * 8 + q) * 128 + row;
            st_shared_v4(outbox + index * 16u, r1[4 * q], r1[4 * q + 1], r1[4 * q + 2],
                         r1[4 * q + 3]);
          }
        }
      }
    }
    fence_proxy_async_shared();
    named_barrier_sync(1, 128);
    if (epi_tid == 0) {
      for (int peer = 0; peer < split; ++peer) {
        if (peer == rank) continue;
        const int out_slot = peer < rank ? peer : peer - 1;
        const int in_slot = rank < peer ? rank : rank - 1;  // my slot in the peer's inbox
        bulk_copy_to_peer(cluster_map_shared(inbox + static_cast<uint32_t>(in_slot) * portion, peer),
                          staging + static_cast<uint32_t>(out_slot) * portion, portion,
                          cluster_map_shared(bar_data, peer));
      }
    }
    // The bytes arrive through the async proxy and are counted on the barrier: the plain
    // wait is the one every TMA consumer uses.
    if (!mbar_wait(bar_data, 0, abort_ptr)) {
      report_failure(p, abort_ptr, kStatusClusterTimeout);
      return;
    }
  } else {
  // 1. My pipeline memory is free: tell every peer it may write into it.
  if (epi_tid == 0) {
    for (int peer = 0; peer < split; ++peer) {
      if (peer != rank) mbar_arrive_cluster(cluster_map_shared(bar_ready, peer));
    }
  }
  // 2. Wait until every peer has said the same (one lane polls for its warp).
  int ready = 1;
  if (lane == 0) ready = mbar_wait_cluster(bar_ready, 0, abort_ptr) ? 1 : 0;
  ready = __shfl_sync(0xFFFFFFFFu, ready, 0);
  if (!ready) {
    report_failure(p, abort_ptr, kStatusClusterTimeout);
    return;
  }
  // 3. Send: slot index at the receiver = my rank among its peers.
  for (int peer = 0; peer < split; ++peer) {
    if (peer == rank) continue;
    const int slot = rank < peer ? rank : rank - 1;
    const uint32_t remote = cluster_map_shared(staging, peer);
#pragma unroll 1
    for (int c = 0; c < chunks; ++c) {
#pragma unroll
      for (int h = 0; h < HALVES; ++h) {
        uint32_t r1[32];
        tmem_load_32(taddr + h * Cfg::OUT_BN + peer * width + c * 32, r1);
        tmem_load_wait();
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const uint32_t index = (((slot * chunks + c) * HALVES + h) * 8 + q) * 128 + row;
          st_cluster_v4(remote + index * 16u,
                        make_float4(__uint_as_float(r1[4 * q]), __uint_as_float(r1[4 * q + 1]),
                                    __uint_as_float(r1[4 * q + 2]), __uint_as_float(r1[4 * q + 3])));
        }
      }
    }
  }
  // One lane per warp signals every peer: the warp's stores are ordered before the lane's
  // fence by the __syncwarp, the fence makes them visible at cluster scope before the
  // (relaxed) arrives. A releasing arrive per thread and peer - 128 x (split - 1) remote
  // operations that each wait for the thread's stores - cost several microseconds for
  // clusters of four.
  __syncwarp();
  if (lane == 0) {
    fence_acq_rel_cluster();
    for (int peer = 0; peer < split; ++peer) {
      if (peer != rank) mbar_arrive_peer(cluster_map_shared(bar_data, peer));
    }
  }
  // 4. Wait for every peer's columns: one lane acquires for its warp.
  int arrived = 1;
  if (lane == 0) arrived = mbar_wait_cluster(bar_data, 0, abort_ptr) ? 1 : 0;
  arrived = __shfl_sync(0xFFFFFFFFu, arrived, 0);
  if (!arrived) {
    report_failure(p, abort_ptr, kStatusClusterTimeout);
    return;
  }
  }
  // 5. Own columns: add in rank order, finish, store.
  const int n0 = s.n_tile * Cfg::OUT_BN + rank * width;
#pragma unroll 1
  for (int c = 0; c < chunks; ++c) {
    float sum[HALVES][32];
#pragma unroll
    for (int h = 0; h < HALVES; ++h) {
      uint32_t own[32];
      tmem_load_32(taddr + h * Cfg::OUT_BN + rank * width + c * 32, own);
      tmem_load_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) sum[h][i] = 0.0f;
      for (int src = 0; src < split; ++src) {
        if (src == rank) {
#pragma unroll
          for (int i = 0; i < 32; ++i) sum[h][i] += __uint_as_float(own[i]);
        } else {
          const int slot = src < rank ? src : src - 1;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint32_t index = (((slot * chunks + c) * HALVES + h) * 8 + q) * 128 + row;
            const uint4 t = ld_shared_v4(inbox + index * 16u);
            sum[h][4 * q + 0] += __uint_as_float(t.x);
            sum[h][4 * q + 1] += __uint_as_float(t.y);
            sum[h][4 * q + 2] += __uint_as_float(t.z);
            sum[h][4 * q + 3] += __uint_as_float(t.w);
          }
        }
      }
    }
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if constexpr (Cfg::DUAL) {
        v[i] = silu_f32(sum[0][i] * alpha) * (sum[HALVES - 1][i] * alpha);
      } else {
        v[i] = sum[0][i] * alpha;
      }
    }
    if constexpr (Cfg::DUAL) {
      // Two accumulators are live here; the staged store on top of them spills.
      if (grow < pd.m) store_row_chunk<OutT>(out_row, n0 + c * 32, pd.n, v);
    } else {
      unshuffle_columns(v, p.b_shuffle);
      store_warp_chunk<OutT>(store_stage, out_block, out_row, grow < pd.m, n0 + c * 32, pd.n,
                             rows_valid, row & 31, v);
    }
  }
}

// STALLED is the failure-detection self-test: the producer issues no copy at all, so every
// other role waits on a barrier that nothing completes, and the wait limit is a few
// milliseconds instead of about a second. The kernel must then report the abandoned wait in
// the status word, stop all roles through the abort flag, free its tensor memory and return
// by itself. Instantiated once, for nvfp4_selftest_abandoned_wait.
template <class Cfg, bool STALLED = false>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
nvfp4_gemm_kernel(const __grid_constant__ KernelParams p) {
  constexpr int BN = Cfg::BN;
  constexpr uint32_t kLimit = STALLED ? (1u << 17) : kWaitLimitSpins;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int ACC_BUFS = Cfg::ACC_BUFS;
  using OutT = typename Cfg::OutT;

  extern __shared__ uint8_t dyn_smem[];
  // A stage is full when A and B have landed (the producer's arrive + transaction bytes)
  // and the four scale movers have put its scales into tensor memory: five arrivals.
  __shared__ alignas(8) uint64_t bar_full[STAGES];
  __shared__ alignas(8) uint64_t bar_empty[STAGES];
  __shared__ alignas(8) uint64_t bar_acc_full[ACC_BUFS];
  __shared__ alignas(8) uint64_t bar_acc_empty[ACC_BUFS];
  __shared__ alignas(8) uint64_t bar_sf_full[STAGES];  // a stage's scale atoms have landed
  __shared__ alignas(8) uint64_t bar_peer_ready;  // every peer's pipeline memory is free
  __shared__ alignas(8) uint64_t bar_peer_data;   // every peer's partial columns have arrived
  __shared__ alignas(16) uint8_t epi_stage[4][2048];  // per epilogue warp: 32 rows x 64 bytes
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int epi_last_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(dyn_smem) + 1023u) & ~1023u;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 5);
      mbar_init(smem_u32(&bar_empty[s]), 1);
      mbar_init(smem_u32(&bar_sf_full[s]), 1);
    }
#pragma unroll
    for (int a = 0; a < ACC_BUFS; ++a) {
      mbar_init(smem_u32(&bar_acc_full[a]), 1);
      mbar_init(smem_u32(&bar_acc_empty[a]), 128);
    }
    const uint32_t peers = p.split > 1 ? static_cast<uint32_t>(p.split - 1) : 1u;
    mbar_init(smem_u32(&bar_peer_ready), peers);
    // Inbox path: one local arrival (expect_tx) + the peers' bytes. Otherwise one arrival
    // per epilogue warp and peer.
    mbar_init(smem_u32(&bar_peer_data), p.inbox_offset >= 0 ? 1u : 4u * peers);
    abort_flag = 0;
    epi_last_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_slot), Cfg::TMEM_COLS);
  }
  tc_fence_before_sync();
  __syncthreads();
  // Peers arrive on this CTA's barriers, so they must be initialised cluster-wide before the
  // first remote access, which comes only after the mainloop: every thread announces itself
  // here and collects the others' announcements when it first needs them (the epilogue
  // before the exchange, everyone else at the exit), instead of stalling the start.
  if (p.split > 1) cluster_arrive();
  bool cluster_joined = false;
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abort_ptr = &abort_flag;
  const int ring = p.ring_stages;  // <= STAGES
  // Everything above touched only this CTA's shared and tensor memory, so under
  // programmatic dependent launch it overlaps the previous kernel's tail; nothing below
  // may read or write global memory before that kernel has finished.
  grid_dependency_wait();
  grid_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    // The whole warp runs the loop (waits included); one elected lane issues the copies.
    {
      const uint64_t pol_a = l2_policy_evict_last();
      const uint64_t pol_b = p.b_streams ? l2_policy_evict_first() : l2_policy_evict_last();
      if constexpr (!Cfg::GROUPED) {
        if (elect_one()) {
          prefetch_tensormap(&p.map_a);
          prefetch_tensormap(&p.map_b);
          if constexpr (Cfg::DUAL) prefetch_tensormap(&p.map_b2);
        }
      }
      WorkIter<Cfg::GROUPED> it(p);
      Segment s;
      int stage = 0;
      uint32_t phase = 0;
      uint32_t stage_smem = smem_base;
      const uint32_t full0 = smem_u32(&bar_full[0]);
      const uint32_t sf_full0 = smem_u32(&bar_sf_full[0]);
      const uint32_t empty0 = smem_u32(&bar_empty[0]);
      bool ok = true;
      int acquired_prob = -1;
      while (ok && it.next(s)) {
        const ProblemDesc& pd = it.pd;
        const CUtensorMap* group_maps = p.maps + p.maps_per_group * s.prob;  // grouped only
        const bool routed = Cfg::GROUPED && p.routed_tiles != nullptr;
        const CUtensorMap* map_a = Cfg::GROUPED ? (routed ? p.maps : group_maps) : &p.map_a;
        const CUtensorMap* map_b = Cfg::GROUPED ? group_maps + 1 : &p.map_b;
        const CUtensorMap* map_b2 = Cfg::GROUPED ? group_maps + 2 : &p.map_b2;
        if constexpr (Cfg::GROUPED) {
          // A group's tensor maps were copied into the workspace by the host; an earlier
          // plan's maps may have lived at the same addresses.
          if (s.prob != acquired_prob) {
            if (elect_one()) {
              tensormap_acquire(map_a);
              tensormap_acquire(map_b);
              if constexpr (Cfg::DUAL) tensormap_acquire(map_b2);
            }
            __syncwarp();
            acquired_prob = s.prob;
          }
        }
        const int m0 = s.m_tile * Cfg::BM + (Cfg::GROUPED ? pd.a_row0 : 0);
        const int n0 = s.n_tile * Cfg::OUT_BN;
        // Scale atoms of this tile's rows: one 512-byte atom per 64 K elements, four per
        // k-tile, contiguous along K.
        const long long atom_row_a = static_cast<long long>(s.batch) * pd.sf_mb + s.m_tile;
        const uint8_t* sfa_src = pd.sfa + (atom_row_a * pd.sf_kb + 4ll * s.k0) * 512;
        const int nb0 = n0 / 128;  // first 128-row scale atom row of the tile's B rows
        const uint8_t* sfb_src[Cfg::SFB_BLOCKS];
        int sfb_valid = 0;
#pragma unroll
        for (int i = 0; i < Cfg::SFB_BLOCKS; ++i) {
          const int nb = Cfg::DUAL ? nb0 : nb0 + i;
          const uint8_t* base = (Cfg::DUAL && i == 1) ? pd.sfb2 : pd.sfb;
          const long long atom_row_b = static_cast<long long>(s.batch) * pd.sf_nb + nb;
          sfb_src[i] = nb < pd.sf_nb ? base + (atom_row_b * pd.sf_kb + 4ll * s.k0) * 512 : nullptr;
          if (nb < pd.sf_nb) ++sfb_valid;
        }
        constexpr uint32_t ab_bytes = Cfg::A_BYTES + Cfg::B_BYTES;
        int atoms_left = pd.sf_kb - 4 * s.k0;
        int kbyte = s.k0 * 128;
        for (int kt = s.k0; kt < s.k1; ++kt) {
          if (!mbar_wait<kLimit>(empty0 + 8 * stage, phase ^ 1u, abort_ptr)) {
            report_failure(p, abort_ptr, kStatusProducerTimeout);
            ok = false;
            break;
          }
          const uint32_t sf_bytes = atoms_left >= 4 ? 2048u : static_cast<uint32_t>(atoms_left) * 512u;
          const uint32_t bar = full0 + 8 * stage;
          const uint32_t sf_bar = sf_full0 + 8 * stage;
          const uint32_t a_dst = stage_smem;
          const uint32_t b_dst = a_dst + Cfg::A_BYTES;
          const uint32_t sfa_dst = b_dst + Cfg::B_BYTES;
          const uint32_t sfb_dst = sfa_dst + Cfg::SFA_BYTES;
          // Scales first, on their own barrier: they are small, land early, and the
          // scale movers can put them into tensor memory while A and B are still in
          // flight.
          if (!STALLED && elect_one()) {
            mbar_expect_tx(sf_bar, sf_bytes * (1u + sfb_valid));
            bulk_load(sfa_dst, sfa_src, sf_bytes, sf_bar, pol_a);
#pragma unroll
            for (int i = 0; i < Cfg::SFB_BLOCKS; ++i) {
              if (sfb_src[i] != nullptr) {
                bulk_load(sfb_dst + i * 2048, sfb_src[i], sf_bytes, sf_bar, pol_b);
              }
            }
            mbar_expect_tx(bar, ab_bytes);
            tma_load_3d(a_dst, map_a, bar, kbyte, m0, s.batch, pol_a);
            tma_load_3d(b_dst, map_b, bar, kbyte, n0, s.batch, pol_b);
            if constexpr (Cfg::DUAL) {
              tma_load_3d(b_dst + Cfg::B_BYTES / 2, map_b2, bar, kbyte, n0, s.batch, pol_b);
            }
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < Cfg::SFB_BLOCKS; ++i) {
            if (sfb_src[i] != nullptr) sfb_src[i] += 2048;
          }
          sfa_src += 2048;
          atoms_left -= 4;
          kbyte += 128;
          stage_smem += Cfg::STAGE_BYTES;
          if (++stage == ring) {
            stage = 0;
            phase ^= 1u;
            stage_smem = smem_base;
          }
        }
      }
      if (!ok || *abort_ptr != 0) {
        // Abandoned run: give copies still in flight time to land before the CTA exits.
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs the loop; one elected lane (the same one every time, since a
    // commit covers the instructions of the thread that issues it) issues the MMAs.
    {
      constexpr uint32_t idesc = nvf4_instr_desc(128, BN);
      // Descriptor words that never change: the high half (stride between eight-row
      // groups 1024 bytes, version, 128-byte swizzle) and, per stage, the low half
      // (address >> 4, leading offset). A stage is STAGE_BYTES / 16 further in the
      // address field; a K = 64 step is 32 bytes = 2 further along the swizzled row.
      constexpr uint32_t kHiOperand = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t kStage16 = Cfg::STAGE_BYTES >> 4;
      const uint32_t lo_a0 = ((smem_base >> 4) & 0x3FFFu) | (1u << 16);
      const uint32_t lo_b0 = lo_a0 + (Cfg::A_BYTES >> 4);
      const uint32_t full0 = smem_u32(&bar_full[0]);
      const uint32_t empty0 = smem_u32(&bar_empty[0]);
      WorkIter<Cfg::GROUPED> it(p);
      Segment s;
      int stage = 0;
      uint32_t phase = 0;
      uint32_t stage16 = 0;
      uint32_t t_sf = tmem_base + Cfg::SF_COL;  // this stage's scale columns
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      while (ok && it.next(s)) {
        const ProblemDesc& pd = it.pd;
        if (!mbar_wait<kLimit>(smem_u32(&bar_acc_empty[acc]), acc_phase ^ 1u, abort_ptr)) {
          report_failure(p, abort_ptr, kStatusMmaAccumTimeout);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        // A 64-column tile uses half of a 128-row scale atom: columns 0-1 or 2-3.
        const uint32_t sfb_half = (BN == 64) ? 2u * (s.n_tile & 1) : 0u;
        int atoms_left = pd.sf_kb - 4 * s.k0;
        uint32_t accumulate = 0;
        for (int kt = s.k0; kt < s.k1; ++kt) {
          if (!mbar_wait<kLimit>(full0 + 8 * stage, phase, abort_ptr)) {
            report_failure(p, abort_ptr, kStatusMmaInputTimeout);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t lo_a = lo_a0 + stage16;
          const uint32_t lo_b = lo_b0 + stage16;
          const uint32_t t_sfb = t_sf + 16 + sfb_half;
          if (elect_one()) {
            if (atoms_left >= 4) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                tc_mma_nvf4(d_tmem, pack_desc(lo_a + 2 * j, kHiOperand),
                            pack_desc(lo_b + 2 * j, kHiOperand), idesc, t_sf + 4 * j,
                            t_sfb + j * Cfg::SFB_COLS, j > 0 ? 1u : accumulate);
              }
            } else {
              // K tail: fewer than four 64-wide blocks left.
              const int mmas = min(4, atoms_left);
              for (int j = 0; j < mmas; ++j) {
                tc_mma_nvf4(d_tmem, pack_desc(lo_a + 2 * j, kHiOperand),
                            pack_desc(lo_b + 2 * j, kHiOperand), idesc, t_sf + 4 * j,
                            t_sfb + j * Cfg::SFB_COLS, j > 0 ? 1u : accumulate);
              }
            }
            tc_commit(empty0 + 8 * stage);
          }
          __syncwarp();
          accumulate = 1;
          atoms_left -= 4;
          stage16 += kStage16;
          t_sf += Cfg::SF_STAGE_COLS;
          if (++stage == ring) {
            stage = 0;
            phase ^= 1u;
            stage16 = 0;
            t_sf = tmem_base + Cfg::SF_COL;
          }
        }
        if (!ok) break;
        if (elect_one()) tc_commit(smem_u32(&bar_acc_full[acc]));
        __syncwarp();
        if (++acc == ACC_BUFS) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ scale movers
    // Warp q of the four owns tensor-memory lanes 32q..32q+31. For every stage it copies
    // the stage's scale atoms (shared memory, written by the producer's bulk copies)
    // into the stage's scale columns: lane i takes the atom's 16-byte row i, which holds
    // the scales of rows i, 32+i, 64+i, 96+i for one 64-wide K block = four columns.
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t sf_full0 = smem_u32(&bar_sf_full[0]);
    const uint32_t full0 = smem_u32(&bar_full[0]);
    const uint32_t row_off = static_cast<uint32_t>(lane) * 16u;
    WorkIter<Cfg::GROUPED> it(p);
    Segment s;
    int stage = 0;
    uint32_t phase = 0;
    uint32_t sf_smem = smem_base + Cfg::A_BYTES + Cfg::B_BYTES;
    uint32_t t_sf = tmem_base + lane_base + Cfg::SF_COL;
    bool ok = true;
    while (ok && it.next(s)) {
      int atoms_left = it.pd.sf_kb - 4 * s.k0;
      const bool upper_half = (s.n_tile & 1) != 0;  // narrow dual: rows 64-127 of the atoms
      for (int kt = s.k0; kt < s.k1; ++kt) {
        if (!mbar_wait<kLimit>(sf_full0 + 8 * stage, phase, abort_ptr)) {
          report_failure(p, abort_ptr, kStatusScaleTimeout);
          ok = false;
          break;
        }
        const int atoms = min(4, atoms_left);
        if (atoms == 4) {
          uint4 va[4];
          uint4 vb[4][Cfg::SFB_BLOCKS];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            va[j] = ld_shared_v4(sf_smem + 512 * j + row_off);
#pragma unroll
            for (int i = 0; i < Cfg::SFB_BLOCKS; ++i) {
              vb[j][i] = ld_shared_v4(sf_smem + Cfg::SFA_BYTES + 2048 * i + 512 * j + row_off);
            }
          }
          // The stage's columns are contiguous (A: k-block j at 4j; B: k-block j, atom i
          // at 16 + j * SFB_COLS + 4i), so whole 16-column stores cover them: the cost of
          // a tensor-memory store is per instruction, not per column.
          tmem_store_16(t_sf, va[0], va[1], va[2], va[3]);
          if constexpr (Cfg::NARROW_DUAL) {
            // Two of an atom row's four words belong to the tile's 64 rows of B.
            uint4 w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              w[j] = upper_half ? make_uint4(vb[j][0].z, vb[j][0].w, vb[j][1].z, vb[j][1].w)
                                : make_uint4(vb[j][0].x, vb[j][0].y, vb[j][1].x, vb[j][1].y);
            }
            tmem_store_16(t_sf + 16, w[0], w[1], w[2], w[3]);
          } else if constexpr (Cfg::SFB_BLOCKS == 1) {
            tmem_store_16(t_sf + 16, vb[0][0], vb[1][0], vb[2][0], vb[3][0]);
          } else {
            tmem_store_16(t_sf + 16, vb[0][0], vb[0][1], vb[1][0], vb[1][1]);
            tmem_store_16(t_sf + 32, vb[2][0], vb[2][1], vb[3][0], vb[3][1]);
          }
        } else {
          for (int j = 0; j < atoms; ++j) {
            tmem_store_4(t_sf + 4 * j, ld_shared_v4(sf_smem + 512 * j + row_off));
            if constexpr (Cfg::NARROW_DUAL) {
              const uint4 b1 = ld_shared_v4(sf_smem + Cfg::SFA_BYTES + 512 * j + row_off);
              const uint4 b2 = ld_shared_v4(sf_smem + Cfg::SFA_BYTES + 2048 + 512 * j + row_off);
              tmem_store_4(t_sf + 16 + 4 * j, upper_half ? make_uint4(b1.z, b1.w, b2.z, b2.w)
                                                         : make_uint4(b1.x, b1.y, b2.x, b2.y));
            } else {
#pragma unroll
              for (int i = 0; i < Cfg::SFB_BLOCKS; ++i) {
                tmem_store_4(t_sf + 16 + j * Cfg::SFB_COLS + 4 * i,
                             ld_shared_v4(sf_smem + Cfg::SFA_BYTES + 2048 * i + 512 * j + row_off));
              }
            }
          }
        }
        tmem_store_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(full0 + 8 * stage);
        atoms_left -= 4;
        sf_smem += Cfg::STAGE_BYTES;
        t_sf += Cfg::SF_STAGE_COLS;
        if (++stage == ring) {
          stage = 0;
          phase ^= 1u;
          sf_smem = smem_base + Cfg::A_BYTES + Cfg::B_BYTES;
          t_sf = tmem_base + lane_base + Cfg::SF_COL;
        }
      }
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // the 32 tensor-memory lanes this warp may read
    const int row = quarter * 32 + lane;
    const int epi_tid = threadIdx.x - 64;
    const float alpha = p.alpha != nullptr ? __ldg(p.alpha) : 1.0f;
    const long long grid = gridDim.x;
    const long long cta = blockIdx.x;
    WorkIter<Cfg::GROUPED> it(p);
    Segment s;
    int acc = 0;
    uint32_t acc_phase = 0;
    while (it.next(s)) {
      const ProblemDesc& pd = it.pd;
      if (!mbar_wait<kLimit>(smem_u32(&bar_acc_full[acc]), acc_phase, abort_ptr)) {
        report_failure(p, abort_ptr, kStatusEpilogueTimeout);
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      const int grow = s.m_tile * Cfg::BM + row;
      const int n0 = s.n_tile * Cfg::OUT_BN;
      OutT* out_row = reinterpret_cast<OutT*>(pd.d) +
                      (static_cast<long long>(s.batch) * pd.m + grow) * pd.n;
      // First row of this warp's 32 rows, and how many of them exist.
      OutT* out_block = out_row - static_cast<long long>(lane) * pd.n;
      const int rows_valid = pd.m - (grow - lane);
      const uint32_t stage_smem = smem_u32(&epi_stage[quarter][0]);
      const bool whole = (s.k0 == 0 && s.k1 == pd.k_tiles);

      if constexpr (Cfg::FP4_OUT) {
        // NVFP4 output (whole tiles only: such plans are data parallel). Per row and 16
        // columns: scale = e4m3(amax / 6), codes = E2M1(v / scale) - the arithmetic of
        // quantize_nvfp4_kernel, so the bytes equal quantising the FP32 result afterwards.
        // A thread owns one row: 32 columns give 16 packed bytes, 64 columns give four
        // scale bytes that are contiguous in the blocked layout.
        uint8_t* d_row = static_cast<uint8_t*>(pd.d) +
                         (static_cast<long long>(s.batch) * pd.m + grow) * (pd.n / 2);
        const int sf_cb = (pd.n + 63) / 64;
        uint8_t* sf_row = pd.sfd +
                          (static_cast<long long>(s.batch) * pd.sf_mb + s.m_tile) * sf_cb * 512 +
                          (row % 32) * 16 + ((row / 32) % 4) * 4;
#pragma unroll 1
        for (int c2 = 0; c2 < Cfg::OUT_BN / 64; ++c2) {
          uint32_t scale_word = 0;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int c = 2 * c2 + half;
            uint32_t r1[32];
            tmem_load_32(taddr + c * 32, r1);
            if constexpr (Cfg::DUAL) {
              uint32_t r2[32];
              tmem_load_32(taddr + Cfg::OUT_BN + c * 32, r2);
              tmem_load_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                r1[i] = __float_as_uint(silu_f32(__uint_as_float(r1[i]) * alpha) *
                                        (__uint_as_float(r2[i]) * alpha));
              }
            } else {
              tmem_load_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) r1[i] = __float_as_uint(__uint_as_float(r1[i]) * alpha);
            }
            if (c == Cfg::OUT_BN / 32 - 1) {
              tc_fence_before_sync();
              mbar_arrive(smem_u32(&bar_acc_empty[acc]));
            }
            uint32_t words[4];
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
              float v[16];
              float amax = 0.0f;
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                v[i] = __uint_as_float(r1[16 * blk + i]);
                amax = fmaxf(amax, fabsf(v[i]));
              }
              const uint32_t bits = nvfp4_scale_bits(amax);
              const float scale = nvfp4_scale_value(bits);
              scale_word |= bits << (8 * (2 * half + blk));
              const uint2 codes =
                  scale > 0.0f ? nvfp4_block_codes(v, amax, scale) : make_uint2(0u, 0u);
              words[2 * blk] = codes.x;
              words[2 * blk + 1] = codes.y;
            }
            if (grow < pd.m && n0 + c * 32 < pd.n) {
              *reinterpret_cast<uint4*>(d_row + (n0 + c * 32) / 2) =
                  make_uint4(words[0], words[1], words[2], words[3]);
            }
          }
          if (grow < pd.m && n0 + c2 * 64 < pd.n) {
            *reinterpret_cast<uint32_t*>(sf_row + static_cast<long long>((n0 + c2 * 64) / 64) * 512) =
                scale_word;
          }
        }
      } else if (whole) {
#pragma unroll 1
        for (int c = 0; c < Cfg::OUT_BN / 32; ++c) {
          uint32_t r1[32];
          float v[32];
          tmem_load_32(taddr + c * 32, r1);
          if constexpr (Cfg::DUAL) {
            uint32_t r2[32];
            tmem_load_32(taddr + Cfg::OUT_BN + c * 32, r2);
            tmem_load_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              v[i] = silu_f32(__uint_as_float(r1[i]) * alpha) * (__uint_as_float(r2[i]) * alpha);
            }
          } else {
            tmem_load_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r1[i]) * alpha;
          }
          if (c == Cfg::OUT_BN / 32 - 1) {
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&bar_acc_empty[acc]));
          }
          if constexpr (!Cfg::DUAL) unshuffle_columns(v, p.b_shuffle);
          store_warp_chunk<OutT>(stage_smem, out_block, out_row, grow < pd.m, n0 + c * 32, pd.n,
                                 rows_valid, lane, v);
        }
      } else if (!Cfg::GROUPED && p.split > 1) {  // grouped plans never split in clusters
        if (!cluster_joined) {
          cluster_wait();
          cluster_joined = true;
        }
        cluster_reduce<Cfg>(p, pd, s, taddr, smem_base, smem_u32(&bar_peer_ready),
                            smem_u32(&bar_peer_data), abort_ptr, alpha, row, epi_tid, grow,
                            out_row, out_block, rows_valid, stage_smem);
        tc_fence_before_sync();
        mbar_arrive(smem_u32(&bar_acc_empty[acc]));
      } else {
        // Partial sum of this segment -> workspace slot as float4 [column / 4][row], so
        // that the 32 rows of a warp write (and later read) 512 contiguous bytes.
        const long long my_start = p.total_units * cta / grid;
        const long long my_slot = 2 * cta + (my_start < s.tile_unit0 ? 1 : 0);
        float4* ws = reinterpret_cast<float4*>(p.partials + my_slot * p.slot_floats);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r1[32];
          tmem_load_32(taddr + c * 32, r1);
          tmem_load_wait();
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            ws[(c * 8 + q) * 128 + row] =
                make_float4(__uint_as_float(r1[4 * q]), __uint_as_float(r1[4 * q + 1]),
                            __uint_as_float(r1[4 * q + 2]), __uint_as_float(r1[4 * q + 3]));
          }
        }
        __threadfence();
        named_barrier_sync(1, 128);
        const long long unit_last = s.tile_unit0 + pd.k_tiles - 1;
        const long long first_cta = ((s.tile_unit0 + 1) * grid - 1) / p.total_units;
        const long long last_cta = ((unit_last + 1) * grid - 1) / p.total_units;
        if (epi_tid == 0) {
          const unsigned int parts = static_cast<unsigned int>(last_cta - first_cta + 1);
          const unsigned int old = atomicAdd(&p.counters[s.tile_global], 1u);
          const int last = (old == parts - 1u) ? 1 : 0;
          if (last) p.counters[s.tile_global] = 0u;
          epi_last_flag = last;
        }
        named_barrier_sync(1, 128);
        if (epi_last_flag) {
          __threadfence();
#pragma unroll 1
          for (int c = 0; c < Cfg::OUT_BN / 32; ++c) {
            float s1[32];
            float s2[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              s1[i] = 0.0f;
              s2[i] = 0.0f;
            }
            // Partials are added in segment order, so the sum does not depend on which
            // CTA arrives last: the segments before this CTA's from the workspace, its
            // own straight from tensor memory (it is still there), then the rest.
            add_partials<Cfg>(p, s1, s2, first_cta, cta - 1, s.tile_unit0, grid, c, row);
            {
              uint32_t own[32];
              tmem_load_32(taddr + c * 32, own);
              tmem_load_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) s1[i] += __uint_as_float(own[i]);
              if constexpr (Cfg::DUAL) {
                tmem_load_32(taddr + Cfg::OUT_BN + c * 32, own);
                tmem_load_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) s2[i] += __uint_as_float(own[i]);
              }
            }
            add_partials<Cfg>(p, s1, s2, cta + 1, last_cta, s.tile_unit0, grid, c, row);
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if constexpr (Cfg::DUAL) {
                v[i] = silu_f32(s1[i] * alpha) * (s2[i] * alpha);
              } else {
                v[i] = s1[i] * alpha;
              }
            }
            if constexpr (!Cfg::DUAL) unshuffle_columns(v, p.b_shuffle);
            store_warp_chunk<OutT>(stage_smem, out_block, out_row, grow < pd.m, n0 + c * 32, pd.n,
                                   rows_valid, lane, v);
          }
        }
        tc_fence_before_sync();
        mbar_arrive(smem_u32(&bar_acc_empty[acc]));
      }
      if (++acc == ACC_BUFS) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  // No CTA of a cluster leaves while a peer could still write into its shared memory.
  if (p.split > 1) {
    if (!cluster_joined) cluster_wait();
    cluster_sync_all();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    __syncwarp();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace nvfp4
