// NVFP4 block-scaled GEMM for large dense problems: two CTAs on neighbouring SMs work as
// a pair on one 256 x 256 output tile with tcgen05.mma.cta_group::2.
//
// Why a pair: an SM can take in about 64 bytes per clock from L2. A single CTA on a
// 128 x 256 tile needs 54 KB per 256-wide k-tile for 512 clocks of MMA work (105 B/clk),
// so it is bound by that intake, not by the tensor pipe. In a pair each CTA loads its own
// 128 rows of A and only *half* of the B tile (the MMA reads both halves from the two
// CTAs' shared memory): 38 KB per k-tile for the same 512 clocks. No cluster multicast is
// involved: every byte a CTA needs is loaded by that CTA.
//
// Per CTA (448 threads):
//   warp 0      TMA producer: own A rows, own half of B, own SFA atoms, all SFB atoms.
//               The A/B copies of both CTAs complete on the *leader's* full barrier
//               (cp.async.bulk.tensor ... .cta_group::2), which the leader arms for the
//               bytes of both.
//   warps 6-9   scale movers: this CTA's scale atoms -> this CTA's tensor memory (shared ->
//               registers -> tcgen05.st, one warp per 32-lane quarter); the movers of both
//               CTAs arrive on the leader's full barrier (shared::cluster), so a stage is
//               full after nine arrivals: the leader's producer + 8 movers.
//   warp 1      leader CTA only: issues the MMAs (M = 256, N = 256, K = 64 each); its
//               tcgen05.commit is multicast to both CTAs' barriers.
//   warps 2-5,  epilogue, two groups of four warps (one warp per 32-lane quarter of tensor
//   10-13       memory in each). 16-bit output: a group owns half of the CTA's output
//               columns. It reads them out of tensor memory into registers (rounded and
//               packed), hands the accumulator back to the MMA issuer - the next tile's MMAs
//               start here - and only then writes them, 64 columns at a time, into a 16 KB
//               staging box in the 128-byte-swizzled layout and stores the box with one
//               cp.async.bulk.tensor (which clips rows and columns beyond the tensor). The
//               accumulator is single-buffered (tensor memory holds 256 accumulator columns
//               and five stages of scales), so what the MMA issuer waits for per tile is
//               four tcgen05.ld and two conversions per epilogue warp. FP32 output (the
//               dual-GEMM stage) keeps one group and per-thread stores.
// The producer and MMA warps run their loops with all lanes and elect one to issue.
// Tiles are dealt round-robin to the pairs (data parallel, persistent); 5 stages of 38 KB.
#pragma once

#include "nvfp4_gemm_kernel.cuh"

namespace nvfp4 {

__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols)
               : "memory");
}

// Arrive once on the barrier at this shared-memory offset in every CTA of `mask` when all
// tcgen05 operations issued so far by this thread (for the pair) have completed.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(bar),
      "h"(mask)
      : "memory");
}

__device__ __forceinline__ void tc_mma_nvf4_pair(uint32_t tmem_d, uint64_t desc_a,
                                                 uint64_t desc_b, uint32_t idesc,
                                                 uint32_t tmem_sfa, uint32_t tmem_sfb,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], "
      "p;\n\t"
      "}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}

// Tiled copy into this CTA's shared memory whose completion is counted on a barrier that
// may live in the peer CTA of the pair (`cluster_bar` is a shared::cluster address).
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const void* map,
                                                 uint32_t cluster_bar, int c0, int c1, int c2,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(c0), "r"(c1), "r"(c2),
      "l"(policy)
      : "memory");
}

// DUAL: the pair's 256 B rows are a 128-row tile of B1 (loaded by the leader) and the same
// rows of B2 (loaded by the peer); the epilogue writes silu(h1) * h2 for 128 output columns.
template <typename OutT_, bool DUAL_ = false>
struct PairConfig {
  using OutT = OutT_;
  static constexpr bool DUAL = DUAL_;
  static constexpr int OUT_N = DUAL ? 128 : 256;  // output columns per tile
  static constexpr int TILE_M = 256, TILE_N = 256;
  static constexpr int A_BYTES = 128 * 128;       // this CTA's 128 rows x 256 E2M1
  static constexpr int B_BYTES = 128 * 128;       // this CTA's half of the B tile
  static constexpr int SFA_BYTES = 4 * 512;       // this CTA's rows, four k-blocks
  static constexpr int SFB_BYTES = 2 * 4 * 512;   // all 256 B rows
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr int STAGES = 5;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
  static constexpr int SF_STAGE_COLS = 16 + 4 * 8;
  static constexpr int SF_COL = TILE_N;  // after the accumulator's 256 columns
  static constexpr int TMEM_COLS = 512;
  static constexpr int THREADS = 448;
  // 16-bit outputs leave through staged tensor stores; FP32 through per-thread stores.
  static constexpr bool TMA_STORE = sizeof(OutT_) == 2;
  // D quantised to NVFP4 (Fp4Out, the one one-byte tag): per-thread stores of packed codes
  // and scale words, both epilogue groups at work as for 16-bit output.
  static constexpr bool FP4_OUT = sizeof(OutT_) == 1;
  static constexpr bool TWO_GROUPS = TMA_STORE || FP4_OUT;
  static constexpr int STAGING_BYTES = TMA_STORE ? 2 * 16384 : FP4_OUT ? 1024 : 4 * 2048;
  static_assert(SF_COL + STAGES * SF_STAGE_COLS <= TMEM_COLS, "tensor memory exceeded");
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
nvfp4_gemm_pair_kernel(const __grid_constant__ KernelParams p) {
  constexpr int STAGES = Cfg::STAGES;
  using OutT = typename Cfg::OutT;

  extern __shared__ uint8_t dyn_smem[];
  __shared__ alignas(8) uint64_t bar_full[STAGES];     // leader: A/B + scales of both CTAs
  __shared__ alignas(8) uint64_t bar_empty[STAGES];    // each CTA: stage may be refilled
  __shared__ alignas(8) uint64_t bar_sf_full[STAGES];  // each CTA: own scale atoms landed
  __shared__ alignas(8) uint64_t bar_acc_full;         // each CTA: tile accumulated
  __shared__ alignas(8) uint64_t bar_acc_empty;        // leader: both epilogues have drained
  // TMA_STORE: per epilogue group one box of 128 rows x 128 bytes (64 columns), swizzled;
  // otherwise per epilogue warp 32 rows x 64 bytes.
  __shared__ alignas(1024) uint8_t epi_stage[Cfg::STAGING_BYTES];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(dyn_smem) + 1023u) & ~1023u;
  const uint32_t rank = cluster_cta_rank();  // 0 = leader
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 9);
      mbar_init(smem_u32(&bar_empty[s]), 1);
      mbar_init(smem_u32(&bar_sf_full[s]), 1);
    }
    mbar_init(smem_u32(&bar_acc_full), 1);
    // One arrival per epilogue warp of both CTAs (16-bit output: eight warps per CTA).
    mbar_init(smem_u32(&bar_acc_empty), Cfg::TWO_GROUPS ? 16 : 8);
    abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc_pair(smem_u32(&tmem_base_slot), Cfg::TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers and tensor memory exist before anyone uses them
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abort_ptr = &abort_flag;
  grid_dependency_wait();
  grid_launch_dependents();

  const ProblemDesc& pd = p.dense;
  const int pair_tiles_m = (pd.m + 255) / 256;
  const int pair_tiles_n = (pd.n + Cfg::OUT_N - 1) / Cfg::OUT_N;
  const long long tiles = static_cast<long long>(pair_tiles_m) * pair_tiles_n * pd.batches;
  const long long pairs = gridDim.x / 2;
  const long long first_tile = blockIdx.x / 2;

  // Tile index -> (batch, m, n): bands of eight tile rows, as in the single-CTA kernel.
  auto decode = [&](long long t, int& batch, int& m_tile, int& n_tile) {
    const int per_batch = pair_tiles_m * pair_tiles_n;
    batch = static_cast<int>(t / per_batch);
    const int r = static_cast<int>(t % per_batch);
    const int band_tiles = 8 * pair_tiles_n;
    const int band = r / band_tiles;
    const int in_band = r % band_tiles;
    const int height = min(8, pair_tiles_m - band * 8);
    m_tile = band * 8 + in_band % height;
    n_tile = in_band / height;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    {
      const uint64_t pol = l2_policy_evict_last();
      if (elect_one()) {
        prefetch_tensormap(&p.map_a);
        prefetch_tensormap(&p.map_b);
        if constexpr (Cfg::DUAL) prefetch_tensormap(&p.map_b2);
        if constexpr (Cfg::TMA_STORE) prefetch_tensormap(&p.map_d);
      }
      const uint32_t leader_full0 = cluster_map_shared(smem_u32(&bar_full[0]), 0);
      const uint32_t sf_full0 = smem_u32(&bar_sf_full[0]);
      const uint32_t empty0 = smem_u32(&bar_empty[0]);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t stage_smem = smem_base;
      bool ok = true;
      for (long long t = first_tile; ok && t < tiles; t += pairs) {
        int batch, m_tile, n_tile;
        decode(t, batch, m_tile, n_tile);
        const int m0 = m_tile * 256 + static_cast<int>(rank) * 128;
        // Rows of B this CTA loads: its half of the 256-row tile, or (dual) the tile's 128
        // rows of its own B.
        const int n0 = Cfg::DUAL ? n_tile * 128 : n_tile * 256 + static_cast<int>(rank) * 128;
        const void* map_b = (Cfg::DUAL && rank == 1) ? static_cast<const void*>(&p.map_b2)
                                                     : static_cast<const void*>(&p.map_b);
        const int mb = m_tile * 2 + static_cast<int>(rank);  // this CTA's SFA atom row
        const int nb = Cfg::DUAL ? n_tile : n_tile * 2;       // first of the tile's SFB atom rows
        const bool sfa_valid = mb < pd.sf_mb;
        const uint8_t* sfa_src =
            pd.sfa + (static_cast<long long>(batch) * pd.sf_mb + mb) * pd.sf_kb * 512;
        const uint8_t* sfb_src0 =
            pd.sfb + (static_cast<long long>(batch) * pd.sf_nb + nb) * pd.sf_kb * 512;
        // Second scale atom row: the next 128 rows of B, or (dual) the same rows of B2.
        const uint8_t* sfb_src1 =
            Cfg::DUAL ? pd.sfb2 + (static_cast<long long>(batch) * pd.sf_nb + nb) * pd.sf_kb * 512
                      : sfb_src0 + static_cast<long long>(pd.sf_kb) * 512;
        const bool sfb1_valid = Cfg::DUAL || nb + 1 < pd.sf_nb;
        int atoms_left = pd.sf_kb;
        int kbyte = 0;
        for (int kt = 0; kt < pd.k_tiles; ++kt) {
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1u, abort_ptr)) {
            report_failure(p, abort_ptr, kStatusProducerTimeout);
            ok = false;
            break;
          }
          const uint32_t sf_bytes =
              atoms_left >= 4 ? 2048u : static_cast<uint32_t>(atoms_left) * 512u;
          const uint32_t a_dst = stage_smem;
          const uint32_t b_dst = a_dst + Cfg::A_BYTES;
          const uint32_t sfa_dst = b_dst + Cfg::B_BYTES;
          const uint32_t sfb_dst = sfa_dst + Cfg::SFA_BYTES;
          const uint32_t sf_bar = sf_full0 + 8 * stage;
          if (elect_one()) {
            mbar_expect_tx(sf_bar,
                           sf_bytes * ((sfa_valid ? 1u : 0u) + 1u + (sfb1_valid ? 1u : 0u)));
            if (sfa_valid) bulk_load(sfa_dst, sfa_src, sf_bytes, sf_bar, pol);
            bulk_load(sfb_dst, sfb_src0, sf_bytes, sf_bar, pol);
            if (sfb1_valid) bulk_load(sfb_dst + 2048, sfb_src1, sf_bytes, sf_bar, pol);
            // The leader arms its full barrier for the A and B bytes of both CTAs.
            if (leader) {
              mbar_expect_tx(smem_u32(&bar_full[stage]), 2u * (Cfg::A_BYTES + Cfg::B_BYTES));
            }
            tma_load_3d_pair(a_dst, &p.map_a, leader_full0 + 8 * stage, kbyte, m0, batch, pol);
            tma_load_3d_pair(b_dst, map_b, leader_full0 + 8 * stage, kbyte, n0, batch, pol);
          }
          __syncwarp();
          sfa_src += 2048;
          sfb_src0 += 2048;
          sfb_src1 += 2048;
          atoms_left -= 4;
          kbyte += 128;
          stage_smem += Cfg::STAGE_BYTES;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
            stage_smem = smem_base;
          }
        }
      }
      if (!ok || *abort_ptr != 0) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader)
    if (leader) {
      constexpr uint32_t idesc = nvf4_instr_desc(256, 256);
      constexpr uint32_t kHiOperand = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t kStage16 = Cfg::STAGE_BYTES >> 4;
      const uint32_t lo_a0 = ((smem_base >> 4) & 0x3FFFu) | (1u << 16);
      const uint32_t lo_b0 = lo_a0 + (Cfg::A_BYTES >> 4);
      const uint32_t full0 = smem_u32(&bar_full[0]);
      const uint32_t empty0 = smem_u32(&bar_empty[0]);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t stage16 = 0;
      uint32_t t_sf = tmem_base + Cfg::SF_COL;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (long long t = first_tile; ok && t < tiles; t += pairs) {
        if (!mbar_wait(smem_u32(&bar_acc_empty), acc_phase ^ 1u, abort_ptr)) {
          report_failure(p, abort_ptr, kStatusMmaAccumTimeout);
          break;
        }
        tc_fence_after_sync();
        int atoms_left = pd.sf_kb;
        uint32_t accumulate = 0;
        for (int kt = 0; kt < pd.k_tiles; ++kt) {
          if (!mbar_wait(full0 + 8 * stage, phase, abort_ptr)) {
            report_failure(p, abort_ptr, kStatusMmaInputTimeout);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t lo_a = lo_a0 + stage16;
          const uint32_t lo_b = lo_b0 + stage16;
          if (elect_one()) {
            if (atoms_left >= 4) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                tc_mma_nvf4_pair(tmem_base, pack_desc(lo_a + 2 * j, kHiOperand),
                                 pack_desc(lo_b + 2 * j, kHiOperand), idesc, t_sf + 4 * j,
                                 t_sf + 16 + 8 * j, j > 0 ? 1u : accumulate);
              }
            } else {
              const int mmas = min(4, atoms_left);
              for (int j = 0; j < mmas; ++j) {
                tc_mma_nvf4_pair(tmem_base, pack_desc(lo_a + 2 * j, kHiOperand),
                                 pack_desc(lo_b + 2 * j, kHiOperand), idesc, t_sf + 4 * j,
                                 t_sf + 16 + 8 * j, j > 0 ? 1u : accumulate);
              }
            }
            tc_commit_pair(empty0 + 8 * stage, 3);
          }
          __syncwarp();
          accumulate = 1;
          atoms_left -= 4;
          stage16 += kStage16;
          t_sf += Cfg::SF_STAGE_COLS;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
            stage16 = 0;
            t_sf = tmem_base + Cfg::SF_COL;
          }
        }
        if (!ok) break;
        if (elect_one()) tc_commit_pair(smem_u32(&bar_acc_full), 3);
        __syncwarp();
        acc_phase ^= 1u;
      }
    }
  } else if (warp >= 6 && warp < 10) {
    // ------------------------------------------------------------------ scale movers
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t sf_full0 = smem_u32(&bar_sf_full[0]);
    const uint32_t leader_full0 = cluster_map_shared(smem_u32(&bar_full[0]), 0);
    const uint32_t row_off = static_cast<uint32_t>(lane) * 16u;
    int stage = 0;
    uint32_t phase = 0;
    uint32_t sf_smem = smem_base + Cfg::A_BYTES + Cfg::B_BYTES;
    uint32_t t_sf = tmem_base + lane_base + Cfg::SF_COL;
    bool ok = true;
    for (long long t = first_tile; ok && t < tiles; t += pairs) {
      int atoms_left = pd.sf_kb;
      for (int kt = 0; kt < pd.k_tiles; ++kt) {
        if (!mbar_wait(sf_full0 + 8 * stage, phase, abort_ptr)) {
          report_failure(p, abort_ptr, kStatusScaleTimeout);
          ok = false;
          break;
        }
        const int atoms = min(4, atoms_left);
        if (atoms == 4) {
          // All twelve loads first, then the twelve stores: the loads overlap.
          uint4 va[4], vb0[4], vb1[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            va[j] = ld_shared_v4(sf_smem + 512 * j + row_off);
            vb0[j] = ld_shared_v4(sf_smem + Cfg::SFA_BYTES + 512 * j + row_off);
            vb1[j] = ld_shared_v4(sf_smem + Cfg::SFA_BYTES + 2048 + 512 * j + row_off);
          }
          // 48 contiguous columns: A's k-blocks at 4j, B's at 16 + 8j (+4 for atom row 1).
          tmem_store_16(t_sf, va[0], va[1], va[2], va[3]);
          tmem_store_16(t_sf + 16, vb0[0], vb1[0], vb0[1], vb1[1]);
          tmem_store_16(t_sf + 32, vb0[2], vb1[2], vb0[3], vb1[3]);
        } else {
          for (int j = 0; j < atoms; ++j) {
            tmem_store_4(t_sf + 4 * j, ld_shared_v4(sf_smem + 512 * j + row_off));
            tmem_store_4(t_sf + 16 + 8 * j,
                         ld_shared_v4(sf_smem + Cfg::SFA_BYTES + 512 * j + row_off));
            tmem_store_4(t_sf + 16 + 8 * j + 4,
                         ld_shared_v4(sf_smem + Cfg::SFA_BYTES + 2048 + 512 * j + row_off));
          }
        }
        tmem_store_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_peer(leader_full0 + 8 * stage);
        atoms_left -= 4;
        sf_smem += Cfg::STAGE_BYTES;
        t_sf += Cfg::SF_STAGE_COLS;
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
          sf_smem = smem_base + Cfg::A_BYTES + Cfg::B_BYTES;
          t_sf = tmem_base + lane_base + Cfg::SF_COL;
        }
      }
    }
  } else if (Cfg::FP4_OUT) {
    // ------------------------------------------------------------------ epilogue, NVFP4 D
    // Two groups of four warps, each owning half of the tile's output columns; a thread owns
    // one row of them. Per 32 columns: two block scales and 32 codes with the quantiser
    // kernel's arithmetic (nvfp4_block_codes), so the bytes equal quantising the FP32 result.
    // The accumulator goes back to the MMA issuer once the group's last chunk is in
    // registers; packed codes (16 bytes per 32 columns) and scale words (four scale bytes per
    // 64 columns, contiguous in the blocked layout) are stored by the thread itself.
    if constexpr (Cfg::FP4_OUT) {
      const int group = warp >= 10 ? 1 : 0;
      const int quarter = warp & 3;
      const int row = quarter * 32 + lane;
      const float alpha = p.alpha != nullptr ? __ldg(p.alpha) : 1.0f;
      const uint32_t leader_acc_empty = cluster_map_shared(smem_u32(&bar_acc_empty), 0);
      constexpr int GROUP_COLS = Cfg::DUAL ? 64 : 128;
      constexpr int CHUNKS = GROUP_COLS / 32;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(group * GROUP_COLS);
      uint32_t acc_phase = 0;
      for (long long t = first_tile; t < tiles; t += pairs) {
        int batch, m_tile, n_tile;
        decode(t, batch, m_tile, n_tile);
        if (!mbar_wait(smem_u32(&bar_acc_full), acc_phase, abort_ptr)) {
          report_failure(p, abort_ptr, kStatusEpilogueTimeout);
          break;
        }
        tc_fence_after_sync();
        const int row_block = m_tile * 2 + static_cast<int>(rank);  // 128-row block of D
        const int grow = row_block * 128 + row;
        const int col0 = n_tile * Cfg::OUT_N + group * GROUP_COLS;
        uint32_t words[CHUNKS][4];
        uint32_t scale_word[CHUNKS / 2];
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
          uint32_t r1[32];
          tmem_load_32(taddr + c * 32, r1);
          if constexpr (Cfg::DUAL) {
            uint32_t r2[32];
            tmem_load_32(taddr + 128 + c * 32, r2);
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
          if (c == CHUNKS - 1) {
            // Everything this warp needs has left tensor memory: hand the accumulator back.
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_peer(leader_acc_empty);
          }
          if (c % 2 == 0) scale_word[c / 2] = 0;
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
            scale_word[c / 2] |= bits << (8 * (2 * (c % 2) + blk));
            const uint2 codes =
                scale > 0.0f ? nvfp4_block_codes(v, amax, scale) : make_uint2(0u, 0u);
            words[c][2 * blk] = codes.x;
            words[c][2 * blk + 1] = codes.y;
          }
        }
        if (grow < pd.m) {
          uint8_t* d_row = static_cast<uint8_t*>(pd.d) +
                           (static_cast<long long>(batch) * pd.m + grow) * (pd.n / 2);
          const int sf_cb = (pd.n + 63) / 64;
          uint8_t* sf_row = pd.sfd +
                            (static_cast<long long>(batch) * pd.sf_mb + row_block) * sf_cb * 512 +
                            (row % 32) * 16 + ((row / 32) % 4) * 4;
#pragma unroll
          for (int c = 0; c < CHUNKS; ++c) {
            if (col0 + c * 32 < pd.n) {
              *reinterpret_cast<uint4*>(d_row + (col0 + c * 32) / 2) =
                  make_uint4(words[c][0], words[c][1], words[c][2], words[c][3]);
            }
          }
#pragma unroll
          for (int h = 0; h < CHUNKS / 2; ++h) {
            if (col0 + h * 64 < pd.n) {
              *reinterpret_cast<uint32_t*>(sf_row + static_cast<long long>((col0 + h * 64) / 64) * 512) =
                  scale_word[h];
            }
          }
        }
        acc_phase ^= 1u;
      }
    }
  } else if (Cfg::TMA_STORE) {
    // ------------------------------------------------------------------ epilogue, 16-bit D
    if constexpr (Cfg::TMA_STORE) {
      const int group = warp >= 10 ? 1 : 0;
      const int quarter = warp & 3;
      const int row = quarter * 32 + lane;
      const bool issuer = (warp == 2 || warp == 10) && lane == 0;  // one thread per group
      const uint32_t barrier_id = 1u + static_cast<uint32_t>(group);
      const float alpha = p.alpha != nullptr ? __ldg(p.alpha) : 1.0f;
      const uint32_t leader_acc_empty = cluster_map_shared(smem_u32(&bar_acc_empty), 0);
      // The group's accumulator columns: half of the 256 (dual: the group's 64 columns of h1
      // at 64 g and of h2 at 128 + 64 g).
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(group) * (Cfg::DUAL ? 64u : 128u);
      const uint32_t box = smem_u32(epi_stage) + static_cast<uint32_t>(group) * 16384u;
      // Row `row` of the box: eight 16-byte pieces, piece j at position j ^ (row % 8).
      const uint32_t box_row = box + static_cast<uint32_t>(row) * 128u;
      const uint32_t swizzle = static_cast<uint32_t>(row) & 7u;
      constexpr int BOXES = Cfg::DUAL ? 1 : 2;  // 64-column boxes per group and tile
      uint32_t acc_phase = 0;
      for (long long t = first_tile; t < tiles; t += pairs) {
        int batch, m_tile, n_tile;
        decode(t, batch, m_tile, n_tile);
        if (!mbar_wait(smem_u32(&bar_acc_full), acc_phase, abort_ptr)) {
          report_failure(p, abort_ptr, kStatusEpilogueTimeout);
          break;
        }
        tc_fence_after_sync();
        uint32_t packed[BOXES][32];
#pragma unroll
        for (int b = 0; b < BOXES; ++b) {
          uint32_t r1[32], r2[32];
          if constexpr (Cfg::DUAL) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              tmem_load_32(taddr + 32 * half, r1);
              tmem_load_32(taddr + 128 + 32 * half, r2);
              tmem_load_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                packed[b][16 * half + i] = pack_pair<OutT>(
                    silu_f32(__uint_as_float(r1[2 * i]) * alpha) *
                        (__uint_as_float(r2[2 * i]) * alpha),
                    silu_f32(__uint_as_float(r1[2 * i + 1]) * alpha) *
                        (__uint_as_float(r2[2 * i + 1]) * alpha));
              }
            }
          } else {
            tmem_load_32(taddr + 64 * b, r1);
            tmem_load_32(taddr + 64 * b + 32, r2);
            tmem_load_wait();
            float v1[32], v2[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              v1[i] = __uint_as_float(r1[i]) * alpha;
              v2[i] = __uint_as_float(r2[i]) * alpha;
            }
            unshuffle_columns(v1, p.b_shuffle);
            unshuffle_columns(v2, p.b_shuffle);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              packed[b][i] = pack_pair<OutT>(v1[2 * i], v1[2 * i + 1]);
              packed[b][16 + i] = pack_pair<OutT>(v2[2 * i], v2[2 * i + 1]);
            }
          }
        }
        // Everything this warp needs has left tensor memory: hand the accumulator back.
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_peer(leader_acc_empty);
        const int row0 = m_tile * 256 + static_cast<int>(rank) * 128;
        const int col0 = n_tile * Cfg::OUT_N + group * (Cfg::DUAL ? 64 : 128);
#pragma unroll
        for (int b = 0; b < BOXES; ++b) {
          // The box is free once the previous store has read it.
          if (issuer) bulk_wait_group_read_all();
          named_barrier_sync(barrier_id, 128);
#pragma unroll
          for (uint32_t j = 0; j < 8; ++j) {
            st_shared_v4(box_row + ((j ^ swizzle) << 4), packed[b][4 * j], packed[b][4 * j + 1],
                         packed[b][4 * j + 2], packed[b][4 * j + 3]);
          }
          fence_proxy_async_shared();
          named_barrier_sync(barrier_id, 128);
          if (issuer && row0 < pd.m && col0 + 64 * b < pd.n) {
            tma_store_3d(&p.map_d, box, col0 + 64 * b, row0, batch);
            bulk_commit_group();
          }
        }
        acc_phase ^= 1u;
      }
      // The staging box must outlive the reads of the last stores.
      if (issuer) bulk_wait_group_read_all();
    }
  } else if (warp >= 2 && warp < 6) {
    // ------------------------------------------------------------------ epilogue, FP32 D
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const float alpha = p.alpha != nullptr ? __ldg(p.alpha) : 1.0f;
    const uint32_t leader_acc_empty = cluster_map_shared(smem_u32(&bar_acc_empty), 0);
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    uint32_t acc_phase = 0;
    for (long long t = first_tile; t < tiles; t += pairs) {
      int batch, m_tile, n_tile;
      decode(t, batch, m_tile, n_tile);
      if (!mbar_wait(smem_u32(&bar_acc_full), acc_phase, abort_ptr)) {
        report_failure(p, abort_ptr, kStatusEpilogueTimeout);
        break;
      }
      tc_fence_after_sync();
      const int grow = m_tile * 256 + static_cast<int>(rank) * 128 + row;
      const int n0 = n_tile * Cfg::OUT_N;
      OutT* out_row = reinterpret_cast<OutT*>(pd.d) +
                      (static_cast<long long>(batch) * pd.m + grow) * pd.n;
      OutT* out_block = out_row - static_cast<long long>(lane) * pd.n;
      const int rows_valid = pd.m - (grow - lane);
      const uint32_t stage_smem = smem_u32(epi_stage) + static_cast<uint32_t>(quarter) * 2048u;
#pragma unroll 1
      for (int c = 0; c < 8; ++c) {
        uint32_t r1[32];
        float v[32];
        tmem_load_32(taddr + c * 32, r1);
        tmem_load_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r1[i]) * alpha;
        if constexpr (!Cfg::DUAL) unshuffle_columns(v, p.b_shuffle);
        if (c == 7) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_peer(leader_acc_empty);
        }
        store_warp_chunk<OutT>(stage_smem, out_block, out_row, grow < pd.m, n0 + c * 32, pd.n,
                               rows_valid, lane, v);
      }
      acc_phase ^= 1u;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees tensor memory or exits while the pair is in use
  if (warp == 1) {
    tc_fence_after_sync();
    __syncwarp();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace nvfp4
