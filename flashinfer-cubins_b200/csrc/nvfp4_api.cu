// Host side of the C ABI declared in include/nvfp4_b200.h: argument validation,
// schedule choice, tensor-map encoding, workspace layout and launches. No function
// here allocates device memory, throws, or synchronises except nvfp4_plan_status.

#include "../../include/nvfp4_b200.h"

#include <algorithm>
#include <climits>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstddef>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include <cuda.h>
#include <cuda_runtime.h>

#include "nvfp4_gemm_kernel.cuh"
#include "nvfp4_gemm_pair_kernel.cuh"
#include "nvfp4_glue_kernels.cuh"

using namespace nvfp4;

namespace {

thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

int fail_cuda(cudaError_t err, const char* what) {
  // Clear the sticky-free error so that later calls do not see it again.
  cudaGetLastError();
  return fail(static_cast<int>(err), "%s: %s", what, cudaGetErrorString(err));
}

#define CUDA_TRY(expr)                                   \
  do {                                                   \
    cudaError_t err__ = (expr);                          \
    if (err__ != cudaSuccess) return fail_cuda(err__, #expr); \
  } while (0)

struct DeviceGuard {
  int saved = -1;
  bool active = false;
  // Always sets the device, even when it is the current one: in a host thread that has made
  // no CUDA call yet this is what binds the device's primary context to the thread, which
  // driver entry points such as cuTensorMapEncodeTiled need.
  cudaError_t enter(int device) {
    cudaError_t e = cudaGetDevice(&saved);
    if (e != cudaSuccess) return e;
    e = cudaSetDevice(device);
    if (e != cudaSuccess) return e;
    active = saved != device;
    return cudaSuccess;
  }
  ~DeviceGuard() {
    if (active) cudaSetDevice(saved);
  }
};

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled, looked up through the runtime so that the library has no
// link-time dependency on libcuda (it must load on machines without a driver).
int get_encoder(EncodeTiledFn* out) {
  static std::mutex mu;
  static EncodeTiledFn cached = nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (cached == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t err =
        cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (err != cudaSuccess) return fail_cuda(err, "cudaGetDriverEntryPoint");
    if (qres != cudaDriverEntryPointSuccess || fn == nullptr) {
      return fail(NVFP4_E_UNSUPPORTED_DEVICE, "driver has no cuTensorMapEncodeTiled");
    }
    cached = reinterpret_cast<EncodeTiledFn>(fn);
  }
  *out = cached;
  return 0;
}

// Packed E2M1 operand [batches][rows][k/2] bytes as a rank-3 uint8 tensor with a
// 128-byte (256-element) x box_rows box, 128-byte swizzle, zero fill out of bounds.
int encode_operand_map(CUtensorMap* map, const void* ptr, int rows, int k, int batches,
                       int box_rows) {
  EncodeTiledFn encode = nullptr;
  if (int rc = get_encoder(&encode)) return rc;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(k) / 2;
  // The map describes exactly the caller's tensor. (Loads through the map of a tensor below
  // 128 KiB are slower on current drivers, and declaring never-addressed extra batches up to
  // that size makes them fast again - but the copy engine then touches memory inside the
  // declared extent beyond the real tensor, which faults when that memory is not mapped.)
  const cuuint64_t declared_batches = static_cast<cuuint64_t>(batches);
  const cuuint64_t dims[3] = {row_bytes, static_cast<cuuint64_t>(rows), declared_batches};
  const cuuint64_t strides[2] = {row_bytes, row_bytes * static_cast<cuuint64_t>(rows)};
  const cuuint32_t box[3] = {128u, static_cast<cuuint32_t>(box_rows), 1u};
  const cuuint32_t elem_strides[3] = {1u, 1u, 1u};
  CUresult res = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims,
                        strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) {
    return fail(static_cast<int>(res),
                "cuTensorMapEncodeTiled failed (%d) for rows=%d k=%d batches=%d box_rows=%d",
                static_cast<int>(res), rows, k, batches, box_rows);
  }
  return 0;
}

// 16-bit output D [batches][m][n] as a rank-3 tensor of 16-bit elements with a box of 64
// columns (128 bytes) x 128 rows and 128-byte swizzle: what the 2-CTA kernel's epilogue
// stores from its staging boxes. Needs rows of D 16-byte aligned (n a multiple of 8).
int encode_output_map(CUtensorMap* map, void* ptr, int m, int n, int batches) {
  EncodeTiledFn encode = nullptr;
  if (int rc = get_encoder(&encode)) return rc;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(n) * 2;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(m),
                              static_cast<cuuint64_t>(batches)};
  const cuuint64_t strides[2] = {row_bytes, row_bytes * static_cast<cuuint64_t>(m)};
  const cuuint32_t box[3] = {64u, 128u, 1u};
  const cuuint32_t elem_strides[3] = {1u, 1u, 1u};
  CUresult res = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, ptr, dims, strides, box,
                        elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) {
    return fail(static_cast<int>(res), "cuTensorMapEncodeTiled failed (%d) for D m=%d n=%d batches=%d",
                static_cast<int>(res), m, n, batches);
  }
  return 0;
}

int ceil_div(int a, int b) { return (a + b - 1) / b; }
size_t round_up(size_t a, size_t b) { return (a + b - 1) / b * b; }

enum PlanKind { kDense = 0, kDual = 1, kGrouped = 2 };

// Whether large dense GEMMs (at least two 256 x 256 tiles per SM) use the 2-CTA kernel
// without being asked to: measured 209 us against 232 us single-CTA on 8192^3.
constexpr bool kPairByDefault = true;

using KernelFn = void (*)(const KernelParams);

struct KernelChoice {
  KernelFn fn;
  int smem_bytes;
  int stages;
  int threads;
  int stage_bytes;
};

template <class Cfg>
KernelChoice make_choice() {
  return KernelChoice{&nvfp4_gemm_kernel<Cfg>, Cfg::SMEM_BYTES, Cfg::STAGES, Cfg::THREADS,
                      Cfg::STAGE_BYTES};
}

template <class Cfg>
KernelChoice make_pair_choice() {
  return KernelChoice{&nvfp4_gemm_pair_kernel<Cfg>, Cfg::SMEM_BYTES, Cfg::STAGES, Cfg::THREADS,
                      Cfg::STAGE_BYTES};
}

// kind, out_kind, tile_n -> kernel instantiation. Returns fn == nullptr if absent.
KernelChoice select_kernel(int kind, int out_kind, int tile_n) {
  if (kind == kDual && out_kind == NVFP4_OUT_FP4) {
    switch (tile_n) {
      case 128: return make_choice<GemmConfig<128, true, Fp4Out, false>>();
      case 256: return make_choice<GemmConfig<256, true, Fp4Out, false>>();
    }
    return KernelChoice{nullptr, 0, 0, 0, 0};
  }
  if (kind == kDual) {
    switch (tile_n) {
      case 128: return make_choice<GemmConfig<128, true, __half, false>>();
      case 256: return make_choice<GemmConfig<256, true, __half, false>>();
    }
    return KernelChoice{nullptr, 0, 0, 0, 0};
  }
  if (kind == kGrouped && out_kind == NVFP4_OUT_FP4) {  // grouped dual GEMM, NVFP4 output
    switch (tile_n) {
      case 128: return make_choice<GemmConfig<128, true, Fp4Out, true>>();
      case 256: return make_choice<GemmConfig<256, true, Fp4Out, true>>();
    }
    return KernelChoice{nullptr, 0, 0, 0, 0};
  }
  if (kind == kGrouped) {
    switch (tile_n) {
      case 64: return make_choice<GemmConfig<64, false, __half, true>>();
      case 128: return make_choice<GemmConfig<128, false, __half, true>>();
      case 256: return make_choice<GemmConfig<256, false, __half, true>>();
    }
  } else if (out_kind == NVFP4_OUT_FP4) {
    switch (tile_n) {
      case 64: return make_choice<GemmConfig<64, false, Fp4Out, false>>();
      case 128: return make_choice<GemmConfig<128, false, Fp4Out, false>>();
      case 256: return make_choice<GemmConfig<256, false, Fp4Out, false>>();
    }
  } else if (out_kind == NVFP4_OUT_BF16) {
    switch (tile_n) {
      case 64: return make_choice<GemmConfig<64, false, __nv_bfloat16, false>>();
      case 128: return make_choice<GemmConfig<128, false, __nv_bfloat16, false>>();
      case 256: return make_choice<GemmConfig<256, false, __nv_bfloat16, false>>();
    }
  } else if (out_kind == NVFP4_OUT_F16) {
    switch (tile_n) {
      case 64: return make_choice<GemmConfig<64, false, __half, false>>();
      case 128: return make_choice<GemmConfig<128, false, __half, false>>();
      case 256: return make_choice<GemmConfig<256, false, __half, false>>();
    }
  } else {
    switch (tile_n) {
      case 64: return make_choice<GemmConfig<64, false, float, false>>();
      case 128: return make_choice<GemmConfig<128, false, float, false>>();
      case 256: return make_choice<GemmConfig<256, false, float, false>>();
    }
  }
  return KernelChoice{nullptr, 0, 0, 0, 0};
}

}  // namespace

struct nvfp4_plan {
  int kind = kDense;
  int device = 0;
  int out_kind = NVFP4_OUT_F16;
  int sm_count = 0;
  int tile_n = 128;   // MMA N
  int out_tile_n = 128;
  int schedule = 1;   // 1 data parallel, 2 stream-K, 3 cluster split-K
  int ctas = 1;
  int split = 1;      // cluster size of schedule 3
  bool pair = false;  // 2-CTA kernel: 256 x 256 tiles, one cluster of two CTAs per tile
  int b_shuffle = 0;  // 16 / 32: B's rows are in FlashInfer's epilogue-shuffled order
  int maps_per_group = 2;  // grouped: tensor maps per group in the workspace (dual: 3)
  double estimate_us = 0.0;  // the time model's figure for the chosen schedule (mainloop + tail)
  int ring_stages = 0;       // pipeline stages the kernel cycles through
  int inbox_offset = -1;     // cluster split-K: byte offset of the peers' inbox, or -1
  KernelChoice kernel{};
  std::vector<ProblemDesc> problems;  // shapes and tile counts; operand pointers stay null
  long long total_tiles = 0, total_units = 0;
  long long slot_floats = 0;
  size_t off_counters = 0, off_table = 0, off_maps = 0, off_partials = 0, ws_bytes = 0;
  // Routed groups (nvfp4_moe_plan_create): every group's row count is decided on the device
  // before each launch; the groups share A, D and scale buffers of `routed_rows` rows.
  bool routed = false;
  int routed_rows = 0;
  size_t off_routed = 0;  // RoutedHeader in the workspace
  // Everything above is fixed once the plan has been created. The only state a launch may
  // touch is this cache of encoded kernel parameters (tensor maps are ~2 us each to encode),
  // keyed by the operand and workspace addresses and guarded by `mutex`; a launch copies its
  // entry out under the lock and launches from the copy, so concurrent launches of one plan
  // from several threads and streams are safe.
  struct BoundParams {
    const void* key[10];
    KernelParams params;
    unsigned long long last_use;
  };
  static constexpr size_t kMaxBound = 16;
  mutable std::mutex mutex;
  mutable std::vector<BoundParams> bound;
  mutable unsigned long long use_counter = 0;
  mutable bool group_bound = false;  // grouped: a workspace has been bound at least once
};

namespace {

int env_int(const char* name, int fallback) {
  const char* v = std::getenv(name);
  if (v == nullptr || *v == '\0') return fallback;
  return std::atoi(v);
}

// Time of one k-tile step of one CTA in microseconds by tile width (see finish_schedule).
double kStepUs(int tile_n) { return tile_n <= 64 ? 0.30 : tile_n <= 128 ? 0.38 : 0.52; }
constexpr double kPairStepUs = 0.44;  // a CTA of a pair on its half of a 256 x 256 tile

// How many clusters of `size` CTAs of this kernel the device can hold at once (0 if the
// query fails). Clusters must fit inside one GPC, so this is less than SMs / size.
int max_active_clusters(int device, const KernelChoice& kernel, int size) {
  if (kernel.fn == nullptr) return 0;
  DeviceGuard guard;
  if (guard.enter(device) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  const void* fn = reinterpret_cast<const void*>(kernel.fn);
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kernel.smem_bytes) !=
      cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = static_cast<unsigned int>(size);
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = 1;
  cudaLaunchConfig_t launch = {};
  launch.gridDim = dim3(static_cast<unsigned int>(size), 1, 1);
  launch.blockDim = dim3(static_cast<unsigned int>(kernel.threads), 1, 1);
  launch.dynamicSmemBytes = static_cast<size_t>(kernel.smem_bytes);
  launch.attrs = &attribute;
  launch.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, fn, &launch) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return clusters;
}

// Tile width, schedule and grid for a list of problems whose tile counts are already
// filled for every candidate width. Data parallel when whole tiles fill the SMs
// evenly enough; otherwise stream-K over (tile, k-tile) units.
void finish_schedule(nvfp4_plan* plan, const nvfp4_config* config) {
  long long tiles = 0, units = 0;
  for (ProblemDesc& pd : plan->problems) {
    pd.tile_begin = tiles;
    pd.unit_begin = units;
    const long long t = static_cast<long long>(pd.tiles_m) * pd.tiles_n * pd.batches;
    tiles += t;
    units += t * pd.k_tiles;
  }
  plan->total_tiles = tiles;
  plan->total_units = units;

  const int sms = plan->sm_count;
  int schedule = config != nullptr && config->schedule > 0 ? config->schedule
                                                            : env_int("NVFP4_SCHEDULE", 0);
  int ctas = config != nullptr && config->ctas > 0 ? config->ctas : env_int("NVFP4_CTAS", 0);
  if (ctas > sms) ctas = sms;

  // Cluster split-K (dense and dual GEMM): `split` CTAs of a cluster share a tile's K and
  // reduce through peer shared memory. Candidates are the power-of-two cluster sizes
  // that keep at least one k-tile per CTA, own 32-column multiples, and fit the SMs.
  int split = 1;
  if (plan->kind != kGrouped && plan->problems.size() == 1 && tiles < sms) {
    const int k_tiles = plan->problems[0].k_tiles;
    const int forced = env_int("NVFP4_SPLIT", 0);
    const KernelChoice kernel = select_kernel(plan->kind, plan->out_kind, plan->tile_n);
    for (int s = 2; s <= 8; s *= 2) {
      if (tiles * s > sms || s > k_tiles || (plan->out_tile_n / s) % 32 != 0) break;
      // All clusters must be resident at once, or the grid runs in two waves.
      const int resident = max_active_clusters(plan->device, kernel, s);
      if (resident > 0 && tiles > resident) break;
      if (forced == 0 || s <= forced) split = s;
    }
  }
  if (schedule == 3 && split < 2) schedule = 0;
  {
    // The time model (microseconds, without the per-launch constant). Measured on B200: a
    // k-tile step of one CTA takes about 0.30 / 0.38 / 0.52 us with 64 / 128 / 256-column
    // tiles once the pipeline is full (the shared-memory pipe: TMA writes + MMA operand
    // reads + scale reads), whatever the schedule; a 256-column tile's epilogue (~1.2 us)
    // is not overlapped because its accumulator is single-buffered; finishing split tiles
    // through the workspace costs 8 us and up at the end of the kernel, through a
    // cluster's shared memory 3.5 us and up (below).
    const double step_us = kStepUs(plan->tile_n);
    const double tile_tail_us = plan->tile_n > 128 ? 1.2 : 0.0;
    const double k_per_tile = static_cast<double>(units) / static_cast<double>(tiles);
    const long long waves = (tiles + sms - 1) / sms;
    const double t_whole = static_cast<double>(waves) * (k_per_tile * step_us + tile_tail_us);
    const long long sk_ctas = std::min<long long>(sms, std::max<long long>(tiles, units / 4));
    // The workspace fix-up moves whole FP32 tiles and the last CTA of a tile adds the
    // others' partials one after the other: with 128-column tiles about 6 us for two
    // contributors per tile and ~2.2 us for every further one (39 us measured with sixteen),
    // four times that with 256-column tiles.
    const double units_per_cta = static_cast<double>(units) / static_cast<double>(sk_ctas);
    const double contributors = std::ceil(k_per_tile / units_per_cta) + 1.0;
    const double fixup_us = (plan->tile_n > 128 ? 4.0 : 1.0) * (4.0 + 2.2 * (contributors - 1.0));
    const double t_stream = units_per_cta * step_us + fixup_us;
    double t_cluster = 1e30;
    if (split >= 2) {
      const int k_tiles = plan->problems[0].k_tiles;
      // Against a data-parallel launch of the same tiles a cluster launch measured 2.4-5 us
      // dearer for pairs and more for larger clusters and wider tiles (cluster launch and
      // barriers, the exchange itself, fewer idle SMs for the next launch's prologue).
      const double exchange_us = (split == 2 ? 3.5 : split == 4 ? 5.0 : 8.0) *
                                 (plan->tile_n > 128 ? 1.5 : 1.0);
      t_cluster = static_cast<double>((k_tiles + split - 1) / split) * step_us + tile_tail_us +
                  exchange_us;
    }
    if (schedule != 1 && schedule != 2 && schedule != 3) {
      schedule = 1;
      double best = t_whole;
      if (t_stream < best && units > tiles) {
        schedule = 2;
        best = t_stream;
      }
      if (t_cluster < best) schedule = 3;
    }
    plan->estimate_us = schedule == 1 ? t_whole : schedule == 2 ? t_stream : t_cluster;
  }
  if (ctas <= 0) {
    if (schedule == 1) {
      ctas = static_cast<int>(std::min<long long>(sms, tiles));
    } else {
      const long long by_units = std::max<long long>(tiles, units / 4);
      ctas = static_cast<int>(std::min<long long>(sms, std::max<long long>(1, by_units)));
    }
  }
  if (schedule == 1) ctas = static_cast<int>(std::min<long long>(ctas, tiles));
  if (schedule == 2) ctas = static_cast<int>(std::min<long long>(ctas, units));
  if (schedule == 3) ctas = static_cast<int>(tiles) * split;
  if (ctas < 1) ctas = 1;
  plan->schedule = schedule;
  plan->ctas = ctas;
  plan->split = schedule == 3 ? split : 1;

  // Workspace: [status 256 B][counters][group table][group maps][partials].
  size_t off = 256;
  plan->off_counters = off;
  off += round_up(static_cast<size_t>(tiles) * sizeof(unsigned int), 256);
  plan->off_table = off;
  if (plan->kind == kGrouped) {
    off += round_up(plan->problems.size() * sizeof(ProblemDesc), 256);
    plan->off_maps = off;
    off += round_up(plan->problems.size() * plan->maps_per_group * sizeof(CUtensorMap), 256);
  } else {
    plan->off_maps = off;
  }
  plan->off_partials = off;
  plan->slot_floats = 128ll * plan->tile_n;
  if (schedule == 2) {
    off += static_cast<size_t>(2) * ctas * plan->slot_floats * sizeof(float);
  }
  // (Cluster split-K exchanges partials through shared memory: no slots.)
  plan->ws_bytes = off;
}

int fill_problem(ProblemDesc* pd, int m, int n, int k, int batches, int out_tile_n) {
  std::memset(pd, 0, sizeof(*pd));
  pd->m = m;
  pd->n = n;
  pd->k = k;
  pd->batches = batches;
  pd->tiles_m = ceil_div(m, 128);
  pd->tiles_n = ceil_div(n, out_tile_n);
  pd->k_tiles = ceil_div(k, 256);
  pd->sf_kb = ceil_div(k, 64);
  pd->sf_mb = ceil_div(m, 128);
  pd->sf_nb = ceil_div(n, 128);
  return 0;
}

int check_device(int device, int* sm_count) {
  int count = 0;
  CUDA_TRY(cudaGetDeviceCount(&count));
  if (device < 0 || device >= count) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "device %d out of range (%d devices)", device, count);
  }
  int major = 0, minor = 0;
  CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  CUDA_TRY(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device));
  if (major != 10 || minor != 0) {
    return fail(NVFP4_E_UNSUPPORTED_DEVICE,
                "device %d has compute capability %d.%d; these kernels are built for 10.0 "
                "(sm_100a) only",
                device, major, minor);
  }
  if (sm_count != nullptr) {
    CUDA_TRY(cudaDeviceGetAttribute(sm_count, cudaDevAttrMultiProcessorCount, device));
  }
  return 0;
}

int default_tile_n(const nvfp4_config* config, int fallback) {
  int t = config != nullptr && config->tile_n > 0 ? config->tile_n : env_int("NVFP4_TILE_N", 0);
  if (t == 0) t = fallback;
  return t;
}

int prepare_kernel(nvfp4_plan* plan) {
  if (plan->pair && plan->kind == kDual) {
    plan->kernel = plan->out_kind == NVFP4_OUT_FP4 ? make_pair_choice<PairConfig<Fp4Out, true>>()
                                                   : make_pair_choice<PairConfig<__half, true>>();
  } else if (plan->pair) {
    plan->kernel = plan->out_kind == NVFP4_OUT_F16    ? make_pair_choice<PairConfig<__half>>()
                   : plan->out_kind == NVFP4_OUT_BF16 ? make_pair_choice<PairConfig<__nv_bfloat16>>()
                   : plan->out_kind == NVFP4_OUT_FP4  ? make_pair_choice<PairConfig<Fp4Out>>()
                                                      : make_pair_choice<PairConfig<float>>();
  } else {
    plan->kernel = select_kernel(plan->kind, plan->out_kind, plan->tile_n);
  }
  if (plan->kernel.fn == nullptr) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "no kernel for tile_n=%d", plan->tile_n);
  }
  DeviceGuard guard;
  CUDA_TRY(guard.enter(plan->device));
  CUDA_TRY(cudaFuncSetAttribute(reinterpret_cast<const void*>(plan->kernel.fn),
                                cudaFuncAttributeMaxDynamicSharedMemorySize,
                                plan->kernel.smem_bytes));
  // Cluster split-K: set the last pipeline stages aside as the inbox for the peers' partial
  // columns when at least four stages remain; peers then need no permission to write.
  plan->ring_stages = plan->kernel.stages;
  plan->inbox_offset = -1;
  if (!plan->pair && plan->schedule == 3 && plan->split >= 2 && plan->split <= 4) {
    const int halves = plan->kind == kDual ? 2 : 1;
    const int portion = (plan->out_tile_n / plan->split / 32) * halves * 16384;
    const int inbox = (plan->split - 1) * portion;
    const int reserve = ceil_div(inbox, plan->kernel.stage_bytes);
    if (plan->kernel.stages - reserve >= 4) {
      plan->ring_stages = plan->kernel.stages - reserve;
      plan->inbox_offset = plan->ring_stages * plan->kernel.stage_bytes;
    }
  }
  // Experiments: fewer pipeline stages than the kernel has room for (single-CTA kernel).
  const int fewer = env_int("NVFP4_STAGES", 0);
  if (!plan->pair && fewer >= 2 && fewer < plan->ring_stages) plan->ring_stages = fewer;
  return 0;
}

void fill_common_params(const nvfp4_plan* plan, KernelParams& kp, void* workspace) {
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  kp.status = reinterpret_cast<int*>(ws);
  kp.counters = reinterpret_cast<unsigned int*>(ws + plan->off_counters);
  kp.partials = reinterpret_cast<float*>(ws + plan->off_partials);
  kp.problems = reinterpret_cast<const ProblemDesc*>(ws + plan->off_table);
  kp.maps = reinterpret_cast<const CUtensorMap*>(ws + plan->off_maps);
  kp.total_tiles = plan->total_tiles;
  kp.total_units = plan->total_units;
  kp.slot_floats = plan->slot_floats;
  kp.num_problems = static_cast<int>(plan->problems.size());
  kp.mode = plan->schedule == 1 ? kModeDataParallel : kModeStreamK;
  kp.split = plan->split;
  kp.ring_stages = plan->ring_stages > 0 ? plan->ring_stages : plan->kernel.stages;
  kp.inbox_offset = plan->inbox_offset;
  bool streams = true;
  for (const ProblemDesc& pd : plan->problems) {
    if (pd.tiles_m > 1) streams = false;
  }
  if (plan->routed) streams = false;  // the groups' sizes are not known here
  kp.b_streams = streams ? 1 : 0;
  kp.b_shuffle = plan->b_shuffle;
  kp.maps_per_group = plan->maps_per_group;
  kp.routed_tiles =
      plan->routed ? &reinterpret_cast<const RoutedHeader*>(ws + plan->off_routed)->total_tiles
                   : nullptr;
}

// The kernel parameters of a dense or dual launch on the operands named by `key`: taken from
// the plan's cache, or built by `encode` and remembered (least recently used entry dropped
// when the cache is full). `*out` is the caller's own copy.
template <class Encode>
int bound_params(const nvfp4_plan* plan, const void* const (&key)[10], Encode encode,
                 KernelParams* out) {
  std::lock_guard<std::mutex> lock(plan->mutex);
  for (nvfp4_plan::BoundParams& entry : plan->bound) {
    if (std::memcmp(entry.key, key, sizeof(key)) == 0) {
      entry.last_use = ++plan->use_counter;
      *out = entry.params;
      return 0;
    }
  }
  nvfp4_plan::BoundParams fresh{};
  std::memcpy(fresh.key, key, sizeof(key));
  if (int rc = encode(fresh.params)) return rc;
  fresh.last_use = ++plan->use_counter;
  *out = fresh.params;
  if (plan->bound.size() < nvfp4_plan::kMaxBound) {
    plan->bound.push_back(fresh);
  } else {
    auto oldest = std::min_element(plan->bound.begin(), plan->bound.end(),
                                   [](const nvfp4_plan::BoundParams& x,
                                      const nvfp4_plan::BoundParams& y) {
                                     return x.last_use < y.last_use;
                                   });
    *oldest = fresh;
  }
  return 0;
}

int launch_plan(const nvfp4_plan* plan, KernelParams& kp, void* stream,
                KernelFn kernel_override = nullptr) {
  DeviceGuard guard;
  CUDA_TRY(guard.enter(plan->device));
  void* args[1] = {&kp};
  const KernelFn kernel = kernel_override != nullptr ? kernel_override : plan->kernel.fn;
  // Programmatic stream serialization (as the reference's dense launches use,
  // harness/workloads/nvfp4_gemm.py:143-147): this kernel's prologue may overlap the
  // tail of the kernel before it; it waits on the device before touching global memory.
  static const bool use_pdl = env_int("NVFP4_PDL", 1) != 0;
  cudaLaunchAttribute attribute[2];
  int attributes = 0;
  if (use_pdl) {
    attribute[attributes].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[attributes].val.programmaticStreamSerializationAllowed = 1;
    ++attributes;
  }
  if (plan->split > 1) {
    attribute[attributes].id = cudaLaunchAttributeClusterDimension;
    attribute[attributes].val.clusterDim.x = static_cast<unsigned int>(plan->split);
    attribute[attributes].val.clusterDim.y = 1;
    attribute[attributes].val.clusterDim.z = 1;
    ++attributes;
  }
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(plan->ctas);
  config.blockDim = dim3(plan->kernel.threads);
  config.dynamicSmemBytes = plan->kernel.smem_bytes;
  config.stream = static_cast<cudaStream_t>(stream);
  config.attrs = attribute;
  config.numAttrs = attributes;
  CUDA_TRY(cudaLaunchKernelExC(&config, reinterpret_cast<const void*>(kernel), args));
  return 0;
}

// SM count of the current device (the glue kernels run on whichever device the caller has
// made current, like any runtime launch), remembered per device; 148 if the query fails.
int current_sm_count() {
  static std::mutex mu;
  static int cached[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) {
    cudaGetLastError();
    return 148;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (cached[device] == 0) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        sms < 1) {
      cudaGetLastError();
      sms = 148;
    }
    cached[device] = sms;
  }
  return cached[device];
}

bool aligned(const void* p, uintptr_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; }

int check_dense_shape(int m, int n, int k, int l, int out_bytes) {
  if (m < 1 || n < 1 || k < 1 || l < 1 || k % 32 != 0 || (static_cast<long long>(n) * out_bytes) % 16 != 0) {
    return fail(NVFP4_E_UNSUPPORTED_SHAPE, "unsupported problem m=%d n=%d k=%d l=%d", m, n, k, l);
  }
  if (l > 1) {
    const long long mk = static_cast<long long>(m) * k, nk = static_cast<long long>(n) * k,
                    mn = static_cast<long long>(m) * n;
    if (std::max(mk, std::max(nk, mn)) > INT_MAX) {
      return fail(NVFP4_E_UNSUPPORTED_SHAPE, "batch stride exceeds the 32-bit range");
    }
  }
  return 0;
}

int create_dense_like(nvfp4_plan** out, int kind, int device, int out_kind, int m, int n, int k,
                      int l, const nvfp4_config* config, int b_shuffle = 0) {
  if (out == nullptr) return fail(NVFP4_E_INVALID_ARGUMENT, "plan is null");
  *out = nullptr;
  if (b_shuffle != 0) {
    if (b_shuffle != 16 && b_shuffle != 32) {
      return fail(NVFP4_E_INVALID_ARGUMENT, "the shuffle block is 16 or 32 rows");
    }
    if (kind != kDense || out_kind == NVFP4_OUT_FP4 || n % b_shuffle != 0) {
      return fail(NVFP4_E_UNSUPPORTED_SHAPE,
                  "shuffled weights: dense GEMM with FP16, BF16 or FP32 output and n a "
                  "multiple of the shuffle block");
    }
  }
  double chosen_us = 1e30;  // the time model's figure for the best single-CTA plan
  if (out_kind != NVFP4_OUT_F16 && out_kind != NVFP4_OUT_F32 && out_kind != NVFP4_OUT_FP4 &&
      out_kind != NVFP4_OUT_BF16) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "unknown output kind %d", out_kind);
  }
  if (out_kind == NVFP4_OUT_FP4 && n % 64 != 0) {
    return fail(NVFP4_E_UNSUPPORTED_SHAPE,
                "NVFP4 output needs n to be a multiple of 64 (whole scale atoms)");
  }
  // The fused dual GEMM also takes n % 8 == 4 (8-byte aligned FP16 rows), because its
  // FP32-output stage does.
  const bool two_byte_rows = (out_kind == NVFP4_OUT_F16 || out_kind == NVFP4_OUT_BF16) && kind != kDual;
  if (int rc = check_dense_shape(m, n, k, l, two_byte_rows ? 2 : 4)) {
    return rc;
  }
  // The NVFP4-output epilogue quantises whole rows of a finished tile: such plans keep
  // every tile's K in one CTA or one pair of CTAs (data parallel).
  nvfp4_config whole_tiles = {};
  const bool fp4_schedule_left_open =
      out_kind == NVFP4_OUT_FP4 && (config == nullptr || config->schedule == 0);
  if (out_kind == NVFP4_OUT_FP4) {
    if (config != nullptr) whole_tiles = *config;
    if (whole_tiles.schedule > 1) {
      return fail(NVFP4_E_INVALID_ARGUMENT, "NVFP4 output supports the data-parallel schedule only");
    }
    whole_tiles.schedule = 1;
    config = &whole_tiles;
  }
  int sms = 0;
  if (int rc = check_device(device, &sms)) return rc;
  nvfp4_plan* plan = new (std::nothrow) nvfp4_plan();
  if (plan == nullptr) return fail(NVFP4_E_INVALID_ARGUMENT, "out of host memory");
  plan->kind = kind;
  plan->device = device;
  plan->out_kind = out_kind;
  plan->sm_count = sms;
  plan->b_shuffle = b_shuffle;
  if (kind == kDual) {
    // The MMA is as wide as both B tiles together: 2 x 128 columns, or 2 x 64 when that
    // fills the SMs better (its accumulator is double-buffered and it needs no K split).
    plan->problems.resize(1);
    int chosen = default_tile_n(config, 0);
    if (chosen == 0) {
      for (int tile_n : {128, 256}) {
        plan->tile_n = tile_n;
        plan->out_tile_n = tile_n / 2;
        fill_problem(&plan->problems[0], m, n, k, l, tile_n / 2);
        finish_schedule(plan, config);
        if (plan->estimate_us < chosen_us) {
          chosen_us = plan->estimate_us;
          chosen = tile_n;
        }
      }
    }
    plan->tile_n = chosen;
    plan->out_tile_n = chosen / 2;
  } else {
    // Tile width: the one whose best schedule the time model puts first, unless the
    // caller names one. Pairs of CTAs on 256 x 256 tiles (tcgen05.mma.cta_group::2, each
    // CTA loads only half of every B tile) compete in the same model.
    plan->problems.resize(1);
    int chosen = default_tile_n(config, 0);
    if (chosen == 0) {
      for (int tile_n : {64, 128, 256}) {
        plan->tile_n = tile_n;
        plan->out_tile_n = tile_n;
        fill_problem(&plan->problems[0], m, n, k, l, tile_n);
        finish_schedule(plan, config);
        if (plan->estimate_us < chosen_us) {
          chosen_us = plan->estimate_us;
          chosen = tile_n;
        }
      }
    }
    plan->tile_n = chosen;
    plan->out_tile_n = chosen;
  }
  {
    // The 2-CTA kernel: 256 x 256 output tiles (dual: 256 x 128, B1 in one CTA and B2 in
    // the other).
    const int pair_out_n = kind == kDual ? 128 : 256;
    const long long pair_tiles =
        static_cast<long long>(ceil_div(m, 256)) * ceil_div(n, pair_out_n) * l;
    int want_pair = config != nullptr ? config->pair : 0;
    if (want_pair == 0) want_pair = env_int("NVFP4_PAIR", 0);
    // The 2-CTA kernel stores 16-bit output through a tensor map: rows 16-byte aligned.
    if (out_kind != NVFP4_OUT_F32 && n % 8 != 0) {
      if (want_pair > 0) {
        delete plan;
        return fail(NVFP4_E_UNSUPPORTED_SHAPE,
                    "the 2-CTA kernel needs n to be a multiple of 8 for 16-bit output");
      }
      want_pair = -1;
    }
    // (The data-parallel schedule that NVFP4 output forces above is not the caller's choice.)
    const bool explicit_choice =
        (config != nullptr && (config->tile_n > 0 || (config->schedule > 0 && !fp4_schedule_left_open) ||
                               config->ctas > 0)) ||
        env_int("NVFP4_TILE_N", 0) > 0 || env_int("NVFP4_SCHEDULE", 0) > 0 ||
        env_int("NVFP4_CTAS", 0) > 0;
    const long long pair_waves = (pair_tiles + sms / 2 - 1) / (sms / 2);
    // Beside the waves of tiles, a launch of pairs costs about 2.5 us more than a launch of
    // single CTAs (cluster launch, the pair's barriers at both ends): on 2048^3, one wave
    // either way, the pairs take 9.8 us and 128 x 256 tiles 7.8 us.
    const double pair_us =
        static_cast<double>(pair_waves) * (ceil_div(k, 256) * kPairStepUs + 1.2) + 2.5;
    plan->pair = want_pair > 0 || (want_pair == 0 && !explicit_choice && kPairByDefault &&
                                   pair_tiles >= sms / 4 && pair_us < chosen_us);
    if (plan->pair) {
      plan->tile_n = 256;
      plan->out_tile_n = pair_out_n;
    }
  }
  plan->problems.resize(1);
  fill_problem(&plan->problems[0], m, n, k, l, plan->out_tile_n);
  if (plan->pair) {
    // One schedule only: pair tiles dealt round-robin to the pairs of SMs.
    ProblemDesc& pd = plan->problems[0];
    const long long pair_tiles =
        static_cast<long long>(ceil_div(m, 256)) * ceil_div(n, plan->out_tile_n) * l;
    pd.tiles_m = ceil_div(m, 256);
    pd.tile_begin = 0;
    pd.unit_begin = 0;
    plan->total_tiles = pair_tiles;
    plan->total_units = pair_tiles * pd.k_tiles;
    plan->schedule = 1;
    plan->split = 2;
    plan->ctas = 2 * static_cast<int>(std::min<long long>(sms / 2, pair_tiles));
    plan->off_counters = 256;
    plan->off_table = 512;
    plan->off_maps = 512;
    plan->off_partials = 512;
    plan->slot_floats = 0;
    plan->ws_bytes = 512;
  } else {
    finish_schedule(plan, config);
  }
  if (int rc = prepare_kernel(plan)) {
    delete plan;
    return rc;
  }
  *out = plan;
  return 0;
}

}  // namespace

extern "C" {

int nvfp4_version(void) { return 1000; }

const char* nvfp4_last_error(void) { return g_last_error.c_str(); }

int nvfp4_device_supported(int device) {
  int rc = check_device(device, nullptr);
  if (rc == 0) return 1;
  if (rc == NVFP4_E_UNSUPPORTED_DEVICE) return 0;
  return rc;
}

int nvfp4_gemm_plan_create(nvfp4_plan** plan, int device, int out_kind, int m, int n, int k,
                           int l, const nvfp4_config* config) {
  return create_dense_like(plan, kDense, device, out_kind, m, n, k, l, config);
}

int nvfp4_gemm_plan_create_shuffled(nvfp4_plan** plan, int device, int out_kind, int m, int n,
                                    int k, int l, int shuffle_block, const nvfp4_config* config) {
  if (shuffle_block != 16 && shuffle_block != 32) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "the shuffle block is 16 or 32 rows");
  }
  return create_dense_like(plan, kDense, device, out_kind, m, n, k, l, config, shuffle_block);
}

int nvfp4_dual_gemm_plan_create(nvfp4_plan** plan, int device, int m, int n, int k, int l,
                                const nvfp4_config* config) {
  return create_dense_like(plan, kDual, device, NVFP4_OUT_F16, m, n, k, l, config);
}

int nvfp4_dual_gemm_plan_create_fp4(nvfp4_plan** plan, int device, int m, int n, int k, int l,
                                    const nvfp4_config* config) {
  return create_dense_like(plan, kDual, device, NVFP4_OUT_FP4, m, n, k, l, config);
}

int nvfp4_group_gemm_plan_create(nvfp4_plan** out, int device, int groups, const int* mnk,
                                 const nvfp4_config* config) {
  if (out == nullptr) return fail(NVFP4_E_INVALID_ARGUMENT, "plan is null");
  *out = nullptr;
  if (groups < 1 || mnk == nullptr) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "expected at least one group");
  }
  for (int g = 0; g < groups; ++g) {
    const int m = mnk[3 * g], n = mnk[3 * g + 1], k = mnk[3 * g + 2];
    if (m < 1 || n < 1 || k < 1 || k % 32 != 0 || n % 8 != 0) {
      return fail(NVFP4_E_UNSUPPORTED_SHAPE, "group %d: unsupported problem m=%d n=%d k=%d", g,
                  m, n, k);
    }
  }
  int sms = 0;
  if (int rc = check_device(device, &sms)) return rc;
  nvfp4_plan* plan = new (std::nothrow) nvfp4_plan();
  if (plan == nullptr) return fail(NVFP4_E_INVALID_ARGUMENT, "out of host memory");
  plan->kind = kGrouped;
  plan->device = device;
  plan->out_kind = NVFP4_OUT_F16;
  plan->sm_count = sms;
  long long wide_tiles = 0;
  for (int g = 0; g < groups; ++g) {
    wide_tiles += static_cast<long long>(ceil_div(mnk[3 * g], 128)) * ceil_div(mnk[3 * g + 1], 256);
  }
  plan->tile_n = default_tile_n(config, wide_tiles >= 2ll * sms ? 256 : 128);
  plan->out_tile_n = plan->tile_n;
  plan->problems.resize(groups);
  for (int g = 0; g < groups; ++g) {
    fill_problem(&plan->problems[g], mnk[3 * g], mnk[3 * g + 1], mnk[3 * g + 2], 1,
                 plan->out_tile_n);
  }
  finish_schedule(plan, config);
  if (int rc = prepare_kernel(plan)) {
    delete plan;
    return rc;
  }
  *out = plan;
  return 0;
}

int nvfp4_group_dual_gemm_plan_create_fp4(nvfp4_plan** out, int device, int groups,
                                          const int* mnk, const nvfp4_config* config) {
  if (out == nullptr) return fail(NVFP4_E_INVALID_ARGUMENT, "plan is null");
  *out = nullptr;
  if (groups < 1 || mnk == nullptr) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "expected at least one group");
  }
  for (int g = 0; g < groups; ++g) {
    const int m = mnk[3 * g], n = mnk[3 * g + 1], k = mnk[3 * g + 2];
    if (m < 1 || n < 1 || k < 1 || k % 32 != 0 || n % 64 != 0) {
      return fail(NVFP4_E_UNSUPPORTED_SHAPE,
                  "group %d: unsupported problem m=%d n=%d k=%d (NVFP4 output needs n to be a "
                  "multiple of 64)", g, m, n, k);
    }
  }
  if (config != nullptr && (config->schedule > 1 || config->pair > 0)) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "NVFP4 output supports the data-parallel schedule only");
  }
  int sms = 0;
  if (int rc = check_device(device, &sms)) return rc;
  nvfp4_plan* plan = new (std::nothrow) nvfp4_plan();
  if (plan == nullptr) return fail(NVFP4_E_INVALID_ARGUMENT, "out of host memory");
  plan->kind = kGrouped;
  plan->device = device;
  plan->out_kind = NVFP4_OUT_FP4;
  plan->sm_count = sms;
  plan->maps_per_group = 3;
  // Two 128-row B tiles side by side (128 output columns per tile) when that still gives
  // every SM two tiles, else two 64-row tiles.
  long long wide_tiles = 0;
  for (int g = 0; g < groups; ++g) {
    wide_tiles += static_cast<long long>(ceil_div(mnk[3 * g], 128)) * ceil_div(mnk[3 * g + 1], 128);
  }
  plan->tile_n = default_tile_n(config, wide_tiles >= 2ll * sms ? 256 : 128);
  if (plan->tile_n != 128 && plan->tile_n != 256) {
    delete plan;
    return fail(NVFP4_E_INVALID_ARGUMENT, "the grouped dual GEMM has tile_n 128 or 256");
  }
  plan->out_tile_n = plan->tile_n / 2;
  plan->problems.resize(groups);
  for (int g = 0; g < groups; ++g) {
    fill_problem(&plan->problems[g], mnk[3 * g], mnk[3 * g + 1], mnk[3 * g + 2], 1,
                 plan->out_tile_n);
  }
  nvfp4_config whole_tiles = {};
  if (config != nullptr) whole_tiles = *config;
  whole_tiles.schedule = 1;
  finish_schedule(plan, &whole_tiles);
  if (int rc = prepare_kernel(plan)) {
    delete plan;
    return rc;
  }
  *out = plan;
  return 0;
}

int nvfp4_moe_plan_create(nvfp4_plan** out, int device, int experts, int n, int k, int max_rows,
                          int out_kind, const nvfp4_config* config) {
  if (out == nullptr) return fail(NVFP4_E_INVALID_ARGUMENT, "plan is null");
  *out = nullptr;
  const bool dual = out_kind == NVFP4_OUT_FP4;
  if (out_kind != NVFP4_OUT_F16 && !dual) {
    return fail(NVFP4_E_INVALID_ARGUMENT,
                "a routed plan is the gate/up projection with NVFP4 output or a GEMM with FP16 output");
  }
  if (experts < 1 || experts > kMoeMaxExperts) {
    return fail(NVFP4_E_UNSUPPORTED_SHAPE, "1 to %d experts", kMoeMaxExperts);
  }
  if (n < 1 || k < 32 || k % 32 != 0 || n % (dual ? 64 : 8) != 0 || max_rows < 128 ||
      max_rows % 128 != 0) {
    return fail(NVFP4_E_UNSUPPORTED_SHAPE,
                "unsupported routed problem n=%d k=%d rows=%d (rows a multiple of 128)", n, k,
                max_rows);
  }
  if (config != nullptr && (config->schedule > 1 || config->pair > 0)) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "routed plans are data parallel on single CTAs");
  }
  int sms = 0;
  if (int rc = check_device(device, &sms)) return rc;
  nvfp4_plan* plan = new (std::nothrow) nvfp4_plan();
  if (plan == nullptr) return fail(NVFP4_E_INVALID_ARGUMENT, "out of host memory");
  plan->kind = kGrouped;
  plan->device = device;
  plan->out_kind = out_kind;
  plan->sm_count = sms;
  plan->maps_per_group = dual ? 3 : 2;
  plan->tile_n = default_tile_n(config, 256);
  if ((plan->tile_n != 128 && plan->tile_n != 256) && (dual || plan->tile_n != 64)) {
    delete plan;
    return fail(NVFP4_E_INVALID_ARGUMENT, "no kernel for tile_n=%d", plan->tile_n);
  }
  plan->out_tile_n = dual ? plan->tile_n / 2 : plan->tile_n;
  plan->problems.resize(experts);
  for (int g = 0; g < experts; ++g) {
    fill_problem(&plan->problems[g], 0, n, k, 1, plan->out_tile_n);
  }
  nvfp4_config whole_tiles = {};
  if (config != nullptr) whole_tiles = *config;
  whole_tiles.schedule = 1;
  finish_schedule(plan, &whole_tiles);
  // The groups' sizes are known on the device only: every SM gets a CTA, and the table that
  // the layout kernel fills in follows the maps in the workspace.
  plan->ctas = config != nullptr && config->ctas > 0 ? std::min(config->ctas, sms) : sms;
  plan->routed = true;
  plan->routed_rows = max_rows;
  plan->off_routed = round_up(plan->ws_bytes, 256);
  plan->ws_bytes = plan->off_routed + round_up(sizeof(RoutedHeader), 256);
  if (int rc = prepare_kernel(plan)) {
    delete plan;
    return rc;
  }
  *out = plan;
  return 0;
}

void nvfp4_plan_destroy(nvfp4_plan* plan) { delete plan; }

size_t nvfp4_plan_workspace_bytes(const nvfp4_plan* plan) {
  return plan != nullptr ? plan->ws_bytes : 0;
}

int nvfp4_plan_init_workspace(const nvfp4_plan* plan, void* workspace, void* stream) {
  if (plan == nullptr || workspace == nullptr) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "plan or workspace is null");
  }
  if (!aligned(workspace, 256)) return fail(NVFP4_E_MISALIGNED, "workspace must be 256-byte aligned");
  DeviceGuard guard;
  CUDA_TRY(guard.enter(plan->device));
  CUDA_TRY(cudaMemsetAsync(workspace, 0, plan->off_table, static_cast<cudaStream_t>(stream)));
  return 0;
}

int nvfp4_plan_info_get(const nvfp4_plan* plan, nvfp4_plan_info* info) {
  if (plan == nullptr || info == nullptr) return fail(NVFP4_E_INVALID_ARGUMENT, "null argument");
  info->tile_m = plan->pair ? 256 : 128;
  info->tile_n = plan->out_tile_n;
  info->tile_k = 256;
  info->stages = plan->ring_stages > 0 ? plan->ring_stages : plan->kernel.stages;
  info->schedule = plan->schedule;
  info->ctas = plan->ctas;
  info->threads = plan->kernel.threads;
  info->smem_bytes = plan->kernel.smem_bytes;
  info->tiles = plan->total_tiles;
  info->units = plan->total_units;
  info->sm_count = plan->sm_count;
  return 0;
}

}  // extern "C"

namespace {

// The dense launch behind nvfp4_gemm_launch and nvfp4_gemm_launch_fp4 (`sfd` is null for
// the former).
int launch_dense(const nvfp4_plan* plan, const void* a, const void* b, const void* sfa,
                 const void* sfb, const float* alpha, void* d, void* sfd, void* workspace,
                 void* stream, KernelFn kernel_override = nullptr) {
  if (a == nullptr || b == nullptr || sfa == nullptr || sfb == nullptr || alpha == nullptr ||
      d == nullptr || workspace == nullptr) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "null operand");
  }
  if (!aligned(a, 16) || !aligned(b, 16) || !aligned(sfa, 16) || !aligned(sfb, 16) ||
      !aligned(d, 16) || !aligned(sfd, 16) || !aligned(alpha, 4) || !aligned(workspace, 256)) {
    return fail(NVFP4_E_MISALIGNED, "misaligned operand address");
  }
  DeviceGuard guard;
  CUDA_TRY(guard.enter(plan->device));
  const void* key[10] = {a, b, nullptr, sfa, sfb, sfd, alpha, d, nullptr, workspace};
  KernelParams kp;
  const int rc = bound_params(
      plan, key,
      [&](KernelParams& fresh) {
        ProblemDesc pd = plan->problems[0];
        if (int rc = encode_operand_map(&fresh.map_a, a, pd.m, pd.k, pd.batches, 128)) return rc;
        if (int rc = encode_operand_map(&fresh.map_b, b, pd.n, pd.k, pd.batches,
                                        plan->pair ? 128 : plan->tile_n)) {
          return rc;
        }
        fresh.map_b2 = fresh.map_b;
        fresh.map_d = fresh.map_a;  // a valid descriptor; used by the 2-CTA kernel only
        if (plan->pair && (plan->out_kind == NVFP4_OUT_F16 || plan->out_kind == NVFP4_OUT_BF16)) {
          if (int rc = encode_output_map(&fresh.map_d, d, pd.m, pd.n, pd.batches)) return rc;
        }
        pd.sfa = static_cast<const uint8_t*>(sfa);
        pd.sfb = static_cast<const uint8_t*>(sfb);
        pd.sfb2 = nullptr;
        pd.d = d;
        pd.sfd = static_cast<uint8_t*>(sfd);
        fresh.dense = pd;
        fresh.alpha = alpha;
        fill_common_params(plan, fresh, workspace);
        return 0;
      },
      &kp);
  if (rc != 0) return rc;
  return launch_plan(plan, kp, stream, kernel_override);
}

}  // namespace

extern "C" {

int nvfp4_selftest_abandoned_wait(const nvfp4_plan* plan, const void* a, const void* b,
                                  const void* sfa, const void* sfb, const float* alpha, void* d,
                                  void* workspace, void* stream) {
  if (plan == nullptr || plan->kind != kDense || plan->out_kind != NVFP4_OUT_F16 || plan->pair ||
      plan->tile_n != 128 || plan->schedule == 3) {
    return fail(NVFP4_E_INVALID_ARGUMENT,
                "the self-test runs dense FP16 plans with 128-column tiles (config.tile_n = 128, "
                "schedule 1 or 2) only");
  }
  using Stalled = GemmConfig<128, false, __half, false>;
  const KernelFn kernel = &nvfp4_gemm_kernel<Stalled, true>;
  {
    DeviceGuard guard;
    CUDA_TRY(guard.enter(plan->device));
    CUDA_TRY(cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel),
                                  cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  Stalled::SMEM_BYTES));
  }
  return launch_dense(plan, a, b, sfa, sfb, alpha, d, nullptr, workspace, stream, kernel);
}

int nvfp4_gemm_launch(const nvfp4_plan* plan, const void* a, const void* b, const void* sfa,
                      const void* sfb, const float* alpha, void* d, void* workspace,
                      void* stream) {
  if (plan == nullptr || plan->kind != kDense || plan->out_kind == NVFP4_OUT_FP4) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "not a dense GEMM plan with FP16 or FP32 output");
  }
  return launch_dense(plan, a, b, sfa, sfb, alpha, d, nullptr, workspace, stream);
}

int nvfp4_gemm_launch_fp4(const nvfp4_plan* plan, const void* a, const void* b, const void* sfa,
                          const void* sfb, const float* alpha, void* d_packed, void* d_scales,
                          void* workspace, void* stream) {
  if (plan == nullptr || plan->kind != kDense || plan->out_kind != NVFP4_OUT_FP4) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "not a dense GEMM plan with NVFP4 output");
  }
  if (d_scales == nullptr) return fail(NVFP4_E_INVALID_ARGUMENT, "null operand");
  return launch_dense(plan, a, b, sfa, sfb, alpha, d_packed, d_scales, workspace, stream);
}

// ---------------------------------------------------------------------------------------
// Dense launch for callers that cannot hand over a workspace.
//
// Some hosts of this library are not allowed to allocate device memory at the point where
// they call it: a runtime that has given all of HBM to its own pool, a plugin that runs
// under an allocator it does not control, a serving loop that forbids cudaMalloc on its
// hot path because the call synchronises the device. For them the scratch that the
// split-K schedules need lives in the array below instead of in a caller buffer. The
// array is part of the loaded module, so every GPU that loads the library holds these
// bytes until the process exits.
// ---------------------------------------------------------------------------------------

constexpr size_t kStaticScratchBytes = 24u << 20;  // 24 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ int g_peak_status;  // status word of nvfp4_measure_mma_peak

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
void* g_scratch_address[kMaxDevices] = {};

// Device address of g_static_scratch on `device`. In host code the array's name is only
// a handle for the runtime, never a device pointer, so the address is looked up once per
// device (with that device current) and remembered.
int static_scratch_address(int device, void** out) {
  if (device < 0 || device >= kMaxDevices) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "device %d out of range", device);
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_address[device] == nullptr) {
    DeviceGuard guard;
    CUDA_TRY(guard.enter(device));
    void* address = nullptr;
    CUDA_TRY(cudaGetSymbolAddress(&address, g_static_scratch));
    if (address == nullptr) return fail(NVFP4_E_INVALID_ARGUMENT, "no address for the scratch array");
    g_scratch_address[device] = address;
  }
  *out = g_scratch_address[device];
  return 0;
}

}  // namespace

int nvfp4_gemm_launch_static(const nvfp4_plan* plan, const void* a, const void* b, const void* sfa,
                             const void* sfb, const float* alpha, void* d, void* stream) {
  if (plan == nullptr || plan->kind != kDense) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "not a dense GEMM plan");
  }
  if (plan->ws_bytes > kStaticScratchBytes) {
    return fail(NVFP4_E_SCRATCH_TOO_LARGE,
                "this plan needs %zu bytes of scratch; the built-in array holds %zu. Use "
                "nvfp4_gemm_launch with a caller workspace, or a plan with fewer CTAs",
                plan->ws_bytes, kStaticScratchBytes);
  }
  void* scratch = nullptr;
  if (int rc = static_scratch_address(plan->device, &scratch)) return rc;
  {
    // The array keeps whatever the previous call (of any plan) left in it; the status
    // word and this plan's tile counters must start at zero.
    DeviceGuard guard;
    CUDA_TRY(guard.enter(plan->device));
    CUDA_TRY(cudaMemsetAsync(scratch, 0, plan->off_table, static_cast<cudaStream_t>(stream)));
  }
  return nvfp4_gemm_launch(plan, a, b, sfa, sfb, alpha, d, scratch, stream);
}

size_t nvfp4_static_scratch_bytes(void) { return kStaticScratchBytes; }

int nvfp4_static_status(int device, void* stream, int* status) {
  if (status == nullptr) return fail(NVFP4_E_INVALID_ARGUMENT, "null argument");
  void* scratch = nullptr;
  if (int rc = static_scratch_address(device, &scratch)) return rc;
  DeviceGuard guard;
  CUDA_TRY(guard.enter(device));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int value = 0;
  CUDA_TRY(cudaMemcpyAsync(&value, scratch, sizeof(int), cudaMemcpyDeviceToHost, s));
  CUDA_TRY(cudaStreamSynchronize(s));
  *status = value;
  if (value != 0) {
    // The next nvfp4_gemm_launch_static clears the word and its counters before it launches.
    return fail(NVFP4_E_DEVICE_TIMEOUT, "kernel abandoned a bounded wait (code %d)", value);
  }
  return 0;
}

}  // extern "C"

namespace {

// The launch behind nvfp4_dual_gemm_launch and nvfp4_dual_gemm_launch_fp4 (`sfd` null for
// the former).
int launch_dual(const nvfp4_plan* plan, const void* a, const void* b1, const void* b2,
                const void* sfa, const void* sfb1, const void* sfb2, const float* alpha, void* d,
                void* sfd, void* workspace, void* stream) {
  if (a == nullptr || b1 == nullptr || b2 == nullptr || sfa == nullptr || sfb1 == nullptr ||
      sfb2 == nullptr || alpha == nullptr || d == nullptr || workspace == nullptr) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "null operand");
  }
  // FP16 rows are stored in 16-byte pieces whenever n is a multiple of 8; only rows of
  // n % 8 == 4 elements (8-byte aligned at best) are stored in 8-byte pieces.
  const uintptr_t d_alignment = (sfd == nullptr && plan->problems[0].n % 8 == 4) ? 8 : 16;
  if (!aligned(a, 16) || !aligned(b1, 16) || !aligned(b2, 16) || !aligned(sfa, 16) ||
      !aligned(sfb1, 16) || !aligned(sfb2, 16) || !aligned(d, d_alignment) ||
      !aligned(sfd, 16) || !aligned(alpha, 4) || !aligned(workspace, 256)) {
    return fail(NVFP4_E_MISALIGNED, "misaligned operand address");
  }
  DeviceGuard guard;
  CUDA_TRY(guard.enter(plan->device));
  const void* key[10] = {a, b1, b2, sfa, sfb1, sfb2, alpha, d, sfd, workspace};
  KernelParams kp;
  const int rc = bound_params(
      plan, key,
      [&](KernelParams& fresh) {
        ProblemDesc pd = plan->problems[0];
        if (int rc = encode_operand_map(&fresh.map_a, a, pd.m, pd.k, pd.batches, 128)) return rc;
        if (int rc = encode_operand_map(&fresh.map_b, b1, pd.n, pd.k, pd.batches,
                                        plan->out_tile_n)) {
          return rc;
        }
        if (int rc = encode_operand_map(&fresh.map_b2, b2, pd.n, pd.k, pd.batches,
                                        plan->out_tile_n)) {
          return rc;
        }
        fresh.map_d = fresh.map_a;
        if (plan->pair && plan->out_kind != NVFP4_OUT_FP4) {
          if (int rc = encode_output_map(&fresh.map_d, d, pd.m, pd.n, pd.batches)) return rc;
        }
        pd.sfa = static_cast<const uint8_t*>(sfa);
        pd.sfb = static_cast<const uint8_t*>(sfb1);
        pd.sfb2 = static_cast<const uint8_t*>(sfb2);
        pd.d = d;
        pd.sfd = static_cast<uint8_t*>(sfd);
        fresh.dense = pd;
        fresh.alpha = alpha;
        fill_common_params(plan, fresh, workspace);
        return 0;
      },
      &kp);
  if (rc != 0) return rc;
  return launch_plan(plan, kp, stream);
}

}  // namespace

extern "C" {

int nvfp4_dual_gemm_launch(const nvfp4_plan* plan, const void* a, const void* b1, const void* b2,
                           const void* sfa, const void* sfb1, const void* sfb2,
                           const float* alpha, void* d, void* workspace, void* stream) {
  if (plan == nullptr || plan->kind != kDual || plan->out_kind == NVFP4_OUT_FP4) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "not a dual GEMM plan with FP16 output");
  }
  return launch_dual(plan, a, b1, b2, sfa, sfb1, sfb2, alpha, d, nullptr, workspace, stream);
}

int nvfp4_dual_gemm_launch_fp4(const nvfp4_plan* plan, const void* a, const void* b1, const void* b2,
                               const void* sfa, const void* sfb1, const void* sfb2,
                               const float* alpha, void* d_packed, void* d_scales,
                               void* workspace, void* stream) {
  if (plan == nullptr || plan->kind != kDual || plan->out_kind != NVFP4_OUT_FP4) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "not a dual GEMM plan with NVFP4 output");
  }
  if (d_scales == nullptr) return fail(NVFP4_E_INVALID_ARGUMENT, "null operand");
  return launch_dual(plan, a, b1, b2, sfa, sfb1, sfb2, alpha, d_packed, d_scales, workspace,
                     stream);
}

}  // extern "C"

namespace {

// Behind nvfp4_group_gemm_bind and nvfp4_group_dual_gemm_bind_fp4 (`b2`, `sfb2`, `sfd` null
// for the former): checks the pointers, encodes the groups' tensor maps and writes the
// group table into the workspace.
// Host bytes into device memory as kernel parameters, 3.5 KB per launch: parameters are copied
// when a launch is enqueued, so the source may go out of scope when this returns. (An
// asynchronous copy from pageable memory may still be reading its source then.) `bytes` is
// rounded up to 16; the destination has room for that.
int deliver_bytes(uint8_t* dst, const void* src, size_t bytes, void* stream) {
  const uint8_t* from = static_cast<const uint8_t*>(src);
  for (size_t done = 0; done < bytes; done += ParamBlob::kBytes) {
    ParamBlob blob = {};
    const size_t part = std::min<size_t>(ParamBlob::kBytes, bytes - done);
    std::memcpy(blob.data, from + done, part);
    write_blob_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        dst + done, blob, static_cast<int>((part + 15) / 16 * 16));
    CUDA_TRY(cudaGetLastError());
  }
  return 0;
}

int bind_groups(const nvfp4_plan* plan, const void* const* a, const void* const* b,
                const void* const* b2, const void* const* sfa, const void* const* sfb,
                const void* const* sfb2, void* const* d, void* const* sfd, void* workspace,
                void* stream) {
  const bool dual = plan->maps_per_group == 3;
  if (a == nullptr || b == nullptr || sfa == nullptr || sfb == nullptr || d == nullptr ||
      workspace == nullptr || (dual && (b2 == nullptr || sfb2 == nullptr || sfd == nullptr))) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "null pointer array");
  }
  if (!aligned(workspace, 256)) return fail(NVFP4_E_MISALIGNED, "workspace must be 256-byte aligned");
  const size_t groups = plan->problems.size();
  for (size_t g = 0; g < groups; ++g) {
    if (a[g] == nullptr || b[g] == nullptr || sfa[g] == nullptr || sfb[g] == nullptr ||
        d[g] == nullptr || (dual && (b2[g] == nullptr || sfb2[g] == nullptr || sfd[g] == nullptr))) {
      return fail(NVFP4_E_INVALID_ARGUMENT, "group %zu: null operand", g);
    }
    if (!aligned(a[g], 16) || !aligned(b[g], 16) || !aligned(sfa[g], 16) ||
        !aligned(sfb[g], 16) || !aligned(d[g], 16) ||
        (dual && (!aligned(b2[g], 16) || !aligned(sfb2[g], 16) || !aligned(sfd[g], 16)))) {
      return fail(NVFP4_E_MISALIGNED, "group %zu: operands must be 16-byte aligned", g);
    }
  }
  DeviceGuard guard;
  CUDA_TRY(guard.enter(plan->device));
  // The group table and the tensor maps are built in a buffer of this call and copied into
  // the workspace: the plan itself is not modified.
  const size_t table_bytes = plan->off_partials - plan->off_table;
  std::vector<uint8_t> staging(table_bytes, 0);
  ProblemDesc* table = reinterpret_cast<ProblemDesc*>(staging.data());
  uint8_t* maps = staging.data() + (plan->off_maps - plan->off_table);
  const int per_group = plan->maps_per_group;
  // Rows of B per tensor-map box: the tile's rows, or (dual) each B's half of them.
  const int b_box_rows = dual ? plan->out_tile_n : plan->tile_n;
  for (size_t g = 0; g < groups; ++g) {
    ProblemDesc pd = plan->problems[g];
    pd.sfa = static_cast<const uint8_t*>(sfa[g]);
    pd.sfb = static_cast<const uint8_t*>(sfb[g]);
    pd.sfb2 = dual ? static_cast<const uint8_t*>(sfb2[g]) : nullptr;
    pd.d = d[g];
    pd.sfd = dual ? static_cast<uint8_t*>(sfd[g]) : nullptr;
    table[g] = pd;
    CUtensorMap tmp;
    uint8_t* slot = maps + g * per_group * sizeof(CUtensorMap);
    if (int rc = encode_operand_map(&tmp, a[g], pd.m, pd.k, 1, 128)) return rc;
    std::memcpy(slot, &tmp, sizeof(tmp));
    if (int rc = encode_operand_map(&tmp, b[g], pd.n, pd.k, 1, b_box_rows)) return rc;
    std::memcpy(slot + sizeof(tmp), &tmp, sizeof(tmp));
    if (dual) {
      if (int rc = encode_operand_map(&tmp, b2[g], pd.n, pd.k, 1, b_box_rows)) return rc;
      std::memcpy(slot + 2 * sizeof(tmp), &tmp, sizeof(tmp));
    }
  }
  uint8_t* dst = static_cast<uint8_t*>(workspace) + plan->off_table;
  if (int rc = deliver_bytes(dst, staging.data(), table_bytes, stream)) return rc;
  {
    std::lock_guard<std::mutex> lock(plan->mutex);
    plan->group_bound = true;
  }
  return 0;
}

// The bind of a routed plan (nvfp4_moe_bind): what does not depend on the groups' row counts.
int bind_routed(const nvfp4_plan* plan, const void* a, const void* sfa, const void* const* b,
                const void* const* sfb, const void* const* b2, const void* const* sfb2, void* d,
                void* sfd, void* workspace, void* stream) {
  const bool dual = plan->maps_per_group == 3;
  if (a == nullptr || sfa == nullptr || b == nullptr || sfb == nullptr || d == nullptr ||
      workspace == nullptr || (dual && (b2 == nullptr || sfb2 == nullptr || sfd == nullptr))) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "null pointer");
  }
  if (!aligned(workspace, 256)) return fail(NVFP4_E_MISALIGNED, "workspace must be 256-byte aligned");
  if (!aligned(a, 16) || !aligned(sfa, 16) || !aligned(d, 16) || !aligned(sfd, 16)) {
    return fail(NVFP4_E_MISALIGNED, "shared buffers must be 16-byte aligned");
  }
  const size_t groups = plan->problems.size();
  for (size_t g = 0; g < groups; ++g) {
    if (b[g] == nullptr || sfb[g] == nullptr || (dual && (b2[g] == nullptr || sfb2[g] == nullptr))) {
      return fail(NVFP4_E_INVALID_ARGUMENT, "group %zu: null operand", g);
    }
    if (!aligned(b[g], 16) || !aligned(sfb[g], 16) ||
        (dual && (!aligned(b2[g], 16) || !aligned(sfb2[g], 16)))) {
      return fail(NVFP4_E_MISALIGNED, "group %zu: operands must be 16-byte aligned", g);
    }
  }
  DeviceGuard guard;
  CUDA_TRY(guard.enter(plan->device));
  const size_t table_bytes = plan->off_partials - plan->off_table;
  std::vector<uint8_t> staging(table_bytes, 0);
  ProblemDesc* table = reinterpret_cast<ProblemDesc*>(staging.data());
  uint8_t* maps = staging.data() + (plan->off_maps - plan->off_table);
  const int per_group = plan->maps_per_group;
  const int b_box_rows = dual ? plan->out_tile_n : plan->tile_n;
  const ProblemDesc& shape = plan->problems[0];
  CUtensorMap tmp;
  // Slot 0 of group 0: the A buffer all groups share (the other groups' A slots stay unused).
  if (int rc = encode_operand_map(&tmp, a, plan->routed_rows, shape.k, 1, 128)) return rc;
  std::memcpy(maps, &tmp, sizeof(tmp));
  for (size_t g = 0; g < groups; ++g) {
    ProblemDesc pd = plan->problems[g];  // m = 0 until the layout kernel has run
    pd.sfb = static_cast<const uint8_t*>(sfb[g]);
    pd.sfb2 = dual ? static_cast<const uint8_t*>(sfb2[g]) : nullptr;
    table[g] = pd;
    uint8_t* slot = maps + g * per_group * sizeof(CUtensorMap);
    if (int rc = encode_operand_map(&tmp, b[g], pd.n, pd.k, 1, b_box_rows)) return rc;
    std::memcpy(slot + sizeof(tmp), &tmp, sizeof(tmp));
    if (dual) {
      if (int rc = encode_operand_map(&tmp, b2[g], pd.n, pd.k, 1, b_box_rows)) return rc;
      std::memcpy(slot + 2 * sizeof(tmp), &tmp, sizeof(tmp));
    }
  }
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  if (int rc = deliver_bytes(ws + plan->off_table, staging.data(), table_bytes, stream)) return rc;
  RoutedHeader header = {};
  header.sfa_base = static_cast<const uint8_t*>(sfa);
  header.d_base = static_cast<uint8_t*>(d);
  header.sfd_base = dual ? static_cast<uint8_t*>(sfd) : nullptr;
  header.d_row_bytes = dual ? shape.n / 2 : 2ll * shape.n;
  header.sfa_block_bytes = 512ll * shape.sf_kb;
  header.sfd_block_bytes = 512ll * ceil_div(shape.n, 64);
  header.max_rows = plan->routed_rows;
  if (int rc = deliver_bytes(ws + plan->off_routed, &header, sizeof(header), stream)) return rc;
  {
    std::lock_guard<std::mutex> lock(plan->mutex);
    plan->group_bound = true;
  }
  return 0;
}

}  // namespace

extern "C" {

int nvfp4_group_gemm_bind(const nvfp4_plan* plan, const void* const* a, const void* const* b,
                          const void* const* sfa, const void* const* sfb, void* const* d,
                          void* workspace, void* stream) {
  if (plan == nullptr || plan->kind != kGrouped || plan->maps_per_group != 2 || plan->routed) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "not a grouped GEMM plan");
  }
  return bind_groups(plan, a, b, nullptr, sfa, sfb, nullptr, d, nullptr, workspace, stream);
}

int nvfp4_group_dual_gemm_bind_fp4(const nvfp4_plan* plan, const void* const* a,
                                   const void* const* b1, const void* const* b2,
                                   const void* const* sfa, const void* const* sfb1,
                                   const void* const* sfb2, void* const* d_packed,
                                   void* const* d_scales, void* workspace, void* stream) {
  if (plan == nullptr || plan->kind != kGrouped || plan->maps_per_group != 3 || plan->routed) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "not a grouped dual GEMM plan");
  }
  return bind_groups(plan, a, b1, b2, sfa, sfb1, sfb2, d_packed, d_scales, workspace, stream);
}

int nvfp4_moe_bind(const nvfp4_plan* plan, const void* a, const void* sfa, const void* const* b,
                   const void* const* sfb, const void* const* b2, const void* const* sfb2, void* d,
                   void* d_scales, void* workspace, void* stream) {
  if (plan == nullptr || plan->kind != kGrouped || !plan->routed) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "not a routed plan");
  }
  return bind_routed(plan, a, sfa, b, sfb, b2, sfb2, d, d_scales, workspace, stream);
}

int nvfp4_moe_layout(const nvfp4_plan* plan, const int* counts, void* workspace, void* stream) {
  if (plan == nullptr || plan->kind != kGrouped || !plan->routed) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "not a routed plan");
  }
  if (counts == nullptr || workspace == nullptr || !aligned(workspace, 256) || !aligned(counts, 4)) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "counts or workspace is null or misaligned");
  }
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  moe_layout_kernel<<<1, kMoeMaxExperts, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<ProblemDesc*>(ws + plan->off_table),
      reinterpret_cast<RoutedHeader*>(ws + plan->off_routed), counts,
      static_cast<int>(plan->problems.size()));
  CUDA_TRY(cudaGetLastError());
  return 0;
}

int nvfp4_group_gemm_launch(const nvfp4_plan* plan, void* workspace, void* stream) {
  if (plan == nullptr || plan->kind != kGrouped) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "not a grouped GEMM plan");
  }
  if (workspace == nullptr || !aligned(workspace, 256)) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "workspace is null or not 256-byte aligned");
  }
  {
    std::lock_guard<std::mutex> lock(plan->mutex);
    if (!plan->group_bound) {
      return fail(NVFP4_E_NOT_BOUND, "call nvfp4_group_gemm_bind on a workspace first");
    }
  }
  // The group table and tensor maps live in the workspace, so one plan can serve
  // several bound workspaces (different operand sets of the same shapes).
  KernelParams kp{};
  kp.alpha = nullptr;
  fill_common_params(plan, kp, workspace);
  return launch_plan(plan, kp, stream);
}

int nvfp4_plan_status(const nvfp4_plan* plan, void* workspace, void* stream, int* status) {
  if (plan == nullptr || workspace == nullptr || status == nullptr) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "null argument");
  }
  DeviceGuard guard;
  CUDA_TRY(guard.enter(plan->device));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int value = 0;
  CUDA_TRY(cudaMemcpyAsync(&value, workspace, sizeof(int), cudaMemcpyDeviceToHost, s));
  CUDA_TRY(cudaStreamSynchronize(s));
  *status = value;
  if (plan->routed && value == 0) {
    // A layout whose groups did not fit in the shared buffers cut them: say so once.
    uint8_t* header = static_cast<uint8_t*>(workspace) + plan->off_routed;
    int overflow = 0;
    CUDA_TRY(cudaMemcpyAsync(&overflow, header + offsetof(RoutedHeader, overflow), sizeof(int),
                             cudaMemcpyDeviceToHost, s));
    CUDA_TRY(cudaStreamSynchronize(s));
    if (overflow != 0) {
      CUDA_TRY(cudaMemsetAsync(header + offsetof(RoutedHeader, overflow), 0, sizeof(int), s));
      return fail(NVFP4_E_UNSUPPORTED_SHAPE,
                  "a routed layout needed more than the plan's %d rows; groups were cut",
                  plan->routed_rows);
    }
  }
  if (value != 0) {
    // A launch that gave up may have left tile arrival counters of the stream-K schedule
    // non-zero: clear them with the status word, as nvfp4_plan_init_workspace does, so that
    // the workspace can be used again.
    CUDA_TRY(cudaMemsetAsync(workspace, 0, plan->off_table, s));
    return fail(NVFP4_E_DEVICE_TIMEOUT, "kernel abandoned a bounded wait (code %d)", value);
  }
  return 0;
}

int nvfp4_pack_scales(const void* scales, void* packed, int rows, int cols, int batches,
                      void* stream) {
  if (scales == nullptr || packed == nullptr) return fail(NVFP4_E_INVALID_ARGUMENT, "null operand");
  if (rows < 1 || cols < 1 || batches < 1) {
    return fail(NVFP4_E_UNSUPPORTED_SHAPE, "unsupported scales rows=%d cols=%d batches=%d", rows,
                cols, batches);
  }
  if (!aligned(packed, 16)) return fail(NVFP4_E_MISALIGNED, "packed scales must be 16-byte aligned");
  const long long lines =
      static_cast<long long>(batches) * ceil_div(rows, 128) * ceil_div(cols, 4) * 32;
  const int threads = 256;
  const long long blocks =
      std::min<long long>((lines + threads - 1) / threads, 16ll * current_sm_count());
  pack_scales_kernel<<<static_cast<unsigned int>(blocks), threads, 0,
                       static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(scales), static_cast<uint8_t*>(packed), rows, cols, batches);
  CUDA_TRY(cudaGetLastError());
  return 0;
}

}  // extern "C"

namespace {
template <typename In>
void quantize_dispatch(dim3 grid, dim3 block, cudaStream_t s, int mode, const In* in, uint8_t* p8,
                       uint8_t* s8, int rows, int k, int batches, const int* info) {
  if (mode == kQuantBlocks) {
    quantize_nvfp4_kernel<In, kQuantBlocks><<<grid, block, 0, s>>>(in, p8, s8, rows, k, batches, info);
  } else if (mode == kQuantGather) {
    quantize_nvfp4_kernel<In, kQuantGather><<<grid, block, 0, s>>>(in, p8, s8, rows, k, batches, info);
  } else {
    quantize_nvfp4_kernel<In, kQuantDense><<<grid, block, 0, s>>>(in, p8, s8, rows, k, batches, nullptr);
  }
}

int quantize_launch(const void* x, int x_kind, void* packed, void* scales, int rows, int k,
                    int batches, int mode, const int* info, void* stream) {
  if (x == nullptr || packed == nullptr || scales == nullptr) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "null operand");
  }
  if (x_kind != NVFP4_IN_F32 && x_kind != NVFP4_IN_BF16) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "unknown input kind %d", x_kind);
  }
  if (rows < 1 || k < 16 || batches < 1 || k % 16 != 0) {
    return fail(NVFP4_E_UNSUPPORTED_SHAPE, "unsupported tensor rows=%d k=%d batches=%d", rows, k,
                batches);
  }
  if (!aligned(x, 16) || !aligned(packed, 8) || !aligned(scales, 16)) {
    return fail(NVFP4_E_MISALIGNED, "misaligned operand address");
  }
  // One thread per 16-element block of the padded scale grid; see the kernel for the geometry.
  const dim3 block(kQuantBlocksX, kQuantRowsY, 1);
  const dim3 grid(static_cast<unsigned int>(ceil_div(rows, 128) * (128 / kQuantRowsPerCta)),
                  static_cast<unsigned int>(ceil_div(ceil_div(k / 16, 4) * 4, kQuantBlocksX)),
                  static_cast<unsigned int>(std::min(batches, 65535)));
  if (grid.y > 65535u) {
    return fail(NVFP4_E_UNSUPPORTED_SHAPE, "k=%d is too large for the quantiser", k);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* p8 = static_cast<uint8_t*>(packed);
  uint8_t* s8 = static_cast<uint8_t*>(scales);
  if (x_kind == NVFP4_IN_F32) {
    quantize_dispatch(grid, block, s, mode, static_cast<const float*>(x), p8, s8, rows, k, batches,
                      info);
  } else {
    quantize_dispatch(grid, block, s, mode, static_cast<const __nv_bfloat16*>(x), p8, s8, rows, k,
                      batches, info);
  }
  CUDA_TRY(cudaGetLastError());
  return 0;
}
}  // namespace

extern "C" {

int nvfp4_quantize(const void* x, int x_kind, void* packed, void* scales, int rows, int k,
                   int batches, void* stream) {
  return quantize_launch(x, x_kind, packed, scales, rows, k, batches, kQuantDense, nullptr, stream);
}

int nvfp4_quantize_blocks(const void* x, int x_kind, void* packed, void* scales, int rows, int k,
                          const int* block_rows, void* stream) {
  if (block_rows == nullptr || !aligned(block_rows, 4)) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "block_rows is null or misaligned");
  }
  return quantize_launch(x, x_kind, packed, scales, rows, k, 1, kQuantBlocks, block_rows, stream);
}

int nvfp4_quantize_gather(const void* x, int x_kind, void* packed, void* scales, int rows, int k,
                          const int* source_rows, void* stream) {
  if (source_rows == nullptr || !aligned(source_rows, 4)) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "source_rows is null or misaligned");
  }
  return quantize_launch(x, x_kind, packed, scales, rows, k, 1, kQuantGather, source_rows, stream);
}


int nvfp4_measure_mma_peak(int device, int iters, double* tflops) {
  if (tflops == nullptr || iters < 1 || iters > (1 << 22)) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "bad arguments");
  }
  int sms = 0;
  if (int rc = check_device(device, &sms)) return rc;
  DeviceGuard guard;
  CUDA_TRY(guard.enter(device));
  void* status = nullptr;
  CUDA_TRY(cudaGetSymbolAddress(&status, g_peak_status));
  const int smem = 49 * 1024 + 1024;
  CUDA_TRY(cudaFuncSetAttribute(reinterpret_cast<const void*>(&mma_issue_peak_kernel),
                                cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  cudaStream_t stream = nullptr;
  cudaEvent_t start = nullptr, stop = nullptr;
  CUDA_TRY(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  cudaError_t error = cudaEventCreate(&start);
  if (error == cudaSuccess) error = cudaEventCreate(&stop);
  if (error == cudaSuccess) error = cudaMemsetAsync(status, 0, sizeof(int), stream);
  float best_ms = 0.0f;
  for (int run = 0; run < 3 && error == cudaSuccess; ++run) {  // first run warms up
    error = cudaEventRecord(start, stream);
    if (error != cudaSuccess) break;
    mma_issue_peak_kernel<<<sms, 128, smem, stream>>>(iters, static_cast<int*>(status));
    error = cudaGetLastError();
    if (error == cudaSuccess) error = cudaEventRecord(stop, stream);
    if (error == cudaSuccess) error = cudaEventSynchronize(stop);
    float ms = 0.0f;
    if (error == cudaSuccess) error = cudaEventElapsedTime(&ms, start, stop);
    if (run > 0 && (best_ms == 0.0f || ms < best_ms)) best_ms = ms;
  }
  int abandoned = 0;
  if (error == cudaSuccess) {
    error = cudaMemcpyAsync(&abandoned, status, sizeof(int), cudaMemcpyDeviceToHost, stream);
  }
  if (error == cudaSuccess) error = cudaStreamSynchronize(stream);
  if (start != nullptr) cudaEventDestroy(start);
  if (stop != nullptr) cudaEventDestroy(stop);
  cudaStreamDestroy(stream);
  CUDA_TRY(error);
  if (abandoned != 0 || best_ms <= 0.0f) {
    return fail(NVFP4_E_DEVICE_TIMEOUT, "the measurement kernel abandoned its wait");
  }
  const double flops = 2.0 * 128.0 * 256.0 * 64.0 * 4.0 * iters * sms;
  *tflops = flops / (static_cast<double>(best_ms) * 1e-3) / 1e12;
  return 0;
}

int nvfp4_moe_count(const void* ids, int ids_are_64bit, long long pairs, int experts, int* counts,
                    void* stream) {
  if (ids == nullptr || counts == nullptr) return fail(NVFP4_E_INVALID_ARGUMENT, "null operand");
  if (pairs < 0 || experts < 1 || experts > kMoeMaxExperts) {
    return fail(NVFP4_E_UNSUPPORTED_SHAPE, "unsupported routing: %lld pairs, %d experts (at most %d)",
                pairs, experts, kMoeMaxExperts);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(int) * static_cast<size_t>(experts), s));
  if (pairs == 0) return 0;
  const int threads = 256;
  const unsigned int blocks = static_cast<unsigned int>(
      std::min<long long>((pairs + threads - 1) / threads, 4ll * current_sm_count()));
  if (ids_are_64bit) {
    moe_count_kernel<long long><<<blocks, threads, 0, s>>>(static_cast<const long long*>(ids), pairs,
                                                           experts, counts);
  } else {
    moe_count_kernel<int><<<blocks, threads, 0, s>>>(static_cast<const int*>(ids), pairs, experts,
                                                     counts);
  }
  CUDA_TRY(cudaGetLastError());
  return 0;
}

static int moe_place_common(const void* ids, int ids_are_64bit, long long pairs, int choices,
                            int experts, const int* host_first_rows, const int* device_first_rows,
                            int rows, int* cursors, int* row_of_pair, int* token_of_row,
                            void* stream) {
  if (ids == nullptr || (host_first_rows == nullptr && device_first_rows == nullptr) ||
      cursors == nullptr || row_of_pair == nullptr || token_of_row == nullptr) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "null operand");
  }
  if (pairs < 0 || choices < 1 || rows < 0 || experts < 1 || experts > kMoeMaxExperts) {
    return fail(NVFP4_E_UNSUPPORTED_SHAPE, "unsupported routing: %lld pairs, %d experts (at most %d)",
                pairs, experts, kMoeMaxExperts);
  }
  MoeStarts starts = {};
  for (int e = 0; host_first_rows != nullptr && e < experts; ++e) {
    if (host_first_rows[e] < 0 || host_first_rows[e] > rows) {
      return fail(NVFP4_E_INVALID_ARGUMENT, "expert %d: first row %d outside [0, %d]", e,
                  host_first_rows[e], rows);
    }
    starts.first_row[e] = host_first_rows[e];
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CUDA_TRY(cudaMemsetAsync(cursors, 0, sizeof(int) * static_cast<size_t>(experts), s));
  if (rows > 0) {
    CUDA_TRY(cudaMemsetAsync(token_of_row, 0xFF, sizeof(int) * static_cast<size_t>(rows), s));
  }
  if (pairs == 0) return 0;
  const int threads = 256;
  const unsigned int blocks = static_cast<unsigned int>(
      std::min<long long>((pairs + threads - 1) / threads, 4ll * current_sm_count()));
  if (ids_are_64bit) {
    moe_place_kernel<long long><<<blocks, threads, 0, s>>>(static_cast<const long long*>(ids), pairs,
                                                           choices, experts, starts,
                                                           device_first_rows, cursors, row_of_pair,
                                                           token_of_row);
  } else {
    moe_place_kernel<int><<<blocks, threads, 0, s>>>(static_cast<const int*>(ids), pairs, choices,
                                                     experts, starts, device_first_rows, cursors,
                                                     row_of_pair, token_of_row);
  }
  CUDA_TRY(cudaGetLastError());
  return 0;
}

int nvfp4_moe_place(const void* ids, int ids_are_64bit, long long pairs, int choices, int experts,
                    const int* first_rows, int rows, int* cursors, int* row_of_pair,
                    int* token_of_row, void* stream) {
  if (first_rows == nullptr) return fail(NVFP4_E_INVALID_ARGUMENT, "null operand");
  return moe_place_common(ids, ids_are_64bit, pairs, choices, experts, first_rows, nullptr, rows,
                          cursors, row_of_pair, token_of_row, stream);
}

int nvfp4_moe_place_routed(const void* ids, int ids_are_64bit, long long pairs, int choices,
                           const nvfp4_plan* plan, void* workspace, int* cursors, int* row_of_pair,
                           int* token_of_row, void* stream) {
  if (plan == nullptr || !plan->routed || workspace == nullptr) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "not a routed plan and its workspace");
  }
  const RoutedHeader* header =
      reinterpret_cast<const RoutedHeader*>(static_cast<uint8_t*>(workspace) + plan->off_routed);
  return moe_place_common(ids, ids_are_64bit, pairs, choices,
                          static_cast<int>(plan->problems.size()), nullptr, header->first_rows,
                          plan->routed_rows, cursors, row_of_pair, token_of_row, stream);
}

int nvfp4_moe_combine(const void* y, const int* row_of_pair, const float* weights, float* out,
                      int tokens, int choices, int hidden, void* stream) {
  if (y == nullptr || row_of_pair == nullptr || weights == nullptr || out == nullptr) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "null operand");
  }
  if (tokens < 0 || choices < 1 || hidden < 8 || hidden % 8 != 0) {
    return fail(NVFP4_E_UNSUPPORTED_SHAPE, "unsupported combine: %d tokens, %d choices, hidden %d",
                tokens, choices, hidden);
  }
  if (!aligned(y, 16) || !aligned(out, 16) || !aligned(row_of_pair, 4) || !aligned(weights, 4)) {
    return fail(NVFP4_E_MISALIGNED, "misaligned operand address");
  }
  if (tokens == 0) return 0;
  const int threads = 256;
  const long long work = static_cast<long long>(tokens) * (hidden / 8);
  const unsigned int blocks = static_cast<unsigned int>(
      std::min<long long>((work + threads - 1) / threads, 16ll * current_sm_count()));
  moe_combine_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(y), row_of_pair, weights, out, tokens, choices, hidden);
  CUDA_TRY(cudaGetLastError());
  return 0;
}

int nvfp4_silu_product(const float* h1, const float* h2, void* out, int64_t size, void* stream) {
  if (h1 == nullptr || h2 == nullptr || out == nullptr) {
    return fail(NVFP4_E_INVALID_ARGUMENT, "null operand");
  }
  if (size < 1) return fail(NVFP4_E_UNSUPPORTED_SHAPE, "size must be positive");
  if (!aligned(h1, 4) || !aligned(h2, 4) || !aligned(out, 2)) {
    return fail(NVFP4_E_MISALIGNED, "misaligned operand address");
  }
  const int vector_ok = aligned(h1, 16) && aligned(h2, 16) && aligned(out, 16) ? 1 : 0;
  const int threads = 256;
  const long long work = vector_ok ? (size + 7) / 8 : size;
  const long long blocks =
      std::min<long long>((work + threads - 1) / threads, 16ll * current_sm_count());
  silu_product_kernel<<<static_cast<unsigned int>(blocks), threads, 0,
                        static_cast<cudaStream_t>(stream)>>>(
      h1, h2, static_cast<__half*>(out), static_cast<long long>(size), vector_ok);
  CUDA_TRY(cudaGetLastError());
  return 0;
}

}  // extern "C"
