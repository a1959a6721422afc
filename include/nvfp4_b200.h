/*
 * C ABI of the B200 (sm_100a) NVFP4 block-scaled GEMM family: dense/batched GEMM,
 * fused dual GEMM with silu gate, ragged grouped GEMM, and the two glue kernels of
 * the dual-GEMM pipeline. Each entry point names the interface of
 * Aalanli/flashinfer-cubins it stands in for (file:line within that project).
 *
 * Conventions
 *   - Every function returns an int status and never throws, aborts or traps:
 *       0   success
 *      <0   invalid argument (NVFP4_E_*); nothing was launched
 *      >0   a CUDA runtime/driver error code (cudaError_t / CUresult)
 *     nvfp4_last_error() returns text for the calling thread's last failure.
 *   - All data pointers are device pointers on the plan's device unless the
 *     parameter is documented as host memory. Launches are asynchronous on the
 *     stream passed in (a cudaStream_t passed as void*).
 *   - The library allocates no device memory: a plan reports the workspace it needs
 *     (nvfp4_plan_workspace_bytes) and the caller passes that buffer to every
 *     launch. The workspace must be initialised once with nvfp4_plan_init_workspace
 *     (it zeroes the status word and the per-tile arrival counters) and must not be
 *     shared by launches that can overlap on the GPU.
 *   - A plan is immutable once created. Launches of one plan may be issued from several
 *     host threads and on several streams at the same time, each with its own workspace;
 *     the only state a launch shares is a mutex-guarded cache of encoded tensor maps
 *     keyed by the operand addresses. nvfp4_plan_destroy must not race with a launch.
 *   - Operand layout (harness/workloads/quantization.py:1-37): packed E2M1 bytes,
 *     low nibble = even K index, K contiguous, storage [batch][rows][k/2]; UE4M3
 *     scales, one per 16 K elements, in the blocked layout
 *     [batch][ceil(rows/128)][ceil(k/64)][32][4][4] (quantization.py:90-102);
 *     output [batch][m][n] row-major.
 */
#ifndef NVFP4_B200_H_
#define NVFP4_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NVFP4_E_INVALID_ARGUMENT (-1) /* null pointer, bad enum, bad handle */
#define NVFP4_E_UNSUPPORTED_SHAPE (-2) /* m,n,k,l < 1, k % 32, n alignment, int32 range */
#define NVFP4_E_MISALIGNED (-3)        /* operand not 16-byte aligned (alpha: 4) */
#define NVFP4_E_UNSUPPORTED_DEVICE (-4) /* not compute capability 10.0 */
#define NVFP4_E_DEVICE_TIMEOUT (-5)    /* a kernel abandoned a bounded wait (status word) */
#define NVFP4_E_NOT_BOUND (-6)         /* grouped launch before nvfp4_group_gemm_bind */
#define NVFP4_E_SCRATCH_TOO_LARGE (-7) /* plan needs more than the built-in scratch array */

/* Output/element kinds of a plan. */
#define NVFP4_OUT_F16 0 /* nvfp4_gemm: FP16 D (harness/workloads/nvfp4_gemm.py:511-530) */
#define NVFP4_OUT_F32 1 /* nvfp4_dual_gemm_gemm: FP32 D (nvfp4_dual_gemm.py:172-188) */
#define NVFP4_OUT_FP4 2 /* D quantised to NVFP4 in the epilogue; launched by nvfp4_gemm_launch_fp4 */
#define NVFP4_OUT_BF16 3 /* BF16 D, the output type of FlashInfer's mm_fp4 path
                            (harness/workloads/batched_gemm/__init__.py:3-7); nvfp4_gemm_launch */

/* Optional tuning overrides; zero/negative fields mean "choose automatically". */
typedef struct nvfp4_config {
  int tile_n;   /* 64, 128 or 256 */
  int schedule; /* 1 = data parallel (whole tiles), 2 = stream-K (split along K, partials
                   through the workspace), 3 = cluster split-K (partials through peer
                   shared memory; dense and dual GEMM with fewer tiles than SMs only) */
  int ctas;     /* persistent grid size, at most the SM count */
  int pair;     /* dense and dual GEMM: 1 = 256 x 256 tiles (dual: 256 x 128 output tiles) on
                   pairs of CTAs (tcgen05.mma cta_group::2), -1 = never, 0 = automatic */
} nvfp4_config;

/* What a plan decided; filled by nvfp4_plan_info. */
typedef struct nvfp4_plan_info {
  int tile_m, tile_n, tile_k;
  int stages;
  int schedule; /* 1 data parallel, 2 stream-K, 3 cluster split-K */
  int ctas;
  int threads;
  int smem_bytes;
  int64_t tiles;
  int64_t units; /* (tile, 256-wide k-tile) units */
  int sm_count;
} nvfp4_plan_info;

typedef struct nvfp4_plan nvfp4_plan;

/* Library version, major * 1000 + minor. */
int nvfp4_version(void);

/* Text of the calling thread's last error ("" if none). */
const char* nvfp4_last_error(void);

/* 1 if CUDA device `device` can run these kernels (compute capability 10.0), 0 if
 * not, <0 / >0 on error. Replaces Workload.is_supported / _check_supported
 * (harness/workload.py:410-416, harness/workloads/nvfp4_gemm.py:440-443): the check
 * runs on the host, nothing is launched on an unsupported device. */
int nvfp4_device_supported(int device);

/* Dense/batched GEMM plan: D[l] = alpha * (A[l]*SFA[l]) (B[l]*SFB[l])^T.
 * Replaces CutlassFp4Gemm.build_params' shape validation, scheduler and grid choice
 * (harness/workloads/nvfp4_gemm.py:198-387). Requires m,n,k,l >= 1, k % 32 == 0,
 * (n * sizeof(out)) % 16 == 0. */
int nvfp4_gemm_plan_create(nvfp4_plan** plan, int device, int out_kind, int m, int n, int k,
                           int l, const nvfp4_config* config);

/* Dense GEMM plan whose B operand is in the layout FlashInfer prepares for its trtllm-gen
 * `mm_fp4` kernels (`nvfp4_quantize(..., do_shuffle=True)`; the reference's
 * harness/workloads/batched_gemm/trtllm.py:257-288 with formats.py:143-161): the rows of B,
 * and the rows of its scales before they are put into the blocked layout, are permuted inside
 * blocks of `shuffle_block` rows (32 when the producing kernel's epilogue tile is a multiple
 * of 128 rows, else 16), physical row base + map[o] holding logical row base + o. D comes out
 * in logical column order: the epilogue undoes the permutation in registers. Launched with
 * nvfp4_gemm_launch; n must be a multiple of `shuffle_block`; NVFP4_OUT_BF16 is the output
 * type of that path, FP16 and FP32 work as well. */
int nvfp4_gemm_plan_create_shuffled(nvfp4_plan** plan, int device, int out_kind, int m, int n,
                                    int k, int l, int shuffle_block, const nvfp4_config* config);

/* Fused dual GEMM plan: D = half(silu(alpha*A*B1^T) * (alpha*A*B2^T)). The reference
 * runs this as two GEMM launches plus silu_product
 * (harness/workloads/nvfp4_dual_gemm.py:1-30, resources/nvfp4_dual_gemm/task.yml:12-26);
 * here it is one launch. Output FP16, n % 4 == 0 (as for the FP32 stage). */
int nvfp4_dual_gemm_plan_create(nvfp4_plan** plan, int device, int m, int n, int k, int l,
                                const nvfp4_config* config);

/* Grouped GEMM plan for `groups` independent problems; `mnk` is host memory,
 * 3 * groups ints (m_g, n_g, k_g). Replaces NVFP4GroupGEMM.build_params /
 * array_bytes (harness/workloads/nvfp4_group_gemm.py:250-501). Output FP16. */
int nvfp4_group_gemm_plan_create(nvfp4_plan** plan, int device, int groups, const int* mnk,
                                 const nvfp4_config* config);

void nvfp4_plan_destroy(nvfp4_plan* plan);

/* Bytes of caller-provided device workspace the plan's launches need (>= 256). */
size_t nvfp4_plan_workspace_bytes(const nvfp4_plan* plan);

/* Zeroes the workspace's status word and arrival counters; call once per workspace
 * before the first launch (stream-ordered). */
int nvfp4_plan_init_workspace(const nvfp4_plan* plan, void* workspace, void* stream);

int nvfp4_plan_info_get(const nvfp4_plan* plan, nvfp4_plan_info* info);

/* One dense GEMM launch. Replaces CutlassFp4Gemm.launch_config + _launch
 * (harness/workloads/nvfp4_gemm.py:395-435). `alpha` is a device FP32 scalar read by
 * the kernel (nvfp4_gemm.py:35-39); `d` is FP16, BF16 or FP32 per the plan. Tensor maps
 * are encoded once per set of operand addresses (the plan remembers the sixteen most
 * recently used sets). */
int nvfp4_gemm_launch(const nvfp4_plan* plan, const void* a, const void* b, const void* sfa,
                      const void* sfb, const float* alpha, void* d, void* workspace,
                      void* stream);

/* Dense GEMM whose output is quantised to NVFP4 in the epilogue, so that it can be the A
 * operand of the next GEMM without an FP16 round trip (plan created with NVFP4_OUT_FP4;
 * n % 64 == 0; data-parallel schedule, on single CTAs or on pairs). The reference has no
 * such kernel on this path: its
 * NVFP4 convention for a quantised tensor (scale = e4m3(amax / 6) per 16 elements, RNE
 * E2M1 codes, blocked scales: harness/workloads/quantization.py:66-116 and 39-63) is what
 * the bytes follow. `d_packed` is [l][m][n/2] bytes, `d_scales` the blocked layout
 * [l][ceil(m/128)][n/64][32][4][4]; rows beyond m in the last atom row are not written.
 * The result equals nvfp4_quantize applied to the FP32 product alpha * A * B^T. */
int nvfp4_gemm_launch_fp4(const nvfp4_plan* plan, const void* a, const void* b, const void* sfa,
                          const void* sfb, const float* alpha, void* d_packed, void* d_scales,
                          void* workspace, void* stream);

/* The fused dual GEMM with its gated output quantised to NVFP4 in the epilogue: gate/up
 * projection -> packed E2M1 + blocked scales that the down projection's GEMM takes as its A
 * operand. Same conventions as nvfp4_gemm_launch_fp4 (n % 64 == 0, data-parallel
 * schedule); silu is evaluated with ex2.approx / rcp.approx, so codes at E2M1
 * rounding boundaries can differ from an exactly rounded silu. No counterpart in the
 * reference. */
int nvfp4_dual_gemm_plan_create_fp4(nvfp4_plan** plan, int device, int m, int n, int k, int l,
                                    const nvfp4_config* config);
int nvfp4_dual_gemm_launch_fp4(const nvfp4_plan* plan, const void* a, const void* b1, const void* b2,
                               const void* sfa, const void* sfb1, const void* sfb2,
                               const float* alpha, void* d_packed, void* d_scales,
                               void* workspace, void* stream);

/* The dense launch for callers that must not allocate device memory where they call
 * this library (a runtime whose own pool owns all of HBM, a plugin under a foreign
 * allocator, a hot path that bans cudaMalloc because it synchronises the device). It has
 * no counterpart in the reference. Same operands as nvfp4_gemm_launch, but the scratch a
 * split-K schedule needs is a 24 MiB array inside the library
 * (nvfp4_static_scratch_bytes()), which every GPU that loads the library holds until the
 * process exits. A plan whose nvfp4_plan_workspace_bytes() exceeds that is refused with
 * NVFP4_E_SCRATCH_TOO_LARGE; nothing is launched. The call allocates nothing: it zeroes
 * the status word and the plan's tile counters in the array (stream-ordered), then
 * launches. The first call on a device also looks the array's address up; make that
 * first call before any stream capture begins. All calls on a device share the one
 * array, so two such launches that can overlap on the GPU (different streams, no
 * ordering between them) race. The status word of these launches is read with
 * nvfp4_static_status, not nvfp4_plan_status. */
int nvfp4_gemm_launch_static(const nvfp4_plan* plan, const void* a, const void* b, const void* sfa,
                             const void* sfb, const float* alpha, void* d, void* stream);

/* Size in bytes of the built-in scratch array used by nvfp4_gemm_launch_static. */
size_t nvfp4_static_scratch_bytes(void);

/* Synchronises `stream` and reads the status word that nvfp4_gemm_launch_static launches
 * on `device` share into *status; returns NVFP4_E_DEVICE_TIMEOUT if a launch abandoned a
 * bounded wait since the word was last cleared (every nvfp4_gemm_launch_static clears it
 * before it launches). Allocates nothing. No counterpart in the reference. */
int nvfp4_static_status(int device, void* stream, int* status);

/* One fused dual-GEMM launch (see nvfp4_dual_gemm_plan_create). `d` must be 16-byte
 * aligned, except that rows of n % 8 == 4 FP16 elements need only 8 bytes. */
int nvfp4_dual_gemm_launch(const nvfp4_plan* plan, const void* a, const void* b1, const void* b2,
                           const void* sfa, const void* sfb1, const void* sfb2,
                           const float* alpha, void* d, void* workspace, void* stream);

/* Records the groups' device pointers (host arrays of `groups` pointers each),
 * encodes the per-group tensor maps and writes the group table into the workspace,
 * stream-ordered, by small kernel launches that carry the table as parameters (so the
 * call neither synchronises nor depends on host memory after it returns, and can be
 * captured in a graph). Replaces NVFP4GroupGEMM.launch_config
 * (harness/workloads/nvfp4_group_gemm.py:514-591). */
int nvfp4_group_gemm_bind(const nvfp4_plan* plan, const void* const* a, const void* const* b,
                          const void* const* sfa, const void* const* sfb, void* const* d,
                          void* workspace, void* stream);

/* Grouped fused dual GEMM with NVFP4 output, the gate/up projection of a mixture-of-experts
 * layer in one launch: for every group g, D_g = quantise(silu(A_g B1_g^T) * (A_g B2_g^T)) as
 * packed E2M1 [m_g][n_g/2] plus blocked UE4M3 scales [ceil(m_g/128)][n_g/64][32][4][4], ready
 * to be the A operand of the grouped down projection (nvfp4_group_gemm_*). `mnk` as for
 * nvfp4_group_gemm_plan_create (n_g = rows of each B_g, a multiple of 64); data-parallel
 * schedule; silu evaluated as in nvfp4_dual_gemm_launch_fp4. Bound with
 * nvfp4_group_dual_gemm_bind_fp4 (host arrays of `groups` device pointers each) and launched
 * with nvfp4_group_gemm_launch. The reference has no grouped dual kernel: its grouped cases
 * are sized as the expert shards of such a layer (harness/workloads/nvfp4_group_gemm.py:751-785)
 * and its FP8 MoE workload runs the two projections as separate launches
 * (harness/workloads/moe.py:1-33). */
int nvfp4_group_dual_gemm_plan_create_fp4(nvfp4_plan** plan, int device, int groups,
                                          const int* mnk, const nvfp4_config* config);
int nvfp4_group_dual_gemm_bind_fp4(const nvfp4_plan* plan, const void* const* a,
                                   const void* const* b1, const void* const* b2,
                                   const void* const* sfa, const void* const* sfb1,
                                   const void* const* sfb2, void* const* d_packed,
                                   void* const* d_scales, void* workspace, void* stream);

/* One launch covering every group, reading the group table that
 * nvfp4_group_gemm_bind wrote into `workspace` (one plan may be bound to several
 * workspaces, one per operand set). The table holds the operands' addresses: every buffer
 * named at the bind must stay allocated while launches on that workspace can still run.
 * Replaces NVFP4GroupGEMM._launch
 * (harness/workloads/nvfp4_group_gemm.py:593-600). */
int nvfp4_group_gemm_launch(const nvfp4_plan* plan, void* workspace, void* stream);

/* Synchronises `stream` and reads the workspace's status word into *status. If it was
 * non-zero (a kernel abandoned a bounded wait), returns NVFP4_E_DEVICE_TIMEOUT and
 * re-initialises the workspace's status word and tile arrival counters (stream-ordered),
 * so that the workspace can be launched on again; the output of the abandoned launch is
 * undefined. */
int nvfp4_plan_status(const nvfp4_plan* plan, void* workspace, void* stream, int* status);

/* Failure-detection self-test, with no counterpart in the reference: launches the dense
 * kernel of `plan` (FP16 output, 128-column tiles, data-parallel or stream-K schedule; same
 * operands as nvfp4_gemm_launch) in a build whose producer issues no copy and whose waits
 * give up after a few milliseconds. Every role then abandons a wait: the kernel records the
 * first role's code in the workspace's status word, stops, frees its tensor memory and
 * returns by itself; D is left unwritten. nvfp4_plan_status afterwards returns
 * NVFP4_E_DEVICE_TIMEOUT and re-initialises the workspace, and the next nvfp4_gemm_launch
 * on it is correct. Nothing faults and nothing waits without a bound. */
int nvfp4_selftest_abandoned_wait(const nvfp4_plan* plan, const void* a, const void* b,
                                  const void* sfa, const void* sfb, const float* alpha, void* d,
                                  void* workspace, void* stream);

/* Logical E4M3 scales [batches][rows][cols] -> blocked layout, zero padded, flat
 * [batches][round_up(rows,128) * round_up(cols,4)]. Replaces the pack_scales kernel
 * (impls/nvfp4_dual_gemm/kernels/pack_scales.cu:9-19,
 * harness/workloads/nvfp4_dual_gemm.py:269-296). */
int nvfp4_pack_scales(const void* scales, void* packed, int rows, int cols, int batches,
                      void* stream);

/* Input kinds of nvfp4_quantize. */
#define NVFP4_IN_F32 0
#define NVFP4_IN_BF16 1

/* FP32 or BF16 x[batches][rows][k] -> NVFP4: packed E2M1 [batches][rows][k/2] and UE4M3
 * scales written straight into the blocked layout (zero padded). Per 16-element K block
 * scale = e4m3(amax / 6) (round to nearest even, saturating) and each element is the
 * round-to-nearest-even E2M1 code of x / scale; a zero scale gives zero codes. The step
 * before the GEMMs (the reference takes pre-quantised inputs); follows the reference's
 * NVFP4 convention (harness/workloads/batched_gemm/trtllm.py:530-547, formats.py:57-82)
 * and replaces a separate relayout pass (impls/nvfp4_dual_gemm/kernels/pack_scales.cu:9-19).
 * Requires k % 16 == 0; x 16-byte aligned. */
int nvfp4_quantize(const void* x, int x_kind, void* packed, void* scales, int rows, int k,
                   int batches, void* stream);

/* The same for rows that come in 128-row blocks of which only the first block_rows[b] rows
 * hold data (the permuted rows of a mixture-of-experts layer, every expert's rows padded to
 * whole blocks): `block_rows` is a device array of ceil(rows / 128) counts in [0, 128]. Rows
 * beyond a block's count are neither read nor written: their codes and scales keep what the
 * buffers held (zeros, in buffers that were zeroed once). One batch. */
int nvfp4_quantize_blocks(const void* x, int x_kind, void* packed, void* scales, int rows, int k,
                          const int* block_rows, void* stream);

/* Gather and quantise: output row r (of `rows`) is the quantised row source_rows[r] of x
 * ([any number of rows][k]), or, where source_rows[r] < 0, nothing: such rows are neither read
 * nor written. `source_rows` is a device array of `rows` ints. The dispatch of a
 * mixture-of-experts layer (token rows permuted by expert, blocks padded to 128 rows) without
 * a permuted copy of the activations. */
int nvfp4_quantize_gather(const void* x, int x_kind, void* packed, void* scales, int rows, int k,
                          const int* source_rows, void* stream);

/* Routing of a mixture-of-experts layer whose experts' rows are kept in blocks padded to
 * whole 128-row blocks (what the grouped plans and nvfp4_quantize_gather take), around the
 * one host read that the plans' shapes need. `ids` is a device array of `pairs` expert ids
 * (int32, or int64 if ids_are_64bit), pair i = (token i / choices, choice i % choices); at most
 * 512 experts.
 *   nvfp4_moe_count: counts[e] (device, `experts` ints) = number of pairs with id e.
 *   nvfp4_moe_place: with first_rows[e] (HOST array: the caller's prefix over the counts
 *     padded to 128) every pair gets a row of its expert's block: row_of_pair[i] (device,
 *     `pairs` ints) and token_of_row[row] = i / choices (device, `rows` ints, -1 for the rows
 *     that hold no pair). `cursors` is device scratch of `experts` ints. Which pair gets which
 *     row of a block may differ from run to run; the layer's result does not depend on it.
 * The reference routes on the host (harness/workloads/moe.py:1-33 describes its FP8 layer's
 * stages); no counterpart on this path. */
int nvfp4_moe_count(const void* ids, int ids_are_64bit, long long pairs, int experts, int* counts,
                    void* stream);
int nvfp4_moe_place(const void* ids, int ids_are_64bit, long long pairs, int choices, int experts,
                    const int* first_rows, int rows, int* cursors, int* row_of_pair,
                    int* token_of_row, void* stream);

/* Grouped GEMMs whose groups' row counts are decided on the device (the experts of a
 * mixture-of-experts layer under a routing that changes with every forward): one plan and one
 * bind for the life of the layer, no host read of the counts, every step a plain launch, so the
 * whole forward can be captured in a CUDA graph.
 *   nvfp4_moe_plan_create: `experts` groups of [m_g, n, k] with m_g unknown; out_kind
 *     NVFP4_OUT_FP4 = the gate/up dual GEMM with NVFP4 output (n = rows of each of B1, B2, a
 *     multiple of 64), NVFP4_OUT_F16 = a GEMM with FP16 output. All groups share one A buffer,
 *     one D buffer (and their scale buffers) of `max_rows` rows (a multiple of 128): group g
 *     owns a block of ceil(m_g / 128) * 128 rows, blocks in group order.
 *   nvfp4_moe_bind: the shared buffers (a packed [max_rows][k/2], sfa blocked
 *     [max_rows/128][ceil(k/64)][32][4][4], d [max_rows][n] FP16 or packed [max_rows][n/2] with
 *     d_scales [max_rows/128][n/64][32][4][4]) and every expert's weights and scales (host
 *     arrays of `experts` device pointers; b2 / sfb2 / d_scales for NVFP4_OUT_FP4 only).
 *   nvfp4_moe_layout: from `counts` (device, `experts` ints, e.g. nvfp4_moe_count's) fills in
 *     the groups' rows, first rows, tile counts and addresses in the workspace. Groups that do
 *     not fit in max_rows are cut (callers size max_rows as pairs + 127 * experts, rounded up);
 *     nvfp4_plan_status then reports NVFP4_E_UNSUPPORTED_SHAPE once.
 *   nvfp4_moe_place_routed: nvfp4_moe_place with the first rows that nvfp4_moe_layout wrote
 *     (`rows` = max_rows; token_of_row has max_rows entries).
 *   nvfp4_group_gemm_launch launches the plan. Rows of a block beyond m_g are neither
 *     meaningful on input nor written on output.
 * No counterpart in the reference, whose grouped launch takes its shapes from the host
 * (harness/workloads/nvfp4_group_gemm.py:514-591). */
int nvfp4_moe_plan_create(nvfp4_plan** plan, int device, int experts, int n, int k, int max_rows,
                          int out_kind, const nvfp4_config* config);
int nvfp4_moe_bind(const nvfp4_plan* plan, const void* a, const void* sfa, const void* const* b,
                   const void* const* sfb, const void* const* b2, const void* const* sfb2, void* d,
                   void* d_scales, void* workspace, void* stream);
int nvfp4_moe_layout(const nvfp4_plan* plan, const int* counts, void* workspace, void* stream);
int nvfp4_moe_place_routed(const void* ids, int ids_are_64bit, long long pairs, int choices,
                           const nvfp4_plan* plan, void* workspace, int* cursors, int* row_of_pair,
                           int* token_of_row, void* stream);

/* The combine of that layer: out[t][:] = sum over j of weights[t][j] * y[row_of_pair[t * choices
 * + j]][:] in FP32 (`out` [tokens][hidden] FP32, `y` FP16 rows of `hidden` columns, `weights`
 * [tokens][choices] FP32, `row_of_pair` as nvfp4_moe_place wrote it; a negative row adds
 * nothing). hidden % 8 == 0; y and out 16-byte aligned. */
int nvfp4_moe_combine(const void* y, const int* row_of_pair, const float* weights, float* out,
                      int tokens, int choices, int hidden, void* stream);

/* out[i] = half(silu(h1[i]) * h2[i]) over `size` FP32 elements. Replaces the
 * silu_product kernel (impls/nvfp4_dual_gemm/kernels/silu_product.cu:7-9,
 * harness/workloads/nvfp4_dual_gemm.py:352-367). */
int nvfp4_silu_product(const float* h1, const float* h2, void* out, int64_t size, void* stream);

/* Measures the issue rate of the block-scaled FP4 MMA on `device`: one CTA per SM issues
 * `iters` x 4 tcgen05.mma (128 x 256 x 64) back to back from shared memory with nothing else
 * running, and *tflops receives the aggregate TFLOP/s of the best of two timed launches. It
 * is the measured denominator for the tensor-bound rooflines next to the nominal 9 PFLOP/s;
 * the reference has no counterpart. Synchronous; uses its own stream. */
int nvfp4_measure_mma_peak(int device, int iters, double* tflops);

#ifdef __cplusplus
}
#endif

#endif /* NVFP4_B200_H_ */
