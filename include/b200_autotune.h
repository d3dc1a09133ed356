/*
 * b200_autotune.h -- C ABI of libb200_autotune.so
 *
 * The shared library holds hand-written sm_100a kernels for the one hot path of
 * awslabs/nki-autotune: C = lhsT^T . rhs and the fused RMSNorm + matmul, plus the
 * per-candidate timing harness the autotune loop calls.  Every entry point is plain C:
 * device pointers travel as void*, the stream as void* (a cudaStream_t), sizes as long.
 * Every function returns a b200_status (0 = OK) and never throws or aborts; the text
 * of the last error on the calling thread is available from b200_last_error().
 *
 * Reference interfaces each entry point stands in for are cited as
 * <file within awslabs/nki-autotune>:<line>.
 */
#ifndef B200_AUTOTUNE_H
#define B200_AUTOTUNE_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ABI_VERSION 1

/* Status codes.  Mirrors the reference's failure classes: a candidate either runs,
 * is rejected for on-chip capacity ("Out of memory in sbuf/psum" upstream,
 * autotune/src/autotune/runner/output.py:236-239) or fails with a message. */
typedef enum b200_status {
  B200_OK = 0,
  B200_ERR_BAD_ARG = 1,       /* NULL pointer, unknown family, misaligned pointer          */
  B200_ERR_BAD_SHAPE = 2,     /* shape/leading dimension the kernels cannot address        */
  B200_ERR_UNSUPPORTED = 3,   /* meta-parameter outside the implemented grid               */
  B200_ERR_SMEM_OOM = 4,      /* pipeline does not fit the 227 KB shared-memory budget      */
  B200_ERR_TMEM_OOM = 5,      /* accumulators do not fit the 512 tensor-memory columns      */
  B200_ERR_CUDA = 6,          /* a CUDA runtime/driver call failed                          */
  B200_ERR_DEVICE_WAIT = 7,   /* a bounded device-side wait expired; see dev_status[]       */
  B200_ERR_WORKSPACE = 8      /* workspace missing or too small                             */
} b200_status;

/* Meta-parameters of one autotune candidate.  These are what the sweep enumerates in
 * place of the reference's schedule transforms (tensorize Split factors, multi-buffer
 * counts, SoftwarePipeline stages, Reorder; the modules under nkigym/src/nkigym/transforms/) and of
 * KernelJob.lnc (autotune/src/autotune/runner/types.py:50). */
typedef struct b200_cfg {
  int tile_m;     /* output-tile rows per CTA group: 128 or 256; 512 with cluster_m 2 (plain GEMM
                     families: two 2-SM UMMAs along M share each B tile, single accumulator buffer) */
  int tile_n;     /* output-tile columns: 64..256, a multiple of 64 per CTA (128 per pair);
                     512 = two 256-column UMMAs side by side (single accumulator buffer)     */
  int tile_k;     /* K extent of one pipeline stage: 64 or 128 (plain GEMM also 32, 96)     */
  int stages;     /* depth of the TMA -> shared-memory ring, 1..12                          */
  int cluster_m;  /* 1, or 2 = a CTA pair along M (tile_m 256 or 512: 2-SM UMMAs)           */
  int cluster_n;  /* 1 (reserved)                                                          */
  int swizzle;    /* tile rasterisation group width along M (1,2,4,8,16); 0 = default      */
  int split_k;    /* plain GEMM families: 2..16 = every tile's K range is dealt to that many work
                     units (fewer if K has fewer k-blocks), their fp32 partial tiles go to scratch
                     (b200_workspace_bytes) and a second kernel sums them in order; for problems
                     with fewer tiles than SMs.  0 or 1 = none                                 */
  int norm_mode;  /* rmsnorm_matmul, M > 16: where the norm is applied.  1 = inline (x tiles are
                     scaled on their way through tensor memory, no scratch), 2 = prologue (the
                     launch first writes x*gamma and rinv to scratch, then runs the plain main
                     loop; needs b200_workspace_bytes of scratch), 0 = prologue when a large
                     enough workspace is passed, else inline                                */
  int reserved[7]; /* zero in normal use.  [0] 1 = test hook: the TMA producer issues nothing, which makes
                     the consumers' bounded waits run out (values 2..4 are measurement hooks that exist
                     only in a library built with -DB200_MEASURE_HOOKS and are ignored otherwise);
                     [1] limit of a device-side wait in microseconds (default 1 s);
                     [2] 1 = GEMM kernel stores its longest CTA lifetime in dev_status[6] (SM cycles)
                     and [7] (nanoseconds); [3] > 0 = cap on the GEMM kernels' grid in CTAs (the
                     persistent schedule deals the tiles to fewer CTAs), for callers that run
                     another kernel, e.g. a collective, beside it; [4] 1 = the M <= 16 fused
                     kernel is launched without the programmatic-dependent-launch attribute
                     (see b200_rmsnorm_matmul)                                                  */
} b200_cfg;

/* Number of ints in a dev_status block (device memory, caller-owned, zeroed by caller).
 * [0] status code (0 or B200_ERR_DEVICE_WAIT)  [1] role that gave up  [2] barrier id
 * [3] tile index  [4] k-block index  [5] blockIdx.x  -- first failure wins. */
#define B200_DEV_STATUS_INTS 8

const char* b200_last_error(void);
int b200_abi_version(void);

/* Number of CUDA devices visible to the process.
 * Stands in for detect_neuron_cores(), autotune/src/autotune/runner/detect.py:7-20. */
int b200_device_count(int* count);

/* Candidate validation without touching the GPU: computes the shared-memory bytes and
 * tensor-memory columns the candidate needs and returns B200_ERR_SMEM_OOM /
 * B200_ERR_TMEM_OOM / B200_ERR_UNSUPPORTED / B200_ERR_BAD_SHAPE when it cannot run.
 * family is "matmul_lhsT_rhs", "matmul_lhs_rhs" or "rmsnorm_matmul".
 * (rmsnorm_matmul, M > 16, norm_mode 0: which variant runs is only decided at the call, by
 * whether scratch is passed; this check then answers for the inline variant -- ask with
 * norm_mode 2 for the variant that runs with scratch, which is what b200_describe_launch
 * describes and what the sweep does.)
 * Stands in for the compile step, compile_one(), autotune/src/autotune/runner/compile.py:197-244:
 * an over-subscribed candidate is a reported failure, never silently dropped. */
int b200_cfg_check(const char* family, const b200_cfg* cfg, long M, long N, long K,
                   long* smem_bytes, int* tmem_cols);

/* Exchange step of the large-M row split (no counterpart upstream, which gathers on the host,
 * autotune/src/autotune/runner/driver.py:97 being one device): copies `bytes` bytes from src (this
 * GPU's memory) to each of the n_peers (<= 8) destinations, which are pointers into OTHER GPUs'
 * memory mapped into this process (CUDA IPC or any other peer mapping; peer access enabled), with
 * plain 16-byte stores over NVLink.  The kernel reads local memory only and waits for nothing;
 * the data is in place when the kernel has completed, so the ranks need a stream-ordered barrier
 * of their own before they read what the others pushed.  max_ctas > 0 caps the grid (to run beside
 * a GEMM).  src, every destination and bytes must be multiples of 16. */
int b200_peer_store(const void* src, void* const* peer_dst, int n_peers, size_t bytes, int max_ctas, void* stream);

/* Maps memory that another process of this node exported (cudaIpcGetMemHandle: 64 bytes) into the
 * address space of the CURRENT device and returns the base of the exported allocation; peer access
 * from the current device to the owner's is turned on if they differ.  The destinations of
 * b200_peer_store must be mapped this way (under the GPU that will run the kernel).
 * b200_ipc_close unmaps. */
int b200_ipc_open(const void* handle64, void** base);
int b200_ipc_close(void* base);

/* The checked build (libb200_autotune_checked.so, compiled with -DB200_CHECKED_BUILD; the same
 * entry points, for debugging, several times slower): every shared-memory, tensor-memory and
 * barrier address, every TMA coordinate and the kernels' global and schedule indices are
 * validated on the device before use.  A failed check records its code, source line, value and
 * limit and the access is skipped -- nothing traps, nothing out of range is touched; a skipped
 * load leaves its consumer to the bounded wait (B200_ERR_DEVICE_WAIT).  This call synchronises
 * the device and returns out4 = {failed checks, first failure's code << 32 | line, its value, its
 * limit}; flags: 1 = clear the record afterwards, 2 = first run a self-test that passes
 * out-of-range arguments to the checks (all refused: 96 failures).  In the normal library it
 * returns B200_ERR_UNSUPPORTED and zeros.  Stands where the reference leans on its simulator's
 * loud legality errors (nkigym/src/nkigym/ops/base.py:191-215). */
int b200_checked_build_report(long long* out4, int flags);

/* Describes, without launching anything, what a launch of this candidate at this shape is: one
 * JSON object in out[out_bytes] (NUL-terminated) with the kernel variant, grid, cluster, threads,
 * shared-memory bytes, tensor-memory columns, tiles / CTA groups / waves of the persistent schedule,
 * the UMMA-issue-bound SM cycles of the busiest CTA group, and the compiled kernel's registers and
 * local-memory bytes (null without a device).  This is what a detailed profile stores per candidate
 * in place of the reference's per-instruction profile JSON and NEFF
 * (autotune/src/autotune/runner/benchmark.py:81-84, 90-113; output.py:176-199). */
int b200_describe_launch(const char* family, const b200_cfg* cfg, long M, long N, long K,
                         char* out, size_t out_bytes);

/* The candidate the library uses when an entry point is called with cfg == NULL, for this family
 * and shape (the fused family: norm_mode 0 and the tile of the variant that runs without scratch).
 * The reference has no counterpart: its hand kernels carry fixed tile constants
 * (kernel_library/matmul/lhsT_rhs/kernel_hand_90.92mfu.py:103-105). */
int b200_default_cfg(const char* family, long M, long N, long K, b200_cfg* cfg);

/* Bytes of device scratch the candidate can use (0 when it needs none).  The scratch must be
 * zero-filled once before first use; the kernels leave it reusable for the next launch.  After
 * a launch that ended with B200_ERR_DEVICE_WAIT its contents are undefined: zero it again.
 * Launches that share one scratch buffer must not overlap on the GPU. */
size_t b200_workspace_bytes(const char* family, const b200_cfg* cfg, long M, long N, long K);

/* C[M,N] (bf16, row stride ld_out) = lhsT[K,M]^T . rhs[K,N], bf16 operands, fp32
 * accumulation in tensor memory over the whole of K, bf16 result.
 * lhsT has M contiguous (row stride ld_lhsT elements), rhs has N contiguous.
 * Replaces matmul_lhsT_rhs_nkigym, kernel_library/matmul/lhsT_rhs/kernel_hand_90.92mfu.py:101-131.
 * Asynchronous on `stream`; dev_status may be NULL. */
int b200_matmul_lhsT_rhs(const void* lhsT, const void* rhs, void* out,
                         long M, long N, long K, long ld_lhsT, long ld_rhs, long ld_out,
                         const b200_cfg* cfg, void* workspace, size_t workspace_bytes,
                         int* dev_status, void* stream);

/* C[M,N] (bf16) = lhs[M,K] . rhs[K,N] with lhs K-contiguous (row stride ld_lhs): the same
 * kernel with a K-major A operand; no transpose pass is needed on this hardware.
 * Replaces matmul_lhs_rhs_nkigym, kernel_library/matmul/lhs_rhs/kernel_handtuned_89.26mfu.py:226-287. */
int b200_matmul_lhs_rhs(const void* lhs, const void* rhs, void* out,
                        long M, long N, long K, long ld_lhs, long ld_rhs, long ld_out,
                        const b200_cfg* cfg, void* workspace, size_t workspace_bytes,
                        int* dev_status, void* stream);

/* Same contraction in fp32 on the CUDA cores (no tensor cores, no tf32): the 1e-5
 * configuration and the on-device cross-check for the tensor-core candidates.
 * Follows NKIMatmul._run, nkigym/src/nkigym/ops/matmul.py:43-45
 * (stationary.astype(f32).T @ moving.astype(f32)). */
int b200_matmul_lhsT_rhs_f32(const void* lhsT, const void* rhs, void* out,
                             long M, long N, long K, long ld_lhsT, long ld_rhs, long ld_out,
                             void* stream);

/* out[M,N] (bf16) = (x / sqrt(mean_k x^2 + eps) * gamma) . w with x[M,K] (K contiguous),
 * gamma[K] (bf16, may be NULL = all ones), w[K,N] (N contiguous); row statistics and
 * accumulation in fp32.  M <= 16 runs the weight-streaming kernel (only tile_k and stages of
 * cfg apply) and needs b200_workspace_bytes of zero-filled scratch (partial tiles of the
 * 256-column tiles that are shared between CTAs, and their counters); M > 16 see b200_cfg.norm_mode.
 * Replaces rmsnorm_matmul_online, kernel_library/rmsnorm_matmul/kernel_hand_online.py:198-353
 * (gamma is an extension; gamma == NULL reproduces that kernel's maths).
 * The M <= 16 kernel is a programmatic dependent launch: it may begin, and stream w, while the
 * kernel launched before it on the same stream is still finishing; it waits for that kernel before it
 * reads x or gamma, touches the workspace or writes out.  So w must not be written by the kernel
 * launched immediately before this call on `stream` (weights are static in the decode loops this
 * kernel is for); if it is, set b200_cfg.reserved[4] = 1 and the launch is an ordinary one. */
int b200_rmsnorm_matmul(const void* x, const void* gamma, const void* w, void* out,
                        long M, long N, long K, float eps,
                        const b200_cfg* cfg, void* workspace, size_t workspace_bytes,
                        int* dev_status, void* stream);

/* Largest N served by b200_rmsnorm_matmul_noalloc. */
#define B200_NOALLOC_MAX_N 32768

/* The M <= 16 case of b200_rmsnorm_matmul for callers that cannot allocate device memory at the
 * call site (an engine that has handed the whole device heap to its own pools, a thread that
 * must stay out of the allocator's locks): the kernel's scratch lives in a static device array
 * inside the library (one 16 x 256 fp32 partial tile per 256-column tile and per CTA at
 * B200_NOALLOC_MAX_N, plus counters: about 4.7 MB, held by every GPU that loads the library until
 * the process exits) instead of a caller workspace.  No cudaMalloc,
 * cudaFree or other allocating call is made.  Requires 1 <= M <= 16 and N <= B200_NOALLOC_MAX_N
 * (otherwise B200_ERR_BAD_SHAPE).  The first call on each device resolves the array's device
 * address; make that call outside any stream capture.  All calls on a device share the one
 * array: each call clears the counters it uses on `stream` first, and two calls that can overlap
 * on the GPU (different streams without ordering) race and give wrong results.
 * No counterpart in the reference. */
int b200_rmsnorm_matmul_noalloc(const void* x, const void* gamma, const void* w, void* out,
                                long M, long N, long K, float eps, const b200_cfg* cfg,
                                int* dev_status, void* stream);

/* fp32 CUDA-core evaluation of the same fused expression on bf16 inputs (fp32 output),
 * used as the on-device cross-check of b200_rmsnorm_matmul. */
int b200_rmsnorm_matmul_f32(const void* x, const void* gamma, const void* w, void* out_f32,
                            long M, long N, long K, float eps, void* stream);

/* Times one candidate: `warmup` untimed launches, then `iters` launches each bracketed
 * by CUDA events on `stream`; ms_each[iters] receives the per-launch milliseconds.
 * Between launches a scratch buffer of flush_bytes (may be 0/NULL) is overwritten so
 * that operands are not L2-resident from the previous launch.  The launch itself is
 * the same code path as b200_matmul_lhsT_rhs / b200_rmsnorm_matmul.
 * Stands in for benchmark_one() + extract_perf_metrics,
 * autotune/src/autotune/runner/benchmark.py:116-153 and :58-87. */
typedef struct b200_problem {
  const char* family;          /* "matmul_lhsT_rhs" | "matmul_lhs_rhs" | "rmsnorm_matmul"   */
  const void* a;               /* lhsT[K,M], lhs[M,K] or x[M,K]                            */
  const void* b;               /* rhs[K,N]  or w[K,N]                                      */
  const void* gamma;           /* rmsnorm only, may be NULL                                */
  void* out;
  long M, N, K;
  long ld_a, ld_b, ld_out;     /* 0 = dense                                                */
  float eps;
  int reserved[7];
} b200_problem;

int b200_time_kernel(const b200_problem* p, const b200_cfg* cfg,
                     void* workspace, size_t workspace_bytes, int* dev_status,
                     void* flush_buf, size_t flush_bytes,
                     int warmup, int iters, float* ms_each, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_AUTOTUNE_H */
