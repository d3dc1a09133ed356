// Host side of libb200_autotune.so: candidate validation, tensor-map construction, launches of
// the tcgen05 kernels, and the CUDA-event timing harness.  Plain C ABI (include/b200_autotune.h).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "gemm_tcgen05.cuh"
#include "rmsnorm_tcgen05.cuh"
#include "rmsnorm_skinny.cuh"
#include "host_api.h"

namespace b200 {

// ---------------------------------------------------------------------------- errors
static thread_local char g_last_error[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return B200_OK;
  return set_error(B200_ERR_CUDA, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}

// ---------------------------------------------------------------------------- plan
constexpr long SMEM_BUDGET = 232448;  // 227 KB: largest opt-in dynamic shared memory per CTA

enum Family { FAM_LHST = 0, FAM_RMSNORM = 1, FAM_LHS = 2, FAM_UNKNOWN = -1 };

static Family parse_family(const char* family) {
  if (family == nullptr) return FAM_UNKNOWN;
  if (strcmp(family, "matmul_lhsT_rhs") == 0) return FAM_LHST;
  if (strcmp(family, "rmsnorm_matmul") == 0) return FAM_RMSNORM;
  if (strcmp(family, "matmul_lhs_rhs") == 0) return FAM_LHS;
  return FAM_UNKNOWN;
}

struct Plan {
  int cta_group;   // 1, or 2 = one UMMA across a CTA pair
  int m_sub;       // 128-row accumulator blocks per CTA
  int cluster;     // launch cluster size
  int tile_m, tile_n, tile_k, stages, group_m;
  int acc_bufs, tmem_cols;
  int a_col0, a_slots;  // fused kernel: tensor-memory ring that holds the scaled x tiles
  int a_stages, groups; // fused kernel: shared-memory ring of x tiles; transform warp groups
  long gamma_bytes;     // fused kernel: shared memory reserved for gamma
  int skinny;           // fused kernel, M <= 16: the weight-streaming kernel
  int prologue;         // fused kernel, M > 16: prologue variant of the plain GEMM (needs scratch)
  int a_kmajor;         // matmul_lhs_rhs: A is [M,K] with K contiguous
  int split_k;          // plain GEMM: parts of the K range (1 = none); parts > 1 need scratch
  int kb_per_part;
  long smem_bytes;
};

// Default candidate when the caller passes no b200_cfg.  For the plain GEMM main loop the choice
// is the candidate with the smallest estimated time: rounds of the persistent schedule (tiles over
// the CTA groups of a 148-SM part) x tile area per SM / relative throughput of that tile shape
// as measured at 4096^3.  Large problems get the 512x256 pair tile; short ones a smaller tile that
// fills the machine.
static b200_cfg default_cfg(Family fam, long M, long N) {
  b200_cfg c;
  memset(&c, 0, sizeof(c));
  c.cluster_n = 1;
  if (fam == FAM_RMSNORM && M > 0 && M <= 16) {  // weight-streaming kernel
    c.tile_m = 16; c.tile_n = 256; c.tile_k = 128; c.stages = 3; c.cluster_m = 1;
    return c;
  }
  if (fam == FAM_RMSNORM) {  // inline norm
    c.tile_m = 128; c.tile_n = 256; c.tile_k = 128; c.stages = 2; c.cluster_m = 1;
    return c;
  }
  struct Option { int tile_m, tile_n, tile_k, stages, cluster_m; double rate; };
  static const Option kOptions[] = {
      {512, 256, 64, 4, 2, 1.00},
      {256, 256, 128, 3, 2, 0.99},
      {256, 128, 128, 3, 2, 0.76},
      {128, 256, 128, 2, 1, 0.74},
      {128, 128, 128, 3, 1, 0.80},
      {128, 64, 128, 4, 1, 0.51},
  };
  const Option* best = &kOptions[1];
  if (M > 0 && N > 0) {
    double best_cost = 0.0;
    for (const Option& o : kOptions) {
      const long tiles = ((M + o.tile_m - 1) / o.tile_m) * ((N + o.tile_n - 1) / o.tile_n);
      const long groups = 148 / o.cluster_m;
      const long rounds = (tiles + groups - 1) / groups;
      const double cost = static_cast<double>(rounds) * o.tile_m * o.tile_n / o.cluster_m / o.rate;  // per-SM work
      if (best_cost == 0.0 || cost < best_cost) { best_cost = cost; best = &o; }
    }
  }
  c.tile_m = best->tile_m; c.tile_n = best->tile_n; c.tile_k = best->tile_k; c.stages = best->stages;
  c.cluster_m = best->cluster_m;
  return c;
}

static int next_pow2_cols(int cols) {
  int v = 32;
  while (v < cols) v <<= 1;
  return v;
}

// Validates a candidate and derives the launch plan.  Shape checks are skipped when M == 0.
static int make_plan(Family fam, const b200_cfg* cfg_in, long M, long N, long K, Plan* plan) {
  if (fam == FAM_UNKNOWN)
    return set_error(B200_ERR_BAD_ARG, "unknown kernel family (expected matmul_lhsT_rhs, matmul_lhs_rhs or rmsnorm_matmul)");
  b200_cfg cfg = cfg_in ? *cfg_in : default_cfg(fam, M, N);
  if (fam == FAM_RMSNORM && M > 0 && M <= SKINNY_ROWS) {
    // skinny activations: the weight-streaming kernel; only tile_k and stages apply
    Plan sp;
    memset(&sp, 0, sizeof(sp));
    sp.skinny = 1;
    sp.cta_group = 1; sp.m_sub = 1; sp.cluster = 1;
    sp.tile_m = SKINNY_ROWS; sp.tile_n = SKINNY_TILE_N;
    sp.tile_k = cfg.tile_k; sp.stages = cfg.stages;
    sp.tmem_cols = SKINNY_TMEM_COLS;
    if (cfg.tile_k != 64 && cfg.tile_k != 128)
      return set_error(B200_ERR_UNSUPPORTED, "tile_k=%d: only 64 and 128 are implemented", cfg.tile_k);
    if (cfg.stages < 1 || cfg.stages > MAX_STAGES)
      return set_error(B200_ERR_UNSUPPORTED, "stages=%d: need 1..%d", cfg.stages, MAX_STAGES);
    const long stage = (SKINNY_TILE_N + SKINNY_ROWS) * cfg.tile_k * 2L;
    sp.smem_bytes = 1024 + cfg.stages * stage + static_cast<long>(sizeof(SkinnyCtrl));
    *plan = sp;
    if (sp.smem_bytes > SMEM_BUDGET)
      return set_error(B200_ERR_SMEM_OOM, "Out of memory in smem: %d stages x %ld B = %ld B > %ld B per CTA",
                       cfg.stages, stage, sp.smem_bytes, SMEM_BUDGET);
    if (N <= 0 || K <= 0 || N % 8 != 0 || K % 64 != 0)
      return set_error(B200_ERR_BAD_SHAPE, "rmsnorm_matmul (skinny): need N %% 8 == 0 and K %% 64 == 0, got N=%ld K=%ld", N, K);
    return B200_OK;
  }
  const bool prologue = (fam == FAM_RMSNORM && cfg.norm_mode == 2);
  const bool lhs_kmajor = (fam == FAM_LHS);
  if (prologue || lhs_kmajor) fam = FAM_LHST;  // same pipeline budgets as the plain GEMM
  const int cluster_m = cfg.cluster_m == 0 ? 1 : cfg.cluster_m;
  const int cluster_n = cfg.cluster_n == 0 ? 1 : cfg.cluster_n;
  if (cfg.tile_m != 128 && cfg.tile_m != 256 && !(cfg.tile_m == 512 && cluster_m == 2 && fam == FAM_LHST))
    return set_error(B200_ERR_UNSUPPORTED,
                     "tile_m=%d: only 128, 256 and (plain GEMM, CTA pair) 512 are implemented", cfg.tile_m);
  if (cluster_m != 1 && cluster_m != 2)
    return set_error(B200_ERR_UNSUPPORTED, "cluster_m=%d: only 1 and 2 are implemented", cluster_m);
  if (cluster_n != 1)
    return set_error(B200_ERR_UNSUPPORTED, "cluster_n=%d: only 1 is implemented", cluster_n);
  Plan p;
  memset(&p, 0, sizeof(p));
  p.prologue = prologue ? 1 : 0;
  p.a_kmajor = lhs_kmajor ? 1 : 0;
  p.cluster = cluster_m;
  p.tile_m = cfg.tile_m;
  if (cluster_m == 2 && cfg.tile_m == 512) { p.cta_group = 2; p.m_sub = 2; }  // two pair-UMMAs per k-step
  else if (cluster_m == 2 && cfg.tile_m == 256) { p.cta_group = 2; p.m_sub = 1; }
  else if (cfg.tile_m == 256) { p.cta_group = 1; p.m_sub = 2; }
  else { p.cta_group = 1; p.m_sub = 1; }
  p.tile_n = cfg.tile_n;
  p.tile_k = cfg.tile_k;
  p.stages = cfg.stages;
  const int nc = cfg.tile_n / p.cta_group;
  const bool wide = (cfg.tile_n == 512 && fam == FAM_LHST);  // two 256-column UMMAs side by side
  if (!wide && (cfg.tile_n < 64 || cfg.tile_n > 256 || cfg.tile_n % 32 != 0 || nc % 64 != 0))
    return set_error(B200_ERR_UNSUPPORTED,
                     "tile_n=%d: need a multiple of %d in [64,256] (64-column operand chunks per CTA), or 512",
                     cfg.tile_n, 64 * p.cta_group);
  if ((fam == FAM_RMSNORM || prologue || lhs_kmajor) ? (cfg.tile_k != 64 && cfg.tile_k != 128)
                         : (cfg.tile_k != 32 && cfg.tile_k != 64 && cfg.tile_k != 96 && cfg.tile_k != 128))
    return set_error(B200_ERR_UNSUPPORTED, "tile_k=%d: only 64 and 128 (plain GEMM also 32 and 96) are implemented", cfg.tile_k);
  if (cfg.stages < 1 || cfg.stages > MAX_STAGES)
    return set_error(B200_ERR_UNSUPPORTED, "stages=%d: need 1..%d", cfg.stages, MAX_STAGES);
  if (cfg.swizzle < 0 || cfg.swizzle > 64)
    return set_error(B200_ERR_UNSUPPORTED, "swizzle=%d: need 0..64", cfg.swizzle);
  // split-K (plain GEMM families): every tile's k-blocks are dealt to split_k work units whose
  // fp32 partial tiles a second kernel sums; parts are sized so that none is empty
  p.split_k = 1;
  p.kb_per_part = 0;
  if (cfg.split_k < 0 || cfg.split_k > 16)
    return set_error(B200_ERR_UNSUPPORTED, "split_k=%d: need 0..16", cfg.split_k);
  if (cfg.split_k > 1) {
    if (fam != FAM_LHST || prologue)
      return set_error(B200_ERR_UNSUPPORTED, "split_k=%d: only the plain GEMM families can split K", cfg.split_k);
    if (K > 0) {
      const int nkb = static_cast<int>((K + cfg.tile_k - 1) / cfg.tile_k);
      p.kb_per_part = (nkb + cfg.split_k - 1) / cfg.split_k;
      p.split_k = (nkb + p.kb_per_part - 1) / p.kb_per_part;
    } else {
      p.split_k = cfg.split_k;
    }
  }
  p.group_m = cfg.swizzle > 0 ? cfg.swizzle : (cfg.tile_m == 512 ? 4 : (p.cta_group == 2 || p.m_sub == 2 ? 8 : 16));
  // prologue variant: narrow groups, so that the first wave of tiles reads few rows of x (about 1024)
  // and can start as soon as the norm pass has covered those
  if (prologue && cfg.swizzle == 0) p.group_m = cfg.tile_m >= 1024 ? 1 : 1024 / cfg.tile_m;

  const int acc_cols = p.m_sub * p.tile_n;
  const long mc = 128L * p.m_sub;
  const long stage_bytes = (mc + nc) * p.tile_k * 2L;
  long ctrl_bytes = static_cast<long>(sizeof(Ctrl));
  int tmem_need = acc_cols;
  if (fam == FAM_RMSNORM) {
    // accumulators first, then as many x-tile slots as fit (at least 2); prefer two accumulator
    // buffers when that still leaves 2 slots
    const int slot_cols = p.m_sub * (p.tile_k / 2);
    p.acc_bufs = (2 * acc_cols + 2 * slot_cols <= 512) ? 2 : 1;
    p.a_col0 = acc_cols * p.acc_bufs;
    int slots = (512 - p.a_col0) / slot_cols;
    if (slots > MAX_A_SLOTS) slots = MAX_A_SLOTS;
    tmem_need = p.a_col0 + 2 * slot_cols;
    p.gamma_bytes = ((K > 0 ? K : 0) + 127) / 128 * 128 * 2L;  // whole k-blocks of either size
    ctrl_bytes = static_cast<long>(sizeof(RmsCtrl)) + p.gamma_bytes;
    // x ring: as deep as fits beside the w ring (8, 6, 4, 3, 2 or 1 stages).  The transform warp
    // groups take k-blocks round-robin, and both the x ring and the slot ring must be multiples
    // of the group count (a stage/slot is then always served by one group, in order).
    const long a_stage_bytes = mc * p.tile_k * 2L;
    const long b_stage_bytes = static_cast<long>(nc) * p.tile_k * 2L;
    static const int kDepths[6] = {8, 6, 4, 3, 2, 1};
    p.a_stages = 1;
    for (int d : kDepths)
      if (1024 + p.stages * b_stage_bytes + d * a_stage_bytes + ctrl_bytes <= SMEM_BUDGET) { p.a_stages = d; break; }
    p.groups = 1;
    for (int g = 4; g >= 1; --g)
      if (p.a_stages % g == 0 && slots >= g) { p.groups = g; break; }
    slots -= slots % p.groups;
    p.a_slots = slots;
    p.tmem_cols = next_pow2_cols(p.a_col0 + (slots > 0 ? slots : 2) * slot_cols);
    p.smem_bytes = 1024 + p.stages * b_stage_bytes + p.a_stages * a_stage_bytes + ctrl_bytes;
  } else {
    p.acc_bufs = (2 * acc_cols <= 512) ? 2 : 1;
    p.tmem_cols = next_pow2_cols(acc_cols * p.acc_bufs);
  }
  if (fam != FAM_RMSNORM) {
    ctrl_bytes += EPI_STAGE_BYTES;  // output staging of the TMA-store epilogue
    p.smem_bytes = 1024 + p.stages * stage_bytes + ctrl_bytes;
  }
  *plan = p;
  if (tmem_need > 512)
    return set_error(B200_ERR_TMEM_OOM, "Out of memory in tmem: accumulator%s need %d of 512 columns",
                     fam == FAM_RMSNORM ? " and two x-tile slots" : "", tmem_need);
  if (p.smem_bytes > SMEM_BUDGET)
    return set_error(B200_ERR_SMEM_OOM,
                     "Out of memory in smem: %d stages x %ld B + %ld B control = %ld B > %ld B per CTA",
                     p.stages, stage_bytes, 1024 + ctrl_bytes, p.smem_bytes, SMEM_BUDGET);
  if (M != 0 || N != 0 || K != 0) {
    if (M <= 0 || N <= 0 || K <= 0) return set_error(B200_ERR_BAD_SHAPE, "empty shape M=%ld N=%ld K=%ld", M, N, K);
    if (M % 8 != 0 || N % 8 != 0)
      return set_error(B200_ERR_BAD_SHAPE, "M=%ld and N=%ld must be multiples of 8 (16-byte rows)", M, N);
    if ((fam == FAM_RMSNORM || prologue) && K % 64 != 0)
      return set_error(B200_ERR_BAD_SHAPE, "rmsnorm_matmul: K=%ld must be a multiple of 64", K);
    if (lhs_kmajor && K % 8 != 0)
      return set_error(B200_ERR_BAD_SHAPE, "matmul_lhs_rhs: K=%ld must be a multiple of 8 (16-byte rows of lhs)", K);
    if (M > (1L << 30) || N > (1L << 30) || K > (1L << 30))
      return set_error(B200_ERR_BAD_SHAPE, "dimension beyond 2^30");
  }
  return B200_OK;
}

// ---------------------------------------------------------------------------- tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D bf16 tensor [rows, cols] with `cols` contiguous and a row pitch of ld elements; the box
// is box_cols x box_rows with the 128-byte swizzle (box_cols * 2 must be 128).
static int make_tmap_bf16(CUtensorMap* tm, const void* base, long rows, long cols, long ld, int box_cols,
                          int box_rows, const char* what) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return set_error(B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return set_error(B200_ERR_BAD_ARG, "%s: base pointer must be 16-byte aligned", what);
  if (ld % 8 != 0 || ld < cols)
    return set_error(B200_ERR_BAD_SHAPE, "%s: leading dimension %ld must be a multiple of 8 and >= %ld", what, ld, cols);
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2u};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(B200_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed with CUresult %d", what, (int)r);
  return B200_OK;
}

// 2-D fp32 tensor [rows, cols] (row pitch ld floats), boxes of 32 columns x box_rows rows with the
// 128-byte swizzle: the split-K partial arrays the epilogue stores into.
static int make_tmap_f32(CUtensorMap* tm, const void* base, long rows, long cols, long ld, int box_rows,
                         const char* what) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return set_error(B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || ld % 4 != 0 || ld < cols)
    return set_error(B200_ERR_BAD_ARG, "%s: base must be 16-byte aligned and the row pitch a multiple of 4 floats", what);
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 4u};
  cuuint32_t box[2] = {32u, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(B200_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed with CUresult %d", what, (int)r);
  return B200_OK;
}

// split-K: out[m, n] = bf16(sum over parts of partial[part][m][n]), parts added in order
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ partial, int parts, size_t part_stride, __nv_bfloat16* __restrict__ out,
                     long ld_out, int M, int N) {
  const long groups_per_row = N / 8;  // N is a multiple of 8
  const long total = static_cast<long>(M) * groups_per_row;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long m = i / groups_per_row;
    const long n = (i - m * groups_per_row) * 8;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
    for (int p = 0; p < parts; ++p) {
      const float4* src = reinterpret_cast<const float4*>(partial + p * part_stride + m * N + n);
      const float4 x = __ldcg(src), y = __ldcg(src + 1);
      a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
      b.x += y.x; b.y += y.y; b.z += y.z; b.w += y.w;
    }
    uint4 o;
    o.x = pack_bf16x2(a.x, a.y); o.y = pack_bf16x2(a.z, a.w);
    o.z = pack_bf16x2(b.x, b.y); o.w = pack_bf16x2(b.z, b.w);
    *reinterpret_cast<uint4*>(out + m * ld_out + n) = o;
  }
}

static size_t splitk_workspace_bytes(const Plan& plan, long M, long N) {
  if (plan.split_k <= 1) return 0;
  const long m_pad = (M + plan.tile_m - 1) / plan.tile_m * plan.tile_m;
  return static_cast<size_t>(plan.split_k) * m_pad * N * sizeof(float);
}

// ---------------------------------------------------------------------------- launch
typedef void (*GemmKernelFn)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const GemmParams);
typedef void (*RmsKernelFn)(const CUtensorMap, const CUtensorMap, const RmsParams);

static GemmKernelFn pick_gemm_kernel(const Plan& p) {
  if (p.prologue) {
    if (p.cta_group == 2 && p.m_sub == 2) return gemm_tcgen05_kernel<2, 2, A_NORM>;
    if (p.cta_group == 2) return gemm_tcgen05_kernel<2, 1, A_NORM>;
    if (p.m_sub == 2) return gemm_tcgen05_kernel<1, 2, A_NORM>;
    return gemm_tcgen05_kernel<1, 1, A_NORM>;
  }
  if (p.a_kmajor) {
    if (p.cta_group == 2 && p.m_sub == 2) return gemm_tcgen05_kernel<2, 2, A_KMAJOR_PLAIN>;
    if (p.cta_group == 2) return gemm_tcgen05_kernel<2, 1, A_KMAJOR_PLAIN>;
    if (p.m_sub == 2) return gemm_tcgen05_kernel<1, 2, A_KMAJOR_PLAIN>;
    return gemm_tcgen05_kernel<1, 1, A_KMAJOR_PLAIN>;
  }
  if (p.cta_group == 2 && p.m_sub == 2) return gemm_tcgen05_kernel<2, 2>;
  if (p.cta_group == 2) return gemm_tcgen05_kernel<2, 1>;
  if (p.m_sub == 2) return gemm_tcgen05_kernel<1, 2>;
  return gemm_tcgen05_kernel<1, 1>;
}

static RmsKernelFn pick_rms_kernel(const Plan& p) {
  if (p.cta_group == 2) return rmsnorm_tcgen05_kernel<2, 1>;
  if (p.m_sub == 2) return rmsnorm_tcgen05_kernel<1, 2>;
  return rmsnorm_tcgen05_kernel<1, 1>;
}

struct DeviceInfo {
  int sm_count = 0;
  int clock_khz = 0;
};

static int device_info(DeviceInfo* out) {
  static DeviceInfo cache[64];
  int dev = 0;
  int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
  if (rc) return rc;
  if (dev < 0 || dev >= 64) return set_error(B200_ERR_CUDA, "device ordinal %d out of range", dev);
  if (cache[dev].sm_count == 0) {
    int major = 0;
    rc = check_cuda(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev), "device attribute");
    if (rc) return rc;
    if (major != 10)
      return set_error(B200_ERR_CUDA, "device %d has compute capability %d.x; these kernels are sm_100a only", dev, major);
    rc = check_cuda(cudaDeviceGetAttribute(&cache[dev].clock_khz, cudaDevAttrClockRate, dev), "device attribute");
    if (rc) return rc;
    rc = check_cuda(cudaDeviceGetAttribute(&cache[dev].sm_count, cudaDevAttrMultiProcessorCount, dev), "device attribute");
    if (rc) return rc;
  }
  *out = cache[dev];
  return B200_OK;
}

struct LaunchArgs {
  Family fam;
  const void* a;
  const void* b;
  const void* gamma;
  void* out;
  long M, N, K, ld_a, ld_b, ld_out;
  float eps;
  void* workspace;
  size_t workspace_bytes;
};

static size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

// prologue variant: [xg: M*K bf16][rinv: M fp32][counters: next row, departed CTAs, one per 128 rows]
static size_t prologue_workspace_bytes(long M, long K) {
  return align256(static_cast<size_t>(M) * K * 2) + align256(static_cast<size_t>(M) * sizeof(float)) +
         align256((2 + static_cast<size_t>((M + 127) / 128)) * sizeof(unsigned int))
#ifdef B200_MEASURE_HOOKS
         + 160 * 8 * sizeof(unsigned long long)  // measurement build: per-CTA stamps behind the counters
#endif
      ;
}

// skinny kernel: [tile counters: one int per 256-column tile, zero between launches]
//                [partial-tile slots: (tiles + SKINNY_MAX_CTAS) x [16][256] fp32, written before read;
//                 slot index = donor CTA + left-over tile, both below those bounds]
static size_t skinny_counter_bytes(long N) {
  const size_t tiles = static_cast<size_t>((N + SKINNY_TILE_N - 1) / SKINNY_TILE_N);
  return align256(tiles * sizeof(int));
}
static size_t skinny_workspace_bytes(long N) {
  const size_t tiles = static_cast<size_t>((N + SKINNY_TILE_N - 1) / SKINNY_TILE_N);
  return skinny_counter_bytes(N) + (tiles + SKINNY_MAX_CTAS) * SKINNY_SLOT_FLOATS * sizeof(float);
}

// A prepared launch: tensor maps and parameters are built once and can be replayed.
struct Prepared {
  GemmKernelFn fn;      // plain GEMM (fam == FAM_LHST)
  RmsKernelFn rms_fn;   // fused kernel (fam == FAM_RMSNORM)
  CUtensorMap tm_a, tm_b, tm_out;
  GemmParams gp;
  const float* sk_partial;   // split-K: partial arrays in the scratch, one per part
  size_t sk_part_stride;     // floats between parts
  RmsParams rp;
  SkinnyParams sp;
  bool fused;
  bool skinny;
  bool skinny_serial;        // skinny kernel launched without the programmatic-dependent-launch attribute
  Plan plan;
  dim3 grid, block;
  size_t smem;
};

static int prepare_skinny(const LaunchArgs& la, const b200_cfg* cfg, const Plan& plan, const DeviceInfo& di,
                          int* dev_status, Prepared* pr) {
  const size_t need = skinny_workspace_bytes(la.N);
  if (la.workspace == nullptr || la.workspace_bytes < need)
    return set_error(B200_ERR_WORKSPACE,
                     "rmsnorm_matmul with M <= 16 needs %zu bytes of zero-initialised device workspace (got %zu)",
                     need, la.workspace ? la.workspace_bytes : static_cast<size_t>(0));
  if ((reinterpret_cast<uintptr_t>(la.workspace) & 15u) != 0 || (reinterpret_cast<uintptr_t>(la.a) & 15u) != 0 ||
      (la.gamma && (reinterpret_cast<uintptr_t>(la.gamma) & 15u) != 0))
    return set_error(B200_ERR_BAD_ARG, "x, gamma and workspace must be 16-byte aligned");
  if (la.ld_a != la.K || la.ld_out != la.N)
    return set_error(B200_ERR_BAD_SHAPE, "rmsnorm_matmul (skinny): x and out must be dense");
  int rc = make_tmap_bf16(&pr->tm_b, la.b, la.K, la.N, la.ld_b, 64, plan.tile_k, "w");
  if (rc) return rc;
  SkinnyParams& sp = pr->sp;
  memset(&sp, 0, sizeof(sp));
  sp.M = static_cast<int>(la.M);
  sp.N = static_cast<int>(la.N);
  sp.K = static_cast<int>(la.K);
  sp.tile_k = plan.tile_k;
  sp.num_k_blocks = static_cast<int>((la.K + plan.tile_k - 1) / plan.tile_k);
  // Work split (see rmsnorm_skinny.cuh): T tiles of 256 columns over G CTAs; floor(T / G) whole tiles
  // each, the R = T mod G left-over tiles get one owner each and the other G - R CTAs donate the
  // first `don` k-blocks of every left-over tile.
  const long T = (la.N + SKINNY_TILE_N - 1) / SKINNY_TILE_N;
  const long nkb = sp.num_k_blocks;
  long grid = di.sm_count;
  if (grid > SKINNY_MAX_CTAS) grid = SKINNY_MAX_CTAS;  // the scratch holds one slot per tile and per CTA
  if (T < grid && T * nkb < grid) grid = T * nkb;  // tiny problem: one k-block per CTA at most
  const long base = T / grid, R = T % grid, D = R > 0 ? grid - R : 0;
  long don = 0;
  if (R > 0 && D > 0) {
    // Owners stream `own` k-blocks of their tile and donors V / D: balanced when own = R nkb / G.
    // Without whole tiles after their range, donors get about 190 KB (4 us of streaming) less
    // than owners so that their partial tiles are published before the owners need them.
    long lead = base > 0 ? 0 : (192 * 1024) / (static_cast<long>(SKINNY_TILE_N) * plan.tile_k * 2);
    if (lead > R * nkb / grid / 8) lead = R * nkb / grid / 8;
    long own = (R * nkb + D * lead + grid - 1) / grid;
    if (own < 1) own = 1;
    if (own > nkb) own = nkb;
    don = nkb - own;
  }
  sp.base_tiles = static_cast<int>(base);
  sp.lo_tiles = static_cast<int>(R);
  sp.donors = static_cast<int>(D);  // CTAs 0..D-1 (with don == 0 they only have whole tiles, or nothing, to do)
  sp.don = static_cast<int>(don);
  sp.rot = 5;  // CTA b starts its whole-K loops 5 b k-blocks in: neighbours never walk the same k-rows together
  sp.stages = plan.stages;
  sp.x = static_cast<const __nv_bfloat16*>(la.a);
  sp.gamma = static_cast<const __nv_bfloat16*>(la.gamma);
  sp.out = static_cast<__nv_bfloat16*>(la.out);
  sp.tile_count = static_cast<int*>(la.workspace);
  sp.partial = reinterpret_cast<float*>(static_cast<uint8_t*>(la.workspace) + skinny_counter_bytes(la.N));
  sp.eps = la.eps;
  sp.inv_k = 1.0f / static_cast<float>(la.K);
  sp.status = dev_status;
  long long limit_us = 1000000;
  if (cfg && cfg->reserved[1] > 0) limit_us = cfg->reserved[1];
  sp.timeout_cycles = limit_us * (di.clock_khz > 0 ? di.clock_khz / 1000 : 1900);
  pr->skinny = true;
  pr->skinny_serial = cfg != nullptr && cfg->reserved[4] != 0;
  pr->fused = false;
  pr->plan = plan;
  pr->smem = static_cast<size_t>(plan.smem_bytes);
  pr->block = dim3(SKINNY_THREADS);
  rc = check_cuda(cudaFuncSetAttribute(reinterpret_cast<const void*>(rmsnorm_skinny_kernel),
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BUDGET)),
                  "cudaFuncSetAttribute(max dynamic shared memory)");
  if (rc) return rc;
  pr->grid = dim3(static_cast<unsigned>(grid));
  if (getenv("B200_AUTOTUNE_DEBUG") != nullptr)
    fprintf(stderr, "[b200] skinny: grid %ld, %ld tiles x %ld k-blocks: %ld whole tiles per CTA, %ld left-over tiles, "
            "%d donors x %ld of their k-blocks, %d stages\n", grid, T, nkb, base, R, sp.donors, don, sp.stages);
  return B200_OK;
}

static int prepare(const LaunchArgs& la, const b200_cfg* cfg, int* dev_status, Prepared* pr) {
  if (!la.a || !la.b || !la.out) return set_error(B200_ERR_BAD_ARG, "NULL operand pointer");
  // fused kernel, M > 16: choose where the norm is applied (b200_cfg.norm_mode)
  b200_cfg eff;
  if (la.fam == FAM_RMSNORM && la.M > SKINNY_ROWS) {
    const int mode = cfg ? cfg->norm_mode : 0;
    const bool have_ws = la.workspace != nullptr && la.workspace_bytes >= prologue_workspace_bytes(la.M, la.K);
    if (mode < 0 || mode > 2) return set_error(B200_ERR_UNSUPPORTED, "norm_mode=%d: need 0, 1 or 2", mode);
    if (mode == 2 && !have_ws)
      return set_error(B200_ERR_WORKSPACE, "rmsnorm_matmul with norm_mode 2 needs %zu bytes of device workspace (got %zu)",
                       prologue_workspace_bytes(la.M, la.K), la.workspace ? la.workspace_bytes : static_cast<size_t>(0));
    if (mode == 2 || (mode == 0 && have_ws)) {
      eff = cfg ? *cfg : default_cfg(FAM_LHST, la.M, la.N);
      eff.norm_mode = 2;
      cfg = &eff;
    } else if (cfg != nullptr) {
      eff = *cfg;
      eff.norm_mode = 1;
      cfg = &eff;
    }
  }
  Plan plan;
  int rc = make_plan(la.fam, cfg, la.M, la.N, la.K, &plan);
  if (rc) return rc;
  DeviceInfo di;
  rc = device_info(&di);
  if (rc) return rc;
  pr->skinny = false;
  if (plan.skinny) return prepare_skinny(la, cfg, plan, di, dev_status, pr);
  if ((reinterpret_cast<uintptr_t>(la.out) & 15u) != 0 || la.ld_out % 8 != 0 || la.ld_out < la.N)
    return set_error(B200_ERR_BAD_SHAPE, "out: pointer must be 16-byte aligned and ld_out a multiple of 8 >= N");
  if (la.gamma && (reinterpret_cast<uintptr_t>(la.gamma) & 15u) != 0)
    return set_error(B200_ERR_BAD_ARG, "gamma: pointer must be 16-byte aligned");

  const int mc = 128 * plan.m_sub;
  uint8_t* ws = static_cast<uint8_t*>(la.workspace);
  if (plan.prologue) {
    if ((reinterpret_cast<uintptr_t>(ws) & 255u) != 0 || (reinterpret_cast<uintptr_t>(la.a) & 15u) != 0)
      return set_error(B200_ERR_BAD_ARG, "workspace must be 256-byte aligned and x 16-byte aligned");
    if (la.gamma != nullptr) rc = make_tmap_bf16(&pr->tm_a, ws, la.M, la.K, la.K, 64, mc, "scaled x (workspace)");
    else rc = make_tmap_bf16(&pr->tm_a, la.a, la.M, la.K, la.K, 64, mc, "x");  // no gamma: x is the A operand as it is
  } else if (la.fam == FAM_LHS) {
    rc = make_tmap_bf16(&pr->tm_a, la.a, la.M, la.K, la.ld_a, 64, mc, "lhs");
  } else if (la.fam == FAM_LHST) {
    rc = make_tmap_bf16(&pr->tm_a, la.a, la.K, la.M, la.ld_a, 64, plan.tile_k, "lhsT");
  } else {
    rc = make_tmap_bf16(&pr->tm_a, la.a, la.M, la.K, la.ld_a, 64, mc, "x");
  }
  if (rc) return rc;
  rc = make_tmap_bf16(&pr->tm_b, la.b, la.K, la.N, la.ld_b, 64, plan.tile_k, la.fam == FAM_RMSNORM ? "w" : "rhs");
  if (rc) return rc;
  pr->sk_partial = nullptr;
  pr->sk_part_stride = 0;
  if (plan.split_k > 1) {
    // the epilogue stores fp32 boxes into [part][padded rows][N] arrays in the scratch; ragged
    // tiles spill into a part's own padding rows and columns past N are clipped
    const size_t need = splitk_workspace_bytes(plan, la.M, la.N);
    if (la.workspace == nullptr || la.workspace_bytes < need)
      return set_error(B200_ERR_WORKSPACE, "split_k=%d needs %zu bytes of device workspace (got %zu)", plan.split_k,
                       need, la.workspace ? la.workspace_bytes : static_cast<size_t>(0));
    const long m_pad = (la.M + plan.tile_m - 1) / plan.tile_m * plan.tile_m;
    rc = make_tmap_f32(&pr->tm_out, la.workspace, static_cast<long>(plan.split_k) * m_pad, la.N, la.N, 32,
                       "split-K partials (workspace)");
    pr->sk_partial = static_cast<const float*>(la.workspace);
    pr->sk_part_stride = static_cast<size_t>(m_pad) * la.N;
  } else {
    // the epilogue stores 32-row x 64-column boxes; rows and columns past M and N are clipped
    rc = make_tmap_bf16(&pr->tm_out, la.out, la.M, la.N, la.ld_out, 64, 32, "out");
  }
  if (rc) return rc;

  GemmParams& gp = pr->gp;
  memset(&gp, 0, sizeof(gp));
  gp.M = static_cast<int>(la.M);
  gp.N = static_cast<int>(la.N);
  gp.K = static_cast<int>(la.K);
  gp.tile_n = plan.tile_n;
  gp.umma_n = plan.tile_n > 256 ? plan.tile_n / 2 : plan.tile_n;
  gp.tile_k = plan.tile_k;
  gp.stages = plan.stages;
  gp.num_m_tiles = static_cast<int>((la.M + plan.tile_m - 1) / plan.tile_m);
  gp.num_n_tiles = static_cast<int>((la.N + plan.tile_n - 1) / plan.tile_n);
  gp.num_k_blocks = static_cast<int>((la.K + plan.tile_k - 1) / plan.tile_k);
  gp.group_m = plan.group_m;
  gp.split_k = plan.split_k;
  gp.kb_per_part = plan.split_k > 1 ? plan.kb_per_part : gp.num_k_blocks;
  gp.part_rows = static_cast<int>((la.M + plan.tile_m - 1) / plan.tile_m * plan.tile_m);
  gp.acc_bufs = plan.acc_bufs;
  // a single-buffered accumulator of exactly two UMMA blocks is handed over in halves (not with
  // split-K, whose epilogue stores the whole fp32 tile)
  gp.acc_halves = (plan.acc_bufs == 1 && plan.split_k <= 1 &&
                   ((plan.m_sub == 2 && plan.tile_n <= 256) || (plan.m_sub == 1 && plan.tile_n == 512))) ? 1 : 0;
  gp.tmem_cols = plan.tmem_cols;
  gp.ld_out = la.ld_out;
  gp.out = static_cast<__nv_bfloat16*>(la.out);
  gp.status = dev_status;
  long long limit_us = 1000000;  // one second per wait
  if (cfg && cfg->reserved[1] > 0) limit_us = cfg->reserved[1];
  gp.timeout_cycles = limit_us * (di.clock_khz > 0 ? di.clock_khz / 1000 : 1900);
  gp.debug_mode = cfg ? cfg->reserved[0] : 0;
  gp.record_clocks = cfg ? cfg->reserved[2] : 0;
  if (plan.prologue) {
    gp.x = static_cast<const __nv_bfloat16*>(la.a);
    gp.gamma = static_cast<const __nv_bfloat16*>(la.gamma);
    gp.xg = la.gamma != nullptr ? reinterpret_cast<__nv_bfloat16*>(ws) : nullptr;  // no gamma: nothing to rewrite
    gp.rinv = reinterpret_cast<float*>(ws + align256(static_cast<size_t>(la.M) * la.K * 2));
    gp.norm_sync = reinterpret_cast<unsigned int*>(reinterpret_cast<uint8_t*>(gp.rinv) +
                                                   align256(static_cast<size_t>(la.M) * sizeof(float)));
    gp.eps = la.eps;
    gp.inv_k = 1.0f / static_cast<float>(la.K);
#ifdef B200_MEASURE_HOOKS
    gp.trace = reinterpret_cast<unsigned long long*>(
        ws + prologue_workspace_bytes(la.M, la.K) - 160 * 8 * sizeof(unsigned long long));
#endif
  }

  const bool fused = (la.fam == FAM_RMSNORM) && !plan.prologue;
  RmsParams& rp = pr->rp;
  memset(&rp, 0, sizeof(rp));
  if (fused) {
    if (plan.a_slots < 2)
      return set_error(B200_ERR_TMEM_OOM, "Out of memory in tmem: fewer than two x-tile slots fit beside the accumulators");
    rp.M = gp.M; rp.N = gp.N; rp.K = gp.K;
    rp.tile_n = gp.tile_n; rp.tile_k = gp.tile_k; rp.stages = gp.stages;
    rp.num_m_tiles = gp.num_m_tiles; rp.num_n_tiles = gp.num_n_tiles; rp.num_k_blocks = gp.num_k_blocks;
    rp.group_m = gp.group_m;
    rp.acc_bufs = plan.acc_bufs;
    rp.tmem_cols = plan.tmem_cols;
    rp.a_col0 = plan.a_col0;
    rp.a_slots = plan.a_slots;
    rp.a_stages = plan.a_stages;
    rp.groups = plan.groups;
    rp.gamma_bytes = la.gamma ? static_cast<int>(plan.gamma_bytes) : 0;
    rp.ld_out = gp.ld_out;
    rp.eps = la.eps;
    rp.inv_k = 1.0f / static_cast<float>(la.K);
    rp.out = gp.out;
    rp.gamma = static_cast<const __nv_bfloat16*>(la.gamma);
    rp.status = gp.status;
    rp.timeout_cycles = gp.timeout_cycles;
    rp.debug_mode = gp.debug_mode;
  }
  pr->fn = pick_gemm_kernel(plan);
  pr->rms_fn = pick_rms_kernel(plan);
  pr->fused = fused;
  pr->plan = plan;
  pr->smem = static_cast<size_t>(plan.smem_bytes);
  pr->block = dim3(static_cast<unsigned>(fused ? RMS_THREADS : GEMM_THREADS));
  const void* kernel_ptr = fused ? reinterpret_cast<const void*>(pr->rms_fn) : reinterpret_cast<const void*>(pr->fn);
  // always the whole budget: the attribute is sticky per function, and a replayed (cached) launch
  // of a larger configuration must not find it lowered by a smaller one prepared in between
  rc = check_cuda(cudaFuncSetAttribute(kernel_ptr, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(SMEM_BUDGET)),
                  "cudaFuncSetAttribute(max dynamic shared memory)");
  if (rc) return rc;

  const long total_tiles = static_cast<long>(gp.num_m_tiles) * gp.num_n_tiles * plan.split_k;  // work units
  long groups = di.sm_count / plan.cluster;  // CTA groups (clusters) that fit the machine
  if (plan.cluster > 1) {
    cudaLaunchConfig_t qc;
    memset(&qc, 0, sizeof(qc));
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = static_cast<unsigned>(plan.cluster);
    qa[0].val.clusterDim.y = 1;
    qa[0].val.clusterDim.z = 1;
    qc.gridDim = dim3(static_cast<unsigned>(groups * plan.cluster));
    qc.blockDim = pr->block;
    qc.dynamicSmemBytes = pr->smem;
    qc.attrs = qa;
    qc.numAttrs = 1;
    int max_clusters = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&max_clusters, kernel_ptr, &qc);
    if (e == cudaSuccess && max_clusters > 0 && max_clusters < groups) groups = max_clusters;
    (void)cudaGetLastError();
  }
  // work units per CTA group: a CTA pair shares one tile, co-scheduled single CTAs take one each
  const long units = (plan.cta_group == 2) ? total_tiles : (total_tiles + plan.cluster - 1) / plan.cluster;
  if (groups > units) groups = units;
  // caller's cap on the grid (b200_cfg.reserved[3], in CTAs): leaves SMs free for kernels that must
  // run beside this one, such as a collective on another stream
  if (cfg && cfg->reserved[3] > 0 && groups > cfg->reserved[3] / plan.cluster) groups = cfg->reserved[3] / plan.cluster;
  if (groups < 1) groups = 1;
  pr->grid = dim3(static_cast<unsigned>(groups * plan.cluster));
  if (getenv("B200_AUTOTUNE_DEBUG") != nullptr)
    fprintf(stderr, "[b200] %d SMs, cluster %d, CTA groups %ld (work units %ld), grid %u, block %u, smem %zu\n",
            di.sm_count, plan.cluster, groups, units, pr->grid.x, pr->block.x, pr->smem);
  return B200_OK;
}

// Replay cache: the entry points are called once per step with the same buffers, shapes and
// candidate, so the last few prepared launches are kept per host thread (tensor-map encoding,
// the occupancy query and the attribute call cost far more host time than the launch itself).
struct PrepKey {
  LaunchArgs la;
  b200_cfg cfg;
  int has_cfg;
  int device;
  int* dev_status;
};

static int prepare_cached(const LaunchArgs& la, const b200_cfg* cfg, int* dev_status, Prepared* pr) {
  constexpr int SLOTS = 8;
  struct Slot { bool used; PrepKey key; Prepared pr; };
  static thread_local Slot slots[SLOTS];
  static thread_local int next_slot = 0;
  PrepKey key;
  memset(&key, 0, sizeof(key));  // padding bytes too: keys are compared with memcmp
  key.la.fam = la.fam; key.la.a = la.a; key.la.b = la.b; key.la.gamma = la.gamma; key.la.out = la.out;
  key.la.M = la.M; key.la.N = la.N; key.la.K = la.K;
  key.la.ld_a = la.ld_a; key.la.ld_b = la.ld_b; key.la.ld_out = la.ld_out;
  key.la.eps = la.eps; key.la.workspace = la.workspace; key.la.workspace_bytes = la.workspace_bytes;
  if (cfg) { memcpy(&key.cfg, cfg, sizeof(b200_cfg)); key.has_cfg = 1; }
  key.dev_status = dev_status;
  if (cudaGetDevice(&key.device) != cudaSuccess) { (void)cudaGetLastError(); key.device = -1; }
  for (int i = 0; i < SLOTS; ++i)
    if (slots[i].used && memcmp(&slots[i].key, &key, sizeof(key)) == 0) {
      *pr = slots[i].pr;
      return B200_OK;
    }
  int rc = prepare(la, cfg, dev_status, pr);
  if (rc) return rc;
  Slot& s = slots[next_slot];
  next_slot = (next_slot + 1) % SLOTS;
  s.used = true;
  s.key = key;
  s.pr = *pr;
  return B200_OK;
}

static int launch(const Prepared& pr, cudaStream_t stream) {
  cudaLaunchConfig_t lc;
  memset(&lc, 0, sizeof(lc));
  lc.gridDim = pr.grid;
  lc.blockDim = pr.block;
  lc.dynamicSmemBytes = pr.smem;
  lc.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(pr.plan.cluster);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  if (pr.skinny) {
    // programmatic dependent launch (see rmsnorm_skinny.cuh): the kernel waits by itself for the
    // kernel before it wherever it depends on it, and streams its weights meanwhile
    cudaLaunchAttribute sk_attr[2];
    sk_attr[0] = attr[0];
    sk_attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    sk_attr[1].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = sk_attr;
    lc.numAttrs = pr.skinny_serial ? 1 : 2;
    return check_cuda(cudaLaunchKernelEx(&lc, rmsnorm_skinny_kernel, pr.tm_b, pr.sp), "skinny RMSNorm GEMM launch");
  }
  if (pr.fused)
    return check_cuda(cudaLaunchKernelEx(&lc, pr.rms_fn, pr.tm_a, pr.tm_b, pr.rp), "fused RMSNorm GEMM launch");
  int rc = check_cuda(cudaLaunchKernelEx(&lc, pr.fn, pr.tm_a, pr.tm_b, pr.tm_out, pr.gp), "tcgen05 GEMM launch");
  if (rc || pr.plan.split_k <= 1) return rc;
  const long groups = static_cast<long>(pr.gp.M) * (pr.gp.N / 8);
  const unsigned blocks = static_cast<unsigned>(groups / 256 + 1 < 148L * 8 ? groups / 256 + 1 : 148L * 8);
  splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(pr.sk_partial, pr.plan.split_k, pr.sk_part_stride, pr.gp.out,
                                                   pr.gp.ld_out, pr.gp.M, pr.gp.N);
  return check_cuda(cudaGetLastError(), "split-K reduction launch");
}

}  // namespace b200

using namespace b200;

// =============================================================================== C ABI
extern "C" const char* b200_last_error(void) { return g_last_error; }
extern "C" int b200_abi_version(void) { return B200_ABI_VERSION; }

extern "C" int b200_device_count(int* count) {
  if (!count) return set_error(B200_ERR_BAD_ARG, "device_count: NULL pointer");
  *count = 0;
  cudaError_t e = cudaGetDeviceCount(count);
  if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) {
    (void)cudaGetLastError();
    *count = 0;
    return B200_OK;
  }
  return check_cuda(e, "cudaGetDeviceCount");
}

extern "C" int b200_cfg_check(const char* family, const b200_cfg* cfg, long M, long N, long K, long* smem_bytes,
                              int* tmem_cols) {
  Plan plan;
  memset(&plan, 0, sizeof(plan));
  int rc = make_plan(parse_family(family), cfg, M, N, K, &plan);
  if (smem_bytes) *smem_bytes = plan.smem_bytes;
  if (tmem_cols) *tmem_cols = plan.tmem_cols;
  return rc;
}

// What a launch of this candidate at this shape looks like, as one JSON object: which kernel, grid,
// cluster, threads, shared and tensor memory, tiles / CTA groups / waves of the persistent schedule,
// the UMMA-issue-bound SM cycles of the busiest CTA group, and the compiled kernel's registers and
// local memory.  No launch is made; without a usable device the device-derived fields are null.
extern "C" int b200_describe_launch(const char* family, const b200_cfg* cfg_in, long M, long N, long K, char* out,
                                    size_t out_bytes) {
  if (!out || out_bytes == 0) return set_error(B200_ERR_BAD_ARG, "describe_launch: no output buffer");
  Family fam = parse_family(family);
  b200_cfg eff;
  const b200_cfg* cfg = cfg_in;
  if (fam == FAM_RMSNORM && M > SKINNY_ROWS && (!cfg || cfg->norm_mode != 1)) {
    // what runs when scratch is supplied: the prologue variant of the plain GEMM
    eff = cfg ? *cfg : default_cfg(FAM_LHST, M, N);
    eff.norm_mode = 2;
    cfg = &eff;
  }
  Plan plan;
  memset(&plan, 0, sizeof(plan));
  int rc = make_plan(fam, cfg, M, N, K, &plan);
  if (rc) return rc;
  DeviceInfo di;
  const bool have_dev = device_info(&di) == B200_OK;
  const long sms = have_dev ? di.sm_count : 148;
  const void* kptr = nullptr;
  const char* kname = "";
  int threads = GEMM_THREADS;
  if (plan.skinny) { kptr = reinterpret_cast<const void*>(rmsnorm_skinny_kernel); kname = "rmsnorm_skinny_kernel"; threads = SKINNY_THREADS; }
  else if (fam == FAM_RMSNORM && !plan.prologue) { kptr = reinterpret_cast<const void*>(pick_rms_kernel(plan)); kname = "rmsnorm_tcgen05_kernel"; threads = RMS_THREADS; }
  else { kptr = reinterpret_cast<const void*>(pick_gemm_kernel(plan)); kname = "gemm_tcgen05_kernel"; }
  int regs = -1, local_bytes = -1;
  if (have_dev) {
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, kptr) == cudaSuccess) { regs = fa.numRegs; local_bytes = static_cast<int>(fa.localSizeBytes); }
    else (void)cudaGetLastError();
  }
  char regs_txt[32] = "null", local_txt[32] = "null";
  if (regs >= 0) { snprintf(regs_txt, sizeof(regs_txt), "%d", regs); snprintf(local_txt, sizeof(local_txt), "%d", local_bytes); }
  int n = 0;
  if (plan.skinny) {
    const long T = (N + SKINNY_TILE_N - 1) / SKINNY_TILE_N, nkb = (K + plan.tile_k - 1) / plan.tile_k;
    long grid = sms > SKINNY_MAX_CTAS ? SKINNY_MAX_CTAS : sms;
    if (T < grid && T * nkb < grid) grid = T * nkb;
    n = snprintf(out, out_bytes,
                 "{\"kernel\": \"%s\", \"grid\": %ld, \"cluster\": 1, \"threads\": %d, \"smem_bytes\": %ld, \"tmem_cols\": %d, "
                 "\"stages\": %d, \"tile_k\": %d, \"tiles_256_columns\": %ld, \"k_blocks\": %ld, \"whole_tiles_per_cta\": %ld, "
                 "\"shared_tiles\": %ld, \"sm_count\": %ld, \"sm_count_from_device\": %s, \"registers\": %s, \"local_bytes\": %s}",
                 kname, grid, threads, plan.smem_bytes, plan.tmem_cols, plan.stages, plan.tile_k, T, nkb, T / grid, T % grid, sms,
                 have_dev ? "true" : "false", regs_txt, local_txt);
  } else {
    const long m_tiles = (M + plan.tile_m - 1) / plan.tile_m, n_tiles = (N + plan.tile_n - 1) / plan.tile_n;
    const long nkb = (K + plan.tile_k - 1) / plan.tile_k;
    const long units = m_tiles * n_tiles * plan.split_k;
    long groups = sms / plan.cluster;
    const long per_group = plan.cta_group == 2 ? units : (units + plan.cluster - 1) / plan.cluster;
    if (groups > per_group) groups = per_group;
    if (cfg && cfg->reserved[3] > 0 && groups > cfg->reserved[3] / plan.cluster) groups = cfg->reserved[3] / plan.cluster;
    if (groups < 1) groups = 1;
    const long ctas = groups * plan.cluster;
    const long streams = plan.cta_group == 2 ? groups : ctas;      // independent tile streams
    const long rounds = (units + streams - 1) / streams;           // tiles the busiest stream works through
    // one UMMA of 128 x tile_n x 16 per SM keeps the tensor pipe busy tile_n / 2 cycles (8192 dense
    // bf16 FLOP per cycle and SM); a tile of one stream is m_sub of them per 16 k
    const double umma_cycles = static_cast<double>(rounds) * (nkb / static_cast<double>(plan.split_k)) *
                               (plan.tile_k / 16) * plan.m_sub * (plan.tile_n / 2.0);
    n = snprintf(out, out_bytes,
                 "{\"kernel\": \"%s<%d,%d,%s>\", \"grid\": %ld, \"cluster\": %d, \"threads\": %d, \"smem_bytes\": %ld, "
                 "\"tmem_cols\": %d, \"acc_bufs\": %d, \"stages\": %d, \"tile\": [%d, %d, %d], \"group_m\": %d, \"split_k\": %d, "
                 "\"tiles\": %ld, \"k_blocks\": %ld, \"cta_groups\": %ld, \"waves\": %.3f, \"tiles_of_busiest_group\": %ld, "
                 "\"umma_bound_sm_cycles\": %.0f, \"x_ring\": {\"a_stages\": %d, \"a_slots\": %d, \"groups\": %d}, "
                 "\"sm_count\": %ld, \"sm_count_from_device\": %s, \"registers\": %s, \"local_bytes\": %s}",
                 kname, plan.cta_group, plan.m_sub,
                 plan.prologue ? "norm" : (plan.a_kmajor ? "kmajor" : (fam == FAM_RMSNORM ? "inline" : "lhsT")), ctas, plan.cluster,
                 threads, plan.smem_bytes, plan.tmem_cols, plan.acc_bufs, plan.stages, plan.tile_m, plan.tile_n, plan.tile_k,
                 plan.group_m, plan.split_k, units, nkb, groups, static_cast<double>(units) / streams, rounds, umma_cycles,
                 plan.a_stages, plan.a_slots, plan.groups, sms,
                 have_dev ? "true" : "false", regs_txt, local_txt);
  }
  if (n < 0 || static_cast<size_t>(n) >= out_bytes) return set_error(B200_ERR_BAD_ARG, "describe_launch: buffer of %zu bytes is too small", out_bytes);
  return B200_OK;
}

extern "C" int b200_default_cfg(const char* family, long M, long N, long K, b200_cfg* cfg) {
  (void)K;
  if (!cfg) return set_error(B200_ERR_BAD_ARG, "default_cfg: NULL pointer");
  Family fam = parse_family(family);
  if (fam == FAM_UNKNOWN)
    return set_error(B200_ERR_BAD_ARG, "unknown kernel family (expected matmul_lhsT_rhs, matmul_lhs_rhs or rmsnorm_matmul)");
  *cfg = default_cfg(fam == FAM_LHS ? FAM_LHST : fam, M, N);
  return B200_OK;
}

extern "C" size_t b200_workspace_bytes(const char* family, const b200_cfg* cfg, long M, long N, long K) {
  if (parse_family(family) != FAM_RMSNORM && cfg != nullptr && cfg->split_k > 1 && M > 0 && N > 0 && K > 0) {
    Plan plan;
    memset(&plan, 0, sizeof(plan));
    if (make_plan(parse_family(family), cfg, M, N, K, &plan) != B200_OK) return 0;
    return splitk_workspace_bytes(plan, M, N);
  }
  if (parse_family(family) != FAM_RMSNORM || M <= 0) return 0;
  if (M <= SKINNY_ROWS) return N > 0 ? skinny_workspace_bytes(N) : 0;
  if (cfg != nullptr && cfg->norm_mode == 1) return 0;  // inline norm needs no scratch
  return K > 0 ? prologue_workspace_bytes(M, K) : 0;
}

extern "C" int b200_matmul_lhsT_rhs(const void* lhsT, const void* rhs, void* out, long M, long N, long K,
                                    long ld_lhsT, long ld_rhs, long ld_out, const b200_cfg* cfg, void* workspace,
                                    size_t workspace_bytes, int* dev_status, void* stream) {
  LaunchArgs la{FAM_LHST, lhsT, rhs, nullptr, out, M, N, K, ld_lhsT ? ld_lhsT : M, ld_rhs ? ld_rhs : N,
                ld_out ? ld_out : N, 0.0f, workspace, workspace_bytes};
  Prepared pr;
  int rc = prepare_cached(la, cfg, dev_status, &pr);
  if (rc) return rc;
  return launch(pr, static_cast<cudaStream_t>(stream));
}

extern "C" int b200_matmul_lhs_rhs(const void* lhs, const void* rhs, void* out, long M, long N, long K, long ld_lhs,
                                   long ld_rhs, long ld_out, const b200_cfg* cfg, void* workspace,
                                   size_t workspace_bytes, int* dev_status, void* stream) {
  LaunchArgs la{FAM_LHS, lhs, rhs, nullptr, out, M, N, K, ld_lhs ? ld_lhs : K, ld_rhs ? ld_rhs : N,
                ld_out ? ld_out : N, 0.0f, workspace, workspace_bytes};
  Prepared pr;
  int rc = prepare_cached(la, cfg, dev_status, &pr);
  if (rc) return rc;
  return launch(pr, static_cast<cudaStream_t>(stream));
}

extern "C" int b200_rmsnorm_matmul(const void* x, const void* gamma, const void* w, void* out, long M, long N,
                                   long K, float eps, const b200_cfg* cfg, void* workspace, size_t workspace_bytes,
                                   int* dev_status, void* stream) {
  LaunchArgs la{FAM_RMSNORM, x, w, gamma, out, M, N, K, K, N, N, eps, workspace, workspace_bytes};
  Prepared pr;
  int rc = prepare_cached(la, cfg, dev_status, &pr);
  if (rc) return rc;
  return launch(pr, static_cast<cudaStream_t>(stream));
}

extern "C" int b200_time_kernel(const b200_problem* p, const b200_cfg* cfg, void* workspace, size_t workspace_bytes,
                                int* dev_status, void* flush_buf, size_t flush_bytes, int warmup, int iters,
                                float* ms_each, void* stream_v) {
  if (!p || !ms_each || iters <= 0 || warmup < 0) return set_error(B200_ERR_BAD_ARG, "time_kernel: bad arguments");
  Family fam = parse_family(p->family);
  if (fam == FAM_UNKNOWN) return set_error(B200_ERR_BAD_ARG, "time_kernel: unknown family");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  LaunchArgs la;
  la.fam = fam;
  la.a = p->a; la.b = p->b; la.gamma = p->gamma; la.out = p->out;
  la.M = p->M; la.N = p->N; la.K = p->K;
  if (fam == FAM_LHST) {
    la.ld_a = p->ld_a ? p->ld_a : p->M;
  } else {  // x[M,K] and lhs[M,K]: K contiguous
    la.ld_a = p->ld_a ? p->ld_a : p->K;
  }
  la.ld_b = p->ld_b ? p->ld_b : p->N;
  la.ld_out = p->ld_out ? p->ld_out : p->N;
  la.eps = p->eps;
  la.workspace = workspace;
  la.workspace_bytes = workspace_bytes;
  Prepared pr;
  int rc = prepare(la, cfg, dev_status, &pr);
  if (rc) return rc;

  std::vector<cudaEvent_t> ev(2 * static_cast<size_t>(iters), nullptr);
  for (auto& e : ev) {
    rc = check_cuda(cudaEventCreate(&e), "cudaEventCreate");
    if (rc) break;
  }
  for (int i = 0; i < warmup && rc == B200_OK; ++i) rc = launch(pr, stream);
  for (int i = 0; i < iters && rc == B200_OK; ++i) {
    if (flush_buf && flush_bytes)
      rc = check_cuda(cudaMemsetAsync(flush_buf, i & 0xff, flush_bytes, stream), "L2 flush memset");
    if (rc == B200_OK) rc = check_cuda(cudaEventRecord(ev[2 * i], stream), "cudaEventRecord");
    if (rc == B200_OK) rc = launch(pr, stream);
    if (rc == B200_OK) rc = check_cuda(cudaEventRecord(ev[2 * i + 1], stream), "cudaEventRecord");
  }
  if (rc == B200_OK) rc = check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
  for (int i = 0; i < iters && rc == B200_OK; ++i)
    rc = check_cuda(cudaEventElapsedTime(&ms_each[i], ev[2 * i], ev[2 * i + 1]), "cudaEventElapsedTime");
  for (auto& e : ev)
    if (e) cudaEventDestroy(e);
  if (rc == B200_OK && dev_status) {
    int host_status[B200_DEV_STATUS_INTS] = {0};
    rc = check_cuda(cudaMemcpy(host_status, dev_status, sizeof(host_status), cudaMemcpyDeviceToHost), "status copy");
    if (rc == B200_OK && host_status[0] != 0)
      rc = set_error(B200_ERR_DEVICE_WAIT,
                     "device-side wait expired: role %d barrier %d tile %d k-block %d CTA %d", host_status[1],
                     host_status[2], host_status[3], host_status[4], host_status[5]);
  }
  return rc;
}

// =============================================================================== allocation-free entry
// Some callers cannot hand the skinny kernel a workspace because they cannot allocate device
// memory at the point of the call: a decode loop running inside a serving engine that has
// already carved the whole device heap into its own pools, or a host thread that must not take
// the allocator's locks.  For them the same kernel runs on a scratch that is part of this
// library's device image: it costs NOALLOC_SCRATCH_BYTES on every GPU that loads the library,
// for the life of the process, and it caps N at B200_NOALLOC_MAX_N.
namespace b200 {
// tile counters + one partial-tile slot per tile and per CTA at the largest N served
// (the same layout skinny_workspace_bytes describes)
constexpr size_t NOALLOC_TILES = B200_NOALLOC_MAX_N / SKINNY_TILE_N;
constexpr size_t NOALLOC_SCRATCH_BYTES = ((NOALLOC_TILES * sizeof(int) + 255) / 256) * 256 +
                                         (NOALLOC_TILES + SKINNY_MAX_CTAS) * SKINNY_SLOT_FLOATS * sizeof(float);
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];
// Device address of the array, per device ordinal.  The symbol name above is only a host-side
// handle: it must be turned into an address with cudaGetSymbolAddress while that device is current.
static void* g_noalloc_addr[64] = {nullptr};
}  // namespace b200

extern "C" int b200_rmsnorm_matmul_noalloc(const void* x, const void* gamma, const void* w, void* out, long M,
                                           long N, long K, float eps, const b200_cfg* cfg, int* dev_status,
                                           void* stream_v) {
  if (M <= 0 || M > SKINNY_ROWS)
    return set_error(B200_ERR_BAD_SHAPE, "rmsnorm_matmul_noalloc: M=%ld, this entry point serves 1..%d rows", M,
                     SKINNY_ROWS);
  if (N <= 0 || N > B200_NOALLOC_MAX_N)
    return set_error(B200_ERR_BAD_SHAPE,
                     "rmsnorm_matmul_noalloc: N=%ld exceeds the built-in scratch (at most %d columns); use "
                     "b200_rmsnorm_matmul with a caller-provided workspace",
                     N, B200_NOALLOC_MAX_N);
  const size_t need = skinny_workspace_bytes(N);
  if (need > NOALLOC_SCRATCH_BYTES)
    return set_error(B200_ERR_BAD_SHAPE, "rmsnorm_matmul_noalloc: N=%ld needs %zu scratch bytes, %zu are built in", N,
                     need, NOALLOC_SCRATCH_BYTES);
  int dev = 0;
  int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
  if (rc) return rc;
  if (dev < 0 || dev >= 64) return set_error(B200_ERR_CUDA, "device ordinal %d out of range", dev);
  if (g_noalloc_addr[dev] == nullptr) {
    // first call on this device: resolve the address (do this before any stream capture)
    void* addr = nullptr;
    rc = check_cuda(cudaGetSymbolAddress(&addr, g_noalloc_scratch), "cudaGetSymbolAddress(built-in scratch)");
    if (rc) return rc;
    if (addr == nullptr) return set_error(B200_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_noalloc_addr[dev] = addr;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  // The array keeps whatever the previous call (or an aborted one) left.  Only the tile counters
  // must start at zero (partial tiles are written before they are read), so they are cleared on
  // the same stream.
  rc = check_cuda(cudaMemsetAsync(g_noalloc_addr[dev], 0, skinny_counter_bytes(N), stream),
                  "clearing the counters of the built-in scratch");
  if (rc) return rc;
  LaunchArgs la{FAM_RMSNORM, x, w, gamma, out, M, N, K, K, N, N, eps, g_noalloc_addr[dev], NOALLOC_SCRATCH_BYTES};
  Prepared pr;
  rc = prepare_cached(la, cfg, dev_status, &pr);  // a repeated call replays the prepared launch
  if (rc) return rc;
  return launch(pr, stream);
}

// ------------------------------------------------------------------- peer stores
// The exchange step of the large-M row split without a collective library: every GPU pushes the
// rows of C it has just computed into the same rows of every other GPU's copy of C, with plain
// 16-byte stores through peer-mapped pointers (NVLink; every peer at full rate through the switch).
// The kernel reads local memory only, waits for nothing and synchronises with nobody: the stores
// are complete when the kernel is, and a stream-ordered barrier among the ranks afterwards makes
// every copy of C whole.
constexpr int PEER_MAX = 8;
struct PeerDst {
  uint4* p[PEER_MAX];
  int n;
};
__global__ void __launch_bounds__(256) peer_store_kernel(const uint4* __restrict__ src, const PeerDst dst, const size_t n16) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  // four independent 16-byte loads in flight per thread, each stored to every peer
  for (; i + 3 * stride < n16; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = __ldcs(src + i + u * stride);
    for (int r = 0; r < dst.n; ++r) {
#pragma unroll
      for (int u = 0; u < 4; ++u) dst.p[r][i + u * stride] = v[u];
    }
  }
  for (; i < n16; i += stride) {
    const uint4 v = __ldcs(src + i);
    for (int r = 0; r < dst.n; ++r) dst.p[r][i] = v;
  }
}

extern "C" int b200_peer_store(const void* src, void* const* peer_dst, int n_peers, size_t bytes, int max_ctas, void* stream) {
  if (n_peers == 0 || bytes == 0) return B200_OK;
  if (!src || !peer_dst || n_peers < 0 || n_peers > PEER_MAX)
    return set_error(B200_ERR_BAD_ARG, "peer_store: need a source, a pointer table and 1..%d peers (got %d)", PEER_MAX, n_peers);
  if ((reinterpret_cast<uintptr_t>(src) & 15u) != 0 || bytes % 16 != 0)
    return set_error(B200_ERR_BAD_ARG, "peer_store: source and byte count must be multiples of 16");
  PeerDst d;
  memset(&d, 0, sizeof(d));
  d.n = n_peers;
  for (int r = 0; r < n_peers; ++r) {
    if (!peer_dst[r] || (reinterpret_cast<uintptr_t>(peer_dst[r]) & 15u) != 0)
      return set_error(B200_ERR_BAD_ARG, "peer_store: destination %d is NULL or not 16-byte aligned", r);
    d.p[r] = static_cast<uint4*>(peer_dst[r]);
  }
  // every destination must be device memory of another GPU that this GPU can reach, and peer
  // access from this GPU to that one must be on in this process (mapping a peer's memory, e.g.
  // through an IPC handle opened under the owner's device, does not turn it on by itself)
  int cur = 0;
  int rc = check_cuda(cudaGetDevice(&cur), "cudaGetDevice");
  if (rc) return rc;
  for (int r = 0; r < n_peers; ++r) {
    cudaPointerAttributes at;
    rc = check_cuda(cudaPointerGetAttributes(&at, peer_dst[r]), "peer_store: cudaPointerGetAttributes");
    if (rc) return rc;
    if (at.type != cudaMemoryTypeDevice)
      return set_error(B200_ERR_BAD_ARG, "peer_store: destination %d is not device memory", r);
    if (at.device == cur) continue;  // a local destination is fine too
    int can = 0;
    rc = check_cuda(cudaDeviceCanAccessPeer(&can, cur, at.device), "cudaDeviceCanAccessPeer");
    if (rc) return rc;
    if (!can) return set_error(B200_ERR_UNSUPPORTED, "peer_store: GPU %d cannot reach GPU %d", cur, at.device);
    const cudaError_t e = cudaDeviceEnablePeerAccess(at.device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) (void)cudaGetLastError();
    else if (e != cudaSuccess) return check_cuda(e, "cudaDeviceEnablePeerAccess");
  }
  DeviceInfo di;
  rc = device_info(&di);
  if (rc) return rc;
  const size_t n16 = bytes / 16;
  long ctas = static_cast<long>(di.sm_count) * 4;
  if (max_ctas > 0 && ctas > max_ctas) ctas = max_ctas;
  const long need = static_cast<long>((n16 + 255) / 256);
  if (ctas > need) ctas = need;
  if (ctas < 1) ctas = 1;
  peer_store_kernel<<<static_cast<unsigned>(ctas), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(src), d, n16);
  return check_cuda(cudaGetLastError(), "peer store launch");
}

// Maps an allocation that another process of this node exported with cudaIpcGetMemHandle into the
// CURRENT device's address space, turning on peer access from the current device to the owner's
// if they differ.  (A mapping made while the owner's device is current is of no use to kernels
// of this GPU: the address is then valid on the owner's device only.)
extern "C" int b200_ipc_open(const void* handle64, void** base) {
  if (!handle64 || !base) return set_error(B200_ERR_BAD_ARG, "ipc_open: NULL pointer");
  cudaIpcMemHandle_t h;
  static_assert(sizeof(h) == 64, "CUDA IPC memory handles are 64 bytes");
  memcpy(&h, handle64, sizeof(h));
  *base = nullptr;
  return check_cuda(cudaIpcOpenMemHandle(base, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
}
extern "C" int b200_ipc_close(void* base) {
  if (!base) return B200_OK;
  return check_cuda(cudaIpcCloseMemHandle(base), "cudaIpcCloseMemHandle");
}

// ------------------------------------------------------------------- checked build
#ifdef B200_CHECKED_BUILD
// Hands the wrappers arguments their checks must refuse.  Every access below is skipped by its
// check, so the kernel touches nothing: no tensor memory is allocated, the tensor map is never
// read.  32 lanes x 3 refusals.
__global__ void checked_selftest_kernel() {
  using namespace b200;
  st_shared_v4(cta_smem_bytes(), 0u, 0u, 0u, 0u);   // one byte past the shared window
  uint32_t r[16];
  tmem_ld_32x32b_x16(600u, r);                      // column 600 of 512
  tma_store_2d(nullptr, 0u, -8, 0);                 // a store at a negative coordinate
  if (r[0] != 0u) st_shared_v4(cta_smem_bytes(), r[0], 0u, 0u, 0u);  // keeps the load's result alive
}
#endif

extern "C" int b200_checked_build_report(long long* out4, int flags) {
  if (!out4) return set_error(B200_ERR_BAD_ARG, "checked_build_report: NULL pointer");
  out4[0] = out4[1] = out4[2] = out4[3] = 0;
#ifdef B200_CHECKED_BUILD
  if (flags & 2) {
    checked_selftest_kernel<<<1, 32>>>();
    int rc = check_cuda(cudaGetLastError(), "self-test launch");
    if (rc) return rc;
  }
  int rc = check_cuda(cudaDeviceSynchronize(), "checked_build_report: synchronize");
  if (rc) return rc;
  unsigned long long log[4];
  rc = check_cuda(cudaMemcpyFromSymbol(log, b200::g_check_log, sizeof log), "checked_build_report: read");
  if (rc) return rc;
  for (int i = 0; i < 4; ++i) out4[i] = static_cast<long long>(log[i]);
  if (flags & 1) {
    const unsigned long long zero[4] = {0, 0, 0, 0};
    rc = check_cuda(cudaMemcpyToSymbol(b200::g_check_log, zero, sizeof zero), "checked_build_report: clear");
    if (rc) return rc;
  }
  return B200_OK;
#else
  (void)flags;
  return set_error(B200_ERR_UNSUPPORTED, "this library was built without -DB200_CHECKED_BUILD");
#endif
}

#ifdef B200_MEASURE_HOOKS
// measurement build only: copies the GEMM kernels' boundary stamps (g_gemm_trace) to the host
extern "C" int b200_debug_gemm_trace(long long* host, size_t count) {
  if (count > 160 * 16) count = 160 * 16;
  return check_cuda(cudaMemcpyFromSymbol(host, b200::g_gemm_trace, count * sizeof(long long)), "trace copy");
}
#endif
