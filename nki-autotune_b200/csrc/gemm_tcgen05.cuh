// Persistent, warp-specialised tcgen05 GEMM for sm_100a:
//     C[M,N] = lhsT[K,M]^T . rhs[K,N]        (bf16 operands, both MN-major; fp32 accumulation)
//
// Replaces the PSUM-tiled Trainium kernel
//   kernel_library/matmul/lhsT_rhs/kernel_hand_90.92mfu.py:72-131  (matmul_block, load_block, store_block)
// with one fp32 accumulation over the whole of K in tensor memory.
//
// Warp roles (one CTA per SM, or a CTA pair sharing 256-row UMMAs):
//   warp 0      TMA producer   : waits empty[s], arms full[s], issues the tile loads of stage s
//   warp 1      UMMA issuer    : waits full[s], issues tile_k/16 UMMAs per accumulator block, commits
//                                to empty[s]; after the last k-block commits acc_full[b]
//   warps 2-9   epilogue       : wait acc_full[b], tcgen05.ld, bf16 into swizzled staging buffers,
//                                bulk tensor stores, arrive acc_empty[b]; two warps per lane quadrant
//                                take alternate 64-column chunks, so a 512-column accumulator (which
//                                cannot be double-buffered) is drained in half the time
// Warps 0 and 1 run their loops with all lanes converged and elect one lane per instruction.
// Work units are (tile, part of the K range); without split-K a unit is a whole tile.
//
// Shared-memory operand layout (what the TMA writes and the UMMA descriptors read), with the
// 128-byte swizzle: an MN-major operand tile [tile_k x W] is W/64 chunks, each chunk = tile_k
// rows of 128 B (64 consecutive m or n of one k).
//
// Every wait is bounded: when a wait gives up it records where in status[] and raises a
// CTA-wide abort flag so every role leaves its loop and the CTA frees its tensor memory.
#pragma once
#include <type_traits>
#include <cuda.h>
#include "ptx_sm100.cuh"

namespace b200 {

constexpr int MAX_STAGES = 12;
constexpr int EPI_WARPS = 8;  // two per tensor-memory lane quadrant; they share a tile's 64-column chunks
constexpr int GEMM_THREADS = 32 * (2 + EPI_WARPS);
// epilogue staging in shared memory: per epilogue warp one buffer of 32 rows x 64 bf16 columns
// (128-byte rows, 128-byte swizzle), written by the warp and read by its TMA store
constexpr int EPI_BUF_BYTES = 32 * 128;
constexpr int EPI_STAGE_BYTES = EPI_WARPS * EPI_BUF_BYTES;

// test hook (b200_cfg.reserved[0]): the producer issues nothing, so the consumers' bounded waits
// run out -- how the tests exercise the give-up path without faulting anything
constexpr int DEBUG_SKIP_PRODUCER = 1;
// measurement hooks, compiled only into builds made with -DB200_MEASURE_HOOKS (they make the
// kernels compute garbage on purpose): 2 = operands loaded once per stage slot, then only the
// barriers cycle; 3 = loads and barriers run, the UMMAs are not issued; 4 = the inline fused
// kernel's transform warps only cycle their barriers
#ifdef B200_MEASURE_HOOKS
constexpr int DEBUG_NO_RELOAD = 2;
constexpr int DEBUG_NO_MMA = 3;
constexpr int DEBUG_NO_TRANSFORM = 4;
#endif

#ifdef B200_MEASURE_HOOKS
// measurement build: clock64 stamps around the boundary between a CTA's third and fourth tile
// ([cta][0] tile start seen by the issuer, [1] its last UMMA and commit issued, [2] next tile's start;
// [3]/[6] accumulator seen full by an epilogue warp of either half, [4]/[7] its last tensor-memory
// load done, [5]/[8] its arrival on acc_empty; [9] issuer's first operands of the next tile seen)
__device__ long long g_gemm_trace[160 * 16];
#endif

struct GemmParams {
  int M, N, K;
  int tile_n, tile_k, stages;
  int umma_n;        // N of one UMMA: tile_n, or tile_n / 2 when the tile is two instructions wide (tile_n 512)
  int num_m_tiles;   // tiles of (128 * M_SUB * CTA_GROUP) rows
  int num_n_tiles;
  int num_k_blocks;
  int group_m;       // rasterisation group width (tiles along M)
  int acc_bufs;      // accumulator buffers in tensor memory: 1 or 2
  int acc_halves;    // 1: a single-buffered accumulator of two UMMA blocks (two row blocks, or two 256-column
                     // blocks) is handed over in halves, each with its own full / empty barrier (see the issuer)
  int tmem_cols;     // allocation size (power of two >= 32)
  long long ld_out;  // elements
  __nv_bfloat16* out;
  int* status;       // B200_DEV_STATUS_INTS ints or nullptr
  long long timeout_cycles;
  int split_k;       // parts the K range of every tile is split into (1 = none); parts are separate work units
  int kb_per_part;   // k-blocks per part
  int part_rows;     // split-K: rows of one part's fp32 partial array (num_m_tiles x tile rows)
  int debug_mode;    // 0, DEBUG_SKIP_PRODUCER, or (measurement builds) one of the other DEBUG_* hooks
  int record_clocks; // measurement aid: status[6]/[7] = longest CTA lifetime in SM cycles / nanoseconds
  // NORM variant only (fused RMSNorm with an in-kernel prologue):
  const __nv_bfloat16* x;      // [M,K] activations
  const __nv_bfloat16* gamma;  // [K] or nullptr
  __nv_bfloat16* xg;           // scratch [M,K]: x * gamma, the K-major A operand of the main loop
  float* rinv;                 // scratch [M]: rsqrt(mean_k x^2 + eps)
  unsigned int* norm_sync;     // scratch: [0] next row to claim, [1] CTAs that have left, [2 + i] rows of
                               // 128-row block i that are ready; all zero between launches
#ifdef B200_MEASURE_HOOKS
  unsigned long long* trace;   // measurement build: 8 globaltimer stamps per CTA (NORM variant)
#endif
  float eps, inv_k;
};

// Control block that follows the operand stages in dynamic shared memory.
struct alignas(16) Ctrl {
  uint64_t full[MAX_STAGES];    // operands of stage s have landed
  uint64_t empty[MAX_STAGES];   // UMMAs reading stage s have finished
  uint64_t acc_full[2];         // accumulator buffer b holds a finished tile
  uint64_t acc_empty[2];        // the epilogue has drained accumulator buffer b
  uint32_t tmem_base;
  volatile int abort_flag;
};

// Position in a ring of `depth` slots plus the parity of the current pass over it.
struct Ring {
  uint32_t s = 0, ph = 0;
  __device__ __forceinline__ void advance(uint32_t depth) {
    if (++s == depth) { s = 0; ph ^= 1u; }
  }
};

enum Role { ROLE_PRODUCER = 1, ROLE_MMA = 2, ROLE_EPILOGUE = 3, ROLE_TRANSFORM = 4 };

struct WaitCtx {
  Ctrl* ctrl;
  int* status;
  long long limit;
  int role;
};

template <bool CLUSTER_SCOPE>
__device__ __forceinline__ bool bounded_wait(const WaitCtx& w, uint32_t bar, uint32_t parity,
                                             int bar_id, int tile, int kb) {
  auto try_once = [&]() {
    if constexpr (CLUSTER_SCOPE) return mbar_try_wait_cluster(bar, parity);
    else return mbar_try_wait(bar, parity);
  };
  if (try_once()) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (!try_once()) {
    if ((++spins & 63u) == 0u) {
      if (w.ctrl->abort_flag) return false;
      if (clock64() - t0 > w.limit) {
        w.ctrl->abort_flag = 1;
        if (w.status != nullptr && atomicCAS(w.status, 0, 7 /* B200_ERR_DEVICE_WAIT */) == 0) {
          w.status[1] = w.role;
          w.status[2] = bar_id;
          w.status[3] = tile;
          w.status[4] = kb;
          w.status[5] = static_cast<int>(blockIdx.x);
        }
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int group_m, int& mt,
                                            int& nt) {
  const int per_group = group_m * num_n;
  const int g = t / per_group;
  const int first_m = g * group_m;
  const int gsize = min(group_m, num_m - first_m);
  const int r = t - g * per_group;
  mt = first_m + r % gsize;
  nt = r / gsize;
}

// A_MODE 0: C = lhsT^T . rhs (A MN-major from lhsT[K,M]).
// A_MODE 1 (NORM): out = (x / rms(x) * gamma) . w in one launch.  The epilogue warps of all CTAs
//   first run the norm pass: rows of x scaled by gamma go to the scratch xg, rinv[m] is stored, and
//   a counter per block of 128 rows says how many of its rows are done.  The same main loop runs
//   with A = xg (K-major); a producer waits (bounded) only for the row blocks of the tile it is
//   about to load, so the main loop of the first tiles overlaps the norm pass over later rows and
//   no CTA depends on the whole grid being resident.  The epilogue multiplies row m by rinv[m].
//   x is read once; xg costs one extra write and read of M*K*2 bytes, hidden under the tensor
//   work.  (kernel_library/rmsnorm_matmul/kernel_hand_online.py:5-17 is the two-pass form of the
//   same maths; its per-K-block interleaving of statistics and matmul, :307-346, is what the
//   overlap stands for.)
// A_MODE 2: C = lhs . rhs with lhs[M,K] K-major (matmul_lhs_rhs): the K-major operand path of
//   the NORM variant without prologue or row scale.  The reference needs a DMA-transpose pass
//   for this layout (kernel_library/matmul/lhs_rhs/kernel_handtuned_89.26mfu.py:226-287); the
//   UMMA takes it directly.
constexpr int A_LHST = 0, A_NORM = 1, A_KMAJOR_PLAIN = 2;

template <int CTA_GROUP, int M_SUB, int A_MODE = A_LHST>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_a,
                    const __grid_constant__ CUtensorMap tm_b,
                    const __grid_constant__ CUtensorMap tm_out, const GemmParams p) {
  constexpr bool NORM = (A_MODE == A_NORM);
  constexpr bool A_KMAJOR = (A_MODE != A_LHST);
  constexpr bool PAIR = (CTA_GROUP == 2);
  constexpr int MC = 128 * M_SUB;  // accumulator rows held by this CTA
  extern __shared__ uint8_t smem_raw[];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;

  const int tile_n = p.tile_n;
  const int tile_k = p.tile_k;
  const int stages = p.stages;
  const int nc = tile_n / CTA_GROUP;  // columns of the B tile this CTA loads
  const int umma_n = p.umma_n;
  const int n_sub = tile_n / umma_n;           // UMMAs side by side along N (1 or 2)
  const int nc_sub = umma_n / CTA_GROUP;       // columns this CTA supplies to one of them
  const uint32_t a_bytes = static_cast<uint32_t>(MC) * tile_k * 2u;
  const uint32_t b_bytes = static_cast<uint32_t>(nc) * tile_k * 2u;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_base = smem_base;
  const uint32_t b_base = a_base + stages * a_bytes;
  const uint32_t out_stage_base = b_base + stages * b_bytes;  // epilogue staging, 1024-byte aligned
  const uint32_t ctrl_addr = out_stage_base + EPI_STAGE_BYTES;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem_raw + (ctrl_addr - smem_u32(smem_raw)));

  const int acc_cols = M_SUB * tile_n;
  const int acc_bufs = p.acc_bufs;
  const int num_k_blocks = p.num_k_blocks;
  // work units: (tile, part of its K range); without split-K a unit is a tile
  const int split_k = p.split_k;
  const int total_tiles = p.num_m_tiles * p.num_n_tiles * split_k;
  const int first_tile = static_cast<int>(blockIdx.x) / CTA_GROUP;
  const int tile_stride = static_cast<int>(gridDim.x) / CTA_GROUP;

  // NORM: every warp claims its first row of the norm pass now; the answer arrives during set-up
  [[maybe_unused]] int norm_claim = 0;
  if constexpr (NORM) {
    if (lane == 0 && warp >= 2) norm_claim = static_cast<int>(atomicAdd(p.norm_sync, 1u));
  }
#ifdef B200_MEASURE_HOOKS
  if constexpr (NORM) {
    if (p.trace != nullptr && threadIdx.x == 0) p.trace[blockIdx.x * 8 + 0] = global_timer_ns();  // entry
  }
#endif
  long long life_c0 = 0;
  unsigned long long life_n0 = 0;
  if (p.record_clocks && threadIdx.x == 0) {
    life_c0 = clock64();
    life_n0 = global_timer_ns();
  }
  // ------------------------------------------------------------------ set-up
  if (threadIdx.x == 0) {
    ctrl->abort_flag = 0;
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
    tma_prefetch_desc(&tm_out);
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctrl->acc_full[b]), 1);
      mbar_init(smem_u32(&ctrl->acc_empty[b]), EPI_WARPS * CTA_GROUP);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<CTA_GROUP>(smem_u32(&ctrl->tmem_base), static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish<CTA_GROUP>();
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) {
    cluster_arrive();
    cluster_wait();
  }
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;

  WaitCtx wctx{ctrl, p.status, p.timeout_cycles, 0};

  // NORM: rows of x are ready for the main loop (xg written, rinv stored) in blocks of 128 rows;
  // norm_ready() waits, bounded, until block `blk` is complete.  Every lane polls the same word
  // (one transaction), so whichever lane is elected for the copies has made the acquire itself.
  constexpr int NORM_BLOCK = 128;
  auto norm_ready = [&](int blk, int tile) -> bool {
    const unsigned want = static_cast<unsigned>(min(NORM_BLOCK, p.M - blk * NORM_BLOCK));
    const int* word = reinterpret_cast<const int*>(p.norm_sync + 2 + blk);
    if (static_cast<unsigned>(ld_acquire_gpu(word)) >= want) return true;
    const long long t0 = clock64();
    while (static_cast<unsigned>(ld_acquire_gpu(word)) < want) {
      if (ctrl->abort_flag) return false;
      if (clock64() - t0 > p.timeout_cycles) {
        ctrl->abort_flag = 1;
        if (p.status != nullptr && atomicCAS(p.status, 0, 7) == 0) {
          p.status[1] = wctx.role;
          p.status[2] = 600;  // rows of x not ready
          p.status[3] = tile;
          p.status[4] = blk;
          p.status[5] = static_cast<int>(blockIdx.x);
        }
        return false;
      }
      __nanosleep(100);
    }
    return true;
  };
  // ---------------------------------------------------------------- the norm pass over x
  // xg = x * gamma (bf16, one rounding) and rinv[m], one row per claim from a global counter (any
  // CTA that runs makes progress; all warps of the grid work on the same thousand rows, so row
  // blocks become ready in the order the tiles need them).  The eight epilogue warps of every
  // CTA do the pass: they have nothing to drain until the first tile is finished.  The producer
  // and issuer warps start the main loop at once; a producer waits for the row blocks of its
  // tile.  All loads of a row (x and gamma, 32 x 16 bytes per lane) are issued before the first
  // store, so nothing serialises them.
  [[maybe_unused]] const int norm_pieces = p.K / 8;  // 16-byte pieces per row (K is a multiple of 64)
  auto norm_row = [&](int row) {
    if (!B200_CHECK(row >= 0 && row < p.M, CHK_GLOBAL, row, p.M)) return;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const uint4 ones = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);  // bf16 1.0 pairs
    const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<long long>(row) * p.K);
    uint4* dst = reinterpret_cast<uint4*>(p.xg + static_cast<long long>(row) * p.K);
    float ss = 0.0f, tt = 0.0f;
    for (int i0 = lane; i0 < norm_pieces; i0 += 512) {
      uint4 v[16], g[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int i = i0 + u * 32;
        v[u] = (i < norm_pieces) ? __ldg(src + i) : zero;
        g[u] = (i < norm_pieces && p.gamma != nullptr) ? __ldg(reinterpret_cast<const uint4*>(p.gamma) + i) : ones;
      }
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int i = i0 + u * 32;
        const uint32_t w4[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const float lo = __uint_as_float(w4[w] << 16), hi = __uint_as_float(w4[w] & 0xffff0000u);
          ss = fmaf(lo, lo, ss);
          tt = fmaf(hi, hi, tt);
        }
        if (i < norm_pieces && p.xg != nullptr)  // without gamma the main loop reads x itself: nothing to write
          dst[i] = make_uint4(mul_bf16x2(v[u].x, g[u].x), mul_bf16x2(v[u].y, g[u].y), mul_bf16x2(v[u].z, g[u].z),
                              mul_bf16x2(v[u].w, g[u].w));
      }
    }
    ss += tt;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    // publish: the row's stores (all lanes'), then one more row of its block
    __syncwarp();
    if (lane == 0) {
      p.rinv[row] = rsqrtf(ss * p.inv_k + p.eps);
      __threadfence();
      atomicAdd(p.norm_sync + 2 + row / NORM_BLOCK, 1u);
    }
  };
  // works on claimed rows until the counter has passed M; the next claim is made before the
  // current row's loads, which hides its latency
  auto norm_pass = [&]() {
    int cur = __shfl_sync(0xffffffffu, norm_claim, 0);
    while (cur < p.M) {
      int nxt = 0;
      if (lane == 0) nxt = static_cast<int>(atomicAdd(p.norm_sync, 1u));
      norm_row(cur);
      cur = __shfl_sync(0xffffffffu, nxt, 0);
    }
  };
  const bool run_roles = true;

  // ------------------------------------------------------------------ TMA producer
  if (!run_roles) {
    // a CTA that gave up at the grid barrier skips straight to the teardown
  } else if (warp == 0) {
    // the whole warp runs the loop converged; one elected lane issues each copy and arrival
    if (p.debug_mode != DEBUG_SKIP_PRODUCER) {
      wctx.role = ROLE_PRODUCER;
      uint32_t it = 0;
      Ring ring;
      bool ok = true;
      [[maybe_unused]] unsigned long long norm_seen = 0;  // 128-row blocks of x already seen complete
      const int b_chunks = nc / 64, sub_chunks = nc_sub / 64, sub_jump = umma_n - nc_sub;
      for (int unit = first_tile; unit < total_tiles && ok; unit += tile_stride) {
        const int tile = unit / split_k, part = unit - tile * split_k;
        const int kb0 = part * p.kb_per_part, kb1 = min(kb0 + p.kb_per_part, num_k_blocks);
        int mt, nt;
        tile_coords(tile, p.num_m_tiles, p.num_n_tiles, p.group_m, mt, nt);
        const int m_base = (mt * CTA_GROUP + static_cast<int>(cta_rank)) * MC;
        const int n_base = nt * tile_n + static_cast<int>(cta_rank) * nc_sub;  // first UMMA's share; next at + umma_n
        // a tile may hang over the edge of C (TMA fills and clips), but it starts inside it
        if (!B200_CHECK(mt * CTA_GROUP * MC < p.M && nt * tile_n < p.N && kb0 < kb1 && kb1 <= num_k_blocks, CHK_SCHEDULE, tile, total_tiles)) break;
        // the loads of one stage
        auto arm_stage = [&](uint32_t s) {
          const uint32_t full_local = smem_u32(&ctrl->full[s]);
          if constexpr (PAIR) {
            if (cta_rank == 0) mbar_arrive_expect_tx_elect(full_local, 2u * (a_bytes + b_bytes));
          } else {
            mbar_arrive_expect_tx_elect(full_local, a_bytes + b_bytes);
          }
        };
        auto load_a = [&](uint32_t s, int kb) {
          const uint32_t a_s = a_base + s * a_bytes;
          const int k0 = kb * tile_k;
          if (!B200_CHECK(s < static_cast<uint32_t>(stages) && k0 < p.K, CHK_SCHEDULE, s, kb)) return;
          const uint32_t full_local = smem_u32(&ctrl->full[s]);
          if constexpr (PAIR) {
            const uint32_t full_leader = map_to_cta(full_local, 0);
            if constexpr (A_KMAJOR) {
              for (int c = 0; c < tile_k / 64; ++c)
                tma_load_2d_pair_elect(a_s + c * MC * 128, &tm_a, full_leader, k0 + 64 * c, m_base);
            } else {
              for (int c = 0; c < MC / 64; ++c)
                tma_load_2d_pair_elect(a_s + c * tile_k * 128, &tm_a, full_leader, m_base + 64 * c, k0);
            }
          } else {
            if constexpr (A_KMAJOR) {
              for (int c = 0; c < tile_k / 64; ++c)
                tma_load_2d_elect(a_s + c * MC * 128, &tm_a, full_local, k0 + 64 * c, m_base);
            } else {
              for (int c = 0; c < MC / 64; ++c)
                tma_load_2d_elect(a_s + c * tile_k * 128, &tm_a, full_local, m_base + 64 * c, k0);
            }
          }
        };
        auto load_b = [&](uint32_t s, int kb) {
          const uint32_t b_s = b_base + s * b_bytes;
          const int k0 = kb * tile_k;
          if (!B200_CHECK(s < static_cast<uint32_t>(stages) && k0 < p.K, CHK_SCHEDULE, s, kb)) return;
          const uint32_t full_local = smem_u32(&ctrl->full[s]);
          // B chunks of 64 columns; after this CTA's share of one UMMA the column jumps to the next UMMA
          if constexpr (PAIR) {
            const uint32_t full_leader = map_to_cta(full_local, 0);
            for (int c = 0, col = n_base, in_sub = 0; c < b_chunks; ++c) {
              tma_load_2d_pair_elect(b_s + c * tile_k * 128, &tm_b, full_leader, col, k0);
              col += 64;
              if (++in_sub == sub_chunks) { in_sub = 0; col += sub_jump; }
            }
          } else {
            for (int c = 0, col = n_base, in_sub = 0; c < b_chunks; ++c) {
              tma_load_2d_elect(b_s + c * tile_k * 128, &tm_b, full_local, col, k0);
              col += 64;
              if (++in_sub == sub_chunks) { in_sub = 0; col += sub_jump; }
            }
          }
        };
        if constexpr (NORM) {
          if (p.xg != nullptr) {  // A = xg: this CTA's rows of the tile must have been written
            for (int blk = m_base / NORM_BLOCK; blk * NORM_BLOCK < min(m_base + MC, p.M) && ok; ++blk)
              if (blk >= 64 || !((norm_seen >> blk) & 1ull)) {
                ok = norm_ready(blk, tile);
                ok = __all_sync(0xffffffffu, ok);
                if (ok && blk < 64) norm_seen |= 1ull << blk;
              }
            if (!ok) break;
            // order the other CTAs' generic-proxy stores to xg before this CTA's TMA (async proxy) loads
            asm volatile("fence.proxy.async;" ::: "memory");
          }
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it, ring.advance(stages)) {
          const uint32_t s = ring.s;
          const uint32_t ph = ring.ph;
          ok = bounded_wait<false>(wctx, smem_u32(&ctrl->empty[s]), ph ^ 1u, 100 + s, tile, kb);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
#ifdef B200_MEASURE_HOOKS
          if (p.debug_mode == DEBUG_NO_RELOAD && it >= static_cast<uint32_t>(stages)) {
            // operands stay as first loaded, only the barrier protocol runs
            if (!PAIR || cta_rank == 0) mbar_arrive_elect(smem_u32(&ctrl->full[s]));
            continue;
          }
#endif
          arm_stage(s);
          load_a(s, kb);
          load_b(s, kb);
        }
      }
      // tail: every stage released, so no UMMA-completion arrival is still on its way to
      // this CTA's barriers when the CTA exits
      for (int i = 0; i < stages && ok; ++i, ring.advance(stages)) {
        ok = bounded_wait<false>(wctx, smem_u32(&ctrl->empty[ring.s]), ring.ph ^ 1u, 150 + ring.s, -1, i);
        ok = __all_sync(0xffffffffu, ok);
      }
    }
    __syncwarp();
  }
  // ------------------------------------------------------------------ UMMA issuer
  else if (warp == 1) {
    // the whole warp runs the issue loop converged; one elected lane issues each UMMA and commit
    if (cta_rank == 0) {
      wctx.role = ROLE_MMA;
      const uint32_t idesc =
          make_idesc_bf16_f32(128 * CTA_GROUP, umma_n, A_KMAJOR ? 0 : 1, 1);
      const uint32_t mn_lbo = static_cast<uint32_t>(tile_k) * 128u;
      // descriptors: the high word (stride offset, version, swizzle) and the leading offset are
      // fixed; only the 14-bit start-address field moves (16-byte units: 128 per 16 k-rows)
      const uint64_t a_desc0 = make_smem_desc_sw128(a_base, mn_lbo, 1024);
      const uint64_t b_desc0 = make_smem_desc_sw128(b_base, mn_lbo, 1024);
      const uint32_t a_step = a_bytes >> 4, b_step = b_bytes >> 4, sub_step = (2u * mn_lbo) >> 4;
      const uint32_t nsub_step = (static_cast<uint32_t>(nc_sub / 64) * mn_lbo) >> 4;  // next UMMA's B chunks
      const int nk16 = tile_k / 16;
#ifdef B200_MEASURE_HOOKS
      const bool issue_enabled = p.debug_mode != DEBUG_NO_MMA;
#else
      constexpr bool issue_enabled = true;
#endif
      Ring ring, acc;
      bool ok = true;
      // A single-buffered accumulator made of two UMMA blocks (512x256: two row blocks; 256x512: two
      // 256-column blocks) is handed over in halves: the tile's last k-block issues all of half 0's
      // UMMAs first and commits half 0, so the epilogue drains half 0 while half 1's UMMAs still run;
      // the next tile's first k-block issues half 0 as soon as half 0 is drained and half 1 after
      // that.  Barriers acc_full[h] / acc_empty[h] then stand for half h (with one buffer, index 1 is
      // free for that), and both flip once per tile.
      const bool halves = p.acc_halves != 0;
      const auto commit_to = [&](uint64_t* bar) {
        if constexpr (PAIR) umma_commit_pair_elect(smem_u32(bar), 3);
        else umma_commit_1cta_elect(smem_u32(bar));
      };
      for (int unit = first_tile; unit < total_tiles && ok; unit += tile_stride, acc.advance(acc_bufs)) {
        const int tile = unit / split_k, part = unit - tile * split_k;
        const int kb0 = part * p.kb_per_part, kb1 = min(kb0 + p.kb_per_part, num_k_blocks);
        const uint32_t b = acc.s;
        ok = bounded_wait<false>(wctx, smem_u32(&ctrl->acc_empty[b]), acc.ph ^ 1u, 200 + b, tile, -1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
#ifdef B200_MEASURE_HOOKS
        if (lane == 0 && unit == first_tile + 2 * tile_stride) g_gemm_trace[blockIdx.x * 16 + 0] = clock64();
        if (lane == 0 && unit == first_tile + 3 * tile_stride) g_gemm_trace[blockIdx.x * 16 + 2] = clock64();
#endif
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + b * static_cast<uint32_t>(acc_cols);
        for (int kb = kb0; kb < kb1; ++kb, ring.advance(stages)) {
          const uint32_t s = ring.s;
          ok = bounded_wait<false>(wctx, smem_u32(&ctrl->full[s]), ring.ph, 300 + s, tile, kb);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
#ifdef B200_MEASURE_HOOKS
          if constexpr (NORM) {
            if (p.trace != nullptr && lane == 0 && unit == first_tile && kb == kb0) p.trace[blockIdx.x * 8 + 3] = global_timer_ns();  // first operands landed
          }
          if (lane == 0 && unit == first_tile + 3 * tile_stride && kb == kb0) g_gemm_trace[blockIdx.x * 16 + 9] = clock64();
#endif
          tc_fence_after();
          const uint64_t adesc0 = a_desc0 + s * a_step;
          const uint64_t bdesc0 = b_desc0 + s * b_step;
          // One k-block of UMMAs.  NS (instructions side by side along N) is a compile-time constant so
          // that the common NS = 1 loop unrolls into a straight run of instructions; HALF = -1 issues
          // every block of the tile (16 k at a time), HALF = 0 / 1 only that half of the accumulator.
          auto issue_k_block = [&](auto ns_const, auto half_const) {
            constexpr int NS = decltype(ns_const)::value;
            constexpr int HALF = decltype(half_const)::value;
            uint64_t adesc = adesc0, bdesc = bdesc0;
#pragma unroll 4
            for (int k16 = 0; k16 < nk16; ++k16, adesc += 128, bdesc += 128) {
#pragma unroll
              for (int mi = 0; mi < M_SUB; ++mi) {
                if (HALF >= 0 && M_SUB == 2 && mi != HALF) continue;
                uint64_t ad = adesc + mi * sub_step;
                if constexpr (A_KMAJOR)  // K-major x tile: 64-wide k chunks of MC rows x 128 B, 32 B per 16 k
                  ad = make_smem_desc_sw128(a_base + s * a_bytes + (k16 >> 2) * (MC * 128) + mi * (128 * 128) +
                                                (k16 & 3) * 32, 16, 1024);
#pragma unroll
                for (int ns = 0; ns < NS; ++ns) {
                  if (HALF >= 0 && M_SUB == 1 && ns != HALF) continue;
                  umma_bf16_elect<CTA_GROUP>(d_tmem + static_cast<uint32_t>(mi * tile_n + ns * umma_n), ad,
                                       bdesc + ns * nsub_step, idesc, ((kb - kb0) | k16) != 0 ? 1u : 0u);
                }
              }
            }
          };
          auto issue = [&](auto half_const) {
            if (!issue_enabled) return;
            if (n_sub == 1) issue_k_block(std::integral_constant<int, 1>{}, half_const);
            else issue_k_block(std::integral_constant<int, 2>{}, half_const);
          };
          if (halves) {
            // Half by half in every k-block, so that the first and last k-block of a tile -- which hand
            // the halves over separately -- run the same instructions as all the others (a path taken
            // once per tile would be fetched cold every time)
            issue(std::integral_constant<int, 0>{});
            if (kb == kb1 - 1) commit_to(&ctrl->acc_full[0]);
            if (kb == kb0) {  // (half 0 was waited for above)
              ok = bounded_wait<false>(wctx, smem_u32(&ctrl->acc_empty[1]), acc.ph ^ 1u, 201, tile, -1);
              ok = __all_sync(0xffffffffu, ok);
              if (!ok) break;
              tc_fence_after();
            }
            issue(std::integral_constant<int, 1>{});
          } else {
            issue(std::integral_constant<int, -1>{});
          }
          commit_to(&ctrl->empty[s]);
        }
        if (!ok) break;
        commit_to(&ctrl->acc_full[halves ? 1 : b]);
#ifdef B200_MEASURE_HOOKS
        if (lane == 0 && unit == first_tile + 2 * tile_stride) g_gemm_trace[blockIdx.x * 16 + 1] = clock64();
        if constexpr (NORM) {
          if (p.trace != nullptr && lane == 0 && unit == first_tile) p.trace[blockIdx.x * 8 + 4] = global_timer_ns();  // first tile issued
          if (p.trace != nullptr && lane == 0) p.trace[blockIdx.x * 8 + 6] = global_timer_ns();  // last tile issued
        }
#endif
      }
    }
    __syncwarp();
  }
  // ------------------------------------------------------------------ epilogue
  else if (warp < 2 + EPI_WARPS) {
    wctx.role = ROLE_EPILOGUE;
    const int q = warp & 3;          // tensor-memory lane quadrant this warp may read
    const int eg = (warp - 2) >> 2;  // which of the quadrant's two warps: it takes chunks eg, eg + 2, ...
    const uint32_t acc_empty_leader =
        PAIR ? map_to_cta(smem_u32(&ctrl->acc_empty[0]), 0) : smem_u32(&ctrl->acc_empty[0]);
    const uint32_t buf = out_stage_base + static_cast<uint32_t>(warp - 2) * EPI_BUF_BYTES;
    Ring acc;
    bool ok = true;
    [[maybe_unused]] unsigned long long norm_seen = 0;
    if constexpr (NORM) {
      // the epilogue warps have nothing to drain until the first tile is finished: they take the
      // rest of the norm pass
      norm_pass();
#ifdef B200_MEASURE_HOOKS
      if (p.trace != nullptr && threadIdx.x == 64) p.trace[blockIdx.x * 8 + 2] = global_timer_ns();  // norm pass done in this CTA
#endif
    }
    for (int unit = first_tile; unit < total_tiles && ok; unit += tile_stride, acc.advance(acc_bufs)) {
      const int tile = unit / split_k, part = unit - tile * split_k;
      int mt, nt;
      tile_coords(tile, p.num_m_tiles, p.num_n_tiles, p.group_m, mt, nt);
      const int m_base = (mt * CTA_GROUP + static_cast<int>(cta_rank)) * MC;
      const int n_base = nt * tile_n;
      const int b = static_cast<int>(acc.s);
      const uint32_t aph = acc.ph;
      [[maybe_unused]] float row_scale[M_SUB];
      if constexpr (NORM) {
        // rinv of this tile's rows comes from other CTAs: make sure their blocks are complete, and
        // fetch the factors while the tile is still being accumulated
        for (int blk = m_base / NORM_BLOCK; blk * NORM_BLOCK < min(m_base + MC, p.M) && ok; ++blk)
          if (blk >= 64 || !((norm_seen >> blk) & 1ull)) {
            ok = norm_ready(blk, tile);
            ok = __all_sync(0xffffffffu, ok);
            if (ok && blk < 64) norm_seen |= 1ull << blk;
          }
        if (!ok) break;
#pragma unroll
        for (int mi = 0; mi < M_SUB; ++mi) {
          const int row = m_base + mi * 128 + q * 32 + lane;
          row_scale[mi] = row < p.M ? __ldcg(p.rinv + row) : 0.0f;
        }
      }
      const bool halves = p.acc_halves != 0;  // then b == 0 and acc_full[h] / acc_empty[h] stand for half h
      ok = bounded_wait<false>(wctx, smem_u32(&ctrl->acc_full[b]), aph, 500 + b, tile, -1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
#ifdef B200_MEASURE_HOOKS
      const bool tr = lane == 0 && (warp == 2 || warp == 6) && unit == first_tile + 2 * tile_stride;
      const int tr0 = blockIdx.x * 16 + (warp == 2 ? 3 : 6);
      if (tr) g_gemm_trace[tr0] = clock64();
      if constexpr (NORM) {
        if (p.trace != nullptr && threadIdx.x == 64 && unit == first_tile) p.trace[blockIdx.x * 8 + 5] = global_timer_ns();  // first tile seen by the epilogue
      }
#endif
      tc_fence_after();
      auto release_accumulator = [&](int which) {
        // every tensor-memory load of this warp has completed (tcgen05.wait::ld): the issuer may
        // overwrite the accumulator.  No data in memory is handed over with this arrival, so the
        // remote form needs no release fence (which costs about 2000 cycles here).
        tc_fence_before();
        __syncwarp();
#ifdef B200_MEASURE_HOOKS
        if (tr) g_gemm_trace[tr0 + 1] = clock64();
#endif
        if (lane == 0) {
          if constexpr (PAIR) mbar_arrive_cluster_relaxed(acc_empty_leader + which * 8);
          else mbar_arrive(acc_empty_leader + which * 8);
        }
#ifdef B200_MEASURE_HOOKS
        if (tr) g_gemm_trace[tr0 + 2] = clock64();
#endif
      };
      if (split_k > 1) {
        // split-K: this unit's fp32 partial goes to its part's array in the scratch (rows
        // part * part_rows + ...), 32 columns = one 128-byte staging row at a time; a second
        // kernel sums the parts.  Same staging buffer and swizzle as the bf16 path.
#pragma unroll
        for (int mi = 0; mi < M_SUB; ++mi) {
          const int row0 = m_base + mi * 128 + q * 32;  // first of this warp's 32 rows
          for (int c = eg; c < tile_n / 64; c += EPI_WARPS / 4) {
            uint32_t r0[32], r1[32];
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                   static_cast<uint32_t>(b * acc_cols + mi * tile_n + c * 64);
            tmem_ld_32x32b_x32(taddr, r0);
            tmem_ld_32x32b_x32(taddr + 32u, r1);
            tmem_ld_wait();
            const int col0 = n_base + c * 64;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              if (row0 < p.M && col0 + 32 * h < p.N) {
                if (lane == 0) tma_store_wait_read<0>();
                __syncwarp();
                const uint32_t row_addr = buf + static_cast<uint32_t>(lane) * 128u;
                const uint32_t sw = static_cast<uint32_t>(lane & 7);
                const uint32_t* r = h ? r1 : r0;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  st_shared_v4(row_addr + ((static_cast<uint32_t>(j) ^ sw) << 4), r[j * 4], r[j * 4 + 1], r[j * 4 + 2],
                               r[j * 4 + 3]);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                  tma_store_2d(&tm_out, buf, col0 + 32 * h, part * p.part_rows + row0);
                  tma_store_commit();
                }
              }
            }
          }
        }
        release_accumulator(b);
      } else {
        // Phase 1: all of this warp's chunks (at most four: two per 128-row block, or four of a
        // 512-column tile) go from tensor memory to registers as packed bf16, 64 accumulator
        // columns of this lane's row at a time, and the accumulator is released -- the issuer
        // starts the next tile while phase 2 runs.  Phase 2: chunk by chunk, one 128-byte row per
        // lane into the staging buffer (16-byte piece j lands at piece j ^ (row & 7): the
        // 128-byte swizzle the store's tensor map undoes, conflict-free for the warp's 16-byte
        // shared stores), then one bulk tensor store; rows / columns past the edge are clipped.
        constexpr int SLOTS = 4, PER_MI = SLOTS / M_SUB;
        uint32_t packed[SLOTS][32];
#pragma unroll
        for (int mi = 0; mi < M_SUB; ++mi) {
          float scale = 1.0f;
          if constexpr (NORM) scale = row_scale[mi];
#pragma unroll
          for (int ci = 0; ci < PER_MI; ++ci) {
            const int c = eg + ci * (EPI_WARPS / 4);
            // accumulator handed over in halves: slots 0, 1 are half 0 (row block 0, or columns 0..255
            // of a 512-column tile), slots 2, 3 half 1.  Before the first chunk of half 1: half 0 goes
            // back to the issuer, and half 1 has to be complete.
            if (mi * PER_MI + ci == SLOTS / 2 && halves) {
              release_accumulator(0);
              ok = bounded_wait<false>(wctx, smem_u32(&ctrl->acc_full[1]), aph, 501, tile, -1);
              ok = __all_sync(0xffffffffu, ok);
              if (!ok) break;
              tc_fence_after();
            }
            if (c < tile_n / 64) {
              const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                     static_cast<uint32_t>(b * acc_cols + mi * tile_n + c * 64);
#pragma unroll
              for (int h = 0; h < 2; ++h) {  // 32 columns at a time keeps the register peak below the cap
                uint32_t r[32];
                tmem_ld_32x32b_x32(taddr + 32u * h, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  packed[mi * PER_MI + ci][16 * h + j] =
                      pack_bf16x2(__uint_as_float(r[2 * j]) * scale, __uint_as_float(r[2 * j + 1]) * scale);
              }
            }
          }
          if (!ok) break;
        }
        if (!ok) break;
        release_accumulator(halves ? 1 : b);
#pragma unroll
        for (int mi = 0; mi < M_SUB; ++mi) {
          const int row0 = m_base + mi * 128 + q * 32;  // first of this warp's 32 rows
#pragma unroll
          for (int ci = 0; ci < PER_MI; ++ci) {
            const int c = eg + ci * (EPI_WARPS / 4);
            const int col0 = n_base + c * 64;
            if (c < tile_n / 64 && row0 < p.M && col0 < p.N) {  // warp-uniform
              if (lane == 0) tma_store_wait_read<0>();  // the store that last read the buffer has drained it
              __syncwarp();
              const uint32_t row_addr = buf + static_cast<uint32_t>(lane) * 128u;
              const uint32_t sw = static_cast<uint32_t>(lane & 7);
              const uint32_t* pk = packed[mi * PER_MI + ci];
#pragma unroll
              for (int j = 0; j < 8; ++j)
                st_shared_v4(row_addr + ((static_cast<uint32_t>(j) ^ sw) << 4), pk[4 * j], pk[4 * j + 1], pk[4 * j + 2],
                             pk[4 * j + 3]);
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_2d(&tm_out, buf, col0, row0);
                tma_store_commit();
              }
            }
          }
        }
      }
    }
    if (lane == 0) tma_store_wait_all<0>();  // staging buffers are read out and the rows written before exit
#ifdef B200_MEASURE_HOOKS
    if constexpr (NORM) {
      if (p.trace != nullptr && threadIdx.x == 64) p.trace[blockIdx.x * 8 + 7] = global_timer_ns();  // epilogue done
    }
#endif
  }
  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (ctrl->abort_flag && threadIdx.x == 0) {
    // give tile loads that are still in flight a bounded time to land before the CTA's
    // shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) __nanosleep(1000);
  }
  if constexpr (PAIR) {
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<CTA_GROUP>(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
  if constexpr (NORM) {
    // the last CTA to leave puts the counters back to zero for the next launch (a CTA that gave
    // up leaves them as they are: the scratch is undefined after a failed launch)
    if (threadIdx.x == 0 && ctrl->abort_flag == 0) {
      __threadfence();
      if (atomicAdd(p.norm_sync + 1, 1u) == gridDim.x - 1) {
        const int blocks = (p.M + NORM_BLOCK - 1) / NORM_BLOCK;
        for (int i = 0; i < blocks + 2; ++i) p.norm_sync[i] = 0u;
        __threadfence();
      }
    }
  }
  if (p.record_clocks && threadIdx.x == 0 && p.status != nullptr) {
    atomicMax(&p.status[6], static_cast<int>(clock64() - life_c0));
    atomicMax(&p.status[7], static_cast<int>(global_timer_ns() - life_n0));
  }
}

}  // namespace b200
