// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   MODE_LHST   : C[M,N] = lhsT[K,M]^T . rhs[K,N]            (both operands MN-major)
//   MODE_RMSNORM: out[M,N] = (x/rms(x) * gamma)[M,K] . w[K,N]  (x K-major, w MN-major)
//
// Replaces the PSUM-tiled Trainium kernels
//   kernel_library/matmul/lhsT_rhs/kernel_hand_90.92mfu.py:72-131  (matmul_block, load_block, store_block)
//   kernel_library/rmsnorm_matmul/kernel_hand_online.py:93-353     (square-sum, rsqrt, scale, drain)
// with one fp32 accumulation over the whole of K in tensor memory.
//
// Warp roles (one CTA per SM, or a CTA pair sharing one 256-row UMMA):
//   warp 0      TMA producer   : waits empty[s], arms full[s], issues the tile loads of stage s
//   warp 1      UMMA issuer    : waits full[s] (ready[s] when fused), issues tile_k/16 UMMAs,
//                                commits to empty[s]; after the last k-block commits acc_full[b]
//   warps 2-5   epilogue       : wait acc_full[b], tcgen05.ld, (x rinv), bf16, global stores,
//                                arrive acc_empty[b]
//   warps 6-9   (fused only)   : per stage read the x tile in shared memory, accumulate the
//                                per-row sum of squares, scale by gamma in place, publish
//                                ready[s]; at the end of a tile publish rinv[row]
//
// Shared-memory operand layout (what the TMA writes and the UMMA descriptors read), all with
// the 128-byte swizzle:
//   MN-major operand tile [tile_k x W]: W/64 chunks, each chunk = tile_k rows of 128 B
//   K-major  operand tile [R x tile_k]: tile_k/64 chunks, each chunk = R rows of 128 B
//
// Every wait is bounded: when a wait gives up it records where in status[] and raises a
// CTA-wide abort flag so every role leaves its loop and the CTA frees its tensor memory.
#pragma once
#include <cuda.h>
#include "ptx_sm100.cuh"

namespace b200 {

constexpr int MODE_LHST = 0;
constexpr int MODE_RMSNORM = 1;

constexpr int MAX_STAGES = 12;

struct GemmParams {
  int M, N, K;
  int tile_n, tile_k, stages;
  int num_m_tiles;   // tiles of (128 * M_SUB * CTA_GROUP) rows
  int num_n_tiles;
  int num_k_blocks;
  int group_m;       // rasterisation group width (tiles along M)
  int acc_bufs;      // accumulator buffers in tensor memory: 1 or 2
  int tmem_cols;     // allocation size (power of two >= 32)
  long long ld_out;  // elements
  float eps, inv_k;
  __nv_bfloat16* out;
  const __nv_bfloat16* gamma;
  int* status;       // B200_DEV_STATUS_INTS ints or nullptr
  long long timeout_cycles;
  int debug_skip_producer;  // test hook: the producer issues nothing, so waits run out
};

// Control block that follows the operand stages in dynamic shared memory.
struct alignas(16) Ctrl {
  uint64_t full[MAX_STAGES];    // operands of stage s have landed (fused: w tile only)
  uint64_t full_a[MAX_STAGES];  // fused: x tile of stage s has landed (local to each CTA)
  uint64_t ready[MAX_STAGES];   // fused: x tile of stage s has been transformed
  uint64_t empty[MAX_STAGES];   // UMMAs reading stage s have finished
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t rinv_full[2];
  uint64_t rinv_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
  float rinv[2][256];
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

__host__ __device__ inline int gemm_threads(int mode) { return mode == MODE_RMSNORM ? 320 : 192; }

template <int CTA_GROUP, int M_SUB, int MODE>
__global__ void __launch_bounds__(MODE == MODE_RMSNORM ? 320 : 192, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_a,
                    const __grid_constant__ CUtensorMap tm_b, const GemmParams p) {
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
  const uint32_t a_bytes = static_cast<uint32_t>(MC) * tile_k * 2u;
  const uint32_t b_bytes = static_cast<uint32_t>(nc) * tile_k * 2u;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_base = smem_base;
  const uint32_t b_base = a_base + stages * a_bytes;
  const uint32_t ctrl_addr = b_base + stages * b_bytes;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem_raw + (ctrl_addr - smem_u32(smem_raw)));

  const int acc_cols = M_SUB * tile_n;
  const int acc_bufs = p.acc_bufs;
  const int num_k_blocks = p.num_k_blocks;
  const int total_tiles = p.num_m_tiles * p.num_n_tiles;
  const int first_tile = static_cast<int>(blockIdx.x) / CTA_GROUP;
  const int tile_stride = static_cast<int>(gridDim.x) / CTA_GROUP;

  // ------------------------------------------------------------------ set-up
  if (threadIdx.x == 0) {
    ctrl->abort_flag = 0;
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->full_a[s]), 1);
      mbar_init(smem_u32(&ctrl->ready[s]), 4 * CTA_GROUP);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctrl->acc_full[b]), 1);
      mbar_init(smem_u32(&ctrl->acc_empty[b]), 4 * CTA_GROUP);
      mbar_init(smem_u32(&ctrl->rinv_full[b]), 4);
      mbar_init(smem_u32(&ctrl->rinv_empty[b]), 4);
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

  // ------------------------------------------------------------------ TMA producer
  if (warp == 0) {
    if (lane == 0 && !p.debug_skip_producer) {
      wctx.role = ROLE_PRODUCER;
      uint32_t it = 0;
      bool ok = true;
      for (int tile = first_tile; tile < total_tiles && ok; tile += tile_stride) {
        int mt, nt;
        tile_coords(tile, p.num_m_tiles, p.num_n_tiles, p.group_m, mt, nt);
        const int m_base = (mt * CTA_GROUP + static_cast<int>(cta_rank)) * MC;
        const int n_base = nt * tile_n + static_cast<int>(cta_rank) * nc;
        for (int kb = 0; kb < num_k_blocks; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1u;
          ok = bounded_wait<PAIR>(wctx, smem_u32(&ctrl->empty[s]), ph ^ 1u, 100 + s, tile, kb);
          if (!ok) break;
          const uint32_t a_s = a_base + s * a_bytes;
          const uint32_t b_s = b_base + s * b_bytes;
          const int k0 = kb * tile_k;
          const uint32_t full_local = smem_u32(&ctrl->full[s]);
          if constexpr (MODE == MODE_LHST) {
            if constexpr (PAIR) {
              const uint32_t full_leader = map_to_cta(full_local, 0);
              if (cta_rank == 0) mbar_arrive_expect_tx(full_local, 2u * (a_bytes + b_bytes));
              for (int c = 0; c < MC / 64; ++c)
                tma_load_2d_pair(a_s + c * tile_k * 128, &tm_a, full_leader, m_base + 64 * c, k0);
              for (int c = 0; c < nc / 64; ++c)
                tma_load_2d_pair(b_s + c * tile_k * 128, &tm_b, full_leader, n_base + 64 * c, k0);
            } else {
              mbar_arrive_expect_tx(full_local, a_bytes + b_bytes);
              for (int c = 0; c < MC / 64; ++c)
                tma_load_2d(a_s + c * tile_k * 128, &tm_a, full_local, m_base + 64 * c, k0);
              for (int c = 0; c < nc / 64; ++c)
                tma_load_2d(b_s + c * tile_k * 128, &tm_b, full_local, n_base + 64 * c, k0);
            }
          } else {
            // x tile completes on this CTA's own barrier (its transform warps wait there);
            // w tile completes on the pair leader's barrier (the UMMA issuer waits there)
            const uint32_t fa = smem_u32(&ctrl->full_a[s]);
            mbar_arrive_expect_tx(fa, a_bytes);
            for (int c = 0; c < tile_k / 64; ++c)
              tma_load_2d(a_s + c * MC * 128, &tm_a, fa, k0 + 64 * c, m_base);
            if constexpr (PAIR) {
              const uint32_t full_leader = map_to_cta(full_local, 0);
              if (cta_rank == 0) mbar_arrive_expect_tx(full_local, 2u * b_bytes);
              for (int c = 0; c < nc / 64; ++c)
                tma_load_2d_pair(b_s + c * tile_k * 128, &tm_b, full_leader, n_base + 64 * c, k0);
            } else {
              mbar_arrive_expect_tx(full_local, b_bytes);
              for (int c = 0; c < nc / 64; ++c)
                tma_load_2d(b_s + c * tile_k * 128, &tm_b, full_local, n_base + 64 * c, k0);
            }
          }
        }
      }
      // tail: every stage released, so no UMMA-completion arrival is still on its way to
      // this CTA's barriers when the CTA exits
      for (int i = 0; i < stages && ok; ++i, ++it) {
        const int s = it % stages;
        const uint32_t ph = (it / stages) & 1u;
        ok = bounded_wait<PAIR>(wctx, smem_u32(&ctrl->empty[s]), ph ^ 1u, 150 + s, -1, i);
      }
    }
    __syncwarp();
  }
  // ------------------------------------------------------------------ UMMA issuer
  else if (warp == 1) {
    if (lane == 0 && cta_rank == 0) {
      wctx.role = ROLE_MMA;
      const uint32_t idesc =
          make_idesc_bf16_f32(128 * CTA_GROUP, tile_n, MODE == MODE_LHST ? 1 : 0, 1);
      const uint32_t mn_lbo = static_cast<uint32_t>(tile_k) * 128u;
      uint32_t it = 0;
      int t = 0;
      bool ok = true;
      for (int tile = first_tile; tile < total_tiles && ok; tile += tile_stride, ++t) {
        const int b = t % acc_bufs;
        const uint32_t aph = (t / acc_bufs) & 1u;
        ok = bounded_wait<PAIR>(wctx, smem_u32(&ctrl->acc_empty[b]), aph ^ 1u, 200 + b, tile, -1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(b * acc_cols);
        for (int kb = 0; kb < num_k_blocks; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1u;
          ok = bounded_wait<PAIR>(wctx, smem_u32(&ctrl->full[s]), ph, 300 + s, tile, kb);
          if (!ok) break;
          if constexpr (MODE == MODE_RMSNORM) {
            ok = bounded_wait<PAIR>(wctx, smem_u32(&ctrl->ready[s]), ph, 400 + s, tile, kb);
            if (!ok) break;
          }
          tc_fence_after();
          const uint32_t a_s = a_base + s * a_bytes;
          const uint32_t b_s = b_base + s * b_bytes;
          for (int k16 = 0; k16 < tile_k / 16; ++k16) {
            const uint64_t bdesc = make_smem_desc_sw128(b_s + k16 * 2048, mn_lbo, 1024);
#pragma unroll
            for (int mi = 0; mi < M_SUB; ++mi) {
              uint64_t adesc;
              if constexpr (MODE == MODE_LHST)
                adesc = make_smem_desc_sw128(a_s + mi * 2 * mn_lbo + k16 * 2048, mn_lbo, 1024);
              else
                adesc = make_smem_desc_sw128(
                    a_s + (k16 >> 2) * (MC * 128) + mi * (128 * 128) + (k16 & 3) * 32, 16, 1024);
              umma_bf16<CTA_GROUP>(d_tmem + static_cast<uint32_t>(mi * tile_n), adesc, bdesc, idesc,
                                   (kb | k16) != 0 ? 1u : 0u);
            }
          }
          if constexpr (PAIR) umma_commit_pair(smem_u32(&ctrl->empty[s]), 3);
          else umma_commit_1cta(smem_u32(&ctrl->empty[s]));
        }
        if (!ok) break;
        if constexpr (PAIR) umma_commit_pair(smem_u32(&ctrl->acc_full[b]), 3);
        else umma_commit_1cta(smem_u32(&ctrl->acc_full[b]));
      }
    }
    __syncwarp();
  }
  // ------------------------------------------------------------------ epilogue
  else if (warp < 6) {
    wctx.role = ROLE_EPILOGUE;
    const int q = warp & 3;  // tensor-memory lane quadrant this warp may read
    const int row_in_cta = q * 32 + lane;
    const uint32_t acc_empty_leader =
        PAIR ? map_to_cta(smem_u32(&ctrl->acc_empty[0]), 0) : smem_u32(&ctrl->acc_empty[0]);
    int t = 0;
    bool ok = true;
    for (int tile = first_tile; tile < total_tiles && ok; tile += tile_stride, ++t) {
      int mt, nt;
      tile_coords(tile, p.num_m_tiles, p.num_n_tiles, p.group_m, mt, nt);
      const int m_base = (mt * CTA_GROUP + static_cast<int>(cta_rank)) * MC;
      const int n_base = nt * tile_n;
      const int b = t % acc_bufs;
      const uint32_t aph = (t / acc_bufs) & 1u;
      ok = bounded_wait<PAIR>(wctx, smem_u32(&ctrl->acc_full[b]), aph, 500 + b, tile, -1);
      if constexpr (MODE == MODE_RMSNORM) {
        if (ok) ok = bounded_wait<false>(wctx, smem_u32(&ctrl->rinv_full[b]), aph, 600 + b, tile, -1);
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int mi = 0; mi < M_SUB; ++mi) {
        const long long grow = static_cast<long long>(m_base) + mi * 128 + row_in_cta;
        float scale = 1.0f;
        if constexpr (MODE == MODE_RMSNORM) scale = ctrl->rinv[b][mi * 128 + row_in_cta];
        __nv_bfloat16* out_row = p.out + grow * p.ld_out;
        for (int c = 0; c < tile_n / 32; ++c) {
          uint32_t r[32];
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                 static_cast<uint32_t>(b * acc_cols + mi * tile_n + c * 32);
          tmem_ld_32x32b_x32(taddr, r);
          tmem_ld_wait();
          if (grow < p.M) {
            const int col0 = n_base + c * 32;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int col = col0 + g * 8;
              if (col + 8 <= p.N) {
                uint4 v;
                v.x = pack_bf16x2(__uint_as_float(r[g * 8 + 0]) * scale,
                                  __uint_as_float(r[g * 8 + 1]) * scale);
                v.y = pack_bf16x2(__uint_as_float(r[g * 8 + 2]) * scale,
                                  __uint_as_float(r[g * 8 + 3]) * scale);
                v.z = pack_bf16x2(__uint_as_float(r[g * 8 + 4]) * scale,
                                  __uint_as_float(r[g * 8 + 5]) * scale);
                v.w = pack_bf16x2(__uint_as_float(r[g * 8 + 6]) * scale,
                                  __uint_as_float(r[g * 8 + 7]) * scale);
                *reinterpret_cast<uint4*>(out_row + col) = v;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR) mbar_arrive_cluster(acc_empty_leader + b * 8);
        else mbar_arrive(acc_empty_leader + b * 8);
        if constexpr (MODE == MODE_RMSNORM) mbar_arrive(smem_u32(&ctrl->rinv_empty[b]));
      }
    }
  }
  // ------------------------------------------------------------------ fused-norm transform
  else {
    if constexpr (MODE == MODE_RMSNORM) {
      wctx.role = ROLE_TRANSFORM;
      const int row = (warp - 6) * 32 + lane;  // 0..127
      const uint32_t sw = static_cast<uint32_t>(row & 7);
      const bool has_gamma = (p.gamma != nullptr);
      uint32_t it = 0;
      int t = 0;
      bool ok = true;
      for (int tile = first_tile; tile < total_tiles && ok; tile += tile_stride, ++t) {
        float ss[M_SUB];
#pragma unroll
        for (int mi = 0; mi < M_SUB; ++mi) ss[mi] = 0.0f;
        for (int kb = 0; kb < num_k_blocks; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1u;
          ok = bounded_wait<false>(wctx, smem_u32(&ctrl->full_a[s]), ph, 700 + s, tile, kb);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          uint8_t* a_s = smem_raw + (a_base + s * a_bytes - smem_u32(smem_raw));
          for (int c = 0; c < tile_k / 64; ++c) {
            const __nv_bfloat16* gptr = p.gamma + kb * tile_k + c * 64;
#pragma unroll
            for (int mi = 0; mi < M_SUB; ++mi) {
              uint8_t* rowp = a_s + c * (MC * 128) + (mi * 128 + row) * 128;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                uint4* cp = reinterpret_cast<uint4*>(rowp + ((static_cast<uint32_t>(j) ^ sw) << 4));
                uint4 v = *cp;
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
                float2 f0 = __bfloat1622float2(h[0]);
                float2 f1 = __bfloat1622float2(h[1]);
                float2 f2 = __bfloat1622float2(h[2]);
                float2 f3 = __bfloat1622float2(h[3]);
                ss[mi] += f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y + f2.x * f2.x +
                          f2.y * f2.y + f3.x * f3.x + f3.y * f3.y;
                if (has_gamma) {
                  uint4 gv = __ldg(reinterpret_cast<const uint4*>(gptr + j * 8));
                  __nv_bfloat162* gh = reinterpret_cast<__nv_bfloat162*>(&gv);
                  float2 g0 = __bfloat1622float2(gh[0]);
                  float2 g1 = __bfloat1622float2(gh[1]);
                  float2 g2 = __bfloat1622float2(gh[2]);
                  float2 g3 = __bfloat1622float2(gh[3]);
                  uint4 o;
                  o.x = pack_bf16x2(f0.x * g0.x, f0.y * g0.y);
                  o.y = pack_bf16x2(f1.x * g1.x, f1.y * g1.y);
                  o.z = pack_bf16x2(f2.x * g2.x, f2.y * g2.y);
                  o.w = pack_bf16x2(f3.x * g3.x, f3.y * g3.y);
                  *cp = o;
                }
              }
            }
          }
          if (has_gamma) fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if constexpr (PAIR) mbar_arrive_cluster(map_to_cta(smem_u32(&ctrl->ready[s]), 0));
            else mbar_arrive(smem_u32(&ctrl->ready[s]));
          }
        }
        if (!ok) break;
        const int b = t % acc_bufs;
        const uint32_t aph = (t / acc_bufs) & 1u;
        ok = bounded_wait<false>(wctx, smem_u32(&ctrl->rinv_empty[b]), aph ^ 1u, 800 + b, tile, -1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
#pragma unroll
        for (int mi = 0; mi < M_SUB; ++mi)
          ctrl->rinv[b][mi * 128 + row] = rsqrtf(ss[mi] * p.inv_k + p.eps);
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctrl->rinv_full[b]));
      }
    }
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
}

}  // namespace b200
