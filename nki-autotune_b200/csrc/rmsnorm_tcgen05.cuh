// Fused RMSNorm + matmul for sm_100a:  out[M,N] = (x / rms(x) * gamma)[M,K] . w[K,N]
//
// Replaces rmsnorm_matmul_online (kernel_library/rmsnorm_matmul/kernel_hand_online.py:198-353).
// The per-row factor commutes out of the K sum, so the kernel makes ONE pass over x:
//     out[m,:] = rinv[m] * sum_k (x[m,k] * gamma[k]) * w[k,:],   rinv[m] = rsqrt(mean_k x[m,k]^2 + eps)
// and the running rescale of the reference's online algorithm (:127-136, :165-192) is not needed
// because the whole K reduction stays in fp32 tensor memory.
//
// Data flow per k-block:
//   TMA    : x tile [rows x tile_k] (K-major) and w tile [tile_k x cols] (MN-major) -> shared memory
//   16 transform warps (four groups of four taking k-blocks round-robin, so four x tiles
//            are in flight): read the x tile from shared memory (each thread owns one row), accumulate the row's sum of squares with fp32 FMAs, multiply by gamma
//            (bf16x2 multiply = one rounding, same as fp32 multiply + round), and write the
//            scaled tile into a ring of TENSOR-MEMORY slots with tcgen05.st
//   UMMA   : D[tmem] += A[tmem slot] . B[smem desc]   (A from tensor memory, so the scaled tile
//            never goes back through shared memory and the MMA's shared-memory reads are w only)
//   epilogue warps: tcgen05.ld, multiply row m by rinv[m], bf16, global stores
//
// Barriers (all waits bounded, see bounded_wait in gemm_tcgen05.cuh):
//   full_a[s]  x tile landed (local)          empty_a[s] transform warps done reading it (local)
//   full_b[s]  w tile landed (pair leader)    empty_b[s] UMMAs reading it finished
//   a_ready[t] slot t written (pair leader)   a_free[t]  UMMAs reading slot t finished
//   acc_full/acc_empty[b], ss_full/ss_empty[b] as in the plain GEMM
#pragma once
#include "gemm_tcgen05.cuh"

namespace b200 {

constexpr int MAX_A_SLOTS = 8;
constexpr int RMS_TRANSFORM_GROUPS = 4;  // groups of four warps (one per tensor-memory lane quadrant)
constexpr int RMS_TRANSFORM_WARPS = 4 * RMS_TRANSFORM_GROUPS;
constexpr int RMS_A_PRODUCER_WARP = 6 + RMS_TRANSFORM_WARPS;  // last warp
constexpr int RMS_THREADS = 32 * (7 + RMS_TRANSFORM_WARPS);

struct RmsParams {
  int M, N, K;
  int tile_n, tile_k, stages;
  int num_m_tiles, num_n_tiles, num_k_blocks;
  int group_m;
  int acc_bufs;
  int tmem_cols;
  int a_col0;     // first tensor-memory column of the A ring
  int a_slots;    // ring depth (a multiple of groups)
  int a_stages;   // depth of the shared-memory ring of x tiles (a multiple of groups)
  int groups;     // transform warp groups in use: 1, 2 or 4
  int gamma_bytes;  // bytes of gamma staged in shared memory (0 when gamma is NULL)
  long long ld_out;
  float eps, inv_k;
  __nv_bfloat16* out;
  const __nv_bfloat16* gamma;
  int* status;
  long long timeout_cycles;
  int debug_mode;  // 0, or (measurement builds) DEBUG_NO_MMA / DEBUG_NO_TRANSFORM
};


struct alignas(16) RmsCtrl {
  uint64_t full_a[MAX_STAGES];
  uint64_t full_b[MAX_STAGES];
  uint64_t empty_a[MAX_STAGES];
  uint64_t empty_b[MAX_STAGES];
  uint64_t a_ready[MAX_A_SLOTS];
  uint64_t a_free[MAX_A_SLOTS];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t ss_full[2];
  uint64_t ss_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
  float ss[2][RMS_TRANSFORM_GROUPS][256];  // [accumulator buffer][warp group][row]: partial sums of squares
};

// bounded_wait works on any control block with an abort_flag: thin adapter
struct RmsWait {
  RmsCtrl* ctrl;
  int* status;
  long long limit;
  int role;
};

template <bool CLUSTER_SCOPE>
__device__ __forceinline__ bool rms_wait(const RmsWait& w, uint32_t bar, uint32_t parity, int bar_id,
                                         int tile, int kb) {
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
        if (w.status != nullptr && atomicCAS(w.status, 0, 7) == 0) {
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

template <int CTA_GROUP, int M_SUB>
__global__ void __launch_bounds__(RMS_THREADS, 1)
rmsnorm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_x,
                       const __grid_constant__ CUtensorMap tm_w, const RmsParams p) {
  constexpr bool PAIR = (CTA_GROUP == 2);
  constexpr int MC = 128 * M_SUB;
  extern __shared__ uint8_t smem_raw[];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;

  const int tile_n = p.tile_n;
  const int tile_k = p.tile_k;
  const int stages = p.stages;
  const int a_slots = p.a_slots;
  const int a_stages = p.a_stages;
  const int nc = tile_n / CTA_GROUP;
  const uint32_t a_bytes = static_cast<uint32_t>(MC) * tile_k * 2u;
  const uint32_t b_bytes = static_cast<uint32_t>(nc) * tile_k * 2u;
  const int slot_cols = M_SUB * (tile_k / 2);  // tensor-memory columns of one A slot

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_base = smem_base;
  const uint32_t b_base = a_base + a_stages * a_bytes;
  const uint32_t gamma_addr = b_base + stages * b_bytes;
  const uint32_t ctrl_addr = gamma_addr + ((static_cast<uint32_t>(p.gamma_bytes) + 15u) & ~15u);
  uint8_t* const smem_gen = smem_raw - smem_u32(smem_raw);  // generic pointer for shared address 0
  RmsCtrl* ctrl = reinterpret_cast<RmsCtrl*>(smem_gen + ctrl_addr);

  const int acc_cols = M_SUB * tile_n;
  const int acc_bufs = p.acc_bufs;
  const int num_k_blocks = p.num_k_blocks;
  const int total_tiles = p.num_m_tiles * p.num_n_tiles;
  const int first_tile = static_cast<int>(blockIdx.x) / CTA_GROUP;
  const int tile_stride = static_cast<int>(gridDim.x) / CTA_GROUP;

  // ------------------------------------------------------------------ set-up
  if (threadIdx.x == 0) {
    ctrl->abort_flag = 0;
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_w);
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&ctrl->full_b[s]), 1);
      mbar_init(smem_u32(&ctrl->empty_b[s]), 1);
    }
    for (int s = 0; s < a_stages; ++s) {
      mbar_init(smem_u32(&ctrl->full_a[s]), 1);
      mbar_init(smem_u32(&ctrl->empty_a[s]), 4);
    }
    for (int t = 0; t < a_slots; ++t) {
      mbar_init(smem_u32(&ctrl->a_ready[t]), 4 * CTA_GROUP);
      mbar_init(smem_u32(&ctrl->a_free[t]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctrl->acc_full[b]), 1);
      mbar_init(smem_u32(&ctrl->acc_empty[b]), 4 * CTA_GROUP);
      mbar_init(smem_u32(&ctrl->ss_full[b]), 4 * p.groups);
      mbar_init(smem_u32(&ctrl->ss_empty[b]), 4);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<CTA_GROUP>(smem_u32(&ctrl->tmem_base), static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish<CTA_GROUP>();
  }
  // gamma -> shared memory (read by every transform warp for every tile)
  if (p.gamma_bytes > 0) {
    const uint4* src = reinterpret_cast<const uint4*>(p.gamma);
    uint4* dst = reinterpret_cast<uint4*>(smem_gen + gamma_addr);
    // staged length is K rounded up to whole k-blocks; the tail is zero so that it multiplies the
    // zero-filled x columns beyond K into zeros (never garbage)
    for (int i = threadIdx.x; i < p.gamma_bytes / 16; i += blockDim.x)
      dst[i] = (i * 8 < p.K) ? __ldg(src + i) : make_uint4(0u, 0u, 0u, 0u);
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) {
    cluster_arrive();
    cluster_wait();
  }
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;

  RmsWait wctx{ctrl, p.status, p.timeout_cycles, 0};

  // ------------------------------------------------------------------ TMA producer, w tiles
  // The x and w rings advance independently (separate producer warps, separate barriers), so
  // the transform of later x tiles runs ahead while earlier w tiles are still being consumed.
  // The producer and issuer warps run their loops with all lanes converged; one elected lane
  // issues each copy, UMMA and commit, so loop state and descriptors stay in uniform registers.
  if (warp == 0) {
    {
      wctx.role = ROLE_PRODUCER;
      Ring ring;
      bool ok = true;
      for (int tile = first_tile; tile < total_tiles && ok; tile += tile_stride) {
        int mt, nt;
        tile_coords(tile, p.num_m_tiles, p.num_n_tiles, p.group_m, mt, nt);
        const int n_base = nt * tile_n + static_cast<int>(cta_rank) * nc;
        for (int kb = 0; kb < num_k_blocks; ++kb, ring.advance(stages)) {
          const uint32_t s = ring.s;
          ok = rms_wait<false>(wctx, smem_u32(&ctrl->empty_b[s]), ring.ph ^ 1u, 100 + s, tile, kb);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          const uint32_t b_s = b_base + s * b_bytes;
          const int k0 = kb * tile_k;
          const uint32_t fb = smem_u32(&ctrl->full_b[s]);
          if constexpr (PAIR) {
            const uint32_t fb_leader = map_to_cta(fb, 0);
            if (cta_rank == 0) mbar_arrive_expect_tx_elect(fb, 2u * b_bytes);
            for (int c = 0; c < nc / 64; ++c)
              tma_load_2d_pair_elect(b_s + c * tile_k * 128, &tm_w, fb_leader, n_base + 64 * c, k0);
          } else {
            mbar_arrive_expect_tx_elect(fb, b_bytes);
            for (int c = 0; c < nc / 64; ++c)
              tma_load_2d_elect(b_s + c * tile_k * 128, &tm_w, fb, n_base + 64 * c, k0);
          }
        }
      }
      for (int i = 0; i < stages && ok; ++i, ring.advance(stages)) {  // tail: all stages released
        ok = rms_wait<false>(wctx, smem_u32(&ctrl->empty_b[ring.s]), ring.ph ^ 1u, 150 + ring.s, -1, i);
        ok = __all_sync(0xffffffffu, ok);
      }
    }
    __syncwarp();
  }
  // ------------------------------------------------------------------ TMA producer, x tiles
  else if (warp == RMS_A_PRODUCER_WARP) {
    {
      wctx.role = ROLE_PRODUCER;
      Ring ring;
      bool ok = true;
      for (int tile = first_tile; tile < total_tiles && ok; tile += tile_stride) {
        int mt, nt;
        tile_coords(tile, p.num_m_tiles, p.num_n_tiles, p.group_m, mt, nt);
        const int m_base = (mt * CTA_GROUP + static_cast<int>(cta_rank)) * MC;
        for (int kb = 0; kb < num_k_blocks; ++kb, ring.advance(a_stages)) {
          const uint32_t s = ring.s;
          ok = rms_wait<false>(wctx, smem_u32(&ctrl->empty_a[s]), ring.ph ^ 1u, 120 + s, tile, kb);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          const uint32_t a_s = a_base + s * a_bytes;
          const int k0 = kb * tile_k;
          const uint32_t fa = smem_u32(&ctrl->full_a[s]);
          mbar_arrive_expect_tx_elect(fa, a_bytes);
          for (int c = 0; c < tile_k / 64; ++c)
            tma_load_2d_elect(a_s + c * MC * 128, &tm_x, fa, k0 + 64 * c, m_base);
        }
      }
      for (int i = 0; i < a_stages && ok; ++i, ring.advance(a_stages)) {
        ok = rms_wait<false>(wctx, smem_u32(&ctrl->empty_a[ring.s]), ring.ph ^ 1u, 170 + ring.s, -1, i);
        ok = __all_sync(0xffffffffu, ok);
      }
    }
    __syncwarp();
  }
  // ------------------------------------------------------------------ UMMA issuer
  else if (warp == 1) {
    if (cta_rank == 0) {
      wctx.role = ROLE_MMA;
      const uint32_t idesc = make_idesc_bf16_f32(128 * CTA_GROUP, tile_n, 0, 1);
      const uint32_t mn_lbo = static_cast<uint32_t>(tile_k) * 128u;
      const uint64_t b_desc0 = make_smem_desc_sw128(b_base, mn_lbo, 1024);
      const uint32_t b_step = b_bytes >> 4;
      const int nk16 = tile_k / 16;
      Ring ring, slot, acc;
      bool ok = true;
      for (int tile = first_tile; tile < total_tiles && ok; tile += tile_stride, acc.advance(acc_bufs)) {
        const uint32_t b = acc.s;
        ok = rms_wait<false>(wctx, smem_u32(&ctrl->acc_empty[b]), acc.ph ^ 1u, 200 + b, tile, -1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + b * static_cast<uint32_t>(acc_cols);
        for (int kb = 0; kb < num_k_blocks; ++kb, ring.advance(stages), slot.advance(a_slots)) {
          const uint32_t s = ring.s;
          const uint32_t ta = slot.s;
          ok = rms_wait<false>(wctx, smem_u32(&ctrl->full_b[s]), ring.ph, 300 + s, tile, kb);
          ok = __all_sync(0xffffffffu, ok);
          if (ok) ok = rms_wait<false>(wctx, smem_u32(&ctrl->a_ready[ta]), slot.ph, 400 + ta, tile, kb);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          uint64_t bdesc = b_desc0 + s * b_step;
          uint32_t a_tmem = tmem_base + static_cast<uint32_t>(p.a_col0) + ta * static_cast<uint32_t>(slot_cols);
#pragma unroll 4
          for (int k16 = 0; k16 < nk16; ++k16, bdesc += 128, a_tmem += 8) {
#pragma unroll
            for (int mi = 0; mi < M_SUB; ++mi)
#ifdef B200_MEASURE_HOOKS
              if (p.debug_mode != DEBUG_NO_MMA)
#endif
                umma_bf16_ts_elect<CTA_GROUP>(d_tmem + static_cast<uint32_t>(mi * tile_n),
                                      a_tmem + static_cast<uint32_t>(mi * (tile_k / 2)), bdesc, idesc,
                                      (kb | k16) != 0 ? 1u : 0u);
          }
          if constexpr (PAIR) {
            umma_commit_pair_elect(smem_u32(&ctrl->empty_b[s]), 3);
            umma_commit_pair_elect(smem_u32(&ctrl->a_free[ta]), 3);
          } else {
            umma_commit_1cta_elect(smem_u32(&ctrl->empty_b[s]));
            umma_commit_1cta_elect(smem_u32(&ctrl->a_free[ta]));
          }
        }
        if (!ok) break;
        if constexpr (PAIR) umma_commit_pair_elect(smem_u32(&ctrl->acc_full[b]), 3);
        else umma_commit_1cta_elect(smem_u32(&ctrl->acc_full[b]));
      }
    }
    __syncwarp();
  }
  // ------------------------------------------------------------------ epilogue
  else if (warp < 6) {
    wctx.role = ROLE_EPILOGUE;
    const int q = warp & 3;
    const int row_in_cta = q * 32 + lane;
    const uint32_t acc_empty_leader =
        PAIR ? map_to_cta(smem_u32(&ctrl->acc_empty[0]), 0) : smem_u32(&ctrl->acc_empty[0]);
    Ring acc;
    bool ok = true;
    for (int tile = first_tile; tile < total_tiles && ok; tile += tile_stride, acc.advance(acc_bufs)) {
      int mt, nt;
      tile_coords(tile, p.num_m_tiles, p.num_n_tiles, p.group_m, mt, nt);
      const int m_base = (mt * CTA_GROUP + static_cast<int>(cta_rank)) * MC;
      const int n_base = nt * tile_n;
      const int b = static_cast<int>(acc.s);
      const uint32_t aph = acc.ph;
      ok = rms_wait<false>(wctx, smem_u32(&ctrl->acc_full[b]), aph, 500 + b, tile, -1);
      if (ok) ok = rms_wait<false>(wctx, smem_u32(&ctrl->ss_full[b]), aph, 600 + b, tile, -1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int mi = 0; mi < M_SUB; ++mi) {
        const int r = mi * 128 + row_in_cta;
        const long long grow = static_cast<long long>(m_base) + r;
        float sumsq = 0.0f;
#pragma unroll
        for (int gidx = 0; gidx < RMS_TRANSFORM_GROUPS; ++gidx)
          if (gidx < p.groups) sumsq += ctrl->ss[b][gidx][r];
        const float scale = rsqrtf(sumsq * p.inv_k + p.eps);
        __nv_bfloat16* out_row = p.out + grow * p.ld_out;
        for (int c = 0; c < tile_n / 32; ++c) {
          uint32_t v[32];
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                 static_cast<uint32_t>(b * acc_cols + mi * tile_n + c * 32);
          tmem_ld_32x32b_x32(taddr, v);
          tmem_ld_wait();
          if (grow < p.M) {
            const int col0 = n_base + c * 32;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int col = col0 + g * 8;
              if (col + 8 <= p.N) {
                uint4 o;
                o.x = pack_bf16x2(__uint_as_float(v[g * 8 + 0]) * scale, __uint_as_float(v[g * 8 + 1]) * scale);
                o.y = pack_bf16x2(__uint_as_float(v[g * 8 + 2]) * scale, __uint_as_float(v[g * 8 + 3]) * scale);
                o.z = pack_bf16x2(__uint_as_float(v[g * 8 + 4]) * scale, __uint_as_float(v[g * 8 + 5]) * scale);
                o.w = pack_bf16x2(__uint_as_float(v[g * 8 + 6]) * scale, __uint_as_float(v[g * 8 + 7]) * scale);
                *reinterpret_cast<uint4*>(out_row + col) = o;
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
        mbar_arrive(smem_u32(&ctrl->ss_empty[b]));
      }
    }
  }
  // ------------------------------------------------------------------ transform warps
  else {
    wctx.role = ROLE_TRANSFORM;
    const int q = warp & 3;                 // tensor-memory lane quadrant of this warp
    const int group = (warp - 6) >> 2;      // groups of four warps take k-blocks round-robin
    const int row = q * 32 + lane;          // row within a 128-row block
    const uint32_t sw = static_cast<uint32_t>(row & 7);
    const bool has_gamma = p.gamma_bytes > 0;
    const uint8_t* gamma_s = smem_gen + gamma_addr;
    const uint32_t a_ready_leader_base =
        PAIR ? map_to_cta(smem_u32(&ctrl->a_ready[0]), 0) : smem_u32(&ctrl->a_ready[0]);
    uint32_t it = 0;
    Ring ring, slot, acc;
    bool ok = true;
    const int groups = p.groups;
    if (group >= groups) ok = false;  // this group is not used by the current configuration
    for (int tile = first_tile; tile < total_tiles && ok; tile += tile_stride, acc.advance(acc_bufs)) {
      float ss[M_SUB];
#pragma unroll
      for (int mi = 0; mi < M_SUB; ++mi) ss[mi] = 0.0f;
      for (int kb = 0; kb < num_k_blocks; ++kb, ++it, ring.advance(a_stages), slot.advance(a_slots)) {
        // Round-robin over the groups.  Both ring depths are multiples of `groups`, so a given
        // stage and a given slot are always served by the same group, in order: a group never
        // waits on a barrier that is more than one phase behind (parity waits would alias).
        if (static_cast<int>(it % static_cast<uint32_t>(groups)) != group) continue;
        const uint32_t s = ring.s;
        const uint32_t ph = ring.ph;
        const uint32_t ta = slot.s;
        const uint32_t tph = slot.ph;
        ok = rms_wait<false>(wctx, smem_u32(&ctrl->full_a[s]), ph, 700 + s, tile, kb);
        if (ok) ok = rms_wait<false>(wctx, smem_u32(&ctrl->a_free[ta]), tph ^ 1u, 720 + ta, tile, kb);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint8_t* a_s = smem_gen + a_base + s * a_bytes;
        const int k0 = kb * tile_k;
#ifdef B200_MEASURE_HOOKS
        const int n_grp = p.debug_mode == DEBUG_NO_TRANSFORM ? 0 : tile_k / 32;
#else
        const int n_grp = tile_k / 32;
#endif
        for (int grp = 0; grp < n_grp; ++grp) {
          const int e0 = grp * 32;        // first k element (within the stage) of this group of 32
          const int chunk = e0 >> 6;      // 64-wide shared-memory chunk
          const int j0 = (e0 & 63) >> 3;  // first 16-byte piece within the row
          const uint4* g4 = reinterpret_cast<const uint4*>(gamma_s + (k0 + e0) * 2);
#pragma unroll
          for (int mi = 0; mi < M_SUB; ++mi) {
            const uint8_t* rowp = a_s + chunk * (MC * 128) + (mi * 128 + row) * 128;
            uint32_t r[16];
            float acc = ss[mi], acc2 = 0.0f;  // two chains halve the dependent-FMA latency
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              const uint4 v = *reinterpret_cast<const uint4*>(rowp + ((static_cast<uint32_t>(j0 + jj) ^ sw) << 4));
              const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
              uint32_t g[4] = {0, 0, 0, 0};
              if (has_gamma) {
                const uint4 gv = g4[jj];
                g[0] = gv.x; g[1] = gv.y; g[2] = gv.z; g[3] = gv.w;
              }
#pragma unroll
              for (int w = 0; w < 4; ++w) {
                const float lo = __uint_as_float(w4[w] << 16);
                const float hi = __uint_as_float(w4[w] & 0xffff0000u);
                acc = fmaf(lo, lo, acc);
                acc2 = fmaf(hi, hi, acc2);
                r[jj * 4 + w] = has_gamma ? mul_bf16x2(w4[w], g[w]) : w4[w];
              }
            }
            ss[mi] = acc + acc2;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                   static_cast<uint32_t>(p.a_col0 + ta * slot_cols + mi * (tile_k / 2) + (e0 >> 1));
            tmem_st_32x32b_x16(taddr, r);
          }
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&ctrl->empty_a[s]));
          if constexpr (PAIR) mbar_arrive_cluster(a_ready_leader_base + ta * 8);
          else mbar_arrive(a_ready_leader_base + ta * 8);
        }
      }
      if (!ok) break;
      const int b = static_cast<int>(acc.s);
      const uint32_t aph = acc.ph;
      ok = rms_wait<false>(wctx, smem_u32(&ctrl->ss_empty[b]), aph ^ 1u, 800 + b, tile, -1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
#pragma unroll
      for (int mi = 0; mi < M_SUB; ++mi) ctrl->ss[b][group][mi * 128 + row] = ss[mi];
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctrl->ss_full[b]));
    }
    // tail: every slot released, so no UMMA-completion arrival is still on its way to a_free[]
    for (int i = 0; i < a_slots && ok; ++i, slot.advance(a_slots)) {
      ok = rms_wait<false>(wctx, smem_u32(&ctrl->a_free[slot.s]), slot.ph ^ 1u, 750 + slot.s, -1, i);
      ok = __all_sync(0xffffffffu, ok);
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (ctrl->abort_flag && threadIdx.x == 0) {
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
