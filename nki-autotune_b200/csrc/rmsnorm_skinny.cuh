// Fused RMSNorm + matmul for skinny activations (M <= 16 rows, e.g. decode):
//     out[M,N] = (x / rms(x) * gamma)[M,K] . w[K,N]
// The work is streaming w (K*N*2 bytes) once from HBM, so the kernel is built around that:
//
//   * one UMMA per 16 k covers 256 weight columns: D[128, 256 n] += A[128, 16 k] . B[16 k, 256 n]
//     with B = w tile (MN-major, straight from TMA) and A = the scaled x tile (K-major).  Only
//     rows 0..15 of A exist: the descriptor's row groups beyond them read whatever follows in
//     shared memory, which only pollutes accumulator rows 16..127 -- rows of D are independent
//     and those rows are never read.
//   * stream-K: the (n-tile, k-block) units are flattened and cut into one contiguous range per
//     CTA, so all SMs stream equal amounts of w whatever N/256 is.  A CTA that covers only part
//     of a tile's K publishes its fp32 partial tile in a scratch slot of its own and adds its
//     k-blocks to the tile's counter; the contributor that completes the count (or finds it
//     complete but for its own share, in which case it publishes nothing) sums the partials in
//     CTA order, scales by rinv[m], writes bf16 and resets the counter.
//   * x is tiny (M*K): four warps stage x*gamma tiles into shared memory in the swizzled
//     K-major layout the UMMA reads (loads issued one unit ahead), and every CTA computes
//     rinv[m] for itself from x (L2).
//
// Same maths as kernel_library/rmsnorm_matmul/kernel_hand_online.py:5-17 (plus gamma); the
// per-row factor is applied after the K sum.  All waits are bounded (see gemm_tcgen05.cuh).
#pragma once
#include "gemm_tcgen05.cuh"

namespace b200 {

constexpr int SKINNY_ROWS = 16;       // activation rows per launch (rows 0..15 of the UMMA M side)
constexpr int SKINNY_TILE_N = 256;    // weight columns per tile (UMMA N): 512 contiguous bytes per k-row
constexpr int SKINNY_ACC_BUFS = 2;    // 256-column accumulators in tensor memory
constexpr int SKINNY_TMEM_COLS = SKINNY_ACC_BUFS * SKINNY_TILE_N;
constexpr int SKINNY_THREADS = 32 * 10;
constexpr int SKINNY_MAX_CTAS = 160;  // grid cap: bounds the number of partial-tile slots in the scratch
constexpr int SKINNY_SLOT_FLOATS = SKINNY_ROWS * SKINNY_TILE_N;  // one partial tile, [16][256] fp32

struct SkinnyParams {
  int M, N, K;
  int tile_k, stages;
  int num_n_tiles, num_k_blocks;
  const __nv_bfloat16* x;
  const __nv_bfloat16* gamma;   // may be nullptr
  __nv_bfloat16* out;
  float* partial;               // [num_n_tiles + gridDim.x][16][256] fp32 partial tiles, written before read
  int* tile_count;              // [num_n_tiles] k-blocks contributed so far, all zero between launches
  float eps, inv_k;
  int* status;
  long long timeout_cycles;
};

struct alignas(16) SkinnyCtrl {
  uint64_t full_w[MAX_STAGES];   // w tile of stage s has landed
  uint64_t full_x[MAX_STAGES];   // scaled x tile of stage s has been written
  uint64_t empty[MAX_STAGES];    // UMMAs reading stage s have finished
  uint64_t acc_full[SKINNY_ACC_BUFS];
  uint64_t acc_empty[SKINNY_ACC_BUFS];
  uint32_t tmem_base;
  volatile int abort_flag;
  float rinv[SKINNY_ROWS];
  // drain staging: one whole partial tile, 16 rows x 256 fp32 columns, rows padded by 16 bytes so
  // that the row-per-lane writes of the drain and the row-wise reads after it are free of bank
  // conflicts
  alignas(16) float tile_s[SKINNY_ROWS][SKINNY_TILE_N + 4];
};

struct SkinnyWait {
  SkinnyCtrl* ctrl;
  int* status;
  long long limit;
  int role;
};

__device__ __forceinline__ bool skinny_wait(const SkinnyWait& w, uint32_t bar, uint32_t parity, int bar_id,
                                            int unit) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0u) {
      if (w.ctrl->abort_flag) return false;
      if (clock64() - t0 > w.limit) {
        w.ctrl->abort_flag = 1;
        if (w.status != nullptr && atomicCAS(w.status, 0, 7) == 0) {
          w.status[1] = w.role;
          w.status[2] = bar_id;
          w.status[3] = unit;
          w.status[5] = static_cast<int>(blockIdx.x);
        }
        return false;
      }
    }
  }
  return true;
}

__global__ void __launch_bounds__(SKINNY_THREADS, 1)
rmsnorm_skinny_kernel(const __grid_constant__ CUtensorMap tm_w, const SkinnyParams p) {
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tile_k = p.tile_k;
  const int stages = p.stages;
  const uint32_t w_bytes = static_cast<uint32_t>(SKINNY_TILE_N) * tile_k * 2u;
  const uint32_t x_bytes = static_cast<uint32_t>(SKINNY_ROWS) * tile_k * 2u;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // x stages first: the UMMA's reads past row 15 of an x tile then land in the w stages
  const uint32_t x_base = smem_base;
  const uint32_t w_base = x_base + stages * x_bytes;
  const uint32_t ctrl_addr = w_base + stages * w_bytes;
  uint8_t* const smem_gen = smem_raw - smem_u32(smem_raw);
  SkinnyCtrl* ctrl = reinterpret_cast<SkinnyCtrl*>(smem_gen + ctrl_addr);

  // this CTA's contiguous range of (n-tile, k-block) units
  const int nkb = p.num_k_blocks;
  const long long total_units = static_cast<long long>(p.num_n_tiles) * nkb;
  const long long u_begin = total_units * blockIdx.x / gridDim.x;
  const long long u_end = total_units * (blockIdx.x + 1) / gridDim.x;

  if (threadIdx.x == 0) {
    ctrl->abort_flag = 0;
    tma_prefetch_desc(&tm_w);
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&ctrl->full_w[s]), 1);
      mbar_init(smem_u32(&ctrl->full_x[s]), 4);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int b = 0; b < SKINNY_ACC_BUFS; ++b) {
      mbar_init(smem_u32(&ctrl->acc_full[b]), 1);
      mbar_init(smem_u32(&ctrl->acc_empty[b]), 1);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<1>(smem_u32(&ctrl->tmem_base), SKINNY_TMEM_COLS);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;
  SkinnyWait wctx{ctrl, p.status, p.timeout_cycles, 0};

  // ------------------------------------------------------------------ TMA producer (w tiles)
  // producer and issuer loops run with all lanes converged; one elected lane issues each copy,
  // UMMA and commit (loop state and descriptors stay in uniform registers)
  if (warp == 0) {
    {
      wctx.role = ROLE_PRODUCER;
      Ring ring;
      bool ok = true;
      int nt = static_cast<int>(u_begin / nkb);
      int kb = static_cast<int>(u_begin - static_cast<long long>(nt) * nkb);
      for (long long u = u_begin; u < u_end && ok; ++u, ring.advance(stages)) {
        ok = skinny_wait(wctx, smem_u32(&ctrl->empty[ring.s]), ring.ph ^ 1u, 100 + ring.s, static_cast<int>(u - u_begin));
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const uint32_t w_s = w_base + ring.s * w_bytes;
        const uint32_t fw = smem_u32(&ctrl->full_w[ring.s]);
        mbar_arrive_expect_tx_elect(fw, w_bytes);
        for (int c = 0; c < SKINNY_TILE_N / 64; ++c)
          tma_load_2d_elect(w_s + c * tile_k * 128, &tm_w, fw, nt * SKINNY_TILE_N + 64 * c, kb * tile_k);
        if (++kb == nkb) { kb = 0; ++nt; }
      }
      for (int i = 0; i < stages && ok; ++i, ring.advance(stages)) {
        ok = skinny_wait(wctx, smem_u32(&ctrl->empty[ring.s]), ring.ph ^ 1u, 150 + ring.s, -1);
        ok = __all_sync(0xffffffffu, ok);
      }
    }
    __syncwarp();
  }
  // ------------------------------------------------------------------ UMMA issuer
  else if (warp == 1) {
    {
      wctx.role = ROLE_MMA;
      const uint32_t idesc = make_idesc_bf16_f32(128, SKINNY_TILE_N, 0, 1);  // A K-major, B MN-major
      const uint32_t mn_lbo = static_cast<uint32_t>(tile_k) * 128u;
      const uint64_t b_desc0 = make_smem_desc_sw128(w_base, mn_lbo, 1024);
      const int nk16 = tile_k / 16;
      Ring ring, acc;
      bool ok = true;
      long long u = u_begin;
      while (u < u_end && ok) {
        const int nt = static_cast<int>(u / nkb);
        const long long seg_end = min(u_end, static_cast<long long>(nt + 1) * nkb);
        ok = skinny_wait(wctx, smem_u32(&ctrl->acc_empty[acc.s]), acc.ph ^ 1u, 200 + acc.s, static_cast<int>(u - u_begin));
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc.s * SKINNY_TILE_N;
        bool first = true;
        for (; u < seg_end; ++u, ring.advance(stages)) {
          const uint32_t s = ring.s;
          ok = skinny_wait(wctx, smem_u32(&ctrl->full_w[s]), ring.ph, 300 + s, static_cast<int>(u - u_begin));
          ok = __all_sync(0xffffffffu, ok);
          if (ok) ok = skinny_wait(wctx, smem_u32(&ctrl->full_x[s]), ring.ph, 400 + s, static_cast<int>(u - u_begin));
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          uint64_t bdesc = b_desc0 + s * (w_bytes >> 4);
          const uint32_t x_s = x_base + s * x_bytes;
          for (int k16 = 0; k16 < nk16; ++k16, bdesc += 128) {
            const uint64_t adesc =
                make_smem_desc_sw128(x_s + (k16 >> 2) * (SKINNY_ROWS * 128) + (k16 & 3) * 32, 16, 1024);
            umma_bf16_elect<1>(d_tmem, adesc, bdesc, idesc, first ? 0u : 1u);
            first = false;
          }
          umma_commit_1cta_elect(smem_u32(&ctrl->empty[s]));
        }
        if (!ok) break;
        umma_commit_1cta_elect(smem_u32(&ctrl->acc_full[acc.s]));
        acc.advance(SKINNY_ACC_BUFS);

      }
    }
    __syncwarp();
  }
  // ------------------------------------------------------------------ epilogue warps
  else if (warp < 6) {
    wctx.role = ROLE_EPILOGUE;
    const int q = warp & 3;          // tensor-memory lane quadrant
    const int et = (warp - 2) * 32 + lane;  // 0..127
    // rinv[m] for every row, from x itself: 8 threads per row, 16-byte loads, shuffle reduction
    {
      const int row = et >> 3, part = et & 7;
      float ss = 0.0f;
      if (row < p.M) {
        const int per = p.K / 8;  // K is a multiple of 64
        const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<long long>(row) * p.K + part * per);
        for (int i0 = 0; i0 < per / 8; i0 += 8) {  // eight independent 16-byte loads in flight
          uint4 v8[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v8[i] = (i0 + i < per / 8) ? __ldg(src + i0 + i) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t w4[4] = {v8[i].x, v8[i].y, v8[i].z, v8[i].w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              const float lo = __uint_as_float(w4[w] << 16), hi = __uint_as_float(w4[w] & 0xffff0000u);
              ss = fmaf(lo, lo, ss);
              ss = fmaf(hi, hi, ss);
            }
          }
        }
      }
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      ss += __shfl_xor_sync(0xffffffffu, ss, 4);
      if (part == 0) ctrl->rinv[row] = (row < p.M) ? rsqrtf(ss * p.inv_k + p.eps) : 0.0f;
      // the four epilogue warps meet here once, before any bounded wait (no early exit possible)
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    // Accumulator rows 0..15 (tensor-memory lanes 0..15) hold the result; only the warp that owns
    // lane quadrant 0 can read them, so it alone drains: lane m holds out[m, n0 .. n0+255].
    Ring acc;
    bool ok = (q == 0);
    long long u = u_begin;
    while (u < u_end && ok) {
      const int nt = static_cast<int>(u / nkb);
      const long long seg_end = min(u_end, static_cast<long long>(nt + 1) * nkb);
      const int seg_blocks = static_cast<int>(seg_end - u);
      ok = skinny_wait(wctx, smem_u32(&ctrl->acc_full[acc.s]), acc.ph, 500 + acc.s, static_cast<int>(u - u_begin));
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int n0 = nt * SKINNY_TILE_N;
      const bool whole_k = (seg_blocks == nkb);  // this CTA summed the tile's whole K range
      // Lane m holds row m of the accumulator.  Stores straight from that layout would put 16
      // different rows into every instruction, so the tile first goes to shared memory (which also
      // frees the accumulator early); everything after reads it row-wise, 512 bytes per instruction.
      for (int c = 0; c < SKINNY_TILE_N / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + acc.s * SKINNY_TILE_N + c * 32, v);
        tmem_ld_wait();
        if (lane < SKINNY_ROWS) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(&ctrl->tile_s[lane][c * 32 + j * 4]) =
                make_uint4(v[j * 4], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctrl->acc_empty[acc.s]));
      static_assert(SKINNY_TILE_N == 256 && SKINNY_ROWS == 16, "row-wise passes cover 2 x 128 columns, 2 x 8 rows");
      const long long G = gridDim.x;
      bool last = whole_k;
      if (!whole_k) {
        // Contributors publish their partial tile (slot index = CTA index + tile index, unique along
        // the chain of K ranges) and then add their k-blocks to the tile's counter; whoever brings
        // it to nkb sums up.  A contributor that finds all the others already counted is known to
        // be the last without publishing anything: its own partial stays in shared memory.
        int before = 0;
        if (lane == 0) before = ld_acquire_gpu(p.tile_count + nt);
        before = __shfl_sync(0xffffffffu, before, 0);
        last = (before + seg_blocks == nkb);
        if (!last) {
          float* const slot = p.partial + static_cast<size_t>(blockIdx.x + nt) * SKINNY_SLOT_FLOATS;
#pragma unroll
          for (int m = 0; m < SKINNY_ROWS; ++m)
#pragma unroll
            for (int j = 0; j < 2; ++j)
              __stcg(reinterpret_cast<float4*>(slot + m * SKINNY_TILE_N + j * 128 + lane * 4),
                     *reinterpret_cast<const float4*>(&ctrl->tile_s[m][j * 128 + lane * 4]));
          __threadfence();
          __syncwarp();
          int seen = 0;
          if (lane == 0) seen = atomicAdd(p.tile_count + nt, seg_blocks) + seg_blocks;
          seen = __shfl_sync(0xffffffffu, seen, 0);
          last = (seen == nkb);  // the others finished in the meantime
        }
        if (last) __threadfence();  // the other contributors' partials are visible from here on
      }
      if (last) {
        // sum of the contributors' partials in CTA order, whoever does the summing (the result does
        // not depend on which contributor came last): this CTA's from shared memory, the others'
        // from their slots, found from the same partition arithmetic; scale, store, and leave the
        // counter zero for the next launch
        int c_lo = static_cast<int>(blockIdx.x), c_hi = static_cast<int>(blockIdx.x);
        if (!whole_k) {
          c_lo = static_cast<int>(((static_cast<long long>(nt) * nkb + 1) * G - 1) / total_units);
          c_hi = static_cast<int>(((static_cast<long long>(nt + 1) * nkb) * G - 1) / total_units);
        }
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          float4 v[8][2];
#pragma unroll
          for (int r = 0; r < 8; ++r)
#pragma unroll
            for (int j = 0; j < 2; ++j) v[r][j] = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int cc = c_lo; cc <= c_hi; ++cc) {
            if (total_units * cc / G == total_units * (cc + 1) / G) continue;     // a CTA with no units
            const bool mine = (cc == static_cast<int>(blockIdx.x));
            const float* other = p.partial + static_cast<size_t>(cc + nt) * SKINNY_SLOT_FLOATS;
            // 16 independent 16-byte loads in flight per lane (8 rows x 2 column groups)
            float4 t[8][2];
#pragma unroll
            for (int r = 0; r < 8; ++r)
#pragma unroll
              for (int j = 0; j < 2; ++j)
                t[r][j] = mine ? *reinterpret_cast<const float4*>(&ctrl->tile_s[half * 8 + r][j * 128 + lane * 4])
                               : __ldcg(reinterpret_cast<const float4*>(other + (half * 8 + r) * SKINNY_TILE_N + j * 128 + lane * 4));
#pragma unroll
            for (int r = 0; r < 8; ++r)
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                v[r][j].x += t[r][j].x; v[r][j].y += t[r][j].y; v[r][j].z += t[r][j].z; v[r][j].w += t[r][j].w;
              }
          }
#pragma unroll
          for (int r = 0; r < 8; ++r)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const int m = half * 8 + r, nn = n0 + j * 128 + lane * 4;
              if (m < p.M && nn < p.N) {  // N is a multiple of 8: a group of four columns never straddles N
                const float ri = ctrl->rinv[m];
                uint2 o;
                o.x = pack_bf16x2(v[r][j].x * ri, v[r][j].y * ri);
                o.y = pack_bf16x2(v[r][j].z * ri, v[r][j].w * ri);
                *reinterpret_cast<uint2*>(p.out + static_cast<long long>(m) * p.N + nn) = o;
              }
            }
        }
        if (!whole_k && lane == 0) p.tile_count[nt] = 0;
      }
      __syncwarp();  // the next segment's drain overwrites the staging tile
      u = seg_end;
      acc.advance(SKINNY_ACC_BUFS);
    }
  }
  // ------------------------------------------------------------------ x-tile staging warps
  else {
    wctx.role = ROLE_TRANSFORM;
    const int tt = (warp - 6) * 32 + lane;  // 0..127
    const int pieces_per_row = tile_k / 8;  // 16-byte pieces of one row of a stage
    const int pieces = SKINNY_ROWS * pieces_per_row;  // 128 (tile_k 64) or 256 (tile_k 128)
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    const uint4 one4 = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);  // bf16 1.0 pairs
    // x and gamma pieces of unit u; loads are issued one unit ahead of their use so that the
    // L2 latency overlaps the previous stage instead of adding to every stage
    auto load_unit = [&](long long u, uint4 (&xv)[2], uint4 (&gv)[2]) {
      const int nt = static_cast<int>(u / nkb);
      const int kb = static_cast<int>(u - static_cast<long long>(nt) * nkb);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int c = tt + i * 128;
        xv[i] = zero4;
        gv[i] = one4;
        if (c < pieces) {
          const int row = c / pieces_per_row;
          const int k = kb * tile_k + (c - row * pieces_per_row) * 8;
          if (row < p.M && k < p.K) {
            xv[i] = __ldg(reinterpret_cast<const uint4*>(p.x + static_cast<long long>(row) * p.K + k));
            if (p.gamma != nullptr) gv[i] = __ldg(reinterpret_cast<const uint4*>(p.gamma + k));
          }
        }
      }
    };
    uint4 cur_x[2], cur_g[2], nxt_x[2], nxt_g[2];
    if (u_begin < u_end) load_unit(u_begin, cur_x, cur_g);
    Ring ring;
    bool ok = true;
    for (long long u = u_begin; u < u_end && ok; ++u, ring.advance(stages)) {
      if (u + 1 < u_end) load_unit(u + 1, nxt_x, nxt_g);
      ok = skinny_wait(wctx, smem_u32(&ctrl->empty[ring.s]), ring.ph ^ 1u, 700 + ring.s, static_cast<int>(u - u_begin));
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      uint8_t* x_s = smem_gen + x_base + ring.s * x_bytes;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int c = tt + i * 128;
        if (c < pieces) {
          const int row = c / pieces_per_row;
          const int j = c - row * pieces_per_row;   // 16-byte piece along k within the stage
          uint4 o;
          o.x = mul_bf16x2(cur_x[i].x, cur_g[i].x); o.y = mul_bf16x2(cur_x[i].y, cur_g[i].y);
          o.z = mul_bf16x2(cur_x[i].z, cur_g[i].z); o.w = mul_bf16x2(cur_x[i].w, cur_g[i].w);
          // K-major, 128-byte swizzle: 64-wide chunk (j / 8), row, piece (j % 8) xor (row % 8)
          uint8_t* dst = x_s + (j >> 3) * (SKINNY_ROWS * 128) + row * 128 +
                         ((static_cast<uint32_t>(j & 7) ^ static_cast<uint32_t>(row & 7)) << 4);
          *reinterpret_cast<uint4*>(dst) = o;
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctrl->full_x[ring.s]));
#pragma unroll
      for (int i = 0; i < 2; ++i) { cur_x[i] = nxt_x[i]; cur_g[i] = nxt_g[i]; }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (ctrl->abort_flag && threadIdx.x == 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, SKINNY_TMEM_COLS);
  }
}

}  // namespace b200
