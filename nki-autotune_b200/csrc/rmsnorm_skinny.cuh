// Fused RMSNorm + matmul for skinny activations (M <= 16 rows, e.g. decode):
//     out[M,N] = (x / rms(x) * gamma)[M,K] . w[K,N]
// The work is streaming w (K*N*2 bytes) once from HBM, so the kernel is built around that:
//
//   * one UMMA per 16 k covers a tile of 256 weight columns: D[128, 256 n] += A[128, 16 k] . B[16 k, 256 n]
//     with B = w tile (MN-major, straight from TMA) and A = the scaled x tile (K-major).  Only
//     rows 0..15 of A exist: the descriptor's row groups beyond them read whatever follows in
//     shared memory, which only pollutes accumulator rows 16..127 -- rows of D are independent
//     and those rows are never read.  Tiles are 256 columns because a k-row of a tile is then 512
//     contiguous, 512-byte-aligned bytes; narrower or unaligned column strips stream at half the rate.
//   * work split over G CTAs (one per SM) for T tiles: every CTA takes floor(T / G) whole tiles over
//     the whole of K (no exchange with anybody).  The R = T mod G tiles left over get one OWNER CTA
//     each; the other G - R CTAs are DONORS.  An owner streams the last k-blocks of its tile, the
//     first `don` k-blocks of every left-over tile are dealt to the donors as one flattened range
//     each.  Donors do their range first and get slightly less work, so every partial tile is in
//     its scratch slot (and counted) before the owners finish streaming; an owner fetches the
//     donors' partials while its own k-blocks are still in flight and ends with drain, add, scale,
//     store, like a CTA that had the tile to itself.  The sum order is fixed (donors in index
//     order, then the owner), so results do not depend on timing.  Donors have the low CTA
//     indices: if the grid is ever not co-resident they run first and no owner waits on a CTA
//     that has not started.
//   * CTAs start their K loops at different k-blocks (and wrap around): CTAs that walk the same
//     k-rows at the same time were measured 15 % slower.
//   * x is tiny (M*K): four warps stage x*gamma tiles into shared memory in the swizzled
//     K-major layout the UMMA reads (loads issued one unit ahead), and every CTA computes
//     rinv[m] for itself from x (L2).
//   * the TMA producer warp initialises the barriers itself and starts loading at once; the
//     other warps join through a named barrier after the tensor-memory allocation.
//   * launched as a programmatic dependent launch: the weights are not produced by the kernel
//     before this one in the stream, so the producer streams them without waiting for it, while
//     every warp that reads x or gamma, touches the scratch or writes out first waits for that
//     kernel to complete.  In a chain of these launches (a decode loop) a CTA's SM is taken by the
//     next launch as soon as the CTA exits, and the next launch's first weight tiles are already
//     in shared memory when the previous launch ends.
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
  int num_k_blocks;
  int base_tiles;               // whole tiles per CTA: tile R + b * base_tiles + i belongs to CTA b
  int lo_tiles;                 // R: left-over tiles 0..R-1, tile t owned by CTA donors + t
  int donors;                   // D = gridDim.x - R when R > 0, else 0: CTAs 0..D-1
  int don;                      // k-blocks 0..don-1 of every left-over tile are streamed by donors
  int rot;                      // CTA b starts its whole-K loops at k-block (b * rot) mod num_k_blocks
  const __nv_bfloat16* x;
  const __nv_bfloat16* gamma;   // may be nullptr
  __nv_bfloat16* out;
  float* partial;               // [R + D][16][256] fp32 partial tiles, written before read
  int* tile_count;              // [R] k-blocks the donors have contributed, all zero between launches
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

__device__ __forceinline__ void skinny_give_up(const SkinnyWait& w, int bar_id, int unit) {
  w.ctrl->abort_flag = 1;
  if (w.status != nullptr && atomicCAS(w.status, 0, 7) == 0) {
    w.status[1] = w.role;
    w.status[2] = bar_id;
    w.status[3] = unit;
    w.status[5] = static_cast<int>(blockIdx.x);
  }
}

__device__ __forceinline__ bool skinny_wait(const SkinnyWait& w, uint32_t bar, uint32_t parity, int bar_id,
                                            int unit) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0u) {
      if (w.ctrl->abort_flag) return false;
      if (clock64() - t0 > w.limit) {
        skinny_give_up(w, bar_id, unit);
        return false;
      }
    }
  }
  return true;
}

enum SkinnyKind { SK_WHOLE = 0, SK_DONATE = 1, SK_OWN = 2 };

// The work of one CTA as a sequence of segments, the same sequence for every role.  A segment is
// a tile and a range of its k-blocks, walked from kb_start upwards with wrap-around.
struct SkinnyWork {
  int nkb, N, b, base, R, D, don, rot;
  long long du, du_end;   // donor: flattened (left-over tile, donated k-block) units still to hand out
  int bt;                 // whole tiles handed out so far
  bool own_pending;       // owner: its left-over tile is still to come
  // current segment
  int kind, tile, n0, width;
  int kb_lo, kb_hi, kb_start;
  int pos;                // unit-by-unit view: position within the segment

  __device__ __forceinline__ SkinnyWork(const SkinnyParams& p) {
    nkb = p.num_k_blocks; N = p.N; b = static_cast<int>(blockIdx.x);
    base = p.base_tiles; R = p.lo_tiles; D = p.donors; don = p.don; rot = p.rot;
    du = du_end = 0;
    if (b < D && don > 0) {
      const long long V = static_cast<long long>(R) * don;
      du = V * b / D;
      du_end = V * (b + 1) / D;
    }
    bt = 0;
    own_pending = (b >= D && b - D < R);
    kind = SK_WHOLE; tile = n0 = width = kb_lo = kb_hi = kb_start = 0;
    pos = 0;
  }
  __device__ __forceinline__ void place(int t) {
    tile = t;
    n0 = t * SKINNY_TILE_N;
    width = min(SKINNY_TILE_N, (N - n0 + 63) & ~63);  // the last chunk may reach past N: the loads fill zeros
    pos = 0;
  }
  __device__ __forceinline__ bool whole_tile() {
    if (bt >= base) return false;
    place(R + b * base + bt);
    kind = SK_WHOLE;
    kb_lo = 0; kb_hi = nkb;
    kb_start = static_cast<int>((static_cast<long long>(b) * rot + 7LL * bt) % nkb);
    ++bt;
    return true;
  }
  __device__ __forceinline__ bool next_segment() {
    if (b < D) {  // donor: its range of the donated k-blocks first, whole tiles after
      if (du < du_end) {
        const int t = static_cast<int>(du / don);
        place(t);
        kind = SK_DONATE;
        kb_lo = static_cast<int>(du - static_cast<long long>(t) * don);
        const long long seg_end = min(du_end, static_cast<long long>(t + 1) * don);
        kb_hi = kb_lo + static_cast<int>(seg_end - du);
        kb_start = kb_lo;
        du = seg_end;
        return true;
      }
      return whole_tile();
    }
    if (whole_tile()) return true;
    if (own_pending) {  // owner: the rest of its left-over tile last
      own_pending = false;
      place(b - D);
      kind = don > 0 ? SK_OWN : SK_WHOLE;
      kb_lo = don; kb_hi = nkb;
      kb_start = don + static_cast<int>((static_cast<long long>(b) * rot) % (nkb - don));
      return true;
    }
    return false;
  }
  __device__ __forceinline__ int len() const { return kb_hi - kb_lo; }
  // k-block at position i of the segment's K loop
  __device__ __forceinline__ int kb_at(int i) const {
    const int k = kb_start + i;
    return k >= kb_hi ? k - (kb_hi - kb_lo) : k;
  }
  // unit-by-unit view of the same sequence (k-block of the next unit)
  __device__ __forceinline__ bool next_unit(int& kb_out) {
    if (pos >= kb_hi - kb_lo && !next_segment()) return false;
    kb_out = kb_at(pos++);
    return true;
  }
};

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

  // ------------------------------------------------------------------ set-up
  // The producer warp initialises the barriers and goes straight to its loads (it needs nothing
  // else); the other nine warps wait for that and for the tensor-memory allocation at a named
  // barrier the producer only arrives at.
  grid_launch_dependents();  // the launch after this one may take SMs as this one's CTAs leave them
  if (warp == 0) {
    if (lane == 0) {
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
      fence_proxy_async_smem();
    }
    __syncwarp();
    asm volatile("bar.arrive 2, %0;" ::"n"(SKINNY_THREADS) : "memory");
  } else {
    if (warp == 1) {
      tmem_alloc<1>(smem_u32(&ctrl->tmem_base), SKINNY_TMEM_COLS);
      tmem_relinquish<1>();
    }
    tc_fence_before();
    asm volatile("bar.sync 2, %0;" ::"n"(SKINNY_THREADS) : "memory");
    tc_fence_after();
  }
  SkinnyWait wctx{ctrl, p.status, p.timeout_cycles, 0};
#ifdef B200_MEASURE_HOOKS
  // measurement build only: per-CTA globaltimer stamps in the last partial-tile slot of the scratch
  // ([0] entry, [2] first weight tile landed, [3] last accumulator committed, [4] seen by the
  // epilogue, [5] epilogue done, [6] donors' partials fetched, [7] rinv done)
  unsigned long long* trace = reinterpret_cast<unsigned long long*>(p.partial + static_cast<size_t>((p.N + 255) / 256 + SKINNY_MAX_CTAS - 1) * SKINNY_SLOT_FLOATS) + blockIdx.x * 8;
  if (threadIdx.x == 0) trace[0] = global_timer_ns();
  if (threadIdx.x == 32) trace[1] = global_timer_ns();
#endif

  // ------------------------------------------------------------------ TMA producer (w tiles)
  // producer and issuer loops run with all lanes converged; one elected lane issues each copy,
  // UMMA and commit (loop state and descriptors stay in uniform registers)
  if (warp == 0) {
    {
      wctx.role = ROLE_PRODUCER;
      Ring ring;
      bool ok = true;
      int unit = 0;
      SkinnyWork work(p);
      while (ok && work.next_segment()) {
        const int chunks = work.width / 64;
        const uint32_t seg_bytes = static_cast<uint32_t>(work.width) * tile_k * 2u;
        const int len = work.len();
        for (int i = 0; i < len; ++i, ++unit, ring.advance(stages)) {
          ok = skinny_wait(wctx, smem_u32(&ctrl->empty[ring.s]), ring.ph ^ 1u, 100 + ring.s, unit);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          const uint32_t w_s = w_base + ring.s * w_bytes;
          const uint32_t fw = smem_u32(&ctrl->full_w[ring.s]);
          const int k0 = work.kb_at(i) * tile_k;
          if (!B200_CHECK(k0 >= 0 && k0 < p.K && work.n0 >= 0 && work.n0 < p.N, CHK_SCHEDULE, k0, work.n0)) { ok = false; break; }
          mbar_arrive_expect_tx_elect(fw, seg_bytes);
          for (int c = 0; c < chunks; ++c)
            tma_load_2d_elect(w_s + c * tile_k * 128, &tm_w, fw, work.n0 + 64 * c, k0);
        }
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
      const uint32_t tmem_base = ctrl->tmem_base;
      const uint32_t mn_lbo = static_cast<uint32_t>(tile_k) * 128u;
      const uint64_t b_desc0 = make_smem_desc_sw128(w_base, mn_lbo, 1024);
      const int nk16 = tile_k / 16;
      Ring ring, acc;
      bool ok = true;
      int unit = 0;
      SkinnyWork work(p);
      while (ok && work.next_segment()) {
        const uint32_t idesc = make_idesc_bf16_f32(128, work.width, 0, 1);  // A K-major, B MN-major
        ok = skinny_wait(wctx, smem_u32(&ctrl->acc_empty[acc.s]), acc.ph ^ 1u, 200 + acc.s, unit);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc.s * SKINNY_TILE_N;
        bool first = true;
        const int len = work.len();
        for (int i = 0; i < len; ++i, ++unit, ring.advance(stages)) {
          const uint32_t s = ring.s;
          ok = skinny_wait(wctx, smem_u32(&ctrl->full_w[s]), ring.ph, 300 + s, unit);
          ok = __all_sync(0xffffffffu, ok);
          if (ok) ok = skinny_wait(wctx, smem_u32(&ctrl->full_x[s]), ring.ph, 400 + s, unit);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
#ifdef B200_MEASURE_HOOKS
          if (lane == 0 && unit == 0) trace[2] = global_timer_ns();
#endif
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
#ifdef B200_MEASURE_HOOKS
        if (lane == 0) trace[3] = global_timer_ns();
#endif
      }
    }
    __syncwarp();
  }
  // ------------------------------------------------------------------ epilogue warps
  else if (warp < 6) {
    wctx.role = ROLE_EPILOGUE;
    const uint32_t tmem_base = ctrl->tmem_base;
    const int q = warp & 3;          // tensor-memory lane quadrant
    const int et = (warp - 2) * 32 + lane;  // 0..127
    grid_dependency_wait();  // x, the scratch and out may belong to the kernel before this one
    // rinv[m] for every row, from x itself: 8 threads per row, 16-byte loads, shuffle reduction
    {
      const int row = et >> 3, part = et & 7;
      float ss = 0.0f, ss2 = 0.0f;
      if (row < p.M) {
        const int per = p.K / 8;  // K is a multiple of 64
        const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<long long>(row) * p.K + part * per);
        for (int i0 = 0; i0 < per / 8; i0 += 32) {  // 32 independent 16-byte loads in flight
          uint4 v16[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v16[i] = (i0 + i < per / 8) ? __ldg(src + i0 + i) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const uint32_t w4[4] = {v16[i].x, v16[i].y, v16[i].z, v16[i].w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              const float lo = __uint_as_float(w4[w] << 16), hi = __uint_as_float(w4[w] & 0xffff0000u);
              ss = fmaf(lo, lo, ss);
              ss2 = fmaf(hi, hi, ss2);
            }
          }
        }
      }
      ss += ss2;
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      ss += __shfl_xor_sync(0xffffffffu, ss, 4);
      if (part == 0) ctrl->rinv[row] = (row < p.M) ? rsqrtf(ss * p.inv_k + p.eps) : 0.0f;
      // the four epilogue warps meet here once, before any bounded wait (no early exit possible)
      asm volatile("bar.sync 1, 128;" ::: "memory");
#ifdef B200_MEASURE_HOOKS
      if (et == 0) trace[7] = global_timer_ns();
#endif
    }
    // Accumulator rows 0..15 (tensor-memory lanes 0..15) hold the result and only the warp that owns
    // lane quadrant 0 can read them, so it alone drains them, to a staging tile in shared memory
    // (lane m holds out[m, n0 .. n0 + width): stores straight from that layout would put 16
    // different rows into every instruction).  Everything row-wise -- fetching the donors'
    // partials, publishing a partial, scaling and storing the result, 512 bytes per instruction
    // -- is shared by the four warps, four rows each.  The warps meet at named barrier 1; the
    // other three never wait on anything else, and every exit from the loop is taken by all four
    // right after a barrier.
    static_assert(SKINNY_TILE_N == 256 && SKINNY_ROWS == 16, "row-wise passes cover 2 x 128 columns, 4 x 4 rows");
    auto epi_sync = []() { asm volatile("bar.sync 1, 128;" ::: "memory"); };
    const int r0 = q * 4;  // first of this warp's rows in the row-wise passes
    Ring acc;
    int unit = 0;
    SkinnyWork work(p);
    while (work.next_segment()) {
      const int nt = work.tile;
      const int kind = work.kind;
      const int width = work.width;
      const int n0 = work.n0;
      // columns of the tile this lane touches in the row-wise passes: j * 128 + lane * 4, j = 0, 1
      const bool col_ok[2] = {lane * 4 < width, 128 + lane * 4 < width};
      if (kind == SK_OWN) {
        // The donors' partials are on their way (or there already) while this CTA's own k-blocks
        // stream.  Wait for the count (bounded like every wait), then their sum, in donor order,
        // goes to the staging tile.
        if (q == 0) {
          const long long t0 = clock64();
          for (;;) {
            int seen = 0;
            if (lane == 0) seen = ld_acquire_gpu(p.tile_count + nt);
            seen = __shfl_sync(0xffffffffu, seen, 0);
            if (seen == p.don || ctrl->abort_flag) break;
            if (clock64() - t0 > wctx.limit) { skinny_give_up(wctx, 600, nt); break; }
            __nanosleep(200);
          }
        }
        epi_sync();
        if (ctrl->abort_flag) break;
        __threadfence();  // the donors' partials are visible from here on
        const long long V = static_cast<long long>(p.lo_tiles) * p.don;
        const int d_lo = static_cast<int>(((static_cast<long long>(nt) * p.don + 1) * p.donors - 1) / V);
        const int d_hi = static_cast<int>(((static_cast<long long>(nt + 1) * p.don) * p.donors - 1) / V);
        float4 v[4][2];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int j = 0; j < 2; ++j) v[r][j] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int d = d_lo; d <= d_hi; ++d) {
          if (V * d / p.donors == V * (d + 1) / p.donors) continue;  // a donor without units
          if (!B200_CHECK(d >= 0 && d < p.donors && nt < (p.N + 255) / 256, CHK_GLOBAL, d, nt)) continue;
          const float* other = p.partial + static_cast<size_t>(d + nt) * SKINNY_SLOT_FLOATS;
          float4 t[4][2];  // 8 independent 16-byte loads in flight per lane
#pragma unroll
          for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int j = 0; j < 2; ++j)
              t[r][j] = col_ok[j] ? __ldcg(reinterpret_cast<const float4*>(other + (r0 + r) * SKINNY_TILE_N + j * 128 + lane * 4))
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              v[r][j].x += t[r][j].x; v[r][j].y += t[r][j].y; v[r][j].z += t[r][j].z; v[r][j].w += t[r][j].w;
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int j = 0; j < 2; ++j)
            *reinterpret_cast<float4*>(&ctrl->tile_s[r0 + r][j * 128 + lane * 4]) = v[r][j];
        if (et == 0) p.tile_count[nt] = 0;  // zero again for the next launch
        epi_sync();
#ifdef B200_MEASURE_HOOKS
        if (et == 0) trace[6] = global_timer_ns();
#endif
      }
      if (q == 0) {
        bool ok = skinny_wait(wctx, smem_u32(&ctrl->acc_full[acc.s]), acc.ph, 500 + acc.s, unit);
        ok = __all_sync(0xffffffffu, ok);
#ifdef B200_MEASURE_HOOKS
        if (lane == 0) trace[4] = global_timer_ns();
#endif
        if (ok) {
          tc_fence_after();
          // the accumulator goes to the staging tile (an owner adds it to the donors' sum that is
          // already there), which also frees it early for the issuer
          for (int c = 0; c < width / 32; ++c) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(tmem_base + acc.s * SKINNY_TILE_N + c * 32, v);
            tmem_ld_wait();
            if (lane < SKINNY_ROWS) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4* dst = reinterpret_cast<float4*>(&ctrl->tile_s[lane][c * 32 + j * 4]);
                float4 a = make_float4(__uint_as_float(v[j * 4]), __uint_as_float(v[j * 4 + 1]),
                                       __uint_as_float(v[j * 4 + 2]), __uint_as_float(v[j * 4 + 3]));
                if (kind == SK_OWN) {
                  const float4 o = *dst;
                  a.x += o.x; a.y += o.y; a.z += o.z; a.w += o.w;
                }
                *dst = a;
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ctrl->acc_empty[acc.s]));
        }
      }
      unit += work.len();
      epi_sync();
      if (ctrl->abort_flag) break;
      if (kind == SK_DONATE) {
        // publish the partial tile (slot index = donor index + tile index, unique along the chain of
        // donated ranges), then add the k-blocks to the tile's counter
        if (!B200_CHECK(static_cast<int>(blockIdx.x) < p.donors && nt < (p.N + 255) / 256, CHK_GLOBAL, blockIdx.x, nt)) break;
        float* const slot = p.partial + static_cast<size_t>(blockIdx.x + nt) * SKINNY_SLOT_FLOATS;
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int j = 0; j < 2; ++j)
            if (col_ok[j])
              __stcg(reinterpret_cast<float4*>(slot + (r0 + r) * SKINNY_TILE_N + j * 128 + lane * 4),
                     *reinterpret_cast<const float4*>(&ctrl->tile_s[r0 + r][j * 128 + lane * 4]));
        __threadfence();
        epi_sync();
        if (et == 0) {
          __threadfence();
          atomicAdd(p.tile_count + nt, work.len());
        }
      } else {
        // scale by rinv[m], round, store
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int m = r0 + r, nn = n0 + j * 128 + lane * 4;
            if (m < p.M && col_ok[j] && nn < p.N) {  // N is a multiple of 8: a group of four columns never straddles N
              const float4 v = *reinterpret_cast<const float4*>(&ctrl->tile_s[m][j * 128 + lane * 4]);
              const float ri = ctrl->rinv[m];
              uint2 o;
              o.x = pack_bf16x2(v.x * ri, v.y * ri);
              o.y = pack_bf16x2(v.z * ri, v.w * ri);
              *reinterpret_cast<uint2*>(p.out + static_cast<long long>(m) * p.N + nn) = o;
            }
          }
        epi_sync();  // the next segment's passes overwrite the staging tile
      }
      acc.advance(SKINNY_ACC_BUFS);
#ifdef B200_MEASURE_HOOKS
      if (et == 0) trace[5] = global_timer_ns();
#endif
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
    // x and gamma pieces of k-block kb; loads are issued one unit ahead of their use so that the
    // L2 latency overlaps the previous stage instead of adding to every stage
    auto load_unit = [&](int kb, uint4 (&xv)[2], uint4 (&gv)[2]) {
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
    grid_dependency_wait();  // x and gamma may be produced by the kernel before this one
    SkinnyWork work(p);
    int kb_next = 0;
    bool have = work.next_unit(kb_next);
    if (have) load_unit(kb_next, cur_x, cur_g);
    Ring ring;
    bool ok = true;
    for (int unit = 0; have && ok; ++unit, ring.advance(stages)) {
      const bool more = work.next_unit(kb_next);
      if (more) load_unit(kb_next, nxt_x, nxt_g);
      ok = skinny_wait(wctx, smem_u32(&ctrl->empty[ring.s]), ring.ph ^ 1u, 700 + ring.s, unit);
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
      have = more;
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
    tmem_dealloc<1>(ctrl->tmem_base, SKINNY_TMEM_COLS);
  }
}

}  // namespace b200
