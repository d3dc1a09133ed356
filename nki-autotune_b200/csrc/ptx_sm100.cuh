// Thin inline-PTX wrappers for the sm_100a features the kernels use: mbarrier, TMA tile
// copies (plain per-CTA form only), tcgen05 (UMMA, tensor memory), cluster addressing.
// Written from the public PTX ISA; one instruction per wrapper.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace b200 {

// ----------------------------------------------------------------------------------
// Checked build (-DB200_CHECKED_BUILD): every wrapper below that takes a shared-memory address,
// a tensor-memory address or TMA coordinates validates them first, and the kernels validate
// their global indices with the same macro.  A failed check records the first offender
// (code, source line, value, limit) in g_check_log, counts the rest, and the access is SKIPPED:
// nothing traps and nothing out of range is touched (a skipped load leaves its consumer to its
// bounded wait).  In the normal build B200_CHECK is the constant true and costs nothing.
// ----------------------------------------------------------------------------------
enum CheckCode : int {
  CHK_SMEM_RANGE = 1,   // shared-memory access outside the CTA's window or misaligned
  CHK_BARRIER = 2,      // mbarrier address outside the window or not 8-byte aligned
  CHK_TMA_LOAD = 3,     // TMA load: destination outside the window / not 128-byte aligned, or x not 16-byte aligned
  CHK_TMA_STORE = 4,    // TMA store: negative coordinate, x not 16-byte aligned, source outside the window
  CHK_TMEM = 5,         // tensor-memory address beyond 512 columns / 128 lanes, or not this warp's lane quarter
  CHK_GLOBAL = 6,       // global index beyond its extent
  CHK_SCHEDULE = 7      // tile / k-block / stage / slot index beyond its extent
};
#ifdef B200_CHECKED_BUILD
__device__ unsigned long long g_check_log[4];   // [0] failures  [1] code << 32 | line  [2] value  [3] limit
__device__ __noinline__ bool check_failed(int code, int line, unsigned long long value, unsigned long long limit) {
  if (atomicAdd(&g_check_log[0], 1ull) == 0ull) {
    g_check_log[1] = (static_cast<unsigned long long>(code) << 32) | static_cast<unsigned>(line);
    g_check_log[2] = value;
    g_check_log[3] = limit;
  }
  return false;
}
#define B200_CHECK(ok, code, value, limit)                                                     \
  ((ok) ? true                                                                                 \
        : ::b200::check_failed((code), __LINE__, static_cast<unsigned long long>(value),        \
                               static_cast<unsigned long long>(limit)))
__device__ __forceinline__ uint32_t cta_smem_bytes() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%total_smem_size;" : "=r"(r));
  return r;
}
// [addr, addr + bytes) inside this CTA's shared window and addr aligned to `align`.  In a cluster
// launch a CTA's own shared addresses carry its rank above bit 24 (they are valid shared::cluster
// addresses of itself), so the offset inside the window is the low 24 bits.
__device__ __forceinline__ bool smem_ok(uint32_t addr, uint32_t bytes, uint32_t align, int code) {
  const uint32_t window = cta_smem_bytes(), off = addr & 0x00FFFFFFu;
  return B200_CHECK(addr % align == 0, code, addr, align) && B200_CHECK(off <= window && bytes <= window - off, code, addr, window);
}
// a tensor-memory address (lane << 16 | column) with `cols` columns behind it
__device__ __forceinline__ bool tmem_ok(uint32_t taddr, uint32_t cols) {
  return B200_CHECK((taddr & 0xFFFFu) + cols <= 512u, CHK_TMEM, taddr, cols) && B200_CHECK((taddr >> 16) < 128u, CHK_TMEM, taddr, 128u);
}
// tcgen05.ld / .st 32x32b: a warp reaches only the lane quarter 32 * (warp index % 4)
__device__ __forceinline__ bool tmem_warp_ok(uint32_t taddr, uint32_t cols) {
  return tmem_ok(taddr, cols) && B200_CHECK((taddr >> 16) == 32u * ((threadIdx.x >> 5) & 3u), CHK_TMEM, taddr, threadIdx.x >> 5);
}
__device__ __forceinline__ uint32_t cta_smem_bytes_or_max() { return cta_smem_bytes(); }
#else
#define B200_CHECK(ok, code, value, limit) (true)
__device__ __forceinline__ uint32_t cta_smem_bytes_or_max() { return 0xFFFFFFFFu; }
__device__ __forceinline__ bool smem_ok(uint32_t, uint32_t, uint32_t, int) { return true; }
__device__ __forceinline__ bool tmem_ok(uint32_t, uint32_t) { return true; }
__device__ __forceinline__ bool tmem_warp_ok(uint32_t, uint32_t) { return true; }
#endif

// ----------------------------------------------------------------------------------
// addresses
// ----------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
}

// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization
// attribute may start while the kernel before it in the stream is still running, once every CTA of
// that kernel has called grid_launch_dependents() (or exited); it must call grid_dependency_wait()
// before it touches anything that kernel may have written.  Without the attribute, or after a kernel
// that never signals, both are no-ops in effect.
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  if (!smem_ok(bar, 8, 8, CHK_BARRIER)) return;
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  if (!smem_ok(bar, 8, 8, CHK_BARRIER)) return;
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  if (!smem_ok(bar, 8, 8, CHK_BARRIER)) return;
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// arrive on a barrier that lives in another CTA of the cluster (address from map_to_cta)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
               : "memory");
}
// the same without the release fence: for arrivals that hand over no data in memory
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  if (!smem_ok(bar, 8, 8, CHK_BARRIER)) return false;
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// cluster-scope acquire: pairs with remote arrivals (mbar_arrive_cluster) and with
// tcgen05.commit / TMA completions issued by the peer CTA
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  if (!smem_ok(bar, 8, 8, CHK_BARRIER)) return false;
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// ----------------------------------------------------------------------------------
// proxies / fences
// ----------------------------------------------------------------------------------
// make generic-proxy writes to shared memory visible to the async proxy (TMA store, UMMA)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  if (!smem_ok(addr, 16, 16, CHK_SMEM_RANGE)) return make_uint4(0, 0, 0, 0);
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  if (!smem_ok(addr, 16, 16, CHK_SMEM_RANGE)) return;
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  if (!smem_ok(addr, 16, 16, CHK_SMEM_RANGE)) return;
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ----------------------------------------------------------------------------------
// TMA (tensor maps are passed as __grid_constant__ kernel parameters)
// ----------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// 2-D tile load into this CTA's shared memory, completion on this CTA's mbarrier
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int c0,
                                            int c1) {
  if (!smem_ok(dst, 128, 128, CHK_TMA_LOAD) || !B200_CHECK((c0 & 7) == 0, CHK_TMA_LOAD, c0, 8)) return;
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
// 2-D tile load for a CTA pair: data lands in this CTA's shared memory, the byte count
// completes on `cluster_bar`, which may be the pair leader's mbarrier (map_to_cta address)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* tmap,
                                                 uint32_t cluster_bar, int c0, int c1) {
  if (!smem_ok(dst, 128, 128, CHK_TMA_LOAD) || !B200_CHECK((c0 & 7) == 0, CHK_TMA_LOAD, c0, 8)) return;
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(cluster_bar), "r"(c0), "r"(c1)
      : "memory");
}
// Whole-warp forms for a producer loop that all 32 lanes run converged with identical arguments:
// one elected lane performs the operation (see umma_bf16_elect for why the loop stays uniform).
__device__ __forceinline__ void tma_load_2d_elect(uint32_t dst, const void* tmap, uint32_t bar, int c0,
                                                  int c1) {
  if (!smem_ok(dst, 128, 128, CHK_TMA_LOAD) || !B200_CHECK((c0 & 7) == 0, CHK_TMA_LOAD, c0, 8)) return;
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];\n\t"
      "}"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair_elect(uint32_t dst, const void* tmap,
                                                       uint32_t cluster_bar, int c0, int c1) {
  if (!smem_ok(dst, 128, 128, CHK_TMA_LOAD) || !B200_CHECK((c0 & 7) == 0, CHK_TMA_LOAD, c0, 8)) return;
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];\n\t"
      "}"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(cluster_bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_elect(uint32_t bar, uint32_t bytes) {
  if (!smem_ok(bar, 8, 8, CHK_BARRIER)) return;
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t"
      "}" ::"r"(bar),
      "r"(bytes)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_elect(uint32_t bar) {
  if (!smem_ok(bar, 8, 8, CHK_BARRIER)) return;
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q mbarrier.arrive.shared::cta.b64 _, [%0];\n\t"
      "}" ::"r"(bar)
      : "memory");
}
// 2-D tile store shared -> global (bulk async group)
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src, int c0, int c1) {
  if (!smem_ok(src, 128, 128, CHK_TMA_STORE) || !B200_CHECK(c0 >= 0 && c1 >= 0 && (c0 & 3) == 0, CHK_TMA_STORE, c0, c1)) return;
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(tmap)), "r"(src), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------------------------
// tensor memory allocation (one warp, all lanes)
// ----------------------------------------------------------------------------------
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols)
                 : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols)
                 : "memory");
}
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}

// ----------------------------------------------------------------------------------
// UMMA: D[tmem] (+)= A[smem desc] . B[smem desc], bf16 x bf16 -> fp32, one thread issues
// ----------------------------------------------------------------------------------
template <int CTA_GROUP>
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  if (!tmem_ok(tmem_d, 1) || !B200_CHECK(((adesc & 0x3FFFull) << 4) < cta_smem_bytes_or_max(), CHK_SMEM_RANGE, adesc, 0) || !B200_CHECK(((bdesc & 0x3FFFull) << 4) < cta_smem_bytes_or_max(), CHK_SMEM_RANGE, bdesc, 0)) return;
  if constexpr (CTA_GROUP == 1)
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Whole-warp form: every lane of a converged warp calls this with identical arguments and one
// elected lane issues the instruction.  Keeping the issuing loop warp-uniform lets the compiler
// hold descriptors, addresses and loop state in uniform registers, which is where the
// instruction reads them from; a loop that runs under a one-lane branch pays a transfer per
// operand per instruction instead.
template <int CTA_GROUP>
__device__ __forceinline__ void umma_bf16_elect(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                                uint32_t idesc, uint32_t accumulate) {
  if (!tmem_ok(tmem_d, 1) || !B200_CHECK(((adesc & 0x3FFFull) << 4) < cta_smem_bytes_or_max(), CHK_SMEM_RANGE, adesc, 0) || !B200_CHECK(((bdesc & 0x3FFFull) << 4) < cta_smem_bytes_or_max(), CHK_SMEM_RANGE, bdesc, 0)) return;
  if constexpr (CTA_GROUP == 1)
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@q tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// same, with the A operand read from tensor memory (128 lanes x K/2 32-bit columns, two
// consecutive-k bf16 per column, K-major) instead of shared memory
template <int CTA_GROUP>
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                             uint32_t idesc, uint32_t accumulate) {
  if (!tmem_ok(tmem_d, 1) || !tmem_ok(tmem_a, 1) || !B200_CHECK(((bdesc & 0x3FFFull) << 4) < cta_smem_bytes_or_max(), CHK_SMEM_RANGE, bdesc, 0)) return;
  if constexpr (CTA_GROUP == 1)
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// whole-warp form of umma_bf16_ts (see umma_bf16_elect)
template <int CTA_GROUP>
__device__ __forceinline__ void umma_bf16_ts_elect(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                                   uint32_t idesc, uint32_t accumulate) {
  if (!tmem_ok(tmem_d, 1) || !tmem_ok(tmem_a, 1) || !B200_CHECK(((bdesc & 0x3FFFull) << 4) < cta_smem_bytes_or_max(), CHK_SMEM_RANGE, bdesc, 0)) return;
  if constexpr (CTA_GROUP == 1)
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@q tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// registers -> tensor memory: lane i of the warp writes TMEM lane (base lane + i), 16 columns
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  if (!tmem_warp_ok(taddr, 16)) return;
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// arrive (count 1) on this CTA's mbarrier once all previously issued UMMAs have finished
__device__ __forceinline__ void umma_commit_1cta(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// CTA-pair form: arrive on the mbarrier at the same offset in every CTA named by cta_mask
// (a barrier arrival broadcast, not a data load)
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::
          "r"(bar),
      "h"(cta_mask)
      : "memory");
}

// whole-warp forms of the two commits (same elected lane as umma_bf16_elect)
__device__ __forceinline__ void umma_commit_1cta_elect(uint32_t bar) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "}" ::"r"(bar)
      : "memory");
}
__device__ __forceinline__ void umma_commit_pair_elect(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t"
      "}" ::"r"(bar),
      "h"(cta_mask)
      : "memory");
}

// tensor memory -> registers: lane i of the warp reads TMEM lane (base lane + i),
// N consecutive 32-bit columns
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  if (!tmem_warp_ok(taddr, 32)) {
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = 0u;
    return;
  }
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  if (!tmem_warp_ok(taddr, 16)) {
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = 0u;
    return;
  }
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ----------------------------------------------------------------------------------
// descriptors
// ----------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a 128-byte-swizzled operand tile.
//   bits  0-13  start address >> 4        bits 16-29  leading byte offset >> 4
//   bits 32-45  stride byte offset >> 4   bits 46-47  descriptor version (1 on sm_100)
//   bits 61-63  layout type (2 = 128-byte swizzle)
// MN-major tile (M or N contiguous, rows of 64 elements = 128 B, 8 k-rows per 1 KB atom):
//   stride offset  = distance between consecutive groups of 8 k-rows
//   leading offset = distance between consecutive 64-element chunks along M/N
// K-major tile (K contiguous, rows of 64 k = 128 B):
//   stride offset  = distance between consecutive groups of 8 M/N rows; leading unused
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor for kind::f16 with bf16 operands and fp32 accumulation.
//   bits 4-5 D format (1 = f32)   bits 7-9 A format (1 = bf16)   bits 10-12 B format
//   bit 15 A major (1 = MN)       bit 16 B major (1 = MN)
//   bits 17-22 N >> 3             bits 24-28 M >> 4
__host__ __device__ constexpr uint32_t make_idesc_bf16_f32(int umma_m, int umma_n, int a_mn_major,
                                                           int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(umma_n >> 3) << 17) |
         (static_cast<uint32_t>(umma_m >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// packed bf16 multiply: one rounding per lane (same result as fp32 multiply then round)
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}

}  // namespace b200
