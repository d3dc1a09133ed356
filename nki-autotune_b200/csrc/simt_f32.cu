// fp32 CUDA-core contraction kernels (no tensor cores, no tf32).
//
//   matmul_lhsT_rhs_f32 : C[M,N] = lhsT[K,M]^T . rhs[K,N], fp32 in, fp32 out.  This is the
//     1e-5 configuration and follows NKIMatmul._run (nkigym/src/nkigym/ops/matmul.py:43-45).
//   rmsnorm_matmul_f32  : out[M,N] = rinv[m] * sum_k x[m,k] gamma[k] w[k,n] on bf16 inputs with
//     fp32 arithmetic, rinv[m] = rsqrt(mean_k x[m,k]^2 + eps): the on-device cross-check of the
//     fused tensor-core kernel (kernel_library/rmsnorm_matmul/kernel_hand_online.py:5-17).
//
// Classic shared-memory tiling: a 64x64 output tile per 256-thread block, 16-deep k slices,
// 4x4 outputs per thread.  Any shape is accepted (edges are predicated).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_api.h"

namespace b200 {

constexpr int SB_M = 64, SB_N = 64, SB_K = 16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

// A_KM: a(k, m) = a[k * lda + m]   (lhsT);   otherwise a(m, k) = a[m * lda + k]   (x)
template <typename T, bool A_KM, bool FUSE_NORM>
__global__ void __launch_bounds__(256)
simt_gemm_kernel(const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ gamma,
                 float* __restrict__ c, long M, long N, long K, long lda, long ldb, long ldc,
                 float eps) {
  __shared__ float as[SB_K][SB_M + 1];
  __shared__ float bs[SB_K][SB_N + 1];
  __shared__ float sumsq[SB_M];

  const int tid = threadIdx.x;
  const int tx = tid & 15;   // 16 column groups of 4
  const int ty = tid >> 4;   // 16 row groups of 4
  const long m0 = static_cast<long>(blockIdx.y) * SB_M;
  const long n0 = static_cast<long>(blockIdx.x) * SB_N;

  float acc[4][4] = {};

  for (long k0 = 0; k0 < K; k0 += SB_K) {
    // stage A: 16 x 64 values, 4 per thread
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;
      int kk, mm;
      if (A_KM) { kk = e >> 6; mm = e & 63; } else { mm = e >> 4; kk = e & 15; }
      const long gk = k0 + kk, gm = m0 + mm;
      float v = 0.0f;
      if (gk < K && gm < M) v = to_f32(A_KM ? a[gk * lda + gm] : a[gm * lda + gk]);
      if (FUSE_NORM && gamma != nullptr && gk < K) {
        as[kk][mm] = v * to_f32(gamma[gk]);
      } else {
        as[kk][mm] = v;
      }
      if (FUSE_NORM) {
        // x values of one row are spread over 16 consecutive threads (kk = e & 15)
        float sq = v * v;
#pragma unroll
        for (int off = 8; off >= 1; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off, 16);
        if ((e & 15) == 0) {
          // row mm visited exactly once per k slice by the lane with kk == 0
          if (k0 == 0) sumsq[mm] = sq; else sumsq[mm] += sq;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;
      const int kk = e >> 6, nn = e & 63;
      const long gk = k0 + kk, gn = n0 + nn;
      bs[kk][nn] = (gk < K && gn < N) ? to_f32(b[gk * ldb + gn]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SB_K; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = as[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
    float scale = 1.0f;
    if (FUSE_NORM) scale = rsqrtf(sumsq[ty * 4 + i] / static_cast<float>(K) + eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long gn = n0 + tx * 4 + j;
      if (gn < N) c[gm * ldc + gn] = acc[i][j] * scale;
    }
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_matmul_lhsT_rhs_f32(const void* lhsT, const void* rhs, void* out, long M, long N,
                                        long K, long ld_lhsT, long ld_rhs, long ld_out,
                                        void* stream) {
  if (!lhsT || !rhs || !out) return set_error(B200_ERR_BAD_ARG, "matmul_lhsT_rhs_f32: NULL pointer");
  if (M <= 0 || N <= 0 || K <= 0) return set_error(B200_ERR_BAD_SHAPE, "matmul_lhsT_rhs_f32: empty shape");
  if (ld_lhsT == 0) ld_lhsT = M;
  if (ld_rhs == 0) ld_rhs = N;
  if (ld_out == 0) ld_out = N;
  if (ld_lhsT < M || ld_rhs < N || ld_out < N)
    return set_error(B200_ERR_BAD_SHAPE, "matmul_lhsT_rhs_f32: leading dimension smaller than row");
  dim3 grid(static_cast<unsigned>((N + SB_N - 1) / SB_N), static_cast<unsigned>((M + SB_M - 1) / SB_M));
  simt_gemm_kernel<float, true, false><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(lhsT), static_cast<const float*>(rhs), nullptr,
      static_cast<float*>(out), M, N, K, ld_lhsT, ld_rhs, ld_out, 0.0f);
  return check_cuda(cudaGetLastError(), "matmul_lhsT_rhs_f32 launch");
}

extern "C" int b200_rmsnorm_matmul_f32(const void* x, const void* gamma, const void* w, void* out_f32,
                                       long M, long N, long K, float eps, void* stream) {
  if (!x || !w || !out_f32) return set_error(B200_ERR_BAD_ARG, "rmsnorm_matmul_f32: NULL pointer");
  if (M <= 0 || N <= 0 || K <= 0) return set_error(B200_ERR_BAD_SHAPE, "rmsnorm_matmul_f32: empty shape");
  dim3 grid(static_cast<unsigned>((N + SB_N - 1) / SB_N), static_cast<unsigned>((M + SB_M - 1) / SB_M));
  simt_gemm_kernel<__nv_bfloat16, false, true><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<const __nv_bfloat16*>(gamma), static_cast<float*>(out_f32), M, N, K, K, N, N, eps);
  return check_cuda(cudaGetLastError(), "rmsnorm_matmul_f32 launch");
}
