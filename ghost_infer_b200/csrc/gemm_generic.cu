// Plain matrix product on CUDA cores with 32-bit accumulation: out[M,N] (op)= A[M,K] * W[N,K]^T.
//
// This is the kernel of the true 32-bit path (no tensor cores, no reduced-precision mode), and the
// reference beside every faster product.  Each output element is summed by one thread walking k in
// increasing order, so a row's result does not depend on what else is in the batch.  Weights are
// row-major [out, in] without bias, as the reference keeps them (src/model.rs:1019, src/quant.rs:73-78).
#include "api.h"
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TA, typename TW, typename TO, int MODE>
__global__ void __launch_bounds__(256)
gemm_tile_kernel(void* __restrict__ out_, const TA* __restrict__ A, const TW* __restrict__ W, int M, int N, int K,
                 long lda, long ldw, long ldo) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid % 16, ty = tid / 16;  // thread owns rows ty*4..+4, cols tx*4..+4
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 k per operand = 1024 elements, 4 per thread; consecutive threads walk k (contiguous)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;
      const int r = idx / BK, kk = idx % BK;
      const int k = k0 + kk;
      float a = 0.f, w = 0.f;
      if (k < K) {
        if (m0 + r < M) a = gi::ldf(A + (size_t)(m0 + r) * lda + k);
        if (n0 + r < N) w = gi::ldf(W + (size_t)(n0 + r) * ldw + k);
      }
      As[kk][r] = a;
      Ws[kk][r] = w;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      if (MODE == GI_GEMM_ACCUM_F32) {
        float* o = (float*)out_ + (size_t)m * ldo + n;
        *o = *o + acc[i][j];
      } else {
        gi::stf((TO*)out_ + (size_t)m * ldo + n, acc[i][j]);
      }
    }
  }
}

template <typename TA, typename TW>
int launch(void* out, int out_dtype, int mode, const void* A, const void* W, int M, int N, int K, long lda, long ldw,
           long ldo, cudaStream_t s) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (mode == GI_GEMM_ACCUM_F32) {
    gemm_tile_kernel<TA, TW, float, GI_GEMM_ACCUM_F32><<<grid, 256, 0, s>>>(out, (const TA*)A, (const TW*)W, M, N, K, lda, ldw, ldo);
  } else if (out_dtype == GI_F32) {
    gemm_tile_kernel<TA, TW, float, GI_GEMM_STORE><<<grid, 256, 0, s>>>(out, (const TA*)A, (const TW*)W, M, N, K, lda, ldw, ldo);
  } else {
    gemm_tile_kernel<TA, TW, __nv_bfloat16, GI_GEMM_STORE><<<grid, 256, 0, s>>>(out, (const TA*)A, (const TW*)W, M, N, K, lda, ldw, ldo);
  }
  return gi::check_launch("gemm_generic");
}

}  // namespace

extern "C" int gi_gemm_generic(void* out, int out_dtype, int mode, const void* A, int a_dtype, const void* W,
                               int w_dtype, int M, int N, int K, long lda, long ldw, long ldo, void* stream) {
  if (M <= 0 || N <= 0) return GI_OK;
  if (K <= 0) return gi::fail(GI_ERR_ARG, "gemm: K must be positive, got %d", K);
  if (mode != GI_GEMM_STORE && mode != GI_GEMM_ACCUM_F32) return gi::fail(GI_ERR_ARG, "gemm: unknown mode %d", mode);
  if (mode == GI_GEMM_ACCUM_F32 && out_dtype != GI_F32) return gi::fail(GI_ERR_ARG, "gemm: accumulation needs a float output");
  if ((N + BN - 1) / BN > 2147483647 || (M + BM - 1) / BM > 65535)
    return gi::fail(GI_ERR_UNSUPPORTED, "gemm: %d rows are more than one launch takes (%d)", M, 65535 * BM);
  GI_DISPATCH_DTYPE(a_dtype, TA, GI_DISPATCH_DTYPE(w_dtype, TW,
      return (launch<TA, TW>(out, out_dtype, mode, A, W, M, N, K, lda, ldw, ldo, (cudaStream_t)stream))));
  return GI_OK;
}
