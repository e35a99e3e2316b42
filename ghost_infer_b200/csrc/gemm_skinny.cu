// Products of a few rows of activations with a bfloat16 weight matrix: out[M,N] (op)= A[M,K] * W[N,K]^T, M <= 64.
//
// This is the decode step's product, bound by the bytes of W (the role of the reference's dp4a decode
// kernels, src/cuda.rs:1425-1434, which keep a fixed summation order so that a token's result is the same
// alone or in a batch, src/cuda.rs:748-766).  A block owns 32 rows of W and all of K; its 8 warps take
// 32-column steps of K in turn, stream their rows straight from global memory into mma.sync fragments
// (16 bytes per thread and row, no shared-memory staging), and multiply them with the activations, which
// stay in L1.  W rows are the "M" side of m16n8k16 and tokens the "N" side, so 8 tokens cost one
// instruction per 16x16 piece of W.  The k positions inside a 32-column step are permuted so that a
// thread's 16 contiguous bytes feed both halves of two instructions; the same permutation is applied to
// the activations, so the dot products are unchanged.  Partial sums of the 8 warps are added in warp
// order through shared memory: a given (row, token) is always summed in the same order.
//
// Epilogues: store (bfloat16 or float), add into the float residual stream, or SwiGLU, for which W holds
// gate and up rows interleaved in blocks of 8 (rows 16b..16b+7 gate j, 16b+8..16b+15 up j).
#include "api.h"
#include "common.cuh"

namespace {

constexpr int ROWS = 32;     // W rows per block
constexpr int WARPS = 8;

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_keep(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT, int UNROLL, int MODE>
__global__ void __launch_bounds__(WARPS * 32)
skinny_kernel(void* __restrict__ out_, const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W, int M, int N,
              int K, long lda, long ldw, long ldo) {
  constexpr int RNT = NT < 4 ? NT : 4;
  __shared__ float red[WARPS][2][RNT][32][4];
  gi::pdl_prologue();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * ROWS;

  // rows of W this thread reads (clamped: rows past N are computed from row N-1 and never stored)
  const __nv_bfloat16* wrow[2][2];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt) {
    wrow[mt][0] = W + (size_t)min(n0 + mt * 16 + g, N - 1) * ldw + t * 8;
    wrow[mt][1] = W + (size_t)min(n0 + mt * 16 + g + 8, N - 1) * ldw + t * 8;
  }
  const __nv_bfloat16* arow[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) arow[nt] = A + (size_t)min(nt * 8 + g, M - 1) * lda + t * 8;

  float acc[2][NT][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[mt][nt][c] = 0.f;

  const int steps = (K + 31) / 32;
  for (int s0 = warp; s0 < steps; s0 += WARPS * UNROLL) {
    uint4 w[UNROLL][2][2], x[UNROLL][NT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int s = s0 + u * WARPS;
      const int k = s * 32;
      const bool live = s < steps && k + t * 8 < K;    // K is a multiple of 8: a thread's 8 columns are all in or all out
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        w[u][mt][0] = live ? ld_stream(wrow[mt][0] + k) : make_uint4(0, 0, 0, 0);
        w[u][mt][1] = live ? ld_stream(wrow[mt][1] + k) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) x[u][nt] = live ? ld_keep(arow[nt] + k) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          mma_bf16(acc[mt][nt], w[u][mt][0].x, w[u][mt][1].x, w[u][mt][0].y, w[u][mt][1].y, x[u][nt].x, x[u][nt].y);
          mma_bf16(acc[mt][nt], w[u][mt][0].z, w[u][mt][1].z, w[u][mt][0].w, w[u][mt][1].w, x[u][nt].z, x[u][nt].w);
        }
  }

  // partial sums of the 8 warps, added in warp order; at most 4 token tiles go through shared memory at a time
  for (int ntb = 0; ntb < NT; ntb += RNT) {
    if (ntb) __syncthreads();
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < RNT; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) red[warp][mt][nt][lane][c] = acc[mt][ntb + nt][c];
    __syncthreads();

    if (MODE == GI_SKINNY_SWIGLU) {
      // 16 activations x (8 RNT) tokens: feature j = n0/2 + mt*8 + g, gate at tile row g, up at tile row g + 8
      for (int idx = threadIdx.x; idx < 16 * 8 * RNT; idx += WARPS * 32) {
        const int ml = idx / 16, fl = idx % 16;
        const int mt = fl / 8, gg = fl % 8, nt = ml / 8, tt = (ml % 8) / 2, c = ml % 2;
        const int ln = gg * 4 + tt;
        float gate = 0.f, up = 0.f;
#pragma unroll
        for (int wv = 0; wv < WARPS; ++wv) {
          gate += red[wv][mt][nt][ln][c];
          up += red[wv][mt][nt][ln][2 + c];
        }
        const int f = n0 / 2 + fl, m = ntb * 8 + ml;
        if (m < M && f < N / 2) ((__nv_bfloat16*)out_)[(size_t)m * ldo + f] = __float2bfloat16_rn(gi::silu_mul_bf16(gate, up));
      }
      continue;
    }
    for (int idx = threadIdx.x; idx < ROWS * 8 * RNT; idx += WARPS * 32) {
      const int ml = idx / ROWS, fl = idx % ROWS;
      const int mt = fl / 16, r = fl % 16, gg = r % 8, hi = r / 8, nt = ml / 8, tt = (ml % 8) / 2;
      const int c = hi * 2 + (ml % 2), ln = gg * 4 + tt;
      float v = 0.f;
#pragma unroll
      for (int wv = 0; wv < WARPS; ++wv) v += red[wv][mt][nt][ln][c];
      const int f = n0 + fl, m = ntb * 8 + ml;
      if (m >= M || f >= N) continue;
      if (MODE == GI_SKINNY_ACCUM_F32) {
        float* o = (float*)out_ + (size_t)m * ldo + f;
        *o += v;
      } else if (MODE == GI_SKINNY_STORE_F32) {
        ((float*)out_)[(size_t)m * ldo + f] = v;
      } else {
        ((__nv_bfloat16*)out_)[(size_t)m * ldo + f] = __float2bfloat16_rn(v);
      }
    }
  }
}

template <int NT, int UNROLL>
int launch_mode(int mode, dim3 grid, cudaStream_t s, void* out, const __nv_bfloat16* A, const __nv_bfloat16* W, int M, int N,
                int K, long lda, long ldw, long ldo) {
  cudaError_t e = cudaSuccess;
  switch (mode) {
    case GI_SKINNY_STORE_BF16:
      e = gi::launch(skinny_kernel<NT, UNROLL, GI_SKINNY_STORE_BF16>, grid, dim3(WARPS * 32), 0, s, out, A, W, M, N, K, lda, ldw, ldo);
      break;
    case GI_SKINNY_STORE_F32:
      e = gi::launch(skinny_kernel<NT, UNROLL, GI_SKINNY_STORE_F32>, grid, dim3(WARPS * 32), 0, s, out, A, W, M, N, K, lda, ldw, ldo);
      break;
    case GI_SKINNY_ACCUM_F32:
      e = gi::launch(skinny_kernel<NT, UNROLL, GI_SKINNY_ACCUM_F32>, grid, dim3(WARPS * 32), 0, s, out, A, W, M, N, K, lda, ldw, ldo);
      break;
    case GI_SKINNY_SWIGLU:
      e = gi::launch(skinny_kernel<NT, UNROLL, GI_SKINNY_SWIGLU>, grid, dim3(WARPS * 32), 0, s, out, A, W, M, N, K, lda, ldw, ldo);
      break;
    default:
      return gi::fail(GI_ERR_ARG, "skinny product: unknown mode %d", mode);
  }
  return gi::check(e, "skinny product");
}

}  // namespace

extern "C" int gi_gemm_skinny_bf16(void* out, int mode, const void* A, const void* W, int M, int N, int K, long lda,
                                   long ldw, long ldo, void* stream) {
  if (M <= 0 || N <= 0) return GI_OK;
  if (M > 64) return gi::fail(GI_ERR_UNSUPPORTED, "skinny product: %d rows of activations, at most 64", M);
  if (K <= 0 || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0)
    return gi::fail(GI_ERR_UNSUPPORTED, "skinny product: K (%d) and the row strides (%ld, %ld) must be multiples of 8", K, lda, ldw);
  if (((uintptr_t)A | (uintptr_t)W) & 15) return gi::fail(GI_ERR_UNSUPPORTED, "skinny product: operands must be 16-byte aligned");
  if (mode == GI_SKINNY_SWIGLU && N % 16 != 0) return gi::fail(GI_ERR_UNSUPPORTED, "skinny product: SwiGLU needs interleaved rows, N (%d) a multiple of 16", N);
  dim3 grid((N + ROWS - 1) / ROWS);
  cudaStream_t s = (cudaStream_t)stream;
  const __nv_bfloat16* a = (const __nv_bfloat16*)A;
  const __nv_bfloat16* w = (const __nv_bfloat16*)W;
  if (M <= 8) return launch_mode<1, 4>(mode, grid, s, out, a, w, M, N, K, lda, ldw, ldo);
  if (M <= 16) return launch_mode<2, 4>(mode, grid, s, out, a, w, M, N, K, lda, ldw, ldo);
  if (M <= 32) return launch_mode<4, 2>(mode, grid, s, out, a, w, M, N, K, lda, ldw, ldo);
  return launch_mode<8, 1>(mode, grid, s, out, a, w, M, N, K, lda, ldw, ldo);
}
