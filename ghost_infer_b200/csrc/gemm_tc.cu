// Prefill matrix product on Blackwell's tensor cores: out[M,N] (op)= A[M,K] * W[N,K]^T, bfloat16 operands,
// 32-bit accumulation in tensor memory.
//
// The role of the reference's prompt GEMM (matmul_mma, src/cuda.rs:2986-3200: 64x64 tiles of int8 mma.sync with
// a register-prefetch pipeline) rebuilt for sm_100a: a block owns a 128 x BN tile of the output; one thread
// feeds a ring of shared-memory stages with TMA (128-byte-swizzled boxes of 64 k-columns of A and of W),
// one thread issues tcgen05.mma (M 128, N BN, K 16, four per stage) whose accumulator lives in tensor
// memory, and four warps read the accumulator back with tcgen05.ld and write the epilogue: store
// (bfloat16 or float), add into the float residual stream (src/cuda.rs:9774: the reference's accumulate=1),
// or SwiGLU over gate/up rows interleaved in blocks of 8.  Stages are handed over with mbarriers:
// TMA completes `full`, tcgen05.commit arrives on `empty` when the products that read a stage are done.
// Rows and columns past M, N or K are zero-filled by TMA and masked at the store, so every size whose rows
// are 16 bytes apart is taken.  Every wait has an iteration limit; a wait that runs out records a status
// word and the block leaves through its normal exit (tensor memory freed).
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "api.h"
#include "common.cuh"
#include "tc_utils.cuh"

namespace {

constexpr int BM = 128;      // rows of A per block = tensor-memory lanes
constexpr int BK = 64;       // k-columns per stage = one 128-byte swizzle row
constexpr int THREADS = 192; // warp 0: TMA, warp 1: MMA and tensor-memory allocation, warps 2-5: epilogue

__device__ int g_status = 0;   // 0 = fine; else which wait ran out (1 producer, 2 mma, 3 epilogue)

using namespace gi::tc;

template <int BN, int STAGES, int MODE>
__global__ void __launch_bounds__(THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, void* __restrict__ out_,
               int M, int N, int K, long ldo) {
  constexpr uint32_t A_BYTES = BM * BK * 2, W_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + W_BYTES;
  // instruction descriptor: float accumulator (bits 4-5 = 1), bfloat16 A and B (bits 7-9, 10-12 = 1), both K-major,
  // N / 8 in bits 17-22, M / 16 in bits 24-28
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);   // full[STAGES], empty[STAGES], accumulator ready
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int num_kb = (K + BK - 1) / BK;
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES), done = smem_u32(bars + 2 * STAGES);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t round = (uint32_t)(kb / STAGES);
        if (!mbar_wait(empty0 + 8 * s, (round & 1) ^ 1, 1, &g_status)) break;     // a fresh barrier passes the first round
        mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
        const uint32_t dst = smem_u32(smem + (size_t)s * STAGE_BYTES);
        tma_load_2d(dst, &map_a, kb * BK, m0, full0 + 8 * s);
        tma_load_2d(dst + A_BYTES, &map_w, kb * BK, n0, full0 + 8 * s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % STAGES;
        const uint32_t round = (uint32_t)(kb / STAGES);
        ok = mbar_wait(full0 + 8 * s, round & 1, 2, &g_status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
        const uint64_t da = smem_desc(a_addr), dw = smem_desc(a_addr + A_BYTES);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)     // 16 k-columns = 32 bytes further along the swizzled row
          tc_mma(tmem, da + (uint64_t)(2 * k), dw + (uint64_t)(2 * k), IDESC, (kb > 0 || k > 0) ? 1u : 0u);
        tc_commit(empty0 + 8 * s);            // arrives when these products no longer read the stage
      }
      tc_commit(done);                        // arrives when the accumulator is complete
    }
  } else {
    const int quarter = warp & 3;             // the tensor-memory lanes this warp may read: 32 * (warp % 4)
    const int row = quarter * 32 + lane;
    const long m = (long)m0 + row;
    const bool live = mbar_wait(done, 0, 3, &g_status);
    tc_fence_after();
    if (live) {
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tc_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 32), r);
        tc_wait_ld();
        const int nb = n0 + c * 32;
        if (m >= M || nb >= N) {
          // nothing to store for this thread; it still takes part in the next (warp-wide) tensor-memory load
        } else if (MODE == GI_TC_SWIGLU) {
          // columns [8 gate | 8 up | 8 gate | 8 up] -> 16 activations
          __nv_bfloat16* o = (__nv_bfloat16*)out_ + m * ldo + nb / 2;
#pragma unroll
          for (int blk = 0; blk < 2; ++blk) {
            if (nb + blk * 16 >= N) break;
            uint32_t packed[4];
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
              const float g0 = __uint_as_float(r[blk * 16 + j]), g1 = __uint_as_float(r[blk * 16 + j + 1]);
              const float u0 = __uint_as_float(r[blk * 16 + 8 + j]), u1 = __uint_as_float(r[blk * 16 + 8 + j + 1]);
              __nv_bfloat162 v = __floats2bfloat162_rn(g0 / (1.0f + expf(-g0)) * u0, g1 / (1.0f + expf(-g1)) * u1);
              packed[j / 2] = *reinterpret_cast<uint32_t*>(&v);
            }
            *reinterpret_cast<uint4*>(o + blk * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        } else if (MODE == GI_TC_ACCUM_F32) {
          float* o = (float*)out_ + m * ldo + nb;
          if (nb + 32 <= N) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float4 v = *reinterpret_cast<float4*>(o + j);
              v.x += __uint_as_float(r[j]);
              v.y += __uint_as_float(r[j + 1]);
              v.z += __uint_as_float(r[j + 2]);
              v.w += __uint_as_float(r[j + 3]);
              *reinterpret_cast<float4*>(o + j) = v;
            }
          } else {
            for (int j = 0; j < 32 && nb + j < N; ++j) o[j] += __uint_as_float(r[j]);
          }
        } else if (MODE == GI_TC_STORE_F32) {
          float* o = (float*)out_ + m * ldo + nb;
          if (nb + 32 <= N) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(o + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                              __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
          } else {
            for (int j = 0; j < 32 && nb + j < N; ++j) o[j] = __uint_as_float(r[j]);
          }
        } else {
          __nv_bfloat16* o = (__nv_bfloat16*)out_ + m * ldo + nb;
          if (nb + 32 <= N) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint32_t p[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[j + 2 * e]), __uint_as_float(r[j + 2 * e + 1]));
                p[e] = *reinterpret_cast<uint32_t*>(&v);
              }
              *reinterpret_cast<uint4*>(o + j) = make_uint4(p[0], p[1], p[2], p[3]);
            }
          } else {
            for (int j = 0; j < 32 && nb + j < N; ++j) o[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
          }
        }
        __syncwarp();
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)BN) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------- host
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encoder() {
  static EncodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiled)p;
  });
  return fn;
}

// Tensor maps by (address, rows, columns, row stride, box rows): a map is pure data, and the same weights
// and the same activation buffers come back step after step.
}  // namespace

int gi::tensor_map_2d(CUtensorMap* out, const void* base, int rows, int cols, long ld, int box_rows) {
  typedef std::tuple<const void*, int, int, long, int> Key;
  static std::map<Key, CUtensorMap> cache;
  static std::mutex lock;
  const Key key(base, rows, cols, ld, box_rows);
  std::lock_guard<std::mutex> guard(lock);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return GI_OK;
  }
  EncodeTiled enc = encoder();
  if (!enc) return gi::fail(GI_ERR_CUDA, "tensor-core product: the driver does not export cuTensorMapEncodeTiled");
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return gi::fail(GI_ERR_CUDA, "tensor-core product: cuTensorMapEncodeTiled failed with %d", (int)r);
  if (cache.size() > 4096) cache.clear();
  cache[key] = *out;
  return GI_OK;
}

namespace {

template <int BN, int STAGES, int MODE>
int launch(void* out, const CUtensorMap& ma, const CUtensorMap& mw, int M, int N, int K, long ldo, cudaStream_t s) {
  constexpr size_t smem = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + (2 * STAGES + 1) * 8 + 16 + 1024;
  auto kern = gemm_tc_kernel<BN, STAGES, MODE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "tensor-core product: %s", cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid((M + BM - 1) / BM, (N + BN - 1) / BN);
  kern<<<grid, THREADS, smem, s>>>(ma, mw, out, M, N, K, ldo);
  return gi::check_launch("tensor-core product");
}

template <int BN, int STAGES>
int launch_mode(int mode, void* out, const CUtensorMap& ma, const CUtensorMap& mw, int M, int N, int K, long ldo, cudaStream_t s) {
  switch (mode) {
    case GI_TC_STORE_BF16: return launch<BN, STAGES, GI_TC_STORE_BF16>(out, ma, mw, M, N, K, ldo, s);
    case GI_TC_STORE_F32: return launch<BN, STAGES, GI_TC_STORE_F32>(out, ma, mw, M, N, K, ldo, s);
    case GI_TC_ACCUM_F32: return launch<BN, STAGES, GI_TC_ACCUM_F32>(out, ma, mw, M, N, K, ldo, s);
    case GI_TC_SWIGLU: return launch<BN, STAGES, GI_TC_SWIGLU>(out, ma, mw, M, N, K, ldo, s);
  }
  return gi::fail(GI_ERR_ARG, "tensor-core product: unknown mode %d", mode);
}

}  // namespace

extern "C" int gi_gemm_tc_bf16(void* out, int mode, const void* A, const void* W, int M, int N, int K, long lda, long ldw,
                               long ldo, int tile_n, void* stream) {
  if (M <= 0 || N <= 0) return GI_OK;
  if (K <= 0 || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0)
    return gi::fail(GI_ERR_UNSUPPORTED, "tensor-core product: K (%d) and the row strides (%ld, %ld) must be multiples of 8", K, lda, ldw);
  if (((uintptr_t)A | (uintptr_t)W | (uintptr_t)out) & 15) return gi::fail(GI_ERR_UNSUPPORTED, "tensor-core product: operands must be 16-byte aligned");
  const int out_align = (mode == GI_TC_STORE_BF16 || mode == GI_TC_SWIGLU) ? 8 : 4;
  if (ldo % out_align != 0) return gi::fail(GI_ERR_UNSUPPORTED, "tensor-core product: the output's row stride (%ld) must be a multiple of %d", ldo, out_align);
  if (mode == GI_TC_SWIGLU && N % 16 != 0) return gi::fail(GI_ERR_UNSUPPORTED, "tensor-core product: SwiGLU needs interleaved rows, N (%d) a multiple of 16", N);
  if (tile_n != 128 && tile_n != 256) return gi::fail(GI_ERR_ARG, "tensor-core product: tile width %d, 128 or 256", tile_n);
  if ((M + BM - 1) / BM > 2147483647 || (N + tile_n - 1) / tile_n > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "tensor-core product: too many tiles");
  CUtensorMap ma, mw;
  int rc = gi::tensor_map_2d(&ma, A, M, K, lda, BM);
  if (rc != GI_OK) return rc;
  rc = gi::tensor_map_2d(&mw, W, N, K, ldw, tile_n);
  if (rc != GI_OK) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  if (tile_n == 128) return launch_mode<128, 3>(mode, out, ma, mw, M, N, K, ldo, s);
  return launch_mode<256, 4>(mode, out, ma, mw, M, N, K, ldo, s);
}

// Reads and clears the status word of the tensor-core product (0 = every wait was met).  Synchronises the device.
extern "C" int gi_gemm_tc_status(int* status) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(status, g_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
  if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "tensor-core product status: %s", cudaGetErrorString(e));
  return GI_OK;
}
