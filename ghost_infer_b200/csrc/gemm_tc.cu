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
// are 16 bytes apart is taken.  When the tiles do not fill the last round of blocks, the last columns are cut
// into narrower tiles (their own TMA box and instruction width) that fit one round: 256 tiles of 128 x 256 on
// 148 blocks cost two rounds of 256 columns, 144 of them plus 128 tiles of 128 x 224 cost 256 + 224.  Every wait has an iteration limit; a wait that runs out records a status
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
constexpr int THREADS = 192; // warp 0: TMA loads, warp 1: MMA and tensor-memory allocation, warps 2-5: epilogue

__device__ int g_status = 0;   // 0 = fine; else which wait ran out (1 producer, 2 mma, 3 epilogue)
bool g_tail_tiles = true;      // narrower tiles for an unfilled last round

using namespace gi::tc;

// Writes one staged row (128 bytes = eight 16-byte chunks) into a 128-byte-swizzled staging tile.
__device__ __forceinline__ void stage_chunk(unsigned char* stg, int row, int j, uint4 v) {
  *reinterpret_cast<uint4*>(stg + row * 128 + ((j ^ (row & 7)) << 4)) = v;
}

// How the output is cut into tiles: `wide_cols` column tiles of BN, then column tiles of `narrow` (<= BN) columns.
struct TilePlan {
  int wide_cols;     // column tiles of full width
  int narrow;        // width of the column tiles after them (0: none)
  int n_tiles;       // all tiles
};

// What the q/k/v product's epilogue needs to rotate and store by itself (mode GI_TC_QKV_ROPE): the output's columns are
// heads of `hd` values, first n_heads of queries, then n_kv of keys, then n_kv of values.  Queries are rotated and
// stored in the packed rows, keys rotated into the cache, values copied into the cache (src/model.rs:1046-1048);
// the keys' and values' columns of the packed rows are not written at all.
struct RopeEpilogue {
  const float2* table;        // [M][hd / 2] (cos, sin) of each token's position
  const int* positions;       // [M]
  const int* slots;           // [M] the sequence's slot, -1: a padding row (the trash page)
  const int* block_table;
  int max_pages;
  __nv_bfloat16* kcache;
  __nv_bfloat16* vcache;
  int n_heads, n_kv, hd;      // hd 64 or 128, all of it rotated, pairs (i, i + hd / 2)
  int write_cache;
};

template <int BN, int STAGES, int MODE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_w2, const __grid_constant__ CUtensorMap map_o, int M, int N, int K,
               const TilePlan plan, const RopeEpilogue rope) {
  constexpr uint32_t A_BYTES = BM * BK * 2, W_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + W_BYTES;
  constexpr uint32_t STG_BYTES = BM * 128;     // a staging tile: 128 rows of 128 bytes
  // instruction descriptor: float accumulator (bits 4-5 = 1), bfloat16 A and B (bits 7-9, 10-12 = 1), both K-major,
  // N / 8 in bits 17-22, M / 16 in bits 24-28
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  // accumulator columns that make one 128-byte row of output: 32 floats, 64 bfloat16, or 128 gate/up values -> 64 activations
  constexpr int CW = (MODE == GI_TC_SWIGLU) ? 128 : ((MODE == GI_TC_STORE_BF16 || MODE == GI_TC_QKV_ROPE) ? 64 : 32);
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* staging = smem + STAGES * STAGE_BYTES;                 // two staging tiles
  uint64_t* bars = (uint64_t*)(staging + 2 * STG_BYTES);               // full[S], empty[S], acc_full[2], acc_empty[2]
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM;
  const int n_tiles = plan.n_tiles;
  const int wide_tiles = plan.wide_cols * tiles_m;
  const int num_kb = (K + BK - 1) / BK;
  // Tiles in an order that keeps a tile of W in use by neighbouring blocks: the row tile runs fastest.
  auto geometry = [&](int tile, int& m0, int& n0, int& width) {
    if (tile < wide_tiles) {
      m0 = (tile % tiles_m) * BM;
      n0 = (tile / tiles_m) * BN;
      width = BN;
    } else {
      const int t = tile - wide_tiles;
      m0 = (t % tiles_m) * BM;
      n0 = plan.wide_cols * BN + (t / tiles_m) * plan.narrow;
      width = plan.narrow;
    }
  };
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
  const uint32_t accf0 = smem_u32(bars + 2 * STAGES), acce0 = smem_u32(bars + 2 * STAGES + 2);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(accf0 + 8 * b, 1);
      mbar_init(acce0 + 8 * b, 4);      // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)(2 * BN)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  gi::pdl_prologue();      // set-up overlapped the previous kernel's end; its results are visible from here on

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        int m0, n0, width;
        geometry(tile, m0, n0, width);
        const CUtensorMap* mw = width == BN ? &map_w : &map_w2;        // the box of W's rows is as tall as the tile is wide
        const uint32_t bytes = A_BYTES + (uint32_t)width * BK * 2;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(empty0 + 8 * s, (((uint32_t)(it / STAGES)) & 1) ^ 1, 1, &g_status);   // a fresh barrier passes
          if (!ok) break;
          mbar_expect_tx(full0 + 8 * s, bytes);
          const uint32_t dst = smem_u32(smem + (size_t)s * STAGE_BYTES);
          tma_load_2d(dst, &map_a, kb * BK, m0, full0 + 8 * s);
          tma_load_2d(dst + A_BYTES, mw, kb * BK, n0, full0 + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int it = 0, seg = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++seg) {
        const int buf = seg & 1;
        ok = mbar_wait(acce0 + 8 * buf, (((uint32_t)(seg >> 1)) & 1) ^ 1, 2, &g_status);      // the buffer was drained
        if (!ok) break;
        tc_fence_after();
        const uint32_t d = tmem + (uint32_t)(buf * BN);
        const uint32_t idesc = tile < wide_tiles ? IDESC : ((IDESC & ~(0x3fu << 17)) | ((uint32_t)(plan.narrow >> 3) << 17));
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(full0 + 8 * s, ((uint32_t)(it / STAGES)) & 1, 2, &g_status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
          const uint64_t da = smem_desc(a_addr), dw = smem_desc(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)     // 16 k-columns = 32 bytes further along the swizzled row
            tc_mma(d, da + (uint64_t)(2 * k), dw + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit(empty0 + 8 * s);            // arrives when these products no longer read the stage
        }
        if (ok) tc_commit(accf0 + 8 * buf);     // arrives when the accumulator is complete
      }
    }
  } else {
    // Epilogue: tensor memory -> registers -> swizzled staging tile -> TMA store (or TMA add into the float
    // residual stream: the addition happens at the memory side, nothing is read back here).
    const int quarter = warp & 3;               // the tensor-memory lanes this warp may read: 32 * (warp % 4)
    const int row = quarter * 32 + lane;
    const bool issuer = (warp == 2 && lane == 0);
    int seg = 0, chunk_no = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++seg) {
      int m0, n0, width;
      geometry(tile, m0, n0, width);
      const int chunks = MODE == GI_TC_QKV_ROPE ? 0 : width / CW;      // that mode has its own loop over the columns
      const int buf = seg & 1;
      ok = mbar_wait(accf0 + 8 * buf, ((uint32_t)(seg >> 1)) & 1, 3, &g_status);
      if (!ok) break;
      tc_fence_after();
      const uint32_t tbase = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN);
      if (MODE == GI_TC_QKV_ROPE) {
        // This thread's row is one token.  The tile is worked through in groups of 128 columns: one head of 128
        // values (its first half goes to staging tile A, its second to B) or two heads of 64 (one to each tile).
        // A value is rounded to bfloat16 as the plain store would round it, rotated in 32-bit with the token's
        // angles (the same function as the rotary kernels: the same bits), and rounded again.
        const int tok = m0 + row;
        const bool live = tok < M;
        const int hd = rope.hd, half = hd >> 1;
        size_t cache_tok = 0;       // this token's row of kv head 0 in the cache, in elements
        if (live && rope.write_cache) {
          const int pos = rope.positions[tok], slot = rope.slots[tok];
          const int page = slot >= 0 ? rope.block_table[(size_t)slot * rope.max_pages + pos / PAGE_TOKENS] : 0;
          cache_tok = ((size_t)page * rope.n_kv * PAGE_TOKENS + (pos % PAGE_TOKENS)) * hd;
        }
        const float2* cs = rope.table + (size_t)(live ? tok : 0) * half;
        const int heads_all = rope.n_heads + 2 * rope.n_kv;
        auto kind_of = [&](int head) { return head < rope.n_heads ? 0 : (head < rope.n_heads + rope.n_kv ? 1 : (head < heads_all ? 2 : 3)); };
        const int groups = width / 128;
#pragma unroll 1
        for (int gi_ = 0; gi_ < groups; ++gi_) {
          const int gcol = n0 + gi_ * 128;
          if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");    // both staging tiles are free again
          asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll 1
          for (int pass = 0; pass < 2; ++pass) {
            // head size 128: the head's pairs 32 pass .. 32 pass + 31; head size 64: head `pass` of the group
            const int lo_col = hd == 128 ? 32 * pass : 64 * pass, hi_col = lo_col + half;
            const int lo_dim = hd == 128 ? 32 * pass : 0;
            const int head = (gcol + lo_col) / hd;
            const int kind = kind_of(head);
            if (kind == 3) continue;                          // past the last head (the same for every thread)
            uint32_t lo[32], hi[32];
            tc_ld32(tbase + (uint32_t)(gi_ * 128 + lo_col), lo);
            tc_ld32(tbase + (uint32_t)(gi_ * 128 + hi_col), hi);
            tc_wait_ld();
            uint32_t plo[16], phi[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float a0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(lo[j]))), a1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(lo[j + 1])));
              float b0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(hi[j]))), b1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(hi[j + 1])));
              if (kind != 2 && live) {
                const float4 c2 = *reinterpret_cast<const float4*>(cs + lo_dim + j);    // two pairs' (cos, sin)
                gi::rotate_pair(a0, b0, make_float2(c2.x, c2.y), &a0, &b0);
                gi::rotate_pair(a1, b1, make_float2(c2.z, c2.w), &a1, &b1);
              }
              __nv_bfloat162 v = __floats2bfloat162_rn(a0, a1);
              plo[j / 2] = *reinterpret_cast<uint32_t*>(&v);
              v = __floats2bfloat162_rn(b0, b1);
              phi[j / 2] = *reinterpret_cast<uint32_t*>(&v);
            }
            if (kind == 0) {
              // head size 128: the first half's chunks 4 pass .. in tile A, the second half's in tile B;
              // head size 64: the head's eight chunks in tile A (pass 0) or B (pass 1)
              unsigned char* stg_lo = (hd == 128 || pass == 0) ? staging : staging + STG_BYTES;
              unsigned char* stg_hi = hd == 128 ? staging + STG_BYTES : stg_lo;
              const int c_lo = hd == 128 ? 4 * pass : 0, c_hi = hd == 128 ? 4 * pass : 4;
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                stage_chunk(stg_lo, row, c_lo + e, make_uint4(plo[4 * e], plo[4 * e + 1], plo[4 * e + 2], plo[4 * e + 3]));
                stage_chunk(stg_hi, row, c_hi + e, make_uint4(phi[4 * e], phi[4 * e + 1], phi[4 * e + 2], phi[4 * e + 3]));
              }
            } else if (live && rope.write_cache) {
              const int kvh = head - rope.n_heads - (kind == 2 ? rope.n_kv : 0);
              __nv_bfloat16* dst = (kind == 1 ? rope.kcache : rope.vcache) + cache_tok + (size_t)kvh * PAGE_TOKENS * hd;
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                *reinterpret_cast<uint4*>(dst + lo_dim + 8 * e) = make_uint4(plo[4 * e], plo[4 * e + 1], plo[4 * e + 2], plo[4 * e + 3]);
                *reinterpret_cast<uint4*>(dst + lo_dim + half + 8 * e) = make_uint4(phi[4 * e], phi[4 * e + 1], phi[4 * e + 2], phi[4 * e + 3]);
              }
            }
          }
          if (gi_ == groups - 1) {
            // the whole accumulator is in registers, staged or stored: hand the buffer back to the MMA thread
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce0 + 8 * buf);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // staged rows become visible to the TMA engine
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (issuer) {
            // tile A holds columns gcol .. gcol + 63, tile B the next 64: stored where they are queries
            if (kind_of(gcol / hd) == 0)
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(&map_o), "r"(smem_u32(staging)), "r"(gcol), "r"(m0) : "memory");
            if (kind_of((gcol + 64) / hd) == 0)
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(&map_o), "r"(smem_u32(staging + STG_BYTES)), "r"(gcol + 64), "r"(m0) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
      }
#pragma unroll 1
      for (int c = 0; c < chunks; ++c, ++chunk_no) {
        unsigned char* stg = staging + (chunk_no & 1) * STG_BYTES;
        // the TMA operation that last read this staging tile (two chunks ago) must be done with it
        if (issuer) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (int q = 0; q < CW / 32; ++q) {
          uint32_t r[32];
          tc_ld32(tbase + (uint32_t)(c * CW + q * 32), r);
          tc_wait_ld();
          if (MODE == GI_TC_SWIGLU) {
            // columns [8 gate | 8 up | 8 gate | 8 up] -> 16 activations = 32 bytes = chunks 2q, 2q + 1 of the row
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
              uint32_t p[4];
#pragma unroll
              for (int j = 0; j < 8; j += 2) {
                const float g0 = __uint_as_float(r[blk * 16 + j]), g1 = __uint_as_float(r[blk * 16 + j + 1]);
                const float u0 = __uint_as_float(r[blk * 16 + 8 + j]), u1 = __uint_as_float(r[blk * 16 + 8 + j + 1]);
                __nv_bfloat162 v = __floats2bfloat162_rn(gi::silu_mul_bf16(g0, u0), gi::silu_mul_bf16(g1, u1));
                p[j / 2] = *reinterpret_cast<uint32_t*>(&v);
              }
              stage_chunk(stg, row, q * 2 + blk, make_uint4(p[0], p[1], p[2], p[3]));
            }
          } else if (MODE == GI_TC_STORE_BF16) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint32_t p[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[j + 2 * e]), __uint_as_float(r[j + 2 * e + 1]));
                p[e] = *reinterpret_cast<uint32_t*>(&v);
              }
              stage_chunk(stg, row, q * 4 + j / 8, make_uint4(p[0], p[1], p[2], p[3]));
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; j += 4) stage_chunk(stg, row, j / 4, make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]));
          }
        }
        if (c == chunks - 1) {
          // the whole accumulator is in registers or staged: hand the buffer back to the MMA thread
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(acce0 + 8 * buf);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // staged rows become visible to the TMA engine
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (issuer) {
          const int x = (MODE == GI_TC_SWIGLU) ? (n0 + c * CW) / 2 : n0 + c * CW;   // in elements of the output
          const int limit = (MODE == GI_TC_SWIGLU) ? N / 2 : N;
          if (x < limit) {     // rows and columns past the matrix's edge are clipped by the TMA engine
            if (MODE == GI_TC_ACCUM_F32)
              asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(&map_o), "r"(smem_u32(stg)), "r"(x), "r"(m0) : "memory");
            else
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(&map_o), "r"(smem_u32(stg)), "r"(x), "r"(m0) : "memory");
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
    }
    if (issuer) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // every store has landed before the block leaves
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)(2 * BN)) : "memory");
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

// Tensor maps by (address, rows, columns, row stride, element, box): a map is pure data, and the same weights
// and the same activation buffers come back step after step.
}  // namespace

int gi::tensor_map_2d_ex(CUtensorMap* out, const void* base, long rows, long cols, long ld, int elem, int box_cols, int box_rows) {
  typedef std::tuple<const void*, long, long, long, int, int, int> Key;
  static std::map<Key, CUtensorMap> cache;
  static std::mutex lock;
  const Key key(base, rows, cols, ld, elem, box_cols, box_rows);
  std::lock_guard<std::mutex> guard(lock);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return GI_OK;
  }
  EncodeTiled enc = encoder();
  if (!enc) return gi::fail(GI_ERR_CUDA, "tensor-core product: the driver does not export cuTensorMapEncodeTiled");
  const int bytes = elem == GI_F32 ? 4 : 2;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * bytes};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, elem == GI_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return gi::fail(GI_ERR_CUDA, "tensor-core product: cuTensorMapEncodeTiled failed with %d", (int)r);
  if (cache.size() > 4096) cache.clear();
  cache[key] = *out;
  return GI_OK;
}

int gi::tensor_map_2d(CUtensorMap* out, const void* base, int rows, int cols, long ld, int box_rows) {
  return gi::tensor_map_2d_ex(out, base, rows, cols, ld, GI_BF16, BK, box_rows);
}

namespace {

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

// The cut of the output for BN-wide tiles on `sms` blocks.  Whole rounds of wide tiles first; if what is left would be
// a round that is not full, its columns are cut into narrower tiles (a multiple of `gran` columns, the epilogue's
// unit) of which one round holds all.
TilePlan plan_tiles(int M, int N, int bn, int gran, int sms) {
  const int tiles_m = (M + BM - 1) / BM, cols = (N + bn - 1) / bn;
  TilePlan p = {cols, 0, tiles_m * cols};
  const int per_round = sms / tiles_m;                  // column tiles one round of blocks holds
  if (bn != 256 || per_round < 1 || p.n_tiles <= sms || p.n_tiles % sms == 0) return p;
  const int rounds = p.n_tiles / sms;
  const int wide = (int)((long)rounds * sms / tiles_m);
  const int rest = N - wide * bn;
  if (wide >= cols || rest <= 0) return p;
  int narrow = ((rest + per_round - 1) / per_round + gran - 1) / gran * gran;
  if (narrow < 32) narrow = 32;
  if (narrow >= bn) return p;
  const int narrow_cols = (rest + narrow - 1) / narrow;
  p.wide_cols = wide;
  p.narrow = narrow;
  p.n_tiles = tiles_m * (wide + narrow_cols);
  return p;
}

template <int BN, int STAGES, int MODE>
int launch(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& mo, int M, int N, int K,
           const TilePlan& plan, const RopeEpilogue& rope, cudaStream_t s) {
  constexpr size_t smem = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 2 * BM * 128 + (2 * STAGES + 4) * 8 + 16 + 1024;
  auto kern = gemm_tc_kernel<BN, STAGES, MODE>;
  static bool configured[gi::MAX_DEVICES_SEEN] = {false};
  int dev;
  if (gi::unconfigured_here(configured, &dev)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "tensor-core product: %s", cudaGetErrorString(e));
    if (dev >= 0) configured[dev] = true;
  }
  const long tiles = plan.n_tiles;
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  return gi::check(gi::launch(kern, dim3(grid), dim3(THREADS), smem, s, ma, mw, mw2, mo, M, N, K, plan, rope), "tensor-core product");
}

template <int BN, int STAGES>
int launch_mode(int mode, const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& mo, int M, int N,
                int K, const TilePlan& plan, cudaStream_t s) {
  const RopeEpilogue none = {nullptr, nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0, 0, 0, 0};
  switch (mode) {
    case GI_TC_STORE_BF16: return launch<BN, STAGES, GI_TC_STORE_BF16>(ma, mw, mw2, mo, M, N, K, plan, none, s);
    case GI_TC_STORE_F32: return launch<BN, STAGES, GI_TC_STORE_F32>(ma, mw, mw2, mo, M, N, K, plan, none, s);
    case GI_TC_ACCUM_F32: return launch<BN, STAGES, GI_TC_ACCUM_F32>(ma, mw, mw2, mo, M, N, K, plan, none, s);
    case GI_TC_SWIGLU: return launch<BN, STAGES, GI_TC_SWIGLU>(ma, mw, mw2, mo, M, N, K, plan, none, s);
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
  CUtensorMap ma, mw, mo;
  int rc = gi::tensor_map_2d(&ma, A, M, K, lda, BM);
  if (rc != GI_OK) return rc;
  rc = gi::tensor_map_2d(&mw, W, N, K, ldw, tile_n);
  if (rc != GI_OK) return rc;
  // the output as the TMA engine sees it: rows of 128 bytes per box (32 floats or 64 bfloat16)
  const bool f32 = (mode == GI_TC_STORE_F32 || mode == GI_TC_ACCUM_F32);
  const long out_cols = mode == GI_TC_SWIGLU ? N / 2 : N;
  rc = gi::tensor_map_2d_ex(&mo, out, M, out_cols, ldo, f32 ? GI_F32 : GI_BF16, f32 ? 32 : 64, BM);
  if (rc != GI_OK) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const int gran = mode == GI_TC_SWIGLU ? 128 : (mode == GI_TC_STORE_BF16 ? 64 : 32);
  const TilePlan plan = g_tail_tiles ? plan_tiles(M, N, tile_n, gran, sm_count()) : plan_tiles(M, N, tile_n, gran, 0);
  CUtensorMap mw2 = mw;
  if (plan.narrow > 0) {
    rc = gi::tensor_map_2d(&mw2, W, N, K, ldw, plan.narrow);
    if (rc != GI_OK) return rc;
  }
  if (tile_n == 128) return launch_mode<128, 6>(mode, ma, mw, mw2, mo, M, N, K, plan, s);
  return launch_mode<256, 4>(mode, ma, mw, mw2, mo, M, N, K, plan, s);
}

// The q/k/v product of a prompt step with rotation and cache write in its epilogue: out[M, N] holds the packed rows,
// of which only the queries' columns are written (rotated); keys (rotated) and values go to the cache pages of each
// token's slot and position.  N = (n_heads + 2 n_kv) * hd, hd 64 or 128, all of a head rotated, pairs (i, i + hd / 2);
// table [M][hd / 2] (cos, sin).  The same bits as gi_gemm_tc_bf16 (GI_TC_STORE_BF16) followed by gi_rope_cache_write.
extern "C" int gi_gemm_tc_qkv_rope(void* out, const void* A, const void* W, int M, int N, int K, long lda, long ldw, long ldo,
                                   const float* table, const int* positions, const int* slots, const int* block_table,
                                   int max_pages, void* kcache, void* vcache, int n_heads, int n_kv, int hd, int write_cache,
                                   void* stream) {
  if (M <= 0 || N <= 0) return GI_OK;
  if (K <= 0 || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || ldo % 8 != 0)
    return gi::fail(GI_ERR_UNSUPPORTED, "q/k/v product: K (%d) and the row strides (%ld, %ld, %ld) must be multiples of 8", K, lda, ldw, ldo);
  if (((uintptr_t)A | (uintptr_t)W | (uintptr_t)out | (uintptr_t)table | (uintptr_t)kcache | (uintptr_t)vcache) & 15)
    return gi::fail(GI_ERR_UNSUPPORTED, "q/k/v product: operands must be 16-byte aligned");
  if (hd != 64 && hd != 128) return gi::fail(GI_ERR_UNSUPPORTED, "q/k/v product with rotation: head size %d, only 64 and 128", hd);
  if (n_heads <= 0 || n_kv <= 0 || N != (n_heads + 2 * n_kv) * hd)
    return gi::fail(GI_ERR_ARG, "q/k/v product with rotation: %d columns are not (%d + 2 x %d) heads of %d", N, n_heads, n_kv, hd);
  if (!table || !positions) return gi::fail(GI_ERR_ARG, "q/k/v product with rotation: no table of angles or no positions");
  if (write_cache && (!kcache || !vcache || !block_table || !slots)) return gi::fail(GI_ERR_ARG, "q/k/v product with rotation: cache write without a cache");
  if ((N + 255) / 256 > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "q/k/v product: too many tiles");
  CUtensorMap ma, mw, mo;
  int rc = gi::tensor_map_2d(&ma, A, M, K, lda, BM);
  if (rc != GI_OK) return rc;
  rc = gi::tensor_map_2d(&mw, W, N, K, ldw, 256);
  if (rc != GI_OK) return rc;
  rc = gi::tensor_map_2d_ex(&mo, out, M, N, ldo, GI_BF16, 64, BM);
  if (rc != GI_OK) return rc;
  // full-width tiles only: a narrower tile would cut a head
  const TilePlan plan = plan_tiles(M, N, 256, 64, 0);
  const RopeEpilogue rope = {(const float2*)table, positions, slots, block_table, max_pages, (__nv_bfloat16*)kcache,
                             (__nv_bfloat16*)vcache, n_heads, n_kv, hd, write_cache};
  return launch<256, 4, GI_TC_QKV_ROPE>(ma, mw, mw, mo, M, N, K, plan, rope, (cudaStream_t)stream);
}

// Switches the narrower tiles of an unfilled last round on (the default) or off; for measurements.
extern "C" int gi_gemm_tc_tail_tiles(int on) {
  g_tail_tiles = on != 0;
  return GI_OK;
}

// Reads and clears the status word of the tensor-core product (0 = every wait was met).  Synchronises the device.
extern "C" int gi_gemm_tc_status(int* status) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(status, g_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
  if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "tensor-core product status: %s", cudaGetErrorString(e));
  return GI_OK;
}
