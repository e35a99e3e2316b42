// Causal grouped-query attention of a step's prompt tokens over the paged cache on tcgen05 tensor cores
// (bfloat16, head size 64 or 128).
//
// Formula: src/model.rs:1320-1419.  The reference's prompt attention (attention_prefill_tc, src/cuda.rs:2408-2613)
// keeps scores in registers of mma.sync fragments; on sm_100a the same algorithm is laid out around tensor memory:
// a block takes 128 queries of one head.  One thread issues the TMA loads of the queries and of 64-key tiles of K
// (fetched page by page through the sequence's page table, two tiles ahead) and the score products S = Q K^T into
// one of two score buffers in tensor memory; another thread issues the loads of V and the output products
// O += P V, with P read from tensor memory and V in its stored (dimension-contiguous) layout.  Four warps own one
// query row per thread: they read a row of S with tcgen05.ld, keep the running maximum and sum in 32-bit (base-2
// exponentials), write the probabilities as bfloat16 over the scores they have just read (tcgen05.st), and
// rescale the accumulator in tensor memory when a row's reference point moves.  Two blocks share an SM, so one
// block's softmax overlaps the other's products.  Where that makes the launch one round of blocks (a prompt of 2,048
// tokens: 256 blocks on 296 places), a block takes two query tiles one after the other, the i-th from the end and
// the i-th from the start: under the causal mask every block then visits the same number of key tiles, instead of
// one full round and a ragged one.  Longer prompts keep one tile per block, longest first (measured: paired blocks
// are 10% slower at 8,192 tokens, where the many rounds even out by themselves).
// Every wait has an iteration limit and reports through a status word.
#include <cuda.h>
#include <math.h>

#include "api.h"
#include "common.cuh"
#include "tc_utils.cuh"

namespace {

using namespace gi::tc;

constexpr int BQ = 128;          // queries per block = tensor-memory lanes
constexpr int BKV = 64;          // keys per tile = one page
constexpr int THREADS = 192;     // warps 0-3: one query row per thread; warp 4: queries, keys and the score products;
                                 // warp 5: values and the output products
constexpr int TMEM_COLS = 256;   // two score buffers of 64 columns (tile j in buffer j & 1; its probabilities, two bfloat16 to a
                                 // column, take the buffer's first 32 columns once the scores are read), then O: head size columns
constexpr uint32_t Q_HALF = BQ * 128, KV_HALF = BKV * 128;   // a 64-dimension half of a tile: rows of 128 bytes, swizzled

__device__ int g_attn_status = 0;
int g_pairing = 1;      // two query tiles per block: 0 never, 1 when that gives one round of blocks, 2 always

__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31]) : "memory");
}
// 2^x in one instruction (32-bit, about 2 units in the last place): the softmax of this kernel is bound by the
// number of instructions per score, and its probabilities are rounded to bfloat16 right after.
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// D (+)= A B with A read from tensor memory: 128 lanes = rows, each 32-bit column two neighbouring bfloat16 of K.
__device__ __forceinline__ void tc_mma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Descriptor of an operand whose rows (the M or N side) are contiguous along that side ("MN-major"), stored as
// 64-element-wide, 128-byte-swizzled blocks: 8 rows of K are 1024 bytes apart (SBO), the next 64-wide block of the
// M/N side is `lbo_bytes` away.
__device__ __forceinline__ uint64_t smem_desc_mn(uint32_t addr, uint32_t lbo_bytes) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}

template <int HD>
__global__ void __launch_bounds__(THREADS, 2)
attn_prefill_t5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, long ldo,
                       const int* __restrict__ block_table, int max_pages, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ seq_slots, const int* __restrict__ seq_pos0, int n_heads, int n_kv, float scale,
                       int window, int q_tiles, int paired) {
  constexpr int HALVES = HD / 64;
  constexpr uint32_t Q_BYTES = HALVES * Q_HALF, KV_BYTES = HALVES * KV_HALF;
  // instruction descriptors: float accumulator, bfloat16 operands, M 128; S = Q K^T has N 64 and both operands K-major,
  // O = P V has N 128 and B (V) MN-major (bit 16)
  constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BKV >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
  constexpr uint32_t IDESC_O = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
  // Two blocks must fit one SM (2 x 113 KB at head size 128), which leaves no room for alignment slack: the tiles need 1024-byte
  // alignment, the dynamic shared memory of a kernel without static shared memory starts on such a boundary, and
  // the block checks that before it does anything.
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* q_s = smem;                              // [halves][128 rows][64 dims]
  unsigned char* k_s = q_s + Q_BYTES;                     // [2 stages][halves][64 keys][64 dims]
  unsigned char* v_s = k_s + 2 * KV_BYTES;                // the same
  uint64_t* bars = (uint64_t*)(v_s + 2 * KV_BYTES);       // q_full, k_full[2], v_full[2], kv_empty[2], s_full[2], p_full[2], o_full
  uint32_t* tmem_slot = (uint32_t*)(bars + 12);

  // Blocks start in the order x, y, z: heads fastest (the heads of a group read the same keys and values at the
  // same time), then sequences, then query tiles from the latest down: the blocks with the most keys to visit start
  // first, for every head and sequence of the launch, and the short ones fill the gaps at the end.
  const int h = blockIdx.x, b = blockIdx.y;
  const int tok0 = cu_seqlens[b], qlen = cu_seqlens[b + 1] - tok0;
  // the block's two query tiles: the later one first (it has the most keys to visit), then its mirror from the start
  // (not paired: the later one only)
  const int tile_a = q_tiles - 1 - (int)blockIdx.z, tile_b = paired ? (int)blockIdx.z : tile_a;
  if (tile_b * BQ >= qlen) return;                         // the earlier tile lies past this sequence: so does the later one
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicCAS(&g_attn_status, 0, 9);
    return;
  }
  const int slot = seq_slots[b], pos0 = seq_pos0[b];
  const int kvh = h / (n_heads / n_kv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const uint32_t bar0 = smem_u32(bars);
  const uint32_t q_full = bar0, k_full0 = bar0 + 8, v_full0 = bar0 + 24, kv_empty0 = bar0 + 40;
  // The probabilities' barrier is one per score buffer, not one for both: a row warp may be a whole tile ahead of
  // another (one that rescales the accumulator, or zeroes values at a tile's edge, while the others do not), and with
  // one barrier its arrival for tile j + 1 would have counted as the slow warp's for tile j: the output product would
  // have started without that warp's probabilities, and the count would have been one off from then on.  On the
  // buffer's own barrier nobody can be a tile ahead: tile j + 2 needs the buffer back, which needs tile j's product.
  const uint32_t s_full0 = bar0 + 56, p_full0 = bar0 + 72, o_full = bar0 + 88;

  auto init_barriers = [&](bool again) {
    if (again)                                             // the objects of the tile before are no longer in use
      for (int i = 0; i < 12; ++i) asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar0 + 8 * i) : "memory");
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full0 + 8 * s, 1);
      mbar_init(v_full0 + 8 * s, 1);
      mbar_init(kv_empty0 + 8 * s, 1);
    }
    mbar_init(s_full0, 1);
    mbar_init(s_full0 + 8, 1);
    mbar_init(p_full0, 4);
    mbar_init(p_full0 + 8, 4);
    mbar_init(o_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  };
  if (threadIdx.x == 0) init_barriers(false);
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_s = tmem, tmem_o = tmem + 128;
  gi::pdl_prologue();      // set-up overlapped the previous kernel's end; its results are visible from here on

  bool first_pass = true;
  for (int pass = 0; pass < 2; ++pass) {
  const int q_tile = pass == 0 ? tile_a : tile_b;
  if (pass == 1 && tile_b == tile_a) break;                // an odd count's middle tile has no mirror
  const int q0 = q_tile * BQ;
  if (q0 >= qlen) continue;                                // (uniform over the block)
  if (!first_pass) {
    // everybody is done with the tile before (its output is read out of tensor memory): fresh barriers for this one
    if (threadIdx.x == 0) init_barriers(true);
    __syncthreads();
  }
  first_pass = false;
  const int rows_here = min(BQ, qlen - q0);
  const int p_last = pos0 + q0 + rows_here - 1;
  int t_first = 0;
  if (window > 0) t_first = max(0, pos0 + q0 - window + 1);
  const int kt_begin = (t_first / BKV) * BKV;
  const int n_tiles = (p_last - kt_begin) / BKV + 1;

  // Two threads issue the products, each with its own loads, so that neither chain waits behind the other's
  // barriers: S(j+1) = Q K(j+1)^T wants only the keys and the score buffer back (the rows of S(j) read into
  // registers), O += P(j) V(j) wants the probabilities staged.  One thread for both spent half a tile's time in
  // the one chain's waits while the other chain was ready.
  auto row_of = [&](int tile) {        // where a tile's keys and values lie: the page comes from the sequence's page table
    const int kt = kt_begin + tile * BKV;
    const int page = block_table[(size_t)slot * max_pages + kt / PAGE_TOKENS];
    return (page * n_kv + kvh) * PAGE_TOKENS;
  };
  if (warp == 4) {
    if (lane == 0) {
      bool ok = true;
      auto load_k = [&](int tile) {
        const int s = tile & 1, row0 = row_of(tile);
        mbar_expect_tx(k_full0 + 8 * s, KV_BYTES);
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf) tma_load_2d(smem_u32(k_s + s * KV_BYTES + hf * KV_HALF), &map_k, hf * 64, row0, k_full0 + 8 * s);
      };
      mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int hf = 0; hf < HALVES; ++hf) tma_load_2d(smem_u32(q_s + hf * Q_HALF), &map_q, h * HD + hf * 64, tok0 + q0, q_full);
      load_k(0);
      if (n_tiles > 1) load_k(1);
      ok = mbar_wait(q_full, 0, 1, &g_attn_status);
      // the operands' descriptors do not change from tile to tile (but for the stage): made once
      uint64_t dq[HD / 16], dk[2][HD / 16];
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        dq[ks] = smem_desc(smem_u32(q_s) + (ks / 4) * Q_HALF + (ks % 4) * 32);
        dk[0][ks] = smem_desc(smem_u32(k_s) + (ks / 4) * KV_HALF + (ks % 4) * 32);
        dk[1][ks] = smem_desc(smem_u32(k_s) + KV_BYTES + (ks / 4) * KV_HALF + (ks % 4) * 32);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        // the keys are here, and this score buffer is free: the output product of tile j - 2, which read its
        // probabilities from it, is done (the barrier that frees that tile's values says so)
        ok = mbar_wait(k_full0 + 8 * s, (uint32_t)((j >> 1) & 1), 2, &g_attn_status);
        if (ok && j >= 2) ok = mbar_wait(kv_empty0 + 8 * s, (uint32_t)(((j - 2) >> 1) & 1), 2, &g_attn_status);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) tc_mma(tmem_s + (uint32_t)(s * 64), dq[ks], s ? dk[1][ks] : dk[0][ks], IDESC_S, ks > 0 ? 1u : 0u);
        tc_commit(s_full0 + 8 * s);
        // keys two tiles ahead go into this tile's stage as soon as its scores are complete: a whole tile's softmax
        // before they are wanted
        if (j + 2 < n_tiles) {
          ok = mbar_wait(s_full0 + 8 * s, (uint32_t)((j >> 1) & 1), 2, &g_attn_status);
          if (!ok) break;
          load_k(j + 2);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      bool ok = true;
      auto load_v = [&](int tile) {
        const int s = tile & 1, row0 = row_of(tile);
        mbar_expect_tx(v_full0 + 8 * s, KV_BYTES);
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf) tma_load_2d(smem_u32(v_s + s * KV_BYTES + hf * KV_HALF), &map_v, hf * 64, row0, v_full0 + 8 * s);
      };
      load_v(0);
      if (n_tiles > 1) load_v(1);
      uint64_t dv[2][BKV / 16];
#pragma unroll
      for (int kk = 0; kk < BKV / 16; ++kk) {
        dv[0][kk] = smem_desc_mn(smem_u32(v_s) + kk * 2048, KV_HALF);
        dv[1][kk] = smem_desc_mn(smem_u32(v_s) + KV_BYTES + kk * 2048, KV_HALF);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        // O += P V once the probabilities are staged (which also says: O has been rescaled) and the values are here
        ok = mbar_wait(p_full0 + 8 * s, (uint32_t)((j >> 1) & 1), 2, &g_attn_status);
        if (ok) ok = mbar_wait(v_full0 + 8 * s, (uint32_t)((j >> 1) & 1), 2, &g_attn_status);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk)      // 16 keys of the probabilities = 8 columns of the tile's score buffer
          tc_mma_a_tmem(tmem_o, tmem_s + (uint32_t)(s * 64 + kk * 8), s ? dv[1][kk] : dv[0][kk], IDESC_O, (j > 0 || kk > 0) ? 1u : 0u);
        // `o_full` first: the barrier asked last by the row warps (the stage's, at the end of the tile loop) is then the
        // one whose arrival is issued last, and no arrival can still be on its way when the barriers are made anew
        // for the block's second query tile
        tc_commit(o_full);
        tc_commit(kv_empty0 + 8 * s);
        // values two tiles ahead go into this tile's stage once this product no longer reads it
        if (j + 2 < n_tiles) {
          ok = mbar_wait(kv_empty0 + 8 * s, (uint32_t)((j >> 1) & 1), 1, &g_attn_status);
          if (!ok) break;
          load_v(j + 2);
        }
      }
    }
  } else {
    const int row = warp * 32 + lane;                 // query row = tensor-memory lane
    const int p_row = pos0 + q0 + row;                // its position
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const float sl2 = scale * 1.4426950408889634f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j & 1;
      const int kt = kt_begin + j * BKV;
      ok = mbar_wait(s_full0 + 8 * s, (uint32_t)((j >> 1) & 1), 3, &g_attn_status);
      if (!ok) break;
      tc_fence_after();
      const uint32_t my_s = tmem_s + lane_base + (uint32_t)(s * 64);
      uint32_t sr[2][32];
      tc_ld32(my_s, sr[0]);
      tc_ld32(my_s + 32, sr[1]);
      tc_wait_ld();
      // scores -> probabilities.  A tile every row of the block sees in full needs no mask: one maximum, then one
      // fused multiply-add, one exponential and one addition per score.  Tiles on the diagonal (or at a window's
      // edge) take the masked path.
      const bool interior = (kt + BKV - 1 <= pos0 + q0) && kt >= t_first && (window <= 0 || kt > pos0 + q0 + BQ - 1 - window);
      float tmax = -INFINITY;
      if (interior) {
#pragma unroll
        for (int q = 0; q < 2; ++q)
#pragma unroll
          for (int c = 0; c < 32; ++c) tmax = fmaxf(tmax, __uint_as_float(sr[q][c]));
        tmax *= sl2;
      } else {
#pragma unroll
        for (int q = 0; q < 2; ++q)
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int key = kt + q * 32 + c;
            const bool vis = key <= p_row && key >= t_first && (window <= 0 || key > p_row - window);
            const float v = vis ? __uint_as_float(sr[q][c]) : -INFINITY;
            sr[q][c] = __float_as_uint(v);
            tmax = fmaxf(tmax, v * sl2);
          }
      }
      // The reference point of the exponentials moves only when the row's maximum has grown by more than 2^8 since
      // it was set: probabilities may then exceed 1 (by at most 2^8, harmless in bfloat16 and float), and the
      // accumulator in tensor memory is rescaled rarely instead of at every new maximum.  The result O / l does not
      // depend on the reference point.
      float alpha = 1.0f;
      if (m_run == -INFINITY || tmax > m_run + 8.0f) {
        const float m_new = fmaxf(m_run, tmax);
        alpha = (m_run == -INFINITY) ? 0.f : ex2(m_run - m_new);
        m_run = m_new;
      }
      const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
      float psum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int q = 0; q < 2; ++q)
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          // a masked score is -inf: -inf * sl2 - m = -inf, and 2^-inf = 0
          const float p0 = ex2(fmaf(__uint_as_float(sr[q][c]), sl2, neg_m)), p1 = ex2(fmaf(__uint_as_float(sr[q][c + 1]), sl2, neg_m));
          psum += p0 + p1;
          __nv_bfloat162 pv = __floats2bfloat162_rn(p0, p1);
          pk[q * 16 + c / 2] = *reinterpret_cast<uint32_t*>(&pv);
        }
      l_run = l_run * alpha + psum;
      // The accumulator is rescaled only when some row of the warp moved its reference point (rare): then the
      // previous output product must be done first.  Nothing else here waits for it: the probabilities go into
      // this tile's own score buffer, which no product reads before they are announced.
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
        ok = mbar_wait(o_full, (uint32_t)((j - 1) & 1), 3, &g_attn_status);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t orow[32];
          tc_ld32(tmem_o + lane_base + c * 32, orow);
          tc_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) orow[e] = __float_as_uint(__uint_as_float(orow[e]) * alpha);
          tc_st32(tmem_o + lane_base + c * 32, orow);
        }
        tc_wait_st();
      }
      // the row of probabilities: 64 bfloat16, two to a column, over the first 32 columns of the scores just read
      tc_st32(my_s, pk);
      tc_wait_st();
      // keys of this tile that no row of the block may see (past the block's last position, or before every window)
      // get zero values: their probabilities are zero, but zero times a stale non-number would still be a non-number
      const int lo = max(0, t_first - kt), hi = min(BKV, p_last + 1 - kt);
      if (lo > 0 || hi < BKV) {
        ok = mbar_wait(v_full0 + 8 * s, (uint32_t)((j >> 1) & 1), 3, &g_attn_status);
        if (!ok) break;
        unsigned char* vt = v_s + s * KV_BYTES;
        for (int idx = threadIdx.x; idx < BKV * (HD / 8); idx += 128) {
          const int r = idx / (HD / 8), cidx = idx % (HD / 8);   // key row, 16-byte chunk of the row (its halves lie apart)
          if (r < lo || r >= hi) *reinterpret_cast<uint4*>(vt + (cidx / 8) * KV_HALF + r * 128 + (cidx % 8) * 16) = make_uint4(0, 0, 0, 0);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full0 + 8 * s);
    }
    // The last output product is done when the barrier that frees its stage of values says so.  That barrier belongs
    // to one stage: it completes a phase every second tile, and the phase before the awaited one (tile n - 3's) is known
    // to be complete, since the scores of tile n - 1 were not issued before it.  `o_full`, which completes a phase
    // at every tile, cannot be asked here: a warp that has finished its last tile while another is still two tiles back
    // finds it two phases behind, and a wait by parity takes that for the awaited phase: the warp then read its rows
    // of the output before the last two products had added to them (seen as one warp's rows wrong, once in some
    // dozens of launches with few tiles per block).  During the loop `o_full` is safe: at tile j the product of tile
    // j - 2 is known to be done, so the barrier is at most one phase behind.
    if (ok) ok = mbar_wait(kv_empty0 + 8 * ((n_tiles - 1) & 1), (uint32_t)(((n_tiles - 1) >> 1) & 1), 3, &g_attn_status);
    tc_fence_after();
    if (ok) {
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      __nv_bfloat16* orow_g = out + (size_t)(tok0 + q0 + row) * ldo + (size_t)h * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t orow[32];
        tc_ld32(tmem_o + lane_base + c * 32, orow);
        tc_wait_ld();
        if (row < rows_here) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint32_t pkd[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              __nv_bfloat162 v2 = __floats2bfloat162_rn(__uint_as_float(orow[e + 2 * u]) * inv, __uint_as_float(orow[e + 2 * u + 1]) * inv);
              pkd[u] = *reinterpret_cast<uint32_t*>(&v2);
            }
            *reinterpret_cast<uint4*>(orow_g + c * 32 + e) = make_uint4(pkd[0], pkd[1], pkd[2], pkd[3]);
          }
        }
        __syncwarp();
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  }  // the block's two query tiles
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS) : "memory");
  }
}

template <int HD>
int launch_t5(dim3 grid, cudaStream_t stream, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, __nv_bfloat16* out,
              long ldo, const int* block_table, int max_pages, const int* cu_seqlens, const int* seq_slots, const int* seq_pos0,
              int n_heads, int n_kv, float scale, int window, int q_tiles, int paired) {
  constexpr size_t smem = (HD / 64) * (Q_HALF + 4 * KV_HALF) + 12 * 8 + 16;
  static bool configured[gi::MAX_DEVICES_SEEN] = {false};
  int dev;
  if (gi::unconfigured_here(configured, &dev)) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_t5_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "attention prefill (tcgen05): %s", cudaGetErrorString(e));
    if (dev >= 0) configured[dev] = true;
  }
  return gi::check(gi::launch(attn_prefill_t5_kernel<HD>, grid, dim3(THREADS), smem, stream, mq, mk, mv, out, ldo, block_table, max_pages,
                              cu_seqlens, seq_slots, seq_pos0, n_heads, n_kv, scale, window, q_tiles, paired),
                   "attention prefill (tcgen05)");
}

}  // namespace

extern "C" int gi_attn_prefill_t5(void* out, long ldo, const void* q, long ldq, long q_rows, const void* kcache,
                                  const void* vcache, long cache_pages, const int* block_table, int max_pages,
                                  const int* cu_seqlens, const int* seq_slots, const int* seq_pos0, int n_seqs,
                                  int max_q_len, int n_heads, int n_kv, int hd, float scale, int window, void* stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return GI_OK;
  if (hd != 64 && hd != 128) return gi::fail(GI_ERR_UNSUPPORTED, "attention prefill (tcgen05): head size %d, only 64 and 128", hd);
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0)
    return gi::fail(GI_ERR_ARG, "attention: %d heads do not divide into %d kv heads", n_heads, n_kv);
  if (ldq % 8 != 0 || ldo % 8 != 0 || (((uintptr_t)q | (uintptr_t)kcache | (uintptr_t)vcache | (uintptr_t)out) & 15))
    return gi::fail(GI_ERR_UNSUPPORTED, "attention prefill (tcgen05): rows must be 16-byte aligned");
  if (n_seqs > 65535 || (max_q_len + BQ - 1) / BQ > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "attention: more than 65535 sequences or query tiles in one launch");
  CUtensorMap mq, mk, mv;
  int rc = gi::tensor_map_2d_ex(&mq, q, q_rows, (long)(n_heads + 2 * n_kv) * hd, ldq, GI_BF16, 64, BQ);
  if (rc != GI_OK) return rc;
  const long cache_rows = cache_pages * n_kv * PAGE_TOKENS;
  if (cache_rows > 0x7fffffffL || q_rows > 0x7fffffffL)       // TMA coordinates are 32-bit
    return gi::fail(GI_ERR_UNSUPPORTED, "attention prefill (tcgen05): more than 2^31 - 1 rows of queries or of cached keys");
  rc = gi::tensor_map_2d_ex(&mk, kcache, cache_rows, hd, hd, GI_BF16, 64, BKV);
  if (rc != GI_OK) return rc;
  rc = gi::tensor_map_2d_ex(&mv, vcache, cache_rows, hd, hd, GI_BF16, 64, BKV);
  if (rc != GI_OK) return rc;
  const int q_tiles = (max_q_len + BQ - 1) / BQ;
  // two query tiles per block where that makes the launch a single round of blocks (two blocks per SM)
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long paired_blocks = (long)n_heads * n_seqs * ((q_tiles + 1) / 2);
  const int paired = (g_pairing != 0 && q_tiles > 1 && (g_pairing == 2 || paired_blocks <= 2L * (sms > 0 ? sms : 148))) ? 1 : 0;
  dim3 grid(n_heads, n_seqs, paired ? (q_tiles + 1) / 2 : q_tiles);
  if (hd == 128)
    return launch_t5<128>(grid, (cudaStream_t)stream, mq, mk, mv, (__nv_bfloat16*)out, ldo, block_table, max_pages, cu_seqlens, seq_slots,
                          seq_pos0, n_heads, n_kv, scale, window, q_tiles, paired);
  return launch_t5<64>(grid, (cudaStream_t)stream, mq, mk, mv, (__nv_bfloat16*)out, ldo, block_table, max_pages, cu_seqlens, seq_slots,
                       seq_pos0, n_heads, n_kv, scale, window, q_tiles, paired);
}

// Query tiles two to a block: 0 never, 1 where the launch then is one round of blocks (default), 2 always; for
// measurements and tests.
extern "C" int gi_attn_prefill_t5_pairing(int mode) {
  g_pairing = mode;
  return GI_OK;
}

extern "C" int gi_attn_prefill_t5_status(int* status) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(status, g_attn_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_attn_status, &zero, sizeof(int));
  if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "attention prefill status: %s", cudaGetErrorString(e));
  return GI_OK;
}
