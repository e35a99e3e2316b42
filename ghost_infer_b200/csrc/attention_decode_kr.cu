// Decode attention over the paged cache with the keys on the rows of the tensor-core tile: one token per sequence,
// bfloat16, head size 64 or 128.
//
// The same operation and the same cut of the work as attention_decode_tc.cu (src/model.rs:1320-1419; a block takes one
// kv head of one sequence and one slice of its context, src/cuda.rs:1684-1865), with the two products turned
// around.  There the group's query heads are the 16 rows of an m16n8k16 tile, of which a group of 4 heads uses 4.
// Here a tile of 16 keys is the rows and up to 8 heads are the columns:
//   S^T[16 keys x 8 heads] = K[16 x hd] Q^T[hd x 8]          hd / 16 products a tile instead of hd / 8
//   O^T[hd x 8 heads]     += V^T[hd x 16] P^T[16 x 8]          hd / 16 products a tile instead of hd / 8
// P^T comes out of the first product with a thread holding (key g, heads 2t, 2t + 1) and goes into the second with
// (keys 2t, 2t + 1, head g): one movmatrix per 8 keys turns it.  A thread then holds two heads' scores of two keys:
// half the exponentials, a quarter of the masks, half the accumulators of the other layout, which leaves registers for
// more warps per SM.  Per-head maxima run over lanes of equal t (three exchanges); the per-head sums stay per thread
// until the end.  Everything else is as in the other kernel: keys and values by cp.async into per-warp rings of
// swizzled stages, the first tiles requested before the dependency wait, warps merged through shared memory in warp
// order, slices left to gi_attn_combine in slice order.
#include <math.h>

#include "api.h"
#include "common.cuh"
#include "mma_utils.cuh"

namespace {

constexpr int KT = 16;       // keys per tile
constexpr int COLS = 8;      // heads per block: the columns of the tile

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

template <int HD, int WARPS, int STAGES>
__global__ void __launch_bounds__(WARPS * 32)
attn_decode_kr_kernel(__nv_bfloat16* __restrict__ out, long ldo, float* __restrict__ part_o, float* __restrict__ part_ml,
                      const __nv_bfloat16* q /* written by the kernel before: see gi::pdl_wait */, long ldq,
                      const __nv_bfloat16* __restrict__ kcache, const __nv_bfloat16* __restrict__ vcache,
                      const int* __restrict__ block_table, int max_pages, const int* __restrict__ seq_slots,
                      const int* __restrict__ seq_lens, int n_heads, int n_kv, float scale, int window, int n_splits,
                      int own_tiles) {
  constexpr int CH = HD / 8;                     // 16-byte chunks per row
  constexpr int TILE_BYTES = KT * HD * 2;        // one K or V tile
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;    // K then V
  constexpr int MT = HD / 16;                    // 16-dim row tiles of O^T, and 16-dim steps of S^T
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* q_s = smem;                                       // [8][HD] bf16, swizzled
  unsigned char* ring = smem + COLS * HD * 2;                      // [WARPS][STAGES][K tile | V tile]
  // Lengths, slots and the block table were uploaded before the step's first kernel, and no kernel of the step
  // writes a cached position other than each sequence's last one: the first tiles are requested before the
  // dependency wait; only the tile that holds the last position waits.
  gi::pdl_launch_dependents();

  const int group = n_heads / n_kv;
  const int chunks = (group + COLS - 1) / COLS;
  const int b = blockIdx.z, kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks, sp = blockIdx.x;
  const int g0 = chunk * COLS, gcount = min(COLS, group - g0);
  const int h0 = kvh * group + g0;
  const int slot = gi::ld_step(seq_slots + b);
  const int len = gi::ld_step(seq_lens + b);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  int t_first = 0;
  if (window > 0) t_first = max(0, len - window);
  const int t_base = (t_first / KT) * KT;
  const int tiles = len > t_base ? (len - t_base + KT - 1) / KT : 0;
  const int per = own_tiles > 0 ? own_tiles : (tiles + n_splits - 1) / n_splits;
  const int used = per > 0 ? max(1, (tiles + per - 1) / per) : 1;      // slices of this sequence that hold keys
  const int tile_lo = sp * per, tile_hi = min(tiles, tile_lo + per);
  if (sp >= used) {
    // nothing of this sequence lies in this slice: the combine kernel must find it marked empty
    if (n_splits > 1) {
      for (int r = threadIdx.x; r < gcount; r += WARPS * 32) {
        const size_t pi = ((size_t)b * n_heads + h0 + r) * n_splits + sp;
        part_ml[pi * 2] = -INFINITY;
        part_ml[pi * 2 + 1] = 0.f;
      }
    }
    return;
  }

  unsigned char* my_ring = ring + (size_t)warp * STAGES * STAGE_BYTES;
  const float sl2 = scale * 1.4426950408889634f;

  auto issue = [&](int tile, int stage) {
    const int t0 = t_base + tile * KT;
    const int page = slot >= 0 ? gi::ld_step(block_table + (size_t)slot * max_pages + t0 / PAGE_TOKENS) : 0;
    const size_t base = (((size_t)page * n_kv + kvh) * PAGE_TOKENS + (t0 % PAGE_TOKENS)) * HD;
    unsigned char* ks = my_ring + (size_t)stage * STAGE_BYTES;
    unsigned char* vs = ks + TILE_BYTES;
#pragma unroll
    for (int i = 0; i < KT * CH / 32; ++i) {
      const int idx = i * 32 + lane;
      const int r = idx / CH, c = idx % CH;
      const int ok = (t0 + r < len && t0 + r >= t_first) ? 16 : 0;   // rows outside the visible span are zero-filled, not read
      const size_t off = base + (size_t)(ok ? r : 0) * HD + c * 8;
      gi::cp_async_16(gi::smem_u32(ks + gi::swz<CH>(r, c)), kcache + off, ok);
      gi::cp_async_16(gi::smem_u32(vs + gi::swz<CH>(r, c)), vcache + off, ok);
    }
  };

  // per thread: heads 2t and 2t + 1 (index j), keys g and g + 8 of a tile
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[MT][4];                      // O^T: [0], [1] dim 16 mt + g of heads 2t, 2t + 1; [2], [3] dim 16 mt + g + 8
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[i][c] = 0.f;

  // prologue: STAGES - 1 tiles in flight; the tile with the sequence's last position only after the wait
  int next = tile_lo + warp;
  int late_stage = -1;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (next < tile_hi) {
      if (next == tiles - 1) late_stage = s;
      else issue(next, s);
    }
    gi::cp_async_commit();
    next += WARPS;
  }
  gi::pdl_wait();
  if (late_stage >= 0) {          // a short slice: its last tile is among the first ones; fetch it now and let it land
    issue(tiles - 1, late_stage);
    gi::cp_async_commit();
    gi::cp_async_wait<0>();
  }
  // queries of the block's heads as rows 0..gcount-1 of an 8-row tile (the others zero)
  for (int idx = tid; idx < COLS * CH; idx += WARPS * 32) {
    const int r = idx / CH, c = idx % CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < gcount) v = *reinterpret_cast<const uint4*>(q + (size_t)b * ldq + (size_t)(h0 + r) * HD + c * 8);
    *reinterpret_cast<uint4*>(q_s + gi::swz<CH>(r, c)) = v;
  }
  __syncthreads();
  // Q^T as the second operand: for 32 dims at a time, four 8x8 matrices (heads 0-7, dims +0, +8, +16, +24)
  uint32_t qb[HD / 32][4];
#pragma unroll
  for (int kp = 0; kp < HD / 32; ++kp) gi::ldmatrix_x4(qb[kp], gi::smem_u32(q_s + gi::swz<CH>(lane & 7, kp * 4 + (lane >> 3))));

  int stage = 0;
  for (int tile = tile_lo + warp; tile < tile_hi; tile += WARPS) {
    // keep the ring full, then wait for the oldest tile
    if (next < tile_hi) issue(next, (stage + STAGES - 1) % STAGES);
    gi::cp_async_commit();
    next += WARPS;
    gi::cp_async_wait<STAGES - 1>();
    __syncwarp();
    const unsigned char* ks = my_ring + (size_t)stage * STAGE_BYTES;
    const unsigned char* vs = ks + TILE_BYTES;
    const int t0 = t_base + tile * KT;

    // S^T = K Q^T: rows are the tile's 16 keys
    float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int kk = 0; kk < MT; ++kk) {
      // matrices: (keys 0-7, dims lo), (keys 8-15, dims lo), (keys 0-7, dims hi), (keys 8-15, dims hi)
      uint32_t ka[4];
      gi::ldmatrix_x4(ka, gi::smem_u32(ks + gi::swz<CH>((lane & 7) + ((lane >> 3) & 1) * 8, kk * 2 + (lane >> 4))));
      gi::mma_16816(s, ka, qb[kk >> 1][(kk & 1) * 2], qb[kk >> 1][(kk & 1) * 2 + 1]);
    }
    // mask (two keys per thread) and running softmax (two heads per thread)
    const bool ok0 = t0 + g < len && t0 + g >= t_first, ok1 = t0 + g + 8 < len && t0 + g + 8 >= t_first;
    s[0] = ok0 ? s[0] * sl2 : -INFINITY;
    s[1] = ok0 ? s[1] * sl2 : -INFINITY;
    s[2] = ok1 ? s[2] * sl2 : -INFINITY;
    s[3] = ok1 ? s[3] * sl2 : -INFINITY;
    float alpha[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float tmax = fmaxf(s[j], s[2 + j]);
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 8));
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 16));
      const float m_new = fmaxf(m_run[j], tmax);          // finite: every tile holds at least one live key
      alpha[j] = (m_run[j] == -INFINITY) ? 0.f : exp2f(m_run[j] - m_new);
      m_run[j] = m_new;
    }
    const float p0 = exp2f(s[0] - m_run[0]), p1 = exp2f(s[1] - m_run[1]);
    const float p2 = exp2f(s[2] - m_run[0]), p3 = exp2f(s[3] - m_run[1]);
    l_run[0] = l_run[0] * alpha[0] + (p0 + p2);           // this thread's keys only; lanes are added at the end
    l_run[1] = l_run[1] * alpha[1] + (p1 + p3);
    // P^T from (key g, heads 2t, 2t + 1) to (keys 2t, 2t + 1, head g)
    const uint32_t pb0 = movmatrix_trans(gi::pack_bf16(p0, p1)), pb1 = movmatrix_trans(gi::pack_bf16(p2, p3));
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[1];
      o[i][2] *= alpha[0];
      o[i][3] *= alpha[1];
    }
    // O^T += V^T P^T: rows are 16 dims of the head
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      // transposed matrices: (keys 0-7, dims lo), (keys 0-7, dims hi), (keys 8-15, dims lo), (keys 8-15, dims hi)
      uint32_t va[4];
      gi::ldmatrix_x4_trans(va, gi::smem_u32(vs + gi::swz<CH>((lane & 7) + (lane >> 4) * 8, mt * 2 + ((lane >> 3) & 1))));
      gi::mma_16816(o[mt], va, pb0, pb1);
    }
    __syncwarp();
    stage = (stage + 1) % STAGES;
  }
  gi::cp_async_wait<0>();
  // the sums over this warp's keys: lanes of equal t hold the same two heads
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    l_run[j] += __shfl_xor_sync(0xffffffffu, l_run[j], 4);
    l_run[j] += __shfl_xor_sync(0xffffffffu, l_run[j], 8);
    l_run[j] += __shfl_xor_sync(0xffffffffu, l_run[j], 16);
  }
  __syncthreads();

  // merge the warps (reusing the ring): natural-log maxima so that the combine kernel can go on
  constexpr int MROW = HD + 8;
  float* Mo = reinterpret_cast<float*>(ring);            // [WARPS][8][MROW]
  float* Mm = Mo + WARPS * COLS * MROW;                  // [WARPS][8]
  float* Ml = Mm + WARPS * COLS;                         // [WARPS][8]
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int r = 2 * t + j;
    if (r >= gcount) continue;
    if (g == 0) {
      Mm[warp * COLS + r] = m_run[j];
      Ml[warp * COLS + r] = l_run[j];
    }
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      Mo[(warp * COLS + r) * MROW + i * 16 + g] = o[i][j];
      Mo[(warp * COLS + r) * MROW + i * 16 + g + 8] = o[i][2 + j];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < gcount * HD; idx += WARPS * 32) {
    const int r = idx / HD, d = idx % HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, Mm[w * COLS + r]);
    float tot = 0.f, val = 0.f;
    if (mm != -INFINITY) {
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float mw = Mm[w * COLS + r];
        if (mw == -INFINITY) continue;
        const float wgt = exp2f(mw - mm);
        tot += Ml[w * COLS + r] * wgt;
        val += Mo[(w * COLS + r) * MROW + d] * wgt;
      }
    }
    const int h = h0 + r;
    if (n_splits == 1) {
      out[(size_t)b * ldo + (size_t)h * HD + d] = __float2bfloat16_rn(tot > 0.f ? val / tot : 0.f);
    } else {
      const size_t pi = ((size_t)b * n_heads + h) * n_splits + sp;
      part_o[pi * HD + d] = val;
      if (d == 0) {
        part_ml[pi * 2] = mm * 0.6931471805599453f;      // back to natural-log units
        part_ml[pi * 2 + 1] = tot;
      }
    }
  }
}

template <int HD, int WARPS, int STAGES>
int launch(dim3 grid, cudaStream_t s, __nv_bfloat16* out, long ldo, float* po, float* pml, const __nv_bfloat16* q, long ldq,
           const __nv_bfloat16* kc, const __nv_bfloat16* vc, const int* bt, int max_pages, const int* slots, const int* lens,
           int H, int KV, float scale, int window, int n_splits, int own_tiles) {
  constexpr size_t ring = (size_t)WARPS * STAGES * 2 * KT * HD * 2;
  constexpr size_t merge = (size_t)(WARPS * COLS * (HD + 8) + 2 * WARPS * COLS) * sizeof(float);
  constexpr size_t smem = COLS * HD * 2 + (ring > merge ? ring : merge);
  auto kern = attn_decode_kr_kernel<HD, WARPS, STAGES>;
  static bool configured[gi::MAX_DEVICES_SEEN] = {false};
  int dev;
  if (gi::unconfigured_here(configured, &dev)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "attention decode: %s", cudaGetErrorString(e));
    if (dev >= 0) configured[dev] = true;
  }
  return gi::check(gi::launch(kern, grid, dim3(WARPS * 32), smem, s, out, ldo, po, pml, q, ldq, kc, vc, bt, max_pages, slots, lens, H, KV,
                              scale, window, n_splits, own_tiles), "attention decode (keys on rows)");
}

}  // namespace

// The decode attention with the keys on the rows of the tile.  Arguments as gi_attn_decode_tc_merged's without the
// counters (slices are merged by gi_attn_combine); warps: 4, 6 or 8 per block; stages: 2 or 3 tiles deep per warp.
extern "C" int gi_attn_decode_kr(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq, const void* kcache,
                                 const void* vcache, const int* block_table, int max_pages, const int* seq_slots,
                                 const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd, float scale, int window,
                                 int n_splits, int own_tiles, int warps, int stages, void* stream) {
  if (n_seqs <= 0) return GI_OK;
  if (own_tiles < 0) return gi::fail(GI_ERR_ARG, "attention: tiles per slice cannot be negative");
  if (hd != 64 && hd != 128) return gi::fail(GI_ERR_UNSUPPORTED, "attention decode (keys on rows): head size %d, only 64 and 128", hd);
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0)
    return gi::fail(GI_ERR_ARG, "attention: %d heads do not divide into %d kv heads", n_heads, n_kv);
  if (n_splits < 1) return gi::fail(GI_ERR_ARG, "attention: at least one slice");
  if (n_splits > 1 && (!part_o || !part_ml)) return gi::fail(GI_ERR_ARG, "attention: slices need scratch memory");
  if (ldq % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)kcache & 15) || ((uintptr_t)vcache & 15))
    return gi::fail(GI_ERR_UNSUPPORTED, "attention decode (keys on rows): queries and cache must be 16-byte aligned");
  const int group = n_heads / n_kv;
  const int chunks = (group + COLS - 1) / COLS;
  if ((long)n_kv * chunks > 65535 || n_seqs > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "attention: more than 65535 sequences or kv heads in one launch");
  dim3 grid(n_splits, n_kv * chunks, n_seqs);
  cudaStream_t s = (cudaStream_t)stream;
  int rc;
#define GI_DECODE_KR(HD_, W_, ST_)                                                                                          \
  rc = launch<HD_, W_, ST_>(grid, s, (__nv_bfloat16*)out, ldo, part_o, part_ml, (const __nv_bfloat16*)q, ldq,               \
                            (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, block_table, max_pages, seq_slots, \
                            seq_lens, n_heads, n_kv, scale, window, n_splits, own_tiles)
  if (stages != 2 && stages != 3) return gi::fail(GI_ERR_ARG, "attention decode (keys on rows): rings of %d stages, 2 or 3", stages);
  if (warps != 4 && warps != 6 && warps != 8) return gi::fail(GI_ERR_ARG, "attention decode (keys on rows): %d warps, 4, 6 or 8", warps);
  if (hd == 64) {
    if (warps == 4 && stages == 2) GI_DECODE_KR(64, 4, 2);
    else if (warps == 4) GI_DECODE_KR(64, 4, 3);
    else if (warps == 6 && stages == 2) GI_DECODE_KR(64, 6, 2);
    else if (warps == 6) GI_DECODE_KR(64, 6, 3);
    else if (stages == 2) GI_DECODE_KR(64, 8, 2);
    else GI_DECODE_KR(64, 8, 3);
  } else {
    if (warps == 4 && stages == 2) GI_DECODE_KR(128, 4, 2);
    else if (warps == 4) GI_DECODE_KR(128, 4, 3);
    else if (warps == 6 && stages == 2) GI_DECODE_KR(128, 6, 2);
    else if (warps == 6) GI_DECODE_KR(128, 6, 3);
    else if (stages == 2) GI_DECODE_KR(128, 8, 2);
    else GI_DECODE_KR(128, 8, 3);
  }
#undef GI_DECODE_KR
  if (rc != GI_OK) return rc;
  if (n_splits > 1) return gi_attn_combine(out, ldo, GI_BF16, part_o, part_ml, n_seqs, n_heads, hd, n_splits, stream);
  return GI_OK;
}
