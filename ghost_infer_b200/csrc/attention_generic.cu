// Causal grouped-query attention over the paged cache on CUDA cores, 32-bit arithmetic throughout.
//
// Formula (src/model.rs:1320-1419): head h reads kv head h / (H / KV); score_t = (q . k_t) / sqrt(hd)
// for every cached position t <= the query's own position (and, with a window w, t > pos - w);
// softmax with the maximum subtracted; output = sum_t p_t v_t.  Two kernels:
//  * prefill: a block takes 32 queries of one head and walks key tiles of 32 with a running softmax
//    (the role of the reference's attention_prefill, src/cuda.rs:1940-2039);
//  * decode: a block takes one kv head of one sequence and one slice of its context, every query
//    head of the group sharing each key/value row it reads; slices are merged by a second kernel
//    (the roles of attention_partial_gqa and attention_combine, src/cuda.rs:1684-1865, :2806-2839).
// Keys and values live in pages of 64 positions: [page][kv head][64][hd].
#include <math.h>

#include "api.h"
#include "common.cuh"

namespace {

constexpr int QT = 32;  // queries per block (prefill)
constexpr int KT = 32;  // keys per tile

// ------------------------------------------------------------------------------------ prefill
template <typename T, int DPT>
__global__ void __launch_bounds__(128)
attn_prefill_kernel(T* __restrict__ out, long ldo, const T* __restrict__ q, long ldq, const T* __restrict__ kcache,
                    const T* __restrict__ vcache, const int* __restrict__ block_table, int max_pages,
                    const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slots,
                    const int* __restrict__ seq_pos0, int n_heads, int n_kv, int hd, float scale, int window) {
  extern __shared__ float smem[];
  const int ldk = hd + 1;
  float* Qs = smem;                  // [QT][hd+1]
  float* Ks = Qs + QT * ldk;         // [KT][hd+1]
  float* Vs = Ks + KT * ldk;         // [KT][hd+1]
  float* Ps = Vs + KT * ldk;         // [QT][KT+1]

  const int b = blockIdx.z, h = blockIdx.y;
  const int tok0 = cu_seqlens[b], qlen = cu_seqlens[b + 1] - tok0;
  const int q0 = blockIdx.x * QT;
  if (q0 >= qlen) return;
  const int slot = seq_slots[b], pos0 = seq_pos0[b];
  const int kvh = h / (n_heads / n_kv);
  const int tid = threadIdx.x, row = tid >> 2, sub = tid & 3;
  const int rows_here = min(QT, qlen - q0);

  for (int idx = tid; idx < QT * hd; idx += 128) {
    const int r = idx / hd, d = idx % hd;
    Qs[r * ldk + d] = r < rows_here ? gi::ldf(q + (size_t)(tok0 + q0 + r) * ldq + (size_t)h * hd + d) : 0.f;
  }
  const bool row_ok = row < rows_here;
  const int p_row = pos0 + q0 + row;               // this row's position
  const int p_last = pos0 + q0 + rows_here - 1;    // the block's last position
  int t_first = 0;                                 // the first key any row of this block may see
  if (window > 0) t_first = max(0, pos0 + q0 - window + 1);
  const int t_begin = (t_first / KT) * KT;

  float m = -INFINITY, l = 0.f;
  float acc[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) acc[i] = 0.f;

  for (int kt = t_begin; kt <= p_last; kt += KT) {
    __syncthreads();
    const int page = block_table[(size_t)slot * max_pages + kt / PAGE_TOKENS];
    const size_t base = (((size_t)page * n_kv + kvh) * PAGE_TOKENS + (kt % PAGE_TOKENS)) * hd;
    for (int idx = tid; idx < KT * hd; idx += 128) {
      const int j = idx / hd, d = idx % hd;
      const bool live = kt + j <= p_last && kt + j >= t_first;   // rows no query here sees are not read
      Ks[j * ldk + d] = live ? gi::ldf(kcache + base + (size_t)j * hd + d) : 0.f;
      Vs[j * ldk + d] = live ? gi::ldf(vcache + base + (size_t)j * hd + d) : 0.f;
    }
    __syncthreads();
    float s[8];
    float tile_max = -INFINITY;
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const int j = sub + 4 * jj;
      const int t = kt + j;
      float dot = 0.f;
      const float* qr = Qs + row * ldk;
      const float* kr = Ks + j * ldk;
      for (int d = 0; d < hd; ++d) dot = fmaf(qr[d], kr[d], dot);
      const bool ok = row_ok && t <= p_row && (window <= 0 || t > p_row - window);
      s[jj] = ok ? dot * scale : -INFINITY;
      tile_max = fmaxf(tile_max, s[jj]);
    }
    tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
    tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
    const float m_new = fmaxf(m, tile_max);
    float alpha = 1.f, psum = 0.f;
    if (m_new != -INFINITY) {
      alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const float p = (s[jj] == -INFINITY) ? 0.f : expf(s[jj] - m_new);
        Ps[row * (KT + 1) + sub + 4 * jj] = p;
        psum += p;
      }
    } else {
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) Ps[row * (KT + 1) + sub + 4 * jj] = 0.f;
    }
    psum += __shfl_xor_sync(0xffffffffu, psum, 1);
    psum += __shfl_xor_sync(0xffffffffu, psum, 2);
    l = l * alpha + psum;
    m = m_new;
    __syncwarp();
#pragma unroll
    for (int i = 0; i < DPT; ++i) acc[i] *= alpha;
    for (int j = 0; j < KT; ++j) {
      const float p = Ps[row * (KT + 1) + j];
      const float* vr = Vs + j * ldk;
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        const int d = sub + 4 * i;
        if (d < hd) acc[i] = fmaf(p, vr[d], acc[i]);
      }
    }
    __syncwarp();
  }
  if (row_ok) {
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    T* o = out + (size_t)(tok0 + q0 + row) * ldo + (size_t)h * hd;
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      const int d = sub + 4 * i;
      if (d < hd) gi::stf(o + d, acc[i] * inv);
    }
  }
}

// ------------------------------------------------------------------------------------- decode
// One token per sequence.  grid = (splits, kv heads * head chunks, sequences); 4 warps; a warp takes
// key tiles of 32 (one key per lane for the scores, one output dimension stripe per lane for values).
template <typename T, int GC, int DC>
__global__ void __launch_bounds__(128)
attn_decode_kernel(T* __restrict__ out, long ldo, float* __restrict__ part_o, float* __restrict__ part_ml,
                   const T* __restrict__ q, long ldq, const T* __restrict__ kcache, const T* __restrict__ vcache,
                   const int* __restrict__ block_table, int max_pages, const int* __restrict__ seq_slots,
                   const int* __restrict__ seq_lens, int n_heads, int n_kv, int hd, float scale, int window,
                   int n_splits, int own_tiles) {
  extern __shared__ float smem[];
  float* Qs = smem;                       // [GC][hd]
  float* Mo = Qs + GC * hd;               // [4][GC][hd] warp outputs
  float* Mm = Mo + 4 * GC * hd;           // [4][GC] warp maxima
  float* Ml = Mm + 4 * GC;                // [4][GC] warp sums

  const int group = n_heads / n_kv;
  const int chunks = (group + GC - 1) / GC;
  const int b = blockIdx.z, kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks, sp = blockIdx.x;
  const int g0 = chunk * GC, gcount = min(GC, group - g0);
  const int h0 = kvh * group + g0;
  const int slot = seq_slots[b];
  const int len = seq_lens[b];            // cached positions including this step's token
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int idx = tid; idx < GC * hd; idx += 128) {
    const int g = idx / hd, d = idx % hd;
    Qs[idx] = g < gcount ? gi::ldf(q + (size_t)b * ldq + (size_t)(h0 + g) * hd + d) : 0.f;
  }
  __syncthreads();

  int t_first = 0;
  if (window > 0) t_first = max(0, len - window);
  const int t_base = (t_first / KT) * KT;
  const int tiles = len > t_base ? (len - t_base + KT - 1) / KT : 0;
  // own_tiles > 0: a slice is that many tiles of the sequence's own span, so its sums do not depend on what else
  // the launch holds (slices past the span stay empty); else the span is cut into n_splits equal slices
  const int per = own_tiles > 0 ? own_tiles : (tiles + n_splits - 1) / n_splits;
  const int tile_lo = sp * per, tile_hi = min(tiles, tile_lo + per);

  float m[GC], l[GC], o[GC][DC];
#pragma unroll
  for (int g = 0; g < GC; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int c = 0; c < DC; ++c) o[g][c] = 0.f;
  }

  for (int tile = tile_lo + warp; tile < tile_hi; tile += 4) {
    const int t0 = t_base + tile * KT;
    const int page = slot >= 0 ? block_table[(size_t)slot * max_pages + t0 / PAGE_TOKENS] : 0;
    const size_t base = (((size_t)page * n_kv + kvh) * PAGE_TOKENS + (t0 % PAGE_TOKENS)) * hd;
    const int t = t0 + lane;
    const bool ok = t < len && t >= t_first;
    float s[GC];
#pragma unroll
    for (int g = 0; g < GC; ++g) s[g] = 0.f;
    if (ok) {
      const T* kr = kcache + base + (size_t)lane * hd;
      for (int d = 0; d < hd; ++d) {
        const float kv = gi::ldf(kr + d);
#pragma unroll
        for (int g = 0; g < GC; ++g) s[g] = fmaf(Qs[g * hd + d], kv, s[g]);
      }
    }
    float p[GC];
#pragma unroll
    for (int g = 0; g < GC; ++g) {
      const float sc = ok ? s[g] * scale : -INFINITY;
      const float tmax = gi::warp_max(sc);
      const float m_new = fmaxf(m[g], tmax);      // finite: a tile always holds at least one live key
      const float alpha = (m[g] == -INFINITY) ? 0.f : expf(m[g] - m_new);
      p[g] = ok ? expf(sc - m_new) : 0.f;
      l[g] = l[g] * alpha + gi::warp_sum(p[g]);
      m[g] = m_new;
#pragma unroll
      for (int c = 0; c < DC; ++c) o[g][c] *= alpha;
    }
    const int n_here = min(KT, len - t0);
    for (int j = 0; j < n_here; ++j) {
      float v[DC];
#pragma unroll
      for (int c = 0; c < DC; ++c) {
        const int d = lane + 32 * c;
        v[c] = (d < hd && t0 + j >= t_first) ? gi::ldf(vcache + base + (size_t)j * hd + d) : 0.f;
      }
#pragma unroll
      for (int g = 0; g < GC; ++g) {
        const float pj = __shfl_sync(0xffffffffu, p[g], j);
#pragma unroll
        for (int c = 0; c < DC; ++c) o[g][c] = fmaf(pj, v[c], o[g][c]);
      }
    }
  }

  // merge the four warps in a fixed order
#pragma unroll
  for (int g = 0; g < GC; ++g) {
    if (lane == 0) {
      Mm[warp * GC + g] = m[g];
      Ml[warp * GC + g] = l[g];
    }
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      const int d = lane + 32 * c;
      if (d < hd) Mo[(warp * GC + g) * hd + d] = o[g][c];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < gcount * hd; idx += 128) {
    const int g = idx / hd, d = idx % hd;
    float mm = -INFINITY;
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, Mm[w * GC + g]);
    float tot = 0.f, val = 0.f;
    if (mm != -INFINITY) {
      for (int w = 0; w < 4; ++w) {
        const float mw = Mm[w * GC + g];
        if (mw == -INFINITY) continue;
        const float wgt = expf(mw - mm);
        tot += Ml[w * GC + g] * wgt;
        val += Mo[(w * GC + g) * hd + d] * wgt;
      }
    }
    const int h = h0 + g;
    if (n_splits == 1) {
      gi::stf(out + (size_t)b * ldo + (size_t)h * hd + d, tot > 0.f ? val / tot : 0.f);
    } else {
      const size_t pi = ((size_t)b * n_heads + h) * n_splits + sp;
      part_o[pi * hd + d] = val;
      if (d == 0) {
        part_ml[pi * 2] = mm;
        part_ml[pi * 2 + 1] = tot;
      }
    }
  }
}

// Merges the slices of one (sequence, head): weights exp(m_s - m), summed in slice order.
template <typename T>
__global__ void attn_combine_kernel(T* __restrict__ out, long ldo, const float* __restrict__ part_o,
                                    const float* __restrict__ part_ml, int n_heads, int hd, int n_splits) {
  // The loads of eight slices are issued together (a slice past the end counts as an empty one): the merge costs
  // a trip or two to the L2 cache, not one per slice.  The arithmetic and its order are those of a plain loop.
  gi::pdl_prologue();
  const int b = blockIdx.y, h = blockIdx.x;
  const size_t p0 = ((size_t)b * n_heads + h) * n_splits;
  const float2* ml = reinterpret_cast<const float2*>(part_ml) + p0;
  if (n_splits <= 8) {
    // the usual case: the maxima, the sums and this thread's values of all slices in one round of loads
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
      float2 m8[8];
      float o8[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool in = j < n_splits;
        m8[j] = in ? __ldcg(ml + j) : make_float2(-INFINITY, 0.f);
        o8[j] = in ? __ldcg(part_o + (p0 + j) * hd + d) : 0.f;
      }
      float mm = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) mm = fmaxf(mm, m8[j].x);
      float tot = 0.f, val = 0.f;
      if (mm != -INFINITY) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (m8[j].x == -INFINITY) continue;
          const float w = expf(m8[j].x - mm);
          tot += m8[j].y * w;
          val += o8[j] * w;
        }
      }
      gi::stf(out + (size_t)b * ldo + (size_t)h * hd + d, tot > 0.f ? val / tot : 0.f);
    }
    return;
  }
  float mm = -INFINITY;
  for (int s0 = 0; s0 < n_splits; s0 += 8) {
    float m8[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) m8[j] = (s0 + j < n_splits) ? __ldcg(ml + s0 + j).x : -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) mm = fmaxf(mm, m8[j]);
  }
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float tot = 0.f, val = 0.f;
    if (mm != -INFINITY) {
      for (int s0 = 0; s0 < n_splits; s0 += 8) {
        float2 m8[8];
        float o8[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const bool in = s0 + j < n_splits;
          m8[j] = in ? __ldcg(ml + s0 + j) : make_float2(-INFINITY, 0.f);
          o8[j] = in ? __ldcg(part_o + (p0 + s0 + j) * hd + d) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (m8[j].x == -INFINITY) continue;
          const float w = expf(m8[j].x - mm);
          tot += m8[j].y * w;
          val += o8[j] * w;
        }
      }
    }
    gi::stf(out + (size_t)b * ldo + (size_t)h * hd + d, tot > 0.f ? val / tot : 0.f);
  }
}

template <typename T>
int launch_prefill(int dpt, dim3 grid, size_t smem, cudaStream_t s, T* out, long ldo, const T* q, long ldq,
                   const T* kc, const T* vc, const int* bt, int max_pages, const int* cu, const int* slots,
                   const int* pos0, int H, int KV, int hd, float scale, int window) {
#define GI_PREFILL_CASE(D)                                                                                       \
  case D: {                                                                                                      \
    auto kern = attn_prefill_kernel<T, D>;                                                                       \
    if (smem > 48 * 1024) {                                                                                      \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
      if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "attention prefill: %s", cudaGetErrorString(e));        \
    }                                                                                                            \
    kern<<<grid, 128, smem, s>>>(out, ldo, q, ldq, kc, vc, bt, max_pages, cu, slots, pos0, H, KV, hd, scale, window); \
    break;                                                                                                       \
  }
  switch (dpt) {
    GI_PREFILL_CASE(4)
    GI_PREFILL_CASE(8)
    GI_PREFILL_CASE(16)
    GI_PREFILL_CASE(32)
    GI_PREFILL_CASE(64)
    default:
      return gi::fail(GI_ERR_UNSUPPORTED, "attention prefill: head size %d is above 256", hd);
  }
#undef GI_PREFILL_CASE
  return gi::check_launch("attention prefill");
}

template <typename T, int GC>
int launch_decode_dc(int dc, dim3 grid, size_t smem, cudaStream_t s, T* out, long ldo, float* po, float* pml,
                     const T* q, long ldq, const T* kc, const T* vc, const int* bt, int max_pages, const int* slots,
                     const int* lens, int H, int KV, int hd, float scale, int window, int n_splits, int own_tiles) {
#define GI_DECODE_CASE(D)                                                                                        \
  case D: {                                                                                                      \
    auto kern = attn_decode_kernel<T, GC, D>;                                                                    \
    if (smem > 48 * 1024) {                                                                                      \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
      if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "attention decode: %s", cudaGetErrorString(e));         \
    }                                                                                                            \
    kern<<<grid, 128, smem, s>>>(out, ldo, po, pml, q, ldq, kc, vc, bt, max_pages, slots, lens, H, KV, hd, scale, window, n_splits, own_tiles); \
    break;                                                                                                       \
  }
  switch (dc) {
    GI_DECODE_CASE(1)
    GI_DECODE_CASE(2)
    GI_DECODE_CASE(4)
    GI_DECODE_CASE(8)
    default:
      return gi::fail(GI_ERR_UNSUPPORTED, "attention decode: head size %d is above 256", hd);
  }
#undef GI_DECODE_CASE
  return gi::check_launch("attention decode");
}

int pow2_at_least(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

}  // namespace

extern "C" int gi_attn_combine(void* out, long ldo, int dtype, const float* part_o, const float* part_ml, int n_seqs,
                               int n_heads, int hd, int n_splits, void* stream) {
  dim3 cgrid(n_heads, n_seqs);
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T,
      e = gi::launch(attn_combine_kernel<T>, cgrid, dim3(hd <= 64 ? 64 : (hd <= 128 ? 128 : 256)), 0, (cudaStream_t)stream, (T*)out, ldo, part_o, part_ml, n_heads, hd, n_splits));
  return gi::check(e, "attention combine");
}

extern "C" int gi_attn_prefill_generic(void* out, long ldo, const void* q, long ldq, int dtype, const void* kcache,
                                       const void* vcache, const int* block_table, int max_pages,
                                       const int* cu_seqlens, const int* seq_slots, const int* seq_pos0, int n_seqs,
                                       int max_q_len, int n_heads, int n_kv, int hd, float scale, int window,
                                       void* stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return GI_OK;
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0)
    return gi::fail(GI_ERR_ARG, "attention: %d heads do not divide into %d kv heads", n_heads, n_kv);
  if (hd <= 0 || hd > 256) return gi::fail(GI_ERR_UNSUPPORTED, "attention: head size %d is outside 1..256", hd);
  if (n_seqs > 65535 || n_heads > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "attention: more than 65535 sequences or heads in one launch");
  const int dpt = max(4, pow2_at_least((hd + 3) / 4));
  dim3 grid((max_q_len + QT - 1) / QT, n_heads, n_seqs);
  const size_t smem = ((size_t)(QT + 2 * KT) * (hd + 1) + (size_t)QT * (KT + 1)) * sizeof(float);
  GI_DISPATCH_DTYPE(dtype, T,
      return (launch_prefill<T>(dpt, grid, smem, (cudaStream_t)stream, (T*)out, ldo, (const T*)q, ldq, (const T*)kcache,
                                (const T*)vcache, block_table, max_pages, cu_seqlens, seq_slots, seq_pos0, n_heads, n_kv,
                                hd, scale, window)));
  return GI_OK;
}

extern "C" int gi_attn_decode_generic(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq,
                                      int dtype, const void* kcache, const void* vcache, const int* block_table,
                                      int max_pages, const int* seq_slots, const int* seq_lens, int n_seqs,
                                      int n_heads, int n_kv, int hd, float scale, int window, int n_splits,
                                      int own_tiles, void* stream) {
  if (n_seqs <= 0) return GI_OK;
  if (own_tiles < 0) return gi::fail(GI_ERR_ARG, "attention: tiles per slice cannot be negative");
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0)
    return gi::fail(GI_ERR_ARG, "attention: %d heads do not divide into %d kv heads", n_heads, n_kv);
  if (hd <= 0 || hd > 256) return gi::fail(GI_ERR_UNSUPPORTED, "attention: head size %d is outside 1..256", hd);
  if (n_splits < 1) return gi::fail(GI_ERR_ARG, "attention: at least one slice");
  if (n_splits > 1 && (!part_o || !part_ml)) return gi::fail(GI_ERR_ARG, "attention: slices need scratch memory");
  const int group = n_heads / n_kv;
  const int gc = min(8, pow2_at_least(group));
  const int chunks = (group + gc - 1) / gc;
  const int dc = pow2_at_least((hd + 31) / 32);
  if ((long)n_kv * chunks > 65535 || n_seqs > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "attention: more than 65535 sequences or kv heads in one launch");
  dim3 grid(n_splits, n_kv * chunks, n_seqs);
  const size_t smem = ((size_t)gc * hd + 4 * (size_t)gc * hd + 8 * (size_t)gc) * sizeof(float);
  cudaStream_t s = (cudaStream_t)stream;
  int rc = GI_OK;
#define GI_GC_CASE(G)                                                                                              \
  case G:                                                                                                          \
    GI_DISPATCH_DTYPE(dtype, T,                                                                                    \
        rc = (launch_decode_dc<T, G>(dc, grid, smem, s, (T*)out, ldo, part_o, part_ml, (const T*)q, ldq, (const T*)kcache, \
                                     (const T*)vcache, block_table, max_pages, seq_slots, seq_lens, n_heads, n_kv, hd, \
                                     scale, window, n_splits, own_tiles)));                                        \
    break;
  switch (gc) {
    GI_GC_CASE(1)
    GI_GC_CASE(2)
    GI_GC_CASE(4)
    GI_GC_CASE(8)
  }
#undef GI_GC_CASE
  if (rc != GI_OK) return rc;
  if (n_splits > 1) {
    dim3 cgrid(n_heads, n_seqs);
    GI_DISPATCH_DTYPE(dtype, T,
        (attn_combine_kernel<T><<<cgrid, 64, 0, s>>>((T*)out, ldo, part_o, part_ml, n_heads, hd, n_splits)));
    return gi::check_launch("attention combine");
  }
  return GI_OK;
}
