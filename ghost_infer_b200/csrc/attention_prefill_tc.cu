// Causal grouped-query attention of a step's prompt tokens over the paged cache, on tensor cores
// (bfloat16, head size 64 or 128).
//
// Formula: src/model.rs:1320-1419; the shape of the work is the reference's attention_prefill_tc
// (src/cuda.rs:2408-2613): a block takes 64 queries of one head, 4 warps of 16 rows each, and walks the
// cached keys in tiles of 64 with a running softmax (base 2, 32-bit statistics, 32-bit accumulators,
// probabilities rounded to bfloat16 as the second product's operand); the latest query tiles are
// scheduled first, since they have the most keys to visit (src/cuda.rs:2423).  New here: sequences of
// unequal length in one launch (a flat token axis with per-sequence offsets), keys and values fetched from
// pages through the sequence's page table by cp.async into a double-buffered, XOR-swizzled tile that
// ldmatrix reads, and queries that may sit after an already cached prefix (chunked prompts).
#include <math.h>

#include "api.h"
#include "common.cuh"
#include "mma_utils.cuh"

namespace {

constexpr int BQ = 64;     // queries per block
constexpr int BKV = 64;    // keys per tile = one page
constexpr int WARPS = 4;

template <int HD>
__global__ void __launch_bounds__(WARPS * 32)
attn_prefill_tc_kernel(__nv_bfloat16* __restrict__ out, long ldo, const __nv_bfloat16* __restrict__ q, long ldq,
                       const __nv_bfloat16* __restrict__ kcache, const __nv_bfloat16* __restrict__ vcache,
                       const int* __restrict__ block_table, int max_pages, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ seq_slots, const int* __restrict__ seq_pos0, int n_heads, int n_kv,
                       float scale, int window, int q_tiles) {
  constexpr int CH = HD / 8;
  constexpr int TILE_BYTES = BKV * HD * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* q_s = smem;                         // [BQ][HD]
  unsigned char* kv_s = smem + BQ * HD * 2;          // [2 stages][K tile | V tile]

  const int b = blockIdx.z, h = blockIdx.y;
  const int tok0 = cu_seqlens[b], qlen = cu_seqlens[b + 1] - tok0;
  const int q0 = (q_tiles - 1 - (int)blockIdx.x) * BQ;          // latest tiles first
  if (q0 >= qlen) return;
  const int slot = seq_slots[b], pos0 = seq_pos0[b];
  const int kvh = h / (n_heads / n_kv);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int rows_here = min(BQ, qlen - q0);
  const int p_last = pos0 + q0 + rows_here - 1;                 // the block's last position
  int t_first = 0;                                              // the first key any row here may see
  if (window > 0) t_first = max(0, pos0 + q0 - window + 1);
  const int kt_begin = (t_first / BKV) * BKV;
  const int n_tiles = (p_last - kt_begin) / BKV + 1;

  auto issue_kv = [&](int tile, int stage) {
    const int kt = kt_begin + tile * BKV;
    const int page = block_table[(size_t)slot * max_pages + kt / PAGE_TOKENS];
    const size_t base = ((size_t)page * n_kv + kvh) * PAGE_TOKENS * HD;
    unsigned char* ks = kv_s + (size_t)stage * 2 * TILE_BYTES;
    unsigned char* vs = ks + TILE_BYTES;
#pragma unroll
    for (int i = 0; i < BKV * CH / (WARPS * 32); ++i) {
      const int idx = i * WARPS * 32 + tid;
      const int r = idx / CH, c = idx % CH;
      const int ok = (kt + r <= p_last && kt + r >= t_first) ? 16 : 0;     // rows nobody here sees: zeros, not read
      const size_t off = base + (size_t)(ok ? r : 0) * HD + c * 8;
      gi::cp_async_16(gi::smem_u32(ks + gi::swz<CH>(r, c)), kcache + off, ok);
      gi::cp_async_16(gi::smem_u32(vs + gi::swz<CH>(r, c)), vcache + off, ok);
    }
  };

  // queries of this block (rows past the sequence's end: zeros) and the first key tile
#pragma unroll
  for (int i = 0; i < BQ * CH / (WARPS * 32); ++i) {
    const int idx = i * WARPS * 32 + tid;
    const int r = idx / CH, c = idx % CH;
    const int ok = r < rows_here ? 16 : 0;
    gi::cp_async_16(gi::smem_u32(q_s + gi::swz<CH>(r, c)), q + (size_t)(tok0 + q0 + (ok ? r : 0)) * ldq + (size_t)h * HD + c * 8, ok);
  }
  issue_kv(0, 0);
  gi::cp_async_commit();

  const int p_row0 = pos0 + q0 + warp * 16 + g;       // position of this thread's first row; the second is 8 further
  const int p_warp_last = pos0 + q0 + warp * 16 + 15;
  const float sl2 = scale * 1.4426950408889634f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[i][c] = 0.f;
  uint32_t qf[HD / 16][4];

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < n_tiles) issue_kv(tile + 1, stage ^ 1);
    gi::cp_async_commit();
    gi::cp_async_wait<1>();
    __syncthreads();
    if (tile == 0) {
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = ks * 2 + (lane >> 4);
        gi::ldmatrix_x4(qf[ks], gi::smem_u32(q_s + gi::swz<CH>(r, c)));
      }
    }
    const int kt = kt_begin + tile * BKV;
    const unsigned char* ks_ = kv_s + (size_t)stage * 2 * TILE_BYTES;
    const unsigned char* vs_ = ks_ + TILE_BYTES;
    // a warp whose rows all lie before this tile, or whose windows all ended before it, has nothing to do here
    const bool active = kt <= p_warp_last && (window <= 0 || kt + BKV - 1 > p_warp_last - 15 - window);
    if (active) {
      float s[BKV / 8][4];
#pragma unroll
      for (int nt = 0; nt < BKV / 8; ++nt) {
#pragma unroll
        for (int c = 0; c < 4; ++c) s[nt][c] = 0.f;
#pragma unroll
        for (int kp = 0; kp < HD / 32; ++kp) {
          uint32_t kb[4];
          const int r = nt * 8 + (lane & 7), c = kp * 4 + (lane >> 3);
          gi::ldmatrix_x4(kb, gi::smem_u32(ks_ + gi::swz<CH>(r, c)));
          gi::mma_16816(s[nt], qf[kp * 2], kb[0], kb[1]);
          gi::mma_16816(s[nt], qf[kp * 2 + 1], kb[2], kb[3]);
        }
      }
      float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < BKV / 8; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int key = kt + nt * 8 + 2 * t + (c & 1);
          const int p = p_row0 + (c >> 1) * 8;
          const bool ok = key <= p && p <= p_last && (window <= 0 || key > p - window);
          s[nt][c] = ok ? s[nt][c] * sl2 : -INFINITY;
          tmax[c >> 1] = fmaxf(tmax[c >> 1], s[nt][c]);
        }
      float alpha[2], m_use[2];
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        tmax[hh] = fmaxf(tmax[hh], __shfl_xor_sync(0xffffffffu, tmax[hh], 1));
        tmax[hh] = fmaxf(tmax[hh], __shfl_xor_sync(0xffffffffu, tmax[hh], 2));
        const float m_new = fmaxf(m_run[hh], tmax[hh]);
        alpha[hh] = (m_run[hh] == -INFINITY) ? 0.f : exp2f(m_run[hh] - m_new);   // m_new >= m_run, both finite here
        m_run[hh] = m_new;
        m_use[hh] = (m_new == -INFINITY) ? 0.f : m_new;     // a row that has seen no key yet: every p below is 0
      }
      float psum[2] = {0.f, 0.f};
      uint32_t pf[BKV / 16][4];
#pragma unroll
      for (int nt = 0; nt < BKV / 8; ++nt) {
        const float p0 = exp2f(s[nt][0] - m_use[0]), p1 = exp2f(s[nt][1] - m_use[0]);
        const float p2 = exp2f(s[nt][2] - m_use[1]), p3 = exp2f(s[nt][3] - m_use[1]);
        psum[0] += p0 + p1;
        psum[1] += p2 + p3;
        pf[nt / 2][(nt & 1) * 2] = gi::pack_bf16(p0, p1);
        pf[nt / 2][(nt & 1) * 2 + 1] = gi::pack_bf16(p2, p3);
      }
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        psum[hh] += __shfl_xor_sync(0xffffffffu, psum[hh], 1);
        psum[hh] += __shfl_xor_sync(0xffffffffu, psum[hh], 2);
        l_run[hh] = l_run[hh] * alpha[hh] + psum[hh];
      }
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        o[i][0] *= alpha[0];
        o[i][1] *= alpha[0];
        o[i][2] *= alpha[1];
        o[i][3] *= alpha[1];
      }
#pragma unroll
      for (int kk = 0; kk < BKV / 16; ++kk) {
#pragma unroll
        for (int dp = 0; dp < HD / 16; ++dp) {
          uint32_t vb[4];
          const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = dp * 2 + (lane >> 4);
          gi::ldmatrix_x4_trans(vb, gi::smem_u32(vs_ + gi::swz<CH>(r, c)));
          gi::mma_16816(o[dp * 2], pf[kk], vb[0], vb[1]);
          gi::mma_16816(o[dp * 2 + 1], pf[kk], vb[2], vb[3]);
        }
      }
    }
    __syncthreads();     // everyone is done with this stage before the next iteration refills it
  }

#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int row = warp * 16 + g + hh * 8;
    if (row >= rows_here) continue;
    const float inv = l_run[hh] > 0.f ? 1.0f / l_run[hh] : 0.f;
    __nv_bfloat16* orow = out + (size_t)(tok0 + q0 + row) * ldo + (size_t)h * HD;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      __nv_bfloat162 v = __floats2bfloat162_rn(o[i][hh * 2] * inv, o[i][hh * 2 + 1] * inv);
      *reinterpret_cast<__nv_bfloat162*>(orow + i * 8 + 2 * t) = v;
    }
  }
}

template <int HD>
int launch(dim3 grid, cudaStream_t s, __nv_bfloat16* out, long ldo, const __nv_bfloat16* q, long ldq, const __nv_bfloat16* kc,
           const __nv_bfloat16* vc, const int* bt, int max_pages, const int* cu, const int* slots, const int* pos0, int H, int KV,
           float scale, int window, int q_tiles) {
  constexpr size_t smem = (size_t)BQ * HD * 2 + 2 * 2 * (size_t)BKV * HD * 2;
  auto kern = attn_prefill_tc_kernel<HD>;
  static bool configured[gi::MAX_DEVICES_SEEN] = {false};
  int dev;
  if (gi::unconfigured_here(configured, &dev)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "attention prefill: %s", cudaGetErrorString(e));
    if (dev >= 0) configured[dev] = true;
  }
  kern<<<grid, WARPS * 32, smem, s>>>(out, ldo, q, ldq, kc, vc, bt, max_pages, cu, slots, pos0, H, KV, scale, window, q_tiles);
  return gi::check_launch("attention prefill (tensor cores)");
}

}  // namespace

extern "C" int gi_attn_prefill_tc(void* out, long ldo, const void* q, long ldq, const void* kcache, const void* vcache,
                                  const int* block_table, int max_pages, const int* cu_seqlens, const int* seq_slots,
                                  const int* seq_pos0, int n_seqs, int max_q_len, int n_heads, int n_kv, int hd,
                                  float scale, int window, void* stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return GI_OK;
  if (hd != 64 && hd != 128) return gi::fail(GI_ERR_UNSUPPORTED, "attention prefill (tensor cores): head size %d, only 64 and 128", hd);
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0)
    return gi::fail(GI_ERR_ARG, "attention: %d heads do not divide into %d kv heads", n_heads, n_kv);
  if (ldq % 8 != 0 || ldo % 2 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)kcache & 15) || ((uintptr_t)vcache & 15) || ((uintptr_t)out & 3))
    return gi::fail(GI_ERR_UNSUPPORTED, "attention prefill (tensor cores): queries and cache must be 16-byte aligned");
  if (n_seqs > 65535 || n_heads > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "attention: more than 65535 sequences or heads in one launch");
  const int q_tiles = (max_q_len + BQ - 1) / BQ;
  dim3 grid(q_tiles, n_heads, n_seqs);
  cudaStream_t s = (cudaStream_t)stream;
  if (hd == 128)
    return launch<128>(grid, s, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)kcache,
                       (const __nv_bfloat16*)vcache, block_table, max_pages, cu_seqlens, seq_slots, seq_pos0, n_heads, n_kv, scale,
                       window, q_tiles);
  return launch<64>(grid, s, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)kcache,
                    (const __nv_bfloat16*)vcache, block_table, max_pages, cu_seqlens, seq_slots, seq_pos0, n_heads, n_kv, scale,
                    window, q_tiles);
}
