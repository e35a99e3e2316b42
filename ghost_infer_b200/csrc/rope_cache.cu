// Rotary positions on q and k, and the cache write, in one pass over a step's packed [q | k | v] rows.
//
// Formula (src/model.rs:942-953, src/cuda.rs:461-471): for pair i of a head, theta = pos * inv_freq[i]
// in 32-bit, (a, b) <- (a cos - b sin, a sin + b cos).  Pairs are (i, i + rot/2) ("half", the layout
// safetensors checkpoints are trained in) or (2i, 2i + 1) ("adjacent", what GGUF converters permute
// to).  k is stored after rotation, v untouched (src/model.rs:1046-1048).  The frequency table is
// built once on the host; angles are computed here, once per (token, pair), and shared by all heads.
#include "api.h"
#include "common.cuh"

namespace {

template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, long ld, const int* __restrict__ positions,
                                  const int* __restrict__ slots, const int* __restrict__ block_table, int max_pages,
                                  T* __restrict__ kcache, T* __restrict__ vcache, const float* __restrict__ inv_freq,
                                  int n_heads, int n_kv, int hd, int rot, int adjacent, int write_cache) {
  extern __shared__ float2 cs[];  // rot/2 entries: (cos, sin)
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int slot = slots[t];
  const int half = rot / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf((float)pos * inv_freq[i], &s, &c);
    cs[i] = make_float2(c, s);
  }
  __syncthreads();
  T* row = qkv + (size_t)t * ld;
  // queries: rotated in place
  for (int idx = threadIdx.x; idx < n_heads * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half;
    const int ia = adjacent ? 2 * i : i, ib = adjacent ? 2 * i + 1 : i + half;
    T* q = row + (size_t)h * hd;
    const float a = gi::ldf(q + ia), b = gi::ldf(q + ib);
    const float2 f = cs[i];
    gi::stf(q + ia, a * f.x - b * f.y);
    gi::stf(q + ib, a * f.y + b * f.x);
  }
  if (!write_cache) return;
  // a padding row (slot < 0) writes to the trash page, which no live sequence reads
  const int page = slot >= 0 ? block_table[(size_t)slot * max_pages + pos / PAGE_TOKENS] : 0;
  const int off = pos % PAGE_TOKENS;
  const T* k = row + (size_t)n_heads * hd;
  const T* v = k + (size_t)n_kv * hd;
  for (int idx = threadIdx.x; idx < n_kv * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half;
    const int ia = adjacent ? 2 * i : i, ib = adjacent ? 2 * i + 1 : i + half;
    const float a = gi::ldf(k + h * hd + ia), b = gi::ldf(k + h * hd + ib);
    const float2 f = cs[i];
    T* dst = kcache + (((size_t)page * n_kv + h) * PAGE_TOKENS + off) * hd;
    gi::stf(dst + ia, a * f.x - b * f.y);
    gi::stf(dst + ib, a * f.y + b * f.x);
  }
  const int tail = hd - rot;  // dimensions past the rotated ones are kept as they are
  for (int idx = threadIdx.x; idx < n_kv * tail; idx += blockDim.x) {
    const int h = idx / tail, d = rot + idx % tail;
    kcache[(((size_t)page * n_kv + h) * PAGE_TOKENS + off) * hd + d] = k[h * hd + d];
  }
  for (int idx = threadIdx.x; idx < n_kv * hd; idx += blockDim.x) {
    const int h = idx / hd, d = idx % hd;
    vcache[(((size_t)page * n_kv + h) * PAGE_TOKENS + off) * hd + d] = v[idx];
  }
}

}  // namespace

extern "C" int gi_rope_cache_write(void* qkv, int dtype, long ld, const int* positions, const int* slots,
                                   const int* block_table, int max_pages, void* kcache, void* vcache,
                                   const float* inv_freq, int n_tokens, int n_heads, int n_kv, int hd, int rot,
                                   int adjacent, int write_cache, void* stream) {
  if (n_tokens <= 0) return GI_OK;
  if (hd <= 0 || rot < 0 || rot > hd || rot % 2 != 0)
    return gi::fail(GI_ERR_ARG, "rope: rotary size %d does not fit head size %d", rot, hd);
  if (write_cache && (!kcache || !vcache || !block_table)) return gi::fail(GI_ERR_ARG, "rope: cache write without a cache");
  const size_t smem = (size_t)(rot / 2) * sizeof(float2);
  GI_DISPATCH_DTYPE(dtype, T,
      (rope_cache_kernel<T><<<n_tokens, 128, smem, (cudaStream_t)stream>>>((T*)qkv, ld, positions, slots, block_table, max_pages,
          (T*)kcache, (T*)vcache, inv_freq, n_heads, n_kv, hd, rot, adjacent, write_cache)));
  return gi::check_launch("rope_cache_write");
}
