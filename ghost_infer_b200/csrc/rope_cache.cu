// Rotary positions on q and k, and the cache write, in one pass over a step's packed [q | k | v] rows.
//
// Formula (src/model.rs:942-953, src/cuda.rs:461-471): for pair i of a head, theta = pos * inv_freq[i]
// in 32-bit, (a, b) <- (a cos - b sin, a sin + b cos).  Pairs are (i, i + rot/2) ("half", the layout
// safetensors checkpoints are trained in) or (2i, 2i + 1) ("adjacent", what GGUF converters permute
// to).  k is stored after rotation, v untouched (src/model.rs:1046-1048).  The frequency table is
// built once on the host; angles (cos, sin) are computed once per step for every (token, pair) by a small
// kernel and shared by all heads and all layers.
#include "api.h"
#include "common.cuh"

namespace {

// (cos, sin) of pos * inv_freq for every token of a step and every rotated pair: computed once per step and
// shared by all layers, which rotate with the same positions and frequencies.
__global__ void rope_table_kernel(float2* __restrict__ table, const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int half, int total) {
  gi::pdl_prologue();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int t = idx / half, i = idx % half;
  float s, c;
  sincosf((float)positions[t] * inv_freq[i], &s, &c);
  table[idx] = make_float2(c, s);
}

using gi::rotate_pair;

// The value of column f of token t's packed row: what the product stored, or, for a tile of 128 columns that was cut
// between blocks of a deferred product (`sp`, looked up before the dependency wait), the sum of the partial sums in
// the order of the K ranges, rounded to T.
template <typename T>
__device__ __forceinline__ float row_value(const T* row, const gi_settle_t& st, const gi_settle_span& sp, int t, int f) {
  if (sp.c_first != sp.c_last) {
    const float acc = gi_sum_pieces(st, sp, t, f);
    T rounded;
    gi::stf(&rounded, acc);
    return gi::ldf(&rounded);
  }
  return gi::ldf(row + f);
}
__device__ __forceinline__ gi_settle_span span_or_none(const gi_settle_t& st, int f) {
  if (st.partials != nullptr) return gi_span_of(st, f);
  gi_settle_span none = {0, 0, 0};
  return none;
}

// One block per (token, head of the packed row): heads 0..H-1 are queries (rotated in place), H..H+KV-1 keys
// (rotated into the cache), H+KV.. values (copied into the cache).  A thread handles one pair or one value pair.
template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, long ld, const float2* table /* written by a kernel of this step: see gi::pdl_wait */,
                                  const int* __restrict__ positions,
                                  const int* __restrict__ slots, const int* __restrict__ block_table, int max_pages,
                                  T* __restrict__ kcache, T* __restrict__ vcache, int n_heads, int n_kv, int hd, int rot,
                                  int adjacent, int write_cache, gi_settle_t st) {
  // Positions, slots, the block table and the tables of the product's cut were uploaded before the step's first
  // kernel: they are read while the product before this kernel drains.  The rows, the partial sums and the angle
  // table (written by a kernel of this step) are read after the dependency wait.
  gi::pdl_launch_dependents();
  const int t = blockIdx.x, head = blockIdx.y;
  const int half = rot / 2;
  T* row = qkv + (size_t)t * ld;
  const int col0 = head * hd;
  T* src = row + col0;
  T* dst = src;                                 // queries are rotated in place
  if (head >= n_heads) {
    if (!write_cache) return;
    const int pos = gi::ld_step(positions + t), slot = gi::ld_step(slots + t);
    // a padding row (slot < 0) writes to the trash page, which no live sequence reads
    const int page = slot >= 0 ? gi::ld_step(block_table + (size_t)slot * max_pages + pos / PAGE_TOKENS) : 0;
    const int off = pos % PAGE_TOKENS;
    const bool is_k = head < n_heads + n_kv;
    dst = (is_k ? kcache : vcache) + (((size_t)page * n_kv + (head - n_heads - (is_k ? 0 : n_kv))) * PAGE_TOKENS + off) * hd;
  }
  const bool rotate = head < n_heads + n_kv;
  // the first two columns this thread reads (one pair, or two values): their spans are looked up before the wait
  const int i0 = threadIdx.x;
  const int e0 = rotate ? (adjacent ? 2 * i0 : i0) : i0;
  const int e1 = rotate ? (adjacent ? 2 * i0 + 1 : i0 + half) : i0 + (int)blockDim.x;
  gi_settle_span sp0 = {0, 0, 0}, sp1 = {0, 0, 0};
  if (e0 < hd) sp0 = span_or_none(st, col0 + e0);
  if (e1 < hd) sp1 = span_or_none(st, col0 + e1);
  gi::pdl_wait();
  if (rotate) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const int ia = adjacent ? 2 * i : i, ib = adjacent ? 2 * i + 1 : i + half;
      const gi_settle_span sa = (i == i0) ? sp0 : span_or_none(st, col0 + ia), sb = (i == i0) ? sp1 : span_or_none(st, col0 + ib);
      const float a = row_value(row, st, sa, t, col0 + ia), b = row_value(row, st, sb, t, col0 + ib);
      const float2 f = table[(size_t)t * half + i];
      float ra, rb;
      rotate_pair(a, b, f, &ra, &rb);
      gi::stf(dst + ia, ra);
      gi::stf(dst + ib, rb);
    }
    // past the rotated part: as it is (queries only when they are still partial sums: the attention reads the row)
    if (head >= n_heads || st.partials != nullptr)
      for (int d = rot + threadIdx.x; d < hd; d += blockDim.x) gi::stf(dst + d, row_value(row, st, span_or_none(st, col0 + d), t, col0 + d));
  } else {
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
      const gi_settle_span sd = (d == e0) ? sp0 : ((d == e1) ? sp1 : span_or_none(st, col0 + d));
      gi::stf(dst + d, row_value(row, st, sd, t, col0 + d));
    }
  }
}

// The same work for many tokens at once (a prompt): one block per token, 16 bytes per access.  Takes the common
// case only: half-split pairs, rotary and head sizes that are multiples of 16, nothing pending.  A thread takes
// eight neighbouring pairs of a head (two 16-byte loads, 8 apart by half the rotary size), or eight values.
template <typename T>
__global__ void rope_cache_rows_kernel(T* __restrict__ qkv, long ld, const float2* __restrict__ table, const int* __restrict__ positions,
                                       const int* __restrict__ slots, const int* __restrict__ block_table, int max_pages,
                                       T* __restrict__ kcache, T* __restrict__ vcache, int n_heads, int n_kv, int hd, int rot,
                                       int write_cache) {
  constexpr int V = 16 / sizeof(T);            // values per 16-byte access
  gi::pdl_prologue();
  const int t = blockIdx.x;
  const int half = rot / 2;
  T* row = qkv + (size_t)t * ld;
  const int pos = positions[t], slot = slots[t];
  const int page = (write_cache && slot >= 0) ? block_table[(size_t)slot * max_pages + pos / PAGE_TOKENS] : 0;
  const int off = pos % PAGE_TOKENS;
  const float2* cs = table + (size_t)t * half;
  const int chunks = half / V;                 // chunks of V pairs per head
  const int rot_heads = n_heads + (write_cache ? n_kv : 0);
  for (int item = threadIdx.x; item < rot_heads * chunks; item += blockDim.x) {
    const int head = item / chunks, i0 = (item % chunks) * V;
    T* src = row + (size_t)head * hd;
    T* dst = src;
    if (head >= n_heads) dst = kcache + (((size_t)page * n_kv + (head - n_heads)) * PAGE_TOKENS + off) * hd;
    T a[V], b[V];
    *reinterpret_cast<uint4*>(a) = *reinterpret_cast<const uint4*>(src + i0);
    *reinterpret_cast<uint4*>(b) = *reinterpret_cast<const uint4*>(src + i0 + half);
#pragma unroll
    for (int e = 0; e < V; ++e) {
      const float2 f = cs[i0 + e];
      const float x = gi::ldf(a + e), y = gi::ldf(b + e);
      float rx, ry;
      rotate_pair(x, y, f, &rx, &ry);
      gi::stf(a + e, rx);
      gi::stf(b + e, ry);
    }
    *reinterpret_cast<uint4*>(dst + i0) = *reinterpret_cast<const uint4*>(a);
    *reinterpret_cast<uint4*>(dst + i0 + half) = *reinterpret_cast<const uint4*>(b);
  }
  if (!write_cache) return;
  // keys past the rotated part, and the values: copied as they are
  const int tail = (hd - rot) / V, vchunks = hd / V;
  for (int item = threadIdx.x; item < n_kv * (tail + vchunks); item += blockDim.x) {
    const int h = item / (tail + vchunks), c = item % (tail + vchunks);
    const size_t cache_row = (((size_t)page * n_kv + h) * PAGE_TOKENS + off) * hd;
    if (c < tail) {
      const int d = rot + c * V;
      *reinterpret_cast<uint4*>(kcache + cache_row + d) = *reinterpret_cast<const uint4*>(row + (size_t)(n_heads + h) * hd + d);
    } else {
      const int d = (c - tail) * V;
      *reinterpret_cast<uint4*>(vcache + cache_row + d) = *reinterpret_cast<const uint4*>(row + (size_t)(n_heads + n_kv + h) * hd + d);
    }
  }
}

}  // namespace

extern "C" int gi_rope_table(float* table, const int* positions, const float* inv_freq, int n_tokens, int rot, void* stream) {
  const int half = rot / 2, total = n_tokens * half;
  if (total <= 0) return GI_OK;
  return gi::check(gi::launch(rope_table_kernel, dim3((total + 255) / 256), dim3(256), 0, (cudaStream_t)stream, (float2*)table,
                              positions, inv_freq, half, total), "rope table");
}

namespace {
int rope_impl(void* qkv, int dtype, long ld, const float* table, const int* positions, const int* slots, const int* block_table,
              int max_pages, void* kcache, void* vcache, int n_tokens, int n_heads, int n_kv, int hd, int rot, int adjacent,
              int write_cache, gi_settle_t st, void* stream) {
  if (n_tokens <= 0) return GI_OK;
  if (hd <= 0 || rot < 0 || rot > hd || rot % 2 != 0)
    return gi::fail(GI_ERR_ARG, "rope: rotary size %d does not fit head size %d", rot, hd);
  if (write_cache && (!kcache || !vcache || !block_table)) return gi::fail(GI_ERR_ARG, "rope: cache write without a cache");
  if (rot > 0 && !table) return gi::fail(GI_ERR_ARG, "rope: no table of angles");
  // with partial sums pending, the k and v blocks must run even without a cache write, so that nothing stays unsettled;
  // they are only needed for the cache, though, so without a cache they are simply not launched
  // a prompt's worth of tokens in the common layout: one block per token, 16-byte accesses
  const int vals = dtype == GI_F32 ? 4 : 8;
  if (st.partials == nullptr && n_tokens >= 32 && !adjacent && rot > 0 && (rot / 2) % vals == 0 && hd % vals == 0 && ld % vals == 0 &&
      (((uintptr_t)qkv | (uintptr_t)kcache | (uintptr_t)vcache) & 15) == 0) {
    cudaError_t e = cudaSuccess;
    GI_DISPATCH_DTYPE(dtype, T,
        e = gi::launch(rope_cache_rows_kernel<T>, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, (T*)qkv, ld, (const float2*)table,
                       positions, slots, block_table, max_pages, (T*)kcache, (T*)vcache, n_heads, n_kv, hd, rot, write_cache));
    return gi::check(e, "rope_cache_write");
  }
  const int heads = n_heads + (write_cache ? 2 * n_kv : 0);
  if (heads > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "rope: more than 65535 heads in one launch");
  dim3 grid(n_tokens, heads);
  const int threads = hd >= 128 ? 64 : 32;
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T,
      e = gi::launch(rope_cache_kernel<T>, grid, dim3(threads), 0, (cudaStream_t)stream, (T*)qkv, ld, (const float2*)table, positions,
                     slots, block_table, max_pages, (T*)kcache, (T*)vcache, n_heads, n_kv, hd, rot, adjacent, write_cache, st));
  return gi::check(e, "rope_cache_write");
}
}  // namespace

extern "C" int gi_rope_cache_write(void* qkv, int dtype, long ld, const float* table, const int* positions, const int* slots,
                                   const int* block_table, int max_pages, void* kcache, void* vcache, int n_tokens,
                                   int n_heads, int n_kv, int hd, int rot, int adjacent, int write_cache, void* stream) {
  gi_settle_t none = {nullptr, nullptr, nullptr, nullptr, 0};
  return rope_impl(qkv, dtype, ld, table, positions, slots, block_table, max_pages, kcache, vcache, n_tokens, n_heads, n_kv, hd, rot,
                   adjacent, write_cache, none, stream);
}

extern "C" int gi_rope_cache_write_settle(void* qkv, int dtype, long ld, const float* table, const int* positions, const int* slots,
                                          const int* block_table, int max_pages, void* kcache, void* vcache, int n_tokens,
                                          int n_heads, int n_kv, int hd, int rot, int adjacent, int write_cache,
                                          gi_settle_t settle, void* stream) {
  return rope_impl(qkv, dtype, ld, table, positions, slots, block_table, max_pages, kcache, vcache, n_tokens, n_heads, n_kv, hd, rot,
                   adjacent, write_cache, settle, stream);
}
