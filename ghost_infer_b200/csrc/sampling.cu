// Next-token selection on the device: greedy, or temperature + top-k + top-p.
//
// Rule (src/sampler.rs:205-218, :259-291): temperature <= 0 picks the highest logit, the first one on
// ties.  Otherwise the candidates are the top_k highest logits (0 = all), in descending order;
// w_i = exp((l_i - l_max) / T); the list is cut after the first place where the running share of the
// total reaches top_p; then r = u * (kept mass) is walked down the list and the first candidate at
// which the running sum reaches r is taken.  u comes from xorshift64*, top 24 bits (src/sampler.rs:185-191).
//
// No sort is done.  "The first place in descending order where a running sum reaches a target" is
// found by descending the bits of an order-preserving integer key, eight at a time: one sweep builds
// a 256-bin histogram of weights for the keys that share the prefix found so far, a scan of the bins
// picks the next byte.  Weights are 41-bit fixed point and summed as integers, so the result does not
// depend on the order in which threads add.  Equal logits are ordered by token id (lower first), with
// a second descent over the ids.  One block per row.
//
// The usual case, a top_k of at most 2048, takes a shorter way to the same pick: one sweep counts the keys by their
// distance below the highest key (4096 bins of 2^16 key steps: the seven upper bits of the mantissa, 32 octaves),
// which names the bin the k-th highest key lies in; a second sweep collects the keys down to that bin (top_k and
// a few more) into shared memory, where they are sorted (key descending, token id ascending) and the cut and the
// draw are made over at most top_k entries with the same fixed-point weights and the same rules.  Some twenty
// sweeps over the row, with an exponential per logit in half of them, become two sweeps and top_k exponentials.
#include <math.h>
#include <stddef.h>

#include "api.h"
#include "common.cuh"

namespace {

typedef unsigned long long u64;

constexpr int THREADS = 1024;
constexpr float FIXED_ONE = 1099511627776.0f;  // 2^40

__device__ __forceinline__ unsigned order_key(float v) {
  if (v != v) return 0u;  // NaN never wins (src/cuda.rs:3540-3570)
  const unsigned f = __float_as_uint(v);
  return (f & 0x80000000u) ? ~f : (f | 0x80000000u);
}
__device__ __forceinline__ float key_value(unsigned k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ u64 fixed_weight(float logit, float lmax, float temperature) {
  if (logit != logit) return 0;
  return __float2ull_rn(expf((logit - lmax) / temperature) * FIXED_ONE);
}

constexpr int FAST_BINS = 4096;      // keys by their distance below the highest key, in steps of 2^16
constexpr int FAST_CAP = 2048;       // candidates the short way can hold

struct Shared {
  unsigned bins[FAST_BINS];
  u64 list[FAST_CAP];                // (key << 32) | ~id: descending order = key descending, id ascending; the long way
                                     // keeps sixteen copies of its histogram in `bins` and here (64-bit additions to
                                     // shared memory are compare-and-swap loops: a copy per two warps spares them the crowd)
  int n_list, first_bin;
  u64 hist[256];
  u64 red64[32];
  float redv[32];
  int redi[32];
  unsigned prefix;
  u64 before, equal;
  float bestv;
  int besti;
  u64 total;
  float u;
};

// Descends the bytes of `val` from `start_shift` down.  elem(i, val) says whether element i takes part and
// gives its ordering value; weight(i, val) its weight, asked only for elements that still match the bytes found
// so far (an exponential each: after the first byte few elements are left).  On return: `val_out` is the value at which the running
// sum (in descending order if DESC, else ascending) first reaches `target`; `before` is the weight
// ordered strictly before it; `equal` the weight of the elements equal to it.
template <bool DESC, typename F, typename W>
__device__ void radix_descend(Shared& sh, int n, int start_shift, u64 target, F elem, W weight, unsigned& val_out, u64& before_out,
                              u64& equal_out) {
  const int tid = threadIdx.x;
  if (tid == 0) {
    sh.prefix = 0;
    sh.before = 0;
    sh.equal = 0;
  }
  constexpr int COPIES = 16;                               // over `bins` and `list`, which lie one after the other
  static_assert(offsetof(Shared, list) == sizeof(unsigned) * FAST_BINS, "the copies span bins and list");
  u64* copies = reinterpret_cast<u64*>(sh.bins);           // [COPIES][256]
  u64* my_hist = copies + ((tid >> 5) % COPIES) * 256;
  for (int shift = start_shift; shift >= 0; shift -= 8) {
    for (int b = tid; b < COPIES * 256; b += blockDim.x) copies[b] = 0;
    __syncthreads();
    const unsigned prefix = sh.prefix;
    const bool check = shift != start_shift;
    int cur = -1;
    u64 run = 0;
#pragma unroll 8
    for (int i = tid; i < n; i += blockDim.x) {
      unsigned val;
      if (!elem(i, val)) continue;
      if (check && (val >> (shift + 8)) != prefix) continue;
      const u64 wt = weight(i, val);
      const int bin = (int)((val >> shift) & 255u);
      if (bin != cur) {
        if (run) atomicAdd(&my_hist[cur], run);
        cur = bin;
        run = 0;
      }
      run += wt;
    }
    if (run) atomicAdd(&my_hist[cur], run);
    __syncthreads();
    for (int b = tid; b < 256; b += blockDim.x) {
      u64 t = 0;
#pragma unroll
      for (int c = 0; c < COPIES; ++c) t += copies[c * 256 + b];
      sh.hist[b] = t;
    }
    __syncthreads();
    if (tid == 0) {
      u64 acc = sh.before;
      int chosen = -1, last = -1;
      for (int s = 0; s < 256; ++s) {
        const int b = DESC ? 255 - s : s;
        const u64 hb = sh.hist[b];
        if (hb == 0) continue;
        last = b;
        if (acc + hb >= target) {
          chosen = b;
          break;
        }
        acc += hb;
      }
      if (chosen < 0) {  // the target lies beyond the total: the last element in order
        chosen = last < 0 ? 0 : last;
        acc -= sh.hist[chosen];
      }
      sh.prefix = (sh.prefix << 8) | (unsigned)chosen;
      sh.before = acc;
      sh.equal = sh.hist[chosen];
    }
    __syncthreads();
  }
  val_out = sh.prefix;
  before_out = sh.before;
  equal_out = sh.equal;
  __syncthreads();
}

__device__ __forceinline__ int index_start_shift(int n) { return n <= (1 << 8) ? 0 : n <= (1 << 16) ? 8 : n <= (1 << 24) ? 16 : 24; }

__device__ u64 block_sum_u64(Shared& sh, u64 v) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) sh.red64[warp] = v;
  __syncthreads();
  if (warp == 0) {
    u64 t = lane < (int)(blockDim.x >> 5) ? sh.red64[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) sh.total = t;
  }
  __syncthreads();
  return sh.total;
}

// The first place j < count (count <= 2 * blockDim.x) at which base + item(0) + ... + item(j) reaches `target`, found by
// the whole block: every thread takes two neighbouring items, a scan over the threads gives each the sum before its
// pair.  Returns the place (-1: the sum never gets there), `before_out` = base + the items before it, `total_out` =
// the sum of all items.  Sums are integers: no order of additions can change them.
template <typename F>
__device__ int first_reaching(Shared& sh, int count, u64 base, u64 target, F item, u64& before_out, u64& total_out) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int j0 = 2 * tid;
  const u64 a = j0 < count ? item(j0) : 0, b = j0 + 1 < count ? item(j0 + 1) : 0;
  u64 incl = a + b;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const u64 up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  __syncthreads();
  if (lane == 31) sh.red64[warp] = incl;
  if (tid == 0) sh.first_bin = 0x7fffffff;
  __syncthreads();
  if (warp == 0) {
    u64 t = lane < (int)(blockDim.x >> 5) ? sh.red64[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const u64 up = __shfl_up_sync(0xffffffffu, t, o);
      if (lane >= o) t += up;
    }
    sh.red64[lane] = t;                               // inclusive over the warps
  }
  __syncthreads();
  const u64 mine_before = base + (warp > 0 ? sh.red64[warp - 1] : 0) + (incl - a - b);
  int found = 0x7fffffff;
  if (j0 < count && mine_before + a >= target) found = j0;
  else if (j0 + 1 < count && mine_before + a + b >= target) found = j0 + 1;
  if (found != 0x7fffffff) atomicMin(&sh.first_bin, found);
  __syncthreads();
  const int first = sh.first_bin;
  if (found != 0x7fffffff && first == found) sh.before = (found == j0) ? mine_before : mine_before + a;
  __syncthreads();
  before_out = sh.before;
  total_out = sh.red64[(blockDim.x >> 5) - 1];
  const int result = first == 0x7fffffff ? -1 : first;
  __syncthreads();
  return result;
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, long ld, int n, float temperature, int top_k,
              float top_p, u64* __restrict__ rng_state, const int* __restrict__ state_index) {
  __shared__ Shared sh;
  gi::pdl_prologue();
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* row = logits + (size_t)r * ld;

  // ---- highest logit, first index on ties
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  if ((((uintptr_t)row) & 15) == 0) {
    // four logits per load, four loads in flight: a thread's candidates still come in increasing index order
    const int n4 = n / 4;
    const float4* row4 = reinterpret_cast<const float4*>(row);
    for (int i0 = tid; i0 < n4; i0 += 4 * blockDim.x) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        v[u] = i < n4 ? row4[i] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int base = 4 * (i0 + u * blockDim.x);
        if (v[u].x > bv) { bv = v[u].x; bi = base; }
        if (v[u].y > bv) { bv = v[u].y; bi = base + 1; }
        if (v[u].z > bv) { bv = v[u].z; bi = base + 2; }
        if (v[u].w > bv) { bv = v[u].w; bi = base + 3; }
      }
    }
    for (int i = 4 * n4 + tid; i < n; i += blockDim.x) {
      const float v = row[i];
      if (v > bv) { bv = v; bi = i; }
    }
  } else {
    for (int i = tid; i < n; i += blockDim.x) {
      const float v = row[i];
      if (v > bv) {  // strictly greater keeps the first; NaN never enters
        bv = v;
        bi = i;
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) {
      bv = ov;
      bi = oi;
    }
  }
  if (lane == 0) {
    sh.redv[warp] = bv;
    sh.redi[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    bv = lane < (int)(blockDim.x >> 5) ? sh.redv[lane] : -INFINITY;
    bi = lane < (int)(blockDim.x >> 5) ? sh.redi[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      sh.bestv = bv;
      sh.besti = bi == 0x7fffffff ? 0 : bi;
    }
  }
  __syncthreads();
  const float lmax = sh.bestv;
  if (!(temperature > 0.f) || rng_state == nullptr) {
    if (tid == 0) out[r] = sh.besti;
    return;
  }

  // ---- one draw from this row's xorshift64* stream
  if (tid == 0) {
    const int si = state_index ? state_index[r] : r;
    u64 s = rng_state[si];
    if (s == 0) s = 1;
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    rng_state[si] = s;
    sh.u = (float)((s * 0x2545F4914F6CDD1DULL) >> 40) / 16777216.0f;
  }

  // ---- the short way (see the head of this file)
  if (top_k > 0 && top_k < n && top_k <= FAST_CAP) {
    for (int b = tid; b < FAST_BINS; b += blockDim.x) sh.bins[b] = 0;
    if (tid == 0) sh.n_list = 0;
    __syncthreads();
    // (eight loads in flight per thread: one at a time, a sweep waits for the L2 cache 125 times in a row)
    const unsigned top_key = order_key(lmax);
    for (int i0 = 0; i0 < n; i0 += 8 * blockDim.x) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * blockDim.x + tid;
        v[u] = i < n ? row[i] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * blockDim.x + tid;
        const unsigned below = (top_key - order_key(v[u])) >> 16;       // a NaN's key is 0: far below
        if (i < n && below < FAST_BINS) atomicAdd(&sh.bins[below], 1u);
      }
    }
    __syncthreads();
    if (tid == 0) {
      // from the highest key's bin downwards until top_k keys are covered (or the bins end: then the long way)
      unsigned covered = 0;
      int b = 0;
      for (; b < FAST_BINS; ++b) {
        covered += sh.bins[b];
        if (covered >= (unsigned)top_k) break;
      }
      sh.first_bin = b;
      sh.n_list = b < FAST_BINS ? (int)covered : FAST_CAP + 1;
    }
    __syncthreads();
    const int total_c = sh.n_list;
    const unsigned last_bin = (unsigned)sh.first_bin;
    __syncthreads();
    if (total_c <= FAST_CAP) {
      if (tid == 0) sh.n_list = 0;
      __syncthreads();
      for (int i0 = 0; i0 < n; i0 += 8 * blockDim.x) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u * blockDim.x + tid;
          v[u] = i < n ? row[i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u * blockDim.x + tid;
          const unsigned key = order_key(v[u]);
          if (i < n && ((top_key - key) >> 16) <= last_bin) {
            const int at = atomicAdd(&sh.n_list, 1);
            sh.list[at] = ((u64)key << 32) | (u64)(~(unsigned)i);
          }
        }
      }
      __syncthreads();
      // bitonic sort, descending, over the next power of two (the padding, zeros, sorts to the end)
      int m = 1;
      while (m < total_c) m <<= 1;
      for (int i = total_c + tid; i < m; i += blockDim.x) sh.list[i] = 0;
      __syncthreads();
      for (int size = 2; size <= m; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
          for (int t = tid; t < m / 2; t += blockDim.x) {
            const int lo = 2 * t - (t & (stride - 1)), hi = lo + stride;
            const bool down = (lo & size) == 0;                  // this run sorts descending
            const u64 a = sh.list[lo], b = sh.list[hi];
            if ((a < b) == down) {
              sh.list[lo] = b;
              sh.list[hi] = a;
            }
          }
          __syncthreads();
        }
      }
      const int k = top_k < total_c ? top_k : total_c;
      auto weight_at = [&](int j) { return fixed_weight(key_value((unsigned)(sh.list[j] >> 32)), lmax, temperature); };
      u64 upto = 0, total = 0, unused = 0;
      first_reaching(sh, k, 0, ~(u64)0, weight_at, upto, total);                      // (only the total is wanted here)
      int kept = k;
      u64 mass = total;
      if (top_p < 1.0f && total > 0) {
        u64 target = (u64)ceil((double)top_p * (double)total);
        target = target < 1 ? 1 : (target > total ? total : target);
        const int j = first_reaching(sh, k, 0, target, weight_at, upto, unused);
        if (j >= 0) {
          kept = j + 1;
          mass = upto + weight_at(j);
        }
      }
      u64 target = (u64)ceil((double)sh.u * (double)mass);
      target = target < 1 ? 1 : (target > mass ? mass : target);
      int pick = first_reaching(sh, kept, 0, target, weight_at, upto, unused);
      if (pick < 0) pick = kept - 1;
      if (tid == 0) out[r] = mass > 0 ? (int)(~(unsigned)(sh.list[pick] & 0xffffffffu)) : sh.besti;
      return;
    }
  }

  // ---- the short way without a top_k: every logit is a candidate.  Weights are summed by the logits' distance below
  // the highest one, in 2048 equal steps over the 29 T within which a weight is not yet zero in fixed point (the
  // step is monotone in the logit, so the bins keep the descending order); the bins say in which one the cut of
  // top_p and the draw fall, and only that bin's logits are gathered and sorted.  If a bin holds more than the list
  // takes, the long way below does the whole job.
  if (!(top_k > 0 && top_k < n)) {
    constexpr int WBINS = 2048;
    // a bin's sum as two 32-bit words (additions of 32 bits to shared memory are one instruction, those of 64 bits a
    // compare-and-swap loop): the low word's overflow is carried into the high word by whoever caused it
    unsigned* wlo = sh.bins;
    unsigned* whi = sh.bins + WBINS;
    auto wb_at = [&](int b) { return ((u64)whi[b] << 32) | (u64)wlo[b]; };
    const float per_logit = (float)WBINS / (29.0f * temperature);
    auto bin_of = [&](float v) { return (int)fminf((lmax - v) * per_logit, 1.0e9f); };      // >= WBINS: weight 0
    for (int b = tid; b < 2 * WBINS; b += blockDim.x) sh.bins[b] = 0;
    __syncthreads();
    u64 rest_mine = 0;
    for (int i0 = 0; i0 < n; i0 += 8 * blockDim.x) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * blockDim.x + tid;
        v[u] = i < n ? row[i] : __int_as_float(0x7fc00000);        // past the row: not a number, weight 0
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const u64 w = fixed_weight(v[u], lmax, temperature);
        const int below = bin_of(v[u]);
        if (w == 0) continue;
        if (below < WBINS) {
          const unsigned lo = (unsigned)w, hi = (unsigned)(w >> 32);
          const unsigned old = atomicAdd(&wlo[below], lo);
          const unsigned carry = (old + lo < old) ? 1u : 0u;
          if (hi + carry) atomicAdd(&whi[below], hi + carry);
        } else {
          rest_mine += w;                                             // (none, by the choice of the steps)
        }
      }
    }
    const u64 rest = block_sum_u64(sh, rest_mine);                  // (synchronises)
    // gathers bin `b` into the list, sorted; false if it does not fit
    auto gather_sorted = [&](int b) -> bool {
      __syncthreads();
      if (tid == 0) sh.n_list = 0;
      __syncthreads();
      for (int i0 = 0; i0 < n; i0 += 8 * blockDim.x) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u * blockDim.x + tid;
          v[u] = i < n ? row[i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u * blockDim.x + tid;
          const unsigned key = order_key(v[u]);
          if (i < n && bin_of(v[u]) == b && fixed_weight(v[u], lmax, temperature) > 0) {
            const int at = atomicAdd(&sh.n_list, 1);
            if (at < FAST_CAP) sh.list[at] = ((u64)key << 32) | (u64)(~(unsigned)i);
          }
        }
      }
      __syncthreads();
      const int c = sh.n_list;
      if (c > FAST_CAP) return false;
      int m = 1;
      while (m < c) m <<= 1;
      for (int i = c + tid; i < m; i += blockDim.x) sh.list[i] = 0;
      __syncthreads();
      for (int size = 2; size <= m; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
          for (int t = tid; t < m / 2; t += blockDim.x) {
            const int lo = 2 * t - (t & (stride - 1)), hi = lo + stride;
            const bool down = (lo & size) == 0;
            const u64 a = sh.list[lo], bb = sh.list[hi];
            if ((a < bb) == down) {
              sh.list[lo] = bb;
              sh.list[hi] = a;
            }
          }
          __syncthreads();
        }
      }
      return true;
    };
    auto weight_of = [&](int j) { return fixed_weight(key_value((unsigned)(sh.list[j] >> 32)), lmax, temperature); };
    u64 before = 0, bins_total = 0, unused = 0;
    first_reaching(sh, WBINS, 0, ~(u64)0, wb_at, before, bins_total);                 // (only the total is wanted here)
    const u64 total = bins_total + rest;
    bool fits = total > 0;
    u64 mass = total;
    int cut_bin = WBINS;                 // bins before this one are kept whole; of this one, the first cut_count entries
    int cut_count = 0;
    if (fits && top_p < 1.0f) {
      u64 target = (u64)ceil((double)top_p * (double)total);
      target = target < 1 ? 1 : (target > total ? total : target);
      cut_bin = first_reaching(sh, WBINS, 0, target, wb_at, before, unused);
      fits = cut_bin >= 0 && gather_sorted(cut_bin);
      if (fits) {
        u64 upto = 0;
        const int j = first_reaching(sh, sh.n_list, before, target, weight_of, upto, unused);
        fits = j >= 0;                   // (always: the bin's sum reaches the target)
        if (fits) {
          cut_count = j + 1;
          mass = upto + weight_of(j);
        }
      }
    }
    if (fits) {
      u64 target = (u64)ceil((double)sh.u * (double)mass);
      target = target < 1 ? 1 : (target > mass ? mass : target);
      const int draw_bin = first_reaching(sh, WBINS, 0, target, wb_at, before, unused);
      fits = draw_bin >= 0;
      if (fits && draw_bin != cut_bin) fits = gather_sorted(draw_bin);      // (the cut's bin is still in the list)
      if (fits) {
        const int limit = draw_bin == cut_bin ? cut_count : sh.n_list;
        u64 upto = 0;
        int pick = first_reaching(sh, limit, before, target, weight_of, upto, unused);
        if (pick < 0) pick = limit - 1;
        if (tid == 0) out[r] = pick >= 0 ? (int)(~(unsigned)(sh.list[pick] & 0xffffffffu)) : sh.besti;
        return;
      }
    }
    __syncthreads();
  }

  const int ishift = index_start_shift(n);
  unsigned val;
  u64 before, equal;

  // ---- top-k: the k-th highest key, and up to which token id keys equal to it still count
  unsigned kth = 0;
  int kth_last = n;  // ids <= kth_last with key == kth are candidates
  if (top_k > 0 && top_k < n) {
    radix_descend<true>(sh, n, 24, (u64)top_k, [&](int i, unsigned& v) { v = order_key(row[i]); return true; },
                        [&](int, unsigned) { return (u64)1; }, val, before, equal);
    kth = val;
    const u64 need = (u64)top_k - before;
    if (need < equal) {
      radix_descend<false>(sh, n, ishift, need, [&](int i, unsigned& v) { v = (unsigned)i; return order_key(row[i]) == kth; },
                           [&](int, unsigned) { return (u64)1; }, val, before, equal);
      kth_last = (int)val;
    }
  }
  auto candidate = [&](int i, unsigned key) { return key > kth || (key == kth && i <= kth_last); };

  // ---- total weight of the candidates
  u64 mine = 0;
#pragma unroll 8
  for (int i = tid; i < n; i += blockDim.x) {
    const float v = row[i];
    if (candidate(i, order_key(v))) mine += fixed_weight(v, lmax, temperature);
  }
  const u64 total = block_sum_u64(sh, mine);

  // ---- top-p: where the running share first reaches top_p
  unsigned cut = 0;
  int cut_last = n;
  u64 mass = total;
  if (top_p < 1.0f && total > 0) {
    u64 target = (u64)ceil((double)top_p * (double)total);
    target = target < 1 ? 1 : (target > total ? total : target);
    radix_descend<true>(sh, n, 24, target, [&](int i, unsigned& v) { v = order_key(row[i]); return candidate(i, v); },
                        [&](int, unsigned v) { return fixed_weight(key_value(v), lmax, temperature); }, val, before, equal);
    cut = val;
    const u64 wc = fixed_weight(key_value(cut), lmax, temperature);
    if (wc > 0) {
      const u64 n_eq = equal / wc;
      u64 j = (target - before + wc - 1) / wc;
      j = j < 1 ? 1 : (j > n_eq ? n_eq : j);
      mass = before + j * wc;
      if (j < n_eq) {
        radix_descend<false>(sh, n, ishift, j,
                             [&](int i, unsigned& v) { v = (unsigned)i; return order_key(row[i]) == cut && candidate(i, cut); },
                             [&](int, unsigned) { return (u64)1; }, val, before, equal);
        cut_last = (int)val;
      }
    } else {
      mass = before + equal;
    }
  }
  auto kept = [&](int i, unsigned key) { return candidate(i, key) && (key > cut || (key == cut && i <= cut_last)); };

  // ---- the draw: the first kept candidate, in descending order, at which the running sum reaches u * mass
  u64 target = (u64)ceil((double)sh.u * (double)mass);
  target = target < 1 ? 1 : (target > mass ? mass : target);
  radix_descend<true>(sh, n, 24, target, [&](int i, unsigned& v) { v = order_key(row[i]); return kept(i, v); },
                      [&](int, unsigned v) { return fixed_weight(key_value(v), lmax, temperature); }, val, before, equal);
  const unsigned sel = val;
  const u64 ws = fixed_weight(key_value(sel), lmax, temperature);
  u64 jj = 1;
  if (ws > 0) {
    const u64 n_eq = equal / ws;
    jj = (target - before + ws - 1) / ws;
    jj = jj < 1 ? 1 : (jj > n_eq ? n_eq : jj);
  }
  radix_descend<false>(sh, n, ishift, jj, [&](int i, unsigned& v) { v = (unsigned)i; return order_key(row[i]) == sel && kept(i, sel); },
                       [&](int, unsigned) { return (u64)1; }, val, before, equal);
  if (tid == 0) out[r] = equal > 0 ? (int)val : sh.besti;
}

}  // namespace

extern "C" int gi_sample(int* out_tokens, const float* logits, long ld, int n_rows, int vocab, float temperature,
                         int top_k, float top_p, unsigned long long* rng_state, const int* state_index, void* stream) {
  if (n_rows <= 0) return GI_OK;
  if (vocab <= 0) return gi::fail(GI_ERR_ARG, "sample: empty vocabulary");
  if (temperature > 0.f && !rng_state) return gi::fail(GI_ERR_ARG, "sample: temperature sampling needs generator states");
  if (top_k < 0) return gi::fail(GI_ERR_ARG, "sample: top_k must not be negative");
  return gi::check(gi::launch(sample_kernel, dim3(n_rows), dim3(THREADS), 0, (cudaStream_t)stream, out_tokens, logits, ld, vocab,
                              temperature, top_k, top_p, rng_state, state_index), "sample");
}
