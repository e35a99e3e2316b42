// Decode attention over the paged cache on tensor cores: one token per sequence, bfloat16, head size 64 or 128.
//
// Same formula as the plain kernel (src/model.rs:1320-1419) and the same cut of the work as the
// reference's attention_partial_gqa + attention_combine (src/cuda.rs:1684-1865, :2806-2839): a block takes
// one kv head of one sequence and one slice of its context, and all query heads of the group share every
// key and value row that is read.  Here the group's heads (up to 16) are the rows of an m16n8k16 tile:
// scores S = Q K^T and outputs O += P V are mma.sync products with 32-bit accumulators, softmax statistics
// and the running rescale are 32-bit.  Each of the 4 warps walks its own tiles of 16 or 32 keys; keys and values
// arrive by cp.async into a per-warp ring of shared-memory stages (16-byte chunks, XOR-swizzled for
// ldmatrix), so the next tiles are in flight while one is used.  Warps are merged through shared memory in
// warp order.  A context is cut either into a fixed number of equal slices (few sequences: one wave of blocks) or
// into slices of a fixed number of tiles counted from the start of the sequence's own span (many or unequal
// sequences: every block has the same work, short sequences use fewer blocks, and a launch's other slices leave at
// once).  Slices are merged in slice order: by the block of a (sequence, kv head) that finishes last, which an atomic
// counter tells (nobody waits; the role of the reference's attention_combine, src/cuda.rs:2806-2839), or, when the
// caller gives no counters, by the combine kernel.
#include <math.h>

#include <mutex>

#include "api.h"
#include "common.cuh"
#include "mma_utils.cuh"

//
// The kernel can also take the rows as the q/k/v product left them (not rotated, tiles cut between the product's blocks
// still as partial sums) together with the step's table of angles: every block then sums, rotates and rounds its own
// query heads into shared memory, and the block that holds a sequence's newest position does the same for the kv
// head's key and value, stores them in the cache (src/model.rs:1046-1048) and reads them back with the rest of its
// last tile.  That is the rotary kernel's work (rope_cache.cu, the same roundings) without its launch.
namespace {

constexpr int WARPS = 4;

// What the kernel needs to rotate and store by itself; table == nullptr: the queries come rotated, the cache is complete.
struct RopeInside {
  const float2* table;   // [sequences][rot / 2] (cos, sin) of each sequence's newest position; written by a kernel of this step
  gi_settle_t st;        // partial sums that the q/k/v product left (partials == nullptr: none)
  int rot;               // rotated part of a head, pairs (i, i + rot / 2)
};

template <int HD, int KT, int STAGES>
__global__ void __launch_bounds__(WARPS * 32)
attn_decode_tc_kernel(__nv_bfloat16* __restrict__ out, long ldo, float* __restrict__ part_o, float* __restrict__ part_ml,
                      const __nv_bfloat16* q /* written by the kernel before: see gi::pdl_wait */, long ldq, __nv_bfloat16* kcache,
                      __nv_bfloat16* vcache, const int* __restrict__ block_table, int max_pages,
                      const int* __restrict__ seq_slots, const int* __restrict__ seq_lens, int n_heads, int n_kv,
                      float scale, int window, int n_splits, int own_tiles, int* __restrict__ counters, RopeInside rope) {
  constexpr int CH = HD / 8;                     // 16-byte chunks per row
  constexpr int TILE_BYTES = KT * HD * 2;        // one K or V tile
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;    // K then V
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* q_s = smem;                                       // [16][HD] bf16, swizzled
  unsigned char* ring = smem + 16 * HD * 2;                        // [WARPS][STAGES][K tile | V tile]
  // Lengths, slots and the block table were uploaded before the step's first kernel, and no kernel of the step
  // writes a cached position other than each sequence's last one: the first tiles of keys and values are
  // requested before the dependency wait, while the kernel before this one (which writes the last position and
  // the queries) still runs.  Only the tile that holds the last position waits.
  gi::pdl_launch_dependents();

  const int group = n_heads / n_kv;
  const int chunks = (group + 15) / 16;
  const int b = blockIdx.z, kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks, sp = blockIdx.x;
  const int g0 = chunk * 16, gcount = min(16, group - g0);
  const int h0 = kvh * group + g0;
  const int slot = gi::ld_step(seq_slots + b);
  const int len = gi::ld_step(seq_lens + b);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  int t_first = 0;
  if (window > 0) t_first = max(0, len - window);
  const int t_base = (t_first / KT) * KT;
  const int tiles = len > t_base ? (len - t_base + KT - 1) / KT : 0;
  // own_tiles > 0: a slice is that many tiles of the sequence's own span; else the span is cut into n_splits equal slices
  const int per = own_tiles > 0 ? own_tiles : (tiles + n_splits - 1) / n_splits;
  const int used = per > 0 ? max(1, (tiles + per - 1) / per) : 1;      // slices of this sequence that hold keys
  const int tile_lo = sp * per, tile_hi = min(tiles, tile_lo + per);
  if (sp >= used) {
    // nothing of this sequence lies in this slice.  With counters the merging block reads the `used` first slices
    // only; without, the combine kernel reads every slice of the launch and must find this one marked empty.
    if (counters == nullptr && n_splits > 1) {
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
    // 32 keys x CH chunks for K and for V, 16 bytes per lane and instruction
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

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[i][c] = 0.f;

  // Rotating inside: which heads of the packed row this block works on (its query heads; with the newest position in
  // its slice also the kv head's key and value) and, looked up before the wait, which of the product's blocks hold
  // pieces of each (the tables of the product's cut are uploaded once and never written by a kernel).
  __shared__ gi_settle_span s_span[18];
  const bool inside = rope.table != nullptr;
  const bool stores = inside && tile_hi == tiles;
  const int n_items = gcount + (stores ? 2 : 0);
  auto item_col = [&](int item) {
    return (item < gcount ? h0 + item : (item == gcount ? n_heads + kvh : n_heads + n_kv + kvh)) * HD;
  };
  if (inside) {
    if (tid < n_items) {
      gi_settle_span none = {0, 0, 0};
      s_span[tid] = rope.st.partials != nullptr ? gi_span_of(rope.st, item_col(tid)) : none;
    }
    for (int idx = tid; idx < 16 * CH; idx += WARPS * 32)
      if (idx / CH >= gcount) *reinterpret_cast<uint4*>(q_s + gi::swz<CH>(idx / CH, idx % CH)) = make_uint4(0, 0, 0, 0);
  }

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
  if (inside) __syncthreads();    // the spans are in shared memory
  gi::pdl_wait();
  if (!inside) {
    if (late_stage >= 0) {        // a short slice: its last tile is among the first ones; fetch it now and let it land
      issue(tiles - 1, late_stage);
      gi::cp_async_commit();
      gi::cp_async_wait<0>();
    }
    // queries of the group's heads as rows 0..gcount-1 of a 16-row tile (the others zero)
    for (int idx = tid; idx < 16 * CH; idx += WARPS * 32) {
      const int r = idx / CH, c = idx % CH;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < gcount) v = *reinterpret_cast<const uint4*>(q + (size_t)b * ldq + (size_t)(h0 + r) * HD + c * 8);
      *reinterpret_cast<uint4*>(q_s + gi::swz<CH>(r, c)) = v;
    }
    __syncthreads();
  } else {
    // A thread takes two columns of a head at a time: a rotated pair (i, i + rot / 2), or two neighbours past the
    // rotated part or of the value.  Each column is what the product stored or the sum of its pieces in the order of
    // the K ranges, rounded to bfloat16 as the product would have stored it; rotated in 32-bit; rounded again.
    const int half = rope.rot >> 1;
    const __nv_bfloat16* row = q + (size_t)b * ldq;
    const float2* cs = rope.table + (size_t)b * half;
    size_t cache_row = 0;
    if (stores) {
      const int pos = max(len - 1, 0);
      const int page = slot >= 0 ? gi::ld_step(block_table + (size_t)slot * max_pages + pos / PAGE_TOKENS) : 0;
      cache_row = (((size_t)page * n_kv + kvh) * PAGE_TOKENS + (pos % PAGE_TOKENS)) * HD;
    }
    for (int idx = tid; idx < n_items * (HD / 2); idx += WARPS * 32) {
      const int item = idx / (HD / 2), i = idx % (HD / 2);
      const int col0 = item_col(item);
      const bool is_v = item == gcount + 1;
      const bool rotate = !is_v && i < half;
      const int ea = is_v ? 2 * i : (rotate ? i : rope.rot + 2 * (i - half));
      const int eb = rotate ? i + half : ea + 1;
      const gi_settle_span spn = s_span[item];
      float a, c;
      if (spn.c_first != spn.c_last) {
        const float2 sum = gi_sum_pieces2(rope.st, spn, b, col0 + ea, col0 + eb);
        a = __bfloat162float(__float2bfloat16_rn(sum.x));
        c = __bfloat162float(__float2bfloat16_rn(sum.y));
      } else {
        a = __bfloat162float(row[col0 + ea]);
        c = __bfloat162float(row[col0 + eb]);
      }
      if (rotate) gi::rotate_pair(a, c, cs[i], &a, &c);
      const __nv_bfloat16 va = __float2bfloat16_rn(a), vc = __float2bfloat16_rn(c);
      if (item < gcount) {
        *reinterpret_cast<__nv_bfloat16*>(q_s + gi::swz<CH>(item, ea >> 3) + (ea & 7) * 2) = va;
        *reinterpret_cast<__nv_bfloat16*>(q_s + gi::swz<CH>(item, eb >> 3) + (eb & 7) * 2) = vc;
      } else {
        __nv_bfloat16* dst = (is_v ? vcache : kcache) + cache_row;
        dst[ea] = va;
        dst[eb] = vc;
      }
    }
    // the newest key and value go through memory: stored here, fetched below like every other row of the last tile
    if (stores) __threadfence();
    __syncthreads();
    if (late_stage >= 0) {
      issue(tiles - 1, late_stage);
      gi::cp_async_commit();
      gi::cp_async_wait<0>();
    }
  }
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
    // matrices: (rows 0-7, k lo), (rows 8-15, k lo), (rows 0-7, k hi), (rows 8-15, k hi) = a0..a3
    const int r = (lane & 7) + ((lane >> 3) & 1) * 8, c = ks * 2 + (lane >> 4);
    gi::ldmatrix_x4(qf[ks], gi::smem_u32(q_s + gi::swz<CH>(r, c)));
  }

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

    // S = Q K^T : 4 key tiles of 8, HD/16 steps
    float s[KT / 8][4];
#pragma unroll
    for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[nt][c] = 0.f;
#pragma unroll
    for (int nt = 0; nt < KT / 8; ++nt) {
#pragma unroll
      for (int kp = 0; kp < HD / 32; ++kp) {
        // four 8x8 matrices: keys nt*8.., dims [kp*32, +8), [+8, +16), [+16, +24), [+24, +32)
        uint32_t kb[4];
        const int r = nt * 8 + (lane & 7), c = kp * 4 + (lane >> 3);
        gi::ldmatrix_x4(kb, gi::smem_u32(ks + gi::swz<CH>(r, c)));
        gi::mma_16816(s[nt], qf[kp * 2], kb[0], kb[1]);
        gi::mma_16816(s[nt], qf[kp * 2 + 1], kb[2], kb[3]);
      }
    }
    // mask and running softmax (rows g and g + 8)
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key = t0 + nt * 8 + 2 * t + (c & 1);
        const bool ok = key < len && key >= t_first;
        s[nt][c] = ok ? s[nt][c] * sl2 : -INFINITY;
        tmax[c >> 1] = fmaxf(tmax[c >> 1], s[nt][c]);
      }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
      tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
      const float m_new = fmaxf(m_run[h], tmax[h]);       // finite: every tile holds at least one live key
      alpha[h] = (m_run[h] == -INFINITY) ? 0.f : exp2f(m_run[h] - m_new);
      m_run[h] = m_new;
    }
    float psum[2] = {0.f, 0.f};
    uint32_t pf[KT / 16][4];
#pragma unroll
    for (int nt = 0; nt < KT / 8; ++nt) {
      const float p0 = exp2f(s[nt][0] - m_run[0]), p1 = exp2f(s[nt][1] - m_run[0]);
      const float p2 = exp2f(s[nt][2] - m_run[1]), p3 = exp2f(s[nt][3] - m_run[1]);
      psum[0] += p0 + p1;
      psum[1] += p2 + p3;
      pf[nt / 2][(nt & 1) * 2] = gi::pack_bf16(p0, p1);       // a0 / a2: row g
      pf[nt / 2][(nt & 1) * 2 + 1] = gi::pack_bf16(p2, p3);   // a1 / a3: row g + 8
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 1);
      psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 2);
      l_run[h] = l_run[h] * alpha[h] + psum[h];
    }
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[0];
      o[i][2] *= alpha[1];
      o[i][3] *= alpha[1];
    }
    // O += P V : 2 steps of 16 keys, HD/8 output tiles of 8 dims, two tiles per ldmatrix
#pragma unroll
    for (int kk = 0; kk < KT / 16; ++kk) {
#pragma unroll
      for (int dp = 0; dp < HD / 16; ++dp) {
        // transposed 8x8 matrices: (keys kk*16.., dims dp*16..), (keys +8, same dims), (keys, dims +8), (keys +8, dims +8)
        uint32_t vb[4];
        const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = dp * 2 + (lane >> 4);
        gi::ldmatrix_x4_trans(vb, gi::smem_u32(vs + gi::swz<CH>(r, c)));
        gi::mma_16816(o[dp * 2], pf[kk], vb[0], vb[1]);
        gi::mma_16816(o[dp * 2 + 1], pf[kk], vb[2], vb[3]);
      }
    }
    __syncwarp();
    stage = (stage + 1) % STAGES;
  }
  gi::cp_async_wait<0>();
  __syncthreads();

  // merge the warps (reusing the ring): natural-log maxima so that the combine kernel can go on.  Only the rows
  // that hold a head are written (a group of 4 heads uses 4 of the tile's 16 rows); rows are HD + 8 floats apart,
  // which spreads the eight rows a warp writes at once over the banks.
  constexpr int MROW = HD + 8;
  float* Mo = reinterpret_cast<float*>(ring);            // [WARPS][16][MROW]
  float* Mm = Mo + WARPS * 16 * MROW;                    // [WARPS][16]
  float* Ml = Mm + WARPS * 16;                           // [WARPS][16]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = g + h * 8;
    if (r >= gcount) continue;
    if (t == 0) {
      Mm[warp * 16 + r] = m_run[h];
      Ml[warp * 16 + r] = l_run[h];
    }
#pragma unroll
    for (int i = 0; i < HD / 8; ++i)
      *reinterpret_cast<float2*>(Mo + (warp * 16 + r) * MROW + i * 8 + 2 * t) = make_float2(o[i][h * 2], o[i][h * 2 + 1]);
  }
  __syncthreads();
  for (int idx = tid; idx < gcount * HD; idx += WARPS * 32) {
    const int r = idx / HD, d = idx % HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, Mm[w * 16 + r]);
    float tot = 0.f, val = 0.f;
    if (mm != -INFINITY) {
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float mw = Mm[w * 16 + r];
        if (mw == -INFINITY) continue;
        const float wgt = exp2f(mw - mm);
        tot += Ml[w * 16 + r] * wgt;
        val += Mo[(w * 16 + r) * MROW + d] * wgt;
      }
    }
    const int h = h0 + r;
    if (n_splits == 1 || (used == 1 && counters != nullptr)) {
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
  if (counters == nullptr || used == 1 || n_splits == 1) return;

  // The block of this (sequence, kv head, head chunk) that arrives last merges the slices, in slice order and from
  // memory (its own slice too), so the result does not depend on which block that is.  Nobody waits for anybody.
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int* c = counters + (size_t)b * gridDim.y + blockIdx.y;
    const int seen = atomicAdd(c, 1);
    s_last = (seen == used - 1);
    if (s_last) *c = 0;                                   // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // maxima and sums of every slice of the block's heads into shared memory (the ring is free by now): one round of
  // loads for all of them; then each head's largest maximum and every slice's weight exp(m_s - m)
  float* Wt = reinterpret_cast<float*>(ring);             // [gcount][used] weights, then [gcount] totals
  float* Tot = Wt + 16 * n_splits;
  if (32 * n_splits + 16 <= (int)(WARPS * STAGES * STAGE_BYTES / sizeof(float))) {
    for (int i = tid; i < gcount * used; i += WARPS * 32) {
      const int r = i / used, sl = i % used;
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml) + ((size_t)b * n_heads + h0 + r) * n_splits + sl);
      Wt[r * n_splits + sl] = ml.x;
      Wt[16 * n_splits + 16 + r * n_splits + sl] = ml.y;                  // sums, behind the totals
    }
    __syncthreads();
    if (tid < gcount) {
      float mm = -INFINITY;
      for (int sl = 0; sl < used; ++sl) mm = fmaxf(mm, Wt[tid * n_splits + sl]);
      float tot = 0.f;
      for (int sl = 0; sl < used; ++sl) {
        const float m = Wt[tid * n_splits + sl];
        const float w = (m == -INFINITY || mm == -INFINITY) ? 0.f : expf(m - mm);
        Wt[tid * n_splits + sl] = w;
        tot += Wt[16 * n_splits + 16 + tid * n_splits + sl] * w;
      }
      Tot[tid] = tot;
    }
    __syncthreads();
    for (int idx = tid; idx < gcount * HD; idx += WARPS * 32) {
      const int r = idx / HD, d = idx % HD;
      const size_t p0 = ((size_t)b * n_heads + h0 + r) * n_splits;
      float val = 0.f;
      for (int s0 = 0; s0 < used; s0 += 8) {              // eight slices' loads together
        float o8[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o8[j] = (s0 + j < used) ? __ldcg(part_o + (p0 + s0 + j) * HD + d) : 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (s0 + j < used) val += o8[j] * Wt[r * n_splits + s0 + j];
      }
      const float tot = Tot[r];
      out[(size_t)b * ldo + (size_t)(h0 + r) * HD + d] = __float2bfloat16_rn(tot > 0.f ? val / tot : 0.f);
    }
    return;
  }
  for (int idx = tid; idx < gcount * HD; idx += WARPS * 32) {           // more slices than the table holds: the plain way
    const int r = idx / HD, d = idx % HD;
    const int h = h0 + r;
    const size_t p0 = ((size_t)b * n_heads + h) * n_splits;
    const float2* ml = reinterpret_cast<const float2*>(part_ml) + p0;
    float mm = -INFINITY;
    for (int sl = 0; sl < used; ++sl) mm = fmaxf(mm, __ldcg(ml + sl).x);
    float tot = 0.f, val = 0.f;
    if (mm != -INFINITY) {
      for (int sl = 0; sl < used; ++sl) {
        const float2 m = __ldcg(ml + sl);
        if (m.x == -INFINITY) continue;
        const float w = expf(m.x - mm);
        tot += m.y * w;
        val += __ldcg(part_o + (p0 + sl) * HD + d) * w;
      }
    }
    out[(size_t)b * ldo + (size_t)h * HD + d] = __float2bfloat16_rn(tot > 0.f ? val / tot : 0.f);
  }
}

template <int HD, int KT, int STAGES>
int launch(dim3 grid, cudaStream_t s, __nv_bfloat16* out, long ldo, float* po, float* pml, const __nv_bfloat16* q, long ldq,
           __nv_bfloat16* kc, __nv_bfloat16* vc, const int* bt, int max_pages, const int* slots, const int* lens,
           int H, int KV, float scale, int window, int n_splits, int own_tiles, int* counters, RopeInside rope) {
  constexpr size_t ring = (size_t)WARPS * STAGES * 2 * KT * HD * 2;
  constexpr size_t merge = (size_t)(WARPS * 16 * (HD + 8) + 2 * WARPS * 16) * sizeof(float);
  constexpr size_t smem = 16 * HD * 2 + (ring > merge ? ring : merge);
  auto kern = attn_decode_tc_kernel<HD, KT, STAGES>;
  static bool configured[gi::MAX_DEVICES_SEEN] = {false};
  int dev;
  if (gi::unconfigured_here(configured, &dev)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "attention decode: %s", cudaGetErrorString(e));
    if (dev >= 0) configured[dev] = true;
  }
  return gi::check(gi::launch(kern, grid, dim3(WARPS * 32), smem, s, out, ldo, po, pml, q, ldq, kc, vc, bt, max_pages, slots, lens, H, KV,
                              scale, window, n_splits, own_tiles, counters, rope), "attention decode (tensor cores)");
}

}  // namespace

// The combine kernel lives in attention_generic.cu.
extern "C" int gi_attn_combine(void* out, long ldo, int dtype, const float* part_o, const float* part_ml, int n_seqs,
                               int n_heads, int hd, int n_splits, void* stream);

extern "C" int gi_attn_decode_tc_ex(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq,
                                    const void* kcache, const void* vcache, const int* block_table, int max_pages,
                                    const int* seq_slots, const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd,
                                    float scale, int window, int n_splits, int tile_keys, void* stream);
extern "C" int gi_attn_decode_tc_merged(void* out, long ldo, float* part_o, float* part_ml, int* counters, int n_counters,
                                        const void* q, long ldq, const void* kcache, const void* vcache,
                                        const int* block_table, int max_pages, const int* seq_slots, const int* seq_lens,
                                        int n_seqs, int n_heads, int n_kv, int hd, float scale, int window, int n_splits,
                                        int own_tiles, int tile_keys, int stages, void* stream);

extern "C" int gi_attn_decode_tc(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq,
                                 const void* kcache, const void* vcache, const int* block_table, int max_pages,
                                 const int* seq_slots, const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd,
                                 float scale, int window, int n_splits, void* stream) {
  return gi_attn_decode_tc_ex(out, ldo, part_o, part_ml, q, ldq, kcache, vcache, block_table, max_pages, seq_slots, seq_lens, n_seqs,
                              n_heads, n_kv, hd, scale, window, n_splits, 32, stream);
}

// tile_keys: 32 (one block per SM, deep rings) or 16 (two blocks per SM)
extern "C" int gi_attn_decode_tc_ex(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq,
                                    const void* kcache, const void* vcache, const int* block_table, int max_pages,
                                    const int* seq_slots, const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd,
                                    float scale, int window, int n_splits, int tile_keys, void* stream) {
  return gi_attn_decode_tc_merged(out, ldo, part_o, part_ml, nullptr, 0, q, ldq, kcache, vcache, block_table, max_pages, seq_slots,
                                  seq_lens, n_seqs, n_heads, n_kv, hd, scale, window, n_splits, 0, tile_keys, 0, stream);
}

// The same with the merge of the slices inside the kernel.  counters: one int per (sequence, kv head, chunk of 16
// heads), zero before the first use (the kernel leaves them zero); nullptr: the slices are merged by a second kernel.
// own_tiles > 0: slice s of a sequence holds tiles [s * own_tiles, (s + 1) * own_tiles) of `tile_keys` keys of its own
// span, whatever n_splits is (which must cover the longest span); 0: each span is cut into n_splits equal slices.
// stages: depth of each warp's ring of tiles (2, 3 or 4; 0: 3 at head size 128, 4 at head size 64).  Fewer stages
// mean less shared memory per block and so more blocks per SM.
namespace {
int decode_tc_impl(void* out, long ldo, float* part_o, float* part_ml, int* counters, int n_counters, const void* q, long ldq,
                   void* kcache, void* vcache, const int* block_table, int max_pages, const int* seq_slots, const int* seq_lens,
                   int n_seqs, int n_heads, int n_kv, int hd, float scale, int window, int n_splits, int own_tiles, int tile_keys,
                   int stages, RopeInside rope, void* stream) {
  if (n_seqs <= 0) return GI_OK;
  if (own_tiles < 0) return gi::fail(GI_ERR_ARG, "attention: tiles per slice cannot be negative");
  if (tile_keys != 16 && tile_keys != 32) return gi::fail(GI_ERR_ARG, "attention decode (tensor cores): tiles of %d keys, 16 or 32", tile_keys);
  if (hd != 64 && hd != 128) return gi::fail(GI_ERR_UNSUPPORTED, "attention decode (tensor cores): head size %d, only 64 and 128", hd);
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0)
    return gi::fail(GI_ERR_ARG, "attention: %d heads do not divide into %d kv heads", n_heads, n_kv);
  if (n_splits < 1) return gi::fail(GI_ERR_ARG, "attention: at least one slice");
  if (n_splits > 1 && (!part_o || !part_ml)) return gi::fail(GI_ERR_ARG, "attention: slices need scratch memory");
  if (ldq % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)kcache & 15) || ((uintptr_t)vcache & 15))
    return gi::fail(GI_ERR_UNSUPPORTED, "attention decode (tensor cores): queries and cache must be 16-byte aligned");
  const int group = n_heads / n_kv;
  const int chunks = (group + 15) / 16;
  if ((long)n_kv * chunks > 65535 || n_seqs > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "attention: more than 65535 sequences or kv heads in one launch");
  if (counters != nullptr && (long)n_seqs * n_kv * chunks > n_counters)
    return gi::fail(GI_ERR_ARG, "attention: %ld counters are needed for the merge, %d were given", (long)n_seqs * n_kv * chunks, n_counters);
  dim3 grid(n_splits, n_kv * chunks, n_seqs);
  cudaStream_t s = (cudaStream_t)stream;
  int rc;
#define GI_DECODE_TC(HD_, KT_, ST_)                                                                                          \
  rc = launch<HD_, KT_, ST_>(grid, s, (__nv_bfloat16*)out, ldo, part_o, part_ml, (const __nv_bfloat16*)q, ldq,               \
                             (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, block_table, max_pages, seq_slots,             \
                             seq_lens, n_heads, n_kv, scale, window, n_splits, own_tiles, counters, rope)
  if (stages == 0) stages = hd == 128 ? 3 : 4;
  if (stages < 2 || stages > 4) return gi::fail(GI_ERR_ARG, "attention decode (tensor cores): rings of %d stages, 2 to 4", stages);
  if (hd == 128 && tile_keys == 32) GI_DECODE_TC(128, 32, 3);
  else if (hd == 128 && stages == 2) GI_DECODE_TC(128, 16, 2);
  else if (hd == 128) GI_DECODE_TC(128, 16, 3);
  else if (tile_keys == 32) GI_DECODE_TC(64, 32, 4);
  else if (stages == 2) GI_DECODE_TC(64, 16, 2);
  else if (stages == 3) GI_DECODE_TC(64, 16, 3);
  else GI_DECODE_TC(64, 16, 4);
#undef GI_DECODE_TC
  if (rc != GI_OK) return rc;
  if (n_splits > 1 && counters == nullptr) return gi_attn_combine(out, ldo, GI_BF16, part_o, part_ml, n_seqs, n_heads, hd, n_splits, stream);
  return GI_OK;
}
}  // namespace

extern "C" int gi_attn_decode_tc_merged(void* out, long ldo, float* part_o, float* part_ml, int* counters, int n_counters,
                                        const void* q, long ldq, const void* kcache, const void* vcache,
                                        const int* block_table, int max_pages, const int* seq_slots, const int* seq_lens,
                                        int n_seqs, int n_heads, int n_kv, int hd, float scale, int window, int n_splits,
                                        int own_tiles, int tile_keys, int stages, void* stream) {
  const RopeInside none = {nullptr, {nullptr, nullptr, nullptr, nullptr, 0}, 0};
  // without a table of angles the kernel only reads the cache
  return decode_tc_impl(out, ldo, part_o, part_ml, counters, n_counters, q, ldq, const_cast<void*>(kcache), const_cast<void*>(vcache),
                        block_table, max_pages, seq_slots, seq_lens, n_seqs, n_heads, n_kv, hd, scale, window, n_splits, own_tiles,
                        tile_keys, stages, none, stream);
}

// The same for rows that are not rotated yet (one row per sequence: the packed [q | k | v] of its newest token, as the
// q/k/v product left it; `settle`: that product's pending partial sums, partials == nullptr for none).  The kernel
// rotates q and k by `table` ([sequences][rot / 2] (cos, sin)), pairs (i, i + rot / 2), and stores k and v at each
// sequence's position (length - 1) itself: the work of gi_rope_cache_write for a decode step, without its launch.
extern "C" int gi_attn_decode_tc_rope(void* out, long ldo, float* part_o, float* part_ml, int* counters, int n_counters,
                                      const void* qkv, long ld, void* kcache, void* vcache, const int* block_table,
                                      int max_pages, const int* seq_slots, const int* seq_lens, int n_seqs, int n_heads,
                                      int n_kv, int hd, float scale, int window, int n_splits, int own_tiles, int tile_keys,
                                      int stages, const float* table, int rot, gi_settle_t settle, void* stream) {
  if (!table) return gi::fail(GI_ERR_ARG, "attention decode with rotation: no table of angles");
  if (rot < 0 || rot > hd || rot % 2 != 0) return gi::fail(GI_ERR_ARG, "attention decode with rotation: rotary size %d does not fit head size %d", rot, hd);
  if (settle.partials != nullptr && settle.nt < n_seqs)
    return gi::fail(GI_ERR_ARG, "attention decode with rotation: partial sums of a product of %d rows for %d sequences", settle.nt, n_seqs);
  const RopeInside rope = {(const float2*)table, settle, rot};
  return decode_tc_impl(out, ldo, part_o, part_ml, counters, n_counters, qkv, ld, kcache, vcache, block_table, max_pages, seq_slots,
                        seq_lens, n_seqs, n_heads, n_kv, hd, scale, window, n_splits, own_tiles, tile_keys, stages, rope, stream);
}

// ------------------------------------------------------------------------------------------------------
// The variant that brings its own scratch (see attention_decode_noalloc.h for who needs it and its rules).
#include "attention_decode_noalloc.h"

namespace {

// Partial outputs first, then (maximum, sum) pairs.  In host code this name is only a handle for
// cudaGetSymbolAddress: it is not a device address and must never be handed to a kernel as one.
static __device__ __align__(256) float g_noalloc_scratch[GI_NOALLOC_SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;
float* g_noalloc_ptr[MAX_DEVICES] = {nullptr};
std::mutex g_noalloc_lock;

// The array's address on the current device, looked up once per device.
int noalloc_scratch(float** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "attention decode (no allocation): %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= MAX_DEVICES) return gi::fail(GI_ERR_UNSUPPORTED, "attention decode (no allocation): device %d, at most %d", dev, MAX_DEVICES);
  std::lock_guard<std::mutex> guard(g_noalloc_lock);
  if (g_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      return gi::fail(GI_ERR_CUDA, "attention decode (no allocation): the scratch array's address is not to be had: %s", cudaGetErrorString(e));
    g_noalloc_ptr[dev] = p;
  }
  *ptr = g_noalloc_ptr[dev];
  return GI_OK;
}

}  // namespace

extern "C" int gi_attn_decode_tc_noalloc(void* out, long ldo, const void* q, long ldq, const void* kcache,
                                         const void* vcache, const int* block_table, int max_pages,
                                         const int* seq_slots, const int* seq_lens, int n_seqs, int n_heads, int n_kv,
                                         int hd, float scale, int window, int n_splits, void* stream) {
  if (n_seqs <= 0) return GI_OK;
  if (n_splits < 1 || n_heads <= 0 || hd <= 0) return gi::fail(GI_ERR_ARG, "attention decode (no allocation): bad sizes");
  const long long need = (long long)n_seqs * n_heads * n_splits * (hd + 2);
  if (need > GI_NOALLOC_SCRATCH_FLOATS)
    return gi::fail(GI_ERR_UNSUPPORTED,
                    "attention decode (no allocation): %d sequences x %d heads x %d slices x (%d + 2) floats = %lld, the built-in "
                    "scratch holds %d; use fewer slices or the entry point that takes scratch",
                    n_seqs, n_heads, n_splits, hd, need, GI_NOALLOC_SCRATCH_FLOATS);
  float* scratch = nullptr;
  const int rc = noalloc_scratch(&scratch);
  if (rc != GI_OK) return rc;
  float* part_o = scratch;
  float* part_ml = scratch + (size_t)n_seqs * n_heads * n_splits * hd;
  return gi_attn_decode_tc(out, ldo, part_o, part_ml, q, ldq, kcache, vcache, block_table, max_pages, seq_slots, seq_lens,
                           n_seqs, n_heads, n_kv, hd, scale, window, n_splits, stream);
}
