// The decode step's product, bound by the bytes of W: out[M,N] (op)= A[M,K] * W[N,K]^T for up to 64 rows of
// activations, bfloat16, on tcgen05 tensor cores with the operands swapped: 128 rows of W are the "M" side of
// the instruction and the tokens its "N" side (16, 32 or 64), so the accumulator in tensor memory holds
// [128 features x tokens].
//
// One persistent block per SM.  The work is the list of (128-row tile of W, 64-column block of K) units.  Each
// block first takes an equal contiguous range of the units of the "shared" tiles ("stream-K"), then whole tiles
// of its own (see Plan), so every SM streams the same number of bytes whatever the matrix's shape.  Inside a
// block: one thread feeds a deep ring of shared-memory stages with TMA (a 16 KB box of W and the matching small
// box of activations per stage, so far more bytes are in flight than registers could hold); one thread issues
// the tcgen05.mma instructions; four warps drain finished accumulators (two buffers in tensor memory, so
// draining overlaps the next tile's products).  A tile whose K range lies in one block is finished there.  A
// tile cut between blocks leaves its partial sums in scratch; the block that arrives last (an atomic counter per
// tile; nobody waits) adds the partials in the order of the K ranges, so the sum does not depend on which block
// came last; since the shared units come first, that exchange is over long before the block's last tile is.
// Epilogues: store (bfloat16 or float), add into the float residual stream, or SwiGLU over gate/up rows
// interleaved in blocks of 8.  Once a block's own loads are issued it asks the L2 cache for the first units of
// the matrix that the next product in the stream will read, when the caller named it.
//
// The role in the reference: its decode matvec kernels (src/cuda.rs:1425-1434), which are bound by weight
// bytes too and keep a fixed summation order (src/cuda.rs:748-766).
#include <cuda.h>

#include "api.h"
#include "common.cuh"
#include "tc_utils.cuh"

namespace {

using namespace gi::tc;

constexpr int TILE_ROWS = 128;   // rows of W per tile = tensor-memory lanes
constexpr int BK = 64;           // K columns per unit = one 128-byte swizzle row
constexpr int THREADS = 192;     // warp 0: TMA, warp 1: MMA + tensor-memory allocation, warps 2-5: epilogue

// Time stamps for a timeline of a decode step (gi_gemm_stream_timeline): when a launch carries a buffer, each block
// notes the nanosecond clock at eight places of its life.  Without one (the usual case) a stamp is a predicated-off store.
constexpr int TL_EVENTS = 8;       // 0 entry, 1 set up, 2 the SM's number, 3 dependency wait over, 4 first stage landed,
                                   // 5 last load issued, 6 last product issued, 7 last epilogue done
constexpr int TL_BLOCKS = 256;     // blocks per launch that a buffer has room for
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define TL(ev) do { if (next.timeline != nullptr && blockIdx.x < TL_BLOCKS) next.timeline[blockIdx.x * TL_EVENTS + (ev)] = gtime(); } while (0)
constexpr int TMEM_COLS = 128;   // two accumulator buffers of up to 64 columns

__device__ int g_stream_status = 0;

// The matrix [N, K] that the next streamed product will read (units_ahead = 0: unknown), and how that launch cuts it
// (all_shared: it runs in a mode that leaves partial sums to a later kernel).
struct Next {
  int N, K, n_ctas, units_ahead, all_shared;
  unsigned long long* timeline;   // this launch's [TL_BLOCKS][TL_EVENTS] stamps, or null
};

struct Range {
  long first, last;              // units [first, last)
};

__device__ __forceinline__ Range range_of(int cta, int n_ctas, long units) {
  Range r;
  r.first = (long)cta * units / n_ctas;
  r.last = (long)(cta + 1) * units / n_ctas;
  return r;
}
// What one block works through, in this order: a contiguous range of the units of the "shared" tiles (cut evenly
// between all blocks, stream-K), then whole tiles of its own.  With T tiles and G blocks, each block owns
// floor(T / G) whole tiles (tiles [c * W, c * W + W)) and the last T - W * G tiles are shared.  The shared units
// come first so that the exchange of partial sums between blocks happens while the whole tiles still stream;
// a block then ends with a tile that it finishes alone.  The modes that leave partial sums to a later kernel
// keep every tile shared (W = 0): their readers know that cut (gi_gemm_stream_geometry).
struct Plan {
  long shared_base, shared_units;   // the shared tiles' units are [shared_base, shared_base + shared_units)
  int sharers;                      // blocks 0 .. sharers-1 cut them between themselves (every range non-empty)
  long s_first, s_last;             // this block's range of them (absolute unit numbers)
  long w_first, w_last;             // this block's whole tiles, as units
};

__device__ __forceinline__ Plan plan_of(int cta, int n_ctas, int n_tiles, int kb_per_tile, bool all_shared) {
  Plan p;
  const int W = all_shared ? 0 : n_tiles / n_ctas;
  p.shared_base = (long)W * n_ctas * kb_per_tile;
  p.shared_units = (long)(n_tiles - W * n_ctas) * kb_per_tile;
  p.sharers = (int)min((long)n_ctas, p.shared_units);
  p.s_first = p.s_last = p.shared_base;
  if (cta < p.sharers) {
    p.s_first = p.shared_base + (long)cta * p.shared_units / p.sharers;
    p.s_last = p.shared_base + (long)(cta + 1) * p.shared_units / p.sharers;
  }
  p.w_first = (long)cta * W * kb_per_tile;
  p.w_last = p.w_first + (long)W * kb_per_tile;
  return p;
}

// The block whose range holds unit u: the largest c with floor(c * units / n) <= u.
__device__ __forceinline__ int cta_of(long u, int n_ctas, long units) {
  return (int)(((u + 1) * n_ctas + units - 1) / units - 1);
}

template <int NT, int STAGES, int MODE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, void* __restrict__ out_,
                   float* __restrict__ scratch, int* __restrict__ counters, int M, int N, int K, long ldo, int use_pdl,
                   const __grid_constant__ CUtensorMap map_next, Next next) {
  constexpr uint32_t W_BYTES = TILE_ROWS * BK * 2, A_BYTES = NT * BK * 2, STAGE_BYTES = W_BYTES + A_BYTES;
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(TILE_ROWS >> 4) << 24);
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);   // full[S], empty[S], acc_full[2], acc_empty[2]
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
  int* last_flag = (int*)(tmem_slot + 1);

  if (threadIdx.x == 0) TL(0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_per_tile = (K + BK - 1) / BK;
  const int n_tiles = (N + TILE_ROWS - 1) / TILE_ROWS;
  const int n_ctas = gridDim.x;
  const Plan plan = plan_of(blockIdx.x, n_ctas, n_tiles, kb_per_tile, MODE == GI_SKINNY_ACCUM_DEFER || MODE == GI_SKINNY_STORE_DEFER);
  const long n_shared = plan.s_last - plan.s_first, n_mine = n_shared + (plan.w_last - plan.w_first);
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
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // every block of this grid is resident by now (one per SM): the next kernel in the stream may start setting
  // itself up; its own dependency wait still holds it until this grid has finished
  if (use_pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      TL(1);
      // (tile, kb) of the running unit, advanced without divisions: this thread should spend its time issuing loads
      long u = n_shared > 0 ? plan.s_first : plan.w_first;
      int tile = (int)(u / kb_per_tile), kb = (int)(u % kb_per_tile);
      auto advance = [&]() {
        ++u;
        if (++kb == kb_per_tile) {
          kb = 0;
          ++tile;
        }
        if (u == plan.s_last && plan.w_last > plan.w_first) {      // after the shared range: the whole tiles
          u = plan.w_first;
          tile = (int)(u / kb_per_tile);
          kb = 0;
        }
      };
      bool ok = true;
      const int ahead = use_pdl ? (int)min((long)STAGES, n_mine) : 0;
      {
        // Weights do not depend on the kernel before this one: with programmatic launch their first stages are on
        // their way while that kernel is still finishing; activations are only touched after the dependency wait.
        const long u0 = u;
        const int tile0 = tile, kb0 = kb;
        for (int i = 0; i < ahead; ++i) {
          mbar_expect_tx(full0 + 8 * i, STAGE_BYTES);
          tma_load_2d(smem_u32(smem + (size_t)i * STAGE_BYTES), &map_w, kb * BK, tile * TILE_ROWS, full0 + 8 * i);
          advance();
        }
        u = u0;
        tile = tile0;
        kb = kb0;
      }
      if (next.timeline != nullptr && blockIdx.x < TL_BLOCKS) {
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        next.timeline[blockIdx.x * TL_EVENTS + 2] = smid;
      }
      if (use_pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
      TL(3);
      int s = 0;
      uint32_t round = 0;
      for (long it = 0; it < n_mine && ok; ++it) {
        const uint32_t dst = smem_u32(smem + (size_t)s * STAGE_BYTES);
        if (it >= ahead) {
          ok = mbar_wait(empty0 + 8 * s, (round & 1) ^ 1, 1, &g_stream_status);
          if (!ok) break;
          mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
          tma_load_2d(dst, &map_w, kb * BK, tile * TILE_ROWS, full0 + 8 * s);
        }
        tma_load_2d(dst + W_BYTES, &map_a, kb * BK, 0, full0 + 8 * s);
        advance();
        if (++s == STAGES) {
          s = 0;
          ++round;
        }
      }
      TL(5);
      // This block's own loads are all on their way.  When the caller named the matrix that the next product in
      // the stream will read, ask the L2 cache for the first units of that product's blocks now: the memory keeps
      // streaming while this kernel drains and the next one starts, instead of idling across the boundary.
      if (ok && next.units_ahead > 0) {
        const int kbn = (next.K + BK - 1) / BK, tiles_n = (next.N + TILE_ROWS - 1) / TILE_ROWS;
        for (int c = blockIdx.x; c < next.n_ctas; c += gridDim.x) {
          const Plan pn = plan_of(c, next.n_ctas, tiles_n, kbn, next.all_shared != 0);
          int left = next.units_ahead;
          for (long uu = pn.s_first; uu < pn.s_last && left > 0; ++uu, --left)
            tma_prefetch_l2_2d(&map_next, (int)(uu % kbn) * BK, (int)(uu / kbn) * TILE_ROWS);
          for (long uu = pn.w_first; uu < pn.w_last && left > 0; ++uu, --left)
            tma_prefetch_l2_2d(&map_next, (int)(uu % kbn) * BK, (int)(uu / kbn) * TILE_ROWS);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int it = 0, seg = 0;
      bool ok = true;
      for (int part = 0; part < 2; ++part) {                       // the shared range, then the whole tiles
        long u = part ? plan.w_first : plan.s_first;
        const long part_end = part ? plan.w_last : plan.s_last;
        while (u < part_end && ok) {
          const int tile = (int)(u / kb_per_tile);
          const long seg_end = min(part_end, (long)(tile + 1) * kb_per_tile);
          const int buf = seg & 1;
          ok = mbar_wait(acce0 + 8 * buf, (((uint32_t)(seg >> 1)) & 1) ^ 1, 2, &g_stream_status);   // the buffer was drained
          if (!ok) break;
          tc_fence_after();
          const uint32_t d = tmem + (uint32_t)(buf * 64);
          bool first = true;
          for (; u < seg_end; ++u, ++it) {
            const int s = it % STAGES;
            ok = mbar_wait(full0 + 8 * s, ((uint32_t)(it / STAGES)) & 1, 2, &g_stream_status);
            if (!ok) break;
            if (it == 0) TL(4);
            tc_fence_after();
            const uint32_t w_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
            const uint64_t dw = smem_desc(w_addr), da = smem_desc(w_addr + W_BYTES);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              tc_mma(d, dw + (uint64_t)(2 * k), da + (uint64_t)(2 * k), IDESC, first ? 0u : 1u);
              first = false;
            }
            tc_commit(empty0 + 8 * s);
          }
          if (ok) tc_commit(accf0 + 8 * buf);
          ++seg;
        }
      }
      TL(6);
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;           // feature within the tile
    const int etid = (warp - 2) * 32 + lane;       // 0..127 among the epilogue threads
    int seg = 0;
    bool ok = true;
    const int first_shared_tile = (int)(plan.s_first / kb_per_tile);
    if (use_pdl) asm volatile("griddepcontrol.wait;" ::: "memory");    // outputs and scratch are shared with earlier kernels
    for (int part = 0; part < 2; ++part) {
    long u = part ? plan.w_first : plan.s_first;
    const long part_end = part ? plan.w_last : plan.s_last;
    while (u < part_end && ok) {
      const int tile = (int)(u / kb_per_tile);
      const long tile_first = (long)tile * kb_per_tile, tile_end = tile_first + kb_per_tile;
      const long seg_end = min(part_end, tile_end);
      const bool whole = (u == tile_first && seg_end == tile_end);
      const int buf = seg & 1;
      ok = mbar_wait(accf0 + 8 * buf, ((uint32_t)(seg >> 1)) & 1, 3, &g_stream_status);
      if (!ok) break;
      tc_fence_after();
      float v[NT];
      {
        const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * 64);
#pragma unroll
        for (int c = 0; c < NT; c += 16) {
          uint32_t r[16];
          asm volatile(
              "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
              : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
              : "r"(taddr + (uint32_t)c) : "memory");
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) v[c + j] = __uint_as_float(r[j]);
        }
      }
      // the accumulator is in registers: hand the buffer back to the MMA thread
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acce0 + 8 * buf);

      const int f = tile * TILE_ROWS + row;
      bool finish = whole;
      if (!whole && (MODE == GI_SKINNY_ACCUM_DEFER || MODE == GI_SKINNY_STORE_DEFER)) {
        // leave the partial sums for the next reader of the output (the norm after a residual add, the rotary
        // kernel after the q/k/v product), which adds them in the order of the K ranges while it reads the row
        // anyway: no exchange between blocks here
        const int which = (tile == first_shared_tile) ? 0 : 1;
        float* slot = scratch + ((size_t)blockIdx.x * 2 + which) * (TILE_ROWS * NT);
#pragma unroll
        for (int m = 0; m < NT; ++m) __stcg(slot + m * TILE_ROWS + row, v[m]);
      } else if (!whole) {
        // a tile shared with other blocks: leave the partial sums, and see whether everyone else has left theirs
        const int c_first = cta_of(tile_first - plan.shared_base, plan.sharers, plan.shared_units);
        const int c_last = cta_of(tile_end - 1 - plan.shared_base, plan.sharers, plan.shared_units);
        const int which = (tile == first_shared_tile) ? 0 : 1;
        float* slot = scratch + ((size_t)blockIdx.x * 2 + which) * (TILE_ROWS * NT);
#pragma unroll
        for (int m = 0; m < NT; ++m) __stcg(slot + m * TILE_ROWS + row, v[m]);
        // the barrier orders every thread's stores before thread 0's release; its acquire, then the second
        // barrier, order the partial sums of the other blocks before everyone's loads (no full fences needed)
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (etid == 0) {
          int seen;
          asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(seen) : "l"(counters + tile) : "memory");
          const int is_last = (seen == c_last - c_first) ? 1 : 0;
          if (is_last) counters[tile] = 0;            // ready for the next launch
          *last_flag = is_last;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        finish = *last_flag != 0;
        if (finish) {
#pragma unroll
          for (int m = 0; m < NT; ++m) v[m] = 0.f;
          for (int c = c_first; c <= c_last; ++c) {      // in the order of the K ranges
            const int wh = (tile == (int)((plan.shared_base + range_of(c, plan.sharers, plan.shared_units).first) / kb_per_tile)) ? 0 : 1;
            const float* src = scratch + ((size_t)c * 2 + wh) * (TILE_ROWS * NT);
#pragma unroll
            for (int m = 0; m < NT; ++m) v[m] += __ldcg(src + m * TILE_ROWS + row);
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");   // last_flag may be rewritten only after everyone read it
      }
      if (finish) {
        if (MODE == GI_SKINNY_SWIGLU) {
          // rows 16b..16b+7 gate j, 16b+8..16b+15 up j: the partner sits 8 lanes further
          const bool is_gate = (row & 15) < 8;
          const int fo = (f >> 4) * 8 + (f & 7);
          // several tokens at a time (eight of a 16-token tile, sixteen of a wider one): their exchanges and
          // exponentials overlap (one token per turn, each turn ending in a test of M, ran them one after the
          // other: 4.5 us for a tile of 64 tokens)
          constexpr int GROUP = NT >= 32 ? 16 : 8;
#pragma unroll
          for (int m0 = 0; m0 < NT; m0 += GROUP) {
            if (m0 >= M) break;                     // the same for every lane
            float h[GROUP];
#pragma unroll
            for (int j = 0; j < GROUP; ++j) {
              const float up = __shfl_down_sync(0xffffffffu, v[m0 + j], 8);
              h[j] = gi::silu_mul_bf16(v[m0 + j], up);
            }
            if (is_gate && f < N) {
#pragma unroll
              for (int j = 0; j < GROUP; ++j)
                if (m0 + j < M) ((__nv_bfloat16*)out_)[(size_t)(m0 + j) * ldo + fo] = __float2bfloat16_rn(h[j]);
            }
          }
        } else if (f < N) {
#pragma unroll
          for (int m = 0; m < NT; ++m) {
            if (m >= M) break;
            if (MODE == GI_SKINNY_ACCUM_F32 || MODE == GI_SKINNY_ACCUM_DEFER) {
              float* o = (float*)out_ + (size_t)m * ldo + f;
              *o += v[m];
            } else if (MODE == GI_SKINNY_STORE_F32) {
              ((float*)out_)[(size_t)m * ldo + f] = v[m];
            } else {
              ((__nv_bfloat16*)out_)[(size_t)m * ldo + f] = __float2bfloat16_rn(v[m]);
            }
          }
        }
      }
      u = seg_end;
      ++seg;
    }
    }
    if (etid == 0) TL(7);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS) : "memory");
  }
}

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

// How many blocks a launch takes.  Usually one per SM, the units cut evenly between them.  A product that finishes its
// sums itself and has a few tiles fewer than there are SMs takes one block per tile instead (g_whole_percent: at least
// that share of the SMs, 0: never): every tile is then whole, no block ends with an exchange of partial sums, and the
// remaining SMs are fewer than the exchange costs.
int g_whole_percent = 80;   // measured: from about 118 tiles on 148 SMs one block per tile is faster at every K tried, below that the cut is
int grid_for(int N, int K, int mode) {
  const int n_tiles = (N + TILE_ROWS - 1) / TILE_ROWS;
  const long units = (long)n_tiles * ((K + BK - 1) / BK);
  const int sms = sm_count();
  const bool deferred = mode == GI_SKINNY_ACCUM_DEFER || mode == GI_SKINNY_STORE_DEFER;
  if (!deferred && g_whole_percent > 0 && n_tiles < sms && (long)n_tiles * 100 >= (long)sms * g_whole_percent) return n_tiles;
  return (int)(units < sms ? units : sms);
}

template <int NT, int STAGES, int MODE>
int launch(void* out, const CUtensorMap& mw, const CUtensorMap& ma, float* scratch, int* counters, int M, int N, int K, long ldo,
           int use_pdl, cudaStream_t s, const CUtensorMap& mn, Next next) {
  constexpr size_t smem = (size_t)STAGES * (TILE_ROWS * BK * 2 + NT * BK * 2) + (2 * STAGES + 4) * 8 + 16 + 1024;
  auto kern = gemm_stream_kernel<NT, STAGES, MODE>;
  static bool configured[gi::MAX_DEVICES_SEEN] = {false};
  int dev;
  if (gi::unconfigured_here(configured, &dev)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "streamed product: %s", cudaGetErrorString(e));
    if (dev >= 0) configured[dev] = true;
  }
  const int grid = grid_for(N, K, MODE);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, mw, ma, out, scratch, counters, M, N, K, ldo, use_pdl, mn, next);
  if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "streamed product: %s", cudaGetErrorString(e));
  return GI_OK;
}

template <int NT, int STAGES>
int launch_mode(int mode, void* out, const CUtensorMap& mw, const CUtensorMap& ma, float* scratch, int* counters, int M, int N,
                int K, long ldo, int use_pdl, cudaStream_t s, const CUtensorMap& mn, Next next) {
  switch (mode) {
    case GI_SKINNY_STORE_BF16: return launch<NT, STAGES, GI_SKINNY_STORE_BF16>(out, mw, ma, scratch, counters, M, N, K, ldo, use_pdl, s, mn, next);
    case GI_SKINNY_STORE_F32: return launch<NT, STAGES, GI_SKINNY_STORE_F32>(out, mw, ma, scratch, counters, M, N, K, ldo, use_pdl, s, mn, next);
    case GI_SKINNY_ACCUM_F32: return launch<NT, STAGES, GI_SKINNY_ACCUM_F32>(out, mw, ma, scratch, counters, M, N, K, ldo, use_pdl, s, mn, next);
    case GI_SKINNY_SWIGLU: return launch<NT, STAGES, GI_SKINNY_SWIGLU>(out, mw, ma, scratch, counters, M, N, K, ldo, use_pdl, s, mn, next);
    case GI_SKINNY_ACCUM_DEFER: return launch<NT, STAGES, GI_SKINNY_ACCUM_DEFER>(out, mw, ma, scratch, counters, M, N, K, ldo, use_pdl, s, mn, next);
    case GI_SKINNY_STORE_DEFER: return launch<NT, STAGES, GI_SKINNY_STORE_DEFER>(out, mw, ma, scratch, counters, M, N, K, ldo, use_pdl, s, mn, next);
  }
  return gi::fail(GI_ERR_ARG, "streamed product: unknown mode %d", mode);
}

}  // namespace

static unsigned long long* g_timeline = nullptr;
static int g_timeline_slots = 1;
static long g_timeline_launches = 0;

// Scratch the caller provides: `scratch` holds gi_gemm_stream_scratch_floats() floats (partial sums of tiles cut
// between blocks), `counters` one int per 128-row tile of W, zero before the first use (the kernel leaves them zero).
extern "C" long gi_gemm_stream_scratch_floats(void) { return (long)sm_count() * 2 * TILE_ROWS * 64; }

extern "C" int gi_gemm_stream_bf16(void* out, int mode, const void* A, const void* W, float* scratch, int* counters,
                                   int n_counters, int M, int N, int K, long lda, long ldw, long ldo, int use_pdl,
                                   void* stream) {
  return gi_gemm_stream_bf16_ex(out, mode, A, W, scratch, counters, n_counters, M, N, K, lda, ldw, ldo, use_pdl, nullptr, 0, 0, 0, 0, 0, stream);
}

extern "C" int gi_gemm_stream_bf16_ex(void* out, int mode, const void* A, const void* W, float* scratch, int* counters,
                                      int n_counters, int M, int N, int K, long lda, long ldw, long ldo, int use_pdl,
                                      const void* next_W, int next_N, int next_K, long next_ldw, int next_mode,
                                      int units_ahead, void* stream) {
  if (M <= 0 || N <= 0) return GI_OK;
  if (M > 64) return gi::fail(GI_ERR_UNSUPPORTED, "streamed product: %d rows of activations, at most 64", M);
  if (K <= 0 || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0)
    return gi::fail(GI_ERR_UNSUPPORTED, "streamed product: K (%d) and the row strides (%ld, %ld) must be multiples of 8", K, lda, ldw);
  if (((uintptr_t)A | (uintptr_t)W) & 15) return gi::fail(GI_ERR_UNSUPPORTED, "streamed product: operands must be 16-byte aligned");
  if (mode == GI_SKINNY_SWIGLU && N % 16 != 0) return gi::fail(GI_ERR_UNSUPPORTED, "streamed product: SwiGLU needs interleaved rows, N (%d) a multiple of 16", N);
  const int n_tiles = (N + TILE_ROWS - 1) / TILE_ROWS;
  if (!scratch || !counters || n_counters < n_tiles)
    return gi::fail(GI_ERR_ARG, "streamed product: scratch and %d tile counters are needed (got %d)", n_tiles, n_counters);
  if (use_pdl < 0) use_pdl = gi::pdl_enabled() ? 1 : 0;
  const int nt = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  CUtensorMap mw, ma;
  int rc = gi::tensor_map_2d(&mw, W, N, K, ldw, TILE_ROWS);
  if (rc != GI_OK) return rc;
  rc = gi::tensor_map_2d(&ma, A, M, K, lda, nt);
  if (rc != GI_OK) return rc;
  // the next product's matrix, if the caller knows it and it can have a tensor map; otherwise nothing is fetched ahead
  Next next = {0, 0, 0, 0, 0, nullptr};
  CUtensorMap mn = mw;
  if (next_W && units_ahead > 0 && next_N > 0 && next_K > 0 && next_K % 8 == 0 && next_ldw % 8 == 0 && !((uintptr_t)next_W & 15) &&
      gi::tensor_map_2d(&mn, next_W, next_N, next_K, next_ldw, TILE_ROWS) == GI_OK) {
    next = {next_N, next_K, grid_for(next_N, next_K, next_mode), units_ahead,
            (next_mode == GI_SKINNY_ACCUM_DEFER || next_mode == GI_SKINNY_STORE_DEFER) ? 1 : 0, nullptr};
  } else {
    mn = mw;
  }
  if (g_timeline != nullptr) next.timeline = g_timeline + (size_t)(g_timeline_launches++ % g_timeline_slots) * TL_BLOCKS * TL_EVENTS;
  cudaStream_t s = (cudaStream_t)stream;
  if (nt == 16) return launch_mode<16, 10>(mode, out, mw, ma, scratch, counters, M, N, K, ldo, use_pdl, s, mn, next);
  if (nt == 32) return launch_mode<32, 9>(mode, out, mw, ma, scratch, counters, M, N, K, ldo, use_pdl, s, mn, next);
  return launch_mode<64, 8>(mode, out, mw, ma, scratch, counters, M, N, K, ldo, use_pdl, s, mn, next);
}

// How a launch with these sizes cuts its work: blocks, units per tile, token-tile width.  The kernel that settles
// deferred partial sums (gi_rmsnorm with a settle descriptor, gi_settle) needs exactly these numbers.
extern "C" int gi_gemm_stream_geometry(int M, int N, int K, int* n_ctas, int* kb_per_tile, int* nt) {
  *n_ctas = grid_for(N, K, GI_SKINNY_ACCUM_DEFER);
  *kb_per_tile = (K + BK - 1) / BK;
  *nt = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  return GI_OK;
}

// From now on every streamed product writes its blocks' time stamps into slot (launch number mod slots) of `buf`
// ([slots][256 blocks][8 events] 64-bit values on the device); buf = null switches it off.  Returns how many
// launches have been stamped since the last call.  A launch captured in a CUDA graph keeps the slot it was captured with.
extern "C" long gi_gemm_stream_timeline(unsigned long long* buf, int slots) {
  const long n = g_timeline_launches;
  g_timeline = (buf != nullptr && slots > 0) ? buf : nullptr;
  g_timeline_slots = slots > 0 ? slots : 1;
  g_timeline_launches = 0;
  return n;
}

// percent > 0: a product that finishes its own sums and has fewer tiles than SMs, but at least `percent` of them, runs
// one block per tile (no tile is cut); 0: always one block per SM.  Returns the value before.
extern "C" int gi_gemm_stream_whole_tiles(int percent) {
  const int was = g_whole_percent;
  g_whole_percent = percent < 0 ? 0 : (percent > 100 ? 100 : percent);
  return was;
}

extern "C" int gi_gemm_stream_status(int* status) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(status, g_stream_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int));
  if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "streamed product status: %s", cudaGetErrorString(e));
  return GI_OK;
}
