// C entry points of the kernel library.  Every function takes device pointers and a CUDA stream,
// launches on that stream without synchronising, and returns 0 or an error code whose text
// gi_last_error() gives.  Nothing here allocates device memory: callers pass outputs and scratch.
#pragma once

#define GI_ABI_VERSION 1

#define GI_GEMM_STORE 0      // out = A * W^T, stored in out_dtype
#define GI_GEMM_ACCUM_F32 1  // out (float) += A * W^T

#ifdef __cplusplus
extern "C" {
#endif

// Partial sums a deferred product left behind (see GI_SKINNY_ACCUM_DEFER): where they are and how the product cut its work.
typedef struct {
  const float* partials;     // null: nothing to settle
  const int* tile_first_cta; // per 128-row tile: the first and the last block that held a piece of it
  const int* tile_last_cta;
  const int* cta_first_tile; // per block: the tile its range began in (that piece sits in the block's slot 0)
  int nt;                    // token-tile width of the product (16, 32 or 64)
} gi_settle_t;

#ifdef __CUDACC__
// Which blocks of a deferred product hold pieces of the 128-column tile of column f.  Blocks take contiguous ranges
// of K blocks, so every block after the first began its range inside the tile (its piece sits in its slot 0); only
// the first block may have come from an earlier tile (slot 1).  The tables are uploaded once per shape and never
// written by a kernel: a kernel may read them before its dependency wait.
struct gi_settle_span {
  int c_first, c_last, first_slot;
};
__device__ __forceinline__ gi_settle_span gi_span_of(const gi_settle_t& st, int f) {
  gi_settle_span s;
  const int tile = f / 128;
  s.c_first = st.tile_first_cta[tile];
  s.c_last = st.tile_last_cta[tile];
  s.first_slot = (s.c_first != s.c_last && tile != st.cta_first_tile[s.c_first]) ? 1 : 0;
  return s;
}
// The address of block c's piece for token m, column f.
__device__ __forceinline__ const float* gi_piece(const gi_settle_t& st, const gi_settle_span& s, int c, int m, int f) {
  const int slot = (c == s.c_first) ? s.first_slot : 0;
  return st.partials + ((size_t)c * 2 + slot) * (128 * st.nt) + (size_t)m * 128 + f % 128;
}
// The sum of a column's pieces in the order of the K ranges.  The loads of up to eight pieces are issued together
// (absent ones count as +0, which changes no sum), so that the sum costs one trip to the L2 cache, not one per piece.
__device__ __forceinline__ float gi_sum_pieces(const gi_settle_t& st, const gi_settle_span& s, int m, int f) {
  float acc = 0.f;
  for (int c0 = s.c_first; c0 <= s.c_last; c0 += 8) {
    float p[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) p[j] = (c0 + j <= s.c_last) ? __ldcg(gi_piece(st, s, c0 + j, m, f)) : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += p[j];
  }
  return acc;
}
// Two columns of the same tile at once (a rotated pair): both columns' loads are in flight together.
__device__ __forceinline__ float2 gi_sum_pieces2(const gi_settle_t& st, const gi_settle_span& s, int m, int fa, int fb) {
  float2 acc = make_float2(0.f, 0.f);
  for (int c0 = s.c_first; c0 <= s.c_last; c0 += 8) {
    float pa[8], pb[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      pa[j] = (c0 + j <= s.c_last) ? __ldcg(gi_piece(st, s, c0 + j, m, fa)) : 0.f;
      pb[j] = (c0 + j <= s.c_last) ? __ldcg(gi_piece(st, s, c0 + j, m, fb)) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      acc.x += pa[j];
      acc.y += pb[j];
    }
  }
  return acc;
}
__device__ __forceinline__ float4 gi_sum_pieces4(const gi_settle_t& st, const gi_settle_span& s, int m, int f) {
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int c0 = s.c_first; c0 <= s.c_last; c0 += 8) {
    float4 p[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      p[j] = (c0 + j <= s.c_last) ? __ldcg(reinterpret_cast<const float4*>(gi_piece(st, s, c0 + j, m, f))) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      acc.x += p[j].x;
      acc.y += p[j].y;
      acc.z += p[j].z;
      acc.w += p[j].w;
    }
  }
  return acc;
}
#endif

const char* gi_last_error(void);
int gi_abi_version(void);
// Programmatic dependent launch: kernels of a stream may begin while their predecessor drains (off by default).
void gi_set_pdl(int on);
int gi_get_pdl(void);

int gi_embed(float* out, const void* table, int table_dtype, const int* tokens, int n_tokens, int d, int vocab,
             void* stream);
int gi_rmsnorm(void* out, int out_dtype, const float* x, const void* w, int w_dtype, const int* rows, int n_rows,
               int d, float eps, void* stream);
// The same, first adding deferred partial sums to the rows it reads (and writing the settled rows back to x, unless
// `rows` selects: then x is left as it is and must not be read again).
int gi_rmsnorm_settle(void* out, int out_dtype, float* x, const void* w, int w_dtype, const int* rows, int n_rows,
                      int d, float eps, gi_settle_t settle, void* stream);
int gi_silu_mul(void* out, const void* gate_up, int dtype, int n_rows, int f, int interleaved, void* stream);

int gi_gemm_generic(void* out, int out_dtype, int mode, const void* A, int a_dtype, const void* W, int w_dtype, int M,
                    int N, int K, long lda, long ldw, long ldo, void* stream);

// mode of gi_gemm_skinny_bf16
#define GI_SKINNY_STORE_BF16 0
#define GI_SKINNY_STORE_F32 1
#define GI_SKINNY_ACCUM_F32 2   // out (float) += product
#define GI_SKINNY_SWIGLU 3      // W rows interleaved [8 gate | 8 up]; out[M, N/2] bfloat16 = silu(gate) * up
#define GI_SKINNY_STORE_DEFER 5 // the same for STORE_BF16: whole tiles are stored, cut tiles stay as partial sums for gi_rope_cache_write
#define GI_SKINNY_ACCUM_DEFER 4 // gi_gemm_stream_bf16 only: as ACCUM_F32, but tiles cut between blocks leave their partial
                                // sums in `scratch` for gi_rmsnorm / gi_settle to add (no exchange between blocks)
int gi_gemm_skinny_bf16(void* out, int mode, const void* A, const void* W, int M, int N, int K, long lda, long ldw,
                        long ldo, void* stream);

// Persistent stream-K tcgen05 product for at most 64 rows of activations (modes as gi_gemm_skinny_bf16).
// `scratch`: gi_gemm_stream_scratch_floats() floats; `counters`: one int per 128 rows of W, zero at first use.
// use_pdl: launch with programmatic stream serialization (weights are prefetched before the dependency wait).
long gi_gemm_stream_scratch_floats(void);
int gi_gemm_stream_bf16(void* out, int mode, const void* A, const void* W, float* scratch, int* counters, int n_counters,
                        int M, int N, int K, long lda, long ldw, long ldo, int use_pdl, void* stream);
// As gi_gemm_stream_bf16; `next_W` [next_N, next_K] (optional) is the matrix that the next streamed product in this
// stream will read: the kernel asks the L2 cache for the first `units_ahead` 16 KB units of each of that launch's blocks
// once its own loads are issued (`next_mode`: the mode of that launch, which decides how it cuts its work).  A wrong
// guess costs bandwidth, never a result; next_W must be valid memory.
int gi_gemm_stream_bf16_ex(void* out, int mode, const void* A, const void* W, float* scratch, int* counters, int n_counters,
                           int M, int N, int K, long lda, long ldw, long ldo, int use_pdl, const void* next_W, int next_N,
                           int next_K, long next_ldw, int next_mode, int units_ahead, void* stream);
int gi_gemm_stream_status(int* status);
// percent > 0: a product that finishes its own sums and has fewer 128-row tiles than SMs, but at least `percent` of
// them, runs one block per tile, so that no tile is cut between blocks; 0: always one block per SM.  Returns the old value.
int gi_gemm_stream_whole_tiles(int percent);
// Time stamps of the streamed products' blocks, for a timeline of a decode step: see gemm_stream.cu.
long gi_gemm_stream_timeline(unsigned long long* buf, int slots);
int gi_gemm_stream_geometry(int M, int N, int K, int* n_ctas, int* kb_per_tile, int* nt);

// x[rows, :] += the partial sums, in the order of the K ranges.  rows: optional selection; n_features = width of x.
int gi_settle(float* x, gi_settle_t settle, const int* rows, int n_rows, int d, void* stream);

// mode of gi_gemm_tc_bf16 (same meanings as the skinny product's)
#define GI_TC_STORE_BF16 0
#define GI_TC_STORE_F32 1
#define GI_TC_ACCUM_F32 2
#define GI_TC_SWIGLU 3
#define GI_TC_QKV_ROPE 4        // gi_gemm_tc_qkv_rope only: queries rotated and stored, keys and values into the cache
// tcgen05 / TMA product for many rows of activations; tile_n is 128 or 256
int gi_gemm_tc_bf16(void* out, int mode, const void* A, const void* W, int M, int N, int K, long lda, long ldw,
                    long ldo, int tile_n, void* stream);
// The q/k/v product of a prompt step that rotates and stores in its epilogue (the work of gi_rope_cache_write, the same
// bits): out [M, N] packed rows of which the queries' columns are written; N = (n_heads + 2 n_kv) * hd, hd 64 or 128.
int gi_gemm_tc_qkv_rope(void* out, const void* A, const void* W, int M, int N, int K, long lda, long ldw, long ldo,
                        const float* table, const int* positions, const int* slots, const int* block_table, int max_pages,
                        void* kcache, void* vcache, int n_heads, int n_kv, int hd, int write_cache, void* stream);
// narrower tiles for the columns of an unfilled last round of blocks: on (default) or off
int gi_gemm_tc_tail_tiles(int on);
int gi_gemm_tc_status(int* status);

// table[t, i] = (cos, sin)(positions[t] * inv_freq[i]), float2 [n_tokens, rot / 2]
int gi_rope_table(float* table, const int* positions, const float* inv_freq, int n_tokens, int rot, void* stream);
int gi_rope_cache_write(void* qkv, int dtype, long ld, const float* table, const int* positions, const int* slots,
                        const int* block_table, int max_pages, void* kcache, void* vcache, int n_tokens, int n_heads,
                        int n_kv, int hd, int rot, int adjacent, int write_cache, void* stream);
// The same for rows whose product was deferred (GI_SKINNY_STORE_DEFER): values of tiles that were cut between blocks
// are the sums of the partial sums, rounded to the row's dtype as a stored value would have been.
int gi_rope_cache_write_settle(void* qkv, int dtype, long ld, const float* table, const int* positions, const int* slots,
                               const int* block_table, int max_pages, void* kcache, void* vcache, int n_tokens,
                               int n_heads, int n_kv, int hd, int rot, int adjacent, int write_cache, gi_settle_t settle,
                               void* stream);

int gi_attn_prefill_generic(void* out, long ldo, const void* q, long ldq, int dtype, const void* kcache,
                            const void* vcache, const int* block_table, int max_pages, const int* cu_seqlens,
                            const int* seq_slots, const int* seq_pos0, int n_seqs, int max_q_len, int n_heads, int n_kv,
                            int hd, float scale, int window, void* stream);
int gi_attn_decode_generic(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq, int dtype,
                           const void* kcache, const void* vcache, const int* block_table, int max_pages,
                           const int* seq_slots, const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd,
                           float scale, int window, int n_splits, int own_tiles, void* stream);
// own_tiles > 0: slice s of a sequence holds tiles [s * own_tiles, (s + 1) * own_tiles) of 32 keys of its own span,
// whatever n_splits is (which must cover the longest span); 0: each span is cut into n_splits equal slices.

// bfloat16, head size 64 or 128: the same operation as gi_attn_prefill_generic, on tensor cores
int gi_attn_prefill_tc(void* out, long ldo, const void* q, long ldq, const void* kcache, const void* vcache,
                       const int* block_table, int max_pages, const int* cu_seqlens, const int* seq_slots,
                       const int* seq_pos0, int n_seqs, int max_q_len, int n_heads, int n_kv, int hd, float scale,
                       int window, void* stream);
// bfloat16, head size 128: the same on tcgen05 tensor cores (scores and output accumulate in tensor memory).
// q_rows: rows of the packed q/k/v matrix; cache_pages: pages the cache tensors hold.
int gi_attn_prefill_t5(void* out, long ldo, const void* q, long ldq, long q_rows, const void* kcache, const void* vcache,
                       long cache_pages, const int* block_table, int max_pages, const int* cu_seqlens, const int* seq_slots,
                       const int* seq_pos0, int n_seqs, int max_q_len, int n_heads, int n_kv, int hd, float scale, int window,
                       void* stream);
// query tiles two to a block (the i-th from the end with the i-th from the start): 0 never, 1 where the launch then
// is one round of blocks (default), 2 always
int gi_attn_prefill_t5_pairing(int mode);
int gi_attn_prefill_t5_status(int* status);
// bfloat16, head size 64 or 128: the same operation as gi_attn_decode_generic, on tensor cores
int gi_attn_decode_tc(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq, const void* kcache,
                      const void* vcache, const int* block_table, int max_pages, const int* seq_slots,
                      const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd, float scale, int window,
                      int n_splits, void* stream);
// the same with a choice of tile: 32 keys (one block per SM) or 16 keys (two blocks per SM)
int gi_attn_decode_tc_ex(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq, const void* kcache,
                         const void* vcache, const int* block_table, int max_pages, const int* seq_slots,
                         const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd, float scale, int window,
                         int n_splits, int tile_keys, void* stream);
// the same with the slices merged inside the kernel by the block that finishes last (counters: one int per sequence x
// kv head x chunk of 16 heads, zero before the first use; nullptr: merged by a second kernel), and, with own_tiles > 0,
// slices of that many tiles of each sequence's own span instead of n_splits equal ones
int gi_attn_decode_tc_merged(void* out, long ldo, float* part_o, float* part_ml, int* counters, int n_counters, const void* q,
                             long ldq, const void* kcache, const void* vcache, const int* block_table, int max_pages,
                             const int* seq_slots, const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd, float scale,
                             int window, int n_splits, int own_tiles, int tile_keys, int stages, void* stream);
// stages: depth of each warp's ring of tiles, 2 to 4 (0: the default for the head size)
// The same on rows that are not rotated yet: `qkv` holds one packed [q | k | v] row per sequence as the q/k/v product
// left it (`settle`: its pending partial sums), `table` [sequences][rot / 2] the (cos, sin) of each sequence's newest
// position.  The kernel rotates q and k (pairs (i, i + rot / 2)) and stores k and v at position length - 1 itself:
// gi_rope_cache_write's work for a decode step, inside the attention's launch.
int gi_attn_decode_tc_rope(void* out, long ldo, float* part_o, float* part_ml, int* counters, int n_counters, const void* qkv,
                           long ld, void* kcache, void* vcache, const int* block_table, int max_pages, const int* seq_slots,
                           const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd, float scale, int window, int n_splits,
                           int own_tiles, int tile_keys, int stages, const float* table, int rot, gi_settle_t settle,
                           void* stream);
// The decode attention with the keys on the rows of the tensor-core tile and up to 8 heads on its columns (half the
// products per key for groups of up to 8 heads); slices are merged by gi_attn_combine.  warps: 4, 6 or 8 a block;
// stages: 2 or 3 tiles deep per warp.
int gi_attn_decode_kr(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq, const void* kcache,
                      const void* vcache, const int* block_table, int max_pages, const int* seq_slots, const int* seq_lens,
                      int n_seqs, int n_heads, int n_kv, int hd, float scale, int window, int n_splits, int own_tiles,
                      int warps, int stages, void* stream);
int gi_attn_combine(void* out, long ldo, int dtype, const float* part_o, const float* part_ml, int n_seqs, int n_heads,
                    int hd, int n_splits, void* stream);

int gi_sample(int* out_tokens, const float* logits, long ld, int n_rows, int vocab, float temperature, int top_k,
              float top_p, unsigned long long* rng_state, const int* state_index, void* stream);

#ifdef __cplusplus
}
#endif
