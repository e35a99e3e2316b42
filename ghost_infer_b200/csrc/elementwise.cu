// Row kernels that move no matrix: embedding lookup, RMSNorm, SwiGLU's elementwise half.
// All arithmetic is 32-bit; inputs and outputs may be float or bfloat16.
#include "api.h"
#include "common.cuh"

namespace {

// x[t, :] = table[tokens[t], :] as float (the reference's embed: src/cuda.rs:418-432, no scaling).
template <typename TW>
__global__ void embed_kernel(float* __restrict__ out, const TW* __restrict__ table, const int* __restrict__ tokens,
                             int d, int vocab) {
  gi::pdl_prologue();
  const int t = blockIdx.x;
  int id = tokens[t];
  if (id < 0 || id >= vocab) id = 0;  // the host validates ids; padding rows may carry anything
  const TW* row = table + (size_t)id * d;
  float* o = out + (size_t)t * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = gi::ldf(row + i);
}

// Sum of the partial sums a deferred product left for features f..f+3 of token m (see gemm_stream.cu: a tile of
// 128 features whose K range was cut between blocks c_first..c_last has one slot per block; they are added in
// the order of the K ranges, so the result does not depend on any timing).  f is a multiple of 4.
__device__ __forceinline__ float4 pending_sum(const gi_settle_t& st, const gi_settle_span& sp, int m, int f) {
  if (sp.c_first == sp.c_last) return make_float4(0.f, 0.f, 0.f, 0.f);   // one block had the whole tile and added it itself
  return gi_sum_pieces4(st, sp, m, f);
}

// x[row, :] += pending partial sums (for readers of the residual stream that do not settle on their own).
__global__ void settle_kernel(float* __restrict__ x, gi_settle_t st, const int* __restrict__ rows, int d) {
  gi::pdl_prologue();
  const int m = rows ? rows[blockIdx.x] : blockIdx.x;
  float4* xr = reinterpret_cast<float4*>(x + (size_t)m * d);
  for (int i = threadIdx.x; i < d / 4; i += blockDim.x) {
    float4 v = xr[i];
    const float4 p = pending_sum(st, gi_span_of(st, 4 * i), m, 4 * i);
    v.x += p.x;
    v.y += p.y;
    v.z += p.z;
    v.w += p.w;
    xr[i] = v;
  }
}

// y = x * (1 / sqrt(mean(x^2) + eps)) * w, one block per row (src/model.rs:919-928, src/cuda.rs:505-515).
// `rows` (optional) picks which rows of x are normed; output row r is then x[rows[r]].
// The row is read once, four floats at a time, and kept in registers (up to VEC float4 per thread);
// wider rows, or rows that are no multiple of 4, take the plain loop.
// ALIGNED: the weights and the output rows start on 16-byte boundaries too (four values per access there as well).
template <typename TO, typename TW, int VEC, bool SETTLE, bool ALIGNED>
__global__ void rmsnorm_kernel(TO* __restrict__ out, float* __restrict__ x, const TW* __restrict__ w,
                               const int* __restrict__ rows, int d, float eps, gi_settle_t st) {
  __shared__ float scratch[33];
  gi::pdl_launch_dependents();
  const int r = blockIdx.x;
  const int m = rows ? gi::ld_step(rows + r) : r;   // the selection was uploaded before the step's first kernel
  float* xr = x + (size_t)m * d;
  TO* o = out + (size_t)r * d;
  if (VEC > 0) {
    const int n4 = d / 4;
    // what no kernel writes (the norm's weights, the tables of a deferred product's cut) is read before the
    // dependency wait; the rows and the partial sums after it
    float4 wv[VEC > 0 ? VEC : 1];
    gi_settle_span sp[VEC > 0 ? VEC : 1];
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < n4) {
        wv[j] = ALIGNED ? gi::ld4(w + 4 * i)
                        : make_float4(gi::ldf(w + 4 * i), gi::ldf(w + 4 * i + 1), gi::ldf(w + 4 * i + 2), gi::ldf(w + 4 * i + 3));
        if (SETTLE) sp[j] = gi_span_of(st, 4 * i);
      }
    }
    gi::pdl_wait();
    float4 v[VEC > 0 ? VEC : 1];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      v[j] = i < n4 ? reinterpret_cast<const float4*>(xr)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      if (SETTLE && i < n4) {
        const float4 p = pending_sum(st, sp[j], m, 4 * i);
        v[j].x += p.x;
        v[j].y += p.y;
        v[j].z += p.z;
        v[j].w += p.w;
        // the settled row goes back to the residual stream; not for a selection of rows (it may name a row twice,
        // and nothing reads the stream after the norm that selects)
        if (rows == nullptr) reinterpret_cast<float4*>(xr)[i] = v[j];
      }
      ss = fmaf(v[j].x, v[j].x, ss);
      ss = fmaf(v[j].y, v[j].y, ss);
      ss = fmaf(v[j].z, v[j].z, ss);
      ss = fmaf(v[j].w, v[j].w, ss);
    }
    ss = gi::block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < n4) {
        const float4 y = make_float4(v[j].x * scale * wv[j].x, v[j].y * scale * wv[j].y, v[j].z * scale * wv[j].z, v[j].w * scale * wv[j].w);
        if (ALIGNED) {
          gi::st4(o + 4 * i, y);
        } else {
          gi::stf(o + 4 * i, y.x);
          gi::stf(o + 4 * i + 1, y.y);
          gi::stf(o + 4 * i + 2, y.z);
          gi::stf(o + 4 * i + 3, y.w);
        }
      }
    }
    return;
  }
  gi::pdl_wait();
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = xr[i];
    ss = fmaf(v, v, ss);
  }
  ss = gi::block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) gi::stf(o + i, xr[i] * scale * gi::ldf(w + i));
}

// `interleaved`: the row holds blocks of 16 values [gate j..j+7 | up j..j+7] instead of [all gates | all ups].
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int f, size_t total, int interleaved) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t m = i / f, c = i % f;
  const size_t gate_at = interleaved ? (c / 8) * 16 + c % 8 : c;
  const size_t up_at = interleaved ? gate_at + 8 : (size_t)f + c;
  const float g = gi::ldf(gu + m * 2 * (size_t)f + gate_at);
  const float u = gi::ldf(gu + m * 2 * (size_t)f + up_at);
  gi::stf(out + i, g / (1.0f + expf(-g)) * u);
}

}  // namespace

extern "C" int gi_embed(float* out, const void* table, int table_dtype, const int* tokens, int n_tokens, int d,
                        int vocab, void* stream) {
  if (n_tokens <= 0) return GI_OK;
  if (d <= 0 || vocab <= 0) return gi::fail(GI_ERR_ARG, "embed: bad sizes d=%d vocab=%d", d, vocab);
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(table_dtype, TW,
                    e = gi::launch(embed_kernel<TW>, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, out, (const TW*)table, tokens, d, vocab));
  return gi::check(e, "embed");
}

namespace {
template <typename TO, typename TW, bool ALIGNED>
cudaError_t rmsnorm_launch(int per, bool settle, dim3 g, dim3 b, cudaStream_t s, TO* out, float* x, const TW* w, const int* rows, int d,
                           float eps, gi_settle_t st) {
  if (settle) {
    if (per == 1) return gi::launch(rmsnorm_kernel<TO, TW, 1, true, ALIGNED>, g, b, 0, s, out, x, w, rows, d, eps, st);
    if (per == 2) return gi::launch(rmsnorm_kernel<TO, TW, 2, true, ALIGNED>, g, b, 0, s, out, x, w, rows, d, eps, st);
    return gi::launch(rmsnorm_kernel<TO, TW, 4, true, ALIGNED>, g, b, 0, s, out, x, w, rows, d, eps, st);
  }
  if (per == 1) return gi::launch(rmsnorm_kernel<TO, TW, 1, false, ALIGNED>, g, b, 0, s, out, x, w, rows, d, eps, st);
  if (per == 2) return gi::launch(rmsnorm_kernel<TO, TW, 2, false, ALIGNED>, g, b, 0, s, out, x, w, rows, d, eps, st);
  if (per == 3 || per == 4) return gi::launch(rmsnorm_kernel<TO, TW, 4, false, ALIGNED>, g, b, 0, s, out, x, w, rows, d, eps, st);
  return gi::launch(rmsnorm_kernel<TO, TW, 0, false, false>, g, b, 0, s, out, x, w, rows, d, eps, st);
}

int rmsnorm_impl(void* out, int out_dtype, float* x, const void* w, int w_dtype, const int* rows, int n_rows, int d, float eps,
                 gi_settle_t st, void* stream) {
  if (n_rows <= 0) return GI_OK;
  if (d <= 0) return gi::fail(GI_ERR_ARG, "rmsnorm: bad width %d", d);
  const bool settle = st.partials != nullptr;
  // few rows (a decode step): many threads per row; many rows (a prompt): 256 threads with more values each, so that
  // an SM holds eight rows' loads in flight instead of four
  // (a settling norm has several loads per value: more threads, fewer values each)
  // (32-bit output is the path whose sums must not depend on the step's other rows: there the block's size, and
  // with it the order of the row's sum, follows from the width alone)
  const bool many = n_rows >= 512 && out_dtype != GI_F32;
  const int threads = settle ? (d >= 4096 ? 1024 : (d >= 2048 ? 512 : 256)) : ((d >= 2048 && !(many && d <= 4096)) ? 512 : 256);
  // the register path: rows that are a multiple of 4 wide, start on 16-byte boundaries, and fit 4 float4 per thread
  const bool vec = d % 4 == 0 && ((uintptr_t)x & 15) == 0 && d / 4 <= 4 * threads;
  const int per = vec ? (d / 4 + threads - 1) / threads : 0;
  if (settle && per == 0) return gi::fail(GI_ERR_UNSUPPORTED, "rmsnorm: settling partial sums needs rows of a multiple of 4 and at most %d values", 16 * threads);
  cudaError_t e = cudaSuccess;
  // d % 4 == 0 here whenever per > 0, so every output row starts as aligned as the first
  const bool aligned = ((uintptr_t)out & 15) == 0 && ((uintptr_t)w & 15) == 0;
  GI_DISPATCH_DTYPE(out_dtype, TO, GI_DISPATCH_DTYPE(w_dtype, TW,
      e = aligned ? (rmsnorm_launch<TO, TW, true>(per, settle, dim3(n_rows), dim3(threads), (cudaStream_t)stream, (TO*)out, x, (const TW*)w, rows, d, eps, st))
                  : (rmsnorm_launch<TO, TW, false>(per, settle, dim3(n_rows), dim3(threads), (cudaStream_t)stream, (TO*)out, x, (const TW*)w, rows, d, eps, st))));
  return gi::check(e, "rmsnorm");
}
}  // namespace

extern "C" int gi_rmsnorm(void* out, int out_dtype, const float* x, const void* w, int w_dtype, const int* rows,
                          int n_rows, int d, float eps, void* stream) {
  gi_settle_t none = {nullptr, nullptr, nullptr, nullptr, 0};
  return rmsnorm_impl(out, out_dtype, const_cast<float*>(x), w, w_dtype, rows, n_rows, d, eps, none, stream);
}

extern "C" int gi_rmsnorm_settle(void* out, int out_dtype, float* x, const void* w, int w_dtype, const int* rows,
                                 int n_rows, int d, float eps, gi_settle_t settle, void* stream) {
  return rmsnorm_impl(out, out_dtype, x, w, w_dtype, rows, n_rows, d, eps, settle, stream);
}

extern "C" int gi_settle(float* x, gi_settle_t settle, const int* rows, int n_rows, int d, void* stream) {
  if (n_rows <= 0 || settle.partials == nullptr) return GI_OK;
  if (d % 4 != 0 || ((uintptr_t)x & 15)) return gi::fail(GI_ERR_UNSUPPORTED, "settle: rows must be a multiple of 4 wide and 16-byte aligned");
  return gi::check(gi::launch(settle_kernel, dim3(n_rows), dim3(256), 0, (cudaStream_t)stream, x, settle, rows, d), "settle");
}

extern "C" int gi_silu_mul(void* out, const void* gate_up, int dtype, int n_rows, int f, int interleaved, void* stream) {
  if (n_rows <= 0) return GI_OK;
  if (f <= 0) return gi::fail(GI_ERR_ARG, "silu_mul: bad width %d", f);
  if (interleaved && f % 8 != 0) return gi::fail(GI_ERR_ARG, "silu_mul: interleaved rows need a width that is a multiple of 8, got %d", f);
  const size_t total = (size_t)n_rows * f;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  GI_DISPATCH_DTYPE(dtype, T, silu_mul_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>((T*)out, (const T*)gate_up, f, total, interleaved));
  return gi::check_launch("silu_mul");
}
