// Shared device helpers for every kernel file: element load/store for the two activation and
// weight types (float, bfloat16), reductions with a fixed order, and the host-side error record.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define GI_OK 0
#define GI_ERR_ARG 1
#define GI_ERR_CUDA 2
#define GI_ERR_UNSUPPORTED 3

// dtype codes shared with the Python side
#define GI_F32 0
#define GI_BF16 1

#define PAGE_TOKENS 64

namespace gi {

bool pdl_enabled();                                // programmatic dependent launch switched on (gi_set_pdl)
int fail(int code, const char* fmt, ...);          // records the message for gi_last_error(), returns code
int check_launch(const char* what);                // cudaGetLastError() -> GI_OK or a recorded failure

// First statements of a kernel that may be launched with programmatic stream serialization: let the next
// kernel in the stream begin its own set-up, then wait until everything before this kernel has completed and
// is visible.  Both are no-ops for a plain launch.  Nothing a predecessor writes may be touched before this.
__device__ __forceinline__ void pdl_prologue() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// The two halves on their own, for kernels that read data no kernel of the step writes (weights, tables the
// host uploaded before the step's first kernel) between them: such loads overlap the predecessor's end.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// In a kernel that runs code before pdl_wait(), a pointer to data that an earlier kernel of the same stream writes
// must not be declared `const __restrict__`: that promises the compiler that nothing writes the data while the
// kernel runs, and it may then issue the loads above the wait (it did so for the decode attention's queries at head
// size 64, which read the previous step's rows in a replayed graph).  Without the promise the wait's memory clobber
// keeps the loads behind it.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// A read of what the host uploaded for this step (positions, slots, lengths, page tables, row selections) made
// BEFORE the dependency wait.  A kernel that starts while its predecessor still runs finds the SM's L1 as earlier
// kernels left it: a line that held the previous step's value of such an array may still be there, and a plain (or
// read-only-path) load would return it.  These loads go to the L2 cache, which the upload went through.
__device__ __forceinline__ int ld_step(const int* p) { return __ldcg(p); }

// One rotary pair's rotation with its roundings spelled out, so that every kernel that rotates (the rotary kernels, the
// decode attention that rotates its own rows) gives the same bits: (a cos - b sin, a sin + b cos), each as one product
// rounded, then a fused multiply-add.  cs = (cos, sin).
__device__ __forceinline__ void rotate_pair(float a, float b, float2 cs, float* ra, float* rb) {
  *ra = __fmaf_rn(a, cs.x, -__fmul_rn(b, cs.y));
  *rb = __fmaf_rn(a, cs.y, __fmul_rn(b, cs.x));
}

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// silu(g) * u = g / (1 + e^-g) * u for the epilogues that round to bfloat16 right after: 2^x and the division by the
// approximate instructions (each good to about 2 units in the last place of a float; 32-bit arithmetic throughout).
// Six instructions instead of forty, which matters where one warp per scheduler works through a whole tile.
__device__ __forceinline__ float silu_mul_bf16(float g, float u) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * -1.4426950408889634f));
  return __fdividef(g, 1.0f + e) * u;
}

// Four neighbouring values at once (the pointer is aligned to the four of them).
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__bfloat162float(lo.x), __bfloat162float(lo.y), __bfloat162float(hi.x), __bfloat162float(hi.y));
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&lo);
  raw.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block (blockDim.x a multiple of 32, at most 1024); every thread gets the result.
// The order of additions depends only on blockDim.x, so a row gives the same sum in any batch.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

template <typename T> struct DType;
template <> struct DType<float> { static constexpr int code = GI_F32; };
template <> struct DType<__nv_bfloat16> { static constexpr int code = GI_BF16; };

}  // namespace gi

namespace gi {
// Launches `kern` on `s`; with programmatic dependent launch switched on, the kernel may start while its
// predecessor in the stream is still running (it must begin with pdl_prologue()).
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
// A kernel's attributes (its dynamic shared memory limit) belong to the kernel on one device.  `seen` is a table of
// one flag per device that a launcher keeps per kernel; true when the attribute is still to be set on the current device.
constexpr int MAX_DEVICES_SEEN = 64;
inline bool unconfigured_here(bool (&seen)[MAX_DEVICES_SEEN], int* dev) {
  *dev = -1;
  if (cudaGetDevice(dev) != cudaSuccess || *dev < 0 || *dev >= MAX_DEVICES_SEEN) { *dev = -1; return true; }
  return !seen[*dev];
}
inline int check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) return fail(GI_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return check_launch(what);
}
}  // namespace gi

// Calls `body` with `T` bound to the element type named by a dtype code.
#define GI_DISPATCH_DTYPE(code, T, ...)                         \
  do {                                                          \
    if ((code) == GI_F32) { using T = float; __VA_ARGS__; }     \
    else if ((code) == GI_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else return gi::fail(GI_ERR_ARG, "unknown dtype code %d", (int)(code)); \
  } while (0)
