// Warp-level tensor-core pieces shared by the attention kernels: m16n8k16 bfloat16 mma, ldmatrix,
// cp.async with zero fill, and the 16-byte-chunk swizzle that keeps ldmatrix free of bank conflicts.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace gi {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// 16 bytes global -> shared; `bytes` (0 or 16) of them are read, the rest is filled with zeros
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a tile whose rows hold CHUNKS chunks.
// Rows of 128 bytes or more: the chunk index is XORed with the row (mod 8), so that the 8 rows an
// ldmatrix phase touches fall into 8 different bank groups.  Rows of 64 bytes (4 chunks): two rows share
// a 128-byte line, and the XOR uses row / 2.
template <int CHUNKS>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  if (CHUNKS >= 8) return (uint32_t)(row * CHUNKS + (chunk ^ (row & 7))) * 16u;
  return (uint32_t)(row * CHUNKS + (chunk ^ ((row >> 1) & 3))) * 16u;
}

}  // namespace gi
