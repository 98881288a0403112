// Descriptor encodings of the tcgen05 tensor core shared by the matrix-multiply and convolution
// kernels.
#pragma once
#include <cuda.h>
#include <stdint.h>

struct b200_engine;

namespace b200 {

// Shared-memory matrix descriptor, 128-byte swizzle. Fields (bits): start address >> 4 [0,14),
// leading byte offset >> 4 [16,30), stride byte offset >> 4 [32,46), version = 1 [46,48),
// layout type [61,64) with 2 = 128-byte swizzle.
//   K-major tile:  rows of 128 bytes, 8-row groups 1024 bytes apart  -> SBO = 1024, LBO unused (1)
//   MN-major tile: blocks of (k rows x 128 bytes); 8-row k groups 1024 bytes apart -> SBO = 1024,
//                  consecutive 128-byte-wide blocks along m/n `lbo_bytes` apart     -> LBO
//
// 32-bit operands stored MN-major cannot use that swizzle: transposing 4-byte elements needs a
// 32-byte swizzle atom. Their layout type is 1 ("128-byte swizzle, 32-byte base"): the pattern
// repeats every 4 k-rows (512 bytes), so SBO = 512, and TMA writes it with
// CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t layout_type) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)layout_type << 61;
  return d;
}

// The same descriptor in two 32-bit halves, for issue loops that only ever change the address:
// the high word (stride offset, version, layout) is fixed per operand, the low word is
// (address >> 4) | LBO field, and a step of n bytes along a row adds n >> 4 to it.
__device__ __forceinline__ uint32_t desc_hi(uint32_t sbo_bytes, uint32_t layout_type) {
  return ((sbo_bytes >> 4) & 0x3FFF) | (1u << 14) | (layout_type << 29);
}
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr, uint32_t lbo_bytes = 16) {
  return ((saddr >> 4) & 0x3FFF) | (((lbo_bytes >> 4) & 0x3FFF) << 16);
}
__device__ __forceinline__ uint64_t desc_pack(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// Instruction descriptor of kind::f16 / kind::tf32: D format F32 (1) at [4,6), A format [7,10),
// B format [10,13) (1 = BF16, 2 = TF32), A major [15], B major [16] (1 = MN-major),
// N >> 3 at [17,23), M >> 4 at [24,29).
__host__ __device__ constexpr uint32_t make_idesc(int fmt, int a_mn, int b_mn, int M, int N) {
  return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)a_mn << 15) |
         ((uint32_t)b_mn << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}


// A 3-D tensor map (contiguous dim, rows, batch) over a row-major matrix with `ld` elements per
// row, 128-byte swizzle (atom32: the 32-byte-atom variant that 32-bit MN-major operands need).
// es = element size in bytes (2: bfloat16, 4: float32). Defined in gemm_tc.cu.
int encode_map(b200_engine *e, CUtensorMap *map, int es, const void *base, long long inner, long long rows,
               long long batch, long long ld, long long batch_stride, int box_inner, int box_rows, bool atom32);

}  // namespace b200
