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


// ---- sharing a launch's work between the CTAs ---------------------------------------------------
// stream == 0: worker c takes tiles c, c + workers, ... and every k-block of each. stream == 1
// ("stream-K"): tiles [0, first) are taken whole in that same way, and the (tile, k-block) units of
// the tiles from `first` on, tile-major, are cut into `sk_workers` equal contiguous shares (workers
// beyond that number get none), so a launch with fewer tiles than SMs (first == 0), or the ragged
// last wave of a larger one (first == the tiles of the full waves), still keeps every SM busy for
// the same time. A share that holds only part of a tile's k range leaves its fp32 partial tile in a
// workspace; whichever CTA delivers a tile's last missing part adds the parts in k order (the result
// therefore does not depend on who that is) and stores the tile. Every warp role of a kernel walks
// the same pieces through this iterator. Sharing out ALL tiles of a launch of several waves was
// measured and is not done: tiny-YOLO's step went from 2.49 to 3.28 ms (the CTAs then work on tiles
// that are far apart at any one time, and at different k offsets, so the operand slabs that
// neighbouring tiles have in common are no longer asked for together).
struct TilePieces {
  // 32-bit throughout: the host refuses launches of 2^31 tiles or units
  int tile, whole_end, u, u1, num_k, stream, workers, first;
  // worker w of `workers` (CTAs, or CTA pairs that take a tile together)
  __device__ TilePieces(int streamk, int units, int num_k_, int tiles, int w, int workers_, int first_ = 0,
                        int sk_workers = 0) {
    stream = streamk;
    num_k = num_k_;
    workers = workers_;
    first = streamk ? first_ : 0;
    whole_end = streamk ? first_ : tiles;
    tile = w;
    if (sk_workers <= 0) sk_workers = workers_;
    u = w < sk_workers ? (int)((long long)w * units / sk_workers) : units;
    u1 = w < sk_workers ? (int)((long long)(w + 1) * units / sk_workers) : units;
  }
  __device__ TilePieces(int streamk, int units, int num_k_, int tiles)
      : TilePieces(streamk, units, num_k_, tiles, (int)blockIdx.x, (int)gridDim.x) {}
  // the next piece: k-blocks [kb0, kb1) of tile t
  __device__ bool next(int &t, int &kb0, int &kb1) {
    if (tile < whole_end) {
      t = tile;
      kb0 = 0;
      kb1 = num_k;
      tile += workers;
      return true;
    }
    if (!stream || u >= u1) return false;
    const int tr = u / num_k;
    t = first + tr;
    kb0 = u - tr * num_k;
    const int rem = u1 - u;
    kb1 = (num_k - kb0) <= rem ? num_k : kb0 + rem;
    u += kb1 - kb0;
    return true;
  }
};

// The CTA whose share holds unit `unit` (shares start at c * units / grid).
__device__ __forceinline__ int share_of_unit(int unit, int units, int grid) {
  int c = (int)((long long)unit * grid / units);
  while (c + 1 < grid && (int)((long long)(c + 1) * units / grid) <= unit) ++c;
  while (c > 0 && (int)((long long)c * units / grid) > unit) --c;
  return c;
}
// Workspace slot of the part of a tile (whose first unit is tile_u0) that CTA c holds: 2c if the
// part begins c's share, 2c + 1 if it ends it (a share has at most one of each).
__device__ __forceinline__ int share_slot(int c, int tile_u0, int units, int grid) {
  return 2 * c + ((int)((long long)c * units / grid) >= tile_u0 ? 0 : 1);
}

// Whether a launch of `tiles` tiles of `num_k` k-blocks shares out the k range, and over how many
// CTAs. Measured on B200: a k-block costs a CTA about 0.6 microseconds (one SM's share of the L2
// bandwidth), the CTA that finishes a tile reads its parts one after the other at about a
// microsecond each, and handing partial tiles over costs about 3 microseconds per launch. A tile is
// cut into at most sqrt(0.6 num_k) parts (beyond that the fix-up costs more than the shorter k loop
// saves), and the k range is shared only where this estimate says it saves a tenth of the time.
inline bool streamk_pays(long long tiles, int num_k, int sm_count, int *grid) {
  if (num_k < 4 || tiles < 1) return false;
  int parts = 1;
  while ((parts + 1) * (parts + 1) <= 0.6 * num_k) ++parts;
  long long g = tiles * parts;
  if (g > sm_count) g = sm_count;
  if (g > tiles * (long long)num_k / 2) g = tiles * (long long)num_k / 2;
  if (g < 1) return false;
  const long long waves = (tiles + sm_count - 1) / sm_count;
  const double t_whole = 0.6 * (double)waves * num_k;
  const long long units = tiles * (long long)num_k;
  const double parts_per_tile = g > tiles ? (double)((g + tiles - 1) / tiles) : 2.0;
  const double t_shared = 0.6 * (double)((units + g - 1) / g) + parts_per_tile + 3.0;
  if (t_shared >= 0.9 * t_whole) return false;
  *grid = (int)g;
  return true;
}

// The same question for a launch of more tiles than SMs: whether the tiles beyond the full waves
// (tiles % sm_count of them) share their k range out. *first = the tiles taken whole, *sk = the CTAs
// that take a share.
inline bool streamk_tail_pays(long long tiles, int num_k, int sm_count, int *first, int *sk) {
  if (tiles <= sm_count) return false;
  const long long rem = tiles % sm_count;
  if (rem == 0) return false;
  int g = sm_count;
  if (!streamk_pays(rem, num_k, sm_count, &g)) return false;
  *first = (int)(tiles - rem);
  *sk = g;
  return true;
}

// A 3-D tensor map (contiguous dim, rows, batch) over a row-major matrix with `ld` elements per
// row, 128-byte swizzle (atom32: the 32-byte-atom variant that 32-bit MN-major operands need).
// es = element size in bytes (2: bfloat16, 4: float32). Defined in gemm_tc.cu.
int encode_map(b200_engine *e, CUtensorMap *map, int es, const void *base, long long inner, long long rows,
               long long batch, long long ld, long long batch_stride, int box_inner, int box_rows, bool atom32);

}  // namespace b200
