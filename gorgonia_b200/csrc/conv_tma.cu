// Implicit-GEMM 2-D convolution whose col operand is built by the TMA unit (float32 as 3xTF32).
//
//   y[b][k][p] = sum_q  col[(b,p)][q] * Wf[k][q],   q' = (tap, channel),  p = oh*Wo + ow
//
// The same tensor-core mapping as conv_tc.cu (pixels on the 128 TMEM lanes, output channels on
// the columns, hi*hi and cross terms in two accumulators folded every 256 k by the epilogue
// warps), but no thread gathers anything: the activations are first rewritten once, channels
// innermost (NHWC) and split into TF32 head and tail, and every 128-pixel x CK-channel slab of col
// is then ONE im2col-mode TMA load per head/tail. The TMA unit walks the 128 consecutive output
// positions across rows and images, applies the tap offset, fills padding with zeros and writes
// the slab in the swizzled K-major layout the tensor core reads. The rewrite costs 12 bytes per
// input element; the 9 (kh*kw) re-reads of the activations come from L2.
//
// CK = 32 channels per k-block (128-byte rows, 128-byte swizzle), so C must be a multiple of 32.
// (The kernel is also correct with CK = 16, 64-byte rows and swizzle, but at C = 16 the col slabs
// are re-read from L2 nine times at 8 bytes per element and the gather kernel, which reads 4, wins.)
// A 1x1 convolution has no re-reads to save, but it runs here as well: in a chain its input arrives
// already split, and the last layers of a network have few tiles, which this kernel can share out
// over all SMs along k (see ConvTmaParams::streamk).
// Warp roles (10 warps): 0 TMA producer, 1 MMA issuer + TMEM owner, 2-9 epilogue.
// No multicast, no clusters. Every wait is bounded; a time-out raises the engine's error word.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>

#include <atomic>

#include "engine.h"
#include "epilogue.cuh"
#include "ptx.cuh"
#include "tc_common.cuh"
#include "tc_operand.h"

namespace b200 {

// conv_tc.cu: filters split into TF32 head/tail and reordered to (tap, channel); cached for constants
int conv_filters_tap_major(b200_engine *e, const float *w, int K, int C, int taps, TcOperand *wf, void **blk);

constexpr int CT_BM = 128;
constexpr int CT_THREADS = 320;  // 10 warps

struct ConvTmaParams {
  float *y;               // NCHW output, or null when only the split form is wanted
  float *y_hi, *y_lo;     // the output as NHWC TF32 head / tail for the next convolution, or null
  long long Mtot;  // B * Ho * Wo
  int K, Wo, hw;
  int kw, padH, padW, sH, sW, dH, dW;
  int cblocks;     // C / CK
  int num_k;       // taps * cblocks
  int chunk_k;     // k-blocks per accumulation chain
  int tiles_m, tiles_n;
  int stages;
  // how the work is shared between the CTAs (TilePieces, tc_common.cuh)
  int streamk;
  int units;        // tiles * num_k (0 when the k range is not shared)
  int sk_first, sk_workers;  // k ranges are shared from this tile on, among this many CTAs (TilePieces)
  float *ws;        // partial tiles: slot 2c (a part that begins CTA c's share) and 2c + 1 (one that ends it)
  int *tile_count;  // parts delivered per tile; zero between launches
  Epilogue ep;     // bias_kind ROW = per output channel
  int *err_flag;
};

__device__ __forceinline__ float ct_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}
__device__ __forceinline__ void ct_tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

template <int BN, int CK>
__global__ void __launch_bounds__(CT_THREADS, 1)
    conv_tma_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                    const __grid_constant__ CUtensorMap tmW0, const __grid_constant__ CUtensorMap tmW1,
                    const __grid_constant__ ConvTmaParams p) {
  constexpr int ROW_BYTES = CK * 4;               // one pixel's (or one filter's) channels of a k-block
  constexpr int A_BYTES = CT_BM * ROW_BYTES;      // one copy (head or tail) of the col slab
  constexpr int B_BYTES = BN * ROW_BYTES;
  constexpr int STAGE_BYTES = 2 * (A_BYTES + B_BYTES);
  constexpr uint32_t SBO = 8 * ROW_BYTES;         // 8-row groups of the swizzle pattern
  constexpr uint32_t LAYOUT = CK == 32 ? 2 : 4;   // 128-byte / 64-byte swizzle
  constexpr int KK = CK / 8;                      // MMAs (k = 8) per k-block
  constexpr uint32_t IDESC = make_idesc(2, 0, 0, CT_BM, BN);
  // head x [filter head | filter tail] as ONE instruction of width 2*BN: the tail slab follows the
  // head slab in shared memory, the cross-term accumulator follows the main one in tensor memory
  constexpr uint32_t IDESC_WIDE = make_idesc(2, 0, 0, CT_BM, 2 * BN);
  constexpr int ACC_COLS = 2 * BN;
  constexpr int TMEM_COLS = 2 * ACC_COLS;
  constexpr int HALF = BN / 2;
  constexpr int MAX_STAGES = 8;

  extern __shared__ __align__(1024) unsigned char ct_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], acc_full[2], acc_empty[2];
  __shared__ __align__(8) uint64_t epi_bar;  // the 8 epilogue warps meet here when a partial tile is handed over
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_fail, s_last;
  __shared__ float bias_s[8][BN / 2];

  unsigned char *smem = reinterpret_cast<unsigned char *>(((uintptr_t)ct_smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages;
  const long long total_tiles = (long long)p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&acc_full[b], 1);
      ptx::mbar_init(&acc_empty[b], 8);  // one arrival per epilogue warp
    }
    ptx::mbar_init(&epi_bar, 8);
    ptx::fence_mbar_init();
    s_fail = 0;
    s_last = 0;
  }
  if (warp == 1) {
    ptx::tmem_alloc(&tmem_base_s, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tmap(&tmA0);
    ptx::prefetch_tmap(&tmA1);
    ptx::prefetch_tmap(&tmW0);
    ptx::prefetch_tmap(&tmW1);
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    // ---------------- TMA producer: col slabs (im2col mode) and filter slabs ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      TilePieces pieces(p.streamk, p.units, p.num_k, (int)total_tiles, (int)blockIdx.x, (int)gridDim.x, p.sk_first, p.sk_workers);
      int tile, kb0, kb1;
      while (ok && pieces.next(tile, kb0, kb1)) {
        const int mt = (int)(tile / p.tiles_n), nt = (int)(tile % p.tiles_n);
        // first output position of the tile -> window origin in the input
        const long long m0 = (long long)mt * CT_BM;
        const int n = (int)(m0 / p.hw);
        const int pix = (int)(m0 - (long long)n * p.hw);
        const int oh = pix / p.Wo, ow = pix - oh * p.Wo;
        const int w0 = ow * p.sW - p.padW, h0 = oh * p.sH - p.padH;
        const int tap0 = kb0 / p.cblocks;
        int cb = kb0 - tap0 * p.cblocks, r = tap0 / p.kw, sx = tap0 - (tap0 / p.kw) * p.kw;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!ptx::mbar_wait_relaxed(&empty_bar[stage], phase ^ 1, 32)) {
            ok = false;
            break;
          }
          unsigned char *sa = smem + (size_t)stage * STAGE_BYTES;
          unsigned char *sb = sa + 2 * A_BYTES;
          ptx::mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
          const uint16_t off_w = (uint16_t)(sx * p.dW), off_h = (uint16_t)(r * p.dH);
          ptx::tma_load_im2col_4d(sa, &tmA0, cb * CK, w0, h0, n, off_w, off_h, &full_bar[stage]);
          ptx::tma_load_im2col_4d(sa + A_BYTES, &tmA1, cb * CK, w0, h0, n, off_w, off_h, &full_bar[stage]);
          ptx::tma_load_3d(sb, &tmW0, kb * CK, nt * BN, 0, &full_bar[stage]);
          ptx::tma_load_3d(sb + B_BYTES, &tmW1, kb * CK, nt * BN, 0, &full_bar[stage]);
          if (++cb == p.cblocks) {  // q' = (tap, channel): channel blocks run fastest
            cb = 0;
            if (++sx == p.kw) {
              sx = 0;
              ++r;
            }
          }
          if (++stage == stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) s_fail = 1;
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int use = 0;
      bool ok = true;
      TilePieces pieces(p.streamk, p.units, p.num_k, (int)total_tiles, (int)blockIdx.x, (int)gridDim.x, p.sk_first, p.sk_workers);
      int tile, kb0, kb1;
      while (ok && pieces.next(tile, kb0, kb1)) {
        for (int kc = kb0; kc < kb1 && ok; kc += p.chunk_k, ++use) {
          const int buf = use & 1;
          const uint32_t acc_phase = (uint32_t)((use >> 1) & 1);
          if (!ptx::mbar_wait(&acc_empty[buf], acc_phase ^ 1)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t d_main = tmem_base + (uint32_t)(buf * ACC_COLS);
          const uint32_t d_tail = d_main + BN;
          const int kend = kc + p.chunk_k < kb1 ? kc + p.chunk_k : kb1;
          for (int kb = kc; kb < kend; ++kb) {
            if (!ptx::mbar_wait(&full_bar[stage], phase)) {
              ok = false;
              break;
            }
            ptx::tc_fence_after_sync();
            const uint32_t st = ptx::smem_addr(smem + (size_t)stage * STAGE_BYTES);
#pragma unroll
            for (int kk = 0; kk < KK; ++kk) {
              const uint64_t a_hi = make_smem_desc(st + kk * 32, 16, SBO, LAYOUT);
              const uint64_t a_lo = make_smem_desc(st + A_BYTES + kk * 32, 16, SBO, LAYOUT);
              const uint64_t b_hi = make_smem_desc(st + 2 * A_BYTES + kk * 32, 16, SBO, LAYOUT);
              const uint32_t accumulate = (kb > kc || kk > 0) ? 1u : 0u;
              ptx::mma_tf32(d_main, a_hi, b_hi, IDESC_WIDE, accumulate);
              ptx::mma_tf32(d_tail, a_lo, b_hi, IDESC, 1u);
            }
            ptx::mma_commit(&empty_bar[stage]);
            if (++stage == stages) {
              stage = 0;
              phase ^= 1;
            }
          }
          if (ok) ptx::mma_commit(&acc_full[buf]);
        }
      }
      if (!ok) s_fail = 1;
    }
  } else {
    // ---------------- epilogue: warps 2..9 ----------------
    const int quarter = warp & 3;           // TMEM lanes 32*quarter .. +31
    const int half = (warp - 2) >> 2;       // which half of the BN columns
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const bool has_bias = p.ep.bias_kind != B200_BIAS_NONE;
    const float *bias_g = reinterpret_cast<const float *>(p.ep.bias);
    int use = 0;
    uint32_t epi_phase = 0;
    bool ok = true;
    // the epilogue warps' own rendezvous: an mbarrier, so that this wait is bounded like every other
    auto epi_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&epi_bar);
      const bool done = ptx::mbar_wait_relaxed(&epi_bar, epi_phase, 32);
      epi_phase ^= 1;
      return done;
    };
    TilePieces pieces(p.streamk, p.units, p.num_k, (int)total_tiles, (int)blockIdx.x, (int)gridDim.x, p.sk_first, p.sk_workers);
    int tile, kb0, kb1;
    while (ok && pieces.next(tile, kb0, kb1)) {
      const int mt = (int)(tile / p.tiles_n), nt = (int)(tile % p.tiles_n);
      float acc[HALF];
#pragma unroll
      for (int j = 0; j < HALF; ++j) acc[j] = 0.f;
      for (int kc = kb0; kc < kb1 && ok; kc += p.chunk_k) {
        const int buf = use & 1;
        const uint32_t acc_phase = (uint32_t)((use >> 1) & 1);
        ++use;
        if (!ptx::mbar_wait_relaxed(&acc_full[buf], acc_phase)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < HALF; c += 16) {
          uint32_t rm[16], rt[16];
          ct_tmem_ld16(lane_addr + (uint32_t)(buf * ACC_COLS + half * HALF + c), rm);
          ct_tmem_ld16(lane_addr + (uint32_t)(buf * ACC_COLS + BN + half * HALF + c), rt);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j)
            acc[c + j] = __fadd_rn(acc[c + j], __fadd_rn(__uint_as_float(rm[j]), __uint_as_float(rt[j])));
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&acc_empty[buf]);
      }
      if (kb0 != 0 || kb1 != p.num_k) {
        // part of a tile: leave it in the workspace; the CTA that delivers the last part finishes the tile
        const int tile_u0 = (tile - p.sk_first) * p.num_k;  // among the units that are shared out
        const size_t slot_floats = (size_t)CT_BM * BN;
        const size_t within = ((size_t)(warp - 2) * HALF) * 32 + lane;
        if (ok) {
          float *wsp = p.ws + (size_t)share_slot(blockIdx.x, tile_u0, p.units, p.sk_workers) * slot_floats + within;
#pragma unroll
          for (int j = 0; j < HALF; ++j) __stcg(wsp + j * 32, acc[j]);
        } else {
          s_fail = 1;
        }
        __threadfence();
        const int c_first = share_of_unit(tile_u0, p.units, p.sk_workers);
        const int c_last = share_of_unit(tile_u0 + p.num_k - 1, p.units, p.sk_workers);
        bool met = epi_sync();
        if (warp == 2 && lane == 0) {
          s_last = (atomicAdd(p.tile_count + (tile - p.sk_first), 1) == c_last - c_first) ? 1 : 0;
          if (s_last) p.tile_count[tile - p.sk_first] = 0;  // zero again for the next launch
        }
        met = epi_sync() && met;
        if (!met || *(volatile int *)&s_fail) {
          ok = false;
          break;
        }
        if (!*(volatile int *)&s_last) continue;
        __threadfence();
#pragma unroll
        for (int j = 0; j < HALF; ++j) acc[j] = 0.f;
        for (int c = c_first; c <= c_last; ++c) {  // k order: CTA c's share precedes CTA c + 1's
          const float *src = p.ws + (size_t)share_slot(c, tile_u0, p.units, p.sk_workers) * slot_floats + within;
#pragma unroll
          for (int j = 0; j < HALF; ++j) acc[j] = __fadd_rn(acc[j], ptx::ld_cg_ordered(src + j * 32));
        }
      }
      if (!ok) break;
      const long long m = (long long)mt * CT_BM + quarter * 32 + lane;
      const int n0 = nt * BN + half * HALF;
      float *yb = nullptr;
      if (m < p.Mtot) {
        long long b;
        int pix;
        if (p.Mtot < (1LL << 31)) {  // the usual case: 32-bit division
          const uint32_t mu = (uint32_t)m, bu = mu / (uint32_t)p.hw;
          b = bu;
          pix = (int)(mu - bu * (uint32_t)p.hw);
        } else {
          b = m / p.hw;
          pix = (int)(m % p.hw);
        }
        yb = p.y ? p.y + (b * p.K + n0) * (long long)p.hw + pix : nullptr;
      }
      // this warp's biases, staged once per tile (lane l holds channels l and l + 32)
      if (has_bias) {
        __syncwarp();
#pragma unroll
        for (int j = lane; j < HALF; j += 32) bias_s[warp - 2][j] = n0 + j < p.K ? bias_g[n0 + j] : 0.f;
        __syncwarp();
      }
      if (p.y_hi)  // position m of the flattened (b, oh, ow) index is row m of the NHWC tensor
        store_channels_split<HALF, false>(acc, yb, p.hw, p.K - n0, has_bias ? bias_s[warp - 2] : nullptr, p.ep.act,
                                          (float)p.ep.alpha, m < p.Mtot, p.y_hi + (m < p.Mtot ? m : 0) * p.K + n0,
                                          p.y_lo + (m < p.Mtot ? m : 0) * p.K + n0);
      else if (yb)
        store_channels<HALF>(acc, yb, p.hw, p.K - n0, has_bias ? bias_s[warp - 2] : nullptr, p.ep.act,
                             (float)p.ep.alpha);
    }
    if (!ok) s_fail = 1;
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && s_fail) atomicExch(p.err_flag, 1);
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// x (B, C, HW) -> head/tail (B, HW, C): channels innermost, each value split into its TF32 head
// and the TF32 rounding of the remainder. One 32 x 32 tile per step through shared memory, so both
// the reads (along HW) and the writes (along C) are contiguous.
__global__ void __launch_bounds__(256) nhwc_split_kernel(const float *__restrict__ x, float *__restrict__ hi,
                                                         float *__restrict__ lo, long long B, int C, int HW) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int ptiles = (HW + 31) / 32, ctiles = (C + 31) / 32;
  const long long per_image = (long long)ptiles * ctiles, total = B * per_image;
  for (long long t = blockIdx.x; t < total; t += gridDim.x) {
    const long long b = t / per_image;
    const int rem = (int)(t - b * per_image);
    const int ct = rem / ptiles, pt = rem - ct * ptiles;
    const int c0 = ct * 32, p0 = pt * 32;
    const float *xb = x + b * (long long)C * HW;
#pragma unroll
    for (int j = ty; j < 32; j += 8) {
      const int c = c0 + j, pp = p0 + tx;
      tile[j][tx] = (c < C && pp < HW) ? __ldg(xb + (long long)c * HW + pp) : 0.f;
    }
    __syncthreads();
    const long long ob = b * (long long)HW * C;
#pragma unroll
    for (int j = ty; j < 32; j += 8) {
      const int pp = p0 + j, c = c0 + tx;
      if (pp < HW && c < C) {
        const float v = tile[tx][j];
        const float h = ct_tf32(v);
        const long long o = ob + (long long)pp * C + c;
        hi[o] = h;
        lo[o] = ct_tf32(__fsub_rn(v, h));
      }
    }
    __syncthreads();
  }
}

// The same rewrite for planes whose size is a multiple of 4 (so every channel row starts on a
// 16-byte boundary): a tile of CT channels x 128 positions is read as float4 along the positions
// (512 contiguous bytes per warp and channel), turned in shared memory (row pitch 129 words: the
// four channels a thread gathers for one position fall into distinct banks), and written as float4
// along the channels, CT * 4 contiguous bytes per position.
template <int CT>
__global__ void __launch_bounds__(256) nhwc_split4_kernel(const float *__restrict__ x, float *__restrict__ hi,
                                                          float *__restrict__ lo, long long B, int C, int HW) {
  constexpr int PT = 128, PITCH = PT + 1;
  __shared__ float tile[CT * PITCH];
  const int ptiles = (HW + PT - 1) / PT, ctiles = C / CT;
  const long long per_image = (long long)ptiles * ctiles, total = B * per_image;
  for (long long t = blockIdx.x; t < total; t += gridDim.x) {
    const long long b = t / per_image;
    const int rem = (int)(t - b * per_image);
    const int ct = rem / ptiles, pt = rem - ct * ptiles;
    const int c0 = ct * CT, p0 = pt * PT;
    const float *xb = x + (b * C + c0) * (long long)HW + p0;
    // load: float4 q of channel row c covers positions 4q .. 4q+3
#pragma unroll
    for (int i = threadIdx.x; i < CT * (PT / 4); i += 256) {
      const int c = i / (PT / 4), q = i - c * (PT / 4);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (p0 + 4 * q < HW) v = __ldg(reinterpret_cast<const float4 *>(xb + (long long)c * HW) + q);
      float *d = &tile[c * PITCH + 4 * q];
      d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
    }
    __syncthreads();
    // store: thread -> (position, group of 4 channels), channel groups fastest
    float *ho = hi + (b * HW + p0) * (long long)C + c0;
    float *lo_o = lo + (b * HW + p0) * (long long)C + c0;
#pragma unroll
    for (int i = threadIdx.x; i < PT * (CT / 4); i += 256) {
      const int pp = i / (CT / 4), cg = i - pp * (CT / 4);
      if (p0 + pp < HW) {
        float v[4], h[4], l[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          v[k] = tile[(4 * cg + k) * PITCH + pp];
          h[k] = ct_tf32(v[k]);
          l[k] = ct_tf32(__fsub_rn(v[k], h[k]));
        }
        *reinterpret_cast<float4 *>(ho + (long long)pp * C + 4 * cg) = make_float4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<float4 *>(lo_o + (long long)pp * C + 4 * cg) = make_float4(l[0], l[1], l[2], l[3]);
      }
    }
    __syncthreads();
  }
}

// The same rewrite for small planes of any size (7x7, 13x13): a block takes 32 channels of one
// image, which are 32 * HW contiguous floats starting on a 16-byte boundary whatever HW is, loads
// them as float4, and writes every position's 32 channels as float4. The shared-memory pitch is
// HW rounded up to 1 (mod 8), which spreads the (position, channel group) reads over all banks.
__global__ void __launch_bounds__(256) nhwc_split_img_kernel(const float *__restrict__ x, float *__restrict__ hi,
                                                             float *__restrict__ lo, long long B, int C, int HW,
                                                             int pitch) {
  extern __shared__ __align__(16) float img[];
  const int chunks = C >> 5;
  const long long total = B * chunks;
  const int n4 = (32 * HW) >> 2;
  for (long long t = blockIdx.x; t < total; t += gridDim.x) {
    const long long b = t / chunks;
    const int c0 = (int)(t - b * chunks) << 5;
    const float4 *src = reinterpret_cast<const float4 *>(x + (b * C + c0) * (long long)HW);
    for (int i = threadIdx.x; i < n4; i += 256) {
      const float4 v = __ldg(src + i);
      const int e0 = i << 2;
      const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {  // the four elements may straddle two channel rows
        const int e = e0 + k, c = e / HW, pp = e - c * HW;
        img[c * pitch + pp] = vv[k];
      }
    }
    __syncthreads();
    float *ho = hi + (b * HW) * (long long)C + c0;
    float *lo_o = lo + (b * HW) * (long long)C + c0;
    for (int i = threadIdx.x; i < HW * 8; i += 256) {
      const int pp = i >> 3, cg = i & 7;
      float h[4], l[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float v = img[(4 * cg + k) * pitch + pp];
        h[k] = ct_tf32(v);
        l[k] = ct_tf32(__fsub_rn(v, h[k]));
      }
      *reinterpret_cast<float4 *>(ho + (long long)pp * C + 4 * cg) = make_float4(h[0], h[1], h[2], h[3]);
      *reinterpret_cast<float4 *>(lo_o + (long long)pp * C + 4 * cg) = make_float4(l[0], l[1], l[2], l[3]);
    }
    __syncthreads();
  }
}

// Rewrites x (B, C, HW) as NHWC TF32 head/tail into two fresh arena blocks xs[0], xs[1], which the
// caller releases.
static int launch_nhwc_split(b200_engine *e, const float *x, long long B, int C, int HW, void **xs);
int conv_nhwc_split(b200_engine *e, const float *x, long long B, int C, int HW, void **xs) {
  const long long xbytes = B * C * HW * 4;
  xs[0] = xs[1] = nullptr;
  int rc = b200_get(e, xbytes, &xs[0]);
  if (rc == B200_OK) rc = b200_get(e, xbytes, &xs[1]);
  if (rc != B200_OK) return rc;
  return launch_nhwc_split(e, x, B, C, HW, xs);
}
static int launch_nhwc_split(b200_engine *e, const float *x, long long B, int C, int HW, void **xs) {
  if (HW % 4 == 0 && C % 16 == 0 && (uintptr_t)x % 16 == 0) {
    const int ct = C % 32 == 0 ? 32 : 16;
    const long long tiles = B * ((HW + 127) / 128) * (C / ct);
    const int blocks = (int)std::max<long long>(1, std::min<long long>(tiles, e->sm_count * 32LL));
    if (ct == 32)
      nhwc_split4_kernel<32><<<blocks, 256, 0, e->stream>>>(x, (float *)xs[0], (float *)xs[1], B, C, HW);
    else
      nhwc_split4_kernel<16><<<blocks, 256, 0, e->stream>>>(x, (float *)xs[0], (float *)xs[1], B, C, HW);
    B200_CHECK_LAUNCH(e, "nhwc_split4_kernel");
    return B200_OK;
  }
  if (C % 32 == 0 && HW <= 360 && (uintptr_t)x % 16 == 0) {  // 32 * pitch floats fit the default 48 KB
    int pitch = HW;
    while (pitch % 8 != 1) ++pitch;
    const long long work = B * (C / 32);
    const int blocks = (int)std::max<long long>(1, std::min<long long>(work, e->sm_count * 16LL));
    nhwc_split_img_kernel<<<blocks, 256, (size_t)32 * pitch * 4, e->stream>>>(x, (float *)xs[0], (float *)xs[1], B, C,
                                                                             HW, pitch);
    B200_CHECK_LAUNCH(e, "nhwc_split_img_kernel");
    return B200_OK;
  }
  const long long tiles = B * ((HW + 31) / 32) * ((C + 31) / 32);
  const int blocks = (int)std::max<long long>(1, std::min<long long>(tiles, e->sm_count * 16LL));
  nhwc_split_kernel<<<blocks, 256, 0, e->stream>>>(x, (float *)xs[0], (float *)xs[1], B, C, HW);
  B200_CHECK_LAUNCH(e, "nhwc_split_kernel");
  return B200_OK;
}

// The same rewrite into buffers the caller owns (B * C * HW floats each).
int conv_nhwc_split_into(b200_engine *e, const float *x, long long B, int C, int HW, float *hi, float *lo) {
  void *xs[2] = {hi, lo};
  return launch_nhwc_split(e, x, B, C, HW, xs);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const int *, const int *, cuuint32_t, cuuint32_t,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static void *driver_entry(const char *name) {
  void *sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
    return sym;
  return nullptr;
}

template <int BN, int CK>
static int launch_conv_tma(b200_engine *e, const CUtensorMap *tm, ConvTmaParams &p) {
  constexpr int STAGE_BYTES = 2 * (CT_BM + BN) * CK * 4;
  auto kern = conv_tma_kernel<BN, CK>;
  static std::atomic<int> attr_dev_mask{0};  // devices on which the attribute is set; engines on other threads share it
  const size_t optin = std::min<size_t>(e->smem_optin, 227 * 1024);
  if (!(attr_dev_mask & (1 << (e->device & 31)))) {
    cudaFuncAttributes fa;
    B200_CHECK_CUDA(e, cudaFuncGetAttributes(&fa, kern));
    B200_CHECK_CUDA(e, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)(optin - fa.sharedSizeBytes)));
    attr_dev_mask |= 1 << (e->device & 31);
  }
  p.stages = (int)std::max<size_t>(2, std::min<size_t>(8, (optin - 4096) / STAGE_BYTES));
  const size_t smem = (size_t)p.stages * STAGE_BYTES + 1024;
  const long long tiles = (long long)p.tiles_m * p.tiles_n;
  int grid = (int)std::min<long long>(tiles, e->sm_count);
  // Whole tiles per CTA leave SMs idle when the tiles do not fill the last wave: with fewer tiles
  // than SMs, or e.g. 169 tiles on 148 SMs. Then the k range is shared out instead (TilePieces).
  void *ws = nullptr;
  p.streamk = 0;
  p.units = 0;
  p.sk_first = 0;
  p.sk_workers = grid;
  if (tiles >= (1LL << 31))
    return set_error(e, B200_ERR_UNSUPPORTED, "convolution: %lld output tiles are more than one launch takes", tiles);
  int sk_grid = grid;
  if (!(e->flags & B200_ENGINE_NO_STREAMK) && tiles <= b200_engine::kSkCounters &&
      streamk_pays(tiles, p.num_k, e->sm_count, &sk_grid)) {
    if (b200_get(e, 2LL * sk_grid * CT_BM * BN * 4, &ws) == B200_OK) {
      grid = sk_grid;
      p.streamk = 1;
      p.units = (int)(tiles * p.num_k);  // small: k sharing is for launches of few tiles
      p.sk_workers = grid;
      p.tile_count = e->sk_counters;
      p.ws = (float *)ws;
    }  // else: no room for the partial tiles, whole tiles per CTA
  } else if (int first = 0, sk = 0; !(e->flags & B200_ENGINE_NO_STREAMK) && tiles % e->sm_count <= b200_engine::kSkCounters &&
                                    streamk_tail_pays(tiles, p.num_k, e->sm_count, &first, &sk)) {
    // several waves of tiles and a ragged last one: the full waves whole, the rest along k
    if (b200_get(e, 2LL * sk * CT_BM * BN * 4, &ws) == B200_OK) {
      p.streamk = 1;
      p.sk_first = first;
      p.sk_workers = sk;
      p.units = (int)((tiles - first) * p.num_k);
      p.tile_count = e->sk_counters;
      p.ws = (float *)ws;
    }
  }
  kern<<<grid, CT_THREADS, smem, e->stream>>>(tm[0], tm[1], tm[2], tm[3], p);
  cudaError_t le = cudaGetLastError();
  if (ws) b200_put(e, ws, 0);  // stream order: whoever gets the block next runs after this kernel
  if (le != cudaSuccess)
    return set_error(e, B200_ERR_CUDA, "launch of conv_tma_kernel failed: %s", cudaGetErrorString(le));
  e->launches++;
  e->flags_dirty = true;
  return B200_OK;
}

// Whether the TMA unit builds the col operand of this convolution: channels a multiple of 32,
// window corners and tap offsets inside the ranges an im2col tensor map can
// encode, and an input of at least 128 KB.
bool conv_tma_eligible(long long B, int C, int H, int W, int kh, int kw, int padH, int padW, int sH, int sW, int dH,
                       int dW) {
  if (C % 32 != 0) return false;
  const int spanH = (kh - 1) * dH, spanW = (kw - 1) * dW;
  if (padH > 128 || padW > 128 || padH - spanH < -128 || padW - spanW < -128) return false;
  if (spanH > 255 || spanW > 255) return false;
  if (sH > 8 || sW > 8) return false;
  if (B >= (1LL << 31)) return false;
  if (B * C * H * W * 4 < 131072) return false;
  return true;
}

// x (B,C,H,W) * w (K,C,kh,kw) -> y (B,K,Ho,Wo), float32. ep.bias_kind ROW = one value per channel.
int conv2d_tma(b200_engine *e, const float *x, const float *w, float *y, long long B, int C, int H, int W, int K,
               int kh, int kw, int padH, int padW, int sH, int sW, int dH, int dW, int Ho, int Wo,
               const Epilogue &ep, const float *x_hi, const float *x_lo, float *y_hi, float *y_lo) {
  static EncodeTiledFn enc_tiled = (EncodeTiledFn)driver_entry("cuTensorMapEncodeTiled");
  static EncodeIm2colFn enc_im2col = (EncodeIm2colFn)driver_entry("cuTensorMapEncodeIm2col");
  if (!enc_tiled || !enc_im2col)
    return set_error(e, B200_ERR_CUDA, "cuTensorMapEncodeTiled / cuTensorMapEncodeIm2col are not available");
  const int taps = kh * kw, crs = C * taps;
  const int ck = 32;
  const CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B;

  TcOperand wf;
  void *wblk[2] = {nullptr, nullptr};
  int rc = conv_filters_tap_major(e, w, K, C, taps, &wf, wblk);
  if (rc != B200_OK) return rc;

  // activations: NHWC, TF32 head and tail
  void *xs[2] = {nullptr, nullptr};
  const void *xin[2] = {x_hi, x_lo};  // the caller's pre-split input, or this call's own rewrite
  if (!x_hi) {
    rc = conv_nhwc_split(e, x, B, C, H * W, xs);
    xin[0] = xs[0];
    xin[1] = xs[1];
  }

  int bn = 128;
  while (bn > 32 && bn / 2 >= K) bn /= 2;
  ConvTmaParams p = ConvTmaParams();
  p.y = y;
  p.y_hi = y_hi;
  p.y_lo = y_lo;
  p.Mtot = B * Ho * Wo;
  p.K = K; p.Wo = Wo; p.hw = Ho * Wo;
  p.kw = kw; p.padH = padH; p.padW = padW; p.sH = sH; p.sW = sW; p.dH = dH; p.dW = dW;
  p.cblocks = C / ck;
  p.num_k = taps * p.cblocks;
  p.chunk_k = 256 / ck;
  p.tiles_m = (int)((p.Mtot + CT_BM - 1) / CT_BM);
  p.tiles_n = (K + bn - 1) / bn;
  p.ep = ep;
  p.err_flag = e->d_flags + 2;

  CUtensorMap tm[4];
  memset((void *)tm, 0, sizeof tm);
  if (rc == B200_OK) {
    // activations as (C, W, H, N); the bounding box of window origins runs from -pad to the last
    // origin whose window still touches the padded image
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)C * 4, (cuuint64_t)W * C * 4, (cuuint64_t)H * W * C * 4};
    int lower[2] = {-padW, -padH};
    int upper[2] = {padW - (kw - 1) * dW, padH - (kh - 1) * dH};
    cuuint32_t estr[4] = {1, (cuuint32_t)sW, (cuuint32_t)sH, 1};
    for (int h = 0; h < 2 && rc == B200_OK; ++h) {
      CUresult r = enc_im2col(&tm[h], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void *>(xin[h]), dims, strides,
                              lower, upper,
                              (cuuint32_t)ck, CT_BM, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS)
        rc = set_error(e, B200_ERR_CUDA, "cuTensorMapEncodeIm2col failed (%d): C %d W %d H %d N %lld", (int)r, C, W,
                       H, B);
    }
    // filters as (crs, K, 1), box ck x bn
    cuuint64_t wdims[3] = {(cuuint64_t)crs, (cuuint64_t)K, 1};
    cuuint64_t wstrides[2] = {(cuuint64_t)wf.ld * 4, (cuuint64_t)K * wf.ld * 4};
    cuuint32_t wbox[3] = {(cuuint32_t)ck, (cuuint32_t)bn, 1};
    cuuint32_t westr[3] = {1, 1, 1};
    for (int h = 0; h < 2 && rc == B200_OK; ++h) {
      CUresult r = enc_tiled(&tm[2 + h], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(h ? wf.p1 : wf.p0),
                             wdims, wstrides, wbox, westr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) rc = set_error(e, B200_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for filters", (int)r);
    }
  }
  if (rc == B200_OK) {
    if (bn == 128) rc = launch_conv_tma<128, 32>(e, tm, p);
    else if (bn == 64) rc = launch_conv_tma<64, 32>(e, tm, p);
    else rc = launch_conv_tma<32, 32>(e, tm, p);
  }
  for (int h = 0; h < 2; ++h) {
    if (xs[h]) b200_put(e, xs[h], 0);
    if (wblk[h]) b200_put(e, wblk[h], 0);
  }
  return rc;
}

}  // namespace b200
