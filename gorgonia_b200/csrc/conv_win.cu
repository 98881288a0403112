// Implicit-GEMM 2-D convolution (stride 1) that keeps an input WINDOW in shared memory and lets
// every filter tap read it in place (float32 as 3xTF32).
//
// A CTA tile is 16 x 16 output positions of one image. Its inputs, for one block of CK channels,
// are the (16 + (kh-1)*dil) x (16 + (kw-1)*dil) window around it, which one tiled TMA load brings
// from the NHWC TF32 head/tail copy of the activations into shared memory as rows of CK channels
// (pitch = window width, swizzled, padding filled with zeros by the TMA unit). The col operand of
// tap (r, s) for the left or right 16 x 8 half of the tile is then that same buffer read from a
// shifted start row: tensor-core row m = 8*i + j is window row (r*dil + i) * pitch + s*dil + j
// (+8 for the right half), i.e. groups of 8 consecutive rows one window pitch apart, which is
// exactly what a K-major shared-memory descriptor expresses (group stride = pitch). The swizzle
// is a function of the shared-memory address, so a shifted start row reads what TMA wrote.
// Each input element therefore crosses L2 -> shared memory about 1.3 times instead of kh*kw times
// (im2col mode) and no thread touches it; each filter slab serves 256 positions.
//
// Accumulation as in the other tensor-core kernels: hi*hi in one TMEM accumulator, the two cross
// terms in a second, chains cut every 256 k and folded in fp32 registers by the epilogue warps.
// Warp roles (12 warps): 0 window producer, 1 and 11 MMA issuers (left / right tile half; 1 owns
// tensor memory), 2-9 epilogue (4 lane quarters x 2 tile halves), 10 filter producer. No multicast, no clusters; every wait is bounded.
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

int conv_filters_tap_major(b200_engine *e, const float *w, int K, int C, int taps, TcOperand *wf, void **blk);
int conv_nhwc_split(b200_engine *e, const float *x, long long B, int C, int HW, void **xs);

constexpr int CW_THREADS = 384;  // 12 warps
constexpr int CW_ISSUERS = 2;    // one MMA-issuing warp per tile half
constexpr int CW_TILE = 16;      // output tile edge
constexpr int CW_WIN_STAGES = 2;
constexpr int CW_MAX_BSTAGES = 12;

struct ConvWinParams {
  float *y;               // NCHW output, or null when only the split form is wanted
  float *y_hi, *y_lo;     // the (pooled) output as NHWC TF32 head / tail for the next convolution, or null
  int K, Ho, Wo;
  int kh, kw, dH, dW, padH, padW;
  int win_w;         // window pitch in rows: 16 + (kw-1)*dW
  int win_bytes;     // one copy (head or tail) of the window, padded to 1024
  int cblocks;       // C / CK
  int C;
  int chunk_k;       // k-blocks per accumulation chain
  int tiles_h, tiles_w, tiles_n;
  long long total_tiles;  // B * tiles_h * tiles_w * tiles_n
  int b_stages;
  Epilogue ep;       // bias_kind ROW = per output channel
  int pool2;         // fold a 2x2 / stride-2 max-pool into the store: y is (B, K, Ho/2, Wo/2)
  int *err_flag;
};

__device__ __forceinline__ void cw_tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void cw_tma_load_4d(void *smem_dst, const void *tmap, int c0, int c1, int c2, int c3,
                                               uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, "
      "%6}], [%2];" ::"r"(ptx::smem_addr(smem_dst)),
      "l"(tmap), "r"(ptx::smem_addr(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

template <int BN, int CK>
__global__ void __launch_bounds__(CW_THREADS, 1)
    conv_win_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                    const __grid_constant__ CUtensorMap tmW0, const __grid_constant__ CUtensorMap tmW1,
                    const __grid_constant__ ConvWinParams p) {
  constexpr int ROW_BYTES = CK * 4;
  constexpr int B_BYTES = BN * ROW_BYTES;
  constexpr int B_STAGE_BYTES = 2 * B_BYTES;      // head + tail
  constexpr uint32_t B_SBO = 8 * ROW_BYTES;
  constexpr uint32_t LAYOUT = CK == 32 ? 2 : 4;   // 128-byte / 64-byte swizzle
  constexpr int KK = CK / 8;                      // MMAs (k = 8) per k-block
  constexpr uint32_t IDESC = make_idesc(2, 0, 0, 128, BN);
  constexpr uint32_t IDESC2 = make_idesc(2, 0, 0, 128, 2 * BN);  // [head | tail] filter slabs as one operand
  constexpr int ACC_COLS = 4 * BN;                // two tile halves x (main + cross-term)
  constexpr int TMEM_COLS = 2 * ACC_COLS;         // double-buffered: 256 (BN 32) or 512 (BN 64)

  extern __shared__ __align__(1024) unsigned char cw_smem_raw[];
  __shared__ __align__(8) uint64_t win_full[CW_WIN_STAGES], win_empty[CW_WIN_STAGES];
  __shared__ __align__(8) uint64_t b_full[CW_MAX_BSTAGES], b_empty[CW_MAX_BSTAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_fail;
  __shared__ float bias_s[8][BN];

  unsigned char *smem = reinterpret_cast<unsigned char *>(((uintptr_t)cw_smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char *smem_b = smem + (size_t)CW_WIN_STAGES * 2 * p.win_bytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b_stages = p.b_stages;
  const int taps = p.kh * p.kw;
  const uint32_t a_sbo = (uint32_t)p.win_w * ROW_BYTES;  // one window row of positions further

  if (threadIdx.x == 0) {
    for (int s = 0; s < CW_WIN_STAGES; ++s) {
      ptx::mbar_init(&win_full[s], 1);
      ptx::mbar_init(&win_empty[s], CW_ISSUERS);
    }
    for (int s = 0; s < b_stages; ++s) {
      ptx::mbar_init(&b_full[s], 1);
      ptx::mbar_init(&b_empty[s], CW_ISSUERS);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&acc_full[b], CW_ISSUERS);
      ptx::mbar_init(&acc_empty[b], 8);  // one arrival per epilogue warp
    }
    ptx::fence_mbar_init();
    s_fail = 0;
  }
  if (warp == 1) {
    ptx::tmem_alloc(&tmem_base_s, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tmap(&tmA0);
    ptx::prefetch_tmap(&tmA1);
  }
  if (warp == 10 && lane == 0) {
    ptx::prefetch_tmap(&tmW0);
    ptx::prefetch_tmap(&tmW1);
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  const int tiles_per_image = p.tiles_h * p.tiles_w;

  if (warp == 0) {
    // ---------------- window producer ----------------
    if (lane == 0) {
      int ws = 0;
      uint32_t wphase = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
        const long long st = tile / p.tiles_n;  // spatial tile; the column tile runs fastest
        const int b = (int)(st / tiles_per_image);
        const int rem = (int)(st - (long long)b * tiles_per_image);
        const int th = rem / p.tiles_w, tw = rem - th * p.tiles_w;
        const int h0 = th * CW_TILE - p.padH, w0 = tw * CW_TILE - p.padW;
        for (int cb = 0; cb < p.cblocks; ++cb) {
          if (!ptx::mbar_wait_relaxed(&win_empty[ws], wphase ^ 1, 32)) {
            ok = false;
            break;
          }
          unsigned char *sa = smem + (size_t)ws * 2 * p.win_bytes;
          ptx::mbar_arrive_expect_tx(&win_full[ws], 2u * (uint32_t)(p.win_w * (CW_TILE + (p.kh - 1) * p.dH)) * ROW_BYTES);
          cw_tma_load_4d(sa, &tmA0, cb * CK, w0, h0, b, &win_full[ws]);
          cw_tma_load_4d(sa + p.win_bytes, &tmA1, cb * CK, w0, h0, b, &win_full[ws]);
          if (++ws == CW_WIN_STAGES) {
            ws = 0;
            wphase ^= 1;
          }
        }
      }
      if (!ok) s_fail = 1;
    }
  } else if (warp == 10) {
    // ---------------- filter producer ----------------
    if (lane == 0) {
      int bs = 0;
      uint32_t bphase = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
        const int nt = (int)(tile % p.tiles_n);
        for (int cb = 0; cb < p.cblocks && ok; ++cb) {
          for (int tap = 0; tap < taps; ++tap) {
            if (!ptx::mbar_wait_relaxed(&b_empty[bs], bphase ^ 1, 32)) {
              ok = false;
              break;
            }
            unsigned char *sb = smem_b + (size_t)bs * B_STAGE_BYTES;
            ptx::mbar_arrive_expect_tx(&b_full[bs], B_STAGE_BYTES);
            ptx::tma_load_3d(sb, &tmW0, tap * p.C + cb * CK, nt * BN, 0, &b_full[bs]);
            ptx::tma_load_3d(sb + B_BYTES, &tmW1, tap * p.C + cb * CK, nt * BN, 0, &b_full[bs]);
            if (++bs == b_stages) {
              bs = 0;
              bphase ^= 1;
            }
          }
        }
      }
      if (!ok) s_fail = 1;
    }
  } else if (warp == 1 || warp == 11) {
    // ---------------- MMA issuers ----------------
    // Two warps, one per 16 x 8 half of the tile: each waits on the same stages and issues only its
    // half's instructions into its half's accumulators, and the stage / accumulator barriers count
    // one arrival per issuer. An issuing thread spends about as long on an instruction as the
    // tensor core does at these widths, so two of them keep it fed where one did not.
    // The whole warp runs the loops and votes on every wait, so that stage indices, addresses and
    // descriptors are warp-uniform values; one elected lane issues the tensor-core instructions.
    const uint32_t mh = warp == 1 ? 0u : 1u;
    int ws = 0, bs = 0;
    uint32_t wphase = 0, bphase = 0;
    int use = 0;
    bool ok = true;
    const int num_k = taps * p.cblocks;
    const uint32_t a_hi32 = desc_hi(a_sbo, LAYOUT), b_hi32 = desc_hi(B_SBO, LAYOUT);
    const uint32_t smem_u = ptx::smem_addr(smem), smem_b_u = ptx::smem_addr(smem_b);
    for (long long tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
      int kb = 0;       // k-block of this tile: (channel block, tap), taps fastest
      int in_chain = 0; // k-blocks issued into the open accumulation chain
      uint32_t d_base = 0;
      for (int cb = 0; cb < p.cblocks && ok; ++cb) {
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(&win_full[ws], wphase));
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t win = smem_u + (uint32_t)ws * 2u * (uint32_t)p.win_bytes;
        for (int r = 0; r < p.kh && ok; ++r) {
          for (int sx = 0; sx < p.kw; ++sx, ++kb) {
            if (in_chain == 0) {  // open a chain: needs a free accumulator buffer
              const int buf = use & 1;
              const uint32_t acc_phase = (uint32_t)((use >> 1) & 1);
              ok = __all_sync(0xffffffffu, ptx::mbar_wait(&acc_empty[buf], acc_phase ^ 1));
              if (!ok) break;
              d_base = tmem_base + (uint32_t)(buf * ACC_COLS);
            }
            ok = __all_sync(0xffffffffu, ptx::mbar_wait(&b_full[bs], bphase));
            if (!ok) break;
            ptx::tc_fence_after_sync();
            const uint32_t sb = smem_b_u + (uint32_t)bs * B_STAGE_BYTES;
            const uint32_t row0 = (uint32_t)((r * p.dH) * p.win_w + sx * p.dW);
            // low descriptor words: (address >> 4) | LBO field; a k step of 8 floats adds 32 bytes = 2
            const uint32_t a_lo32 = desc_lo(win + row0 * ROW_BYTES);
            const uint32_t a_lo32_tail = desc_lo(win + (uint32_t)p.win_bytes + row0 * ROW_BYTES);
            const uint32_t b_lo32 = desc_lo(sb);
            const uint32_t first = in_chain > 0 ? 1u : 0u;
            if (lane == 0) {
              const uint32_t ah = mh * ((8u * ROW_BYTES) >> 4);  // right half: 8 window rows further
              const uint32_t d = d_base + mh * (2 * BN);
#pragma unroll
              for (int kk = 0; kk < KK; ++kk) {
                const uint64_t b_hi = desc_pack(b_lo32 + 2u * kk, b_hi32);
                const uint64_t a_hi = desc_pack(a_lo32 + ah + 2u * kk, a_hi32);
                const uint64_t a_lo = desc_pack(a_lo32_tail + ah + 2u * kk, a_hi32);
                const uint32_t accumulate = kk > 0 ? 1u : first;
                // head x [head | tail] of the filters is ONE instruction of width 2*BN: the filter
                // tail slab follows the head slab in shared memory, the cross-term accumulator
                // follows the main one in tensor memory.
                ptx::mma_tf32(d, a_hi, b_hi, IDESC2, accumulate);
                ptx::mma_tf32(d + BN, a_lo, b_hi, IDESC, 1u);
              }
              ptx::mma_commit(&b_empty[bs]);
            }
            if (++bs == b_stages) {
              bs = 0;
              bphase ^= 1;
            }
            if (++in_chain == p.chunk_k || kb + 1 == num_k) {  // close the chain
              if (lane == 0) ptx::mma_commit(&acc_full[use & 1]);
              ++use;
              in_chain = 0;
            }
            __syncwarp();
          }
        }
        if (ok && lane == 0) ptx::mma_commit(&win_empty[ws]);
        __syncwarp();
        if (++ws == CW_WIN_STAGES) {
          ws = 0;
          wphase ^= 1;
        }
      }
    }
    if (!ok && lane == 0) s_fail = 1;
  } else {
    // ---------------- epilogue: warps 2..9 ----------------
    const int quarter = warp & 3;          // TMEM lanes 32*quarter .. +31
    const int half = (warp - 2) >> 2;      // left / right 16 x 8 half of the tile
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int m = quarter * 32 + lane;     // tensor-core row: position (m / 8, m % 8 + 8*half) of the tile
    const int num_k = taps * p.cblocks;
    const bool has_bias = p.ep.bias_kind != B200_BIAS_NONE;
    const float *bias_g = reinterpret_cast<const float *>(p.ep.bias);
    int use = 0;
    bool ok = true;
    for (long long tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
      float acc[BN];
#pragma unroll
      for (int j = 0; j < BN; ++j) acc[j] = 0.f;
      for (int kc = 0; kc < num_k && ok; kc += p.chunk_k) {
        const int buf = use & 1;
        const uint32_t acc_phase = (uint32_t)((use >> 1) & 1);
        ++use;
        if (!ptx::mbar_wait_relaxed(&acc_full[buf], acc_phase)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < BN; c += 16) {
          uint32_t rm[16], rt[16];
          cw_tmem_ld16(lane_addr + (uint32_t)(buf * ACC_COLS + half * 2 * BN + c), rm);
          cw_tmem_ld16(lane_addr + (uint32_t)(buf * ACC_COLS + half * 2 * BN + BN + c), rt);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j)
            acc[c + j] = __fadd_rn(acc[c + j], __fadd_rn(__uint_as_float(rm[j]), __uint_as_float(rt[j])));
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&acc_empty[buf]);
      }
      if (!ok) break;
      const int nt = (int)(tile % p.tiles_n);
      const long long st = tile / p.tiles_n;
      const int b = (int)(st / tiles_per_image);
      const int rem = (int)(st - (long long)b * tiles_per_image);
      const int th = rem / p.tiles_w, tw = rem - th * p.tiles_w;
      const int oh = th * CW_TILE + (m >> 3), ow = tw * CW_TILE + (m & 7) + 8 * half;
      // this column tile's biases, one copy per epilogue warp (lane l holds channels l and l + 32)
      const int n0 = nt * BN;
      if (has_bias) {
        __syncwarp();
#pragma unroll
        for (int j = lane; j < BN; j += 32) bias_s[warp - 2][j] = n0 + j < p.K ? bias_g[n0 + j] : 0.f;
        __syncwarp();
      }
      const float *bias_w = has_bias ? bias_s[warp - 2] : nullptr;
      if (p.pool2) {
        // Ho and Wo are even, so a pooling window lies wholly inside the image or wholly outside
        const int Hq = p.Ho >> 1, Wq = p.Wo >> 1;
        const long long plane = (long long)Hq * Wq;
        const bool inside = oh < p.Ho && ow < p.Wo;
        const long long pos = inside ? ((long long)b * Hq + (oh >> 1)) * Wq + (ow >> 1) : 0;
        float *yb = p.y ? p.y + ((long long)b * p.K + n0) * plane + (long long)(oh >> 1) * Wq + (ow >> 1) : nullptr;
        float *nh = p.y_hi ? p.y_hi + pos * p.K + n0 : nullptr, *nl = p.y_hi ? p.y_lo + pos * p.K + n0 : nullptr;
        // the short way (the window's four lanes share the channels out); the long way for warps that
        // met a number that is not finite
        if (!store_channels_pool4<BN>(acc, yb, plane, p.K - n0, bias_w, p.ep.act, (float)p.ep.alpha, inside, nh, nl)) {
          const bool writer = inside && (lane & 9) == 0;
          if (p.y_hi)
            store_channels_split<BN, true>(acc, yb, plane, p.K - n0, bias_w, p.ep.act, (float)p.ep.alpha, writer, nh, nl);
          else
            store_channels_pooled<BN>(acc, yb, plane, p.K - n0, bias_w, p.ep.act, (float)p.ep.alpha, writer);
        }
      } else if (p.y_hi) {
        const long long plane = (long long)p.Ho * p.Wo;
        const bool writer = oh < p.Ho && ow < p.Wo;
        const long long pos = writer ? ((long long)b * p.Ho + oh) * p.Wo + ow : 0;
        float *yb = p.y ? p.y + ((long long)b * p.K + n0) * plane + (long long)oh * p.Wo + ow : nullptr;
        store_channels_split<BN, false>(acc, yb, plane, p.K - n0, bias_w, p.ep.act, (float)p.ep.alpha, writer,
                                        p.y_hi + pos * p.K + n0, p.y_lo + pos * p.K + n0);
      } else if (oh < p.Ho && ow < p.Wo) {
        const long long plane = (long long)p.Ho * p.Wo;
        float *yb = p.y + ((long long)b * p.K + n0) * plane + (long long)oh * p.Wo + ow;
        store_channels<BN>(acc, yb, plane, p.K - n0, bias_w, p.ep.act, (float)p.ep.alpha);
      }
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

typedef CUresult (*CwEncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static CwEncodeTiledFn cw_encode_fn() {
  void *sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
      q == cudaDriverEntryPointSuccess)
    return (CwEncodeTiledFn)sym;
  return nullptr;
}

static size_t cw_smem_budget(const b200_engine *e) { return std::min<size_t>(e->smem_optin, 227 * 1024) - 4096; }

static void cw_geometry(int C, int K, int kh, int kw, int dH, int dW, int *ck, int *bn, int *win_w, int *win_h,
                        int *win_bytes) {
  *ck = C % 32 == 0 ? 32 : 16;
  *bn = K <= 32 ? 32 : 64;
  *win_w = CW_TILE + (kw - 1) * dW;
  *win_h = CW_TILE + (kh - 1) * dH;
  *win_bytes = ((*win_w) * (*win_h) * (*ck) * 4 + 1023) / 1024 * 1024;
}

// Whether the window kernel takes a convolution: stride 1, channels 16 or a multiple of 32 (and
// few enough that the re-reads of the im2col path, not the tensor core, are what bounds it), a
// window that fits twice into shared memory beside three filter slabs, output planes that 16 x 16
// tiles cover without much waste, and coordinates a tensor map can hold.
bool conv_win_eligible(const b200_engine *e, long long B, int C, int H, int W, int K, int kh, int kw, int padH,
                       int padW, int sH, int sW, int dH, int dW, int Ho, int Wo) {
  if (sH != 1 || sW != 1) return false;
  if (!(C == 16 || (C % 32 == 0 && C <= 64))) return false;
  if (kh * kw == 1) return false;
  if (B >= (1LL << 31) || B * C * H * W * 4 < 131072) return false;
  int ck, bn, win_w, win_h, win_bytes;
  cw_geometry(C, K, kh, kw, dH, dW, &ck, &bn, &win_w, &win_h, &win_bytes);
  if (win_w > 256 || win_h > 256) return false;
  const size_t need = (size_t)CW_WIN_STAGES * 2 * win_bytes + 3 * (size_t)(2 * bn * ck * 4) + 1024;
  if (need > cw_smem_budget(e)) return false;
  const long long th = (Ho + CW_TILE - 1) / CW_TILE, tw = (Wo + CW_TILE - 1) / CW_TILE;
  if ((double)Ho * Wo < 0.7 * (double)(th * tw * CW_TILE * CW_TILE)) return false;
  (void)padH;
  (void)padW;
  return true;
}

template <int BN, int CK>
static int launch_conv_win(b200_engine *e, const CUtensorMap *tm, ConvWinParams &p) {
  constexpr int B_STAGE_BYTES = 2 * BN * CK * 4;
  auto kern = conv_win_kernel<BN, CK>;
  static std::atomic<int> attr_dev_mask{0};  // devices on which the attribute is set; engines on other threads share it
  const size_t optin = std::min<size_t>(e->smem_optin, 227 * 1024);
  if (!(attr_dev_mask & (1 << (e->device & 31)))) {
    cudaFuncAttributes fa;
    B200_CHECK_CUDA(e, cudaFuncGetAttributes(&fa, kern));
    B200_CHECK_CUDA(e, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)(optin - fa.sharedSizeBytes)));
    attr_dev_mask |= 1 << (e->device & 31);
  }
  const size_t win_total = (size_t)CW_WIN_STAGES * 2 * p.win_bytes;
  p.b_stages = (int)std::max<size_t>(
      2, std::min<size_t>(CW_MAX_BSTAGES, (cw_smem_budget(e) - 1024 - win_total) / B_STAGE_BYTES));
  const size_t smem = win_total + (size_t)p.b_stages * B_STAGE_BYTES + 1024;
  const int grid = (int)std::min<long long>(p.total_tiles, e->sm_count);
  kern<<<grid, CW_THREADS, smem, e->stream>>>(tm[0], tm[1], tm[2], tm[3], p);
  B200_CHECK_LAUNCH(e, "conv_win_kernel");
  e->flags_dirty = true;
  return B200_OK;
}

// x (B,C,H,W) * w (K,C,kh,kw) -> y (B,K,Ho,Wo), float32, stride 1. ep.bias_kind ROW = per channel.
// pool2 (Ho, Wo even): y is (B,K,Ho/2,Wo/2), the 2x2 / stride-2 max-pool of the activated output.
// x_hi / x_lo: the input already in NHWC TF32 head / tail form (x is then unused). y_hi / y_lo: the
// (pooled) output additionally in that form, K a multiple of 4; y may then be null.
int conv2d_win(b200_engine *e, const float *x, const float *w, float *y, long long B, int C, int H, int W, int K,
               int kh, int kw, int padH, int padW, int dH, int dW, int Ho, int Wo, const Epilogue &ep, bool pool2,
               const float *x_hi, const float *x_lo, float *y_hi, float *y_lo) {
  static CwEncodeTiledFn enc = cw_encode_fn();
  if (!enc) return set_error(e, B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const int taps = kh * kw, crs = C * taps;
  int ck, bn, win_w, win_h, win_bytes;
  cw_geometry(C, K, kh, kw, dH, dW, &ck, &bn, &win_w, &win_h, &win_bytes);
  const CUtensorMapSwizzle swz = ck == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;

  TcOperand wf;
  void *wblk[2] = {nullptr, nullptr};
  int rc = conv_filters_tap_major(e, w, K, C, taps, &wf, wblk);
  if (rc != B200_OK) return rc;
  void *xs[2] = {nullptr, nullptr};
  const void *xin[2] = {x_hi, x_lo};  // the caller's pre-split input, or this call's own rewrite
  if (!x_hi) {
    rc = conv_nhwc_split(e, x, B, C, H * W, xs);
    xin[0] = xs[0];
    xin[1] = xs[1];
  }

  ConvWinParams p = ConvWinParams();
  p.y = y;
  p.y_hi = y_hi;
  p.y_lo = y_lo;
  p.K = K; p.Ho = Ho; p.Wo = Wo;
  p.kh = kh; p.kw = kw; p.dH = dH; p.dW = dW; p.padH = padH; p.padW = padW;
  p.win_w = win_w;
  p.win_bytes = win_bytes;
  p.cblocks = C / ck;
  p.C = C;
  p.chunk_k = 256 / ck;
  p.tiles_h = (Ho + CW_TILE - 1) / CW_TILE;
  p.tiles_w = (Wo + CW_TILE - 1) / CW_TILE;
  p.tiles_n = (K + bn - 1) / bn;
  p.total_tiles = B * p.tiles_h * p.tiles_w * p.tiles_n;
  p.ep = ep;
  p.pool2 = pool2 ? 1 : 0;
  p.err_flag = e->d_flags + 2;

  CUtensorMap tm[4];
  memset((void *)tm, 0, sizeof tm);
  if (rc == B200_OK) {
    // activations as (C, W, H, N), box = CK channels x window; positions outside the image read as zero
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)C * 4, (cuuint64_t)W * C * 4, (cuuint64_t)H * W * C * 4};
    cuuint32_t box[4] = {(cuuint32_t)ck, (cuuint32_t)win_w, (cuuint32_t)win_h, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    for (int h = 0; h < 2 && rc == B200_OK; ++h) {
      CUresult r = enc(&tm[h], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void *>(xin[h]), dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS)
        rc = set_error(e, B200_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for a %d x %d window", (int)r, win_w,
                       win_h);
    }
    cuuint64_t wdims[3] = {(cuuint64_t)crs, (cuuint64_t)K, 1};
    cuuint64_t wstrides[2] = {(cuuint64_t)wf.ld * 4, (cuuint64_t)K * wf.ld * 4};
    cuuint32_t wbox[3] = {(cuuint32_t)ck, (cuuint32_t)bn, 1};
    cuuint32_t westr[3] = {1, 1, 1};
    for (int h = 0; h < 2 && rc == B200_OK; ++h) {
      CUresult r = enc(&tm[2 + h], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(h ? wf.p1 : wf.p0), wdims,
                       wstrides, wbox, westr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) rc = set_error(e, B200_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for filters", (int)r);
    }
  }
  if (rc == B200_OK) {
    if (ck == 32) {
      if (bn == 64) rc = launch_conv_win<64, 32>(e, tm, p);
      else rc = launch_conv_win<32, 32>(e, tm, p);
    } else {
      if (bn == 64) rc = launch_conv_win<64, 16>(e, tm, p);
      else rc = launch_conv_win<32, 16>(e, tm, p);
    }
  }
  for (int h = 0; h < 2; ++h) {
    if (xs[h]) b200_put(e, xs[h], 0);
    if (wblk[h]) b200_put(e, wblk[h], 0);
  }
  return rc;
}

}  // namespace b200
