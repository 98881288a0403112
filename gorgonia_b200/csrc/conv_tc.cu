// Implicit-GEMM 2-D convolution on the tensor cores (float32 as 3xTF32).
//
//   y[b][k][p] = sum_q  col[(b,p)][q] * Wf[k][q],    q = (c, r, s) in the order of gorgonia's im2col
//                                                     (op_nn.go:418-441), p = oh*Wo + ow
//
// The col matrix is never written to memory. Mapping onto tcgen05:
//   M (128 TMEM lanes)  = pixels (b, p), flattened over the whole batch, so tiles are full whatever
//                         the image size; a lane <-> pixel mapping also makes the NCHW store of one
//                         output channel a run of consecutive addresses across a warp;
//   N (BN columns)      = output channels, BN = 32..128;
//   K                   = q, in blocks of 32 (one 128-byte swizzle row of float32).
// A operand: eight gather warps build each 128 x 32 slab of col directly in shared memory, in the
// K-major 128-byte-swizzle layout the tensor core reads, already split into TF32 head and tail.
// Two threads share a tile row (one pixel), 16 q each; for a fixed q the 32 lanes of a warp read
// consecutive input pixels, so the gather is coalesced and x is re-read from L1/L2, not HBM. The
// (c, r, s) decomposition of q is the same for every lane: 16 lanes compute one entry each per
// k-block and the warp shares them by shuffle. Loads of the next k-block are issued before the
// current one is converted and stored, so their latency overlaps the conversion.
// B operand: the filters, split once into head/tail (K x C*kh*kw row-major is already K-major),
// loaded by TMA.
// Accumulation, as in the matrix multiply: hi*hi in one TMEM accumulator, the two cross terms in
// a second one, chains cut every 8 k-blocks and folded into fp32 registers by the epilogue warps
// (the tensor core's adder truncates; see gemm_tc.cu). Eight epilogue warps: two per TMEM lane
// quarter, each folding half of the BN columns, which keeps them at 64 accumulator registers.
//
// Warp roles (18 warps): 0 TMA (filters), 1 MMA issuer + TMEM owner, 2-9 epilogue, 10-17 gather.
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

int split_operand_tf32(b200_engine *e, const float *src, long long rows, long long cols, long long ld,
                       long long batch, long long batch_stride, TcOperand *out, void **blk_hi, void **blk_lo);

constexpr int CV_BM = 128;
constexpr int CV_BK = 32;                 // q per stage: one 128-byte row of float32
constexpr int CV_THREADS = 576;           // 18 warps
constexpr int CV_GATHER_WARP0 = 10;
constexpr int CV_GATHER_THREADS = 256;    // two threads per tile row, 16 q each
constexpr int CV_A_BYTES = CV_BM * 128;   // one copy (head or tail) of the A slab

struct ConvTcParams {
  const float *x;
  float *y;
  long long Mtot;  // B * Ho * Wo
  int C, H, W, K, Ho, Wo, hw;
  int kh, kw, padH, padW, sH, sW, dH, dW;
  int crs;         // C * kh * kw
  int num_k;       // k-blocks of 32
  int chunk_k;     // k-blocks per accumulation chain
  int tiles_m, tiles_n;
  int stages;
  Epilogue ep;     // bias_kind ROW = per output channel
  const float *zero;  // one word of device memory that always holds 0.0f
  int *err_flag;
};

__device__ __forceinline__ float cv_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}
__device__ __forceinline__ void cv_sts128(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
// 32 lanes x 16 columns of 32-bit accumulators
__device__ __forceinline__ void cv_tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// MODE 0: general. MODE 1 ("fast"): at most 32 taps per channel (kh*kw <= 32) and fewer than 2^31
// input elements in total, which lets the gather run on 32-bit indices and a per-pixel tap mask.
// MODE 2 ("tap-major"): additionally C is a multiple of 16; the reduction index is reordered to
// q' = (tap, channel) (the filters are permuted to match when they are split), so the 16 elements
// a gather thread owns in a k-block are ONE tap and 16 consecutive channels: one bounds decision
// and a constant stride instead of a (c, r, s) decomposition per element. Reordering a sum changes
// its rounding, not its value; the result stays within the matrix-multiply tolerance.
template <int BN, int MODE>
__global__ void __launch_bounds__(CV_THREADS, 1)
    conv_tc_kernel(const __grid_constant__ CUtensorMap tmW0, const __grid_constant__ CUtensorMap tmW1,
                   const __grid_constant__ ConvTcParams p) {
  constexpr int B_BYTES = BN * 128;
  constexpr int STAGE_BYTES = 2 * (CV_A_BYTES + B_BYTES);
  constexpr uint32_t IDESC = make_idesc(2, 0, 0, CV_BM, BN);
  // head x [filter head | filter tail] as ONE instruction of width 2*BN: the tail slab follows the
  // head slab in shared memory, the cross-term accumulator follows the main one in tensor memory
  constexpr uint32_t IDESC_WIDE = make_idesc(2, 0, 0, CV_BM, 2 * BN);
  constexpr int ACC_COLS = 2 * BN;          // main + cross-term accumulator
  constexpr int TMEM_COLS = 2 * ACC_COLS;   // double-buffered; power of two >= 128 for BN >= 32
  constexpr int HALF = BN / 2;              // columns folded by one epilogue warp
  constexpr int MAX_STAGES = 6;

  extern __shared__ __align__(1024) unsigned char cv_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_fail;
  __shared__ float bias_s[8][BN / 2];

  unsigned char *smem = reinterpret_cast<unsigned char *>(((uintptr_t)cv_smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages;
  const long long total_tiles = (long long)p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(&full_bar[s], CV_GATHER_THREADS + 1);  // gather threads + the TMA thread's expect_tx arrival
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&acc_full[b], 1);
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
    ptx::prefetch_tmap(&tmW0);
    ptx::prefetch_tmap(&tmW1);
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    // ---------------- TMA: filter slabs ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int nt = (int)(tile % p.tiles_n);
        for (int kb = 0; kb < p.num_k; ++kb) {
          if (!ptx::mbar_wait_relaxed(&empty_bar[stage], phase ^ 1, 64)) {
            ok = false;
            break;
          }
          unsigned char *sb = smem + (size_t)stage * STAGE_BYTES + 2 * CV_A_BYTES;
          ptx::mbar_arrive_expect_tx(&full_bar[stage], 2 * B_BYTES);
          ptx::tma_load_3d(sb, &tmW0, kb * CV_BK, nt * BN, 0, &full_bar[stage]);
          ptx::tma_load_3d(sb + B_BYTES, &tmW1, kb * CV_BK, nt * BN, 0, &full_bar[stage]);
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
      for (long long tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        for (int kc = 0; kc < p.num_k && ok; kc += p.chunk_k, ++use) {
          const int buf = use & 1;
          const uint32_t acc_phase = (uint32_t)((use >> 1) & 1);
          if (!ptx::mbar_wait(&acc_empty[buf], acc_phase ^ 1)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t d_main = tmem_base + (uint32_t)(buf * ACC_COLS);
          const uint32_t d_tail = d_main + BN;
          const int kend = kc + p.chunk_k < p.num_k ? kc + p.chunk_k : p.num_k;
          for (int kb = kc; kb < kend; ++kb) {
            if (!ptx::mbar_wait(&full_bar[stage], phase)) {
              ok = false;
              break;
            }
            ptx::tc_fence_after_sync();
            const uint32_t st = ptx::smem_addr(smem + (size_t)stage * STAGE_BYTES);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint64_t a_hi = make_smem_desc(st + kk * 32, 16, 1024, 2);
              const uint64_t a_lo = make_smem_desc(st + CV_A_BYTES + kk * 32, 16, 1024, 2);
              const uint64_t b_hi = make_smem_desc(st + 2 * CV_A_BYTES + kk * 32, 16, 1024, 2);
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
  } else if (warp < CV_GATHER_WARP0) {
    // ---------------- epilogue: warps 2..9 ----------------
    const int quarter = warp & 3;           // TMEM lanes 32*quarter .. +31
    const int half = (warp - 2) >> 2;       // which half of the BN columns
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const bool has_bias = p.ep.bias_kind != B200_BIAS_NONE;
    const float *bias_g = reinterpret_cast<const float *>(p.ep.bias);
    int use = 0;
    bool ok = true;
    for (long long tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int mt = (int)(tile / p.tiles_n), nt = (int)(tile % p.tiles_n);
      float acc[HALF];
#pragma unroll
      for (int j = 0; j < HALF; ++j) acc[j] = 0.f;
      for (int kc = 0; kc < p.num_k && ok; kc += p.chunk_k) {
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
          cv_tmem_ld16(lane_addr + (uint32_t)(buf * ACC_COLS + half * HALF + c), rm);
          cv_tmem_ld16(lane_addr + (uint32_t)(buf * ACC_COLS + BN + half * HALF + c), rt);
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
      const long long m = (long long)mt * CV_BM + quarter * 32 + lane;
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
        yb = p.y + (b * p.K + n0) * (long long)p.hw + pix;
      }
      // this warp's biases, staged once per tile (lane l holds channels l and l + 32)
      if (has_bias) {
        __syncwarp();
#pragma unroll
        for (int j = lane; j < HALF; j += 32) bias_s[warp - 2][j] = n0 + j < p.K ? bias_g[n0 + j] : 0.f;
        __syncwarp();
      }
      if (yb)
        store_channels<HALF>(acc, yb, p.hw, p.K - n0, has_bias ? bias_s[warp - 2] : nullptr, p.ep.act,
                             (float)p.ep.alpha);
    }
    if (!ok) s_fail = 1;
  } else {
    // ---------------- gather: warps 10..17 ----------------
    // thread g: tile row (g & 127), q-half (g >> 7): the 16 q's [16*half, 16*half + 16) of each block
    const int g = threadIdx.x - CV_GATHER_WARP0 * 32;
    const int t = g & 127, qhalf = g >> 7;
    const int khw = p.kh * p.kw;
    const long long n_blocks = (blockIdx.x < total_tiles ? (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0) *
                               (long long)p.num_k;

    // per-tile pixel state of this thread
    bool live = false;
    int ih0 = 0, iw0 = 0;
    const float *xpix = p.x;  // x + image base + ih0*W + iw0 (may point before the image; only
                              // dereferenced together with offsets that land inside it)
    int pix_idx = 0;          // modes 1, 2: the same position as an index into x
    uint32_t tap_mask = 0;    // modes 1, 2: bit (r*kw + s) set iff that tap of this pixel lies inside the image
    auto set_tile = [&](long long tile) {
      const int mt = (int)(tile / p.tiles_n);
      const long long m = (long long)mt * CV_BM + t;
      live = m < p.Mtot;
      long long b = 0;
      int pix = 0;
      if (live) {
        if (p.Mtot < (1LL << 31)) {
          const uint32_t mu = (uint32_t)m, bu = mu / (uint32_t)p.hw;
          b = bu;
          pix = (int)(mu - bu * (uint32_t)p.hw);
        } else {
          b = m / p.hw;
          pix = (int)(m % p.hw);
        }
      }
      const int oh = pix / p.Wo, ow = pix - oh * p.Wo;
      ih0 = oh * p.sH - p.padH;
      iw0 = ow * p.sW - p.padW;
      if (MODE >= 1) {
        pix_idx = (int)(b * (long long)p.C * p.H * p.W) + ih0 * p.W + iw0;
        tap_mask = 0;
        if (live)
          for (int r = 0; r < p.kh; ++r)
            for (int sx = 0; sx < p.kw; ++sx) {
              const int ih = ih0 + r * p.dH, iw = iw0 + sx * p.dW;
              if ((unsigned)ih < (unsigned)p.H && (unsigned)iw < (unsigned)p.W) tap_mask |= 1u << (r * p.kw + sx);
            }
      } else {
        xpix = p.x + b * (long long)p.C * p.H * p.W + (long long)ih0 * p.W + iw0;
      }
    };
    // Issues the loads of the 16 values of block kb for this thread. A tap outside the image (or a
    // q past the end of the filter) is read from p.zero, a word that always holds 0.0f, so every
    // load is valid and nothing has to look at the loaded values here: an instruction that
    // consumed a load at this point would make the warp wait for it and undo the prefetch.
    int m2_tap = 0, m2_c0 = 0, m2_r = 0, m2_sx = 0;  // MODE 2: tap / first channel of the next block
    auto load_block = [&](int kb, float(&v)[16]) {
      if (MODE == 2) {
        // q' = 32*kb + 16*qhalf + j = tap*C + channel; C % 16 == 0, so the 16 share one tap
        if (kb == 0) {
          m2_tap = (qhalf * 16) / p.C;
          m2_c0 = qhalf * 16 - m2_tap * p.C;
          m2_r = m2_tap / p.kw;
          m2_sx = m2_tap - m2_r * p.kw;
        }
        const bool in = m2_tap < khw && ((tap_mask >> (m2_tap & 31)) & 1u) != 0;
        const int idx = pix_idx + ((m2_c0 * p.H) + m2_r * p.dH) * p.W + m2_sx * p.dW;
        const float *base = in ? p.x + idx : p.zero;
        const int step = in ? p.H * p.W : 0;
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = __ldg(base + (long long)j * step);
        // step to the next block: 32 channels further, wrapping into the next tap(s)
        m2_c0 += CV_BK;
        while (m2_c0 >= p.C) {
          m2_c0 -= p.C;
          ++m2_tap;
          if (++m2_sx == p.kw) {
            m2_sx = 0;
            ++m2_r;
          }
        }
        return;
      }
      // lane j < 16 decomposes q = 32*kb + 16*qhalf + j once for the whole warp
      const int q = kb * CV_BK + qhalf * 16 + (lane & 15);
      const int c = q / khw, rs = q - c * khw;
      const int r = rs / p.kw, sx = rs - r * p.kw;
      const int my_off = (c * p.H + r * p.dH) * p.W + sx * p.dW;
      if (MODE == 1) {
        const int my_bit = q < p.crs ? rs : 32;  // 32 = no tap: a q past the end of the filter
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int off = __shfl_sync(0xffffffffu, my_off, j);
          const int bit = __shfl_sync(0xffffffffu, my_bit, j);
          const bool in = bit < 32 && ((tap_mask >> (bit & 31)) & 1u) != 0;
          v[j] = __ldg(in ? p.x + (pix_idx + off) : p.zero);
        }
      } else {
        const int my_rs = q < p.crs ? ((r * p.dH) << 16) | (sx * p.dW) : 0x40004000;  // out of any image
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int off = __shfl_sync(0xffffffffu, my_off, j);
          const int drs = __shfl_sync(0xffffffffu, my_rs, j);
          const int ih = ih0 + (drs >> 16), iw = iw0 + (drs & 0xffff);
          const bool in = live && (unsigned)ih < (unsigned)p.H && (unsigned)iw < (unsigned)p.W;
          v[j] = __ldg(in ? xpix + off : p.zero);
        }
      }
    };

    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    // Load cursor: runs two k-blocks ahead of the block being converted, so that two blocks of
    // loads (32 KB per CTA) are in flight while a third is converted and stored. Bytes in flight
    // over the L2 latency is what bounds the gather.
    long long ltile = blockIdx.x, issued = 0;
    int lkb = 0;
    auto issue_next = [&](float(&dst)[16]) {
      if (issued >= n_blocks) return;
      if (lkb == 0) set_tile(ltile);
      load_block(lkb, dst);
      if (++lkb == p.num_k) {
        lkb = 0;
        ltile += gridDim.x;
      }
      ++issued;
    };
    // waits for the ring slot, converts one block to TF32 head/tail and publishes it
    auto convert_store = [&](const float(&v)[16]) -> bool {
      if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1)) return false;
      const uint32_t row_hi = ptx::smem_addr(smem + (size_t)stage * STAGE_BYTES) + (uint32_t)t * 128;
      const uint32_t row_lo = row_hi + CV_A_BYTES;
      const uint32_t sw = (uint32_t)(t & 7);
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        float h[4], l[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          h[j] = cv_tf32(v[ch * 4 + j]);
          l[j] = cv_tf32(__fsub_rn(v[ch * 4 + j], h[j]));
        }
        // 128-byte swizzle: 16-byte chunk index XOR (row mod 8)
        const uint32_t off = ((uint32_t)(qhalf * 4 + ch) ^ sw) * 16;
        cv_sts128(row_hi + off, h[0], h[1], h[2], h[3]);
        cv_sts128(row_lo + off, l[0], l[1], l[2], l[3]);
      }
      ptx::fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core
      ptx::mbar_arrive(&full_bar[stage]);
      if (++stage == stages) {
        stage = 0;
        phase ^= 1;
      }
      return true;
    };
    // three register buffers in rotation, spelled out so that every index is static
    float va[16], vb[16], vc[16];
    issue_next(va);
    issue_next(vb);
    long long it = 0;
    while (it < n_blocks) {
      issue_next(vc);
      if (!(ok = convert_store(va))) break;
      if (++it >= n_blocks) break;
      issue_next(va);
      if (!(ok = convert_store(vb))) break;
      if (++it >= n_blocks) break;
      issue_next(vb);
      if (!(ok = convert_store(vc))) break;
      ++it;
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

// w (K, C, taps) -> head/tail (K, taps, C): out[k][tap*C + c] = split(w[k][c*taps + tap])
__global__ void __launch_bounds__(256) split_permute_filters_kernel(const float *__restrict__ w, float *__restrict__ hi,
                                                                    float *__restrict__ lo, int K, int C, int taps) {
  const long long total = (long long)K * C * taps;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int c = (int)(t % C);
    const int tap = (int)((t / C) % taps);
    const long long k = t / ((long long)C * taps);
    const float v = w[(k * C + c) * taps + tap];
    const float h = cv_tf32(v);
    hi[t] = h;
    lo[t] = cv_tf32(__fsub_rn(v, h));
  }
}

// Filters (K, C, taps) split into TF32 head/tail AND reordered to (tap, channel) along the
// reduction index. blk[] receives the arena blocks the caller must release, or nulls when the
// result came from (or went into) the cache of a buffer declared constant.
int conv_filters_tap_major(b200_engine *e, const float *w, int K, int C, int taps, TcOperand *wf, void **blk) {
  const int crs = C * taps;
  blk[0] = blk[1] = nullptr;
  wf->ld = crs;
  if (CachedSplit *cached = find_cached(e, w, 1, K, C, taps, crs)) {
    wf->p0 = cached->hi;
    wf->p1 = cached->lo;
    return B200_OK;
  }
  int rc = b200_get(e, (long long)K * crs * 4, &blk[0]);
  if (rc == B200_OK) rc = b200_get(e, (long long)K * crs * 4, &blk[1]);
  if (rc != B200_OK) {
    if (blk[0]) b200_put(e, blk[0], 0);
    blk[0] = nullptr;
    return rc;
  }
  const long long total = (long long)K * crs;
  const int blocks = (int)std::max<long long>(1, std::min<long long>((total + 255) / 256, e->sm_count * 16LL));
  split_permute_filters_kernel<<<blocks, 256, 0, e->stream>>>(w, (float *)blk[0], (float *)blk[1], K, C, taps);
  B200_CHECK_LAUNCH(e, "split_permute_filters_kernel");
  wf->p0 = blk[0];
  wf->p1 = blk[1];
  if (is_constant(e, w)) {  // filters declared constant: keep the permuted split for the next call
    add_cached(e, w, CachedSplit{1, K, C, taps, crs, blk[0], blk[1], crs});
    blk[0] = blk[1] = nullptr;
  }
  return B200_OK;
}

template <int BN, int MODE>
static int launch_conv_tc(b200_engine *e, const CUtensorMap *tm, ConvTcParams &p) {
  constexpr int STAGE_BYTES = 2 * (CV_A_BYTES + BN * 128);
  auto kern = conv_tc_kernel<BN, MODE>;
  static std::atomic<int> attr_dev_mask{0};  // devices on which the attribute is set; engines on other threads share it
  const size_t optin = std::min<size_t>(e->smem_optin, 227 * 1024);
  if (!(attr_dev_mask & (1 << (e->device & 31)))) {
    cudaFuncAttributes fa;
    B200_CHECK_CUDA(e, cudaFuncGetAttributes(&fa, kern));
    B200_CHECK_CUDA(e, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)(optin - fa.sharedSizeBytes)));
    attr_dev_mask |= 1 << (e->device & 31);
  }
  p.stages = (int)std::max<size_t>(2, std::min<size_t>(6, (optin - 4096) / STAGE_BYTES));
  const size_t smem = (size_t)p.stages * STAGE_BYTES + 1024;
  const long long tiles = (long long)p.tiles_m * p.tiles_n;
  const int grid = (int)std::min<long long>(tiles, e->sm_count);
  kern<<<grid, CV_THREADS, smem, e->stream>>>(tm[0], tm[1], p);
  B200_CHECK_LAUNCH(e, "conv_tc_kernel");
  e->flags_dirty = true;
  return B200_OK;
}

// x (B,C,H,W) * w (K,C,kh,kw) -> y (B,K,Ho,Wo), float32. ep.bias_kind ROW = one value per channel.
int conv2d_tc(b200_engine *e, const float *x, const float *w, float *y, long long B, int C, int H, int W, int K,
              int kh, int kw, int padH, int padW, int sH, int sW, int dH, int dW, int Ho, int Wo,
              const Epilogue &ep) {
  const int crs = C * kh * kw;
  const bool fast = kh * kw <= 32 && B * (long long)C * H * W < (1LL << 31);
  const int mode = !fast ? 0 : (C % 16 == 0 ? 2 : 1);
  TcOperand wf;
  void *blk[2] = {nullptr, nullptr};
  int rc;
  if (mode == 2)
    rc = conv_filters_tap_major(e, w, K, C, kh * kw, &wf, blk);
  else
    rc = split_operand_tf32(e, w, K, crs, crs, 1, 0, &wf, &blk[0], &blk[1]);
  if (rc != B200_OK) return rc;
  int bn = 128;
  while (bn > 32 && bn / 2 >= K) bn /= 2;
  ConvTcParams p = ConvTcParams();
  p.x = x;
  p.y = y;
  p.Mtot = B * Ho * Wo;
  p.C = C; p.H = H; p.W = W; p.K = K; p.Ho = Ho; p.Wo = Wo; p.hw = Ho * Wo;
  p.kh = kh; p.kw = kw; p.padH = padH; p.padW = padW; p.sH = sH; p.sW = sW; p.dH = dH; p.dW = dW;
  p.crs = crs;
  p.num_k = (crs + CV_BK - 1) / CV_BK;
  p.chunk_k = 8;
  p.tiles_m = (int)((p.Mtot + CV_BM - 1) / CV_BM);
  p.tiles_n = (K + bn - 1) / bn;
  p.ep = ep;
  // the kernel indexes the bias by output channel, which it passes as the "row" of the epilogue
  p.err_flag = e->d_flags + 2;
  p.zero = reinterpret_cast<const float *>(e->d_flags + 8);  // zeroed at engine creation, never written
  CUtensorMap tm[2];
  memset(tm, 0, sizeof tm);
  rc = encode_map(e, &tm[0], 4, wf.p0, crs, K, 1, wf.ld, (long long)K * wf.ld, CV_BK, bn, false);
  if (rc == B200_OK) rc = encode_map(e, &tm[1], 4, wf.p1, crs, K, 1, wf.ld, (long long)K * wf.ld, CV_BK, bn, false);
  if (rc == B200_OK) {
    if (mode == 2) {
      if (bn == 128) rc = launch_conv_tc<128, 2>(e, tm, p);
      else if (bn == 64) rc = launch_conv_tc<64, 2>(e, tm, p);
      else rc = launch_conv_tc<32, 2>(e, tm, p);
    } else if (mode == 1) {
      if (bn == 128) rc = launch_conv_tc<128, 1>(e, tm, p);
      else if (bn == 64) rc = launch_conv_tc<64, 1>(e, tm, p);
      else rc = launch_conv_tc<32, 1>(e, tm, p);
    } else {
      if (bn == 128) rc = launch_conv_tc<128, 0>(e, tm, p);
      else if (bn == 64) rc = launch_conv_tc<64, 0>(e, tm, p);
      else rc = launch_conv_tc<32, 0>(e, tm, p);
    }
  }
  if (blk[0]) b200_put(e, blk[0], 0);
  if (blk[1]) b200_put(e, blk[1], 0);
  return rc;
}

}  // namespace b200
