// The im2col-TMA convolution (conv_tma.cu) for launches with many tiles, run by PAIRS of CTAs that
// share their filter slabs (float32 as 3xTF32).
//
// What bounds conv_tma_kernel is the rate at which one SM takes bytes from L2: every k-block of a
// 128 x 128 tile brings 64 KB (col head/tail 32 KB, filter head/tail 32 KB) for 0.41 microseconds of
// tensor work, and 64 KB take an SM 0.5-0.6. Two tiles that differ only in their output positions
// read the SAME filter slab. Here two such tiles run on the two CTAs of a thread-block cluster: each
// CTA loads its own col slab and HALF of the filter slab (64 of the 128 filter rows) from L2 and
// copies that half into its peer's shared memory with a bulk copy over the SM-to-SM network
// (cp.async.bulk.shared::cluster.shared::cta: one source, one destination, no multicast; it
// completes on the peer's stage barrier like a TMA load). Per CTA and k-block 48 KB cross L2 instead
// of 64, which puts the load time under the tensor time. Everything else is conv_tma_kernel: the
// same MMAs into the same two accumulators, the same chains folded every 256 k by the same epilogue,
// so a tile's result is bit-identical to what that kernel computes.
//
// Stage protocol, per stage s and round r, symmetric in the two CTAs X and Y:
//   producer X:  wait empty_X[s] (X's MMAs of round r-1 have read the stage) -> arrive on free_Y[s]
//                (remote: "X's stage s can take round r") -> wait free_X[s] (Y said the same; by then
//                Y's MMAs of round r-1 are done, hence X's push of round r-1 has been read in full and
//                X's half can be overwritten) -> arm full_X[s] for 48 KB (col slab + the half Y will
//                push) and half_X[s] for 16 KB -> TMA loads: col slab on full_X[s], own filter half on
//                half_X[s].
//   forwarder X: wait half_X[s] -> bulk-copy X's filter half (head, tail) into the same place of Y's
//                stage s, completing on full_Y[s].
//   issuer X:    wait full_X[s] and half_X[s] -> MMAs -> commit empty_X[s].
// No CTA ever waits for something its peer can only do after waiting for it; every wait is bounded
// (the engine's error word is raised and all roles leave), and the two CTAs meet on the cluster
// barrier before they initialise and before they exit, so nothing is pushed into a CTA that is gone.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstring>

#include "engine.h"
#include "epilogue.cuh"
#include "ptx.cuh"
#include "tc_common.cuh"

namespace b200 {

constexpr int CP_BM = 128;
constexpr int CP_BN = 128;
constexpr int CP_CK = 32;
constexpr int CP_THREADS = 352;  // 11 warps: TMA, MMA, 8 epilogue, forwarder

struct ConvPairParams {
  float *y;               // NCHW output, or null when only the split form is wanted
  float *y_hi, *y_lo;     // the output as NHWC TF32 head / tail for the next convolution, or null
  long long Mtot;         // B * Ho * Wo
  int K, Wo, hw;
  int kw, padH, padW, sH, sW, dH, dW;
  int cblocks, num_k, chunk_k;
  int tiles_m, tiles_n, stages;
  Epilogue ep;            // bias_kind ROW = per output channel
  int *err_flag;
};

__device__ __forceinline__ void cp_tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(CP_THREADS, 1)
    conv_tma_pair_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                         const __grid_constant__ CUtensorMap tmW0, const __grid_constant__ CUtensorMap tmW1,
                         const __grid_constant__ ConvPairParams p) {
  constexpr int BN = CP_BN, CK = CP_CK;
  constexpr int ROW_BYTES = CK * 4;
  constexpr int A_BYTES = CP_BM * ROW_BYTES;      // 16 KB: one copy (head or tail) of the col slab
  constexpr int B_BYTES = BN * ROW_BYTES;         // 16 KB: one copy of the filter slab
  constexpr int HB_BYTES = B_BYTES / 2;           // the half of it one CTA loads from L2
  constexpr int STAGE_BYTES = 2 * (A_BYTES + B_BYTES);
  constexpr uint32_t SBO = 8 * ROW_BYTES;
  constexpr uint32_t LAYOUT = 2;                  // 128-byte swizzle
  constexpr int KK = CK / 8;
  constexpr uint32_t IDESC = make_idesc(2, 0, 0, CP_BM, BN);
  constexpr uint32_t IDESC_WIDE = make_idesc(2, 0, 0, CP_BM, 2 * BN);
  constexpr int ACC_COLS = 2 * BN;
  constexpr int TMEM_COLS = 2 * ACC_COLS;
  constexpr int HALF = BN / 2;
  constexpr int MAX_STAGES = 4;

  extern __shared__ __align__(1024) unsigned char cp_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES], half_bar[MAX_STAGES], empty_bar[MAX_STAGES],
      free_bar[MAX_STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_fail;
  __shared__ float bias_s[8][BN / 2];

  unsigned char *smem = reinterpret_cast<unsigned char *>(((uintptr_t)cp_smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages;
  const uint32_t rank = ptx::cluster_ctarank(), peer = rank ^ 1u;
  const int pairs = gridDim.x >> 1, pair = blockIdx.x >> 1;
  const long long pair_tiles = (long long)((p.tiles_m + 1) / 2) * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&half_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
      ptx::mbar_init(&free_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&acc_full[b], 1);
      ptx::mbar_init(&acc_empty[b], 8);
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
    ptx::prefetch_tmap(&tmW0);
    ptx::prefetch_tmap(&tmW1);
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::cluster_sync_all();  // both CTAs' barriers exist before either arrives on the other's
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;

  // this CTA's tile of pair-tile pt: the two CTAs take neighbouring position tiles of one column tile;
  // with an odd number of position tiles the last pair's second CTA repeats the first one's tile and
  // stores nothing
  auto my_tile = [&](long long pt, int &mt, int &nt, bool &real) {
    const int mtp = (int)(pt / p.tiles_n);
    nt = (int)(pt - (long long)mtp * p.tiles_n);
    mt = 2 * mtp + (int)rank;
    real = mt < p.tiles_m;
    if (!real) mt = p.tiles_m - 1;
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long pt = pair; pt < pair_tiles && ok; pt += pairs) {
        int mt, nt;
        bool real;
        my_tile(pt, mt, nt, real);
        const long long m0 = (long long)mt * CP_BM;
        const int n = (int)(m0 / p.hw);
        const int pix = (int)(m0 - (long long)n * p.hw);
        const int oh = pix / p.Wo, ow = pix - oh * p.Wo;
        const int w0 = ow * p.sW - p.padW, h0 = oh * p.sH - p.padH;
        int cb = 0, r = 0, sx = 0;
        for (int kb = 0; kb < p.num_k; ++kb) {
          if (!ptx::mbar_wait_relaxed(&empty_bar[stage], phase ^ 1, 32)) {
            ok = false;
            break;
          }
          ptx::mbar_arrive_cluster(ptx::mapa(ptx::smem_addr(&free_bar[stage]), peer));
          if (!ptx::mbar_wait_relaxed(&free_bar[stage], phase, 32)) {
            ok = false;
            break;
          }
          unsigned char *sa = smem + (size_t)stage * STAGE_BYTES;
          unsigned char *sb = sa + 2 * A_BYTES;
          ptx::mbar_arrive_expect_tx(&full_bar[stage], 2 * A_BYTES + 2 * HB_BYTES);
          ptx::mbar_arrive_expect_tx(&half_bar[stage], 2 * HB_BYTES);
          const uint16_t off_w = (uint16_t)(sx * p.dW), off_h = (uint16_t)(r * p.dH);
          ptx::tma_load_im2col_4d(sa, &tmA0, cb * CK, w0, h0, n, off_w, off_h, &full_bar[stage]);
          ptx::tma_load_im2col_4d(sa + A_BYTES, &tmA1, cb * CK, w0, h0, n, off_w, off_h, &full_bar[stage]);
          const int wrow = nt * BN + (int)rank * (BN / 2);
          ptx::tma_load_3d(sb + rank * HB_BYTES, &tmW0, kb * CK, wrow, 0, &half_bar[stage]);
          ptx::tma_load_3d(sb + B_BYTES + rank * HB_BYTES, &tmW1, kb * CK, wrow, 0, &half_bar[stage]);
          if (++cb == p.cblocks) {
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
  } else if (warp == 10) {
    // ---------------- forwarder: this CTA's filter half goes to the peer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long pt = pair; pt < pair_tiles && ok; pt += pairs) {
        for (int kb = 0; kb < p.num_k; ++kb) {
          if (!ptx::mbar_wait_relaxed(&half_bar[stage], phase, 32)) {
            ok = false;
            break;
          }
          unsigned char *sb = smem + (size_t)stage * STAGE_BYTES + 2 * A_BYTES;
          const unsigned char *src_hi = sb + rank * HB_BYTES, *src_lo = sb + B_BYTES + rank * HB_BYTES;
          const uint32_t bar = ptx::mapa(ptx::smem_addr(&full_bar[stage]), peer);
          ptx::bulk_s2peer(ptx::mapa(ptx::smem_addr(src_hi), peer), src_hi, HB_BYTES, bar);
          ptx::bulk_s2peer(ptx::mapa(ptx::smem_addr(src_lo), peer), src_lo, HB_BYTES, bar);
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
      for (long long pt = pair; pt < pair_tiles && ok; pt += pairs) {
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
            if (!ptx::mbar_wait(&full_bar[stage], phase) || !ptx::mbar_wait(&half_bar[stage], phase)) {
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
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const bool has_bias = p.ep.bias_kind != B200_BIAS_NONE;
    const float *bias_g = reinterpret_cast<const float *>(p.ep.bias);
    int use = 0;
    bool ok = true;
    for (long long pt = pair; pt < pair_tiles && ok; pt += pairs) {
      int mt, nt;
      bool real;
      my_tile(pt, mt, nt, real);
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
          cp_tmem_ld16(lane_addr + (uint32_t)(buf * ACC_COLS + half * HALF + c), rm);
          cp_tmem_ld16(lane_addr + (uint32_t)(buf * ACC_COLS + BN + half * HALF + c), rt);
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
      if (!real) continue;  // the repeated tile of an odd tail
      const long long m = (long long)mt * CP_BM + quarter * 32 + lane;
      const int n0 = nt * BN + half * HALF;
      float *yb = nullptr;
      if (m < p.Mtot) {
        long long b;
        int pix;
        if (p.Mtot < (1LL << 31)) {
          const uint32_t mu = (uint32_t)m, bu = mu / (uint32_t)p.hw;
          b = bu;
          pix = (int)(mu - bu * (uint32_t)p.hw);
        } else {
          b = m / p.hw;
          pix = (int)(m % p.hw);
        }
        yb = p.y ? p.y + (b * p.K + n0) * (long long)p.hw + pix : nullptr;
      }
      if (has_bias) {
        __syncwarp();
#pragma unroll
        for (int j = lane; j < HALF; j += 32) bias_s[warp - 2][j] = n0 + j < p.K ? bias_g[n0 + j] : 0.f;
        __syncwarp();
      }
      if (p.y_hi)
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
  ptx::cluster_sync_all();  // nobody leaves while its peer may still push to it or arrive on its barriers
}

// Whether a convolution of tiles_m x tiles_n tiles of 128 x 128 runs on CTA pairs: enough pair-tiles
// to fill the pairs the GPU can hold at least twice, otherwise whole tiles (or shared k ranges) win.
bool conv_pair_pays(const b200_engine *e, int K, long long tiles_m, long long tiles_n) {
  if (K <= 64) return false;  // the column tile is narrower than 128: conv_tma_kernel
  const long long pair_tiles = (tiles_m + 1) / 2 * tiles_n;
  return pair_tiles >= 2LL * (e->sm_count / 2);
}

// tm[0..1]: im2col maps of the input head / tail; tm[2..3]: filter head / tail maps with a box of
// 32 channels x 64 filter rows.
int launch_conv_tma_pair(b200_engine *e, const CUtensorMap *tm, ConvPairParams &p) {
  constexpr int STAGE_BYTES = 2 * (CP_BM + CP_BN) * CP_CK * 4;
  static std::atomic<int> attr_dev_mask{0};
  static std::atomic<int> max_clusters[32];
  const size_t optin = std::min<size_t>(e->smem_optin, 227 * 1024);
  p.stages = (int)std::max<size_t>(2, std::min<size_t>(4, (optin - 4096) / STAGE_BYTES));
  const size_t smem = (size_t)p.stages * STAGE_BYTES + 1024;
  const int dev_bit = 1 << (e->device & 31);
  if (!(attr_dev_mask & dev_bit)) {
    cudaFuncAttributes fa;
    B200_CHECK_CUDA(e, cudaFuncGetAttributes(&fa, conv_tma_pair_kernel));
    B200_CHECK_CUDA(e, cudaFuncSetAttribute(conv_tma_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)(optin - fa.sharedSizeBytes)));
    // how many pairs fit at once: a pair needs two SMs of one GPC
    cudaLaunchConfig_t probe = {};
    probe.gridDim = dim3(2 * (e->sm_count / 2));
    probe.blockDim = dim3(CP_THREADS);
    probe.dynamicSmemBytes = smem;
    cudaLaunchAttribute pa[1];
    pa[0].id = cudaLaunchAttributeClusterDimension;
    pa[0].val.clusterDim.x = 2;
    pa[0].val.clusterDim.y = 1;
    pa[0].val.clusterDim.z = 1;
    probe.attrs = pa;
    probe.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, conv_tma_pair_kernel, &probe) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = e->sm_count / 2;
    }
    max_clusters[e->device & 31] = n;
    attr_dev_mask |= dev_bit;
  }
  const long long pair_tiles = (long long)((p.tiles_m + 1) / 2) * p.tiles_n;
  const int pairs = (int)std::min<long long>(pair_tiles, max_clusters[e->device & 31].load());
  conv_tma_pair_kernel<<<2 * pairs, CP_THREADS, smem, e->stream>>>(tm[0], tm[1], tm[2], tm[3], p);
  B200_CHECK_LAUNCH(e, "conv_tma_pair_kernel");
  e->flags_dirty = true;
  return B200_OK;
}

}  // namespace b200
