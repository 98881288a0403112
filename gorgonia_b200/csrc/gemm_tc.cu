// Matrix multiply on the 5th-generation tensor cores (tcgen05), operands fed by TMA, accumulators
// in tensor memory. Stands where Engine.MatMul calls cuBLAS Sgemm in gorgonia
// (cuda/linalg.go:110-229) and where batchedMatMul loops over slices (operatorLinAlg.go:435-502).
//
// One persistent CTA per SM, 10 warps with fixed roles:
//   warp 0     TMA producer: one lane queues the A and B boxes of each k-block into a ring of
//              shared-memory stages (128-byte swizzle) and arms the stage's "full" mbarrier;
//   warp 1     MMA issuer: one lane issues tcgen05.mma for each 32-byte k-slice of a stage,
//              commits the stage's "empty" mbarrier when the tensor core has read it, and commits
//              the accumulator's "full" mbarrier after the last k-block. Owns the TMEM allocation;
//   warps 2-9  epilogue: each drains one half of the columns of its 32-lane quarter of the
//              accumulator with tcgen05.ld, applies the fused bias/activation and stores rows of C
//              with 128-bit stores.
// The accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue of tile i runs
// while the MMAs of tile i+1 are issued.
//
// Operand layouts. tcgen05 takes either operand K-major (k contiguous in memory) or MN-major
// (m resp. n contiguous). Row-major A (M x K) is K-major, row-major B (K x N) is MN-major; the
// transposed storages swap that. All four combinations run without a transposing pass: only the
// TMA box shape and two fields of the shared-memory descriptor differ.
//
// float32 runs as 3xTF32: each operand is split once into a TF32 head and a TF32 tail
// (x = hi + lo up to 2^-22 relative), and three products hi*lo, lo*hi, hi*hi are accumulated in
// fp32 into the same accumulator, smallest terms first. The split is one streaming pass into
// arena scratch; the main loop then loads four tiles per stage and issues three MMAs per slice.
//
// CTA pairs (PAIR, bf16 only): large problems run as clusters of two CTAs on neighbouring SMs that
// share one 256-row tile: each CTA loads its own 128 rows of A and only half of the tile's B rows,
// the even CTA issues tcgen05.mma.cta_group::2 (M = 256), which reads both halves of B across the
// pair, and each CTA drains its own 128 rows of the accumulator. A CTA then brings a third less
// into shared memory per k-block. The stage's "full" barrier lives in the even CTA and counts the
// bytes of both CTAs' loads; "empty" and "accumulator full" exist in both and the even CTA's commits
// name each in turn; "accumulator empty" lives in the even CTA and takes the arrivals of both
// epilogues. 3xTF32 does not pair up: its wide instruction A_head x [B_head | B_tail] would take
// B_head from one CTA and B_tail from the other, A_tail x B_head then needs half of B_head in each
// at one common offset, i.e. a second, half-size slab, and with 7/8 of the bytes per CTA the pair
// measured no faster than two CTAs on their own.
//
// No TMA multicast anywhere: every CTA loads its own tiles from local HBM.
// Every mbarrier wait is bounded; a wait that runs out raises the engine's error word and all
// roles leave their loops, TMEM is released and the kernel returns.
#include <cuda.h>
#include <cuda_bf16.h>
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

int gemm_simt(b200_engine *e, int dtype, int transA, int transB, long long M, long long N, long long K,
              const void *A, long long lda, const void *B, long long ldb, void *C, long long ldc, long long batch,
              long long strideA, long long strideB, long long strideC, const Epilogue &ep);

// ------------------------------------------------------------------------------------------
// kernel
// ------------------------------------------------------------------------------------------

constexpr int TC_BM = 128;
constexpr int TC_THREADS = 320;  // 10 warps: TMA, MMA, 8 epilogue
constexpr int TC_ROW_BYTES = 128;  // one swizzle row: 64 bf16 or 32 fp32 along the contiguous dim

struct GemmTcParams {
  long long M, N, K, batch;
  void *C;                      // may be null when only the split form is wanted
  long long ldc, strideC;
  float *C_hi, *C_lo;           // C additionally as TF32 head / tail with row pitch ld_split, or null
  long long ld_split;
  int tiles_m, tiles_n, num_k;  // num_k = k-blocks of BK elements
  int chunk_k;                  // k-blocks accumulated in tensor memory before the epilogue folds them
  int group_m;                  // rasterisation: m-blocks per group
  int stages;
  int c_vec;                    // 1: rows of C can be stored with 128-bit stores
  int a_zmul, b_zmul;           // 0: the operand is shared by all batch entries (z coordinate 0)
  // how the work is shared between the CTAs (TilePieces, tc_common.cuh); 3xTF32 only
  int streamk;
  int units;                    // tiles * num_k (0 when the k range is not shared)
  float *ws;                    // partial tiles, 2 slots of TC_BM x BN floats per CTA
  int *tile_count;              // parts delivered per tile; zero between launches
  int workers;                  // CTAs, or CTA pairs, that share the tiles out
  int sk_first, sk_workers;     // k ranges are shared from this tile on, among this many CTAs (TilePieces)
  Epilogue ep;
  int *err_flag;
};

// TERMS = 1: bf16 operands (kind::f16). TERMS = 3: fp32 as 3xTF32 (kind::tf32), tensor maps
// 0/1 = head/tail of A, 2/3 = head/tail of B.
// PAIR: two CTAs per 256-row tile (see the file comment); then B's map has a box of BN / 2 rows.
template <int TERMS, int BN, bool A_MN, bool B_MN, bool PAIR>
__global__ void __launch_bounds__(TC_THREADS, 1)
    gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                   const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmB1,
                   const __grid_constant__ GemmTcParams p) {
  static_assert(!PAIR || TERMS == 1, "only bf16 tiles are shared by a pair of CTAs");
  constexpr int ES = TERMS == 1 ? 2 : 4;           // operand element size
  constexpr int BK = TC_ROW_BYTES / ES;            // k elements per stage: 64 bf16 / 32 fp32
  constexpr int UK = 32 / ES;                      // k elements per MMA: 16 / 8
  constexpr int NSPLIT = TERMS == 1 ? 1 : 2;       // copies of each operand per stage (head, tail)
  constexpr int A_BYTES = TC_BM * TC_ROW_BYTES;    // 16 KB
  constexpr int B_BYTES = BN * TC_ROW_BYTES;
  constexpr int BH_BYTES = B_BYTES / 2;            // half of the tile's B rows
  // what one CTA holds per stage. Alone: every copy of A and B. In a pair: its A rows and its half of B
  constexpr int STAGE_BYTES = !PAIR ? NSPLIT * (A_BYTES + B_BYTES) : A_BYTES + BH_BYTES;
  constexpr int MN_PER_BOX = TC_ROW_BYTES / ES;    // m/n elements covered by one MN-major box
  constexpr int MMA_M = PAIR ? 2 * TC_BM : TC_BM;
  constexpr uint32_t IDESC = make_idesc(TERMS == 1 ? 1 : 2, A_MN, B_MN, MMA_M, BN);
  // 3xTF32: B's head and tail slabs are adjacent in shared memory, and so are the main and the
  // cross-term accumulator in tensor memory, so A_head x [B_head | B_tail] is ONE instruction of
  // width 2*BN. An instruction costs a fixed ~65 cycles on top of its arithmetic: two per k step
  // beat three.
  constexpr uint32_t IDESC_WIDE = make_idesc(2, A_MN, B_MN, MMA_M, TERMS == 1 ? BN : 2 * BN);
  constexpr int MAX_STAGES = 8;
  // TMEM columns of one accumulator buffer: 3xTF32 keeps the cross terms in a second accumulator
  constexpr int ACC_COLS = TERMS == 1 ? BN : 2 * BN;
  constexpr int TMEM_COLS = 2 * ACC_COLS;  // double-buffered; a power of two >= 32 for every BN used

  extern __shared__ __align__(1024) unsigned char tc_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], acc_full[2], acc_empty[2];
  __shared__ __align__(8) uint64_t epi_bar;  // the 8 epilogue warps meet here when a partial tile is handed over
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_fail, s_last;

  // the ring must start on a 1024-byte boundary for the 128-byte swizzle
  unsigned char *smem = reinterpret_cast<unsigned char *>(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages;
  const uint32_t rank = PAIR ? ptx::cluster_ctarank() : 0u;  // 0: the CTA that issues the pair's MMAs
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const long long tiles_per_batch = (long long)p.tiles_m * p.tiles_n;
  const long long total_tiles = tiles_per_batch * p.batch;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&acc_full[b], 1);
      ptx::mbar_init(&acc_empty[b], PAIR ? 16 : 8);  // one arrival per epilogue warp (of both CTAs)
    }
    ptx::mbar_init(&epi_bar, 8);
    ptx::fence_mbar_init();
    s_fail = 0;
    s_last = 0;
  }
  if (warp == 1) {
    if (PAIR) {
      ptx::tmem_alloc_pair(&tmem_base_s, TMEM_COLS);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(&tmem_base_s, TMEM_COLS);
      ptx::tmem_relinquish();
    }
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tmap(&tmA0);
    ptx::prefetch_tmap(&tmB0);
    if (TERMS == 3) {
      ptx::prefetch_tmap(&tmA1);
      ptx::prefetch_tmap(&tmB1);
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (PAIR) ptx::cluster_sync();  // the other CTA's barriers are initialised before anything reaches them
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  // shared::cluster address of a barrier of the even CTA / of the other CTA
  auto at_leader = [&](uint64_t *bar) { return PAIR ? ptx::map_to_rank(ptx::smem_addr(bar), 0u) : ptx::smem_addr(bar); };
  auto at_peer = [&](uint64_t *bar) { return ptx::map_to_rank(ptx::smem_addr(bar), rank ^ 1u); };

  // tile index -> (batch, m block, n block); m blocks are walked in groups so that the CTAs of
  // one wave share B columns and A rows in L2
  auto decode = [&](long long tile, int &bz, int &mb, int &nb) {
    bz = (int)(tile / tiles_per_batch);
    const int t = (int)(tile % tiles_per_batch);
    const int per_group = p.group_m * p.tiles_n;
    const int g = t / per_group;
    const int first_m = g * p.group_m;
    const int gm = (p.tiles_m - first_m) < p.group_m ? (p.tiles_m - first_m) : p.group_m;
    const int r = t % per_group;
    mb = first_m + r % gm;
    nb = r / gm;
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      TilePieces pieces(p.streamk, p.units, p.num_k, (int)total_tiles, worker, p.workers, p.sk_first, p.sk_workers);
      int tile, kb0, kb1;
      while (ok && pieces.next(tile, kb0, kb1)) {
        int bz, mb, nb;
        decode(tile, bz, mb, nb);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1)) {
            ok = false;
            break;
          }
          unsigned char *st = smem + (size_t)stage * STAGE_BYTES;
          const int k0 = kb * BK;
          if (PAIR) {
            // the even CTA arms the stage for the bytes of both CTAs; the odd CTA's bytes may land
            // first, which only drives the pending count below zero for a moment
            if (rank == 0) ptx::mbar_arrive_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
            const uint32_t fb = at_leader(&full_bar[stage]);
            const int m0 = (mb * 2 + (int)rank) * TC_BM;
            if (!A_MN) {
              ptx::tma_load_3d_pair(st, &tmA0, k0, m0, bz * p.a_zmul, fb);
            } else {
#pragma unroll
              for (int q = 0; q < TC_BM / MN_PER_BOX; ++q)
                ptx::tma_load_3d_pair(st + q * (BK * TC_ROW_BYTES), &tmA0, m0 + q * MN_PER_BOX, k0, bz * p.a_zmul, fb);
            }
            unsigned char *sb = st + A_BYTES;
            const int nh = nb * BN + (int)rank * (BN / 2);  // this CTA's half of the tile's B rows
            if (!B_MN) {
              ptx::tma_load_3d_pair(sb, &tmB0, k0, nh, bz * p.b_zmul, fb);  // box of BN / 2 rows
            } else {
#pragma unroll
              for (int q = 0; q < BN / 2 / MN_PER_BOX; ++q)
                ptx::tma_load_3d_pair(sb + q * (BK * TC_ROW_BYTES), &tmB0, nh + q * MN_PER_BOX, k0, bz * p.b_zmul, fb);
            }
          } else {
            ptx::mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
#pragma unroll
            for (int h = 0; h < NSPLIT; ++h) {
              const CUtensorMap *ta = h == 0 ? &tmA0 : &tmA1;
              const CUtensorMap *tb = h == 0 ? &tmB0 : &tmB1;
              unsigned char *sa = st + h * A_BYTES;
              unsigned char *sb = st + NSPLIT * A_BYTES + h * B_BYTES;
              if (!A_MN) {
                ptx::tma_load_3d(sa, ta, k0, mb * TC_BM, bz * p.a_zmul, &full_bar[stage]);
              } else {
#pragma unroll
                for (int q = 0; q < TC_BM / MN_PER_BOX; ++q)
                  ptx::tma_load_3d(sa + q * (BK * TC_ROW_BYTES), ta, mb * TC_BM + q * MN_PER_BOX, k0,
                                   bz * p.a_zmul, &full_bar[stage]);
              }
              if (!B_MN) {
                ptx::tma_load_3d(sb, tb, k0, nb * BN, bz * p.b_zmul, &full_bar[stage]);
              } else {
#pragma unroll
                for (int q = 0; q < BN / MN_PER_BOX; ++q)
                  ptx::tma_load_3d(sb + q * (BK * TC_ROW_BYTES), tb, nb * BN + q * MN_PER_BOX, k0,
                                   bz * p.b_zmul, &full_bar[stage]);
              }
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
    // ---------------- MMA issuer (of a pair: the even CTA's only) ----------------
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int use = 0;  // accumulator-buffer uses so far (one per k-chunk)
      bool ok = true;
      // descriptors of stage 0, k-slice 0; a later stage adds its byte offset >> 4, a later k-slice
      // 32 bytes along a K-major row or UK k-rows of an MN-major block (the steps the helpers take)
      constexpr int A_STEP = (A_MN ? UK * TC_ROW_BYTES : 32) >> 4, B_STEP = (B_MN ? UK * TC_ROW_BYTES : 32) >> 4;
      const uint32_t st0 = ptx::smem_addr(smem);
      uint64_t a_desc0[NSPLIT], b_desc0[NSPLIT];
#pragma unroll
      for (int h = 0; h < NSPLIT; ++h) {
        a_desc0[h] = make_smem_desc(st0 + h * A_BYTES, A_MN ? BK * TC_ROW_BYTES : 16, (A_MN && ES == 4) ? 512 : 1024,
                                    (A_MN && ES == 4) ? 1 : 2);
        // pair: this CTA's half of B
        b_desc0[h] = make_smem_desc(st0 + NSPLIT * A_BYTES + h * B_BYTES, B_MN ? BK * TC_ROW_BYTES : 16,
                                    (B_MN && ES == 4) ? 512 : 1024, (B_MN && ES == 4) ? 1 : 2);
      }
      const uint32_t full0 = ptx::smem_addr(&full_bar[0]), empty0 = ptx::smem_addr(&empty_bar[0]);
      const uint32_t empty0_peer = PAIR ? ptx::map_to_rank(empty0, 1u) : 0u;
      uint32_t ready = 0;  // the poll behind the previous k-block saw this stage's barrier complete
      TilePieces pieces(p.streamk, p.units, p.num_k, (int)total_tiles, worker, p.workers, p.sk_first, p.sk_workers);
      int tile, kb0, kb1;
      while (ok && pieces.next(tile, kb0, kb1)) {
        for (int kc = kb0; kc < kb1 && ok; kc += p.chunk_k, ++use) {
          const int buf = use & 1;
          const uint32_t acc_phase = (uint32_t)((use >> 1) & 1);
          // the epilogue must have drained this accumulator buffer (first use passes at once)
          if (!ptx::mbar_wait(&acc_empty[buf], acc_phase ^ 1)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t d_main = tmem_base + (uint32_t)(buf * ACC_COLS);
          const uint32_t d_tail = d_main + BN;  // 3xTF32 only: the small cross terms
          const int kend = kc + p.chunk_k < kb1 ? kc + p.chunk_k : kb1;
          for (int kb = kc; kb < kend; ++kb) {
            if (!ready && !ptx::mbar_wait(&full_bar[stage], phase)) {
              ok = false;
              break;
            }
            ptx::tc_fence_after_sync();
            const int ns = stage + 1 == stages ? 0 : stage + 1;
            const uint32_t nphase = ns == 0 ? phase ^ 1u : phase;
            const uint64_t soff = (uint64_t)((uint32_t)stage * (uint32_t)(STAGE_BYTES >> 4));  // stays inside the address field
            const uint32_t eb = empty0 + (uint32_t)stage * 8u, ebp = empty0_peer + (uint32_t)stage * 8u;
            const uint32_t nf = full0 + (uint32_t)ns * 8u;
            const uint32_t first = kb > kc ? 1u : 0u;  // the chunk's first MMA overwrites the accumulator
            if (TERMS == 1)
              ready = ptx::kblock_f16<PAIR, A_STEP, B_STEP>(d_main, a_desc0[0] + soff, b_desc0[0] + soff, IDESC, first, eb,
                                                            ebp, nf, nphase);
            else  // hi * [hi | lo] into d_main (width 2 BN), lo * hi into d_tail
              ready = ptx::kblock_tf32x3<false, A_STEP, B_STEP>(d_main, d_tail, a_desc0[0] + soff, a_desc0[NSPLIT - 1] + soff,
                                                                b_desc0[0] + soff, b_desc0[0] + soff, IDESC_WIDE, IDESC, first,
                                                                eb, ebp, nf, nphase);
            stage = ns;
            phase = nphase;
          }
          if (ok) {  // this chunk's accumulators are complete
            if (PAIR) {
              ptx::mma_commit_pair(ptx::smem_addr(&acc_full[buf]));
              ptx::mma_commit_pair(at_peer(&acc_full[buf]));
            } else {
              ptx::mma_commit(&acc_full[buf]);
            }
          }
        }
      }
      if (!ok) s_fail = 1;
    }
  } else {
    // ---------------- epilogue: warps 2..9 ----------------
    constexpr int HALF = BN / 2;
    const int quarter = warp & 3;        // the TMEM lanes this warp may read: 32*quarter .. +31
    const int half = (warp - 2) >> 2;    // which half of the tile's columns it takes
    const int ch0 = half * HALF;
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
    TilePieces pieces(p.streamk, p.units, p.num_k, (int)total_tiles, worker, p.workers, p.sk_first, p.sk_workers);
    int tile, kb0, kb1;
    while (ok && pieces.next(tile, kb0, kb1)) {
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);

      // where the tile lies is worked out when a store needs it, not before the k loop: the fold
      // below wants every register it can get
      auto store32 = [&](const float(&v)[32], int c) {
        int bz, mb, nb;
        decode(tile, bz, mb, nb);
        const long long m = (long long)(PAIR ? mb * 2 + (int)rank : mb) * TC_BM + quarter * 32 + lane;
        float *crow = reinterpret_cast<float *>(p.C) + (long long)bz * p.strideC + m * p.ldc;
        const long long n0 = (long long)nb * BN;
        if (m >= p.M) return;
        const long long nbase = n0 + ch0 + c;
        if (p.C_hi) {
          // the result as the next product's A operand: TF32 head and tail, 16 bytes at a time;
          // columns between N and the pitch hold zeros
          float *hrow = p.C_hi + m * p.ld_split, *lrow = p.C_lo + m * p.ld_split;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            if (nbase + j >= p.ld_split) break;
            float h[4], l[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              float o = 0.f;
              if (nbase + j + t < p.N) {
                o = apply_epilogue<float>(v[j + t], p.ep, m, nbase + j + t);
                if (p.C) crow[nbase + j + t] = o;
              }
              uint32_t hb;
              asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(o));
              h[t] = __uint_as_float(hb);
              asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(__fsub_rn(o, h[t])));
              l[t] = __uint_as_float(hb);
            }
            *reinterpret_cast<float4 *>(hrow + nbase + j) = make_float4(h[0], h[1], h[2], h[3]);
            *reinterpret_cast<float4 *>(lrow + nbase + j) = make_float4(l[0], l[1], l[2], l[3]);
          }
          return;
        }
        if (p.c_vec && nbase + 32 <= p.N) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            float4 o;
            o.x = apply_epilogue<float>(v[j + 0], p.ep, m, nbase + j + 0);
            o.y = apply_epilogue<float>(v[j + 1], p.ep, m, nbase + j + 1);
            o.z = apply_epilogue<float>(v[j + 2], p.ep, m, nbase + j + 2);
            o.w = apply_epilogue<float>(v[j + 3], p.ep, m, nbase + j + 3);
            if (p.ep.accumulate) {  // Incr mode: the rounded result is added to what C holds
              const float4 old = *reinterpret_cast<const float4 *>(crow + nbase + j);
              o.x = __fadd_rn(old.x, o.x); o.y = __fadd_rn(old.y, o.y);
              o.z = __fadd_rn(old.z, o.z); o.w = __fadd_rn(old.w, o.w);
            }
            *reinterpret_cast<float4 *>(crow + nbase + j) = o;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (nbase + j < p.N) {
              const float o = apply_epilogue<float>(v[j], p.ep, m, nbase + j);
              crow[nbase + j] = p.ep.accumulate ? __fadd_rn(crow[nbase + j], o) : o;
            }
        }
      };

      if (TERMS == 1) {
        // one chunk per tile: straight from tensor memory to C
        const int buf = use & 1;
        const uint32_t acc_phase = (uint32_t)((use >> 1) & 1);
        ++use;
        if (!ptx::mbar_wait_relaxed(&acc_full[buf], acc_phase)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after_sync();
#pragma unroll 1
        for (int c = 0; c < HALF; c += 32) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(lane_addr + (uint32_t)(buf * ACC_COLS + ch0 + c), r);
          ptx::tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          store32(v, c);
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (PAIR) ptx::mbar_arrive_cluster(at_leader(&acc_empty[buf]));
          else ptx::mbar_arrive(&acc_empty[buf]);
        }
      } else {
        // 3xTF32: the tensor core adds into its accumulator with truncation, a bias that grows
        // with the length of the accumulation chain. Chains are therefore cut into k-chunks; each
        // chunk's two accumulators (main and cross terms) are folded here into fp32 registers
        // with round-to-nearest adds while the next chunk is being multiplied.
        float acc[TERMS == 3 ? HALF : 1];
#pragma unroll
        for (int j = 0; j < (TERMS == 3 ? HALF : 1); ++j) acc[j] = 0.f;
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
          for (int c = 0; c < (TERMS == 3 ? HALF : 0); c += 16) {
            uint32_t rm[16], rt[16];
            ptx::tmem_ld_32x16(lane_addr + (uint32_t)(buf * ACC_COLS + ch0 + c), rm);
            ptx::tmem_ld_32x16(lane_addr + (uint32_t)(buf * ACC_COLS + BN + ch0 + c), rt);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j)
              acc[c + j] = __fadd_rn(acc[c + j], __fadd_rn(__uint_as_float(rm[j]), __uint_as_float(rt[j])));
          }
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if (PAIR) ptx::mbar_arrive_cluster(at_leader(&acc_empty[buf]));
            else ptx::mbar_arrive(&acc_empty[buf]);
          }
        }
        if (kb0 != 0 || kb1 != p.num_k) {
          // part of a tile: leave it in the workspace; the CTA that delivers the last part finishes the tile
          constexpr int NACC = TERMS == 3 ? HALF : 1;
          const int tile_u0 = (tile - p.sk_first) * p.num_k;  // among the units that are shared out
          const size_t slot_floats = (size_t)TC_BM * BN;
          const size_t within = ((size_t)(warp - 2) * HALF) * 32 + lane;
          if (ok) {
            float *wsp = p.ws + (size_t)share_slot(worker, tile_u0, p.units, p.sk_workers) * slot_floats + within;
#pragma unroll
            for (int j = 0; j < NACC; ++j) __stcg(wsp + j * 32, acc[j]);
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
          for (int j = 0; j < NACC; ++j) acc[j] = 0.f;
          for (int c = c_first; c <= c_last; ++c) {  // k order: CTA c's share precedes CTA c + 1's
            const float *src = p.ws + (size_t)share_slot(c, tile_u0, p.units, p.sk_workers) * slot_floats + within;
#pragma unroll
            for (int j = 0; j < NACC; ++j) acc[j] = __fadd_rn(acc[j], ptx::ld_cg_ordered(src + j * 32));
          }
        }
        if (ok) {
#pragma unroll
          for (int c = 0; c < (TERMS == 3 ? HALF : 0); c += 32) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = acc[c + j];
            store32(v, c);
          }
        }
      }
    }
    if (!ok) s_fail = 1;
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  // a pair: neither CTA leaves, or gives its tensor memory back, while the other may still read its
  // shared memory or arrive on its barriers (every wait above is bounded, so both get here)
  if (PAIR) ptx::cluster_sync();
  if (threadIdx.x == 0 && s_fail) atomicExch(p.err_flag, 1);
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    if (PAIR) ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------
// What the tensor cores can do with kind::tf32 when nothing else is in the way: every SM issues
// 128 x 256 x 8 MMAs back to back on operands that already sit in shared memory, with no loads
// and no epilogue. The rate it reaches is the denominator of the float32 tensor rooflines.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128, 1) tf32_peak_kernel(int batches, int *err_flag) {
  constexpr int BN = 256, PER_BATCH = 16;
  extern __shared__ __align__(1024) unsigned char pk_smem_raw[];
  __shared__ __align__(8) uint64_t bar[2];
  __shared__ uint32_t tmem_base_s;
  unsigned char *smem = reinterpret_cast<unsigned char *>(((uintptr_t)pk_smem_raw + 1023) & ~(uintptr_t)1023);
  // operands: TF32 values of both signs and mixed magnitude (all-zero operands would flatter the clocks)
  uint32_t *w = reinterpret_cast<uint32_t *>(smem);
  for (int i = threadIdx.x; i < (TC_BM + BN) * TC_ROW_BYTES / 4; i += blockDim.x) {
    const uint32_t h = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
    w[i] = (h & 0x80000000u) | (0x3F000000u + ((h >> 3) & 0x00FFE000u));
  }
  ptx::fence_proxy_async_smem();
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar[0], 1);
    ptx::mbar_init(&bar[1], 1);
    ptx::fence_mbar_init();
  }
  if (warp == 0) {
    ptx::tmem_alloc(&tmem_base_s, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  if (threadIdx.x == 0) {
    constexpr uint32_t IDESC = make_idesc(2, false, false, TC_BM, BN);
    const uint32_t sa = ptx::smem_addr(smem), sb = sa + TC_BM * TC_ROW_BYTES;
    bool ok = true;
    for (int b = 0; b < batches && ok; ++b) {
#pragma unroll
      for (int i = 0; i < PER_BATCH; ++i) {
        const uint32_t off = (uint32_t)(i & 3) * 32;  // the four 8-wide k-slices of the 32-wide slab
        ptx::mma_tf32(tmem_base + (uint32_t)((i >> 2) & 1) * BN, make_smem_desc(sa + off, 16, 1024, 2),
                      make_smem_desc(sb + off, 16, 1024, 2), IDESC, (b | i) ? 1u : 0u);
      }
      ptx::mma_commit(&bar[b & 1]);
      // one batch stays in flight: wait for the batch before this one
      if (b > 0) ok = ptx::mbar_wait(&bar[(b - 1) & 1], (uint32_t)(((b - 1) >> 1) & 1));
    }
    if (ok && batches > 0) ok = ptx::mbar_wait(&bar[(batches - 1) & 1], (uint32_t)(((batches - 1) >> 1) & 1));
    if (!ok) atomicExch(err_flag, 1);
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------
// TF32 split: x -> (head, tail), both TF32 values in fp32 containers, written densely with the
// row length padded to a multiple of 4 elements (so that TMA row pitches stay 16-byte multiples)
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

__global__ void __launch_bounds__(256) split_tf32_kernel(const float *__restrict__ src, long long ld_in,
                                                         long long stride_in, float *__restrict__ hi,
                                                         float *__restrict__ lo, long long rows, long long cols,
                                                         long long ld_out, long long batch) {
  const long long per = rows * ld_out;
  const long long total = per * batch;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const long long b = t / per, rem = t % per;
    const long long r = rem / ld_out, c = rem % ld_out;
    float x = 0.f;
    if (c < cols) x = src[b * stride_in + r * ld_in + c];
    const float h = to_tf32(x);
    hi[t] = h;
    lo[t] = to_tf32(__fsub_rn(x, h));
  }
}

// The same for rows that can be read 16 bytes at a time (pitch and width multiples of 4, aligned
// base): a block walks whole rows, a thread takes four elements per step, and nothing is divided
// per element.
__global__ void __launch_bounds__(256) split_tf32_rows4_kernel(const float *__restrict__ src, long long ld_in,
                                                               long long stride_in, float *__restrict__ hi,
                                                               float *__restrict__ lo, long long rows, int cols4,
                                                               long long batch) {
  const long long total_rows = rows * batch;
  for (long long row = blockIdx.x; row < total_rows; row += gridDim.x) {
    const long long b = row / rows, r = row - b * rows;
    const float4 *in = reinterpret_cast<const float4 *>(src + b * stride_in + r * ld_in);
    float4 *oh = reinterpret_cast<float4 *>(hi) + row * cols4;
    float4 *ol = reinterpret_cast<float4 *>(lo) + row * cols4;
    for (int c = threadIdx.x; c < cols4; c += blockDim.x) {
      const float4 v = __ldg(in + c);
      float4 h, l;
      h.x = to_tf32(v.x); h.y = to_tf32(v.y); h.z = to_tf32(v.z); h.w = to_tf32(v.w);
      l.x = to_tf32(__fsub_rn(v.x, h.x)); l.y = to_tf32(__fsub_rn(v.y, h.y));
      l.z = to_tf32(__fsub_rn(v.z, h.z)); l.w = to_tf32(__fsub_rn(v.w, h.w));
      oh[c] = h;
      ol[c] = l;
    }
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
  });
  return fn;
}

// A 3-D map (contiguous dim, rows, batch) over a row-major matrix with `ld` elements per row.
int encode_map(b200_engine *e, CUtensorMap *map, int es, const void *base, long long inner, long long rows,
                      long long batch, long long ld, long long batch_stride, int box_inner, int box_rows,
                      bool atom32) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return set_error(e, B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * es, (cuuint64_t)(batch > 1 ? batch_stride : rows * ld) * es};
  cuuint32_t box[3] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, es == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                  const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(e, B200_ERR_CUDA,
                     "cuTensorMapEncodeTiled failed (%d): dims %lld x %lld x %lld, ld %lld, box %d x %d", (int)r,
                     inner, rows, batch, ld, box_inner, box_rows);
  return B200_OK;
}

static bool tc_eligible(int dtype, long long M, long long N, long long K, long long lda, long long ldb,
                        long long ldc, long long batch, long long strideA, long long strideB, const void *A,
                        const void *B, const void *C) {
  if (dtype != B200_F32 && dtype != B200_BF16) return false;
  if (M < 1 || N < 1 || K < 1) return false;
  // tiny problems: a 128-row tile would be mostly padding and the launch is latency-bound anyway
  if (M * N * K < 64LL * 64 * 64) return false;
  // bf16 operands are read in place, so a narrow B cannot meet TMA's pitch rule; float32 operands
  // are re-pitched by the split pass and any N works (the tile is padded with zero columns)
  if (N < 16 && dtype == B200_BF16) return false;
  if (N < 16 && M < 128) return false;
  if ((uintptr_t)C % 4 != 0) return false;
  if (dtype == B200_BF16) {
    if (((uintptr_t)A | (uintptr_t)B) % 16 != 0) return false;
    // TMA reads the caller's buffers directly: row pitch and batch pitch in bytes must be 16-byte multiples
    if ((lda * 2) % 16 || (ldb * 2) % 16) return false;
    if (batch > 1 && ((strideA * 2) % 16 || (strideB * 2) % 16)) return false;
  }
  // float32 goes through the split pass, which re-pitches rows itself: no constraint on lda / ldb
  (void)ldc;
  return true;
}

// Bytes of one ring stage in one CTA (the kernel's STAGE_BYTES).
static size_t tc_stage_bytes(int terms, int bn, bool pair) {
  const size_t a = (size_t)TC_BM * TC_ROW_BYTES, b = (size_t)bn * TC_ROW_BYTES;
  return pair ? a + b / 2 : (terms == 1 ? 1 : 2) * (a + b);
}

// grid = CTAs; pairs launch as clusters of two.
template <int TERMS, int BN, bool A_MN, bool B_MN, bool PAIR>
static int launch_tc(b200_engine *e, const CUtensorMap *tm, const GemmTcParams &p, int grid) {
  auto kern = gemm_tc_kernel<TERMS, BN, A_MN, B_MN, PAIR>;
  const size_t smem = (size_t)p.stages * tc_stage_bytes(TERMS, BN, PAIR) + 1024;
  static std::atomic<int> attr_dev_mask{0};  // devices on which the attribute is set; engines on other threads share it
  if (!(attr_dev_mask & (1 << (e->device & 31)))) {
    // opt in to the large dynamic carve-out: what the SM offers minus this kernel's static part
    cudaFuncAttributes fa;
    B200_CHECK_CUDA(e, cudaFuncGetAttributes(&fa, kern));
    const size_t optin = std::min<size_t>(e->smem_optin, 227 * 1024);
    B200_CHECK_CUDA(e, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)(optin - fa.sharedSizeBytes)));
    attr_dev_mask |= 1 << (e->device & 31);
  }
  if (PAIR) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = e->stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    // Only clusters that are resident together may share the tiles out evenly: a GPU whose SMs do
    // not all pair up would otherwise run the left-over clusters as a second round.
    static std::atomic<int> max_clusters[32];
    int mc = max_clusters[e->device & 31];
    if (mc == 0) {
      B200_CHECK_CUDA(e, cudaOccupancyMaxActiveClusters(&mc, kern, &cfg));
      if (mc < 1) return set_error(e, B200_ERR_CUDA, "gemm_tc_kernel: no pair of CTAs fits this device");
      max_clusters[e->device & 31] = mc;
    }
    GemmTcParams pp = p;
    pp.workers = std::min(p.workers, mc);
    cfg.gridDim = dim3((unsigned)(2 * pp.workers));
    B200_CHECK_CUDA(e, cudaLaunchKernelEx(&cfg, kern, tm[0], tm[1], tm[2], tm[3], pp));
  } else {
    kern<<<grid, TC_THREADS, smem, e->stream>>>(tm[0], tm[1], tm[2], tm[3], p);
  }
  B200_CHECK_LAUNCH(e, "gemm_tc_kernel");
  e->flags_dirty = true;
  return B200_OK;
}

template <int TERMS, int BN, bool PAIR = false>
static int launch_tc_layout(b200_engine *e, bool a_mn, bool b_mn, const CUtensorMap *tm, const GemmTcParams &p,
                            int grid) {
  if (!a_mn && !b_mn) return launch_tc<TERMS, BN, false, false, PAIR>(e, tm, p, grid);
  if (!a_mn && b_mn) return launch_tc<TERMS, BN, false, true, PAIR>(e, tm, p, grid);
  if (a_mn && !b_mn) return launch_tc<TERMS, BN, true, false, PAIR>(e, tm, p, grid);
  return launch_tc<TERMS, BN, true, true, PAIR>(e, tm, p, grid);
}


// terms = 1 (bf16) or 3 (fp32 split into head/tail). a_mn / b_mn: the operand is stored with its
// m / n index contiguous (see the file comment).
int gemm_tc_core(b200_engine *e, int terms, bool a_mn, bool b_mn, long long M, long long N, long long K,
                 const TcOperand &a, const TcOperand &b, void *C, long long ldc, long long batch, long long strideC,
                 const Epilogue &ep, float *C_hi = nullptr, float *C_lo = nullptr, long long ld_split = 0) {
  const int es = terms == 1 ? 2 : 4;
  const int bk = TC_ROW_BYTES / es;
  // tile width: the widest that still gives every SM a tile, to keep small problems spread out
  const int tiles_m = (int)((M + TC_BM - 1) / TC_BM);
  const bool may_share_k = terms == 3 && !(e->flags & B200_ENGINE_NO_STREAMK);
  int bn = terms == 1 ? 256 : 128;
  // tile width: the widest that still gives every SM a tile. A problem too small for that gets the
  // narrow tiles whether or not its k range is shared out as well: one SM pulls operands from L2 at a
  // fixed rate, so more CTAs on more SMs shorten the k loop of each
  while (bn > 64 && (long long)tiles_m * ((N + bn - 1) / bn) * batch < e->sm_count) bn /= 2;
  while (bn > 64 && bn / 2 >= N) bn /= 2;
  const int tiles_n = (int)((N + bn - 1) / bn);
  // CTA pairs on 256-row tiles (bf16), when the widest tiles are in use and there are enough of
  // them to keep every pair busy for several rounds (a pair's tile is twice the size: the last
  // round's idle time doubles with it)
  const int pairs = e->sm_count / 2;
  const long long pair_tiles = (M + 2 * TC_BM - 1) / (2 * TC_BM) * tiles_n * batch;
  const bool pair = !(e->flags & B200_ENGINE_NO_PAIRS) && terms == 1 && bn == 256 && pair_tiles >= 4LL * pairs;

  CUtensorMap tm[4];
  memset(tm, 0, sizeof tm);
  const int mn_box = TC_ROW_BYTES / es;
  const long long a_batch = a.shared ? 1 : batch, b_batch = b.shared ? 1 : batch;
  for (int h = 0; h < (terms == 1 ? 1 : 2); ++h) {
    const void *ap = h == 0 ? a.p0 : a.p1, *bp = h == 0 ? b.p0 : b.p1;
    int rc;
    if (!a_mn)
      rc = encode_map(e, &tm[h], es, ap, K, M, a_batch, a.ld, a.batch_stride, bk, TC_BM, false);
    else
      rc = encode_map(e, &tm[h], es, ap, M, K, a_batch, a.ld, a.batch_stride, mn_box, bk, es == 4);
    if (rc != B200_OK) return rc;
    if (!b_mn)  // a pair's bf16 CTAs load half of the tile's B rows each
      rc = encode_map(e, &tm[2 + h], es, bp, K, N, b_batch, b.ld, b.batch_stride, bk,
                      pair ? bn / 2 : bn, false);
    else
      rc = encode_map(e, &tm[2 + h], es, bp, N, K, b_batch, b.ld, b.batch_stride, mn_box, bk, es == 4);
    if (rc != B200_OK) return rc;
  }
  if (terms == 1) {
    tm[1] = tm[0];
    tm[3] = tm[2];
  }

  GemmTcParams p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.batch = batch;
  p.C = C;
  p.ldc = ldc;
  p.strideC = strideC;
  p.C_hi = C_hi;
  p.C_lo = C_lo;
  p.ld_split = ld_split;
  p.tiles_m = tiles_m;
  p.tiles_n = tiles_n;
  p.num_k = (int)((K + bk - 1) / bk);
  // bf16: one chain per tile. 3xTF32: 8 k-blocks = 256 k = 32 accumulation steps per chain, which
  // keeps the truncation bias of the tensor core's adder near 5e-7 relative.
  p.chunk_k = terms == 1 ? p.num_k : 8;
  p.group_m = std::min(tiles_m, 8);
  p.c_vec = (C && ldc % 4 == 0 && (uintptr_t)C % 16 == 0 && (batch == 1 || strideC % 4 == 0)) ? 1 : 0;
  p.a_zmul = a.shared ? 0 : 1;
  p.b_zmul = b.shared ? 0 : 1;
  p.ep = ep;
  p.err_flag = e->d_flags + 2;
  const size_t stage_bytes = tc_stage_bytes(terms, bn, pair);
  const size_t budget = std::min<size_t>(e->smem_optin, 227 * 1024) - 4096;  // static part + alignment slack
  p.stages = (int)std::max<size_t>(2, std::min<size_t>(8, budget / stage_bytes));
  const long long total_tiles = (long long)tiles_m * tiles_n * batch;
  if (total_tiles >= (1LL << 31))
    return set_error(e, B200_ERR_UNSUPPORTED, "b200_gemm: %lld output tiles are more than one launch takes", total_tiles);
  int grid = (int)std::min<long long>(total_tiles, e->sm_count);
  p.streamk = 0;
  p.units = 0;
  p.ws = nullptr;
  p.tile_count = nullptr;
  p.workers = grid;
  p.sk_first = 0;
  p.sk_workers = grid;
  if (pair) {
    p.tiles_m = (int)((M + 2 * TC_BM - 1) / (2 * TC_BM));
    p.group_m = std::min(p.tiles_m, 4);  // the same 8 x 128 rows of A per raster group
    p.workers = (int)std::min<long long>(pair_tiles, pairs);
    return launch_tc_layout<1, 256, true>(e, a_mn, b_mn, tm, p, 2 * p.workers);
  }

  if (terms == 1) {
    if (bn == 256) return launch_tc_layout<1, 256>(e, a_mn, b_mn, tm, p, grid);
    if (bn == 128) return launch_tc_layout<1, 128>(e, a_mn, b_mn, tm, p, grid);
    return launch_tc_layout<1, 64>(e, a_mn, b_mn, tm, p, grid);
  }
  // whole tiles per CTA would leave SMs idle: share out the k range instead (TilePieces)
  void *ws = nullptr;
  int sk_grid = grid;
  if (may_share_k && total_tiles <= b200_engine::kSkCounters &&
      streamk_pays(total_tiles, p.num_k, e->sm_count, &sk_grid)) {
    if (b200_get(e, 2LL * sk_grid * TC_BM * bn * 4, &ws) == B200_OK) {
      p.streamk = 1;
      p.units = (int)(total_tiles * p.num_k);  // small: k sharing is for launches of few tiles
      grid = sk_grid;
      p.workers = grid;
      p.sk_workers = grid;
      p.tile_count = e->sk_counters;
      p.ws = (float *)ws;
    }  // else: no room for the partial tiles, whole tiles per CTA
  } else if (int first = 0, sk = 0; may_share_k && total_tiles - total_tiles / e->sm_count * e->sm_count <= b200_engine::kSkCounters &&
                                    streamk_tail_pays(total_tiles, p.num_k, e->sm_count, &first, &sk)) {
    // several waves of tiles and a ragged last one: the full waves whole, the rest along k
    if (b200_get(e, 2LL * sk * TC_BM * bn * 4, &ws) == B200_OK) {
      p.streamk = 1;
      p.sk_first = first;
      p.sk_workers = sk;
      p.units = (int)((total_tiles - first) * p.num_k);
      p.tile_count = e->sk_counters;
      p.ws = (float *)ws;
    }
  }
  const int rc = bn == 128 ? launch_tc_layout<3, 128>(e, a_mn, b_mn, tm, p, grid)
                           : launch_tc_layout<3, 64>(e, a_mn, b_mn, tm, p, grid);
  if (ws) b200_put(e, ws, 0);  // stream order: whoever gets the block next runs after this kernel
  return rc;
}

// Splits a row-major fp32 matrix (rows x cols, pitch ld, `batch` of them) into TF32 head and tail
// in arena scratch with a pitch that is a multiple of 4 elements. The caller hands the two
// blocks back with b200_put once the consuming kernel has been launched.
int split_operand_tf32(b200_engine *e, const float *src, long long rows, long long cols, long long ld,
                       long long batch, long long batch_stride, TcOperand *out, void **blk_hi, void **blk_lo) {
  const long long ldo = (cols + 3) / 4 * 4;
  const long long elems = rows * ldo * batch;
  *blk_hi = *blk_lo = nullptr;
  // a buffer declared constant (weights) is split once; the split is kept until the buffer is
  // released or un-declared, and the caller gets no blocks to hand back
  const bool constant = is_constant(e, src);
  if (constant) {
    if (CachedSplit *c = find_cached(e, src, 0, rows, cols, batch, ld)) {
      out->p0 = c->hi;
      out->p1 = c->lo;
      out->ld = c->ld_out;
      out->batch_stride = rows * c->ld_out;
      out->shared = false;
      return B200_OK;
    }
  }
  int rc = b200_get(e, elems * 4, blk_hi);
  if (rc != B200_OK) return rc;
  rc = b200_get(e, elems * 4, blk_lo);
  if (rc != B200_OK) {
    b200_put(e, *blk_hi, 0);
    *blk_hi = nullptr;
    return rc;
  }
  if (cols % 4 == 0 && ld % 4 == 0 && batch_stride % 4 == 0 && (uintptr_t)src % 16 == 0 && cols >= 256) {
    const int blocks = (int)std::max<long long>(1, std::min<long long>(rows * batch, e->sm_count * 16LL));
    split_tf32_rows4_kernel<<<blocks, 256, 0, e->stream>>>(src, ld, batch_stride, (float *)*blk_hi, (float *)*blk_lo,
                                                           rows, (int)(cols / 4), batch);
  } else {
    const int blocks = (int)std::max<long long>(1, std::min<long long>((elems + 255) / 256, e->sm_count * 16LL));
    split_tf32_kernel<<<blocks, 256, 0, e->stream>>>(src, ld, batch_stride, (float *)*blk_hi, (float *)*blk_lo, rows,
                                                     cols, ldo, batch);
  }
  cudaError_t le = cudaGetLastError();
  if (le != cudaSuccess) {
    b200_put(e, *blk_hi, 0);
    b200_put(e, *blk_lo, 0);
    *blk_hi = *blk_lo = nullptr;
    return set_error(e, B200_ERR_CUDA, "launch of split_tf32_kernel failed: %s", cudaGetErrorString(le));
  }
  e->launches++;
  out->p0 = *blk_hi;
  out->p1 = *blk_lo;
  out->ld = ldo;
  out->batch_stride = rows * ldo;
  out->shared = false;
  if (constant) {
    add_cached(e, src, CachedSplit{0, rows, cols, batch, ld, *blk_hi, *blk_lo, ldo});
    *blk_hi = *blk_lo = nullptr;  // kept: nothing for the caller to release
  }
  return B200_OK;
}

static int gemm_tc(b200_engine *e, int dtype, int transA, int transB, long long M, long long N, long long K,
                   const void *A, long long lda, const void *B, long long ldb, void *C, long long ldc,
                   long long batch, long long strideA, long long strideB, long long strideC, const Epilogue &ep) {
  const bool a_mn = transA != 0;   // stored K x M: m contiguous
  const bool b_mn = transB == 0;   // stored K x N: n contiguous
  TcOperand a, b;
  if (dtype == B200_BF16) {
    a.p0 = A;
    a.ld = lda;
    a.batch_stride = strideA;
    b.p0 = B;
    b.ld = ldb;
    b.batch_stride = strideB;
    return gemm_tc_core(e, 1, a_mn, b_mn, M, N, K, a, b, C, ldc, batch, strideC, ep);
  }
  // stored shapes (rows x contiguous)
  const long long a_rows = transA ? K : M, a_cols = transA ? M : K;
  const long long b_rows = transB ? N : K, b_cols = transB ? K : N;
  void *blk[4] = {nullptr, nullptr, nullptr, nullptr};
  int rc = split_operand_tf32(e, (const float *)A, a_rows, a_cols, lda, batch, strideA, &a, &blk[0], &blk[1]);
  if (rc == B200_OK) rc = split_operand_tf32(e, (const float *)B, b_rows, b_cols, ldb, batch, strideB, &b, &blk[2], &blk[3]);
  if (rc == B200_OK) rc = gemm_tc_core(e, 3, a_mn, b_mn, M, N, K, a, b, C, ldc, batch, strideC, ep);
  // stream order makes handing the scratch back safe: later users run after this kernel
  for (void *s2 : blk)
    if (s2) b200_put(e, s2, 0);
  return rc;
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_gemm_chain(b200_engine *e, int transB, int64_t M, int64_t N, int64_t K, const void *A, const void *A_hi,
                    const void *A_lo, int64_t lda, const void *B, int64_t ldb, void *C, void *C_hi, void *C_lo,
                    int64_t ldc, int64_t ld_split, const b200_epilogue *epi) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, M >= 0 && N > 0 && K > 0, "b200_gemm_chain: bad extent");
  B200_REQUIRE(e, (A_hi == nullptr) == (A_lo == nullptr) && (C_hi == nullptr) == (C_lo == nullptr),
               "b200_gemm_chain: a head needs its tail");
  B200_REQUIRE(e, A || A_hi, "b200_gemm_chain: no A");
  B200_REQUIRE(e, C || C_hi, "b200_gemm_chain: no output");
  B200_REQUIRE(e, B, "b200_gemm_chain: B is null");
  B200_REQUIRE(e, lda >= K && ldb >= (transB ? K : N) && (!C || ldc >= N), "b200_gemm_chain: leading dimension too small");
  B200_REQUIRE(e, !A_hi || (lda % 4 == 0 && ((uintptr_t)A_hi | (uintptr_t)A_lo) % 16 == 0),
               "b200_gemm_chain: a split A needs a pitch that is a multiple of 4 and 16-byte aligned pointers");
  B200_REQUIRE(e, !C_hi || (ld_split == (N + 3) / 4 * 4 && ((uintptr_t)C_hi | (uintptr_t)C_lo) % 16 == 0),
               "b200_gemm_chain: the split output needs the pitch N rounded up to a multiple of 4 and aligned pointers");
  if (epi) {
    B200_REQUIRE(e, epi->bias_kind >= 0 && epi->bias_kind <= 2 && epi->act >= 0 && epi->act <= 2,
                 "b200_gemm_chain: bad epilogue");
    B200_REQUIRE(e, epi->bias_kind == 0 || epi->bias != nullptr, "b200_gemm_chain: bias is null");
    B200_REQUIRE(e, epi->accumulate == 0, "b200_gemm_chain: accumulate cannot be combined with a chain");
  }
  if (M == 0) return B200_OK;
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  const Epilogue ep = make_epilogue(epi);
  const void *probe = A ? A : A_hi;
  if (tc_eligible(B200_F32, M, N, K, lda, ldb, ldc, 1, 0, 0, probe, B, C ? C : C_hi)) {
    TcOperand a, b;
    void *blk[4] = {nullptr, nullptr, nullptr, nullptr};
    if (A_hi) {
      a.p0 = A_hi;
      a.p1 = A_lo;
      a.ld = lda;
      a.batch_stride = M * lda;
    } else {
      rc = split_operand_tf32(e, (const float *)A, M, K, lda, 1, 0, &a, &blk[0], &blk[1]);
    }
    const long long b_rows = transB ? N : K, b_cols = transB ? K : N;
    if (rc == B200_OK) rc = split_operand_tf32(e, (const float *)B, b_rows, b_cols, ldb, 1, 0, &b, &blk[2], &blk[3]);
    if (rc == B200_OK)
      rc = gemm_tc_core(e, 3, false, transB == 0, M, N, K, a, b, C, ldc, 1, M * ldc, ep, (float *)C_hi, (float *)C_lo,
                        ld_split);
    for (void *s2 : blk)
      if (s2) b200_put(e, s2, 0);
    return rc;
  }
  // small or oddly shaped: the plain product, then the rewrite pass; both need the tensors unsplit
  if (!A)
    return set_error(e, B200_ERR_UNSUPPORTED,
                     "b200_gemm_chain: this shape runs on the CUDA-core kernel, which reads an unsplit A; pass A");
  void *tmp = nullptr;
  float *cf = (float *)C;
  long long ldc_eff = ldc;
  if (!C) {
    rc = b200_get(e, M * N * 4, &tmp);
    if (rc != B200_OK) return rc;
    cf = (float *)tmp;
    ldc_eff = N;
  }
  rc = gemm_simt(e, B200_F32, 0, transB, M, N, K, A, lda, B, ldb, cf, ldc_eff, 1, 0, 0, 0, ep);
  if (rc == B200_OK && C_hi) {
    const long long elems = M * ld_split;
    const int blocks = (int)std::max<long long>(1, std::min<long long>((elems + 255) / 256, e->sm_count * 16LL));
    split_tf32_kernel<<<blocks, 256, 0, e->stream>>>(cf, ldc_eff, 0, (float *)C_hi, (float *)C_lo, M, N, ld_split, 1);
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) rc = set_error(e, B200_ERR_CUDA, "launch of split_tf32_kernel failed: %s", cudaGetErrorString(le));
    else e->launches++;
  }
  if (tmp) b200_put(e, tmp, 0);
  return rc;
}

int b200_tf32_peak(b200_engine *e, int batches, double *tflops) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, tflops != nullptr, "b200_tf32_peak: null pointer");
  B200_REQUIRE(e, batches >= 1 && batches <= 1000000, "b200_tf32_peak: 1 .. 1000000 batches of 16 instructions");
  B200_NOT_WHILE_CAPTURING(e, "b200_tf32_peak");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  const size_t smem = (size_t)(TC_BM + 256) * TC_ROW_BYTES + 1024;
  B200_CHECK_CUDA(e, cudaFuncSetAttribute(tf32_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cudaEvent_t ev0, ev1;
  B200_CHECK_CUDA(e, cudaEventCreate(&ev0));
  B200_CHECK_CUDA(e, cudaEventCreate(&ev1));
  float best = 0.f;
  for (int rep = 0; rep < 4 && rc == B200_OK; ++rep) {  // the first repetition warms up
    cudaEventRecord(ev0, e->stream);
    tf32_peak_kernel<<<e->sm_count, 128, smem, e->stream>>>(batches, e->d_flags + 2);
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) {
      rc = set_error(e, B200_ERR_CUDA, "launch of tf32_peak_kernel failed: %s", cudaGetErrorString(le));
      break;
    }
    e->launches++;
    e->flags_dirty = true;
    cudaEventRecord(ev1, e->stream);
    rc = sync_stream_checked(e);
    float ms = 0.f;
    if (rc == B200_OK && cudaEventElapsedTime(&ms, ev0, ev1) == cudaSuccess && rep > 0 && (best == 0.f || ms < best))
      best = ms;
  }
  cudaEventDestroy(ev0);
  cudaEventDestroy(ev1);
  if (rc != B200_OK) return rc;
  const double flops = 2.0 * TC_BM * 256 * 8 * 16.0 * batches * e->sm_count;
  *tflops = best > 0.f ? flops / (best * 1e-3) / 1e12 : 0.0;
  return B200_OK;
}

int b200_gemm_path(b200_engine *e, int dtype, int transA, int transB, int64_t M, int64_t N, int64_t K, int64_t lda,
                   int64_t ldb, int64_t ldc, const void *A, const void *B, const void *C) {
  (void)e;
  (void)transA;
  (void)transB;
  return tc_eligible(dtype, M, N, K, lda, ldb, ldc, 1, 0, 0, A, B, C) ? 1 : 0;
}

int b200_gemm(b200_engine *e, int dtype, int transA, int transB, int64_t M, int64_t N, int64_t K, const void *A,
              int64_t lda, const void *B, int64_t ldb, void *C, int64_t ldc, int64_t batch, int64_t strideA,
              int64_t strideB, int64_t strideC, const b200_epilogue *epi) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64 || dtype == B200_BF16, "b200_gemm: dtype %d not supported",
               dtype);
  B200_REQUIRE(e, M >= 0 && N >= 0 && K >= 0 && batch >= 0, "b200_gemm: negative extent");
  if (M == 0 || N == 0 || batch == 0) return B200_OK;
  B200_REQUIRE(e, C != nullptr, "b200_gemm: C is null");
  const int64_t a_cols = transA ? M : K, b_cols = transB ? K : N;
  B200_REQUIRE(e, lda >= a_cols && ldb >= b_cols && ldc >= N, "b200_gemm: leading dimension too small (%lld %lld %lld)",
               (long long)lda, (long long)ldb, (long long)ldc);
  if (epi) {
    B200_REQUIRE(e, epi->bias_kind >= 0 && epi->bias_kind <= 2 && epi->act >= 0 && epi->act <= 2,
                 "b200_gemm: bad epilogue");
    B200_REQUIRE(e, epi->bias_kind == 0 || epi->bias != nullptr, "b200_gemm: bias is null");
  }
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  Epilogue ep = make_epilogue(epi);
  if (K == 0) {
    // empty sum: C = epilogue(0); the CUDA-core kernel handles it with a zero-trip k loop
    if (dtype == B200_BF16) return set_error(e, B200_ERR_UNSUPPORTED, "b200_gemm: bf16 with K = 0");
    return gemm_simt(e, dtype, transA, transB, M, N, 0, C, lda, C, ldb, C, ldc, batch, 0, 0, strideC, ep);
  }
  B200_REQUIRE(e, A && B, "b200_gemm: null operand");
  if (tc_eligible(dtype, M, N, K, lda, ldb, ldc, batch, strideA, strideB, A, B, C)) {
    rc = gemm_tc(e, dtype, transA, transB, M, N, K, A, lda, B, ldb, C, ldc, batch, strideA, strideB, strideC, ep);
    // The float32 tensor-core path keeps TF32 splits of both operands in arena scratch (about
    // 2 x (|A| + |B|) bytes). The reference's MatMul needs no workspace, so an arena too full for
    // the splits still gets its product, from the CUDA-core kernel, which needs none.
    if (rc != B200_ERR_OOM || dtype != B200_F32) return rc;
  }
  if (dtype == B200_BF16)
    return set_error(e, B200_ERR_UNSUPPORTED,
                     "b200_gemm: bf16 operands need 16-byte aligned bases and row pitches (lda %lld, ldb %lld) and "
                     "at least 64^3 work",
                     (long long)lda, (long long)ldb);
  return gemm_simt(e, dtype, transA, transB, M, N, K, A, lda, B, ldb, C, ldc, batch, strideA, strideB, strideC, ep);
}

}  // extern "C"
