// Thin inline-PTX wrappers for the sm_100a features the kernels use: mbarriers, bulk (TMA)
// copies, tensor-map TMA loads, tcgen05 (tensor memory + MMA). Every wait is bounded: it gives
// up after a wall-clock limit and reports failure instead of spinning forever.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {
namespace ptx {

__device__ __forceinline__ uint32_t smem_addr(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// A 4-byte load that bypasses L1 and keeps its place among other such loads (volatile): used where
// a long unrolled run of loads must not be hoisted into one block of live registers.
__device__ __forceinline__ float ld_cg_ordered(const float *p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

// ---- mbarrier ------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint64_t *bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// makes mbarrier initialisation visible to the async proxy (TMA, tcgen05.commit)
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity to complete. Returns false if it did not within
// `limit_ns` of wall-clock time (default 2 s): the caller then records the failure and leaves.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint64_t limit_ns = 2000000000ull) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (globaltimer_ns() - t0 > limit_ns) return false;
  }
}

// The same wait for roles with slack (an epilogue that is handed work every few k-blocks, a
// producer that runs stages ahead): it sleeps between polls, so that the polling warp does not
// take issue slots from the warps it is waiting for.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t *bar, uint32_t parity, unsigned sleep_ns = 128,
                                                  uint64_t limit_ns = 2000000000ull) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      __nanosleep(sleep_ns);
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (globaltimer_ns() - t0 > limit_ns) return false;
  }
}

// ---- proxies / fences ---------------------------------------------------------------------------
// generic-proxy writes to shared memory -> visible to the async proxy (TMA store, tcgen05.mma)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- bulk copies (no tensor map): 16-byte aligned addresses, size a multiple of 16 -----------
__device__ __forceinline__ void bulk_g2s(void *smem_dst, const void *gmem_src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void *gmem_dst, const void *smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(smem_addr(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---- tensor-map TMA loads (tile mode), no multicast -----------------------------------------
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const void *tmap, int x, int y, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
          "r"(smem_addr(smem_dst)),
      "l"(tmap), "r"(smem_addr(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *smem_dst, const void *tmap, int x, int y, int z, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], "
      "[%2];" ::"r"(smem_addr(smem_dst)),
      "l"(tmap), "r"(smem_addr(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// im2col-mode load over an NHWC tensor map (dims C, W, H, N): `pixelsPerColumn` consecutive output
// positions starting at the window origin (w, h) of image n, walking W, then H, then N inside the
// map's bounding box, `channelsPerPixel` channels from c each, read at the filter-tap offset
// (off_w, off_h) from every window origin. Positions outside the image read as zero.
__device__ __forceinline__ void tma_load_im2col_4d(void *smem_dst, const void *tmap, int c, int w, int h, int n,
                                                   uint16_t off_w, uint16_t off_h, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, "
      "%6}], [%2], {%7, %8};" ::"r"(smem_addr(smem_dst)),
      "l"(tmap), "r"(smem_addr(bar)), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h)
      : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const void *tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---- tcgen05: tensor memory and MMA ------------------------------------------------------------
// Allocates `ncols` (power of two >= 32) TMEM columns; the base address lands in *smem_result.
// Warp-collective (all 32 lanes execute it).
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; one thread issues it for the whole CTA.
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on `bar` once all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
               : "memory");
}
// 32 lanes x 32 columns of 32-bit accumulators: thread t of the warp gets lane (base_lane + t),
// register j holds column (base_col + j). The warp may only touch lanes 32*(warp_id % 4) .. +31.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, "
      "%23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// The same for 16 columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- CTA pairs: a cluster of two CTAs on neighbouring SMs driving one tcgen05.mma (cta_group::2) --
// The even CTA of the pair (cluster rank 0) issues the instructions; they read A from each CTA's
// own shared memory (128 rows each, M = 256), the first half of B's rows from rank 0 and the second
// half from rank 1, and leave each CTA's 128 rows of D in that CTA's tensor memory. Nothing below is
// a multicast: every load writes the issuing CTA's own shared memory, and a commit names one barrier.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The shared::cluster address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
// Cluster-wide rendezvous of all threads (hardware barrier; a CTA that has exited counts as arrived).
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrives on an mbarrier given by its shared::cluster address (this CTA's or the other's).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_caddr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_caddr) : "memory");
}
// Tile-mode load into this CTA's shared memory whose byte count is credited to the mbarrier at
// `bar_caddr`, which may live in the other CTA of the pair.
__device__ __forceinline__ void tma_load_3d_pair(void *smem_dst, const void *tmap, int x, int y, int z,
                                                 uint32_t bar_caddr) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, "
      "%5}], [%2];" ::"r"(smem_addr(smem_dst)),
      "l"(tmap), "r"(bar_caddr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_im2col_4d_pair(void *smem_dst, const void *tmap, int c, int w, int h, int n,
                                                        uint16_t off_w, uint16_t off_h, uint32_t bar_caddr) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.im2col.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(smem_addr(smem_dst)),
      "l"(tmap), "r"(bar_caddr), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h)
      : "memory");
}
// Tensor-memory allocation for the pair: one warp of EACH CTA executes it (same warp index, same
// shared-memory offset for the result), and likewise the release.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_tf32_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier at `bar_caddr` (either CTA's) once the pair's MMAs issued so far are done.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar_caddr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_caddr)
               : "memory");
}


// ---- one k-block of MMAs as one run of instructions ----------------------------------------------
// The thread that issues the MMAs is a serial bottleneck: an mbarrier poll comes back after about
// 100 cycles, a tcgen05.mma takes about 60 to issue and a commit about 90, against 512 (bf16) or 768
// (3xTF32) cycles of tensor work per k-block. These helpers keep that thread's path short: the four
// k-slices of a stage are issued from descriptors that only step an immediate, the commit that frees
// the stage follows at once, and the poll of the NEXT stage's "full" barrier (non-blocking
// test_wait) is started first and its answer read last, so that its latency passes behind the
// issue. Returns 1 if the next stage was seen complete.
//   CG: "1" or "2" (cta_group); SA / SB: descriptor step between k-slices (bytes >> 4).
// The second commit of a pair names the other CTA's barrier; empty_peer is ignored when CG is 1.

template <bool PAIR, int SA, int SB>
__device__ __forceinline__ uint32_t kblock_f16(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc_first,
                                               uint32_t empty_bar, uint32_t empty_peer, uint32_t next_full,
                                               uint32_t next_parity) {
  uint32_t ready;
#define B200_KB_F16(CG, SECOND_COMMIT)                                                                   \
  asm volatile(                                                                                        \
      "{\n\t"                                                                                          \
      ".reg .pred pn, pa, p1;\n\t"                                                                     \
      ".reg .b64 a1, b1;\n\t"                                                                          \
      "setp.ne.b32 pa, %4, 0;\n\t"                                                                     \
      "setp.eq.b32 p1, %4, %4;\n\t"                                                                    \
      "mbarrier.test_wait.parity.shared::cta.b64 pn, [%7], %8;\n\t"                                    \
      "tcgen05.mma.cta_group::" CG ".kind::f16 [%1], %2, %3, %5, pa;\n\t"                              \
      "add.s64 a1, %2, %9;\n\t"                                                                        \
      "add.s64 b1, %3, %10;\n\t"                                                                       \
      "tcgen05.mma.cta_group::" CG ".kind::f16 [%1], a1, b1, %5, p1;\n\t"                              \
      "add.s64 a1, a1, %9;\n\t"                                                                        \
      "add.s64 b1, b1, %10;\n\t"                                                                       \
      "tcgen05.mma.cta_group::" CG ".kind::f16 [%1], a1, b1, %5, p1;\n\t"                              \
      "add.s64 a1, a1, %9;\n\t"                                                                        \
      "add.s64 b1, b1, %10;\n\t"                                                                       \
      "tcgen05.mma.cta_group::" CG ".kind::f16 [%1], a1, b1, %5, p1;\n\t"                              \
      "tcgen05.commit.cta_group::" CG ".mbarrier::arrive::one.shared::cluster.b64 [%6];\n\t" SECOND_COMMIT \
      "selp.u32 %0, 1, 0, pn;\n\t"                                                                     \
      "}"                                                                                              \
      : "=r"(ready)                                                                                    \
      : "r"(d), "l"(a), "l"(b), "r"(acc_first), "r"(idesc), "r"(empty_bar), "r"(next_full), "r"(next_parity),  \
        "n"(SA), "n"(SB), "r"(empty_peer)                                                              \
      : "memory")
  if (PAIR)
    B200_KB_F16("2", "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%11];\n\t");
  else
    B200_KB_F16("1", "");
#undef B200_KB_F16
  return ready;
}

// 3xTF32: per k-slice a_head x b_wide (width 2 BN, into d_main) and a_tail x b_narrow (width BN,
// into d_tail, always accumulating).
template <bool PAIR, int SA, int SB>
__device__ __forceinline__ uint32_t kblock_tf32x3(uint32_t d_main, uint32_t d_tail, uint64_t a_head, uint64_t a_tail,
                                                  uint64_t b_wide, uint64_t b_narrow, uint32_t idesc_wide,
                                                  uint32_t idesc, uint32_t acc_first, uint32_t empty_bar,
                                                  uint32_t empty_peer, uint32_t next_full, uint32_t next_parity) {
  uint32_t ready;
#define B200_KB_STEP(CG)                                                       \
  "add.s64 ah, ah, %14;\n\t"                                                   \
  "add.s64 al, al, %14;\n\t"                                                   \
  "add.s64 bw, bw, %15;\n\t"                                                   \
  "add.s64 bn, bn, %15;\n\t"                                                   \
  "tcgen05.mma.cta_group::" CG ".kind::tf32 [%1], ah, bw, %7, p1;\n\t"         \
  "tcgen05.mma.cta_group::" CG ".kind::tf32 [%2], al, bn, %8, p1;\n\t"
#define B200_KB_TF32(CG, SECOND_COMMIT)                                                                  \
  asm volatile(                                                                                        \
      "{\n\t"                                                                                          \
      ".reg .pred pn, pa, p1;\n\t"                                                                     \
      ".reg .b64 ah, al, bw, bn;\n\t"                                                                  \
      "setp.ne.b32 pa, %9, 0;\n\t"                                                                     \
      "setp.eq.b32 p1, %9, %9;\n\t"                                                                    \
      "mbarrier.test_wait.parity.shared::cta.b64 pn, [%12], %13;\n\t"                                  \
      "tcgen05.mma.cta_group::" CG ".kind::tf32 [%1], %3, %5, %7, pa;\n\t"                             \
      "tcgen05.mma.cta_group::" CG ".kind::tf32 [%2], %4, %6, %8, p1;\n\t"                             \
      "mov.b64 ah, %3;\n\t"                                                                            \
      "mov.b64 al, %4;\n\t"                                                                            \
      "mov.b64 bw, %5;\n\t"                                                                            \
      "mov.b64 bn, %6;\n\t" B200_KB_STEP(CG) B200_KB_STEP(CG) B200_KB_STEP(CG)                         \
      "tcgen05.commit.cta_group::" CG ".mbarrier::arrive::one.shared::cluster.b64 [%10];\n\t" SECOND_COMMIT \
      "selp.u32 %0, 1, 0, pn;\n\t"                                                                     \
      "}"                                                                                              \
      : "=r"(ready)                                                                                    \
      : "r"(d_main), "r"(d_tail), "l"(a_head), "l"(a_tail), "l"(b_wide), "l"(b_narrow), "r"(idesc_wide),      \
        "r"(idesc), "r"(acc_first), "r"(empty_bar), "r"(empty_peer), "r"(next_full), "r"(next_parity),       \
        "n"(SA), "n"(SB)                                                                               \
      : "memory")
  if (PAIR)
    B200_KB_TF32("2", "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%11];\n\t");
  else
    B200_KB_TF32("1", "");
#undef B200_KB_TF32
#undef B200_KB_STEP
  return ready;
}

}  // namespace ptx
}  // namespace b200
