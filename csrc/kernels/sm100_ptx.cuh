// Thin inline-PTX wrappers for the Blackwell (sm_100a) execution model:
// mbarrier, TMA (cp.async.bulk.tensor, never with a cluster-wide broadcast), tensor memory
// (TMEM) allocation, tcgen05.mma / tcgen05.commit / tcgen05.ld.
//
// Every wait in this file is bounded: it polls, and after a clock budget it
// raises a CTA-wide abort flag instead of spinning forever, so that a logic
// error surfaces as a status code on the host and never as a hung GPU.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fdb {

// Clock budget of one bounded wait (~1.5 s at 1.9 GHz).
constexpr long long kWaitClockLimit = 3000000000LL;

// Status word values written by kernels (0 = ok).
enum KernelStatus : int {
  kStatusOk = 0,
  kStatusTimeoutProducer = 1,
  kStatusTimeoutMma = 2,
  kStatusTimeoutEpilogue = 3,
  kStatusTimeoutPeer = 4,
  kStatusBadShape = 5,
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
  uint32_t l;
  asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
  return l;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait on an mbarrier phase. Returns false when the CTA is aborting or
// the clock budget ran out (then it raises *abort_flag with `code`).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int code) {
  long long t0 = -1;
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 0xff) == 0) {
      if (*abort_flag) return false;
      long long now = clock64();
      if (t0 < 0) {
        t0 = now;
      } else if (now - t0 > kWaitClockLimit) {
        *abort_flag = code;
        return false;
      }
    }
  }
}

// Same wait executed by a fully converged warp; the verdict is made warp-uniform so that the
// lanes never part ways before a later elect.sync / __syncwarp.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                               int code) {
  const bool ok = mbar_wait(bar, parity, abort_flag, code);
  return __all_sync(0xffffffffu, ok) != 0;
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tensormap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, uint32_t bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1), "r"(c2),
      "r"(c3)
      : "memory");
}

// Untiled bulk copies (no cluster broadcast): global -> this CTA's shared memory with mbarrier completion, and
// shared memory -> global as a bulk group. Addresses and sizes are multiples of 16 bytes.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(reinterpret_cast<uint64_t>(dst)),
               "r"(src_smem), "r"(bytes)
               : "memory");
}

// ---------------------------------------------------------------- TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; kind::f16 covers fp16 and bf16 inputs.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One elected lane of a fully converged warp (the same lane every time while all 32 are active).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "elect.sync _|P, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// The four K=16 steps of one 64-element K block in a single instruction group: the descriptors of
// steps 1..3 are the first one advanced by 32 bytes each (+2 in the 16-byte address field). Keeping
// this in one asm block keeps the issuing thread's instruction count per MMA small, which is what
// bounds the rate for narrow tiles.
__device__ __forceinline__ void umma_f16_kblock(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                                uint32_t idesc, uint32_t accumulate_first) {
  asm volatile(
      "{\n"
      ".reg .pred p0, p1;\n"
      ".reg .b64 a1, a2, a3, b1, b2, b3;\n"
      "setp.ne.b32 p0, %4, 0;\n"
      "setp.eq.u32 p1, %3, %3;\n"
      "add.s64 a1, %1, 2;\n"
      "add.s64 b1, %2, 2;\n"
      "add.s64 a2, %1, 4;\n"
      "add.s64 b2, %2, 4;\n"
      "add.s64 a3, %1, 6;\n"
      "add.s64 b3, %2, 6;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, p1;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, p1;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, p1;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate_first)
      : "memory");
}

// The same K block with only the first `nsteps` (1..4) K = 16 steps issued: the tail slab of a
// reduction whose length is not a multiple of 64 skips the steps that would multiply zero padding.
__device__ __forceinline__ void umma_f16_ksteps(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate_first, uint32_t nsteps) {
  asm volatile(
      "{\n"
      ".reg .pred p0, p1, q1, q2, q3;\n"
      ".reg .b64 a1, a2, a3, b1, b2, b3;\n"
      "setp.ne.b32 p0, %4, 0;\n"
      "setp.eq.u32 p1, %3, %3;\n"
      "setp.gt.u32 q1, %5, 1;\n"
      "setp.gt.u32 q2, %5, 2;\n"
      "setp.gt.u32 q3, %5, 3;\n"
      "add.s64 a1, %1, 2;\n"
      "add.s64 b1, %2, 2;\n"
      "add.s64 a2, %1, 4;\n"
      "add.s64 b2, %2, 4;\n"
      "add.s64 a3, %1, 6;\n"
      "add.s64 b3, %2, 6;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p0;\n"
      "@q1 tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, p1;\n"
      "@q2 tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, p1;\n"
      "@q3 tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, p1;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate_first), "r"(nsteps)
      : "memory");
}

// kind::f8f6f4: e4m3 / e5m2 inputs, fp32 accumulate, K = 32 per instruction.
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One K block of e4m3 operands: up to four K = 32 steps (32 bytes each, so the descriptors advance
// exactly like the 16-bit form), the first `nsteps` issued.
__device__ __forceinline__ void umma_f8_ksteps(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate_first, uint32_t nsteps) {
  asm volatile(
      "{\n"
      ".reg .pred p0, p1, q1, q2, q3;\n"
      ".reg .b64 a1, a2, a3, b1, b2, b3;\n"
      "setp.ne.b32 p0, %4, 0;\n"
      "setp.eq.u32 p1, %3, %3;\n"
      "setp.gt.u32 q1, %5, 1;\n"
      "setp.gt.u32 q2, %5, 2;\n"
      "setp.gt.u32 q3, %5, 3;\n"
      "add.s64 a1, %1, 2;\n"
      "add.s64 b1, %2, 2;\n"
      "add.s64 a2, %1, 4;\n"
      "add.s64 b2, %2, 4;\n"
      "add.s64 a3, %1, 6;\n"
      "add.s64 b3, %2, 6;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p0;\n"
      "@q1 tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a1, b1, %3, p1;\n"
      "@q2 tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a2, b2, %3, p1;\n"
      "@q3 tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a3, b3, %3, p1;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate_first), "r"(nsteps)
      : "memory");
}

// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread retired.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread t of the warp receives lane (base+t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// Same wait, but tied to the destination registers of an earlier tmem_ld_32x32 so the
// compiler cannot move a use of those registers above the wait.
__device__ __forceinline__ void tmem_ld_wait_dep(uint32_t (&v)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]),
                 "+r"(v[7]), "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]),
                 "+r"(v[13]), "+r"(v[14]), "+r"(v[15]), "+r"(v[16]), "+r"(v[17]), "+r"(v[18]),
                 "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]), "+r"(v[24]),
                 "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]),
                 "+r"(v[31])
               :
               : "memory");
}

// ---------------------------------------------------------------- CTA pairs (cta_group::2)
// Two CTAs of a cluster (ranks 2k and 2k+1) act as one MMA unit: each stages its own 128 rows of A and
// half of the B tile, the even CTA issues tcgen05.mma.cta_group::2 (M = 256), and each CTA's tensor
// memory receives the accumulator of its own 128 rows. Every B byte then feeds twice the rows, which
// halves the weight traffic per SM. Loads use the cta_group::2 form WITHOUT any cluster broadcast: each
// CTA fetches its own bytes from global memory; only the completion signal goes to the even CTA's
// mbarrier (same shared-memory offset, CTA-rank bit cleared).
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the mbarrier at the same shared-memory offset in CTA `rank` of the cluster. Relaxed: the
// arrival hands back tensor memory whose reads this thread has already waited for (tcgen05.wait::ld); no
// data written through the generic proxy travels with it, and a release here would first drain the
// thread's earlier shared-memory stores, which was measured at over a microsecond per tile.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar, uint32_t rank) {
  asm volatile(
      "{\n"
      ".reg .b32 ra;\n"
      "mapa.shared::cluster.u32 ra, %0, %1;\n"
      "mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [ra];\n"
      "}\n" ::"r"(bar), "r"(rank)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* tmap, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar & kPeerBitMask), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1, int c2,
                                                 int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar & kPeerBitMask), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrive (once every MMA issued so far by this thread has retired) on the mbarrier at this offset in BOTH CTAs.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          bar & kPeerBitMask),
      "h"(static_cast<uint16_t>(3))
      : "memory");
}
// K block of up to four K = 16 steps issued for the CTA pair (M = 256 over both CTAs).
__device__ __forceinline__ void umma_f16_ksteps_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                     uint32_t accumulate_first, uint32_t nsteps) {
  asm volatile(
      "{\n"
      ".reg .pred p0, p1, q1, q2, q3;\n"
      ".reg .b64 a1, a2, a3, b1, b2, b3;\n"
      "setp.ne.b32 p0, %4, 0;\n"
      "setp.eq.u32 p1, %3, %3;\n"
      "setp.gt.u32 q1, %5, 1;\n"
      "setp.gt.u32 q2, %5, 2;\n"
      "setp.gt.u32 q3, %5, 3;\n"
      "add.s64 a1, %1, 2;\n"
      "add.s64 b1, %2, 2;\n"
      "add.s64 a2, %1, 4;\n"
      "add.s64 b2, %2, 4;\n"
      "add.s64 a3, %1, 6;\n"
      "add.s64 b3, %2, 6;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p0;\n"
      "@q1 tcgen05.mma.cta_group::2.kind::f16 [%0], a1, b1, %3, p1;\n"
      "@q2 tcgen05.mma.cta_group::2.kind::f16 [%0], a2, b2, %3, p1;\n"
      "@q3 tcgen05.mma.cta_group::2.kind::f16 [%0], a3, b3, %3, p1;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate_first), "r"(nsteps)
      : "memory");
}

// The same K block for e4m3 operands (K = 32 per step) on a CTA pair.
__device__ __forceinline__ void umma_f8_ksteps_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                    uint32_t accumulate_first, uint32_t nsteps) {
  asm volatile(
      "{\n"
      ".reg .pred p0, p1, q1, q2, q3;\n"
      ".reg .b64 a1, a2, a3, b1, b2, b3;\n"
      "setp.ne.b32 p0, %4, 0;\n"
      "setp.eq.u32 p1, %3, %3;\n"
      "setp.gt.u32 q1, %5, 1;\n"
      "setp.gt.u32 q2, %5, 2;\n"
      "setp.gt.u32 q3, %5, 3;\n"
      "add.s64 a1, %1, 2;\n"
      "add.s64 b1, %2, 2;\n"
      "add.s64 a2, %1, 4;\n"
      "add.s64 b2, %2, 4;\n"
      "add.s64 a3, %1, 6;\n"
      "add.s64 b3, %2, 6;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p0;\n"
      "@q1 tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], a1, b1, %3, p1;\n"
      "@q2 tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], a2, b2, %3, p1;\n"
      "@q3 tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], a3, b3, %3, p1;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate_first), "r"(nsteps)
      : "memory");
}

// ---------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor for a K-major operand tile whose rows are
// `row_bytes` (32/64/128) wide and stored with the matching TMA swizzle.
// Groups of 8 rows are `8*row_bytes` apart (the stride byte offset).
__device__ __forceinline__ uint64_t make_kmajor_desc(uint32_t smem_addr, uint32_t row_bytes) {
  uint64_t layout = row_bytes == 128 ? 2ull : (row_bytes == 64 ? 4ull : 6ull);
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);          // start address
  d |= (uint64_t)1 << 16;                               // leading byte offset (unused when swizzled)
  d |= (uint64_t)((8u * row_bytes) >> 4) << 32;         // stride byte offset
  d |= (uint64_t)1 << 46;                               // descriptor version (Blackwell)
  d |= layout << 61;                                    // swizzle mode
  return d;
}

// Instruction descriptor: fp32 accumulate, A and B both K-major, dense.
// ab_format: kind::f16 -> 0 fp16, 1 bf16 ; kind::f8f6f4 -> 0 e4m3, 1 e5m2.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t ab_format, uint32_t m, uint32_t n) {
  return (1u << 4) | (ab_format << 7) | (ab_format << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

}  // namespace fdb
