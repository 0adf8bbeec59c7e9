// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the attention
// kernel uses: mbarriers, TMA tiled loads, tensor memory (TMEM) management,
// tcgen05 MMA issue / commit and TMEM <-> register moves, plus the 64-bit
// shared-memory matrix descriptor and the 32-bit instruction descriptor.
//
// Every wait in this file is bounded in wall-clock time: a role that gives up
// records a status code and returns, it never spins forever.
#pragma once
#include <cstdint>
#include <cuda.h>

namespace rsfa {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
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

// Status codes a kernel can leave in its status word (0 = fine).
enum : int {
  kStatusOk = 0,
  kStatusWaitExpired = 1,  // a bounded wait ran out; low bits say which role
};

// try_wait with an explicit suspend-time hint: the hardware may park the thread for up to
// `hint_ns` nanoseconds (waking it when the phase completes), so a waiting warp does not take
// issue slots from the warps that are computing on the same scheduler.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}

// Longest time the hardware may park a waiting thread per try (it is woken when the phase completes).
constexpr uint32_t kWaitHintNs = 20000;

// Bounded wait.  `abort_flag` lives in shared memory and is shared by all roles
// of the CTA: the first role whose wait runs out sets it, every other role sees
// it at its next poll and leaves as well.  Returns false when the caller must
// stop.  `tag` identifies the waiting site in the status word.
__device__ __forceinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                               uint64_t limit_ns, int tag) {
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait_hint(bar, parity, kWaitHintNs)) return true;
    if ((++spins & 0x3u) == 0) {   // abort flag and clock every fourth try
      if (*abort_flag != 0) return false;
      if (global_timer_ns() - t0 > limit_ns) {
        *abort_flag = (kStatusWaitExpired << 16) | (tag & 0xffff);
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          uint64_t limit_ns, int tag) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, limit_ns, tag);
}

// The same for a role that all 32 lanes of a warp run together (MMA issuers, softmax and epilogue
// warps): every lane polls, and the warp must leave the wait as one.  The warp is brought together
// first (__syncwarp: cheap when it is converged already, which it is in practice); the first try is
// then a single instruction executed by all 32 lanes at once, so every lane sees the same answer and no
// vote is needed when the phase has completed already - the usual case for the MMA warps, whose waits
// pace the whole CTA (the vote and the branch on its result cost them 20 to 30 clk per wait, 1.3 % of a
// step).  Only the slow path, in which lanes loop on their own, ends in a vote.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                               uint64_t limit_ns, int tag) {
  __syncwarp();
  if (mbar_try_wait(bar, parity)) return true;
  const bool r = mbar_wait_slow(bar, parity, abort_flag, limit_ns, tag);
  return __all_sync(0xffffffffu, r) != 0;
}

// ------------------------------------------------- programmatic dependent launch
// A kernel launched with programmatic stream serialisation may start while the kernel in front of
// it on the stream is still running.  griddep_wait() returns once that kernel has completed and its
// writes are visible: nothing a predecessor may have written (inputs, queue counters, outputs it
// still reads) is touched before it.  griddep_launch_dependents() lets the kernel behind this one
// start its own set-up as soon as every CTA of this grid has called it or exited.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ----------------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// One tiled 4-D box, global -> this CTA's shared memory, completion counted in
// bytes on `bar`.  c0 is the innermost coordinate (must be a multiple of 8 for
// 16-bit elements).
__device__ __forceinline__ void tma_load_4d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// The same box on its way into L2 only (no shared-memory destination, no completion to wait for).
__device__ __forceinline__ void tma_prefetch_l2_4d(const CUtensorMap* map, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(map), "r"(c0),
               "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

// One tiled 4-D box, this CTA's shared memory -> global (rows outside the tensor are clipped).
// Completion is tracked per thread in bulk groups.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t smem_src, int c0, int c1, int c2,
                                             int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
               "r"(smem_src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until the bulk stores of this thread have finished READING shared memory (it may be reused),
// except that the newest kPending store groups may still be reading.
template <int kPending>
__device__ __forceinline__ void tma_store_wait_read_but() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
// Wait until the bulk stores of this thread are complete.
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// ---------------------------------------------------------------------- TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result),
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
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// Make `bar` complete once every MMA this thread issued so far has finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}


// 128 rows x 256 bits (eight 32-bit columns per lane) from shared memory, described like an MMA
// operand, into tensor memory at [t_dst]; runs in order with the MMAs issued by the same thread and
// is covered by the next tcgen05.commit.
__device__ __forceinline__ void tmem_cp_128x256b(uint32_t t_dst, uint64_t s_desc) {
  asm volatile("tcgen05.cp.cta_group::1.128x256b [%0], %1;" ::"r"(t_dst), "l"(s_desc) : "memory");
}

// One lane of a converged warp.  The MMA warp keeps its control flow and operand arithmetic
// warp-uniform (so descriptors live in uniform registers) and elects a lane only for the
// instruction itself; with a full mask the elected lane is the same every time, which is what
// lets tcgen05.commit track the MMAs issued before it.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void umma_commit_elect(uint32_t bar) {
  if (elect_one()) umma_commit(bar);
}
// Two commits from one elected region (0 = no barrier): an elect.sync and a branch per instruction
// cost the issuing warp more than the instruction itself.
__device__ __forceinline__ void umma_commit2_elect(uint32_t bar_a, uint32_t bar_b) {
  if (elect_one()) {
    if (bar_a != 0) umma_commit(bar_a);
    if (bar_b != 0) umma_commit(bar_b);
  }
  __syncwarp();
}

// Shared-memory matrix descriptor, 128-byte swizzle (the layout TMA writes with
// CU_TENSOR_MAP_SWIZZLE_128B: rows of 128 bytes, 8-row atoms of 1024 bytes).
//   bits  0..13  start address >> 4        bits 16..29  leading byte offset >> 4
//   bits 32..45  stride byte offset >> 4   bits 46..47  descriptor version (1)
//   bits 61..63  layout type (2 = 128-byte swizzle)
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
  return static_cast<uint64_t>((saddr & 0x3ffffu) >> 4) |
         (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16) |
         (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor for kind::f16 with fp32 accumulation.
//   bits 4..5 D format (1 = f32), 7..9 A format, 10..12 B format (0 = f16, 1 = bf16),
//   bit 15 A major, bit 16 B major (0 = K-major, 1 = MN-major),
//   bits 17..22 N >> 3, bits 24..28 M >> 4.
__host__ __device__ constexpr uint32_t make_idesc_f16(int m, int n, bool bf16, bool a_mn_major,
                                                      bool b_mn_major) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) |
         ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// TMEM <-> registers, "32 lanes x 32 bit" shape: lane i of the warp moves N
// consecutive 32-bit columns of TMEM lane (base lane + i).  A warp may only
// touch the 32 lanes starting at 32 * (warp index % 4).
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr));
}

__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
               :
               : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
               : "memory");
}

// The compiler does not know that the registers written by tcgen05.ld are only
// valid after tcgen05.wait::ld.  Passing them through an empty asm placed after
// the wait pins every later use behind it.

__device__ __forceinline__ void reg_fence_x32(uint32_t (&r)[32]) {
  asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]) :: "memory");
}

}  // namespace rsfa
