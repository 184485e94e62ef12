// Thin wrappers over the sm_100a PTX used by the tensor-core attention kernel: mbarriers with
// bounded waits, TMA tile loads, tensor-memory allocation / loads, tcgen05 integer MMAs and the
// shared-memory matrix descriptors they take.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace risa_b200 {
namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier ------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// Non-blocking test of a phase (no suspend): used for the fast path and by the issue warps, whose
// waits sit on the critical path of every tile.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
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
// Same with a suspend-time hint: the hardware may park the thread until the phase completes (or the
// time passes) instead of spinning through issue slots that the working warps of the same
// scheduler need.  Used by the softmax and correction groups when a first test fails.
constexpr uint32_t kSuspendHintNs = 2000;
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
      : "memory");
  return ok != 0;
}

// Every wait in the kernel is bounded: after the limit without progress the waiter records the
// site and reports failure, so a protocol bug ends the kernel instead of hanging the GPU.  Two
// words take the record.  `gave_up` is a word in the CTA's own shared memory (zeroed before the
// first wait): the other waiters of the same CTA poll it and leave as soon as one of them has given
// up; it dies with the CTA, so one expired wait never poisons a later launch.  g_wait_status is the
// process-wide report the host reads (first failing site since the last query).
constexpr uint64_t kWaitLimitNs = 2000000000ull;
__device__ unsigned int g_wait_status;

__device__ __forceinline__ uint32_t gave_up_read(uint32_t gave_up) {
  uint32_t v;
  asm volatile("ld.volatile.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(gave_up) : "memory");
  return v;
}

template <bool SPIN = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t gave_up,
                                          unsigned int site, uint64_t limit_ns = kWaitLimitNs) {
  if (mbar_test(bar, parity)) return true;
  const uint64_t start = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < (SPIN ? 256 : 16); ++i)
      if (SPIN ? mbar_test(bar, parity) : mbar_try_wait(bar, parity)) return true;
    if (gave_up_read(gave_up) != 0) return false;  // another waiter of this CTA gave up
    if (global_timer_ns() - start > limit_ns) {
      atomicCAS(&g_wait_status, 0u, site);
      asm volatile("st.volatile.shared::cta.u32 [%0], %1;" ::"r"(gave_up), "r"(site) : "memory");
      return false;
    }
  }
}

// Wait used while draining after a failure: ignores the give-up word (it is set by then) and only
// stops on completion or on the limit.
__device__ __forceinline__ bool mbar_drain(uint32_t bar, uint32_t parity,
                                           uint64_t limit_ns = kWaitLimitNs) {
  const uint64_t start = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - start > limit_ns) return false;
  }
}

// Waits for several phases at once: the tests are issued back to back so their latencies overlap
// (in steady state all of them are already complete), then any that failed is waited for in turn.
template <bool SPIN = false>
__device__ __forceinline__ bool mbar_wait2(uint32_t b0, uint32_t p0, uint32_t b1, uint32_t p1,
                                           uint32_t gave_up, unsigned int site) {
  const bool r0 = mbar_test(b0, p0), r1 = mbar_test(b1, p1);
  if (r0 & r1) return true;
  return (r0 || mbar_wait<SPIN>(b0, p0, gave_up, site)) &&
         (r1 || mbar_wait<SPIN>(b1, p1, gave_up, site + 1));
}
template <bool SPIN = false>
__device__ __forceinline__ bool mbar_wait3(uint32_t b0, uint32_t p0, uint32_t b1, uint32_t p1,
                                           uint32_t b2, uint32_t p2, uint32_t gave_up,
                                           unsigned int site) {
  const bool r0 = mbar_test(b0, p0), r1 = mbar_test(b1, p1), r2 = mbar_test(b2, p2);
  if (r0 & r1 & r2) return true;
  return (r0 || mbar_wait<SPIN>(b0, p0, gave_up, site)) &&
         (r1 || mbar_wait<SPIN>(b1, p1, gave_up, site + 1)) &&
         (r2 || mbar_wait<SPIN>(b2, p2, gave_up, site + 2));
}

// ---- proxies / fences --------------------------------------------------------------------------
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- TMA ------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// Untiled bulk copy global -> this CTA's shared memory (both addresses 16-byte aligned, `bytes` a
// multiple of 16), completing `bytes` on the mbarrier; no multicast.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar)
      : "memory");
}
// Orders this thread's earlier accesses through the generic proxy (and those it has observed)
// with later accesses through the async proxy, in every state space.
__device__ __forceinline__ void fence_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
// Asks L2 to fetch `bytes` (a multiple of 16) starting at a 16-byte aligned global address; one
// thread, no destination, no completion to wait for.
__device__ __forceinline__ void l2_prefetch_run(const void* address, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(address), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tensor memory --------------------------------------------------------------------------------
// Whole-warp calls.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_result),
               "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address),
               "r"(columns)
               : "memory");
}

// 32 lanes x 32 columns of 32-bit cells: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_load32(uint32_t address, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(address)
      : "memory");
}
// 32 lanes x 16 columns.
__device__ __forceinline__ void tmem_load16(uint32_t address, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(address)
      : "memory");
}
// Store counterpart of tmem_load32: thread i of the warp writes 32 columns of row (lane base + i).
__device__ __forceinline__ void tmem_store32(uint32_t address, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(address), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_store_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_load_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// The registers a tcgen05.ld names are undefined until the wait above, but the wait does not
// mention them, so the compiler sees no dependency and may schedule their readers in front of it.
// This empty volatile statement, placed right after the wait (volatile statements keep their
// order), takes the registers in and out: every later reader now depends on it.  No instruction.
template <int N>
__device__ __forceinline__ void tmem_regs_ready(uint32_t* r) {
  static_assert(N % 16 == 0, "register block");
#pragma unroll
  for (int i = 0; i < N; i += 16)
    asm volatile(""
                 : "+r"(r[i]), "+r"(r[i + 1]), "+r"(r[i + 2]), "+r"(r[i + 3]), "+r"(r[i + 4]),
                   "+r"(r[i + 5]), "+r"(r[i + 6]), "+r"(r[i + 7]), "+r"(r[i + 8]), "+r"(r[i + 9]),
                   "+r"(r[i + 10]), "+r"(r[i + 11]), "+r"(r[i + 12]), "+r"(r[i + 13]),
                   "+r"(r[i + 14]), "+r"(r[i + 15]));
}

// ---- register budget per warpgroup (all four warps of an aligned group of 128 threads) ----------
template <int N> __device__ __forceinline__ void regs_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N> __device__ __forceinline__ void regs_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

// ---- MMA -------------------------------------------------------------------------------------------
// Shared-memory operand descriptor for a K-major tile whose rows are 128 bytes wide and stored with
// the 128-byte swizzle (what a TMA box of 128 bytes x rows produces): 8-row groups are 1024 bytes
// apart (stride byte offset), descriptor version 1, layout type 2 (SWIZZLE_128B).  Advancing along
// K by 32 bytes adds 2 to the (address >> 4) field.
__device__ __forceinline__ uint64_t smem_desc_k128(uint32_t smem_address) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_address & 0x3ffffu) >> 4);  // start address
  desc |= static_cast<uint64_t>(1) << 16;                         // leading byte offset (unused)
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;                 // stride byte offset
  desc |= static_cast<uint64_t>(1) << 46;                         // descriptor version
  desc |= static_cast<uint64_t>(2) << 61;                         // SWIZZLE_128B
  return desc;
}

// Same for tiles whose rows are ROW_BYTES wide: 128 -> 128-byte swizzle (8-row groups 1024 bytes
// apart), 64 -> 64-byte swizzle (layout type 4, 8-row groups 512 bytes apart), which is what a TMA
// box of that inner width with the matching swizzle mode produces.
template <int ROW_BYTES>
__device__ __forceinline__ uint64_t smem_desc_kmajor(uint32_t smem_address) {
  static_assert(ROW_BYTES == 64 || ROW_BYTES == 128, "row width");
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_address & 0x3ffffu) >> 4);
  desc |= static_cast<uint64_t>(1) << 16;
  desc |= static_cast<uint64_t>((8 * ROW_BYTES) >> 4) << 32;
  desc |= static_cast<uint64_t>(1) << 46;
  desc |= static_cast<uint64_t>(ROW_BYTES == 128 ? 2 : 4) << 61;
  return desc;
}

// Instruction descriptor of kind::i8: S32 accumulator, A and B K-major, M = 128.
__host__ __device__ constexpr uint32_t idesc_i8(bool a_signed, bool b_signed, int n) {
  return (2u << 4) | ((a_signed ? 1u : 0u) << 7) | ((b_signed ? 1u : 0u) << 10) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}

// One thread issues; D[tmem] (+)= A[smem] * B[smem]^T, 128 x N x 32.
__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

}  // namespace tc
}  // namespace risa_b200
