// Device-side building blocks for the sm_100a kernels of this package.
//
// Everything a Blackwell tensor-core kernel needs that is not arithmetic lives here:
//   * mbarrier primitives with a *bounded* wait (a wait that runs out records an error
//     word and lets the kernel drain instead of hanging the GPU),
//   * TMA (cp.async.bulk.tensor) tile loads and stores WITHOUT cluster multicast,
//   * tcgen05 tensor-memory allocation, MMA issue, commit and accumulator read-back,
//   * shared-memory matrix descriptors and instruction descriptors for bf16 UMMA,
//   * the 128-byte swizzle address map used when threads build an operand tile by hand.
//
// No kernel in this package issues a TMA load with cluster multicast; tiles that several
// CTAs need are read by each CTA from L2.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ubm {

// ----------------------------------------------------------------------------------------
// Error status written by kernels, read by the host after a synchronisation point.
// code 0 = ok. The first failing thread wins (atomicCAS on code).
struct KernelStatus {
  unsigned int code;   // 0 ok, 1 = mbarrier wait ran out, 2 = peer flag wait ran out, 3 = bad argument
  unsigned int where;  // site id of the wait that gave up
  unsigned int block;  // blockIdx.x of the reporter
  unsigned int aux;    // site-specific (stage / tile / rank)
};

constexpr unsigned int kErrBarrierTimeout = 1;
constexpr unsigned int kErrPeerTimeout = 2;
constexpr unsigned int kErrBadArgument = 3;

// Wall-clock limits of device-side waits (nanoseconds of %globaltimer).
constexpr unsigned long long kBarrierLimitNs = 1500ull * 1000ull * 1000ull;  // local pipeline waits
constexpr unsigned long long kPeerLimitNs = 4000ull * 1000ull * 1000ull;     // waits on another GPU
constexpr uint32_t kWaitHintNs = 20000u;   // suspend-time hint of a barrier wait (the thread wakes when the phase completes)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31u; }

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
      "elect.sync _|P1, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P1;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------------------
// mbarrier

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
  // makes barrier initialisation visible to the async proxy (TMA, tcgen05.commit)
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar_addr, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar_addr), "r"(parity)
      : "memory");
  return ok != 0;
}

// The same test with a suspend-time hint: the thread may sleep in hardware up to `hint_ns` and is woken when the
// phase completes, so a long wait costs a handful of instructions instead of a spin loop's worth of issue slots
// (measured in the attention kernel: spinning role warps took about an eighth of all issued instructions).
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar_addr, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar_addr), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}

// Shared by all threads of a CTA: `abort` turns every later wait into a no-op so that the
// CTA drains in bounded time after one wait has run out.
struct WaitScope {
  volatile uint32_t* abort;  // in shared memory, zero-initialised by the kernel
  KernelStatus* status;      // in global memory, may be nullptr
};

__device__ __forceinline__ void report_failure(const WaitScope& ws, unsigned int code, unsigned int where,
                                               unsigned int aux) {
  *ws.abort = 1u;
  if (ws.status != nullptr) {
    if (atomicCAS(&ws.status->code, 0u, code) == 0u) {
      ws.status->where = where;
      ws.status->block = blockIdx.x;
      ws.status->aux = aux;
    }
    __threadfence_system();
  }
}

// Wait for the phase with the given parity. Returns false when the wait was abandoned
// (either this wait ran past the limit, or another thread of the CTA already gave up).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitScope& ws, unsigned int where,
                                          unsigned int aux = 0) {
  const uint32_t addr = smem_u32(bar);
  if (mbar_try_wait(addr, parity)) return true;
  if (*ws.abort) return false;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t it = 0;
  for (;;) {
    if (mbar_try_wait_hint(addr, parity, kWaitHintNs)) return true;
    // the hardware may resume the thread long before the hint: look at the clock only now and then
    if (((++it) & 0xFu) == 0u) {
      if (*ws.abort) return false;
      if (globaltimer_ns() - t0 > kBarrierLimitNs) {
        report_failure(ws, kErrBarrierTimeout, where, aux);
        return false;
      }
    }
  }
}

// ----------------------------------------------------------------------------------------
// Flags in global memory written by another GPU (or another CTA): bounded acquire-spin.

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Spin until *flag >= want (monotonic epoch counters). Bounded; see kPeerLimitNs.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t want, const WaitScope& ws,
                                             unsigned int where, unsigned int aux = 0,
                                             unsigned long long limit_ns = kPeerLimitNs) {
  if (ld_acquire_sys(flag) >= want) return true;
  if (*ws.abort) return false;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t it = 0;
  for (;;) {
    if (ld_acquire_sys(flag) >= want) return true;
    __nanosleep(64);
    if (((++it) & 0x3Fu) == 0u) {
      if (*ws.abort) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        report_failure(ws, kErrPeerTimeout, where, aux);
        return false;
      }
    }
  }
}

// ----------------------------------------------------------------------------------------
// Proxy fences

// generic-proxy writes to shared memory -> visible to the async proxy (TMA store, tcgen05.mma)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// generic-proxy writes (any state space) -> visible to the async proxy
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ----------------------------------------------------------------------------------------
// TMA: tiled tensor copies, no multicast. Coordinates are innermost-first; the innermost
// coordinate times the element size must be a multiple of 16 bytes.

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], "
      "[%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y,
                                            int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, "
      "%6}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// wait until at most N of this thread's bulk store groups still READ shared memory
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// wait until at most N bulk store groups are incomplete (writes visible)
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------------------------------
// Tensor memory (TMEM) and tcgen05

// One warp allocates `ncols` (power of two, 32..512) columns; the base address is written to
// shared memory at `dst`.
__device__ __forceinline__ void tmem_alloc(uint32_t* dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], bf16/f16 inputs, fp32 accumulate, one CTA.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same with 8-bit floating-point operands (kind::f8f6f4; the formats come from the instruction descriptor).
__device__ __forceinline__ void umma_ss_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrive once on `bar` when all tcgen05.mma issued so far by this thread have completed
// (their shared-memory operands may be overwritten, their accumulators may be read).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// Accumulator read-back: each thread of a warp reads 32 consecutive fp32 columns of its own
// TMEM lane (lane = 32 * (warp_id % 4) + lane_id). `taddr` = (lane << 16) | column.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Write 32 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// TMEM address of (lane quadrant of this warp, column)
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t warp_in_group, uint32_t col) {
  return base + ((warp_in_group * 32u) << 16) + col;
}

// ----------------------------------------------------------------------------------------
// Descriptors

// Instruction descriptor of tcgen05.mma kind::f16 with bf16 A/B and fp32 accumulation.
// a_mn / b_mn: operand is MN-major (1) instead of K-major (0).
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N, int a_mn = 0, int b_mn = 0) {
  return (1u << 4)                          // D format: fp32
         | (1u << 7)                        // A format: bf16
         | (1u << 10)                       // B format: bf16
         | (static_cast<uint32_t>(a_mn) << 15) | (static_cast<uint32_t>(b_mn) << 16) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

// Same with fp16 inputs (A/B format 0).
__host__ __device__ constexpr uint32_t umma_idesc_f16(int M, int N, int a_mn = 0, int b_mn = 0) {
  return (1u << 4) | (static_cast<uint32_t>(a_mn) << 15) | (static_cast<uint32_t>(b_mn) << 16) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

// kind::f8f6f4 with e4m3 A/B (format 0 of that kind), K-major, fp32 accumulation; K = 32 per instruction.
__host__ __device__ constexpr uint32_t umma_idesc_e4m3(int M, int N) {
  return (1u << 4) | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

enum : uint64_t { kSwizzleNone = 0, kSwizzle128 = 2, kSwizzle64 = 4, kSwizzle32 = 6 };

// Shared-memory matrix descriptor. Offsets are in bytes (multiples of 16).
//   K-major, 128B swizzle : rows of 128 bytes, 8-row groups `sbo` bytes apart (1024 when dense);
//                           `lbo` is ignored by the hardware (set 16).
//   MN-major, 128B swizzle: 64-element (128 B) runs along MN, K rows 128 B apart inside an
//                           8-row group, groups `sbo` bytes apart, next 64 MN elements `lbo` away.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint64_t swizzle) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // descriptor version of sm_100
  d |= swizzle << 61;
  return d;
}

// Byte offset of element (row, 16-byte chunk) inside a [rows][128 B] tile stored with the
// 128-byte swizzle (tile base 1024-byte aligned): chunk index XOR (row mod 8).
__device__ __forceinline__ uint32_t swz128_offset(uint32_t row, uint32_t chunk16) {
  return row * 128u + ((chunk16 ^ (row & 7u)) << 4);
}
// 64-byte swizzle for [rows][64 B] tiles: 16-byte chunk XOR ((row / 2) mod 4).
__device__ __forceinline__ uint32_t swz64_offset(uint32_t row, uint32_t chunk16) {
  return row * 64u + ((chunk16 ^ ((row >> 1) & 3u)) << 4);
}

// ----------------------------------------------------------------------------------------
// Small numeric helpers

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// sigmoid through one special-function instruction: sigmoid(x) = 0.5 tanh(x/2) + 0.5 (tanh.approx has a
// relative error near 2^-11, far inside bf16 resolution of the gated values; the exp + reciprocal form
// costs two special-function instructions per element and bounded the SwiGLU and gate epilogues)
__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float sigmoidf_fast(float x) { return fmaf(fast_tanh(0.5f * x), 0.5f, 0.5f); }
__device__ __forceinline__ float siluf_fast(float x) {
  const float hx = 0.5f * x;
  return fmaf(hx, fast_tanh(hx), hx);
}

// 32-byte global store (one full sector per lane in one instruction; address 32-byte aligned)
__device__ __forceinline__ void st_global_256(void* ptr, uint4 a, uint4 b) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(a.x), "r"(a.y), "r"(a.z),
               "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
               : "memory");
}

// 32-byte read-only global load (address 32-byte aligned)
__device__ __forceinline__ void ld_global_256(const void* ptr, uint4& a, uint4& b) {
  asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w)
               : "l"(ptr));
}
// 16 fp32 values -> 16 bf16 = 32 bytes, one store.  A lane that writes half a sector (16 bytes) per
// instruction, as a row-per-lane epilogue does with 16-byte stores, costs the L2 two partial-sector writes;
// measured on the plane writer of the triangle projection, 32-byte stores cut the kernel from 1.6 to 1.0 ms.
__device__ __forceinline__ void st_bf16x16(__nv_bfloat16* dst, const float* f) {
  uint4 a, b;
  a.x = pack_bf16x2(f[0], f[1]);
  a.y = pack_bf16x2(f[2], f[3]);
  a.z = pack_bf16x2(f[4], f[5]);
  a.w = pack_bf16x2(f[6], f[7]);
  b.x = pack_bf16x2(f[8], f[9]);
  b.y = pack_bf16x2(f[10], f[11]);
  b.z = pack_bf16x2(f[12], f[13]);
  b.w = pack_bf16x2(f[14], f[15]);
  st_global_256(dst, a, b);
}
// 16 bf16 values (32 bytes, 32-byte aligned) added to / multiplied into 16 fp32 values
__device__ __forceinline__ void ld_bf16x16(const __nv_bfloat16* src, float* e) {
  uint4 a, b;
  ld_global_256(src, a, b);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    e[2 * j] = bf16_lo(w[j]);
    e[2 * j + 1] = bf16_hi(w[j]);
  }
}

// LayerNorm folded into a GEMM, applied to two adjacent accumulator columns in two packed instructions:
//   out = rstd * (acc - mu * colsum) + colbias = acc * a + (b * colsum + colbias),  a = rstd, b = -mu * rstd
__device__ __forceinline__ float2 ln_fold2(uint32_t acc0, uint32_t acc1, float2 a2, float2 b2, float cs0, float cs1,
                                           float cb0, float cb1) {
  return __ffma2_rn(make_float2(__uint_as_float(acc0), __uint_as_float(acc1)), a2,
                    __ffma2_rn(b2, make_float2(cs0, cs1), make_float2(cb0, cb1)));
}
// 32 accumulator columns at once; cs / cb point at 16-byte aligned shared-memory constants of those columns
__device__ __forceinline__ void ln_fold32(const uint32_t (&acc)[32], float2 a2, float2 b2, const float* cs,
                                          const float* cb, float (&out)[32]) {
  const float4* cs4 = reinterpret_cast<const float4*>(cs);
  const float4* cb4 = reinterpret_cast<const float4*>(cb);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float4 s4 = cs4[j], b4 = cb4[j];
    const float2 v01 = ln_fold2(acc[4 * j], acc[4 * j + 1], a2, b2, s4.x, s4.y, b4.x, b4.y);
    const float2 v23 = ln_fold2(acc[4 * j + 2], acc[4 * j + 3], a2, b2, s4.z, s4.w, b4.z, b4.w);
    out[4 * j] = v01.x;
    out[4 * j + 1] = v01.y;
    out[4 * j + 2] = v23.x;
    out[4 * j + 3] = v23.y;
  }
}

// 2^x for x <= 0 on the FMA and ALU pipes (no special-function instruction): split x into a rounded integer n
// (magic-number add; the integer lands in the low mantissa bits) and f = x - n in [-0.5, 0.5], evaluate a
// degree-3 polynomial of 2^f (largest relative error 7.5e-5, far inside bf16 resolution) and add n to the
// exponent field.  Measured in the attention softmax: it pays for head dimension 64 (one exponential in four
// moved off the special-function unit: 0.128 -> 0.115 ms together with packed adds) and costs time for head
// dimension 32, whose loop is short of issue slots rather than of special-function throughput.
__device__ __forceinline__ float poly_exp2(float x) {
  x = fmaxf(x, -125.0f);
  const float t = x + 12582912.0f;
  const float f = x - (t - 12582912.0f);
  float p = fmaf(f, 0.0551716685f, 0.2426111251f);
  p = fmaf(p, f, 0.6932609677f);
  p = fmaf(p, f, 0.9999280572f);
  return __uint_as_float(__float_as_uint(p) + (__float_as_uint(t) << 23));
}

// three-input maximum (one instruction on sm_100)
__device__ __forceinline__ float max3f(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace ubm
