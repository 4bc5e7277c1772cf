// Thin wrappers over the sm_100a PTX this library uses: mbarrier, cp.async, bulk-tensor
// (TMA) loads, tcgen05 (5th-gen tensor core) MMA / TMEM management, proxy fences.
// Every blocking wait is bounded: it gives up after a fixed number of polls and reports
// failure to its caller, so a protocol bug ends in an error status, never a hung GPU.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace cb2 {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

// ---------------------------------------------------------------- optional event trace
// Built only with -DCB2_TRACE (a debugging aid): CTA 0 records (global timer, code, step)
// triples per role into a device buffer so a pipeline timeline can be read back.
#ifdef CB2_TRACE
struct TraceBuf {
  unsigned long long ev[8][512][2];  // [role][event][time, (code << 32) | step]
  int count[8];
  unsigned long long cta[256][3];    // per CTA: start time, end time, steps
  long long prof[256][12];           // per CTA: clock cycles the MMA warp spent per phase
  long long prof2[256][12];          // per CTA: the same for thread 0 of the epilogue
  long long prof3[256][8];           // per CTA: the scheduler warp
};
__device__ TraceBuf g_trace;
// 1 in the CTA whose events are recorded (a shared-memory flag: testing it must cost next to
// nothing in the CTAs that are not recorded)
__device__ __forceinline__ volatile int &trace_on() {
  __shared__ int v;
  return v;
}
__device__ __forceinline__ void trace_event(int role, int code, int step) {
  if (!trace_on() || blockIdx.y != 0)
    return;
  int n = g_trace.count[role];
  if (n >= 512)
    return;
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  g_trace.ev[role][n][0] = t;
  g_trace.ev[role][n][1] = (static_cast<unsigned long long>(code) << 32) | static_cast<unsigned>(step);
  g_trace.count[role] = n + 1;
}
__device__ __forceinline__ void trace_cta(int which, unsigned long long value) {
  if (blockIdx.x >= 256 || blockIdx.y != 0)
    return;
  if (which < 2) {
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(value));
  }
  g_trace.cta[blockIdx.x][which] = value;
}
#ifdef CB2_PROF_ONLY
#define CB2_TRACE_EVENT(role, code, step) ((void)0)
#else
#define CB2_TRACE_EVENT(role, code, step) ::cb2::trace_event(role, code, step)
#endif
#define CB2_TRACE_CTA(which, value) ::cb2::trace_cta(which, value)
#define CB2_TRACE_SELECT(on) (::cb2::trace_on() = (on))
#define CB2_PROF_BEGIN() long long prof_c[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}; long long prof_prev = clock64()
#define CB2_PROF_MARK(i) do { long long prof_t = clock64(); prof_c[i] += prof_t - prof_prev; prof_prev = prof_t; } while (0)
#define CB2_PROF_END() do { for (int i = 0; i < 12; ++i) ::cb2::g_trace.prof[blockIdx.x & 255][i] = prof_c[i]; } while (0)
#define CB2_PROF_END2() do { for (int i = 0; i < 12; ++i) ::cb2::g_trace.prof2[blockIdx.x & 255][i] = prof_c[i]; } while (0)
#else
#define CB2_PROF_BEGIN() ((void)0)
#define CB2_PROF_MARK(i) ((void)0)
#define CB2_PROF_END() ((void)0)
#define CB2_PROF_END2() ((void)0)
#define CB2_TRACE_EVENT(role, code, step) ((void)0)
#define CB2_TRACE_CTA(which, value) ((void)0)
#define CB2_TRACE_SELECT(on) ((void)0)
#endif

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n"
               ".reg .pred p;\n"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
               "selp.u32 %0, 1, 0, p;\n"
               "}\n"
               : "=r"(ok)
               : "r"(bar), "r"(parity)
               : "memory");
  return ok != 0;
}

// The same test without any waiting: try_wait may suspend the thread for a while when the phase
// is still open (which is what a waiter wants), test_wait returns at once (which is what a
// thread that has other work to do wants).
__device__ __forceinline__ bool mbar_poll(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n"
               ".reg .pred p;\n"
               "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
               "selp.u32 %0, 1, 0, p;\n"
               "}\n"
               : "=r"(ok)
               : "r"(bar), "r"(parity)
               : "memory");
  return ok != 0;
}

// Time limit of every wait, in nanoseconds of the global timer.  Far above any legitimate
// delay on this path (whole kernels run for tens of microseconds), far below anything an
// operator would notice.
#ifndef CB2_WAIT_SLEEP_MIN
#define CB2_WAIT_SLEEP_MIN 20
#endif
#ifndef CB2_WAIT_SLEEP_MAX
#define CB2_WAIT_SLEEP_MAX 160
#endif
constexpr unsigned long long kWaitLimitNs = 1000ull * 1000ull * 1000ull;

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait.  `abort_flag` (shared memory) is polled so that once any thread of the
// CTA has given up, everybody else leaves quickly too.  Returns false on give-up.
// A waiter that does not get through at once sleeps between polls (20 ns growing to
// 160 ns): a CTA has a dozen waiters most of the time, and pollers that spin take issue
// slots away from the warps that do the work.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  if (mbar_test(bar, parity))
    return true;
  unsigned long long t0 = 0;
  uint32_t backoff = CB2_WAIT_SLEEP_MIN;
  for (uint32_t i = 0;; ++i) {
    if (CB2_WAIT_SLEEP_MAX > 0)
      __nanosleep(backoff);
    if (mbar_test(bar, parity))
      return true;
    if (backoff < CB2_WAIT_SLEEP_MAX)
      backoff += backoff;
    if ((i & 63u) == 63u) {
      if (*abort_flag)
        return false;
      unsigned long long now = global_timer_ns();
      if (t0 == 0)
        t0 = now;
      else if (now - t0 > kWaitLimitNs)
        break;
    }
  }
  *abort_flag = 1;
  return false;
}

// Warp-collective wait: lane 0 polls, the other lanes sleep at the shuffle.  Keeps the
// number of spinning threads per SM small (one per warp), which matters because pollers
// compete for issue slots with the warps that do the work.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  int ok = 1;
  if (lane_id() == 0)
    ok = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// Non-blocking, warp-uniform test (lane 0 tests, the result is broadcast).
__device__ __forceinline__ bool mbar_test_warp(uint32_t bar, uint32_t parity) {
  int ok = 0;
  if (lane_id() == 0)
    ok = mbar_poll(bar, parity) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

__device__ __forceinline__ void st_shared_zero16(uint32_t addr) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0) : "memory");
}

// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched with the programmatic-serialisation attribute may start while the kernel
// before it on the stream still runs; it must not touch that kernel's results before
// grid_dep_wait(), which returns once the earlier grid has completed and its writes are visible.
// grid_dep_launch() in the earlier kernel allows the later one to be scheduled from then on.
// Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------- named barriers
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---------------------------------------------------------------- cp.async (16 B, zero-fill)
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
// Asynchronous arrive on `bar`, triggered when all cp.async issued so far by this thread
// have completed.  .noinc: the arrival is one of the barrier's expected count.
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Makes generic-proxy writes to shared memory (st.shared, completed cp.async) visible to
// the async proxy (tcgen05.mma operand reads, TMA).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------- flags in global memory
__device__ __forceinline__ int ld_acquire_gpu(const int *p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_relaxed_gpu(const int *p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int *p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// ---------------------------------------------------------------- TMA (no multicast)
__device__ __forceinline__ void tma_prefetch_desc(const void *tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void *tmap, uint32_t bar, int c0,
                                            int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
               "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
               "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}

// Four rows r0..r3 of a 2-D tensor, gathered into four consecutive 128-byte rows of `dst`.
__device__ __forceinline__ void tma_gather4(uint32_t dst, const void *tmap, uint32_t bar, int c0, int r0, int r1,
                                            int r2, int r3) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes "
               "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(dst),
               "l"(tmap), "r"(bar), "r"(c0), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
               : "memory");
}
// ---------------------------------------------------------------- tcgen05 / TMEM
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
// Arrives on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem];  KIND 0: kind::f16 (fp16 in, fp32 acc), 1: kind::i8.
template <int KIND>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
  if constexpr (KIND == 0) {
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "setp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
                 "}\n" ::"r"(d_tmem),
                 "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
                 : "memory");
  } else {
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "setp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
                 "}\n" ::"r"(d_tmem),
                 "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
                 : "memory");
  }
}
// 32 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor, 128-byte swizzle, sm_100 format:
//   [0,14) start address >> 4, [16,30) leading byte offset >> 4, [32,46) stride byte
//   offset >> 4, [46,48) version = 1, [61,64) layout = 2 (SWIZZLE_128B).
// K-major operand: rows of 128 B (one swizzle atom along K), 8-row groups `sbo` apart.
// MN-major operand: rows of 128 B along M/N, 8 K-rows per group, groups `sbo` apart,
//   successive 64-element (128 B) blocks along M/N `lbo` apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor (32 bit) for tcgen05.mma kind::f16 / kind::i8:
//   [4,6) D format (1 = f32, 2 = s32), [7,10) A format, [10,13) B format
//   (kind::f16: 0 = f16; kind::i8: 1 = s8), bit 15 A is MN-major, bit 16 B is MN-major,
//   [17,23) N >> 3, [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc(int kind, bool a_mn, bool b_mn, int M, int N) {
  uint32_t d = 0;
  d |= (kind == 0 ? 1u : 2u) << 4;
  d |= (kind == 0 ? 0u : 1u) << 7;
  d |= (kind == 0 ? 0u : 1u) << 10;
  d |= (a_mn ? 1u : 0u) << 15;
  d |= (b_mn ? 1u : 0u) << 16;
  d |= static_cast<uint32_t>(N >> 3) << 17;
  d |= static_cast<uint32_t>(M >> 4) << 24;
  return d;
}

} // namespace cb2
