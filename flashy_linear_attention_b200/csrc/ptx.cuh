// Thin inline-PTX wrappers for the sm_100a features the linear-attention kernels use:
// mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (TMEM alloc / mma / ld / st / commit / fences).
// Every wait in here is bounded: it gives up after a time limit and reports failure, so a
// protocol bug ends in an error status rather than a hung GPU.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include <utility>

namespace fla {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// One lane of a fully active warp (deterministic for a given mask).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\t"
      "elect.sync rx|px, 0xffffffff;\n\t"
      "@px mov.s32 %0, 1;\n\t}"
      : "+r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done;
}

// Default limit of one wait: 2 s of the GPU's global timer, far above any legitimate wait of these
// kernels, which are microseconds. Waits are timed with %globaltimer, not clock64(): a CTA that is
// preempted (another context's time slice on a shared GPU) may resume on another SM, whose cycle
// counter has nothing to do with the one read before, and the time it spent switched out must not
// count against a 0.4 s limit either (a wait of a process's first launch, taken while the previous
// process's context was still being torn down, did run out that way).
constexpr unsigned long long kWaitLimitNs = 2000ull * 1000ull * 1000ull;
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Diagnostics for the status bit: the first few waits that ran out (since the last read-out) leave
// a record of which barrier they were waiting on. Only the give-up path touches these.
constexpr int kTimeoutRecords = 32;
static __device__ unsigned g_timeout_records[kTimeoutRecords * 8];
static __device__ unsigned g_timeout_count;
__device__ __noinline__ void record_timeout(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  const unsigned slot = atomicAdd(&g_timeout_count, 1u);
  if (slot >= static_cast<unsigned>(kTimeoutRecords)) return;
  unsigned* r = &g_timeout_records[slot * 8];
  r[0] = bar;      // shared-memory address of the mbarrier
  r[1] = parity;
  r[2] = threadIdx.x;
  r[3] = blockIdx.x;
  r[4] = blockIdx.y;
  r[5] = blockIdx.z;
  r[6] = static_cast<unsigned>(__cvta_generic_to_shared(const_cast<int*>(abort_flag)));  // locates the barrier area
  r[7] = static_cast<unsigned>(global_timer_ns() >> 10);
}

// Waits for the phase with the given parity. Returns false when the CTA-wide abort flag is set
// or the limit ran out (in which case it sets the flag so that every other wait of the CTA
// gives up too). `abort_flag` points at two shared-memory words: [0] the flag, [1] the limit in
// microseconds (0 = kWaitLimitNs), which the host can shorten for tests.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
#pragma unroll 1
  for (int spin = 0; spin < 64; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  const unsigned long long t0 = global_timer_ns();
  const unsigned lim_us = static_cast<unsigned>(abort_flag[1]);
  const unsigned long long limit = lim_us ? static_cast<unsigned long long>(lim_us) * 1000ull : kWaitLimitNs;
#pragma unroll 1
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 63u) == 0u) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > limit) {
        if (*abort_flag == 0) record_timeout(bar, parity, abort_flag);
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// Barrier between CTAs of one launch that are all resident (cooperative launch). Called by ONE
// thread per CTA, after the CTA's earlier global writes have been fenced. bar[0] counts arrivals,
// bar[1] is the generation: the last arrival resets the count and bumps the generation, so the
// two words need no initialisation beyond being zero before their first use and may serve
// launches with different CTA counts one after the other. `gen_before` is the generation read at
// any time before this CTA arrives (it cannot change until it does; reading it early, see
// barrier_generation(), takes a memory round trip off the barrier). The wait is bounded like every
// other wait here; a CTA that gives up withdraws its arrival and sets the abort flag.
__device__ __forceinline__ unsigned barrier_generation(const unsigned* bar) {
  unsigned gen;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(gen) : "l"(bar + 1) : "memory");
  return gen;
}
__device__ __forceinline__ bool grid_barrier(unsigned* bar, unsigned n_ctas, unsigned gen_before,
                                             volatile int* abort_flag) {
  unsigned prev;
  asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(prev) : "l"(bar) : "memory");
  if (prev == n_ctas - 1u) {
    // Release first, reset after: nobody arrives at these words again before the launch ends, and
    // a release that had to wait for the reset to land would cost the waiters a memory round trip.
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(bar + 1), "r"(gen_before + 1u) : "memory");
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(bar), "r"(0u) : "memory");
    return true;
  }
  const unsigned long long t_start = global_timer_ns();
  const unsigned lim_us = static_cast<unsigned>(abort_flag[1]);
  const unsigned long long limit = lim_us ? static_cast<unsigned long long>(lim_us) * 1000ull : kWaitLimitNs;
#pragma unroll 1
  for (uint32_t spin = 1;; ++spin) {
    unsigned now;  // relaxed polls, one acquire fence once the generation has moved
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(now) : "l"(bar + 1) : "memory");
    if (now != gen_before) {
      asm volatile("fence.acq_rel.gpu;" ::: "memory");
      return true;
    }
    if ((spin & 15u) == 0u && (*abort_flag || global_timer_ns() - t_start > limit)) {
      atomicSub(bar, 1u);
      *abort_flag = 1;
      return false;
    }
  }
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, uint32_t src, int c0, int c1,
                                             int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::
          "l"(reinterpret_cast<uint64_t>(m)),
      "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_group_read0() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_group0() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
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
__device__ __forceinline__ void tc_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// Arrives (count 1) on the mbarrier once every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
      : "memory");
}

// Shared-memory matrix descriptors are passed as two 32-bit halves so that the issuing thread
// only adds a constant to the low word between instructions (start address field, 16-byte units).
// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t hi,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Instruction descriptor for kind::f16 with 16-bit operands (bf16, or fp16 when `half`) and an
// fp32 accumulator.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool a_mn_major, bool b_mn_major,
                                                  bool half = false) {
  return (1u << 4)                                // accumulator format: f32
         | ((half ? 0u : 1u) << 7)                // A format: 0 = f16, 1 = bf16
         | ((half ? 0u : 1u) << 10)               // B format
         | ((a_mn_major ? 1u : 0u) << 15)         // A major-ness
         | ((b_mn_major ? 1u : 0u) << 16)         // B major-ness
         | (static_cast<uint32_t>(n >> 3) << 17)  // N / 8
         | (static_cast<uint32_t>(m >> 4) << 24); // M / 16
}

// Shared-memory matrix descriptor, 128-byte swizzle, as two words.
// High word: stride byte offset (1024 B between 8-row groups) | descriptor version | swizzle mode.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
// Low word: start address | leading byte offset, both in 16-byte units.
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
  return ((saddr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (base lane + t).
// tcgen05.ld is asynchronous: its destination registers hold the data only after
// tcgen05.wait::ld. Load and wait therefore sit in ONE asm statement whose outputs are the
// destination registers -- with the wait in a statement of its own the compiler is free to schedule
// arithmetic on those registers between the two (nothing ties a register-only instruction to a
// volatile asm with a memory clobber), and then it computes on whatever the registers held before.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// Two such blocks with one wait: both loads are in flight together.
__device__ __forceinline__ void tmem_ld32x2(uint32_t taddr_a, uint32_t (&a)[32], uint32_t taddr_b,
                                            uint32_t (&b)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%64];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%65];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7]), "=r"(a[8]), "=r"(a[9]), "=r"(a[10]), "=r"(a[11]), "=r"(a[12]), "=r"(a[13]), "=r"(a[14]), "=r"(a[15]), "=r"(a[16]), "=r"(a[17]), "=r"(a[18]), "=r"(a[19]), "=r"(a[20]), "=r"(a[21]), "=r"(a[22]), "=r"(a[23]), "=r"(a[24]), "=r"(a[25]), "=r"(a[26]), "=r"(a[27]), "=r"(a[28]), "=r"(a[29]), "=r"(a[30]), "=r"(a[31]), "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]), "=r"(b[4]), "=r"(b[5]), "=r"(b[6]), "=r"(b[7]), "=r"(b[8]), "=r"(b[9]), "=r"(b[10]), "=r"(b[11]), "=r"(b[12]), "=r"(b[13]), "=r"(b[14]), "=r"(b[15]), "=r"(b[16]), "=r"(b[17]), "=r"(b[18]), "=r"(b[19]), "=r"(b[20]), "=r"(b[21]), "=r"(b[22]), "=r"(b[23]), "=r"(b[24]), "=r"(b[25]), "=r"(b[26]), "=r"(b[27]), "=r"(b[28]), "=r"(b[29]), "=r"(b[30]), "=r"(b[31])
      : "r"(taddr_a), "r"(taddr_b)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);  // .x (low 16 bits) = lo, .y = hi
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Two fp32 values rounded to the 16-bit operand type of the kernel instance.
template <bool HALF>
__device__ __forceinline__ uint32_t pack16x2(float lo, float hi) {
  return HALF ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
}
// L2-only (cache-global) load; volatile, so that a run of them is issued in program order and stays
// ahead of the code that consumes the values.
__device__ __forceinline__ uint32_t ld_global_cg_b32(const float* p) {
  uint32_t v;
  asm volatile("ld.global.cg.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// The same for 16 bytes at a compile-time byte offset from `p` (the offset becomes the immediate
// of the instruction, so a run of these from one base pointer costs one instruction each).
template <int OFF>
__device__ __forceinline__ void ld_global_cg_v4(const float* p, uint32_t& a, uint32_t& b, uint32_t& c,
                                                uint32_t& d) {
  asm volatile("ld.global.cg.v4.b32 {%0, %1, %2, %3}, [%4 + %5];"
               : "=r"(a), "=r"(b), "=r"(c), "=r"(d)
               : "l"(p), "n"(OFF)
               : "memory");
}
template <int OFF>
__device__ __forceinline__ uint32_t ld_global_cg_b32_at(const float* p) {
  uint32_t v;
  asm volatile("ld.global.cg.b32 %0, [%1 + %2];" : "=r"(v) : "l"(p), "n"(OFF) : "memory");
  return v;
}
template <int OFF>
__device__ __forceinline__ void st_global_cg_v4(float* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.global.cg.v4.b32 [%0 + %1], {%2, %3, %4, %5};"
               :
               : "l"(p), "n"(OFF), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}
template <int OFF>
__device__ __forceinline__ void st_global_cg_b32_at(float* p, uint32_t v) {
  asm volatile("st.global.cg.b32 [%0 + %1], %2;" ::"l"(p), "n"(OFF), "r"(v) : "memory");
}
// f(std::integral_constant<int, 0>{}) ... f(std::integral_constant<int, N - 1>{}): a loop whose
// index is a constant expression in the body (template arguments, asm immediates).
template <class F, int... I>
__device__ __forceinline__ void static_for_impl(F&& f, std::integer_sequence<int, I...>) {
  (f(std::integral_constant<int, I>{}), ...);
}
template <int N, class F>
__device__ __forceinline__ void static_for(F&& f) {
  static_for_impl(f, std::make_integer_sequence<int, N>{});
}
// Compiler-only fence over 32 registers: everything that produces them (a run of loads) is placed
// before it and everything that reads them after it, so the loads of a batch are all issued before
// the first of them is waited for. Emits no instruction.
__device__ __forceinline__ void keep_together(uint32_t (&r)[32]) {
  asm volatile(""
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]),
                 "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]),
                 "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]),
                 "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]),
                 "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]));
}
__device__ __forceinline__ void st_shared_b32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_shared_b32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}

}  // namespace ptx
}  // namespace fla
