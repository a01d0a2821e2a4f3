// Shared device helpers: pool-format arithmetic and sm_100a PTX wrappers (mbarrier, asynchronous
// copies, tcgen05 tensor-memory and MMA instructions). Every wait is bounded by a cycle budget:
// when it runs out the waiter raises the CTA's abort flag and the caller's status word and
// falls through, so a protocol error ends the kernel instead of hanging the GPU.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "../../include/foscar_b200.h"

namespace fq {

constexpr int PAGE = FQ_PAGE_SIZE;

// ---------------------------------------------------------------------------------------------
// Pool format
// ---------------------------------------------------------------------------------------------

// Exponent bin of a page maximum (f32 bit pattern): lp = floor(log2(448/x)) = 135 - bin.
__host__ __device__ inline uint32_t vmax_bucket(uint32_t bits) {
  uint32_t m = bits & 0x7FFFFFFFu;
  if (m > 0x7F800000u) m = 0x7F800000u;
  return (m + 0x1FFFFFu) >> 23;
}

// Bit offset, inside a token row, of channel c: word c/W, field 2*(w%(W/2)) + w/(W/2).
template <int BITS>
__host__ __device__ inline int code_bit_offset(int c) {
  constexpr int W = 32 / BITS;
  const int within = c % W;
  const int field = 2 * (within % (W / 2)) + within / (W / 2);
  return (c / W) * 32 + BITS * field;
}

// The order in which byte-expansion of a packed row yields channels. A 32-bit word w expands to
// BITS*... output words ((w >> (BITS*k)) & mask); byte j of output word k is field 4j+k (INT2)
// or 2j+k (INT4). Position p of the expanded row therefore holds this channel.
template <int BITS>
__host__ __device__ inline int channel_of_expanded_pos(int p) {
  if (BITS == 4) return p;
  const int wi = p >> 4, k = (p >> 2) & 3, j = p & 3;
  return 16 * wi + 2 * j + (k >> 1) + 8 * (k & 1);
}

// ---------------------------------------------------------------------------------------------
// PTX: shared addresses, mbarrier
// ---------------------------------------------------------------------------------------------

__device__ inline uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ inline void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ inline void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ inline bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Cycle budget of one wait unless the launch sets another: about a second at B200 clocks.
constexpr long long WAIT_BUDGET_CYCLES = 2000000000LL;

// Wait for a barrier phase, bounded. `abort_flag` is a CTA-shared word: once any waiter has
// given up every later wait returns at once, so the CTA drains in bounded time. The cycle
// budget of a wait sits two words after the flag (set_wait_budget).
// `site` names the call site for the optional wait profile (see FQ_WAIT_PROFILE): the cycles
// lane 0 of each warp spent blocked are summed per site in the words after the budget.
constexpr int WAIT_SITES = 32;
__device__ inline void set_wait_budget(volatile int* abort_flag, long long cycles) {
  *reinterpret_cast<volatile long long*>(abort_flag + 2) = cycles;
}
static __device__ __noinline__ void mbar_wait_slow(uint32_t bar, uint32_t parity,
                                            volatile int* abort_flag, int* status) {
  // mbarrier.try_wait suspends the thread in hardware for a bounded time by itself; the abort
  // flag and the clock are looked at once every 32 failed tries only.
  long long t0 = 0;
  for (uint32_t tries = 1; !mbar_try(bar, parity); ++tries) {
    if ((tries & 31u) != 0) continue;
    if (*abort_flag) return;
    const long long now = clock64();
    if (t0 == 0) t0 = now;
    if (now - t0 > *reinterpret_cast<volatile long long*>(abort_flag + 2)) {
      *abort_flag = 1;
      if (status) atomicOr(status, FQ_STATUS_TIMEOUT);
      return;
    }
  }
}
#ifndef FQ_WAIT_PROFILE
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity,
                                          volatile int* abort_flag, int* status, int = -1,
                                          int* = nullptr) {
  if (!mbar_try(bar, parity)) mbar_wait_slow(bar, parity, abort_flag, status);
}
#else
// Diagnostic build: the cycles each thread spends inside a wait are summed per call site in
// a thread-local array (constant indices, so it stays in registers).
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity,
                                          volatile int* abort_flag, int* status, int site = -1,
                                          int* wprof = nullptr) {
  const long long t0 = clock64();
  if (!mbar_try(bar, parity)) mbar_wait_slow(bar, parity, abort_flag, status);
  if (wprof != nullptr && site >= 0) wprof[site] += static_cast<int>(clock64() - t0);
}
#endif

// Bounded wait for a shared-memory word that only grows (a count of events) to reach `want`.
// One thread polls; the caller follows with a warp or group synchronisation.
static __device__ __noinline__ void count_wait(volatile int* word, int want,
                                               volatile int* abort_flag, int* status) {
  long long t0 = 0;
  for (uint32_t tries = 1; *word < want; ++tries) {
    if ((tries & 31u) != 0) continue;
    if (*abort_flag) return;
    const long long now = clock64();
    if (t0 == 0) t0 = now;
    if (now - t0 > *reinterpret_cast<volatile long long*>(abort_flag + 2)) {
      *abort_flag = 1;
      if (status) atomicOr(status, FQ_STATUS_TIMEOUT);
      return;
    }
  }
}

// Bounded wait that ignores the abort flag: used once, at exit, to let a CTA's own bulk copies
// land before its shared memory is released.
__device__ inline void mbar_wait_drain(uint32_t bar, uint32_t parity, long long budget) {
  const long long t0 = clock64();
  while (!mbar_try(bar, parity)) {
    if (clock64() - t0 > budget) return;
  }
}

__device__ inline void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Make generic-proxy shared-memory writes visible to the async proxy (TMA, tcgen05.mma).
__device__ inline void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ inline void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// Named barrier that also returns whether `pred` held for any of the arriving threads.
__device__ inline bool named_barrier_or(int id, int threads, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %3, 0;\n\t"
      "bar.red.or.pred p, %1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(id), "r"(threads), "r"(static_cast<uint32_t>(pred))
      : "memory");
  return r != 0;
}

// ---------------------------------------------------------------------------------------------
// PTX: asynchronous copies global -> shared
// ---------------------------------------------------------------------------------------------

// 16-byte asynchronous copy global -> shared issued by a thread (LSU path, bypassing L1), and the
// arrive that fires on an mbarrier once all of this thread's earlier copies have landed. The
// barrier's expected count must include these arrivals (".noinc").
__device__ inline void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// The same copy for data read once per launch: marked evict-first in L2, so that the stream of
// cache pages does not push out what is used again (query rows, work items, and above all the
// kernel's own instructions: a phase that runs once per work item otherwise refetches its code
// from DRAM every time).
__device__ inline uint64_t l2_evict_first_policy() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ inline void cp_async16_stream(uint32_t dst, const void* src, uint64_t policy) {
#ifdef FQ_PLAIN_COPIES
  cp_async16(dst, src);
#else
  asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;" ::"r"(dst),
               "l"(src), "l"(policy)
               : "memory");
#endif
}
__device__ inline void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// ---------------------------------------------------------------------------------------------
// PTX: tcgen05 (tensor memory + 5th-generation tensor cores)
// ---------------------------------------------------------------------------------------------

// One full warp allocates `cols` (power of two >= 32) tensor-memory columns; the base address
// lands in shared memory at `dst`.
__device__ inline void tmem_alloc(uint32_t dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ inline void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ inline void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ inline void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on an mbarrier when every tcgen05 operation this thread issued so far has completed.
__device__ inline void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

// Shared-memory matrix descriptor. `layout`: 0 none, 2 = 128-byte swizzle, 4 = 64B, 6 = 32B.
__device__ inline uint64_t make_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                          uint32_t layout) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= 1ull << 46;  // descriptor version of sm_100
  d |= static_cast<uint64_t>(layout & 7) << 61;
  return d;
}

// Instruction descriptor of kind::f8f6f4 with E4M3 operands and an f32 accumulator.
__host__ __device__ constexpr uint32_t make_idesc_e4m3(int m, int n, int a_mn_major,
                                                       int b_mn_major) {
  return (1u << 4)                                 // accumulator f32
         | (0u << 7) | (0u << 10)                  // A, B = E4M3
         | (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// Descriptor halves: the low word carries the start address (and the leading byte offset), the
// high word is constant per operand kind, so an issue loop only adds to the low word.
__device__ inline uint32_t smem_desc_lo(uint32_t addr, uint32_t lbo_bytes) {
  return ((addr >> 4) & 0x3FFFu) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
__host__ __device__ constexpr uint32_t smem_desc_hi(uint32_t sbo_bytes, uint32_t layout) {
  return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | ((layout & 7u) << 29);
}
// Lean issue forms: constant high words, instruction descriptor and accumulate flag.
template <uint32_t A_HI, uint32_t B_HI, uint32_t IDESC, bool ACC>
__device__ inline void umma_ss_c(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %5, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "n"(A_HI), "n"(B_HI), "n"(IDESC), "n"(ACC ? 1 : 0)
      : "memory");
}
template <uint32_t B_HI, uint32_t IDESC, bool ACC>
__device__ inline void umma_ts_c(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "n"(B_HI), "n"(IDESC), "n"(ACC ? 1 : 0)
      : "memory");
}

// The same with the accumulate flag at run time (the first MMA of a chain that either starts or
// continues an accumulator).
template <uint32_t A_HI, uint32_t B_HI, uint32_t IDESC>
__device__ inline void umma_ss_r(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %5, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "n"(A_HI), "n"(B_HI), "n"(IDESC), "r"(acc)
      : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ inline void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ inline void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Tensor-memory loads/stores, shape 32x32b: lane i of the warp addresses TMEM lane
// (taddr.lane + i) and N consecutive 32-bit columns.
__device__ inline void tmem_ld4(uint32_t taddr, uint32_t (&r)[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(taddr)
               : "memory");
}
__device__ inline void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                 "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ inline void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ inline void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ inline void tmem_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(
                   taddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
               "r"(r[7])
               : "memory");
}
__device__ inline void tmem_ld8p(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                 "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ inline void tmem_ld16p(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ inline void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// One 128-byte operand row per lane in one instruction.
__device__ inline void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,"
      "%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ inline void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// Small numeric helpers
// ---------------------------------------------------------------------------------------------

// Two f32 -> packed E4M3 pair (RN, saturating): `lo` in the low byte, `hi` in the high byte.
__device__ inline uint32_t f32x2_to_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
// Packed E4M3 pair -> two f32 (low byte first).
__device__ inline float2 e4m3x2_to_f32x2(uint32_t v) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(v)));
  __half2 h = *reinterpret_cast<__half2*>(&h2);
  return __half22float2(h);
}
__device__ inline float e4m3_to_f32(uint32_t byte) { return e4m3x2_to_f32x2(byte & 0xFF).x; }

__device__ inline float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace fq
