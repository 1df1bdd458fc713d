// Thin inline-PTX wrappers for the sm_100a tensor-core path: tcgen05 (MMA, TMEM alloc/ld/st, commit, fences),
// mbarriers with bounded waits, 1-D bulk copies.  Every wait in here has an iteration limit: on expiry it returns
// false and the caller records a status code and falls through, so a protocol bug yields wrong numbers and a
// Q4B_E_TIMEOUT, never a hung GPU.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace q4b {
namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P;\n\t.reg .b32 R;\n\telect.sync R|P, 0xffffffff;\n\tselp.b32 %0, 1, 0, P;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\tmbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\tselp.b32 %0, 1, 0, P;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking test of a phase: returns at once either way (try_wait may suspend the thread for a hardware-chosen slice
// when the phase is not complete, which is wrong for an opportunistic look).
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\tmbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\tselp.b32 %0, 1, 0, P;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// try_wait with a suspend-time hint: the thread may sleep up to `ns` nanoseconds and is woken when the phase completes.
// Waiting warps then stay out of the issue slots of the working warps on their scheduler.
__device__ __forceinline__ bool mbar_try_hint(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\tmbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\tselp.b32 %0, 1, 0, P;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Bounded wait: about a second at most (each failed try_wait suspends for a hardware-chosen slice first).
constexpr uint32_t WAIT_LIMIT = 1u << 22;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
    if (mbar_try(bar, parity)) return true;
  return false;
}
// The same bound (about a second, by the SM clock) for waits whose failed tries suspend for up to `ns` nanoseconds each: a
// try_wait without the hint comes back within ~100 clocks and the retry loop around it then fills the issue slots of the
// warps that have work; with it a waiting thread costs a handful of instructions per wait and is woken by the completion.
__device__ __forceinline__ bool mbar_wait_parked(uint64_t* bar, uint32_t parity, uint32_t ns = 200000u) {
  if (mbar_try_hint(bar, parity, ns)) return true;
  const long long t0 = clock64();
  do {
    if (mbar_try_hint(bar, parity, ns)) return true;
  } while (clock64() - t0 < (1ll << 31));
  return false;
}

// ---- proxies / fences -------------------------------------------------------------------------------------------
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- TMEM -------------------------------------------------------------------------------------------------------
// One full warp calls these (sync.aligned).  ncols: power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// 32 lanes x 32 bit, 8 / 16 / 32 consecutive columns: thread i of the warp reads/writes TMEM lane (lane base + i).
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- descriptors ------------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, K-major, no swizzle: 8-row x 16-byte core matrices (128 contiguous bytes each);
// `lbo` = byte distance between core matrices adjacent along K, `sbo` = between 8-row groups along M/N.
__device__ __forceinline__ uint64_t smem_desc_kmajor(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version for sm_100
  return d;                 // base offset 0, layout type 0 (no swizzle)
}

// Instruction descriptor for kind::i8, signed x signed -> s32, A and B K-major, dense.
__host__ __device__ constexpr uint32_t idesc_i8(int M, int N) {
  return (2u << 4)                      // D format: s32
         | (1u << 7) | (1u << 10)       // A, B: signed 8-bit
         | ((uint32_t)(N >> 3) << 17)   // N / 8
         | ((uint32_t)(M >> 4) << 24);  // M / 16
}

// Instruction descriptor for kind::f16, fp16 x fp16 -> fp32, A and B K-major, dense.
__host__ __device__ constexpr uint32_t idesc_f16(int M, int N) {
  return (1u << 4)                      // D format: f32 (A, B formats 0 = fp16)
         | ((uint32_t)(N >> 3) << 17)   // N / 8
         | ((uint32_t)(M >> 4) << 24);  // M / 16
}

// D[tmem_d] (+)= A * B, issued by ONE thread.  accumulate = 0 overwrites D.
__device__ __forceinline__ void mma_i8_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_i8_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// fp16 operands, K = 16 per instruction: A = 8 tensor-memory columns (two values per column), B from shared memory
__device__ __forceinline__ void mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` once every MMA issued so far by this thread has completed (implies fence::before_thread_sync).
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Failure path of a kernel that holds tensor memory, called by EVERY thread of the CTA just before the memory is freed.  A
// thread whose bounded wait has expired stops waiting, so the CTA can get here with MMAs still in flight; freeing tensor
// memory under them must not happen.  If any thread reports !ok, the issuing threads (`issuer`; `bar` was initialised with
// their number) commit once more and everybody waits, again bounded, for those MMAs to retire.  One barrier-with-vote per
// kernel when nothing went wrong.
// Returns whether any thread had failed.
__device__ __forceinline__ bool drain_mmas_on_failure(bool ok, bool issuer, uint64_t* bar) {
  const bool failed = __syncthreads_or(ok ? 0 : 1) != 0;
  if (failed) {
    if (issuer) mma_commit(bar);
    mbar_wait_parked(bar, 0u);
    __syncthreads();
  }
  return failed;
}

// ---- packed fp32 pairs (sm_100 has two-wide fp32 add / mul / fma on 64-bit registers) ---------------------------------
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  return (uint64_t)__float_as_uint(lo) | ((uint64_t)__float_as_uint(hi) << 32);
}
__device__ __forceinline__ uint64_t pack2u(uint32_t lo, uint32_t hi) { return (uint64_t)lo | ((uint64_t)hi << 32); }
__device__ __forceinline__ float lo2(uint64_t v) { return __uint_as_float((uint32_t)v); }
__device__ __forceinline__ float hi2(uint64_t v) { return __uint_as_float((uint32_t)(v >> 32)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// int32 -> fp32 without the (slow) conversion unit, for |v| < 2^22: the bits of v + 0x4B400000 are the float
// 2^23 + 2^22 + v, so one integer add and one float subtract give float(v) exactly.  The reference plants the same
// constant in the MMA's C operand (lab/qwen_batched.py:1016-1041, 1237-1243); tcgen05 accumulators start from zero, so
// here it is added after the fact.
constexpr uint32_t I2F_MAGIC = 0x4B400000u;
constexpr float I2F_BIAS = 12582912.f;

// ---- nibble expansion ---------------------------------------------------------------------------------------------
// One 32-bit word = 8 nibbles q (weights 8w..8w+7).  ((q ^ 8) << 4) as a signed byte equals 16 * (q - 8), so two
// logic ops per four weights give signed int8 operands with the Q4_0 offset already applied; the factor 16 is
// exact and divides out of the int32 dot product.  `even` holds weights 0,2,4,6 of the word, `odd` 1,3,5,7.
__device__ __forceinline__ void expand_nibbles(uint32_t w, uint32_t& even, uint32_t& odd) {
  even = ((w << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
  odd = (w & 0xF0F0F0F0u) ^ 0x80808080u;
}
// The matching order for the other operand: bytes (k0,k2,k4,k6) and (k1,k3,k5,k7) of 8 consecutive int8 values
// held as two words lo = k0..k3, hi = k4..k7.
__device__ __forceinline__ void permute_bytes(uint32_t lo, uint32_t hi, uint32_t& even, uint32_t& odd) {
  even = __byte_perm(lo, hi, 0x6420);
  odd = __byte_perm(lo, hi, 0x7531);
}

}  // namespace tc
}  // namespace q4b
