// Per-block integer dot products of Q4_0 weights with int8 activations on the tcgen05 int8 tensor cores:
//   out[n, m, b] = sum_{i<32} (q4[m, 32b+i] - 8) * q8[n, 32b+i]        (exact int32)
// This is the quantity the reference's MMQ computes per k-block with mma.m16n8k32.u8.s8 plus a -8*sum(q8) correction
// in the C operand (lab/qwen_batched.py:1237-1243).  The entry point exists so tests can check the tensor-core
// operand layouts bit for bit; the MMQ kernels use the same expansion, descriptors and TMEM shapes.
//
// One CTA = 128 weight rows (UMMA M = 128) x NT activation rows (UMMA N) and walks the k-blocks one at a time:
// thread t expands row t's 16 bytes of nibbles to 32 signed bytes 16*(q-8) and places them as the A operand, either
// in shared memory (K-major core matrices, mode 0) or directly in tensor memory (tcgen05.st, mode 1); the activation
// tile goes to shared memory in the same k-permutation; one thread issues tcgen05.mma.kind::i8 (K = 32 = one Q4_0
// block); the int32 accumulator is read back from TMEM (tcgen05.ld), shifted right by 4 and stored.
#include "q4b_internal.h"
#include "tc05.cuh"

namespace q4b {

namespace {

constexpr uint32_t TMEM_COLS = 64;   // accumulator in columns [0, 32), A operand in [32, 40)

template <bool A_TMEM, int NT>
__global__ void __launch_bounds__(128) blockdot_kernel(const uint4* __restrict__ W, const int8_t* __restrict__ xq,
                                                       int32_t* __restrict__ out, int M, int K, int P, uint32_t* status) {
  __shared__ __align__(128) uint8_t sA[128 * 32];
  __shared__ __align__(128) uint8_t sB[32 * 32];
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_base_s;
  const int t = threadIdx.x, warp = t >> 5;
  const int row0 = blockIdx.x * 128, n0 = blockIdx.y * NT;
  const int KB = K >> 5;

  if (warp == 0) {
    tc::tmem_alloc(&tmem_base_s, TMEM_COLS);
    tc::tmem_relinquish();
  }
  if (t == 0) {
    tc::mbar_init(&bar, 1);
    tc::mbar_fence_init();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_base_s;
  const uint32_t tmem_d = tmem, tmem_a = tmem + 32;
  const uint32_t lane_off = (uint32_t)(32 * warp) << 16;
  constexpr uint32_t IDESC = tc::idesc_i8(128, NT);
  bool ok = true;
  uint32_t phase = 0;
  const int row = min(row0 + t, M - 1);

  for (int kb = 0; kb < KB; ++kb) {
    const uint4 w = __ldg(W + (size_t)row * KB + kb);
    uint32_t a[8];
    tc::expand_nibbles(w.x, a[0], a[1]);
    tc::expand_nibbles(w.y, a[2], a[3]);
    tc::expand_nibbles(w.z, a[4], a[5]);
    tc::expand_nibbles(w.w, a[6], a[7]);
    if (A_TMEM) {
      tc::tmem_st8(tmem_a + lane_off, a);
      tc::tmem_wait_st();
    } else {
      uint8_t* dst = sA + ((t >> 3) * 2) * 128 + (t & 7) * 16;
      *reinterpret_cast<uint4*>(dst) = make_uint4(a[0], a[1], a[2], a[3]);
      *reinterpret_cast<uint4*>(dst + 128) = make_uint4(a[4], a[5], a[6], a[7]);
    }
    if (t < NT * 2) {
      const int n = t >> 1, kc = t & 1, gn = n0 + n;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (gn < P) v = *reinterpret_cast<const uint4*>(xq + (size_t)gn * K + kb * 32 + kc * 16);
      uint32_t e0, o0, e1, o1;
      tc::permute_bytes(v.x, v.y, e0, o0);
      tc::permute_bytes(v.z, v.w, e1, o1);
      *reinterpret_cast<uint4*>(sB + ((n >> 3) * 2 + kc) * 128 + (n & 7) * 16) = make_uint4(e0, o0, e1, o1);
    }
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    if (t == 0) {
      tc::fence_after_sync();
      const uint64_t bdesc = tc::smem_desc_kmajor(tc::smem_u32(sB), 128, 256);
      if (A_TMEM) {
        tc::mma_i8_ts(tmem_d, tmem_a, bdesc, IDESC, 0u);
      } else {
        const uint64_t adesc = tc::smem_desc_kmajor(tc::smem_u32(sA), 128, 256);
        tc::mma_i8_ss(tmem_d, adesc, bdesc, IDESC, 0u);
      }
      tc::mma_commit(&bar);
    }
    ok = tc::mbar_wait(&bar, phase) && ok;
    phase ^= 1u;
    tc::fence_after_sync();
#pragma unroll
    for (int c0 = 0; c0 < NT; c0 += 8) {
      uint32_t d[8];
      tc::tmem_ld8(tmem_d + lane_off + c0, d);
      tc::tmem_wait_ld();
      if (row0 + t < M) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (n0 + c0 + j < P) out[((size_t)(n0 + c0 + j) * M + row0 + t) * KB + kb] = ((int32_t)d[j]) >> 4;
      }
    }
    tc::fence_before_sync();
    __syncthreads();          // operands and accumulator are reused by the next k-block
    tc::fence_after_sync();
  }
  if (!ok && t == 0) atomicExch(status, 1u);
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, TMEM_COLS);
}

template <bool A_TMEM>
void launch_nt(int nt, dim3 grid, size_t smem, cudaStream_t st, const uint4* W, const int8_t* xq, int32_t* out, int M,
               int K, int P, uint32_t* status) {
  if (nt == 8) blockdot_kernel<A_TMEM, 8><<<grid, 128, smem, st>>>(W, xq, out, M, K, P, status);
  else if (nt == 16) blockdot_kernel<A_TMEM, 16><<<grid, 128, smem, st>>>(W, xq, out, M, K, P, status);
  else blockdot_kernel<A_TMEM, 32><<<grid, 128, smem, st>>>(W, xq, out, M, K, P, status);
}

}  // namespace

int blockdot(const void* W, const void* xq, int32_t* out, int M, int K, int P, int mode, uint32_t* status, cudaStream_t st) {
  if (M <= 0 || P <= 0 || K <= 0 || (K % 32)) return fail(Q4B_E_SHAPE, "blockdot: M, P > 0 and K a positive multiple of 32 required");
  if (!W || !xq || !out || !status || !aligned16(W) || !aligned16(xq)) return fail(Q4B_E_ALIGN, "blockdot: null or misaligned pointer");
  const int a_tmem = mode & 1, nt_sel = mode >> 1;
  const int nt = nt_sel == 0 ? (P <= 8 ? 8 : (P <= 16 ? 16 : 32)) : nt_sel;
  if (nt != 8 && nt != 16 && nt != 32) return fail(Q4B_E_ARG, "blockdot: tile width must be 8, 16 or 32");
  dim3 grid((M + 127) / 128, (P + nt - 1) / nt);
  // 24 KB of unused dynamic shared memory caps residency at 7 CTAs per SM, so 7 x 64 TMEM columns always fit in the
  // 512 an SM has and tcgen05.alloc never has to wait for another CTA.
  const size_t smem = 24 * 1024;
  if (a_tmem) launch_nt<true>(nt, grid, smem, st, (const uint4*)W, (const int8_t*)xq, out, M, K, P, status);
  else launch_nt<false>(nt, grid, smem, st, (const uint4*)W, (const int8_t*)xq, out, M, K, P, status);
  return check_launch("blockdot");
}

}  // namespace q4b
