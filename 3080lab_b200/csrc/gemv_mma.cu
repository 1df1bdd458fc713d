// Q4_0 GEMV for ONE activation vector: bulk-copied weight slab in shared memory, mma.sync int8 with register
// accumulators, exact block dots.
//
//   y[m] = sum_b d[m, b] * 2^e_b * sum_j 256^j * dot_j[m, b],     dot_j[m, b] = sum_{i<32} (q4[m, 32b+i] - 8) * X_j[32b+i]
//
// Each 32-value block of x is written as a block-fixed-point integer X_i = rint(x_i / 2^e_b) of 30 bits and split into
// four signed base-256 digits X_0..X_3; every dot_j is an exact int32, so for fp16 x the result is the reference's
// dequantise-and-dot (lab/qwen_kernels.py:14-113, inner loop lab/experiments/gemv4.py:31-57) with no rounding inside a
// block; the roundings left are the per-block fp32 scale-and-add, as in the reference.  Epilogues are the reference's
// (lab/qwen_kernels.py:21-45) plus the fused RoPE + K/V append of its prefill GEMM (`biasf_kv`,
// lab/qwen_batched.py:1316-1362) applied to the decode QKV projection.
//
// Why this shape (B200):
//   * The weights of a CTA (one 128-row tile x one K slice of the tile-packed layout, pack.cu) are ONE contiguous
//     range.  One thread issues a handful of 1-D bulk (TMA) copies into shared memory BEFORE the programmatic-dependency
//     wait: weights never depend on the previous kernel, so the whole HBM stream of this kernel runs while its
//     predecessor is still computing.  A CTA needs at most ~125 KB of shared memory and 512 threads x <= 64 registers,
//     so the CTAs of two consecutive kernels of the decode chain fit on an SM together; that is what makes the overlap
//     real.
//   * After the wait only latency is left: stage x (RMSNorm fused), then per (32 rows x 32 weights) two
//     mma.sync.m16n8k32.s8: the k extent of the MMA is used block-diagonally (k slots 0..15 carry rows r, r+8 against
//     digit columns 0..3, k slots 16..31 carry rows r+16, r+24 against columns 4..7), so all eight columns and all four
//     accumulator registers of every lane are useful, and there is no cross-lane traffic until the final sum.
//     Per 1024 weights a warp issues ~37 instructions (12 of them the nibble expansion), a third of what the fp32
//     FMA formulation needs, and nothing waits on tensor memory, commits or mbarrier wake-ups.
//   * Split-K over the CTAs of a thread-block cluster; partial sums are pushed into the leader's shared memory and added
//     in rank order, so results are bit-repeatable.
// Every wait is bounded (status word + fall through).
#include <cstdlib>

#include "q4b_internal.h"
#include "tc05.cuh"

namespace q4b {

namespace {

constexpr int GT = 512;                 // threads per CTA: 4 row groups of 32 rows x 4 k groups
constexpr int ROWS = 128;
constexpr int CHK = 8;                  // k-blocks per bulk-copy chunk (one mbarrier each)
constexpr int MAX_CHUNKS = 12;          // at most 96 k-blocks (221 KB of weights) per CTA
constexpr int MODE_X16 = 0, MODE_X32 = 1, MODE_NORM = 3;
constexpr int EPI_ROPE_KV = Q4B_EPI_BIASF_ROPE_KV;
constexpr size_t MAX_DYN_SMEM = 226 * 1024;

struct GemvArgs {
  const uint8_t* W;      // tile-packed nibbles [T, K/32, 128, 16 bytes]
  const __half* S;       // tile-packed scales [T, K/32, 128]
  const void* X;         // fp16 / fp32 [K]; norm mode: the fp32 residual stream
  const float* NW;       // norm mode: RMSNorm weights fp32 [K]
  float eps;
  void* Y;
  const void* AUX;
  uint32_t* status;
  unsigned long long* trace;
  int N, K, KB, epi, ksplit;
  // fused RoPE + K/V append (EPI_ROPE_KV): one sequence, cache fp16 [NKV, max_len, HD]
  const float* cosT;
  const float* sinT;
  const int64_t* pos;
  __half* kc;
  __half* vc;
  int NH, NKV, HD, max_len;
  // look-ahead: up to four ranges (weights of launches further down the chain) that this grid asks to be brought into L2
  const uint8_t* pf[4];
  unsigned long long pf_bytes[4];
  // failure-path exercise (q4b_debug_gemv_mma_expired_wait): polls per wait, and a chunk whose copies are withheld
  uint32_t wait_limit;
  int withhold_chunk;
};

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   tc::smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(tc::smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// first MMA of a block: the C operand is the zero register, no accumulator initialisation
__device__ __forceinline__ void mma_s8_zero(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ bool mbar_wait_n(uint64_t* bar, uint32_t parity, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i)
    if (tc::mbar_try(bar, parity)) return true;
  return false;
}

template <int MODE>
__global__ void __launch_bounds__(GT, 2) gemv_mma_kernel(const GemvArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bar_load[MAX_CHUNKS];
  __shared__ float red_ss[GT / 32];
  __shared__ float ybuf[ROWS];

  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int rg = warp & 3, kg = warp >> 2;               // row group (32 rows), k group
  const int g = lane >> 2, tq = lane & 3;                // MMA fragment coordinates: groupID, thread in group
  const int tile = blockIdx.x, ks = blockIdx.y;
  unsigned long long* tr = (a.trace && t == 0) ? a.trace + (size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 16 : nullptr;
  int tri = 0;
  auto stamp = [&]() {
    if (tr && tri < 15) {
      unsigned long long gt;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
      tr[tri++] = gt;
      tr[15] = (unsigned long long)tri;
    }
  };
  stamp();                                                // 0: start
  pdl_launch_dependents();
  // K slice of this CTA (slices may differ by one k-block)
  const int kb0 = (int)(((long long)a.KB * ks) / a.ksplit), kb1 = (int)(((long long)a.KB * (ks + 1)) / a.ksplit);
  const int nkb = kb1 - kb0;
  const int cap = (a.KB + a.ksplit - 1) / a.ksplit;       // slab capacity in k-blocks (same for every CTA)
  uint8_t* slabW = smem;                                  // [k-block][128 rows][16 bytes]
  uint8_t* slabS = slabW + (size_t)cap * 2048;            // [k-block][128 rows] fp16
  uint8_t* xdig = slabS + (size_t)cap * 256;              // [k-block][digit 0..3][word 0..3][even, odd] int8x4
  float2* xsc = reinterpret_cast<float2*>(xdig + (size_t)cap * 128);   // [k-block] {s, 65536 s}, s = 2^e / 2^29 / 16
  float* red = reinterpret_cast<float*>(xsc + cap);       // [k group][128]
  float* red_buf = red + 4 * ROWS;                        // split-K partials pushed by the peers: [rank - 1][128]
  const int nch = (nkb + CHK - 1) / CHK;

  if (t < nch) {                                          // lane c of warp 0 owns chunk c: barrier, then its two copies
    const int c = t;
    tc::mbar_init(&bar_load[c], 1);
    tc::mbar_fence_init();
    const size_t kbg = (size_t)tile * a.KB + kb0;         // first k-block of this CTA in the packed arrays
    const int n = min(CHK, nkb - c * CHK);
    tc::mbar_expect_tx(&bar_load[c], (uint32_t)n * (2048 + 256));
    if (c != a.withhold_chunk) {                          // (debug: a withheld chunk never completes, its wait must give up)
      bulk_g2s(slabW + (size_t)c * CHK * 2048, a.W + (kbg + (size_t)c * CHK) * 2048, (uint32_t)n * 2048, &bar_load[c]);
      bulk_g2s(slabS + (size_t)c * CHK * 256, a.S + (kbg + (size_t)c * CHK) * 128, (uint32_t)n * 256, &bar_load[c]);
    }
  }
  if (warp == 1) {
    // L2 look-ahead for launches further down the chain: this CTA's share of each range, 16 KB per lane and trip.  A
    // prefetch binds nothing and needs no completion; the later kernels' own bulk copies then find the lines in L2.
    const unsigned long long ncta = (unsigned long long)gridDim.x * gridDim.y, cta = (unsigned long long)blockIdx.y * gridDim.x + blockIdx.x;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      if (!a.pf[r]) continue;
      const unsigned long long share = ((a.pf_bytes[r] + ncta - 1) / ncta + 127) & ~127ull;
      const unsigned long long lo = cta * share, hi = min(a.pf_bytes[r], lo + share);
      for (unsigned long long o = lo + (unsigned long long)lane * 16384; o < hi; o += 32ull * 16384) {
        const uint32_t n = (uint32_t)min(16384ull, hi - o) & ~15u;
        if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(a.pf[r] + o), "r"(n) : "memory");
      }
    }
  }
  __syncwarp();
  if (a.ksplit > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");   // "this CTA exists"
  // operand element of this thread: 8 threads per k-block, 4 consecutive elements each, 64 k-blocks per pass
  constexpr int MAXIT = 2;
  float4 nw[MAXIT];
  if (MODE == MODE_NORM) {
#pragma unroll
    for (int u = 0; u < MAXIT; ++u) {
      const int kbl = (t >> 3) + u * (GT / 8);
      nw[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (kbl < nkb) nw[u] = __ldg(reinterpret_cast<const float4*>(a.NW + (size_t)(kb0 + kbl) * 32 + (t & 7) * 4));
    }
  }
  __syncthreads();                                        // barriers initialised before anyone polls them
  stamp();                                                // 1: copies issued
  pdl_wait();                                             // x comes from the previous kernel
  stamp();                                                // 2: predecessor complete

  const int row = tile * ROWS + (t & (ROWS - 1));
  const bool writer = ks == 0 && t < ROWS;
  float addend = 0.f;
  if (writer && row < a.N) {
    if (a.epi == Q4B_EPI_BIASF || a.epi == EPI_ROPE_KV) addend = reinterpret_cast<const float*>(a.AUX)[row];
    if (a.epi == Q4B_EPI_RESID) addend = reinterpret_cast<const float*>(a.Y)[row];
  }
  int p = 0;
  float rc = 1.f, rs = 0.f;
  if (a.epi == EPI_ROPE_KV && writer) {                   // position -> its cos/sin entry: two dependent loads, hidden
    p = (int)a.pos[0];                                    // behind the main loop
    p = p < 0 ? 0 : (p >= a.max_len ? a.max_len - 1 : p);
    const int half = a.HD >> 1, dd = (row % a.HD) % half;
    rc = a.cosT[(size_t)p * half + dd];
    rs = a.sinT[(size_t)p * half + dd];
  }

  // ---- activations -> four int8 digit planes in shared memory
  // norm mode: this thread's share of the whole residual row (for the sum of squares) is requested first, so that it
  // and the operand elements below are one round trip to memory, not two
  constexpr int HSQ = 2;                                  // float4 per thread held in registers (K <= 4096); the rest loops
  float4 hq[HSQ];
  if (MODE == MODE_NORM) {
    const float4* hv = reinterpret_cast<const float4*>(a.X);
#pragma unroll
    for (int u = 0; u < HSQ; ++u) {
      const int i = t + u * GT;
      hq[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < (a.K >> 2)) hq[u] = hv[i];
    }
  }
  float xin[MAXIT][4];
#pragma unroll
  for (int u = 0; u < MAXIT; ++u) {
    const int kbl = (t >> 3) + u * (GT / 8);
    xin[u][0] = xin[u][1] = xin[u][2] = xin[u][3] = 0.f;
    if (kbl < nkb) {
      const size_t k = (size_t)(kb0 + kbl) * 32 + (t & 7) * 4;
      if (MODE == MODE_X16) {
        const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(a.X) + k);
        const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
        const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
        xin[u][0] = lo.x; xin[u][1] = lo.y; xin[u][2] = hi.x; xin[u][3] = hi.y;
      } else {
        const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.X) + k);
        xin[u][0] = v.x; xin[u][1] = v.y; xin[u][2] = v.z; xin[u][3] = v.w;
      }
    }
  }
  // all of this CTA's weight chunks: warp w polls chunk w (one poll chain per warp, in parallel), the block barrier
  // below publishes the async-proxy writes to everyone; the main loop then runs without touching a barrier (a poll
  // inside the loop, once per trip, was measured: each costs ~0.12 us even on a completed barrier, +40 % loop time)
  bool ok = true;
  if (lane == 0)
    for (int c = warp; c < nch; c += GT / 32) ok = mbar_wait_n(&bar_load[c], 0, a.wait_limit) && ok;
  float rnorm = 1.f;
  if (MODE == MODE_NORM) {
    // RMSNorm of the whole residual row (RMSNORM_F32W_1P, lab/qwen_kernels.py:683-705): every CTA needs the full sum
    // of squares; r = rsqrt(sum(v^2) / K + eps); x = round16(v * r * w), evaluated as (v * w) * r: r arrives last.
    const float4* hv = reinterpret_cast<const float4*>(a.X);
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < HSQ; ++u) ss += hq[u].x * hq[u].x + hq[u].y * hq[u].y + hq[u].z * hq[u].z + hq[u].w * hq[u].w;
    for (int i = t + HSQ * GT; i < (a.K >> 2); i += GT) {
      const float4 v = hv[i];
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
#pragma unroll
    for (int u = 0; u < MAXIT; ++u) {
      xin[u][0] *= nw[u].x; xin[u][1] *= nw[u].y; xin[u][2] *= nw[u].z; xin[u][3] *= nw[u].w;
    }
    ss = warp_sum(ss);
    if (lane == 0) red_ss[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < GT / 32; ++w) tot += red_ss[w];
    rnorm = rsqrtf(tot / (float)a.K + a.eps);
  }
  {
    const int sub = t & 7;
#pragma unroll
    for (int u = 0; u < MAXIT; ++u) {
      const int kbl = (t >> 3) + u * (GT / 8);
      if (kbl >= nkb) continue;                           // whole groups of 8 lanes leave together
      float x[4] = {xin[u][0], xin[u][1], xin[u][2], xin[u][3]};
      if (MODE == MODE_NORM) {
#pragma unroll
        for (int j = 0; j < 4; ++j) x[j] = __half2float(__float2half_rn(x[j] * rnorm));
      }
      float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
      const unsigned grp_mask = 0xFFu << (lane & 24);
#pragma unroll
      for (int o = 4; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(grp_mask, amax, o));
      const bool live = amax > 0.f && amax < INFINITY;
      int e = (__float_as_int(amax) >> 23) & 0xFF;        // biased exponent of the block maximum
      e = max(e, 34);                                     // tiny blocks: keep both scales normal floats
      // |x| < 2^(e - 126) maps below 2^30: X = rint(x * 2^(29 - (e - 127)))
      const float inv = __int_as_float((283 - e) << 23);
      int X[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) X[j] = live ? __float2int_rn(x[j] * inv) : 0;
      // elements 4 sub + {0, 2} are even weights of word sub / 2 (bytes 2 (sub & 1) + {0, 1} of its "even" operand
      // word), elements 4 sub + {1, 3} the same bytes of its "odd" word (see tc::expand_nibbles)
      uint8_t* base = xdig + (size_t)kbl * 128 + (sub >> 1) * 8 + (sub & 1) * 2;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int dg[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          dg[i] = (int)(int8_t)(X[i] & 0xFF);
          X[i] = (X[i] - dg[i]) >> 8;
        }
        *reinterpret_cast<uint16_t*>(base + j * 32) = (uint16_t)((dg[0] & 0xFF) | ((dg[2] & 0xFF) << 8));
        *reinterpret_cast<uint16_t*>(base + j * 32 + 4) = (uint16_t)((dg[1] & 0xFF) | ((dg[3] & 0xFF) << 8));
      }
      if (sub == 0) {
        const float s = live ? __int_as_float((e - 33) << 23) : 0.f;     // 2^(e - 127) / 2^29 / 16
        xsc[kbl] = make_float2(s, s * 65536.f);
      }
    }
  }
  __syncthreads();
  stamp();                                                // 3: activation operand staged

  // ---- main loop: this warp owns rows rg * 32 .. + 31 and k-blocks kg, kg + 4, ...; two k-blocks per trip so that the
  // shared-memory loads and the MMA chain of one overlap the other's
  float acc0 = 0.f, acc1 = 0.f;                           // rows rA, rA + 8, digit pair (tq & 1)
  const int rA = rg * 32 + g + 16 * (tq >> 1);
  const uint32_t m0 = g < 4 ? 0xFFFFFFFFu : 0u, m1 = ~m0;
  const uint8_t* wp0 = slabW + (size_t)(rg * 32 + g) * 16 + 4 * tq;
  const uint8_t* xp0 = xdig + ((g & 3) * 4 + tq) * 8;
  const __half* sp0 = reinterpret_cast<const __half*>(slabS) + rA;
  const float* xs0 = reinterpret_cast<const float*>(xsc) + (tq & 1);
  auto block_dot = [&](int kb, float& sA, float& fA, float& sB, float& fB) {   // -> scale and integer dot of rows rA, rA + 8
    const uint8_t* wp = wp0 + (size_t)kb * 2048;
    const uint32_t w0 = *reinterpret_cast<const uint32_t*>(wp);
    const uint32_t w1 = *reinterpret_cast<const uint32_t*>(wp + 8 * 16);
    const uint32_t w2 = *reinterpret_cast<const uint32_t*>(wp + 16 * 16);
    const uint32_t w3 = *reinterpret_cast<const uint32_t*>(wp + 24 * 16);
    const uint2 xw = *reinterpret_cast<const uint2*>(xp0 + (size_t)kb * 128);
    const float xs = xs0[2 * kb];
    const float dA = __half2float(sp0[kb * 128]), dB = __half2float(sp0[kb * 128 + 8]);
    int c[4];
    uint32_t e0, o0, e1, o1, e2, o2, e3, o3;
    tc::expand_nibbles(w0, e0, o0);
    tc::expand_nibbles(w1, e1, o1);
    tc::expand_nibbles(w2, e2, o2);
    tc::expand_nibbles(w3, e3, o3);
    mma_s8_zero(c, e0, e1, e2, e3, xw.x & m0, xw.x & m1); // even weights of the four words
    mma_s8(c, o0, o1, o2, o3, xw.y & m0, xw.y & m1);      // odd weights
    sA = dA * xs;
    sB = dB * xs;
    fA = (float)(c[0] + (c[1] << 8));
    fB = (float)(c[2] + (c[3] << 8));
  };
  int kb = kg;
  for (; kb + 4 < nkb; kb += 8) {
    float sa0, fa0, sb0, fb0, sa1, fa1, sb1, fb1;
    block_dot(kb, sa0, fa0, sb0, fb0);
    block_dot(kb + 4, sa1, fa1, sb1, fb1);
    stamp();                                              // (thread 0 only) one per trip, while the trace has room
    acc0 = fmaf(sa1, fa1, fmaf(sa0, fa0, acc0));          // k-blocks in ascending order
    acc1 = fmaf(sb1, fb1, fmaf(sb0, fb0, acc1));
  }
  if (kb < nkb) {
    float sa0, fa0, sb0, fb0;
    block_dot(kb, sa0, fa0, sb0, fb0);
    acc0 = fmaf(sa0, fa0, acc0);
    acc1 = fmaf(sb0, fb0, acc1);
  }
  acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);          // low digit pair + high digit pair
  acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
  if ((tq & 1) == 0) {
    red[kg * ROWS + rA] = acc0;
    red[kg * ROWS + rA + 8] = acc1;
  }
  __syncthreads();
  stamp();                                                // 4: main loop done
  float v = 0.f;
  if (t < ROWS) v = (red[t] + red[ROWS + t]) + (red[2 * ROWS + t] + red[3 * ROWS + t]);

  // ---- split-K: peers push their partial sums into the leader's shared memory, the leader adds them in rank order
  if (a.ksplit > 1) {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // pairs with the arrive above
    if (ks != 0 && t < ROWS) {
      uint32_t remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(tc::smem_u32(red_buf)), "r"(0));
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + (uint32_t)(((ks - 1) * ROWS + t) * 4)), "f"(v) : "memory");
    }
    cluster_sync_all();
    if (ks == 0 && t < ROWS)
      for (int r = 1; r < a.ksplit; ++r) v += red_buf[(r - 1) * ROWS + t];
  }
  stamp();                                                // 5: split-K reduced
  if (!ok) atomicOr(a.status, 1u);
  if (ks != 0) return;

  if (a.epi == EPI_ROPE_KV) {
    // bias, round to fp16; q and k heads are then rotated (NeoX pairs d, d + HD/2, both inside this tile) from the
    // ROUNDED values and rounded again; k and v go straight into the cache row of the current position.
    const float y16 = __half2float(__float2half_rn(v + addend));
    if (t < ROWS) ybuf[t] = y16;
    __syncthreads();
    if (t < ROWS && row < a.N) {
      const int head = row / a.HD, d = row - head * a.HD, half = a.HD >> 1;
      const float other = ybuf[d < half ? t + half : t - half];
      const __half rot = __float2half_rn(d < half ? y16 * rc - other * rs : y16 * rc + other * rs);
      __half* Y = reinterpret_cast<__half*>(a.Y);
      if (head < a.NH) {
        Y[row] = rot;
      } else if (head < a.NH + a.NKV) {
        Y[row] = rot;
        a.kc[((size_t)(head - a.NH) * a.max_len + p) * a.HD + d] = rot;
      } else {
        const __half y = __float2half_rn(y16);
        Y[row] = y;
        a.vc[((size_t)(head - a.NH - a.NKV) * a.max_len + p) * a.HD + d] = y;
      }
    }
    return;
  }
  if (t >= ROWS) return;
  const float partner = __shfl_xor_sync(0xffffffffu, v, 1);
  if (row >= a.N) return;
  switch (a.epi) {
    case Q4B_EPI_STORE: reinterpret_cast<__half*>(a.Y)[row] = __float2half_rn(v); break;
    case Q4B_EPI_BIASF: reinterpret_cast<__half*>(a.Y)[row] = __float2half_rn(v + addend); break;
    case Q4B_EPI_RESID: reinterpret_cast<float*>(a.Y)[row] = addend + v; break;
    case Q4B_EPI_LOGITS: reinterpret_cast<float*>(a.Y)[row] = v; break;
    case Q4B_EPI_SWIGLU:
      if ((t & 1) == 0) reinterpret_cast<__half*>(a.Y)[row >> 1] = __float2half_rn(v / (1.f + __expf(-v)) * partner);
      break;
    default: break;
  }
}

unsigned long long* g_trace = nullptr;

size_t smem_for(int cap) { return (size_t)cap * (2048 + 256 + 128 + 8) + (4 + 7) * ROWS * sizeof(float); }

template <int MODE>
int configure(size_t bytes) {
  // cudaFuncSetAttribute is per device: remember, per device, the largest size asked for so far
  static size_t configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(Q4B_E_CUDA, "gemv_q4_0_mma: no current device");
  prefer_max_shared(reinterpret_cast<const void*>(&gemv_mma_kernel<MODE>));
  if (bytes > configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_mma_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_DYN_SMEM);
    if (e != cudaSuccess) {
      set_cuda_error(e, "gemv_q4_0_mma");
      return Q4B_E_CUDA;
    }
    configured[dev] = MAX_DYN_SMEM;
  }
  return Q4B_OK;
}

}  // namespace

void gemv_mma_trace(unsigned long long* buf) { g_trace = buf; }

// Grid geometry: tiles x K slices.  Slices fill the SMs when there are fewer row tiles than SMs (cluster size <= 8) and
// keep a CTA's slab inside shared memory; -1 if the shape cannot be covered.
int gemv_mma_ksplit(int N, int K) {
  const int T = (N + ROWS - 1) / ROWS, KB = K / 32;
  int ks = sm_count() / T;
  ks = ks < 1 ? 1 : (ks > 8 ? 8 : ks);
  if (ks > KB) ks = KB;
  while (ks <= 8 && ((KB + ks - 1) / ks > CHK * MAX_CHUNKS || smem_for((KB + ks - 1) / ks) > MAX_DYN_SMEM)) ++ks;
  return ks <= 8 ? ks : -1;
}

int gemv_mma(const void* W, const void* S, const void* X, void* Y, const void* AUX, int N, int K, int mode, int epi,
             uint32_t* status, cudaStream_t st, const float* norm_w, float eps, const float* cosT, const float* sinT,
             const int64_t* pos, void* kc, void* vc, int NH, int NKV, int HD, int max_len, int withhold_chunk,
             const GemvLookahead* look) {
  if (N <= 0 || K <= 0 || (K % 32)) return fail(Q4B_E_SHAPE, "gemv_q4_0_mma: N > 0 and K a positive multiple of 32 required");
  if (!W || !S || !X || !Y || !status || !aligned16(W) || !aligned16(S) || !aligned16(X))
    return fail(Q4B_E_ALIGN, "gemv_q4_0_mma: null or misaligned pointer");
  if (epi < Q4B_EPI_STORE || epi > EPI_ROPE_KV || epi == Q4B_EPI_SWIGLU_Q8) return fail(Q4B_E_ARG, "gemv_q4_0_mma: unknown epilogue");
  if ((epi == Q4B_EPI_BIASF || epi == EPI_ROPE_KV) && !AUX) return fail(Q4B_E_ALIGN, "gemv_q4_0_mma: this epilogue needs AUX");
  if (epi == Q4B_EPI_SWIGLU && (N % 2)) return fail(Q4B_E_SHAPE, "gemv_q4_0_mma: swiglu needs an even row count");
  if (mode == MODE_NORM && !norm_w) return fail(Q4B_E_ALIGN, "gemv_q4_0_mma: norm weights missing");
  if (epi == EPI_ROPE_KV) {
    if (!cosT || !sinT || !pos || !kc || !vc) return fail(Q4B_E_ALIGN, "gemv_q4_0_mma: rope/kv epilogue needs tables, pos and the cache");
    if (HD <= 0 || (ROWS % HD) || (HD % 2) || NH <= 0 || NKV <= 0 || N != (NH + 2 * NKV) * HD || max_len <= 0)
      return fail(Q4B_E_SHAPE, "gemv_q4_0_mma: rope/kv epilogue needs head_dim dividing 128 and N = (NH + 2 NKV) head_dim");
  }
  const int ks = gemv_mma_ksplit(N, K);
  if (ks < 0) return fail(Q4B_E_SHAPE, "gemv_q4_0_mma: K too long for one cluster of 8 CTAs");
  const int T = (N + ROWS - 1) / ROWS, KB = K / 32, cap = (KB + ks - 1) / ks;
  const size_t smem = smem_for(cap);
  GemvArgs a{};
  a.W = reinterpret_cast<const uint8_t*>(W);
  a.S = reinterpret_cast<const __half*>(S);
  a.X = X;
  a.NW = norm_w;
  a.eps = eps;
  a.Y = Y;
  a.AUX = AUX;
  a.status = status;
  a.trace = g_trace;
  if (unsigned long long* slot = trace_slot(1, T * ks)) a.trace = slot;
  a.N = N; a.K = K; a.KB = KB; a.epi = epi; a.ksplit = ks;
  a.cosT = cosT; a.sinT = sinT; a.pos = pos;
  a.kc = reinterpret_cast<__half*>(kc); a.vc = reinterpret_cast<__half*>(vc);
  a.NH = NH; a.NKV = NKV; a.HD = HD; a.max_len = max_len;
  a.withhold_chunk = withhold_chunk;
  for (int r = 0; r < 4; ++r) {
    const bool on = look && look->ptr[r] && look->bytes[r] >= 16 && aligned16(look->ptr[r]);
    a.pf[r] = on ? reinterpret_cast<const uint8_t*>(look->ptr[r]) : nullptr;
    a.pf_bytes[r] = on ? (unsigned long long)look->bytes[r] : 0ull;
  }
  a.wait_limit = withhold_chunk >= 0 ? 4096u : tc::WAIT_LIMIT;
  dim3 grid(T, ks), block(GT);
  int rc;
  cudaError_t e;
  switch (mode) {
    case MODE_X16:
      if ((rc = configure<MODE_X16>(smem)) != Q4B_OK) return rc;
      e = launch_pdl_cluster(gemv_mma_kernel<MODE_X16>, grid, block, smem, st, 1, ks, a);
      break;
    case MODE_X32:
      if ((rc = configure<MODE_X32>(smem)) != Q4B_OK) return rc;
      e = launch_pdl_cluster(gemv_mma_kernel<MODE_X32>, grid, block, smem, st, 1, ks, a);
      break;
    case MODE_NORM:
      if ((rc = configure<MODE_NORM>(smem)) != Q4B_OK) return rc;
      e = launch_pdl_cluster(gemv_mma_kernel<MODE_NORM>, grid, block, smem, st, 1, ks, a);
      break;
    default: return fail(Q4B_E_ARG, "gemv_q4_0_mma: unknown mode");
  }
  return check_launch(e, "gemv_q4_0_mma");
}

}  // namespace q4b
