// Batched-decode Q4_0 linear for 1 .. 32 activation rows on mma.sync tensor-core instructions, in two arithmetics:
//
// MODE_Q8 (the int8 route of the batched decode step): Q8_1 activations, the block arithmetic of the reference's MMQ
//   (gemm_q4i8_ms_source, lab/qwen_batched.py:1237-1243):
//     Y[b, m] = epilogue( sum_blocks (d_w[m, blk] * d_x[b, blk]) * dot[m, b, blk] ),   dot = exact int32 over 32 weights
//   mma.sync.m16n8k32.s8 with the accumulator started from 0x4B400000, so that float(dot) is one subtraction; the scale
//   product and the fused multiply-add per output and block run on the CUDA cores, accumulators stay in registers.
//   (The tcgen05 form of the same arithmetic, mmq_stream.cu, needs one accumulator tile per block and those retire one per
//   177 clocks; at these row counts the register form is faster.)
//
// MODE_F16: fp16 activations against weights dequantised to fp16, the reference's own batched-decode GEMV
//   (gemv_v2_source, lab/qwen_batched.py:467-641):
//     Y[b, m] = epilogue( sum_k w16[m, k] * X[b, k] ),    w16[m, k] = round_fp16( (q4[m, k] - 8) * d[m, k / 32] )
//   nibbles become exact fp16 integers through the 0x6400 exponent trick, are multiplied by the fp16 block scale with ONE
//   rounding to fp16, and meet the fp16 activations in mma.sync.m16n8k16 with fp32 accumulation.  That rounding is what
//   separates this mode from the exact block-dot kernels; tests compare against an oracle that rounds the same way.
//
// Epilogues as lab/qwen_batched.py:251-267 (+ swiglu_q8, :1363-1396, in MODE_Q8).
//
// Shape of the kernel (B200), shared with the batch-1 GEMV of gemv_mma.cu:
//   * one CTA = one 128-row tile x one K slice of the tile-packed layout (pack.cu): its weights are ONE contiguous range,
//     fetched by a few 1-D bulk copies BEFORE the programmatic-dependency wait; after the wait one bulk copy per
//     activation row brings the K slice of X into a padded (conflict-free) shared-memory image;
//   * 16 warps = 4 row groups (two m16 tiles each) x 4 k groups; a lane reads 4 bytes of nibbles per row and k-block
//     and keeps that natural byte order: logical k slots of the MMA are a permutation of the block's 32 weights, and the
//     activation fragment is permuted to match with two byte-permutes, so no repacked weight copy is needed;
//   * the k groups are added in a fixed order through shared memory, K slices through the thread-block cluster
//     (every CTA pushes the partial sums of the rows it does not finish to their owner, one cluster barrier, the owner
//     adds in rank order): bit-repeatable.
// Every wait is bounded (status word + fall through).
#include <algorithm>
#include <cstdio>
#include <map>
#include <mutex>
#include <tuple>

#include "q4b_internal.h"
#include "tc05.cuh"

namespace q4b {

namespace {

constexpr int GT = 512;
constexpr int ROWS = 128;
constexpr int CHK = 8;                  // k-blocks per weight bulk copy
constexpr int MAX_CHUNKS = 12;
constexpr int PSTR = ROWS + 4;          // row pitch of the partial-sum tile (floats): fragment stores hit 32 banks
constexpr size_t MAX_DYN_SMEM = 226 * 1024;

struct F16Args {
  const uint8_t* W;      // tile-packed nibbles [T, K/32, 128, 16 bytes]
  const __half* S;       // tile-packed scales [T, K/32, 128]
  const __half* X;       // fp16 [B, K]                      (MODE_F16)
  const int8_t* XQ;      // Q8_1 values int8 [B, K]           (MODE_Q8)
  const __half* XD;      // Q8_1 block scales fp16 [B, K/32]  (MODE_Q8)
  void* Y;               // [B, ldy]
  const void* AUX;
  uint32_t* status;
  int N, K, KB, B, epi, ldy, ksplit, cap;
  uint32_t wait_limit;
};

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   tc::smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(tc::smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// int8 MMA whose accumulator starts from the constant 0x4B400000 in every lane: read as a float the result is
// 2^23 + 2^22 + dot, so one subtraction gives float(dot) exactly (|dot| < 2^22); the reference plants the same constant in
// the C operand of its int8 MMQ (lab/qwen_batched.py:1237-1243).
__device__ __forceinline__ void mma_s8_magic(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0x4B400000));
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }

// Two nibbles of `w` (bit positions 0-3 and 16-19, or 4-7 and 20-23) -> fp16 pair round((q - 8) * d).
// low form: (q | 0x6400) is the fp16 1024 + q, minus 1032 is q - 8 exactly; high form (nibble at bits 4-7 / 20-23):
// 1024 + 16 q, times 1/16 minus 72 is q - 8 exactly as well (one fused multiply-add, no rounding: the result is an integer
// of at most 4 bits).  The product with d rounds once, as the reference's __hmul2 does.
__device__ __forceinline__ uint32_t deq_lo(uint32_t w, __half2 d2) {
  const uint32_t h = (w & 0x000F000Fu) | 0x64006400u;
  return h2_as_u32(__hmul2(__hsub2(u32_as_h2(h), __float2half2_rn(1032.f)), d2));
}
__device__ __forceinline__ uint32_t deq_hi(uint32_t w, __half2 d2) {
  const uint32_t h = (w & 0x00F000F0u) | 0x64006400u;
  return h2_as_u32(__hmul2(__hfma2(u32_as_h2(h), __float2half2_rn(0.0625f), __float2half2_rn(-72.f)), d2));
}

__device__ __forceinline__ bool mbar_wait_n(uint64_t* bar, uint32_t parity, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i)
    if (tc::mbar_try(bar, parity)) return true;
  return false;
}

// bytes per staged activation row: an odd multiple of 64, so that the 16-byte fragment reads of a quarter warp (two
// rows x 64 bytes) fall into distinct banks
__host__ __device__ __forceinline__ size_t x_pitch(int cap) { return (size_t)(cap | 1) * 64; }

// bytes per staged row of int8 activations (MODE_Q8): 32 mod 128, so that the 8-byte fragment reads of a half warp (four
// rows x 32 bytes) fall into distinct banks
__host__ __device__ __forceinline__ size_t xq_pitch(int cap) { return ((size_t)cap * 32 + 127) / 128 * 128 + 32; }

// bytes of the region that holds the weight slab during the main loop and the partial-sum tiles after it
__host__ __device__ __forceinline__ size_t slab_region(int cap, int nt) {
  const size_t slab = (size_t)cap * (2048 + 256), part = (size_t)(nt == 1 ? 4 : 1) * nt * 8 * PSTR * sizeof(float);
  return ((slab > part ? slab : part) + 127) / 128 * 128;
}

constexpr int MODE_F16 = 0, MODE_Q8 = 1, MODE_Q8F = 2;   // Q8F: Q8 arithmetic, fp16 activations quantised inside

// MODE_F16: fp16 activations, weights dequantised to fp16 (the reference's batched-decode GEMV).
// MODE_Q8:  Q8_1 activations (int8 values + fp16 block scales), exact int32 block dots by mma.sync.m16n8k32.s8 with register
//           accumulators, rescaled per block in fp32: acc += (d_w / 16 * d_x) * float(dot), the block arithmetic of the
//           reference's MMQ (lab/qwen_batched.py:1237-1243) for up to 32 activation rows.
template <int NT, int MODE>
__global__ void __launch_bounds__(GT, NT <= 2 ? 2 : 1) gemv_f16mma_kernel(const F16Args a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bar_load[MAX_CHUNKS];
  __shared__ __align__(8) uint64_t bar_x;

  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int rg = warp & 3, kg = warp >> 2;
  const int g = lane >> 2, tq = lane & 3;
  const int tile = blockIdx.x, ks = blockIdx.y;
  pdl_launch_dependents();
  if (a.ksplit > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");   // "this CTA exists"
  const int kb0 = (int)(((long long)a.KB * ks) / a.ksplit), kb1 = (int)(((long long)a.KB * (ks + 1)) / a.ksplit);
  const int nkb = kb1 - kb0;
  const int cap = a.cap;                                  // k-blocks per window of the slab (nkb <= cap except for very long K)
  constexpr bool Q8 = MODE != MODE_F16;                   // int8 block-dot arithmetic (activations given as Q8_1, or quantised here)
  const size_t xp = Q8 ? xq_pitch(cap) : x_pitch(cap);
  uint8_t* slabW = smem;                                  // [k-block][128 rows][16 bytes]
  uint8_t* slabS = slabW + (size_t)cap * 2048;            // [k-block][128 rows] fp16
  uint8_t* xs = smem + slab_region(cap, NT);              // [8 NT rows][pitch]: the K window of X (fp16, or int8 permuted)
  float* dxs = reinterpret_cast<float*>(xs + (size_t)NT * 8 * xp);   // MODE_Q8: [k-block][8 NT] block scales / 16 as fp32
  // The partial-sum tiles [8 NT columns][PSTR] live over the weight slab, which is dead once the main loop is done (the
  // slab region is sized for whichever is larger): 17 KB less per CTA at 8 rows, which is what lets gate/up (124 KB) and
  // down (95 KB) share an SM, so that down's weight copies run under gate/up.  The receive buffer of the K-slice reduction
  // is written by PEERS while this CTA may still be in its loop, so it keeps a region of its own.
  // Measured per mode at 8 rows: the int8 step gains 5 % from it (1192 -> 1130 us); the fp16-weight step LOSES 18 % (1040 ->
  // 1230 us: its down launch, then two CTAs per SM, takes 9.8 instead of 7.1 us), so that mode keeps tiles of its own.
  // (The maximum shared-memory carve-out on these kernels was measured too: slower in both modes.)
  float* recv = dxs + (Q8 ? (size_t)cap * NT * 8 : 0);    // [rank][column][maxp] float2
  float* P = Q8 ? reinterpret_cast<float*>(smem)
                : recv + (a.ksplit > 1 ? (size_t)NT * 8 * (ROWS / 2 + 8) * 2 : 0);

  // window `win` covers k-blocks kb0 + win cap .. of this CTA's slice; lane c of warp 0 owns weight chunk c
  auto issue_weights = [&](int win) {
    const int wkb = min(cap, nkb - win * cap), c = t;
    if (c * CHK < wkb) {
      const size_t kbg = (size_t)tile * a.KB + kb0 + (size_t)win * cap;
      const int n = min(CHK, wkb - c * CHK);
      tc::mbar_expect_tx(&bar_load[c], (uint32_t)n * (2048 + 256));
      bulk_g2s(slabW + (size_t)c * CHK * 2048, a.W + (kbg + (size_t)c * CHK) * 2048, (uint32_t)n * 2048, &bar_load[c]);
      bulk_g2s(slabS + (size_t)c * CHK * 256, a.S + (kbg + (size_t)c * CHK) * 128, (uint32_t)n * 256, &bar_load[c]);
    }
  };
  auto issue_x = [&](int win) {                           // warp 1: one bulk copy per activation row
    const int wkb = min(cap, nkb - win * cap);
    if (lane == 0) tc::mbar_expect_tx(&bar_x, (uint32_t)a.B * (uint32_t)wkb * 64u);
    __syncwarp();
    if (lane < a.B)
      bulk_g2s(xs + (size_t)lane * xp, a.X + (size_t)lane * a.K + ((size_t)kb0 + (size_t)win * cap) * 32, (uint32_t)wkb * 64u, &bar_x);
  };

  if (t < MAX_CHUNKS) {
    tc::mbar_init(&bar_load[t], 1);
    tc::mbar_fence_init();
    issue_weights(0);                                     // weights do not depend on the previous kernel
  }
  if (t == 32) {
    tc::mbar_init(&bar_x, 1);
    tc::mbar_fence_init();
  }
  // activation rows B .. 8 NT - 1 do not exist: their MMA columns read zeros
  for (int i = t; i < (NT * 8 - a.B) * (int)(xp / 16); i += GT)
    reinterpret_cast<uint4*>(xs + (size_t)a.B * xp)[i] = make_uint4(0u, 0u, 0u, 0u);
  if (Q8)
    for (int i = t; i < cap * NT * 8; i += GT) dxs[i] = 0.f;
  __syncthreads();
  pdl_wait();                                             // X comes from the previous kernel
  if (MODE == MODE_F16 && warp == 1) issue_x(0);
  // MODE_Q8: up to 16 rows the int8 rows arrive by bulk copy like the fp16 ones (one round trip; as plain loads in a loop
  // they were three dependent ones) and `permute_q8`, after the copies have landed, reorders the bytes of each group of
  // eight in place to (k0, k2, k4, k6 | k1, k3, k5, k7), the order the expansion gives the weights.  With more rows the
  // in-place pass costs more than it saves (down at 32 rows 12.9 against 12.2 us), so they keep plain loads that reorder on
  // the way.  The block scales come by plain loads either way (fp32, with the factor 1/16 of the nibble expansion).
  constexpr bool XQ_BULK = NT <= 2;
  auto stage_q8 = [&](int win) {
    const int wkb = min(cap, nkb - win * cap);
    const size_t kbase = (size_t)kb0 + (size_t)win * cap;
    if (XQ_BULK) {
      if (warp == 1) {
        if (lane == 0) tc::mbar_expect_tx(&bar_x, (uint32_t)a.B * (uint32_t)wkb * 32u);
        __syncwarp();
        if (lane < a.B) bulk_g2s(xs + (size_t)lane * xp, a.XQ + (size_t)lane * a.K + kbase * 32, (uint32_t)wkb * 32u, &bar_x);
      }
    } else {
      for (int i = t; i < a.B * wkb * 4; i += GT) {         // plain 8-byte loads, reordered on the way
        const int col = i / (wkb * 4), r = i - col * (wkb * 4);
        const uint2 v = *reinterpret_cast<const uint2*>(a.XQ + (size_t)col * a.K + kbase * 32 + (size_t)r * 8);
        uint2 o;
        tc::permute_bytes(v.x, v.y, o.x, o.y);
        *reinterpret_cast<uint2*>(xs + (size_t)col * xp + (size_t)r * 8) = o;
      }
    }
    for (int i = t; i < a.B * wkb; i += GT) {
      const int col = i / wkb, kb = i - col * wkb;
      dxs[kb * NT * 8 + col] = __half2float(a.XD[(size_t)col * a.KB + kbase + kb]) * 0.0625f;
    }
  };
  auto permute_q8 = [&](int wkb) {
    for (int i = t; i < a.B * wkb * 4; i += GT) {
      const int col = i / (wkb * 4), r = i - col * (wkb * 4);
      uint2* p8 = reinterpret_cast<uint2*>(xs + (size_t)col * xp + (size_t)r * 8);
      const uint2 v = *p8;
      uint2 o;
      tc::permute_bytes(v.x, v.y, o.x, o.y);
      *p8 = o;
    }
  };
  // MODE_Q8 with fp16 activations given: the Q8_1 quantiser of quant_q8_1.cu (QUANT_Q8, lab/qwen_batched.py:1030-1039) runs
  // here on this CTA's K window, eight lanes per 32-value block, so no separate quantiser launch is needed; values and
  // scales are the ones that launch would have written (the scale goes through fp16 as it does there).
  auto stage_q8_from_f16 = [&](int win) {
    const int wkb = min(cap, nkb - win * cap);
    const size_t kbase = (size_t)kb0 + (size_t)win * cap;
    const int total = a.B * wkb * 8;
    for (int i0 = 0; i0 < total; i0 += GT) {              // whole warps stay in the loop: the shuffles need every lane
      const int i = i0 + t;
      const bool live = i < total;
      const int blk = (live ? i : 0) >> 3, sub = i & 7;
      const int col = blk / wkb, kb = blk - col * wkb;
      float x[4] = {0.f, 0.f, 0.f, 0.f};
      if (live) {
        const uint2 raw = *reinterpret_cast<const uint2*>(a.X + (size_t)col * a.K + (kbase + kb) * 32 + sub * 4);
        const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
        const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
        x[0] = lo.x; x[1] = lo.y; x[2] = hi.x; x[3] = hi.y;
      }
      float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
      for (int o = 4; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float d = amax / 127.f;
      int q[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) q[j] = d > 0.f ? __float2int_rn(x[j] / d) : 0;
      if (live) {
        uint8_t* dst = xs + (size_t)col * xp + (size_t)kb * 32 + (sub >> 1) * 8 + (sub & 1) * 2;
        *reinterpret_cast<uint16_t*>(dst) = (uint16_t)((q[0] & 0xFF) | ((q[2] & 0xFF) << 8));
        *reinterpret_cast<uint16_t*>(dst + 4) = (uint16_t)((q[1] & 0xFF) | ((q[3] & 0xFF) << 8));
        if (sub == 0) dxs[kb * NT * 8 + col] = __half2float(__float2half_rn(d)) * 0.0625f;
      }
    }
  };
  // (the quantising form is a template instance of its own: with both stagings in one kernel the plain Q8_1 form ran
  // 0.9 us per launch slower inside the decode step, though not in isolation)
  if (MODE == MODE_Q8) stage_q8(0);
  if (MODE == MODE_Q8F) stage_q8_from_f16(0);

  // ---- main loop: rows rg * 32 + {g, g + 8, g + 16, g + 24}, k-blocks kg, kg + 4, ... of each window
  // A lane holds word tq of each row's 16 bytes (nibble i = weight 8 tq + i).  Logical k slot -> weight of the block:
  // MMA 0 (nibbles 0, 4, 2, 6) slot 2 tq + {0, 1, 8, 9} = weight 8 tq + {0, 4, 2, 6}; MMA 1 (nibbles 1, 5, 3, 7) the same + 1.
  float c[2][NT][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int n = 0; n < NT; ++n) c[m][n][0] = c[m][n][1] = c[m][n][2] = c[m][n][3] = 0.f;
  const uint8_t* wp0 = slabW + (size_t)(rg * 32 + g) * 16 + 4 * tq;
  const __half* sp0 = reinterpret_cast<const __half*>(slabS) + rg * 32 + g;
  const uint8_t* xp0 = xs + (size_t)g * xp + tq * 16;
  bool ok = true;
  const int nwin = (nkb + cap - 1) / cap;
#pragma unroll 1
  for (int win = 0; win < nwin; ++win) {
    const int wkb = min(cap, nkb - win * cap);
    const uint32_t parity = (uint32_t)win & 1u;
    if (win > 0) {
      // every warp is done reading the previous window (the barrier closing the loop body); order those generic-proxy
      // reads before the bulk copies that overwrite the slab
      tc::fence_async_smem();
      if (t < MAX_CHUNKS) issue_weights(win);
      if (MODE == MODE_F16 && warp == 1) issue_x(win);
      if (MODE == MODE_Q8) stage_q8(win);
      if (MODE == MODE_Q8F) stage_q8_from_f16(win);
    }
    // warp w polls weight chunk w, the last warp the activations; the block barrier publishes the bulk-copied bytes to
    // everyone.  (Polling each chunk inside the loop instead, to start the MMAs while later chunks are in flight, was
    // measured slower: gate/up at 8 rows 7.9 us against 7.0.)
    if (lane == 0) {
      for (int ch = warp; ch * CHK < wkb; ch += GT / 32) ok = mbar_wait_n(&bar_load[ch], parity, a.wait_limit) && ok;
      if ((MODE == MODE_F16 || (MODE == MODE_Q8 && XQ_BULK)) && warp == GT / 32 - 1) ok = mbar_wait_n(&bar_x, parity, a.wait_limit) && ok;
    }
    __syncthreads();
    if (MODE == MODE_Q8 && XQ_BULK) {
      permute_q8(wkb);
      __syncthreads();
    }
    if (Q8) {
      // A fragment of an m16 tile: a0 / a2 = even / odd weights of row g's word tq, a1 / a3 the same of row g + 8; the
      // activation bytes were staged in the matching order, so lane tq reads its 8 bytes of column g in one load.
      const uint8_t* xq0 = xs + (size_t)g * xp + tq * 8;
#pragma unroll 1
      for (int kb = kg; kb < wkb; kb += 4) {
        uint32_t w[4];
        float dw[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          w[r] = *reinterpret_cast<const uint32_t*>(wp0 + (size_t)kb * 2048 + r * 8 * 16);
          dw[r] = __half2float(sp0[kb * 128 + r * 8]);
        }
        uint2 xb[NT];
        float2 dx[NT];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          xb[n] = *reinterpret_cast<const uint2*>(xq0 + (size_t)n * 8 * xp + (size_t)kb * 32);
          dx[n] = *reinterpret_cast<const float2*>(dxs + kb * NT * 8 + n * 8 + 2 * tq);
        }
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          uint32_t eA, oA, eB, oB;
          tc::expand_nibbles(w[2 * m], eA, oA);
          tc::expand_nibbles(w[2 * m + 1], eB, oB);
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            int d[4];
            mma_s8_magic(d, eA, eB, oA, oB, xb[n].x, xb[n].y);
            // (two-wide fp32 instructions for these - half the issue slots at the same lane throughput - were measured:
            // gate/up at 32 rows 15.0 against 14.5 us, at 8 rows 6.6 against 6.8; not kept)
            c[m][n][0] = fmaf(dw[2 * m] * dx[n].x, __int_as_float(d[0]) - 12582912.f, c[m][n][0]);
            c[m][n][1] = fmaf(dw[2 * m] * dx[n].y, __int_as_float(d[1]) - 12582912.f, c[m][n][1]);
            c[m][n][2] = fmaf(dw[2 * m + 1] * dx[n].x, __int_as_float(d[2]) - 12582912.f, c[m][n][2]);
            c[m][n][3] = fmaf(dw[2 * m + 1] * dx[n].y, __int_as_float(d[3]) - 12582912.f, c[m][n][3]);
          }
        }
      }
    } else
#pragma unroll 1
    for (int kb = kg; kb < wkb; kb += 4) {
      uint32_t w[4];
      __half2 d2[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        w[r] = *reinterpret_cast<const uint32_t*>(wp0 + (size_t)kb * 2048 + r * 8 * 16);
        d2[r] = __half2half2(sp0[kb * 128 + r * 8]);
      }
      uint32_t b[NT][4];                                  // {MMA 0 b0, MMA 0 b1, MMA 1 b0, MMA 1 b1}
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const uint4 x = *reinterpret_cast<const uint4*>(xp0 + (size_t)n * 8 * xp + (size_t)kb * 64);   // x[8 tq .. 8 tq + 7]
        b[n][0] = __byte_perm(x.x, x.z, 0x5410);          // x[8 tq + 0], x[8 tq + 4]
        b[n][1] = __byte_perm(x.y, x.w, 0x5410);          // x[8 tq + 2], x[8 tq + 6]
        b[n][2] = __byte_perm(x.x, x.z, 0x7632);          // x[8 tq + 1], x[8 tq + 5]
        b[n][3] = __byte_perm(x.y, x.w, 0x7632);          // x[8 tq + 3], x[8 tq + 7]
      }
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        const uint32_t wA = w[2 * m], wB = w[2 * m + 1];
        const uint32_t wA8 = wA >> 8, wB8 = wB >> 8;
        {
          const uint32_t a0 = deq_lo(wA, d2[2 * m]), a1 = deq_lo(wB, d2[2 * m + 1]);
          const uint32_t a2 = deq_lo(wA8, d2[2 * m]), a3 = deq_lo(wB8, d2[2 * m + 1]);
#pragma unroll
          for (int n = 0; n < NT; ++n) mma_f16(c[m][n], a0, a1, a2, a3, b[n][0], b[n][1]);
        }
        {
          const uint32_t a0 = deq_hi(wA, d2[2 * m]), a1 = deq_hi(wB, d2[2 * m + 1]);
          const uint32_t a2 = deq_hi(wA8, d2[2 * m]), a3 = deq_hi(wB8, d2[2 * m + 1]);
#pragma unroll
          for (int n = 0; n < NT; ++n) mma_f16(c[m][n], a0, a1, a2, a3, b[n][2], b[n][3]);
        }
      }
    }
    __syncthreads();
  }

  // ---- k groups: with up to 8 columns every k group writes its own tile and the sums are formed on reading (one block
  // barrier); with more columns the groups add into one tile in turn (four barriers, a quarter of the shared memory).
  // Either way the order is k group 0, 1, 2, 3.
  constexpr int NPB = NT == 1 ? 4 : 1;
  constexpr size_t PB = (size_t)NT * 8 * PSTR;            // floats per partial tile
  if (NPB == 4) {
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        float* p0 = P + kg * PB + (size_t)(n * 8 + 2 * tq) * PSTR + rg * 32 + 16 * m + g;
        p0[0] = c[m][n][0]; p0[PSTR] = c[m][n][1]; p0[8] = c[m][n][2]; p0[PSTR + 8] = c[m][n][3];
      }
    __syncthreads();
  } else {
#pragma unroll 1
    for (int s = 0; s < 4; ++s) {
      if (kg == s) {
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            float* p0 = P + (size_t)(n * 8 + 2 * tq) * PSTR + rg * 32 + 16 * m + g;
            if (s == 0) {
              p0[0] = c[m][n][0]; p0[PSTR] = c[m][n][1]; p0[8] = c[m][n][2]; p0[PSTR + 8] = c[m][n][3];
            } else {
              p0[0] += c[m][n][0]; p0[PSTR] += c[m][n][1]; p0[8] += c[m][n][2]; p0[PSTR + 8] += c[m][n][3];
            }
          }
      }
      __syncthreads();
    }
  }
  auto partial2 = [&](int col, int pr) {                  // this CTA's sums of rows 2 pr, 2 pr + 1 of column col
    const float* src = P + (size_t)col * PSTR + 2 * pr;
    float2 v = *reinterpret_cast<const float2*>(src);
    if (NPB == 4) {
#pragma unroll
      for (int q = 1; q < 4; ++q) {
        const float2 u = *reinterpret_cast<const float2*>(src + q * PB);
        v.x += u.x;
        v.y += u.y;
      }
    }
    return v;
  };

  // ---- K slices: CTA r of the cluster finishes row pairs [64 r / ksplit, 64 (r + 1) / ksplit) of the tile.  Every CTA
  // PUSHES the pairs it does not own into their owner's receive buffer (remote stores, nothing to wait for), one cluster
  // barrier publishes them, and the owner adds the ksplit contributions in rank order.
  int pr0 = 0, pr1 = ROWS / 2;
  const int maxp = (ROWS / 2 + a.ksplit - 1) / a.ksplit;  // pairs per slice, at most
  if (a.ksplit > 1) {
    pr0 = (ROWS / 2 * ks) / a.ksplit;
    pr1 = (ROWS / 2 * (ks + 1)) / a.ksplit;
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");    // pairs with the arrive at the top: every peer runs
    for (int i = t; i < (ROWS / 2) * a.B; i += GT) {
      const int col = i >> 6, pr = i & 63;
      int r = (pr * a.ksplit) >> 6;
      if (((ROWS / 2) * (r + 1)) / a.ksplit <= pr) ++r;
      const float2 v = partial2(col, pr);
      const int local = pr - ((ROWS / 2) * r) / a.ksplit;
      const float* slot = recv + (((size_t)ks * NT * 8 + col) * maxp + local) * 2;
      uint32_t addr;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(tc::smem_u32(slot)), "r"(r));
      asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(v.x), "f"(v.y) : "memory");
    }
    cluster_sync_all();
  }
  if (a.epi == Q4B_EPI_SWIGLU_Q8) {
    // SwiGLU + re-quantise for `down` (lab/qwen_batched.py:1363-1396; unsplit launches, whole tiles only): the product
    // rounded to fp16, then the Q8_1 quantiser on it.  A 32-value block of the product is 32 row pairs of one column = one
    // warp of this loop (64 B is a multiple of 32, so warps are whole).
    int8_t* qo = reinterpret_cast<int8_t*>(a.Y);
    __half* dout = reinterpret_cast<__half*>(const_cast<void*>(a.AUX));
    for (int i = t; i < (ROWS / 2) * a.B; i += GT) {
      const int col = i >> 6, pr = i & 63;
      const float2 pv = partial2(col, pr);
      const float act = __half2float(__float2half_rn(pv.x / (1.f + __expf(-pv.x)) * pv.y));
      const float d = warp_max(fabsf(act)) / 127.f;
      const int q = d > 0.f ? __float2int_rn(act / d) : 0;
      const size_t f = (size_t)tile * (ROWS / 2) + pr;
      qo[(size_t)col * a.ldy + f] = (int8_t)q;
      if (lane == 0) dout[(size_t)col * (a.ldy >> 5) + (f >> 5)] = __float2half_rn(d);
    }
    if (!ok) atomicOr(a.status, 1u);
    return;
  }
  const int npr = pr1 - pr0;
  // resid: the old values of every item of this thread are loaded first, as 8-byte pairs (at most NT items: npr <= 64,
  // B <= 8 NT).  A load per item in the loop below would wait behind the previous item's store to the same array and pay
  // the global-memory latency once per item.
  const bool resid2 = a.epi == Q4B_EPI_RESID && ((a.ldy | a.N) & 1) == 0 && (reinterpret_cast<uintptr_t>(a.Y) & 7) == 0;
  float2 oldv[NT];
  if (resid2) {
#pragma unroll
    for (int it = 0; it < NT; ++it) {
      const int i = t + it * GT;
      oldv[it] = make_float2(0.f, 0.f);
      if (i < npr * a.B) {
        const int col = i / npr, row = tile * ROWS + 2 * (pr0 + i - col * npr);
        if (row < a.N) oldv[it] = *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(a.Y) + (size_t)col * a.ldy + row);
      }
    }
  }
  int it = -1;
  for (int i = t; i < npr * a.B; i += GT) {
    ++it;
    const int col = i / npr, pl = i - col * npr, pr = pr0 + pl;
    float v0 = 0.f, v1 = 0.f;
    if (a.ksplit > 1) {
      for (int r = 0; r < a.ksplit; ++r) {                                  // rank order
        const float2 pv = *reinterpret_cast<const float2*>(recv + (((size_t)r * NT * 8 + col) * maxp + pl) * 2);
        v0 += pv.x;
        v1 += pv.y;
      }
    } else {
      const float2 pv = partial2(col, pr);
      v0 = pv.x;
      v1 = pv.y;
    }
    const int row = tile * ROWS + 2 * pr;
    if (row >= a.N) continue;
    const bool two = row + 1 < a.N;
    const size_t o = (size_t)col * a.ldy + row;
    switch (a.epi) {
      case Q4B_EPI_STORE: {
        __half* Y = reinterpret_cast<__half*>(a.Y);
        Y[o] = __float2half_rn(v0);
        if (two) Y[o + 1] = __float2half_rn(v1);
        break;
      }
      case Q4B_EPI_BIASF: {
        __half* Y = reinterpret_cast<__half*>(a.Y);
        const float* bias = reinterpret_cast<const float*>(a.AUX);
        Y[o] = __float2half_rn(v0 + bias[row]);
        if (two) Y[o + 1] = __float2half_rn(v1 + bias[row + 1]);
        break;
      }
      case Q4B_EPI_RESID: {
        float* Y = reinterpret_cast<float*>(a.Y);
        if (resid2) {
          float2 ov = make_float2(0.f, 0.f);
#pragma unroll
          for (int q = 0; q < NT; ++q)                                       // static indexing keeps oldv in registers
            if (q == it) ov = oldv[q];
          *reinterpret_cast<float2*>(Y + o) = make_float2(ov.x + v0, ov.y + v1);
        } else {
          Y[o] += v0;
          if (two) Y[o + 1] += v1;
        }
        break;
      }
      case Q4B_EPI_LOGITS: {
        float* Y = reinterpret_cast<float*>(a.Y);
        Y[o] = v0;
        if (two) Y[o + 1] = v1;
        break;
      }
      case Q4B_EPI_SWIGLU:                                                  // rows interleaved gate, up
        if (two) reinterpret_cast<__half*>(a.Y)[(size_t)col * a.ldy + (row >> 1)] = __float2half_rn(v0 / (1.f + __expf(-v0)) * v1);
        break;
      default: break;
    }
  }
  if (!ok) atomicOr(a.status, 1u);
}

size_t smem_for(int cap, int nt, int mode, int ks) {
  const size_t x = mode == MODE_F16 ? (size_t)nt * 8 * x_pitch(cap) : (size_t)nt * 8 * xq_pitch(cap) + (size_t)cap * nt * 8 * sizeof(float);   // Q8 and Q8F alike
  // with K slices: the receive buffer of their reduction (< 64 + 8 pairs per column)
  const size_t recv = ks > 1 ? (size_t)nt * 8 * (ROWS / 2 + 8) * 2 * sizeof(float) : 0;
  const size_t own_tiles = mode == MODE_F16 ? (size_t)(nt == 1 ? 4 : 1) * nt * 8 * PSTR * sizeof(float) : 0;   // see the kernel
  return slab_region(cap, nt) + x + recv + own_tiles;
}

// How many clusters of `ks` CTAs with `smem` bytes each can be resident at once (cached per device and configuration):
// a grid of T clusters that does not fit runs in two waves, which a smaller split avoids.
template <int NT, int MODE>
int resident_clusters(int ks, size_t smem) {
  static std::mutex mu;
  static std::map<std::tuple<int, int, size_t>, int> cache;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  const auto key = std::make_tuple(dev, ks, smem);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(1, ks);
  cfg.blockDim = dim3(GT);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = ks;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemv_f16mma_kernel<NT, MODE>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    n = 1 << 30;                                          // unknown: do not constrain the split
  }
  cache[key] = n;
  return n;
}

template <int NT, int MODE>
int launch(F16Args& a, int T, cudaStream_t st, const char* where) {
  // K slices: fill the SMs when there are fewer row tiles than SMs; the slab holds `cap` k-blocks of one slice (longer
  // slices run as several windows); prefer a split whose clusters are all resident at once
  auto cap_for = [&](int ks) {
    int cap = std::min(CHK * MAX_CHUNKS, (a.KB + ks - 1) / ks);
    while (cap > 1 && smem_for(cap, NT, MODE, ks) > MAX_DYN_SMEM) --cap;
    return cap;
  };
  if (cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(&gemv_f16mma_kernel<NT, MODE>), MAX_DYN_SMEM); e != cudaSuccess) {
    set_cuda_error(e, where);
    return Q4B_E_CUDA;
  }
  int ks = sm_count() / T;
  ks = ks < 1 ? 1 : (ks > 8 ? 8 : ks);
  if (ks > a.KB) ks = a.KB;
  for (; ks > 1; --ks)
    if (resident_clusters<NT, MODE>(ks, smem_for(cap_for(ks), NT, MODE, ks)) >= T) break;
  if (a.epi == Q4B_EPI_SWIGLU_Q8 && ks > 1) return fail(Q4B_E_SHAPE, "mmq_q4_0_q8_1_mma: swiglu_q8 only where the launch is not split along K");
  a.ksplit = ks;
  a.cap = cap_for(ks);
  dim3 grid(T, ks), block(GT);
  return check_launch(launch_pdl_cluster(gemv_f16mma_kernel<NT, MODE>, grid, block, smem_for(a.cap, NT, MODE, ks), st, 1, ks, a), where);
}

int check_common(const char* where, const void* W, const void* S, const void* Y, const void* AUX, int N, int K, int B, int epi, int ldy,
                 const uint32_t* status) {
  static thread_local char msg[160];
  auto say = [&](int code, const char* what) {
    snprintf(msg, sizeof msg, "%s: %s", where, what);
    return fail(code, msg);
  };
  if (N <= 0 || K <= 0 || (K % 32)) return say(Q4B_E_SHAPE, "N > 0 and K a positive multiple of 32 required");
  if (B < 1 || B > 32) return say(Q4B_E_SHAPE, "1 <= B <= 32 activation rows");
  if (!W || !S || !Y || !status || !aligned16(W) || !aligned16(S)) return say(Q4B_E_ALIGN, "null or misaligned pointer");
  if (epi < Q4B_EPI_STORE || epi > Q4B_EPI_SWIGLU_Q8) return say(Q4B_E_ARG, "unknown epilogue");
  if (epi == Q4B_EPI_SWIGLU_Q8 && ((N % 128) || !AUX || (ldy % 32))) return say(Q4B_E_SHAPE, "swiglu_q8 needs N a multiple of 128, AUX (scales out) and ldy a multiple of 32");
  if (epi == Q4B_EPI_BIASF && !AUX) return say(Q4B_E_ALIGN, "biasf needs AUX");
  if (epi == Q4B_EPI_SWIGLU && (N % 2)) return say(Q4B_E_SHAPE, "swiglu needs an even row count");
  if (ldy < (epi == Q4B_EPI_SWIGLU || epi == Q4B_EPI_SWIGLU_Q8 ? N / 2 : N)) return say(Q4B_E_SHAPE, "ldy shorter than an output row");
  return Q4B_OK;
}

template <int MODE>
int dispatch(F16Args& a, int T, int nt, cudaStream_t st, const char* where) {
  switch (nt) {
    case 1: return launch<1, MODE>(a, T, st, where);
    case 2: return launch<2, MODE>(a, T, st, where);
    case 3: return launch<3, MODE>(a, T, st, where);
    default: return launch<4, MODE>(a, T, st, where);
  }
}

}  // namespace

int gemv_f16mma(const void* W, const void* S, const void* X, void* Y, const void* AUX, int N, int K, int B, int epi, int ldy,
                uint32_t* status, cudaStream_t st) {
  const char* where = "gemv_q4_0_f16mma";
  if (int rc = check_common(where, W, S, Y, AUX, N, K, B, epi, ldy, status); rc != Q4B_OK) return rc;
  if (!X || !aligned16(X)) return fail(Q4B_E_ALIGN, "gemv_q4_0_f16mma: null or misaligned pointer");
  if (epi == Q4B_EPI_SWIGLU_Q8) return fail(Q4B_E_ARG, "gemv_q4_0_f16mma: unknown epilogue");
  F16Args a{};
  a.W = reinterpret_cast<const uint8_t*>(W);
  a.S = reinterpret_cast<const __half*>(S);
  a.X = reinterpret_cast<const __half*>(X);
  a.Y = Y;
  a.AUX = AUX;
  a.status = status;
  a.N = N; a.K = K; a.KB = K / 32; a.B = B; a.epi = epi; a.ldy = ldy;
  a.wait_limit = tc::WAIT_LIMIT;
  return dispatch<MODE_F16>(a, (N + ROWS - 1) / ROWS, (B + 7) / 8, st, where);
}

// The same kernel skeleton with Q8_1 activations and exact int8 block dots in registers (MODE_Q8).
int gemv_q8mma(const void* W, const void* S, const void* XQ, const void* XD, void* Y, const void* AUX, int N, int K, int B, int epi,
               int ldy, uint32_t* status, cudaStream_t st) {
  const char* where = "mmq_q4_0_q8_1_mma";
  if (int rc = check_common(where, W, S, Y, AUX, N, K, B, epi, ldy, status); rc != Q4B_OK) return rc;
  // XQ == nullptr: XD is the fp16 activation matrix [B, K] and the quantiser runs inside the kernel
  if (!XD || (XQ && ((reinterpret_cast<uintptr_t>(XQ) & 15u) || (reinterpret_cast<uintptr_t>(XD) & 1u))) || (!XQ && (reinterpret_cast<uintptr_t>(XD) & 7u)))
    return fail(Q4B_E_ALIGN, "mmq_q4_0_q8_1_mma: null or misaligned pointer");
  F16Args a{};
  a.W = reinterpret_cast<const uint8_t*>(W);
  a.S = reinterpret_cast<const __half*>(S);
  a.XQ = reinterpret_cast<const int8_t*>(XQ);
  a.XD = XQ ? reinterpret_cast<const __half*>(XD) : nullptr;
  a.X = XQ ? nullptr : reinterpret_cast<const __half*>(XD);
  a.Y = Y;
  a.AUX = AUX;
  a.status = status;
  a.N = N; a.K = K; a.KB = K / 32; a.B = B; a.epi = epi; a.ldy = ldy;
  a.wait_limit = tc::WAIT_LIMIT;
  if (!XQ) return dispatch<MODE_Q8F>(a, (N + ROWS - 1) / ROWS, (B + 7) / 8, st, where);
  return dispatch<MODE_Q8>(a, (N + ROWS - 1) / ROWS, (B + 7) / 8, st, where);
}

}  // namespace q4b
