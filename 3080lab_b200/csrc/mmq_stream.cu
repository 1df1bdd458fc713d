// Streaming Q4_0 x int8 matrix product for decode (1..32 activation columns) on the tcgen05 int8 tensor cores.
//
//   y[n, m] = sum_b dw[m, b] * sx[n, b] * dot_b[m, n],   dot_b = sum_{i<32} (q4[m, 32b+i] - 8) * x8[n, 32b+i]  (exact)
//
// Two uses of the same kernel:
//   Q8_1 mode   columns are sequences: x8 = Q8_1 int8 values, sx = their fp16 block scales.  This is the reference's
//               MMQ arithmetic (lab/qwen_batched.py:1237-1243: exact int32 block dots, fp32 dw*dx scaling in k-block
//               order) applied to batched decode.
//   exact mode  one activation vector: each 32-value block of x is written as a block-fixed-point integer
//               X_i = x_i / 2^e (24 or 30 bits) split into signed base-256 digits; digit j is column j, so
//               sum_i (q-8) x_i = 2^e * sum_j 256^j dot_b[., j] with every dot an exact integer.  For fp16 x this
//               equals the reference's dequantise-and-dot (lab/qwen_kernels.py:14-113) with no rounding inside a
//               block; the only roundings are the per-block fp32 scale-and-add, as in the reference.
//
// Data movement (per CTA = 128 weight rows x one K slice):
//   * weights arrive tile-packed (pack.cu): a CTA's row tile x K slice is one contiguous range.  Before the
//     programmatic-dependency wait one thread issues two 1-D bulk (TMA) copies per batch of k-blocks (nibbles, fp16
//     scales) into shared memory, each batch completing on its own mbarrier.  Weights never depend on the previous
//     kernel, so with programmatic dependent launch the whole prefetch overlaps the producer of x.  (Per-row copies
//     from the canonical layout were measured first: issuing 256 small bulk copies per CTA cost 1.8 us.)
//   * after the wait the activation slice is staged once into shared memory as the UMMA B operand (K-major 8x16-byte
//     core matrices, bytes permuted to match the nibble expansion order).
//   * per batch of G k-blocks: each thread expands 16 bytes of nibbles to 32 signed bytes 16*(q-8) (two logic ops per
//     four weights) and stores them with tcgen05.st straight into tensor memory as the A operand; one thread issues G
//     tcgen05.mma.kind::i8 (M = 128, N = columns, K = 32 = one Q4_0 block), each into its own TMEM accumulator; the
//     previous batch's accumulators are read back (tcgen05.ld) and folded into fp32 registers with the block scales
//     while the tensor core works on the current one.
//   * split-K: the CTAs of a thread-block cluster share a row tile; partial sums cross through distributed shared
//     memory and are added in rank order, so results are bit-repeatable.
// Measured limits of this formulation on B200: tcgen05.mma instructions that write DIFFERENT accumulator tiles retire
// one every ~177 clocks whatever N (8 or 32; 43 clocks when the same tile is overwritten), so a row tile consumes one
// 2304-byte k-block per 177 clocks: 25 GB/s per SM, 3.8 TB/s per GPU.  A register-accumulator variant of the Q8_1 mode
// (mma.sync.m16n8k32.s8, no tensor memory) was built and measured: faster per kernel when the weights sit in L2, but
// slower inside the real decode step (4.73 K against 5.09 K tok/s at 8 sequences, 12.56 K against 12.73 K at 32), and
// was dropped.
// All waits are bounded (status word + fall through).
#include <algorithm>
#include <cstdlib>

#include "q4b_internal.h"
#include "tc05.cuh"

namespace q4b {

namespace {

constexpr int MODE_X16 = 0, MODE_X32 = 1, MODE_Q8 = 2, MODE_NORM = 3;
constexpr int ROWS = 128;
constexpr int MAX_BATCH = 20;                   // batches (mbarriers) per CTA
constexpr size_t MAX_DYN_SMEM = 226 * 1024;   // 227 KB per CTA on sm_100 minus the static barriers

struct StreamArgs {
  const uint8_t* W;     // tile-packed nibbles [T, K/32, 128, 16 bytes]
  const __half* S;      // tile-packed scales [T, K/32, 128]
  const void* X;        // exact modes: fp16 / fp32 [K]; Q8 mode: int8 [cols, K]
  const __half* XD;     // Q8 mode: fp16 [cols, K/32]
  const float* NW;      // norm mode: RMSNorm weights fp32 [K] (X is then the fp32 residual stream)
  float eps;
  unsigned long long* trace;   // optional: 16 %globaltimer stamps per CTA (thread 0), see q4b_trace_buffer
  void* Y;
  const void* AUX;
  uint32_t* status;
  int N, K, cols, epi, ldy;
  int gps;              // groups (of 8 k-blocks) per K slice
  int ksplit;
  int KBT;              // k-blocks per row of W / S / X in memory (K/32 unless this launch covers a window of K)
  int kbw;              // first k-block of the window
};

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   tc::smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(tc::smem_u32(bar))
               : "memory");
}
// position of element i (0..31) of a k-block inside the 32 operand bytes (see tc::expand_nibbles)

template <int NT>
__device__ __forceinline__ uint32_t b_offset(int kbl, int n, int pos) {
  return (uint32_t)kbl * (NT * 32) + (uint32_t)(((n >> 3) * 2 + (pos >> 4)) * 128 + (n & 7) * 16 + (pos & 15));
}

template <int MODE, int NT>
__global__ void __launch_bounds__(ROWS * ((MODE == MODE_Q8 && NT >= 16) ? 2 : 1)) mmq_stream_kernel(const StreamArgs a) {
  constexpr int G = NT <= 16 ? 8 : 4;                  // k-blocks per MMA batch
  constexpr int NL = (MODE == MODE_X16 || MODE == MODE_NORM) ? 3 : 4;   // digits in exact mode (fp16-valued x: 3)
  // With 16 or 32 activation rows the read-back of the accumulators (columns x k-blocks conversions and FMAs per
  // thread) is the longest stage, so a second warpgroup takes half of the columns.  Warpgroup 0 expands the weights,
  // issues the MMAs and folds columns [0, NT/2); warpgroup 1 only folds columns [NT/2, NT).
  constexpr int FW = (MODE == MODE_Q8 && NT >= 16) ? 2 : 1;
  constexpr int NTHR = ROWS * FW;
  constexpr int NTOT = MODE == MODE_Q8 ? NT : 1;       // accumulator columns of the tile
  constexpr int NACC = NTOT / FW;                      // ... of one thread
  constexpr bool PUSH = NTOT <= 8;                     // split-K partials pushed to the leader (else a reduce-scatter)
  constexpr uint32_t A_COLS = 2 * G * 8, D_COLS = 2 * G * NT;
  constexpr uint32_t TCOLS = (A_COLS + D_COLS) <= 128 ? 128 : ((A_COLS + D_COLS) <= 256 ? 256 : 512);
  constexpr uint32_t IDESC = tc::idesc_i8(128, NT);

  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bar_load[MAX_BATCH];
  __shared__ __align__(8) uint64_t bar_mma[2];
  __shared__ __align__(8) uint64_t bar_free[2];          // warpgroup 1 has read an accumulator slot
  __shared__ __align__(8) uint64_t bar_drain;            // see tc::drain_mmas_on_failure
  __shared__ uint32_t tmem_base_s;

  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int wg = t >> 7, r = t & (ROWS - 1), wq = warp & 3;   // warpgroup, row of the tile, TMEM lane quarter
  const int cbase = wg * NACC;                           // first accumulator column of this thread
  const int row0 = blockIdx.x * ROWS, row = row0 + r;
  const int ks = blockIdx.y;
  unsigned long long* tr = (a.trace && t == 0) ? a.trace + (size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 16 : nullptr;
  int tri = 0;
  auto stamp = [&]() {
    if (tr && tri < 16) {
      unsigned long long g;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g));
      tr[tri++] = g;
    }
  };
  stamp();                                              // 0: start
  pdl_launch_dependents();                              // let the next kernel's CTAs begin their own prologue now
  const int GT = a.K >> 8;
  const int g0 = ks * a.gps, ng = min(a.gps, GT - g0);          // host guarantees ng >= 1
  const int nkb = ng * 8, kb0 = g0 * 8;
  uint8_t* slabW = smem;                                         // [k-block][128 rows][16 bytes]
  uint8_t* slabS = slabW + (size_t)a.gps * 8 * 2048;             // [k-block][128 rows] fp16
  uint8_t* sB = slabS + (size_t)a.gps * 8 * 256;
  float* xs = reinterpret_cast<float*>(sB + (size_t)a.gps * 8 * NT * 32);     // block scales of the activations
  float* red_buf = xs + (size_t)a.gps * 8 * NT;                  // split-K partials pushed by the peers: [rank-1][NACC][128]
  const int nbatch = nkb / G;

  if (warp == 0) {
    tc::tmem_alloc(&tmem_base_s, TCOLS);
    tc::tmem_relinquish();
  }
  if (t == 0) {
    for (int b = 0; b < nbatch; ++b) tc::mbar_init(&bar_load[b], 1);
    tc::mbar_init(&bar_mma[0], 4);                       // one commit per issuing warp
    tc::mbar_init(&bar_mma[1], 4);
    tc::mbar_init(&bar_free[0], 4);
    tc::mbar_init(&bar_free[1], 4);
    tc::mbar_init(&bar_drain, 4);                        // failure path: the four issuing lanes
    tc::mbar_fence_init();
  }
  stamp();                                              // TMEM allocated, barriers initialised
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  stamp();

  // ---- weights: per batch of G k-blocks one bulk copy of nibbles and one of scales, issued by one thread
  if (t == 0) {
    const size_t kbg = (size_t)blockIdx.x * a.KBT + a.kbw + kb0;  // first k-block of this CTA in the packed arrays
    for (int b = 0; b < nbatch; ++b) {
      tc::mbar_expect_tx(&bar_load[b], (uint32_t)G * (2048 + 256));
      bulk_g2s(slabW + (size_t)b * G * 2048, a.W + (kbg + (size_t)b * G) * 2048, (uint32_t)G * 2048, &bar_load[b]);
      bulk_g2s(slabS + (size_t)b * G * 256, a.S + (kbg + (size_t)b * G) * 128, (uint32_t)G * 256, &bar_load[b]);
    }
  }
  stamp();                                              // bulk copies issued
  pdl_wait();                                           // the activations come from the previous kernel
  stamp();                                              // 2: predecessor complete

  // What the epilogue adds to this thread's outputs (residual rows, bias) is requested now, so that its latency hides
  // behind the whole main loop instead of costing one round trip per column at the end.  addend[i] belongs to the
  // i-th column this CTA writes: column i for the leader of a pushed reduction, column ks + i ksplit in a reduce-scatter.
  constexpr int NOWN = PUSH ? NACC : (NTOT / 2 + FW - 1) / FW;   // reduce-scatter: this thread's share of the CTA's columns
  float addend[NOWN];
  auto load_addends = [&]() {
    const bool writer = PUSH ? ks == 0 : true;
    const float bias = (a.epi == Q4B_EPI_BIASF && row < a.N) ? reinterpret_cast<const float*>(a.AUX)[row] : 0.f;
#pragma unroll
    for (int i = 0; i < NOWN; ++i) {
      const int n = PUSH ? i : ks + (wg + FW * i) * a.ksplit;
      addend[i] = bias;
      if (a.epi == Q4B_EPI_RESID && writer && n < a.cols && row < a.N) addend[i] = reinterpret_cast<const float*>(a.Y)[(size_t)n * a.ldy + row];
    }
  };
  if (PUSH) load_addends();                             // few columns: now; many columns: next to the reduce-scatter loads

  // ---- activations -> UMMA B operand in shared memory
  if (MODE == MODE_Q8) {
    const int8_t* xq = reinterpret_cast<const int8_t*>(a.X);
    const int per = nkb * 2;
    for (int c0 = 0; c0 < NT * per; c0 += 4 * NTHR) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * NTHR + t;
        const int n = c / per, r = c - n * per, kbl = r >> 1, kc = r & 1;
        v[u] = make_uint4(0u, 0u, 0u, 0u);
        if (c < NT * per && n < a.cols) v[u] = *reinterpret_cast<const uint4*>(xq + ((size_t)n * a.KBT + a.kbw + kb0 + kbl) * 32 + kc * 16);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * NTHR + t;
        if (c < NT * per) {
          const int n = c / per, r = c - n * per, kbl = r >> 1, kc = r & 1;
          uint32_t e0, o0, e1, o1;
          tc::permute_bytes(v[u].x, v[u].y, e0, o0);
          tc::permute_bytes(v[u].z, v[u].w, e1, o1);
          *reinterpret_cast<uint4*>(sB + b_offset<NT>(kbl, n, kc * 16)) = make_uint4(e0, o0, e1, o1);
        }
      }
    }
    for (int c0 = 0; c0 < NT * nkb; c0 += 4 * NTHR) {
      __half sv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * NTHR + t, n = c / nkb, kbl = c - n * nkb;
        sv[u] = __float2half_rn(0.f);
        if (c < NT * nkb && n < a.cols) sv[u] = a.XD[(size_t)n * a.KBT + a.kbw + kb0 + kbl];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * NTHR + t, n = c / nkb, kbl = c - n * nkb;
        if (c < NT * nkb) xs[kbl * NT + n] = __half2float(sv[u]);
      }
    }
  } else {
    // exact mode: 8 lanes <-> one k-block, 4 consecutive elements per lane.  X_i = rint(x_i * 2^-e) with
    // |X_i| < 2^(8 NL - 2), split into signed base-256 digits, digit j -> column j.
    for (int c = t; c < nkb * 64; c += ROWS)            // columns NL..7 must read as zero
      *reinterpret_cast<uint32_t*>(sB + (size_t)c * 4) = 0u;
    // all global loads of this thread's operand elements are issued before anything waits on them
    constexpr int MAXIT = 5;                            // 16 k-blocks per pass over the CTA's threads, at most 80 per slice
    float xin[MAXIT][4];
#pragma unroll
    for (int u = 0; u < MAXIT; ++u) {
      const int kbl = (t >> 3) + u * (ROWS / 8);
      xin[u][0] = xin[u][1] = xin[u][2] = xin[u][3] = 0.f;
      if (kbl < nkb) {
        const int k = (kb0 + kbl) * 32 + (t & 7) * 4;
        if (MODE == MODE_X16) {
          const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(a.X) + k);
          const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
          const float2 q = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
          xin[u][0] = p.x; xin[u][1] = p.y; xin[u][2] = q.x; xin[u][3] = q.y;
        } else {
          const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.X) + k);
          xin[u][0] = v.x; xin[u][1] = v.y; xin[u][2] = v.z; xin[u][3] = v.w;
          if (MODE == MODE_NORM) {                      // (v * r) * w is evaluated as (v * w) * r: r arrives last
            const float4 w = __ldg(reinterpret_cast<const float4*>(a.NW + k));
            xin[u][0] *= w.x; xin[u][1] *= w.y; xin[u][2] *= w.z; xin[u][3] *= w.w;
          }
        }
      }
    }
    float rnorm = 1.f;
    if (MODE == MODE_NORM) {
      // RMSNorm of the whole residual row (every CTA needs the full sum of squares), as RMSNORM_F32W_1P
      // (lab/qwen_kernels.py:683-705): r = rsqrt(sum(v^2) / K + eps); x = round16(v * r * w).
      float* red = xs + a.gps * 8;                      // 4 floats behind the block scales
      const float4* hv = reinterpret_cast<const float4*>(a.X);
      float ss = 0.f;
      for (int i = t; i < (a.K >> 2); i += ROWS) {
        const float4 v = hv[i];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
      ss = warp_sum(ss);
      if (lane == 0) red[warp] = ss;
      __syncthreads();
      rnorm = rsqrtf((red[0] + red[1] + red[2] + red[3]) / (float)a.K + a.eps);
    } else {
      __syncthreads();
    }
    const int sub = t & 7;
    for (int kbl = t >> 3, it = 0; kbl < nkb; kbl += ROWS / 8, ++it) {
      float x[4];
#pragma unroll
      for (int u = 0; u < MAXIT; ++u)
        if (u == it) {
          x[0] = xin[u][0]; x[1] = xin[u][1]; x[2] = xin[u][2]; x[3] = xin[u][3];
        }
      if (MODE == MODE_NORM) {
#pragma unroll
        for (int j = 0; j < 4; ++j) x[j] = __half2float(__float2half_rn(x[j] * rnorm));   // xin holds v * w
      }
      float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
      for (int o = 4; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const bool live = amax > 0.f && amax < INFINITY;
      int e = (__float_as_int(amax) >> 23) & 0xFF;      // biased exponent of the block maximum
      e = max(e, 8 * NL);                               // tiny blocks: keep the scale a normal float
      // 2^(8 NL - 3) / 2^(e - 127): |x| < 2^(e - 126) maps below 2^(8 NL - 2)
      const float inv = __int_as_float((127 + (8 * NL - 3) - (e - 127)) << 23);
      int X[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) X[j] = live ? __float2int_rn(x[j] * inv) : 0;
      // elements 4 sub + {0, 2} are adjacent operand bytes, and so are 4 sub + {1, 3} (operand byte of element i: 4 (2 (i / 8) + (i & 1)) + (i & 7) / 2)
      const int pos02 = 8 * (sub >> 1) + 2 * (sub & 1), pos13 = pos02 + 4;
#pragma unroll
      for (int j = 0; j < NL; ++j) {
        int dg[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          dg[u] = (int)(int8_t)(X[u] & 0xFF);
          X[u] = (X[u] - dg[u]) >> 8;
        }
        *reinterpret_cast<uint16_t*>(sB + b_offset<NT>(kbl, j, pos02)) = (uint16_t)((dg[0] & 0xFF) | ((dg[2] & 0xFF) << 8));
        *reinterpret_cast<uint16_t*>(sB + b_offset<NT>(kbl, j, pos13)) = (uint16_t)((dg[1] & 0xFF) | ((dg[3] & 0xFF) << 8));
      }
      if (sub == 0) xs[kbl] = live ? __int_as_float((127 - (8 * NL - 3) + (e - 127)) << 23) : 0.f;
    }
  }
  tc::fence_async_smem();
  __syncthreads();
  stamp();                                              // 3: activation operand staged

  bool ok = true;                // slab landed (async-proxy writes made visible by the barrier)

  const uint32_t tmem = tmem_base_s;
  const uint32_t lane_off = (uint32_t)(32 * wq) << 16;
  const uint32_t tmem_a = tmem, tmem_d = tmem + A_COLS;
  float acc[NACC];
#pragma unroll
  for (int n = 0; n < NACC; ++n) acc[n] = 0.f;

  const uint8_t* myW = slabW + r * 16;
  const __half* myS = reinterpret_cast<const __half*>(slabS) + r;

  auto fold = [&](int bi) {                             // accumulators of batch bi -> acc
    const int slot = bi & 1;
    ok = tc::mbar_wait(&bar_mma[slot], (uint32_t)(bi >> 1) & 1u) && ok;
    tc::fence_after_sync();
    if (MODE == MODE_Q8) {
      constexpr int SB = NACC <= 8 ? 8 : 4;                      // k-blocks whose accumulators are in flight together
      static_assert(G % (SB < G ? SB : G) == 0, "batch size");
      constexpr int SBE = SB < G ? SB : G;
#pragma unroll 1
      for (int j0 = 0; j0 < G; j0 += SBE) {
        uint32_t d[SBE][NACC];
#pragma unroll
        for (int j = 0; j < SBE; ++j) {
          const uint32_t dcol = tmem_d + lane_off + (uint32_t)((slot * G + j0 + j) * NT + cbase);
#pragma unroll
          for (int c0 = 0; c0 < NACC; c0 += 8) tc::tmem_ld8(dcol + c0, &d[j][c0]);
        }
        tc::tmem_wait_ld();
        if (FW == 2 && wg == 1 && j0 + SBE >= G) {               // slot read: warpgroup 0 may overwrite it
          tc::fence_before_sync();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&bar_free[slot]);
        }
#pragma unroll
        for (int j = 0; j < SBE; ++j) {
          const int kbl = bi * G + j0 + j;
          const float dw = __half2float(myS[kbl * 128]) * 0.0625f;   // 1/16 undoes the 16*(q-8) operand scaling
#pragma unroll
          for (int c0 = 0; c0 < NACC; c0 += 4) {
            const float4 sx = *reinterpret_cast<const float4*>(xs + kbl * NT + cbase + c0);
            acc[c0 + 0] = fmaf(dw * sx.x, (float)(int32_t)d[j][c0 + 0], acc[c0 + 0]);
            acc[c0 + 1] = fmaf(dw * sx.y, (float)(int32_t)d[j][c0 + 1], acc[c0 + 1]);
            acc[c0 + 2] = fmaf(dw * sx.z, (float)(int32_t)d[j][c0 + 2], acc[c0 + 2]);
            acc[c0 + 3] = fmaf(dw * sx.w, (float)(int32_t)d[j][c0 + 3], acc[c0 + 3]);
          }
        }
      }
    } else {
      uint32_t d[G][4];
#pragma unroll
      for (int j = 0; j < G; ++j) tc::tmem_ld4(tmem_d + lane_off + (uint32_t)((slot * G + j) * NT), d[j]);
      tc::tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < G; ++j) {
        const int kbl = bi * G + j;
        const float dw = __half2float(myS[kbl * 128]) * 0.0625f;
        float f = fmaf(256.f, (float)(int32_t)d[j][1], (float)(int32_t)d[j][0]);
        f = fmaf(65536.f, (float)(int32_t)d[j][2], f);
        if (NL == 4) f = fmaf(16777216.f, (float)(int32_t)d[j][3], f);
        acc[0] = fmaf(dw * xs[kbl], f, acc[0]);
      }
    }
    tc::fence_before_sync();
  };

  for (int bi = 0; bi < nbatch; ++bi) {
    const int slot = bi & 1;
    ok = tc::mbar_wait(&bar_load[bi], 0) && ok;         // this batch's weights landed (async-proxy writes now visible)
    if (FW == 2 && wg == 1) {                           // fold-only warpgroup: needs the batch's scales, then its accumulators
      fold(bi);
      continue;
    }
    // all nibble words of the batch are read before the first tensor-memory store (the stores are ordered asm
    // statements; interleaved with the loads they would expose one shared-memory latency per k-block)
    uint4 wv[G];
#pragma unroll
    for (int j = 0; j < G; ++j) wv[j] = *reinterpret_cast<const uint4*>(myW + (size_t)(bi * G + j) * 2048);
#pragma unroll
    for (int j = 0; j < G; ++j) {
      uint32_t ex[8];
      tc::expand_nibbles(wv[j].x, ex[0], ex[1]);
      tc::expand_nibbles(wv[j].y, ex[2], ex[3]);
      tc::expand_nibbles(wv[j].z, ex[4], ex[5]);
      tc::expand_nibbles(wv[j].w, ex[6], ex[7]);
      tc::tmem_st8(tmem_a + lane_off + (uint32_t)((slot * G + j) * 8), ex);
    }
    tc::tmem_wait_st();
    tc::fence_before_sync();
    if (FW == 1) __syncthreads();
    else asm volatile("bar.sync 1, 128;" ::: "memory");  // warpgroup 0 only
    // the accumulator slot is overwritten: warpgroup 1 must have read batch bi - 2 out of it (this warpgroup has)
    if (FW == 2 && bi >= 2) ok = tc::mbar_wait(&bar_free[slot], (uint32_t)((bi >> 1) - 1) & 1u) && ok;
    // MMA issue is spread over the four warps (one lane each, G / 4 MMAs): a single thread needs ~90 clocks per
    // tcgen05.mma, which at 8 per batch was 0.4 us on the critical path.  Every issuer commits to the batch's barrier.
    if (lane == 0) {
      tc::fence_after_sync();
      const uint32_t b0 = tc::smem_u32(sB);
#pragma unroll
      for (int jj = 0; jj < G / 4; ++jj) {
        const int j = wq * (G / 4) + jj;
        const uint64_t bdesc = tc::smem_desc_kmajor(b0 + (uint32_t)(bi * G + j) * (NT * 32), 128, 256);
        tc::mma_i8_ts(tmem_d + (uint32_t)((slot * G + j) * NT), tmem_a + (uint32_t)((slot * G + j) * 8), bdesc, IDESC, 0u);
      }
      tc::mma_commit(&bar_mma[slot]);
    }
    __syncwarp();
    stamp();                                            // 5, 6, ...: batch expanded and issued
    if (bi > 0) fold(bi - 1);
  }
  if (nbatch > 0 && wg == 0) fold(nbatch - 1);
  __syncthreads();                                      // every thread is done with the slabs and with TMEM
  stamp();                                              // all batches folded

  // one output value: column (sequence) n of this thread's row
  auto emit = [&](int n, float v, float add) {
    const float partner = __shfl_xor_sync(0xffffffffu, v, 1);
    if (n < a.cols && row < a.N) {
      const size_t base = (size_t)n * a.ldy;
      switch (a.epi) {
        case Q4B_EPI_STORE: reinterpret_cast<__half*>(a.Y)[base + row] = __float2half_rn(v); break;
        case Q4B_EPI_BIASF:
          reinterpret_cast<__half*>(a.Y)[base + row] = __float2half_rn(v + add);
          break;
        case Q4B_EPI_RESID: reinterpret_cast<float*>(a.Y)[base + row] = add + v; break;
        case Q4B_EPI_LOGITS: reinterpret_cast<float*>(a.Y)[base + row] = v; break;
        case Q4B_EPI_SWIGLU:
          if ((r & 1) == 0) reinterpret_cast<__half*>(a.Y)[base + (row >> 1)] = __float2half_rn(v / (1.f + __expf(-v)) * partner);
          break;
        default: break;
      }
    }
  };

  // ---- split-K.  Few accumulators per thread: every peer pushes its partial sums into the leader's shared memory
  // (remote stores), one cluster barrier publishes them and the leader adds them in rank order and writes the output.
  // Many accumulators (16 / 32 activation rows): a reduce-scatter.  Every CTA parks its partials in its own dead
  // weight slab; after one cluster barrier rank r sums columns r, r + ksplit, ... over all ranks (in rank order, so
  // the result does not depend on which CTA does it) and writes those columns itself.  Per thread that is NACC remote
  // loads spread over the cluster instead of (ksplit - 1) NACC on the leader.
  // (A variant that pushes every partial to its column's owner and needs one barrier was 0.3-0.9 us faster per launch
  // in isolation and 4.5 % slower in the full 32-sequence step, 12.15 K against 12.75 K tok/s; it was not kept.)
  if (a.ksplit > 1 && !PUSH) {
    float* part = reinterpret_cast<float*>(slabW);      // [NTOT][128], every thread is past its last slab read
#pragma unroll
    for (int n = 0; n < NACC; ++n) part[(cbase + n) * ROWS + r] = acc[n];
    cluster_sync_all();
    load_addends();                                     // in flight together with the remote loads below
    // This CTA sums columns ks, ks + ksplit, ...; its warpgroups take them alternately.  All remote loads of a thread
    // are issued before the first add: own column ii (= ks + (wg + FW ii) ksplit), rank rr -> pv[ii ksplit + rr].
    constexpr int NPV = NTOT / FW + 8;
    float pv[NPV];
#pragma unroll
    for (int q = 0; q < NPV; ++q) {
      const int ii = q / a.ksplit, rr = q - ii * a.ksplit, n = ks + (wg + FW * ii) * a.ksplit;
      pv[q] = n < NTOT ? ld_peer_f32(part + n * ROWS + r, (uint32_t)rr) : 0.f;
    }
    float* fin = reinterpret_cast<float*>(sB);          // [own column][256]: the B operand is dead (all MMAs retired)
    {
      float v = 0.f;
#pragma unroll
      for (int q = 0; q < NPV; ++q) {
        const int ii = q / a.ksplit, rr = q - ii * a.ksplit;
        v += pv[q];                                     // rank order 0, 1, ... within a column
        if (rr == a.ksplit - 1) {
          if (ii < NOWN) fin[ii * NTHR + t] = v;
          v = 0.f;
        }
      }
    }
#pragma unroll
    for (int ii = 0; ii < NOWN; ++ii) {
      const int n = ks + (wg + FW * ii) * a.ksplit;
      if (n < NTOT) emit(n, fin[ii * NTHR + t], addend[ii]);
    }
    cluster_sync_all();                                 // peers stay resident until everyone has read them
    stamp();                                            // split-K reduced
  } else {
    if (a.ksplit > 1) {
      if (ks != 0) {
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(tc::smem_u32(red_buf)), "r"(0));
#pragma unroll
        for (int n = 0; n < NACC; ++n)
          asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + (uint32_t)((((ks - 1) * NACC + n) * ROWS + t) * 4)),
                       "f"(acc[n])
                       : "memory");
      }
      cluster_sync_all();
      if (ks == 0) {
        for (int r = 1; r < a.ksplit; ++r) {
#pragma unroll
          for (int n = 0; n < NACC; ++n) acc[n] += red_buf[((r - 1) * NACC + n) * ROWS + t];
        }
      }
    }
    stamp();                                            // split-K reduced
    if (ks == 0 && a.epi == Q4B_EPI_SWIGLU_Q8) {
      // SwiGLU product rounded to fp16, then the Q8_1 quantiser of quant_q8_1.cu on it (reference QUANT_Q8,
      // lab/qwen_batched.py:1030-1039): a 32-block of the product is 64 weight rows = two warps of this tile.
      float* wmax = xs;                                 // [column][TMEM lane quarter]; the activation scales are dead
      float act[NACC];
#pragma unroll
      for (int n = 0; n < NACC; ++n) {
        const float v = acc[n];
        const float partner = __shfl_xor_sync(0xffffffffu, v, 1);
        const bool live = (r & 1) == 0 && row < a.N && cbase + n < a.cols;
        act[n] = live ? __half2float(__float2half_rn(v / (1.f + __expf(-v)) * partner)) : 0.f;
        const float m = warp_max(fabsf(act[n]));
        if (lane == 0) wmax[(cbase + n) * 4 + wq] = m;
      }
      __syncthreads();
      int8_t* qo = reinterpret_cast<int8_t*>(a.Y);
      __half* dout = reinterpret_cast<__half*>(const_cast<void*>(a.AUX));
#pragma unroll
      for (int n = 0; n < NACC; ++n) {
        const int col = cbase + n;
        const float amax = fmaxf(wmax[col * 4 + wq], wmax[col * 4 + (wq ^ 1)]);
        const float dq = amax / 127.f;
        const int q = dq > 0.f ? __float2int_rn(act[n] / dq) : 0;
        if ((r & 1) == 0 && row < a.N && col < a.cols) qo[(size_t)col * a.ldy + (row >> 1)] = (int8_t)q;
        if ((wq & 1) == 0 && lane == 0 && row < a.N && col < a.cols) dout[(size_t)col * (a.ldy >> 5) + (row >> 6)] = __float2half_rn(dq);
      }
    } else if (ks == 0) {
#pragma unroll
      for (int n = 0; n < NACC; ++n) {
        float add = PUSH ? addend[n < NOWN ? n : 0] : 0.f;
        if (!PUSH) {                                     // unsplit launch with many columns: fetched here
          add = 0.f;
          if (row < a.N && cbase + n < a.cols) {
            if (a.epi == Q4B_EPI_BIASF) add = reinterpret_cast<const float*>(a.AUX)[row];
            if (a.epi == Q4B_EPI_RESID) add = reinterpret_cast<const float*>(a.Y)[(size_t)(cbase + n) * a.ldy + row];
          }
        }
        emit(cbase + n, acc[n], add);
      }
    }
  }
  tc::fence_before_sync();
  if (tc::drain_mmas_on_failure(ok, wg == 0 && lane == 0, &bar_drain) && t == 0) atomicExch(a.status, 1u);   // any thread's expired wait
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, TCOLS);
  stamp();                                              // end
  if (tr) tr[15] = (unsigned long long)tri;
}

unsigned long long* g_trace = nullptr;

struct Geometry {
  int ksplit, gps;
  size_t smem;
  uint32_t tcols;
};

size_t smem_bytes(int gps, int nt, int nacc, int ksplit) {
  size_t s = (size_t)gps * 8 * (2048 + 256);   // weight slabs
  s += (size_t)gps * 8 * nt * 32;              // B operand
  s += (size_t)gps * 8 * nt * 4;               // activation block scales (+ the norm reduction scratch)
  if (nacc <= 8) s += (size_t)(ksplit - 1) * nacc * ROWS * 4;   // split-K partials pushed to the leader
  return s + 128;
}

bool plan(int N, int K, int nt, int nacc, Geometry& g) {
  const int GT = K / 256, tiles = (N + ROWS - 1) / ROWS;
  const int G = nt <= 16 ? 8 : 4;
  const uint32_t need = 2 * G * 8 + 2 * G * nt;
  g.tcols = need <= 128 ? 128 : (need <= 256 ? 256 : 512);
  const int sms = sm_count();
  int best = -1;
  for (int ks = 1; ks <= 8 && ks <= GT; ++ks) {
    const int gps = (GT + ks - 1) / ks;
    if ((ks - 1) * gps >= GT) continue;                 // an empty slice
    if (gps * 8 / G > MAX_BATCH || gps > 10) continue;
    if (smem_bytes(gps, nt, nacc, ks) > MAX_DYN_SMEM) continue;
    if (g.tcols == 512 && best > 0 && (long)tiles * ks > (long)sms) break;   // one CTA per SM: stay within one wave
    best = ks;
    if ((long)tiles * ks >= (long)sms * 3 / 2) break;   // enough CTAs for two per SM on most of the machine
  }
  if (best < 0) return false;
  g.ksplit = best;
  g.gps = (GT + best - 1) / best;
  g.smem = smem_bytes(g.gps, nt, nacc, best);
  // tcgen05.alloc blocks while an SM's 512 TMEM columns are taken; CTAs of one cluster wait for each other, so the
  // number of co-resident CTAs times their columns must never exceed 512.  Shared memory is the limiter we control.
  const size_t max_ctas = 512 / g.tcols;
  const size_t floor_smem = (227 * 1024) / (max_ctas + 1) + 1024;
  if (g.smem < floor_smem) g.smem = floor_smem;
  return true;
}

template <int MODE, int NT>
int launch(const StreamArgs& a, const Geometry& g, cudaStream_t st) {
  auto kern = mmq_stream_kernel<MODE, NT>;
  if (cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), MAX_DYN_SMEM); e != cudaSuccess) {
    set_cuda_error(e, "mmq_stream: cudaFuncSetAttribute");
    return Q4B_E_CUDA;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((a.N + ROWS - 1) / ROWS, g.ksplit, 1);
  cfg.blockDim = dim3(ROWS * ((MODE == MODE_Q8 && NT >= 16) ? 2 : 1), 1, 1);
  cfg.dynamicSmemBytes = g.smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[na].val.programmaticStreamSerializationAllowed = 1;
  ++na;
  if (g.ksplit > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = g.ksplit;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a);
  if (e != cudaSuccess) {
    set_cuda_error(e, "mmq_stream: launch");
    return Q4B_E_CUDA;
  }
  return Q4B_OK;
}

template <int MODE>
int launch_nt(int nt, const StreamArgs& a, const Geometry& g, cudaStream_t st) {
  if (nt == 8) return launch<MODE, 8>(a, g, st);
  if (nt == 16) return launch<MODE, 16>(a, g, st);
  return launch<MODE, 32>(a, g, st);
}

}  // namespace

// Device buffer for the optional timeline stamps of the next launches (16 x uint64 per CTA, up to 4096 CTAs); null = off.
void mmq_stream_trace(unsigned long long* buf) { g_trace = buf; }

// Q8_1 mode over the K window [32 kbw, 32 kbw + Kwin) of matrices whose rows hold Ktot values.
static int mmq_stream_window(const void* W, const void* S, const void* X, const void* XD, void* Y, const void* AUX, int N, int Ktot,
                             int kbw, int Kwin, int cols, int epilogue, int ldy, uint32_t* status, cudaStream_t st) {
  const int nt = cols <= 8 ? 8 : (cols <= 16 ? 16 : 32);
  Geometry g;
  if (!plan(N, Kwin, nt, nt, g)) return fail(Q4B_E_SHAPE, "mmq_stream: K window does not fit");
  StreamArgs a;
  a.W = reinterpret_cast<const uint8_t*>(W);
  a.S = reinterpret_cast<const __half*>(S);
  a.X = X;
  a.XD = reinterpret_cast<const __half*>(XD);
  a.NW = nullptr;
  a.eps = 0.f;
  a.trace = g_trace;
  a.Y = Y;
  a.AUX = AUX;
  a.status = status;
  a.N = N;
  a.K = Kwin;
  a.cols = cols;
  a.epi = epilogue;
  a.ldy = ldy;
  a.gps = g.gps;
  a.ksplit = g.ksplit;
  a.KBT = Ktot / 32;
  a.kbw = kbw;
  return launch_nt<MODE_Q8>(nt, a, g, st);
}

// mode: 0 exact fp16 x, 1 exact fp32 x, 2 Q8_1, 3 exact with RMSNorm of the fp32 row X fused in front.
// cols: 1 for the exact modes, 1..32 sequences for Q8_1.
int mmq_stream(const void* W, const void* S, const void* X, const void* XD, void* Y, const void* AUX, int N, int K,
               int cols, int mode, int epilogue, int ldy, uint32_t* status, cudaStream_t st, const float* norm_w,
               float eps) {
  if (N <= 0 || K <= 0 || (K % 256)) return fail(Q4B_E_SHAPE, "mmq_stream: N > 0 and K a positive multiple of 256 required");
  if (mode < 0 || mode > 3) return fail(Q4B_E_ARG, "mmq_stream: unknown mode");
  if (mode == MODE_NORM && (!norm_w || !aligned16(norm_w))) return fail(Q4B_E_ALIGN, "mmq_stream: norm mode needs 16-byte aligned weights");
  if (epilogue < Q4B_EPI_STORE || epilogue > Q4B_EPI_SWIGLU_Q8) return fail(Q4B_E_ARG, "mmq_stream: unknown epilogue");
  if (epilogue == Q4B_EPI_SWIGLU_Q8 && (mode != MODE_Q8 || (N % 64) || !AUX))
    return fail(Q4B_E_SHAPE, "mmq_stream: swiglu_q8 needs Q8_1 mode, N a multiple of 64 and the scale output");
  if (cols < 1 || cols > 32 || (mode != MODE_Q8 && cols != 1)) return fail(Q4B_E_SHAPE, "mmq_stream: 1..32 columns (1 in exact mode)");
  if (epilogue == Q4B_EPI_SWIGLU && (N % 2)) return fail(Q4B_E_SHAPE, "mmq_stream: swiglu needs an even row count");
  if (!W || !S || !X || !Y || !status || !aligned16(W) || !aligned16(S) || !aligned16(X))
    return fail(Q4B_E_ALIGN, "mmq_stream: W, S, X must be non-null and 16-byte aligned");
  if (mode == MODE_Q8 && !XD) return fail(Q4B_E_ALIGN, "mmq_stream: Q8_1 mode needs the block scales");
  if (epilogue == Q4B_EPI_BIASF && !AUX) return fail(Q4B_E_ALIGN, "mmq_stream: biasf needs AUX");
  const int nt = mode != MODE_Q8 ? 8 : (cols <= 8 ? 8 : (cols <= 16 ? 16 : 32));
  Geometry g;
  if (!plan(N, K, nt, mode == MODE_Q8 ? nt : 1, g)) {
    // K too long for one CTA's shared memory even at the largest split: cover it in windows, accumulating into the
    // fp32 output (epilogues that are linear in K only: the first window stores or adds, the others add).
    if (mode != MODE_Q8 || (epilogue != Q4B_EPI_RESID && epilogue != Q4B_EPI_LOGITS))
      return fail(Q4B_E_SHAPE, "mmq_stream: no K split fits shared memory for this K");
    for (int nwin = 2; nwin <= 8; ++nwin) {
      const int gw = (K / 256 + nwin - 1) / nwin;         // 256-groups per window
      Geometry gt;
      if (!plan(N, gw * 256, nt, nt, gt)) continue;
      for (int w = 0; w * gw < K / 256; ++w) {
        const int kw = std::min(gw, K / 256 - w * gw) * 256;
        int rc = mmq_stream_window(W, S, X, XD, Y, AUX, N, K, w * gw * 8, kw, cols, w == 0 ? epilogue : Q4B_EPI_RESID, ldy, status, st);
        if (rc != Q4B_OK) return rc;
      }
      return Q4B_OK;
    }
    return fail(Q4B_E_SHAPE, "mmq_stream: no K split fits shared memory for this K");
  }
  if (epilogue == Q4B_EPI_SWIGLU_Q8 && g.ksplit > 1 && nt > 8)
    return fail(Q4B_E_SHAPE, "mmq_stream: swiglu_q8 has no split-K form for more than 8 activation rows");
  StreamArgs a;
  a.W = reinterpret_cast<const uint8_t*>(W);
  a.S = reinterpret_cast<const __half*>(S);
  a.X = X;
  a.XD = reinterpret_cast<const __half*>(XD);
  a.NW = norm_w;
  a.eps = eps;
  a.trace = g_trace;
  a.Y = Y;
  a.AUX = AUX;
  a.status = status;
  a.N = N;
  a.K = K;
  a.cols = cols;
  a.epi = epilogue;
  a.ldy = ldy;
  a.gps = g.gps;
  a.ksplit = g.ksplit;
  a.KBT = K / 32;
  a.kbw = 0;
  if (mode == MODE_X16) return launch_nt<MODE_X16>(nt, a, g, st);
  if (mode == MODE_X32) return launch_nt<MODE_X32>(nt, a, g, st);
  if (mode == MODE_NORM) return launch<MODE_NORM, 8>(a, g, st);
  return launch_nt<MODE_Q8>(nt, a, g, st);
}

}  // namespace q4b
