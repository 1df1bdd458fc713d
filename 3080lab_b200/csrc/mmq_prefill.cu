// Q8_1 x Q4_0 matrix product for prefill (hundreds to thousands of activation rows) on the tcgen05 int8 tensor cores.
//
//   Y[p, m] = epilogue( sum_b dw[m, b] * dx[p, b] * dot_b[m, p] ),  dot_b exact int32 over one 32-weight block
//
// the arithmetic of the reference's MMQ (gemm_q4i8_ms_source, lab/qwen_batched.py:1271-1561; block arithmetic
// :1237-1243): one int8 MMA per k-block because every block has its own pair of scales, fp32 rescale-and-add per block
// in ascending k order.  What changes is where things live on Blackwell:
//   * CTA tile = 128 weight rows (UMMA M) x 128 activation rows (UMMA N); one tcgen05.mma.kind::i8 (K = 32) per k-block
//     into one of three TMEM accumulator slots (128 columns each);
//   * weights arrive tile-packed through bulk (TMA) copies in batches of 8 k-blocks (ring of 4); four EXPANDER warps
//     (thread = row) turn nibbles into signed bytes 16 (q - 8) and write them into a ring of eight A operands in tensor
//     memory (tcgen05.st), running ahead of the MMAs by up to eight k-blocks;
//   * activations arrive pre-tiled from the quantiser (quant_q8_1.cu, "tiled" outputs): per (128-row tile, k-block)
//     4096 bytes already in the UMMA K-major core-matrix order + 128 fp32 block scales, one bulk copy per stage
//     (ring of 8), used directly as the B operand;
//   * one thread issues the MMAs, one the bulk copies;
//   * SIXTEEN rescale warps (four per TMEM lane quarter, 32 accumulator columns each) read an accumulator slot back in
//     two halves of 16 columns, scale by dw * dx and add into fp32 registers, on a rolling schedule: the read of the
//     next half is always in flight while the previous one is folded.
// The rescale is CUDA-core work: per output and k-block one integer add (exact int -> float through a magic constant,
// as the reference plants it in the C operand of its mma.sync, lab/qwen_batched.py:1016-1041, 1237-1243) and three fp32
// operations (subtract the constant, scale product, fused multiply-add).  Measured on B200: two-wide fp32 instructions
// (f32x2) retire 128 lane-operations per clock and SM, the same as scalar ones, and integer adds share that rate, so a
// 128 x 128 x 32 k-block costs >= 384 fp32 + integer clocks against 64 tensor-core clocks: this formulation of
// Q4_0 x Q8_1 tops out near a sixth of the int8 peak whatever the pipeline does; the pipeline's job is to keep the
// fp32 pipe busy.  (A variant that pre-loaded the accumulator slot with the magic constant through tcgen05.st, so
// that the words came back as floats, was measured: the extra 64 KB of tensor-memory writes per k-block cost more than
// the integer adds they saved.)
// What sets the pace (clock trace of every role, launch time against K, launches with parts removed): no single stage;
// barriers, waits and commits alone take half of a k-block's time.  A dependent mbarrier wait on a completed phase costs
// 86 clocks on an idle SM and ~180 in this kernel, a k-block costs each rescale warp two of them plus two tensor-memory
// read latencies, and the four rescale warps of a scheduler run in step.  Waits therefore park (suspend-time hint) with
// all lanes polling.  The epilogues are written for latency, not instruction count: loads hoisted above the stores of
// the same array, one SwiGLU product per lane pair and token, fp16 outputs as 4-byte row-pair stores.
// All waits are bounded; after the first expired wait a thread stops waiting (status word, garbage out, no hang).
#include <algorithm>

#include "q4b_internal.h"
#include "tc05.cuh"

namespace q4b {

namespace {

constexpr int NSLOT = 3;                  // accumulator slots in tensor memory (128 columns each)
constexpr int NA = 8;                     // A operands in tensor memory (8 columns each)
constexpr int NRW = 16;                   // rescale warps: (TMEM lane quarter) x (column quarter)
constexpr int NEW = 4;                    // expander warps: one per TMEM lane quarter
constexpr int PF_THREADS = (NRW + NEW + 2) * 32;   // + MMA warp + copy warp
constexpr int W_MMA = NRW + NEW, W_COPY = NRW + NEW + 1;
constexpr int NTOK = 128;                 // activation rows per CTA tile (UMMA N)
constexpr int SB = 8;                     // activation stages (one k-block each)
constexpr int WB = 4;                     // weight batches in flight (8 k-blocks each)
constexpr uint32_t STAGE_BYTES = 4096 + 512;
constexpr uint32_t WBATCH_W = 8 * 2048, WBATCH_S = 8 * 256;
constexpr size_t PF_SMEM = (size_t)WB * (WBATCH_W + WBATCH_S) + (size_t)SB * STAGE_BYTES + 128;
// ---- fp16 mode (the second instance of the kernel; q4b_mm_prefill_q4_0_f16) ------------------------------------------
// The arithmetic of the reference's `cublas` prefill mode (scripts/qwen_prefill.py:37-53 DEQ, :156-160): weights
// dequantised to fp16 ((q - 8) exact, times the block scale, one rounding), fp16 activations, fp32 accumulation - but
// with the dequantisation inside the GEMM instead of through a dense fp16 copy of the matrix: expander warps (two groups
// of four here, each owning one operand slot) write fp16 A operands into tensor memory, tcgen05.mma.kind::f16 accumulates over ALL of K into one
// tensor-memory tile per 128 rows, and the per-block rescale - the int8 mode's bottleneck - does not exist.  A CTA makes
// 256 weight rows x 128 tokens (two accumulators), so every activation record fetched from L2 feeds two MMAs.  The
// pipeline moves UNITS of G k-blocks so that the one MMA-issuing thread pays its waits and commits once per 4 G MMAs.
// CTAs are persistent (one per SM, tiles c, c + #CTAs, ..): rings and parities run on across tiles, so the next tile's
// copies, its first expansion and - once the accumulators are in registers - its first MMAs proceed under the epilogue.
// Measured on B200, gate/up 2048 x 17920 x 1536: 134 - 145 us = 780 - 840 TFLOP/s (about half of the measured cuBLAS bf16
// peak) against 586 us for the int8 mode; ~0.25 us per k-block and 5.6 us fixed per tile (8.1 before the CTAs were
// persistent; removing the copies changes nothing, half of the MMAs -16 %, the expansion -14 %: again no single stage).
constexpr int G16 = 4;                    // k-blocks per unit
constexpr int MH16 = 2;                   // row halves: a CTA makes 256 weight rows x 128 tokens, two accumulators, so that
                                          // an activation record fetched from L2 feeds two MMAs (the copies set the pace)
constexpr int WB16 = 2;                   // weight batches in flight (8 k-blocks x 2 row halves each)
constexpr int NAU = 2;                    // A units in tensor memory (G16 x MH16 x 16 columns each)
constexpr int SBU = 3;                    // activation units in shared memory
constexpr int NXG = (NRW + NEW) / 4;      // groups of four worker warps (one warp per TMEM lane quarter)
constexpr uint32_t REC16 = 128 * 32 * 2;  // one k-block of fp16 activations for 128 tokens
constexpr uint32_t UNIT16 = G16 * REC16;
constexpr uint32_t SCR16 = 128 * 72 * 2;  // fp16 mode's epilogue staging (the weight ring is live then: the next tile's weights)
constexpr size_t PF_SMEM16 = (size_t)WB * (WBATCH_W + WBATCH_S) + (size_t)SBU * UNIT16 + SCR16 + 128;

struct PrefillArgs {
  const uint8_t* Wt;   // tile-packed nibbles
  const __half* St;    // tile-packed scales
  const uint8_t* Xt;   // tiled Q8_1 activations [P/128][K/32][4608]
  void* Y;
  const void* AUX;
  uint32_t* status;
  int N, K, P, epi, ldy;
  int pair16;          // fp16 outputs may go out two rows at a time (N, ldy even, Y 4-byte aligned)
  int tx, ty, ntiles;  // fp16 mode (persistent CTAs): row pairs, token tiles, tiles in all = tx * ty * K parts
  long long* trace;    // per-role clock stamps of CTA (0, 0, 0), [11][64] (see q4b_mmq_prefill_trace); null = off
  int debug_no_copy;   // TRACE instance only: the copy thread issues nothing, every wait of the pipeline runs out (see
                       // q4b_debug_mmq_prefill_expired_wait)
  float* Y2;           // split launch: where parts 1 .. of K store their sums, fp32 [parts - 1][P, ldy]
  int kb_bound[5];     // k-block bounds of the parts (multiples of 8); unsplit: {0, K / 32}
  // fused RoPE + K/V append (Q4B_EPI_BIASF_ROPE_KV): tokens of ONE sequence at positions pos0 .., cache fp16 [NKV, max_len, 128]
  const float* cosT;
  const float* sinT;
  __half* kc;
  __half* vc;
  int NH, NKV, max_len, pos0;
};

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   tc::smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(tc::smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }
// Wait unless an earlier wait of this thread already expired.  Worker warps call it with all 32 lanes (one polling lane
// plus a warp barrier was measured 4 % slower); the tries park the thread (suspend hint) instead of spinning, which was
// worth little by itself but keeps waiting warps out of the issue slots.
__device__ __forceinline__ void waitb(uint64_t* bar, uint32_t parity, bool& ok) {
  if (ok) ok = tc::mbar_wait_parked(bar, parity);
}
// Bits of float(12582912 + d) for -2^22 <= d < 2^22 without an addition: the low 22 bits of d, bit 22 inverted, 0x4B0 on
// top.  One LOP3 with two constant operands that select, per bit, (b, c) = (0,0) d, (0,1) ~d, (1,0) 0, (1,1) 1.
__device__ __forceinline__ uint32_t magic_lop(uint32_t d) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0x9A;" : "=r"(r) : "r"(d), "r"(0xFF800000u), "r"(0x4B400000u));
  return r;
}
// SwiGLU of one gate/up row pair (adjacent TMEM lanes = adjacent threads) for the token pair (2 j, 2 j + 1) held in `acc`:
// the even lane takes token 2 j, the odd lane token 2 j + 1, so each lane evaluates 16 of the 32 products (one exchange
// and one division per token pair instead of two of each).  Returns the product and the token n it belongs to.
// FAST (fp16 mode, whose results are held to a tolerance, not to bits): the quotient through the approximate reciprocal.
template <bool FAST>
__device__ __forceinline__ float swiglu_pair(uint64_t acc, int r, int j, int& n) {
  const bool odd = r & 1;
  const float v0 = tc::lo2(acc), v1 = tc::hi2(acc);
  const float got = __shfl_xor_sync(0xffffffffu, odd ? v0 : v1, 1);
  const float g = odd ? got : v0, u = odd ? v1 : got;
  n = 2 * j + (odd ? 1 : 0);
  if constexpr (FAST) return __fdividef(g, 1.f + __expf(-g)) * u;
  return g / (1.f + __expf(-g)) * u;
}
// Second halves of the two fused epilogues, kept out of line so that they cost the main loop no registers.
// RoPE + cache write from the rounded tile in shared memory: thread = (row pair 2 pr, 2 pr + 1 of the head, 16 tokens), so
// that every access is a 4-byte one and a warp's stores cover 128 contiguous bytes (2-byte stores, one row per thread,
// were measured at ~20 clocks per warp store).
__device__ __noinline__ void rope_kv_phase(const PrefillArgs& a, const __half* ybuf, int head, int tok_base, int t) {
  const int r = 2 * (t & 63), dd = r & 63, row = head * 128 + r;
  const bool rotate = head < a.NH + a.NKV, upper = r >= 64;
#pragma unroll 4
  for (int n = 0; n < 16; ++n) {
    const int tl = (t >> 6) * 16 + n, p = tok_base + tl, pos = a.pos0 + p;
    if (p >= a.P || pos >= a.max_len) continue;
    __half2 outv = *reinterpret_cast<const __half2*>(ybuf + tl * 128 + r);
    if (rotate) {
      const float2 mine = __half22float2(outv);
      const float2 other = __half22float2(*reinterpret_cast<const __half2*>(ybuf + tl * 128 + (r ^ 64)));
      const float2 c = __ldg(reinterpret_cast<const float2*>(a.cosT + (size_t)pos * 64 + dd));   // read-only path: free to move above the stores
      const float2 s = __ldg(reinterpret_cast<const float2*>(a.sinT + (size_t)pos * 64 + dd));
      float lo0, hi0, lo1, hi1;
      if (!upper) {
        rope_pair(mine.x, other.x, c.x, s.x, lo0, hi0);
        rope_pair(mine.y, other.y, c.y, s.y, lo1, hi1);
        outv = __floats2half2_rn(lo0, lo1);
      } else {
        rope_pair(other.x, mine.x, c.x, s.x, lo0, hi0);
        rope_pair(other.y, mine.y, c.y, s.y, lo1, hi1);
        outv = __floats2half2_rn(hi0, hi1);
      }
    }
    *reinterpret_cast<__half2*>(reinterpret_cast<__half*>(a.Y) + (size_t)p * a.ldy + row) = outv;
    if (head >= a.NH + a.NKV) *reinterpret_cast<__half2*>(a.vc + ((size_t)(head - a.NH - a.NKV) * a.max_len + pos) * 128 + r) = outv;
    else if (head >= a.NH) *reinterpret_cast<__half2*>(a.kc + ((size_t)(head - a.NH) * a.max_len + pos) * 128 + r) = outv;
  }
}

// Q8_1 quantiser over the rounded SwiGLU products in shared memory: 128 tokens x 2 blocks x 8 lanes = 4 tasks per thread.
// The two records (k-blocks 2 row_tile, 2 row_tile + 1 of this token tile; adjacent in the operand) are put together in
// shared memory behind the products and leave as 16-byte stores: the quantiser's own stores are 2 bytes wide and scattered.
__device__ __noinline__ void swiglu_q8_phase(const PrefillArgs& a, const __half* abuf, int row_tile, int tok_tile, int t) {
  const int KB2 = a.N >> 6;                                // k-blocks of the product row
  uint8_t* rec = reinterpret_cast<uint8_t*>(const_cast<__half*>(abuf)) + 128 * 64 * 2;   // [2][STAGE_BYTES]
#pragma unroll 1
  for (int j = 0; j < 4; ++j) {
    const int task = t + j * (NRW * 32);
    const int sub = task & 7, hb = (task >> 3) & 1, nn = task >> 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(abuf + nn * 64 + hb * 32 + sub * 4);
    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    const float x4[4] = {lo.x, lo.y, hi.x, hi.y};
    quant_block4_tiled(x4, rec + (size_t)hb * STAGE_BYTES, nn, sub);
  }
  asm volatile("bar.sync 1, %0;" ::"n"(NRW * 32) : "memory");
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a.Y) + ((size_t)tok_tile * KB2 + (size_t)row_tile * 2) * STAGE_BYTES);
  const uint4* src = reinterpret_cast<const uint4*>(rec);
  for (int i = t; i < 2 * (int)STAGE_BYTES / 16; i += NRW * 32) dst[i] = src[i];
}

template <bool TRACE, bool F16>
__global__ void __launch_bounds__(PF_THREADS, 1) mmq_prefill_kernel(const __grid_constant__ PrefillArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  // "empty" barriers are waited on with the inverted parity the first time round (a fresh barrier reads as having
  // completed the phase before its first), so no pre-arrivals are needed
  // "empty" barriers are waited on with the inverted parity the first time round (a fresh barrier reads as having
  // completed the phase before its first), so no pre-arrivals are needed.  (One combined barrier per k-block for the MMA
  // issuer - operand written, stage landed, slot free - was measured: 8 % slower than these separate ones.)
  __shared__ __align__(8) uint64_t w_full[WB], w_empty[WB], b_full[SB], b_empty[SB], a_full[NA], a_empty[NA], d_full[NSLOT],
      d_empty[NSLOT];
  __shared__ __align__(8) uint64_t drain;                  // failure path only (tc::drain_mmas_on_failure)
  __shared__ uint32_t tmem_base_s;

  uint8_t* slabW = smem;                                   // [WB][8][128 rows][16]
  uint8_t* slabS = slabW + (size_t)WB * WBATCH_W;          // [WB][8][128] fp16
  uint8_t* stage = slabS + (size_t)WB * WBATCH_S;          // [SB][4608]

  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  // K range of this CTA: all of K, or with a split launch (gridDim.z = 2 .. 4) part blockIdx.z of it (bounds in whole
  // batches of 8 k-blocks).  Part 0 adds its sums to Y; part z > 0 stores them as fp32 into Y2[z - 1]; whoever reads Y next
  // adds the parts in that fixed order.
  const int KBT = a.K >> 5;
  const int kb_lo = a.kb_bound[blockIdx.z];
  const int KB = a.kb_bound[blockIdx.z + 1] - kb_lo, NBATCH = KB >> 3;
  const int row_tile = F16 ? 2 * (int)blockIdx.x : (int)blockIdx.x, tok_tile = blockIdx.y;   // fp16 mode: row tiles 2 x, 2 x + 1
  [[maybe_unused]] const bool have1 = F16 && (row_tile + 1) * 128 < a.N;
  const size_t wbase = (size_t)row_tile * KBT + kb_lo;     // k-block index of this row tile in the packed arrays
  const uint8_t* xbase = a.Xt + ((size_t)tok_tile * KBT + kb_lo) * (F16 ? REC16 : STAGE_BYTES);

  [[maybe_unused]] long long t_entry = 0;
  if constexpr (TRACE) t_entry = clock64();
  if (warp == 0) {
    tc::tmem_alloc(&tmem_base_s, 512);
    tc::tmem_relinquish();
  }
  if (t == 32) {
    for (int i = 0; i < WB; ++i) {
      tc::mbar_init(&w_full[i], 1);
      tc::mbar_init(&w_empty[i], NEW + NRW);               // nibbles read by the expanders, scales by the rescale warps
    }
    for (int i = 0; i < SB; ++i) {
      tc::mbar_init(&b_full[i], 1);
      tc::mbar_init(&b_empty[i], F16 ? 1 : 1 + NRW);       // operand read by the MMA (commit), block scales by the rescale warps
    }
    for (int i = 0; i < NA; ++i) {
      tc::mbar_init(&a_full[i], NEW);
      tc::mbar_init(&a_empty[i], 1);                       // commit of the MMA that read it
    }
    tc::mbar_init(&drain, 1);
    for (int i = 0; i < NSLOT; ++i) {
      tc::mbar_init(&d_full[i], 1);                        // commit of the MMA that wrote it
      tc::mbar_init(&d_empty[i], NRW);                     // read out by every rescale warp
    }
    tc::mbar_fence_init();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  pdl_launch_dependents();
  const uint32_t tmem = tmem_base_s;
  // int8 mode: A NA x 8 columns, D NSLOT x 128 columns; fp16 mode: A NAU x G16 x MH16 x 16 columns, D MH16 x 128 columns
  const uint32_t tmem_a = tmem, tmem_d = tmem + (F16 ? NAU * G16 * MH16 * 16 : NA * 8);
  constexpr uint32_t IDESC = tc::idesc_i8(128, NTOK);
  bool ok = true;
  // TRACE instance only: timeline of the first 64 k-blocks of one CTA, one row per pipeline role (SM clock).  The stamps
  // cost ~10 % of the kernel's time even when switched off at run time, hence a separate instance.
  auto stamp = [&](int role, int b) {
    if constexpr (TRACE) {
      if (a.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && b < 64) a.trace[role * 64 + b] = clock64();
    }
  };

  if constexpr (TRACE) {
    if (a.trace && t == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) a.trace[10 * 64 + 0] = t_entry;
  }
  if (t == 0) stamp(10, 1);                                // set-up done (tensor memory, barriers)

  // ===================== fp16 mode: every role's main loop =====================
  // Persistent CTAs: CTA c works on tiles c, c + gridDim.x, ..  (tile = row pair fastest, then token tile, then K part).
  // Rings and their parities run on across tiles, so the copies, the first expansions and (once the accumulators have
  // been read out) the MMAs of the next tile proceed under the epilogue of this one.
  struct Tile16 {
    int row_tile, tok_tile, z, KB, NB, NU;
    bool have1;
    size_t wbase;
    const uint8_t* xbase;
  };
  [[maybe_unused]] auto tile16 = [&](int idx) {
    Tile16 q;
    const int rx = idx % a.tx, rest = idx / a.tx;
    q.row_tile = 2 * rx;
    q.tok_tile = rest % a.ty;
    q.z = rest / a.ty;
    const int lo = a.kb_bound[q.z];
    q.KB = a.kb_bound[q.z + 1] - lo;
    q.NB = q.KB >> 3;
    q.NU = q.KB / G16;
    q.have1 = (q.row_tile + 1) * 128 < a.N;
    q.wbase = (size_t)q.row_tile * KBT + lo;
    q.xbase = a.Xt + ((size_t)q.tok_tile * KBT + lo) * REC16;
    return q;
  };
  [[maybe_unused]] int ug0 = 0, wg0 = 0;                   // units / weight batches of this CTA's earlier tiles (expander warps)
  // fp16 mode's waits say where they gave up: the first expired wait leaves (info << 12 | id << 8 | 1) in the status word,
  // id 1 weights landed, 2 A slot free, 3 weight slot free, 4 activation slot free, 5 accumulators read out, 6 A operand
  // written, 7 activations landed, 8 accumulators complete; info = warp and unit, or tile count
  [[maybe_unused]] auto waitf = [&](uint64_t* bar, uint32_t parity, uint32_t id, uint32_t info) {
    if (ok && !tc::mbar_wait_parked(bar, parity)) {
      ok = false;
      atomicCAS(a.status, 0u, (info << 12) | (id << 8) | 1u);
    }
  };
  [[maybe_unused]] auto expand16 = [&](const Tile16& q) {
    // Every worker warp runs this loop (the weight ring counts all twenty), two groups of four warps (one warp per TMEM
    // lane quarter) expand, see below:
    // nibbles -> (q - 8) exactly in fp16 -> times the block scale, rounded once (gemv_v2_source's `dq`,
    // lab/qwen_batched.py:493-498) -> 16 columns of tensor memory per k-block.  A word's 8 weights come out as the pairs
    // (0,4) (1,5) (2,6) (3,7); the activation operand carries the same order within every 8 values.
    const int grp = warp >> 2;
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_off = (uint32_t)(32 * (warp & 3)) << 16;
    const __half2 c1032 = __float2half2_rn(1032.f), c16th = __float2half2_rn(0.0625f), c72 = __float2half2_rn(-72.f);
    const bool have1 = q.have1;
    for (int u = 0; u < q.NU; ++u) {
      const int b0 = u * G16, wg = wg0 + (b0 >> 3), ws = wg % WB16, ug = ug0 + u;
      if ((b0 & 7) == 0) waitb(&w_full[ws], (uint32_t)(wg / WB16) & 1u, ok);
      // EVERY warp waits for the slot of EVERY unit, not only of the units it expands: a parity wait is only sound if the
      // waiter has seen the phase before, and a group that skipped four units could otherwise meet a slot barrier two
      // phases behind (unit u - 4 written but not yet consumed), which reads as "free" and lets it overwrite live data.
      // Each tensor-memory slot belongs to ONE group of four warps: the even units (slot 0) to warps 16 .. 19, which have
      // no epilogue to do and so expand the next tile's first unit while the others still write this tile out, the odd
      // units (slot 1) to warps 0 .. 3.  A group therefore waits for consecutive phases of its own slot's barrier and for
      // nothing else - a parity wait is only sound for a waiter that is neither a phase early (a group that skipped units
      // met a barrier two phases behind and overwrote a live operand) nor a phase late (warps coming out of the epilogue
      // after the MMAs had moved on blocked for good); the other twelve warps do not touch the slots at all.
      static_assert(NAU == 2, "slot = unit parity");
      const int as = ug & 1;
      const int owner = as ? 0 : NXG - 1;
      if (owner == grp)
        waitf(&a_empty[as], ((uint32_t)(ug / NAU) & 1u) ^ 1u, 2u, (uint32_t)(warp << 8) | (uint32_t)(u & 255));
      if (owner == grp) {
        tc::fence_after_sync();
#pragma unroll
        for (int gh = 0; gh < G16 * MH16; ++gh) {
          const int g = gh >> 1, hf = gh & 1;
          if (hf && !have1) continue;
          const int bb = (b0 + g) & 7;
          const uint4 w = *reinterpret_cast<const uint4*>(slabW + (size_t)(ws * MH16 + hf) * WBATCH_W + (size_t)bb * 2048 + r * 16);
          const __half2 d2 = __half2half2(reinterpret_cast<const __half*>(slabS + (size_t)(ws * MH16 + hf) * WBATCH_S)[bb * 128 + r]);
          const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
          uint32_t ex[16];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t w0 = ww[i], w8 = ww[i] >> 8;
            const __half2 l0 = __hsub2(u32_as_h2((w0 & 0x000F000Fu) | 0x64006400u), c1032);
            const __half2 h0 = __hfma2(u32_as_h2((w0 & 0x00F000F0u) | 0x64006400u), c16th, c72);
            const __half2 l1 = __hsub2(u32_as_h2((w8 & 0x000F000Fu) | 0x64006400u), c1032);
            const __half2 h1 = __hfma2(u32_as_h2((w8 & 0x00F000F0u) | 0x64006400u), c16th, c72);
            ex[4 * i + 0] = h2_as_u32(__hmul2(l0, d2));
            ex[4 * i + 1] = h2_as_u32(__hmul2(h0, d2));
            ex[4 * i + 2] = h2_as_u32(__hmul2(l1, d2));
            ex[4 * i + 3] = h2_as_u32(__hmul2(h1, d2));
          }
          tc::tmem_st16(tmem_a + lane_off + (uint32_t)((as * G16 + g) * MH16 + hf) * 16, ex);
        }
        tc::tmem_wait_st();                                // warp-wide
        tc::fence_before_sync();
        if (lane == 0) tc::mbar_arrive(&a_full[as]);
        if ((warp & 3) == 0 && lane == 0) stamp(1, ug);
      }
      if (((b0 + G16 - 1) & 7) == 7) {
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&w_empty[ws]);      // this warp is done with the batch (whether it expanded any of it or not)
      }
    }
    ug0 += q.NU;
    wg0 += q.NB;
  };
  if (warp == W_COPY) {
    // ===================== bulk-copy producer (one thread) =====================
    if constexpr (F16) {
      if (lane == 0) {
        int ug = 0, wg = 0;                                // units / weight batches requested so far, over all tiles
        bool first = true;
        for (int tile = blockIdx.x; tile < a.ntiles && ok; tile += gridDim.x) {
          const Tile16 q = tile16(tile);
          for (int j = 0; j < q.NB && ok; ++j, ++wg) {     // a weight batch (both row halves), then its units
            const int s = wg % WB16;                       // (after an expired wait: no further copies)
            if (wg >= WB16) waitf(&w_empty[s], (uint32_t)(wg / WB16 - 1) & 1u, 3u, (uint32_t)(j & 255));
            tc::mbar_expect_tx(&w_full[s], (q.have1 ? 2u : 1u) * (WBATCH_W + WBATCH_S));
            for (int hf = 0; hf < (q.have1 ? 2 : 1); ++hf) {
              const size_t wb = q.wbase + (size_t)hf * KBT + (size_t)j * 8;
              bulk_g2s(slabW + (size_t)(s * MH16 + hf) * WBATCH_W, a.Wt + wb * 2048, WBATCH_W, &w_full[s]);
              bulk_g2s(slabS + (size_t)(s * MH16 + hf) * WBATCH_S, a.St + wb * 128, WBATCH_S, &w_full[s]);
            }
            if (first) {                                   // weights do not depend on the previous kernel, activations do
              pdl_wait();
              first = false;
            }
            for (int k = 0; k < 8 / G16; ++k, ++ug) {      // G16 consecutive records = one contiguous piece
              const int sb = ug % SBU;
              if (ug >= SBU) waitf(&b_empty[sb], (uint32_t)(ug / SBU - 1) & 1u, 4u, (uint32_t)(j & 255));
              tc::mbar_expect_tx(&b_full[sb], UNIT16);
              bulk_g2s(stage + (size_t)sb * UNIT16, q.xbase + (size_t)(j * (8 / G16) + k) * UNIT16, UNIT16, &b_full[sb]);
              stamp(0, ug);
            }
          }
        }
      }
    } else
    if (lane == 0 && !(TRACE && a.debug_no_copy)) {
      auto load_w = [&](int j) {                           // weight batch j -> slot j % WB
        const int s = j % WB;
        tc::mbar_expect_tx(&w_full[s], WBATCH_W + WBATCH_S);
        bulk_g2s(slabW + (size_t)s * WBATCH_W, a.Wt + (wbase + (size_t)j * 8) * 2048, WBATCH_W, &w_full[s]);
        bulk_g2s(slabS + (size_t)s * WBATCH_S, a.St + (wbase + (size_t)j * 8) * 128, WBATCH_S, &w_full[s]);
      };
      auto load_b = [&](int b) {                           // activation k-block b -> stage b % SB
        const int s = b % SB;
        tc::mbar_expect_tx(&b_full[s], STAGE_BYTES);
        bulk_g2s(stage + (size_t)s * STAGE_BYTES, xbase + (size_t)b * STAGE_BYTES, STAGE_BYTES, &b_full[s]);
        stamp(0, b);
      };
      for (int j = 0; j < WB && j < NBATCH; ++j) load_w(j);   // weights do not depend on the previous kernel
      pdl_wait();                                             // activations do
      for (int b = 0; b < SB && b < KB; ++b) load_b(b);
      for (int ob = 0; ob < KB && ok; ++ob) {                 // refill each ring slot as soon as its k-block is done with
        if (ob + SB < KB) {                                   // (after an expired wait: no further copies into a ring in use)
          waitb(&b_empty[ob % SB], (uint32_t)(ob / SB) & 1u, ok);
          load_b(ob + SB);
        }
        if ((ob & 7) == 7) {
          const int oj = ob >> 3;
          if (oj + WB < NBATCH) {
            waitb(&w_empty[oj % WB], (uint32_t)(oj / WB) & 1u, ok);
            load_w(oj + WB);
          }
        }
      }
    }
  } else if (warp == W_MMA) {
    // ===================== MMA issuer (one thread) =====================
    if constexpr (F16) {
      if (lane == 0) {
        constexpr uint32_t IDESC16 = tc::idesc_f16(128, NTOK);
        const uint32_t stage0 = tc::smem_u32(stage);
        int ug = 0, it = 0;
        for (int tile = blockIdx.x; tile < a.ntiles; tile += gridDim.x, ++it) {
          const Tile16 q = tile16(tile);
          if (it > 0) waitf(&d_empty[0], (uint32_t)(it - 1) & 1u, 5u, (uint32_t)it);
          for (int u = 0; u < q.NU; ++u, ++ug) {
            const int s = ug % SBU, as = ug % NAU;
            waitf(&a_full[as], (uint32_t)(ug / NAU) & 1u, 6u, (uint32_t)(it << 8) | (uint32_t)(u & 255));
            waitf(&b_full[s], (uint32_t)(ug / SBU) & 1u, 7u, (uint32_t)(it << 8) | (uint32_t)(u & 255));
            tc::fence_after_sync();
#pragma unroll
            for (int g = 0; g < G16; ++g) {
#pragma unroll
              for (int j = 0; j < 2; ++j) {                // 16 of the k-block's 32 values per instruction
                // per 8-token group: four 8-value chunks of 128 bytes; chunks 2 j, 2 j + 1 belong to this instruction
                const uint64_t bdesc = tc::smem_desc_kmajor(stage0 + (uint32_t)s * UNIT16 + (uint32_t)g * REC16 + (uint32_t)j * 256, 128, 512);
#pragma unroll
                for (int hf = 0; hf < MH16; ++hf)          // the same activations against both row halves
                  if (hf == 0 || q.have1)
                    tc::mma_f16_ts(tmem_d + (uint32_t)hf * 128, tmem_a + (uint32_t)((as * G16 + g) * MH16 + hf) * 16 + (uint32_t)j * 8, bdesc,
                                   IDESC16, (u | g | j) ? 1u : 0u);
              }
            }
            tc::mma_commit(&a_empty[as]);
            tc::mma_commit(&b_empty[s]);
            stamp(2, ug);
          }
          tc::mma_commit(&d_full[0]);
        }
      }
    } else
    if (lane == 0) {
      const uint32_t stage0 = tc::smem_u32(stage);
      for (int b = 0; b < KB; ++b) {
        const int slot = b % NSLOT, s = b % SB, as = b % NA;
        stamp(6, b);
        waitb(&a_full[as], (uint32_t)(b / NA) & 1u, ok);
        stamp(7, b);
        waitb(&b_full[s], (uint32_t)(b / SB) & 1u, ok);
        stamp(8, b);
        waitb(&d_empty[slot], ((uint32_t)(b / NSLOT) & 1u) ^ 1u, ok);   // the slot has been read out (k-block b - NSLOT)
        stamp(9, b);
        tc::fence_after_sync();
        const uint64_t bdesc = tc::smem_desc_kmajor(stage0 + (uint32_t)s * STAGE_BYTES, 128, 256);
        tc::mma_i8_ts(tmem_d + (uint32_t)slot * 128, tmem_a + (uint32_t)as * 8, bdesc, IDESC, 0u);
        tc::mma_commit(&d_full[slot]);
        tc::mma_commit(&a_empty[as]);
        tc::mma_commit(&b_empty[s]);
        stamp(2, b);
      }
    }
  } else if (warp >= NRW) {
    // ===================== expanders: thread = weight row, nibbles -> signed bytes -> A operand in tensor memory ==========
    if constexpr (F16) {
      for (int tile = blockIdx.x; tile < a.ntiles; tile += gridDim.x) expand16(tile16(tile));
    } else {
    const int r = (warp - NRW) * 32 + lane;                // row of the tile = TMEM lane
    const uint32_t lane_off = (uint32_t)(32 * (warp & 3)) << 16;
    for (int b = 0; b < KB; ++b) {
      const int ws = (b >> 3) % WB, as = b % NA;
      if ((b & 7) == 0) waitb(&w_full[ws], (uint32_t)((b >> 3) / WB) & 1u, ok);
      const uint4 w = *reinterpret_cast<const uint4*>(slabW + (size_t)ws * WBATCH_W + (size_t)(b & 7) * 2048 + r * 16);
      uint32_t ex[8];
      tc::expand_nibbles(w.x, ex[0], ex[1]);
      tc::expand_nibbles(w.y, ex[2], ex[3]);
      tc::expand_nibbles(w.z, ex[4], ex[5]);
      tc::expand_nibbles(w.w, ex[6], ex[7]);
      waitb(&a_empty[as], ((uint32_t)(b / NA) & 1u) ^ 1u, ok);   // the MMA of k-block b - NA has read this operand
      tc::fence_after_sync();
      tc::tmem_st8(tmem_a + lane_off + (uint32_t)as * 8, ex);
      tc::tmem_wait_st();                                  // warp-wide
      tc::fence_before_sync();
      if (lane == 0) {
        tc::mbar_arrive(&a_full[as]);
        if ((b & 7) == 7) tc::mbar_arrive(&w_empty[ws]);   // this warp is done with the batch's nibbles
        if (warp == NRW) stamp(1, b);
      }
    }
    }
  } else {
    // ===================== rescale warps: TMEM lane quarter lq (rows), column quarter cq (32 activation rows) ==========
    const int lq = warp & 3, cq = warp >> 2;
    const int r = lq * 32 + lane;
    const uint32_t lane_off = (uint32_t)(32 * lq) << 16;
    const uint32_t dbase = tmem_d + lane_off + (uint32_t)cq * 32;
    uint64_t acc2[16];                                     // 32 fp32 accumulators as packed pairs
#pragma unroll
    for (int n = 0; n < 16; ++n) acc2[n] = 0ull;
    const uint64_t neg_bias = tc::pack2(-tc::I2F_BIAS, -tc::I2F_BIAS);
    // 16 columns of one k-block: exact int -> float through the magic constant (two integer adds per pair), then three
    // two-wide fp32 ops per pair: subtract the bias, scale product dw * dx, fused multiply-add
    auto fold16 = [&](const uint32_t* d, const ulonglong2* sx, uint64_t dw2, int half) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const ulonglong2 x4 = sx[4 * half + q];            // four block scales = two packed pairs
        // the first pair through one LOP3 each (logic pipe), the second through an integer add (which the compiler puts on
        // the fp32 pipe as IMAD): splitting them evens out the two pipes, measured 1.5 % over adds only (all-LOP3: 0.7 %)
        const uint64_t f0 = tc::add2(tc::pack2u(magic_lop(d[4 * q + 0]), magic_lop(d[4 * q + 1])), neg_bias);
        const uint64_t f1 = tc::add2(tc::pack2u(d[4 * q + 2] + tc::I2F_MAGIC, d[4 * q + 3] + tc::I2F_MAGIC), neg_bias);
        acc2[8 * half + 2 * q + 0] = tc::fma2(tc::mul2(dw2, x4.x), f0, acc2[8 * half + 2 * q + 0]);
        acc2[8 * half + 2 * q + 1] = tc::fma2(tc::mul2(dw2, x4.y), f1, acc2[8 * half + 2 * q + 1]);
      }
    };
    // fp16 mode: one pass of this loop per tile of the CTA; int8 mode: exactly one pass
    for (int it16 = 0, tile = blockIdx.x; F16 ? tile < a.ntiles : it16 < 1; ++it16, tile += gridDim.x) {
    int e_row = row_tile, e_tok = tok_tile, e_z = blockIdx.z;        // what the epilogue below works on
    [[maybe_unused]] bool e_have1 = false;
    if constexpr (F16) {
      // fp16 mode: these warps expand too; then the accumulators (complete sums over K) are read out once
      const Tile16 q = tile16(tile);
      e_row = q.row_tile;
      e_tok = q.tok_tile;
      e_z = q.z;
      e_have1 = q.have1;
      expand16(q);
      waitf(&d_full[0], (uint32_t)it16 & 1u, 8u, (uint32_t)(warp << 8) | (uint32_t)it16);
      tc::fence_after_sync();
    } else {
    // Rolling schedule: the read-back of the next 16 columns is always in flight while the previous 16 are folded, so a
    // warp does not sit idle on tensor-memory latency.  (Handing the slot back before folding anything was measured:
    // slower, the exposed read latency costs more than the earlier release gains.)
    uint32_t dA[16], dB[16];
    if (KB > 0) {
      waitb(&w_full[0], 0u, ok);
      waitb(&d_full[0], 0u, ok);
      tc::fence_after_sync();
      tc::tmem_ld16(dbase, dA);
      tc::tmem_wait_ld();
    }
    int slot = 0, s = 0;                                   // b % NSLOT, b % SB, kept incrementally
    for (int b = 0; b < KB; ++b) {
      const int ws = (b >> 3) & (WB - 1);
      tc::tmem_ld16(dbase + (uint32_t)slot * 128 + 16, dB);      // second half of k-block b
      const float dw = __half2float(reinterpret_cast<const __half*>(slabS + (size_t)ws * WBATCH_S)[(b & 7) * 128 + r]) * 0.0625f;
      const ulonglong2* sx = reinterpret_cast<const ulonglong2*>(stage + (size_t)s * STAGE_BYTES + 4096) + cq * 8;
      const uint64_t dw2 = tc::pack2(dw, dw);
      fold16(dA, sx, dw2, 0);
      tc::tmem_wait_ld();                                  // warp-wide: the slot is now entirely in registers
      tc::fence_before_sync();
      if (lane == 0) tc::mbar_arrive(&d_empty[slot]);      // one arrival per warp: the MMA of k-block b + NSLOT may overwrite it
      if (warp == 0 && lane == 0) stamp(4, b);
      const int nb = b + 1, nslot = slot + 1 == NSLOT ? 0 : slot + 1;
      const uint32_t npar = (uint32_t)(nb / NSLOT) & 1u;
      bool requested = false;
      if (nb < KB) {
        if ((nb & 7) == 0) waitb(&w_full[(nb >> 3) & (WB - 1)], (uint32_t)((nb >> 3) / WB) & 1u, ok);   // next batch's weight scales
        // A look only (non-blocking), by one lane so that the warp-wide read-back below is entered uniformly.  Measured
        // alternatives: all lanes looking + a vote (7 % slower); looking before the first fold (the accumulator is usually
        // not there yet, and the blocking path costs more); a blocking try (suspends the warp for hundreds of clocks).
        if (__shfl_sync(0xffffffffu, lane == 0 && tc::mbar_test(&d_full[nslot], npar) ? 1 : 0, 0)) {
          tc::fence_after_sync();
          tc::tmem_ld16(dbase + (uint32_t)nslot * 128, dA);
          requested = true;
          if (warp == 0 && lane == 0) stamp(3, nb);
        }
      }
      fold16(dB, sx, dw2, 1);
      __syncwarp();
      if (warp == 0 && lane == 0) stamp(5, b);
      if (lane == 0) {
        tc::mbar_arrive(&b_empty[s]);                      // this warp is done with the stage's block scales
        if ((b & 7) == 7) tc::mbar_arrive(&w_empty[ws]);   // ... and with the weight batch's scales
      }
      if (nb < KB && !requested) {
        waitb(&d_full[nslot], npar, ok);
        tc::fence_after_sync();
        tc::tmem_ld16(dbase + (uint32_t)nslot * 128, dA);
        if (warp == 0 && lane == 0) stamp(3, nb);
      }
      tc::tmem_wait_ld();
      slot = nslot;
      s = s + 1 == SB ? 0 : s + 1;
    }

    }
    // ---- epilogue: thread (row r, 32 activation rows); fp16 mode: once per row half, from that half's accumulator
    if (t == 0) stamp(10, 2);                              // main loop left
    pdl_wait();                                            // Y / AUX may be written by the previous kernel
    if (t == 0) stamp(10, 5);                              // previous grid seen complete
    for (int hh = 0; hh < (F16 ? MH16 : 1); ++hh) {
    const int rt = e_row + hh;
    if constexpr (F16) {
      if (hh && !e_have1) break;
      uint32_t dA[16], dB[16];
      tc::tmem_ld16(dbase + (uint32_t)hh * 128, dA);
      tc::tmem_ld16(dbase + (uint32_t)hh * 128 + 16, dB);
      tc::tmem_wait_ld();
      if (hh == (e_have1 ? 1 : 0)) {                       // both accumulators are in registers: the next tile's MMAs may start
        tc::fence_before_sync();
        if (lane == 0) tc::mbar_arrive(&d_empty[0]);
      }
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        acc2[n] = tc::pack2u(dA[2 * n], dA[2 * n + 1]);
        acc2[8 + n] = tc::pack2u(dB[2 * n], dB[2 * n + 1]);
      }
    }
    const int row = rt * 128 + r;
    const int tok0 = e_tok * NTOK + cq * 32;
    const float bias = ((a.epi == Q4B_EPI_BIASF || a.epi == Q4B_EPI_BIASF_ROPE_KV) && row < a.N) ? reinterpret_cast<const float*>(a.AUX)[row] : 0.f;
    if (a.epi == Q4B_EPI_BIASF_ROPE_KV) {
      // The `biasf_kv` epilogue (lab/qwen_batched.py:1316-1362) extended to q: bias, round to fp16, rotate the q and k heads
      // (NeoX pairs d, d + 64: the other half sits 64 TMEM lanes away, so the rounded tile goes through shared memory)
      // from the ROUNDED values, round again; rotated k and raw v also go into the cache rows pos0 + token.  A row tile is
      // exactly one head.  The weight slab is dead here: the last MMA has retired, so the expanders are done with it.
      __half* ybuf = reinterpret_cast<__half*>(slabW);     // [token 128][row 128]
#pragma unroll
      for (int n = 0; n < 32; ++n) {
        const float v = (n & 1) ? tc::hi2(acc2[n >> 1]) : tc::lo2(acc2[n >> 1]);
        ybuf[(cq * 32 + n) * 128 + r] = __float2half_rn(v + bias);
      }
      asm volatile("bar.sync 1, %0;" ::"n"(NRW * 32) : "memory");
      if (t == 0) stamp(10, 6);                            // rounded tile in shared memory
      rope_kv_phase(a, ybuf, rt, e_tok * NTOK, t);
    } else if (a.epi == Q4B_EPI_SWIGLU_Q8) {
      // SwiGLU + re-quantise for `down` (lab/qwen_batched.py:1363-1396): the product rounded to fp16, then the Q8_1
      // quantiser of quant_q8_1.cu on it, written straight into the tiled operand format of the next GEMM.  This row
      // tile makes 64 product columns = k-blocks 2 row_tile + {0, 1} of the product row.  The rounded products go
      // through shared memory (the dead weight slab) so that the quantiser runs in its own thread mapping, eight lanes
      // per 32-value block, instead of 32 warp-wide maxima per thread.
      __half* abuf = reinterpret_cast<__half*>(slabW);     // [token 128][product column 64]
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        int n;
        const float prod = swiglu_pair<F16>(acc2[j], r, j, n);
        abuf[(cq * 32 + n) * 64 + (r >> 1)] = __float2half_rn(row < a.N ? prod : 0.f);
      }
      asm volatile("bar.sync 1, %0;" ::"n"(NRW * 32) : "memory");
      if (t == 0) stamp(10, 6);                            // rounded tile in shared memory
      swiglu_q8_phase(a, abuf, rt, e_tok, t);
    } else if (F16 && a.epi == Q4B_EPI_SWIGLU_F16T) {       // compiled into the fp16 instance only
      // fp16 mode: the rounded products in the operand order of the next fp16 GEMM (see f16_tiled_kernel).  This row tile
      // makes product columns 64 rt .. 64 rt + 63 = k-blocks 2 rt, 2 rt + 1 of the product row.  Through shared memory (the
      // dead weight slab; rows padded to 144 bytes so that eight tokens' 16-byte reads fall into distinct banks), then
      // 16-byte stores, eight tokens = 128 contiguous bytes.
      constexpr int AP = 72;                               // halves per staged token row
      __half* abuf = reinterpret_cast<__half*>(stage + (size_t)SBU * UNIT16);   // its own buffer: the weight ring is live
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        int n;
        const float prod = swiglu_pair<F16>(acc2[j], r, j, n);
        abuf[(cq * 32 + n) * AP + (r >> 1)] = __float2half_rn(row < a.N ? prod : 0.f);
      }
      asm volatile("bar.sync 1, %0;" ::"n"(NRW * 32) : "memory");
      const int KB2 = a.N >> 6;
#pragma unroll
      for (int itx = 0; itx < 2; ++itx) {
        const int item = t + itx * (NRW * 32);
        const int r8 = item & 7, wd = (item >> 3) & 7, gq = item >> 6, tk = gq * 8 + r8;
        if (e_tok * NTOK + tk < a.P) {
          const uint4 v = *reinterpret_cast<const uint4*>(abuf + tk * AP + wd * 8);
          uint4 o;                                           // halves (0..7) -> (0,4,1,5,2,6,3,7)
          o.x = __byte_perm(v.x, v.z, 0x5410);
          o.y = __byte_perm(v.x, v.z, 0x7632);
          o.z = __byte_perm(v.y, v.w, 0x5410);
          o.w = __byte_perm(v.y, v.w, 0x7632);
          uint8_t* rec = reinterpret_cast<uint8_t*>(a.Y) + ((size_t)e_tok * KB2 + (size_t)(2 * rt + (wd >> 2))) * REC16;
          *reinterpret_cast<uint4*>(rec + gq * 512 + (wd & 3) * 128 + r8 * 16) = o;
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(NRW * 32) : "memory");   // the other row half reuses the buffer
    } else if (a.epi == Q4B_EPI_SWIGLU) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        int n;
        const float prod = swiglu_pair<F16>(acc2[j], r, j, n);
        const int p = tok0 + n;
        if (p < a.P && row < a.N) reinterpret_cast<__half*>(a.Y)[(size_t)p * a.ldy + (row >> 1)] = __float2half_rn(prod);
      }
    } else if ((a.epi == Q4B_EPI_STORE || a.epi == Q4B_EPI_BIASF) && a.pair16) {
      // fp16 outputs as 4-byte stores: the even lane of a row pair writes (row, row + 1) of token 2 j, the odd lane of
      // token 2 j + 1 (one exchange per token pair); a warp store then covers two runs of 64 bytes
      const bool odd = r & 1;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float v0 = tc::lo2(acc2[j]) + bias, v1 = tc::hi2(acc2[j]) + bias;
        const float got = __shfl_xor_sync(0xffffffffu, odd ? v0 : v1, 1);
        const int p = tok0 + 2 * j + (odd ? 1 : 0);
        if (p < a.P && row < a.N)
          *reinterpret_cast<__half2*>(reinterpret_cast<__half*>(a.Y) + (size_t)p * a.ldy + (row & ~1)) =
              odd ? __floats2half2_rn(got, v1) : __floats2half2_rn(v0, got);
      }
    } else if (a.epi == Q4B_EPI_RESID && e_z == 0) {
      // h += sum: all 32 loads first (issued back to back), then the adds and stores; one load-add-store per token in turn
      // would pay the global-memory latency 32 times over, the loads being ordered behind the stores to the same array
      float* y = reinterpret_cast<float*>(a.Y) + (size_t)tok0 * a.ldy + row;
      float old[32];
#pragma unroll
      for (int n = 0; n < 32; ++n) old[n] = (tok0 + n < a.P && row < a.N) ? y[(size_t)n * a.ldy] : 0.f;
#pragma unroll
      for (int n = 0; n < 32; ++n) {
        const float v = (n & 1) ? tc::hi2(acc2[n >> 1]) : tc::lo2(acc2[n >> 1]);
        if (tok0 + n < a.P && row < a.N) y[(size_t)n * a.ldy] = old[n] + v;
      }
    } else {
#pragma unroll
    for (int n = 0; n < 32; ++n) {                         // fully unrolled: the accumulators must stay in registers
      const float v = (n & 1) ? tc::hi2(acc2[n >> 1]) : tc::lo2(acc2[n >> 1]);
      const int p = tok0 + n;
      if (p < a.P && row < a.N) {
        const size_t base = (size_t)p * a.ldy;
        switch (a.epi) {
          case Q4B_EPI_STORE: reinterpret_cast<__half*>(a.Y)[base + row] = __float2half_rn(v); break;
          case Q4B_EPI_BIASF: reinterpret_cast<__half*>(a.Y)[base + row] = __float2half_rn(v + bias); break;
          case Q4B_EPI_RESID: a.Y2[(size_t)(e_z - 1) * a.P * a.ldy + base + row] = v; break;   // part z > 0 of a split launch
          case Q4B_EPI_LOGITS: reinterpret_cast<float*>(a.Y)[base + row] = v; break;
          default: break;
        }
      }
    }
    }
    }
    }
  }
  if (t == 0) stamp(10, 3);                                // epilogue written
  if (!ok) atomicCAS(a.status, 0u, 1u);
  tc::fence_before_sync();
  // any thread's expired wait: the MMA issuer sees its MMAs retire before tensor memory is freed (it may itself have met
  // no expired wait: the others' late arrivals satisfy its barriers)
  tc::drain_mmas_on_failure(ok, warp == W_MMA && lane == 0, &drain);
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, 512);
  if (t == 0) stamp(10, 4);                                // tensor memory released
}

long long* g_prefill_trace = nullptr;
bool g_prefill_no_copy = false;

}  // namespace

void mmq_prefill_trace(long long* buf) { g_prefill_trace = buf; }
void mmq_prefill_debug_no_copy(bool on) { g_prefill_no_copy = on; }

size_t f16_tiled_bytes(int P, int K) { return (size_t)((P + NTOK - 1) / NTOK) * (size_t)(K / 32) * REC16; }

// fp16 activations [P, K] -> the fp16 mode's B operand: per (128-token tile, k-block) 8192 bytes in the tensor core's
// K-major core-matrix order ([8-token group 16][8-value chunk 4][token 8][16 bytes]); within a chunk the values sit as
// (0,4,1,5,2,6,3,7), the order in which the expanders' nibble masks deliver a word's weights.  A warp writes 512
// contiguous bytes and reads 64 contiguous bytes of 8 tokens.
__global__ void __launch_bounds__(256) f16_tiled_kernel(const __half* __restrict__ x, uint8_t* __restrict__ xt, int P, int K) {
  pdl_wait();
  pdl_launch_dependents();
  const int KB = K >> 5;
  const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
  const int r = (int)(i & 7), c = (int)(i >> 3) & 3;
  const size_t grp = i >> 5;
  const int g = (int)(grp & 15);
  const size_t rec = grp >> 4;                              // (token tile, k-block)
  const int kb = (int)(rec % KB), tt = (int)(rec / KB);
  const int p = tt * NTOK + g * 8 + r;
  if (p >= P) return;                                       // rows past P stay zero (the buffer is zero-filled once)
  const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)p * K + kb * 32 + c * 8);
  uint4 o;                                                  // halves (0..7) -> (0,4,1,5,2,6,3,7)
  o.x = __byte_perm(v.x, v.z, 0x5410);
  o.y = __byte_perm(v.x, v.z, 0x7632);
  o.z = __byte_perm(v.y, v.w, 0x5410);
  o.w = __byte_perm(v.y, v.w, 0x7632);
  *reinterpret_cast<uint4*>(xt + rec * REC16 + (size_t)g * 512 + c * 128 + r * 16) = o;
}

int f16_tiled(const void* x, void* xt, int P, int K, cudaStream_t st) {
  if (P <= 0 || K <= 0 || (K % 32)) return fail(Q4B_E_SHAPE, "f16_tiled: P > 0 and K a positive multiple of 32 required");
  if (!x || !xt || !aligned16(x) || !aligned16(xt)) return fail(Q4B_E_ALIGN, "f16_tiled: null or misaligned pointer");
  const size_t threads = (size_t)((P + NTOK - 1) / NTOK) * (size_t)(K / 32) * 16 * 32;
  return check_launch(launch_pdl(f16_tiled_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, st,
                                 reinterpret_cast<const __half*>(x), reinterpret_cast<uint8_t*>(xt), P, K),
                      "f16_tiled");
}

size_t q8_tiled_bytes(int P, int K) { return (size_t)((P + NTOK - 1) / NTOK) * (size_t)(K / 32) * STAGE_BYTES; }

// Y2 != nullptr (RESID only): the launch is split along K over gridDim.z = parts; Y += part 0, Y2[z - 1] = part z.
int mmq_prefill(const void* Wt, const void* St, const void* Xt, void* Y, const void* AUX, int N, int K, int P, int epilogue,
                int ldy, uint32_t* status, cudaStream_t st, const float* cosT, const float* sinT, void* kc, void* vc, int NH,
                int NKV, int max_len, int pos0, float* Y2, int parts, int f16) {
  if (f16 && epilogue == Q4B_EPI_SWIGLU_Q8) return fail(Q4B_E_ARG, "mmq_prefill: no swiglu_q8 epilogue in fp16 mode");
  if (epilogue == Q4B_EPI_SWIGLU_F16T && (!f16 || (N % 128) || !aligned16(Y)))
    return fail(Q4B_E_ARG, "mmq_prefill: swiglu_f16t is an fp16-mode epilogue, needs N a multiple of 128 and a tiled fp16 output buffer");
  if (N <= 0 || P <= 0 || K <= 0 || (K % 256)) return fail(Q4B_E_SHAPE, "mmq_prefill: N, P > 0 and K a positive multiple of 256 required");
  if (epilogue < Q4B_EPI_STORE || epilogue > Q4B_EPI_SWIGLU_F16T) return fail(Q4B_E_ARG, "mmq_prefill: unknown epilogue");
  if (epilogue == Q4B_EPI_SWIGLU && (N % 2)) return fail(Q4B_E_SHAPE, "mmq_prefill: swiglu needs an even row count");
  if (epilogue == Q4B_EPI_SWIGLU_Q8 && ((N % 128) || !aligned16(Y)))
    return fail(Q4B_E_SHAPE, "mmq_prefill: swiglu_q8 needs a row count that is a multiple of 128 and a tiled Q8_1 output buffer");
  if (epilogue == Q4B_EPI_BIASF_ROPE_KV) {
    if (!cosT || !sinT || !kc || !vc || !AUX) return fail(Q4B_E_ALIGN, "mmq_prefill: the rope/kv epilogue needs bias, tables and the cache");
    if (reinterpret_cast<uintptr_t>(cosT) % 8 || reinterpret_cast<uintptr_t>(sinT) % 8 || reinterpret_cast<uintptr_t>(kc) % 4 ||
        reinterpret_cast<uintptr_t>(vc) % 4 || reinterpret_cast<uintptr_t>(Y) % 4 || (ldy % 2))
      return fail(Q4B_E_ALIGN, "mmq_prefill: the rope/kv epilogue needs 8-byte aligned tables, 4-byte aligned outputs and an even ldy");
    if (NH <= 0 || NKV <= 0 || N != (NH + 2 * NKV) * 128 || max_len <= 0 || pos0 < 0 || pos0 + P > max_len)
      return fail(Q4B_E_SHAPE, "mmq_prefill: the rope/kv epilogue needs head_dim 128, N = (NH + 2 NKV) 128 and pos0 + P <= max_len");
  }
  if (!Wt || !St || !Xt || !Y || !status || !aligned16(Wt) || !aligned16(St) || !aligned16(Xt))
    return fail(Q4B_E_ALIGN, "mmq_prefill: null or misaligned pointer");
  if (epilogue == Q4B_EPI_BIASF && !AUX) return fail(Q4B_E_ALIGN, "mmq_prefill: biasf needs AUX");
  const bool traced = g_prefill_trace || g_prefill_no_copy;
  auto kern = f16 ? (traced ? mmq_prefill_kernel<true, true> : mmq_prefill_kernel<false, true>)
                  : (traced ? mmq_prefill_kernel<true, false> : mmq_prefill_kernel<false, false>);
  const size_t smem_bytes = f16 ? PF_SMEM16 : PF_SMEM;
  if (cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes); e != cudaSuccess) {
    set_cuda_error(e, "mmq_prefill: cudaFuncSetAttribute");
    return Q4B_E_CUDA;
  }
  PrefillArgs a;
  a.Wt = reinterpret_cast<const uint8_t*>(Wt);
  a.St = reinterpret_cast<const __half*>(St);
  a.Xt = reinterpret_cast<const uint8_t*>(Xt);
  a.Y = Y;
  a.AUX = AUX;
  a.status = status;
  a.N = N;
  a.K = K;
  a.P = P;
  a.epi = epilogue;
  a.ldy = ldy;
  a.pair16 = (N % 2 == 0 && ldy % 2 == 0 && reinterpret_cast<uintptr_t>(Y) % 4 == 0) ? 1 : 0;
  a.cosT = cosT;
  a.sinT = sinT;
  a.kc = reinterpret_cast<__half*>(kc);
  a.vc = reinterpret_cast<__half*>(vc);
  a.NH = NH;
  a.NKV = NKV;
  a.max_len = max_len;
  a.pos0 = pos0;
  a.trace = g_prefill_trace;
  a.debug_no_copy = g_prefill_no_copy ? 1 : 0;
  a.Y2 = Y2;
  a.kb_bound[0] = 0;
  a.kb_bound[1] = a.kb_bound[2] = a.kb_bound[3] = a.kb_bound[4] = K / 32;
  dim3 grid(f16 ? (N + 255) / 256 : (N + 127) / 128, (P + NTOK - 1) / NTOK);
  if (Y2) {
    if (epilogue != Q4B_EPI_RESID || parts < 2 || parts > 4 || K / 256 < parts || !aligned16(Y2))
      return fail(Q4B_E_SHAPE, "mmq_prefill: a K-split launch needs the resid epilogue, 2 .. 4 parts and K >= 256 per part");
    const int batches = K / 256;                         // whole batches of 8 k-blocks, spread as evenly as they go
    for (int z = 1; z < parts; ++z) a.kb_bound[z] = (int)(((long long)batches * z + parts - 1) / parts) * 8;
    grid.z = parts;
  }
  a.tx = a.ty = a.ntiles = 0;
  if (f16) {                                             // persistent CTAs over (row pair, token tile, K part)
    a.tx = (int)grid.x;
    a.ty = (int)grid.y;
    a.ntiles = a.tx * a.ty * (int)grid.z;
    grid = dim3((unsigned)std::min(a.ntiles, sm_count()));
  }
  return check_launch(launch_pdl(kern, grid, dim3(PF_THREADS), smem_bytes, st, a), "mmq_prefill");
}

}  // namespace q4b
