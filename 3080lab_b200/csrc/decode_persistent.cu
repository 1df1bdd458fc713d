// All transformer layers of one batch-1 decode token as ONE persistent cooperative kernel (one CTA per SM).
//
// The per-op kernels of the fused step (mmq_stream.cu, attn_decode.cu) are each a few microseconds of dependent
// latency: launch hand-over, operand staging, one MMA batch, split-K exchange.  With 5 of them per layer the step is
// bound by that chain, not by HBM.  Here the chain is shortened and the weight stream is taken off it entirely:
//
//   * a producer warp walks the STATIC schedule of this CTA's (row tile, K slice) units through every layer and keeps
//     a ring of shared-memory stages full with 1-D bulk (TMA) copies of tile-packed Q4_0 weights.  It never waits for
//     activations, so weights for the next ops arrive while the CTA sits in a grid barrier.
//   * per batch of 8 k-blocks: one warpgroup expands nibbles to signed bytes straight into tensor memory
//     (tcgen05.st), one thread issues tcgen05.mma.kind::i8 (M = 128 rows, N = 8 digit columns, K = 32 = one Q4_0
//     block), another warpgroup reads the int32 accumulators back (tcgen05.ld) and folds them with the block scales.
//     Four TMEM slots keep four batches in flight; all hand-overs are mbarriers with bounded waits.
//   * activations are exact: each 32-block of the fp16-valued input vector becomes a block-fixed-point integer split
//     into three signed base-256 digits (one MMA column each), the same arithmetic as mmq_stream.cu's exact mode and
//     therefore the reference's dequantise-and-dot (lab/qwen_kernels.py:14-113) with no rounding inside a block.
//   * ops are separated by grid barriers (one release-add and an acquire-poll on a global counter, bounded).  Split-K
//     partial sums go to global scratch and are added, in slice order, by the consumer while it stages its operand, so
//     the residual add and the RMSNorm (lab/qwen_kernels.py:683-705) cost no extra pass and results are bit-repeatable.
//   * attention (ATTN4 arithmetic, lab/qwen_kernels.py:517-605: RoPE, fp16 K/V append, soft-max, P.V) runs as (KV head,
//     position chunk) units; its partials (max, sum, unnormalised output) are merged by the o_proj units on read.
//
// Measured on B200 (Qwen2.5-1.5B shape, context 512): 1.63 ms per token against 1.00 ms for the chain of per-op
// kernels, i.e. SLOWER; the library therefore keeps it opt-in (Q4B_STEP_PERSISTENT).  The timeline stamps show why:
// a grid barrier costs 1.9 us (0.5 us fence + 1.3-1.4 us release/acquire round trip through L2) where a
// programmatic-dependent-launch hand-over costs about 1.3 us; every consumer CTA re-reads all split-K partials
// (148 x 80 KB through L2 = 3 us per reduction, where a cluster reduces through distributed shared memory in
// 0.65 us); and one batch through expand -> MMA -> fold is a 1 us dependent chain that the four TMEM slots do not
// overlap.  The reference reports the same outcome for its own persistent decode kernel on sm_86 (17 % slower than
// its 200-kernel graph, docs/reports/llm-inference.md:140-144).
//
// Layer op order and rounding points are those of the fused step (scripts/qwen_fused.py:113-145): fp16 qkv (+bias),
// fp16 attention output, fp16 SwiGLU product, fp32 residual stream.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "q4b_internal.h"
#include "tc05.cuh"

namespace q4b {

namespace {

constexpr int CT = 256;                    // compute threads: warps 0-3 expand, warps 4-7 fold
constexpr int PT = 320;                    // + warp 8 (MMA issue) + warp 9 (weight producer)
constexpr int WARP_MMA = 8, WARP_LOAD = 9;
constexpr int G = 8;                       // k-blocks per batch = per ring stage
constexpr int STAGE_NIB = G * 2048, STAGE_BYTES = G * (2048 + 256);
constexpr int NSLOT = 4;                   // TMEM slots (A: 64 columns each at 0.., D: 64 columns each at 256..)
constexpr int NL = 3;                      // base-256 digits of an fp16-valued block
constexpr int MAX_STAGES = 12;
constexpr int MAX_GRP = 8;                 // query heads per KV head
constexpr int MAX_KSPLIT = 16;             // K slices of one linear
constexpr int MAX_WHEADS = 8;              // heads one K slice of o_proj may touch
constexpr uint32_t IDESC = tc::idesc_i8(128, 8);
constexpr uint32_t GRID_WAIT_LIMIT = 1u << 20;   // acquire polls of a grid barrier (well under a second)
constexpr uint32_t PIPE_WAIT_LIMIT = 1u << 16;   // try_waits (each may sleep up to 20 us) of a pipeline mbarrier
constexpr size_t MAX_DYN_SMEM = 226 * 1024;

struct PLinear {
  const uint8_t* W;   // tile-packed nibbles
  const __half* S;    // tile-packed scales
  int N, KB, tiles, ksplit, rot;
};
struct PLayer {
  PLinear lin[4];     // qkv, o, gate_up, down
  const float* ln1;
  const float* ln2;
  const float* bias;
  __half* kc;
  __half* vc;
};
struct PArgs {
  const PLayer* layer;
  int layers, H, FFN, NH, NKV, HD, max_len;
  float eps, scale;
  const float* cosT;
  const float* sinT;
  const int64_t* pos;
  float* hA;          // residual stream: the embedding row on entry, the last layer's output on exit
  float* hB;
  float* part_qkv;    // [ksplit][rows] fp32 split-K partials
  float* part_o;
  float* part_down;
  float* att_part;    // [NH][nch_max][HD + 2]: unnormalised output, running maximum, running sum
  __half* xm;         // [FFN] SwiGLU product
  uint32_t* sync;     // [0] barrier arrivals, [1] CTAs that have left; both zero between launches
  uint32_t* status;
  unsigned long long* trace;
  int trace_stride;
  int nstage, bkb, nch_max;
};

__device__ __forceinline__ void named_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ void red_release_add(uint32_t* p) {
  asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   tc::smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(tc::smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ float round16(float v) { return __half2float(__float2half_rn(v)); }

struct Unit {
  int tile, ks, kb0, kb1;
};
// idx-th unit of CTA `cta` for one linear.  Units are (tile, K slice) pairs numbered tile-major; CTA c owns units
// c - rot, c - rot + ncta, ...  (more than one per CTA only when ksplit == 1).
__device__ __forceinline__ bool get_unit(const PLinear& g, int cta, int ncta, int idx, Unit& u) {
  int v = cta - g.rot;
  if (v < 0) v += ncta;
  v += idx * ncta;
  if (v >= g.tiles * g.ksplit) return false;
  u.tile = v / g.ksplit;
  u.ks = v - u.tile * g.ksplit;
  u.kb0 = (int)(((long long)g.KB * u.ks) / g.ksplit);
  u.kb1 = (int)(((long long)g.KB * (u.ks + 1)) / g.ksplit);
  return true;
}
// k-blocks of the activation vector a CTA stages for a linear: its K slice, or all of K when it owns whole rows.
__device__ __forceinline__ void staged_range(const PLinear& g, int cta, int ncta, int& kbA, int& nkbA) {
  Unit u;
  if (!get_unit(g, cta, ncta, 0, u)) {
    kbA = 0;
    nkbA = 0;
  } else if (g.ksplit == 1) {
    kbA = 0;
    nkbA = g.KB;
  } else {
    kbA = u.kb0;
    nkbA = u.kb1 - u.kb0;
  }
}

// Chunking of the positions 0..p over the CTAs: chunks of 32 R positions, R the smallest count with at most ncta units.
__device__ __forceinline__ void attn_geometry(int p, int NKV, int ncta, int& chunk, int& nch) {
  const int n32 = (p + 32) >> 5;                       // ceil((p + 1) / 32)
  const int R = (n32 * NKV + ncta - 1) / ncta;
  chunk = 32 * R;
  nch = (p + chunk) / chunk;                           // ceil((p + 1) / chunk)
}

template <int HD>
__global__ void __launch_bounds__(PT, 1) decode_persistent_kernel(const __grid_constant__ PArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t full[MAX_STAGES], empty[MAX_STAGES];
  __shared__ __align__(8) uint64_t aready[NSLOT], dfull[NSLOT], dempty[NSLOT], bar_drain;
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile uint32_t abort_s;                 // a bounded wait expired somewhere in this CTA: stop waiting
  __shared__ float red[8];

  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int cta = blockIdx.x, ncta = gridDim.x;
  const int NST = a.nstage;
  uint8_t* ring = smem;
  uint8_t* sB = ring + (size_t)NST * STAGE_BYTES;                 // [k-block][2 x 128 bytes]: UMMA B operand, 8 columns
  float* xs = reinterpret_cast<float*>(sB + (size_t)a.bkb * 256); // block scales of the staged activations
  float* work = xs + a.bkb;                                       // staging / attention scratch

  if (warp == 0) {
    tc::tmem_alloc(&tmem_base_s, 512);
    tc::tmem_relinquish();
  }
  if (t == 0) {
    abort_s = 0u;
    for (int s = 0; s < NST; ++s) {
      tc::mbar_init(&full[s], 1);
      tc::mbar_init(&empty[s], 8);          // one arrival per expand warp and per fold warp
    }
    for (int s = 0; s < NSLOT; ++s) {
      tc::mbar_init(&aready[s], 4);
      tc::mbar_init(&dfull[s], 1);
      tc::mbar_init(&dempty[s], 4);
    }
    tc::mbar_init(&bar_drain, 1);            // failure path: the MMA-issuing lane (tc::drain_mmas_on_failure)
    tc::mbar_fence_init();
  }
  for (int i = t; i < a.bkb * 64; i += PT) reinterpret_cast<uint32_t*>(sB)[i] = 0u;   // digit columns 3..7 stay zero
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_base_s;
  const uint32_t tmem_a = tmem, tmem_d = tmem + 256;
  bool ok = true;
  // Bounded mbarrier wait.  After the first expiry in the CTA every later wait returns at once, so a protocol error
  // costs one time-out, not one per batch.
  auto wait = [&](uint64_t* bar, uint32_t parity) {
    if (!ok) return;
    for (uint32_t i = 0; i < PIPE_WAIT_LIMIT; ++i) {
      if (tc::mbar_try_hint(bar, parity, 20000u)) return;
      if ((i & 15u) == 15u && abort_s) break;
    }
    ok = false;
    abort_s = 1u;
  };

  if (warp == WARP_LOAD) {
    // ================= weight producer: the whole schedule, limited only by ring space =================
    if (lane == 0) {
      uint32_t q = 0;
      for (int l = 0; l < a.layers; ++l) {
        for (int o = 0; o < 4; ++o) {
          const PLinear g = a.layer[l].lin[o];
          Unit u;
          for (int idx = 0; get_unit(g, cta, ncta, idx, u); ++idx) {
            for (int kb = u.kb0; kb < u.kb1; kb += G, ++q) {
              const int nb = min(G, u.kb1 - kb);
              const uint32_t s = q % (uint32_t)NST;
              if (q >= (uint32_t)NST) wait(&empty[s], ((q / (uint32_t)NST) - 1u) & 1u);
              uint8_t* st = ring + (size_t)s * STAGE_BYTES;
              const size_t kbg = (size_t)u.tile * g.KB + kb;
              tc::mbar_expect_tx(&full[s], (uint32_t)nb * (2048 + 256));
              bulk_g2s(st, g.W + kbg * 2048, (uint32_t)nb * 2048, &full[s]);
              bulk_g2s(st + STAGE_NIB, g.S + kbg * 128, (uint32_t)nb * 256, &full[s]);
            }
          }
        }
      }
    }
  } else if (warp == WARP_MMA) {
    // ================= MMA issue =================
    uint32_t q = 0;
    const uint32_t b0 = tc::smem_u32(sB);
    for (int l = 0; l < a.layers; ++l) {
      for (int o = 0; o < 4; ++o) {
        const PLinear g = a.layer[l].lin[o];
        int kbA, nkbA;
        staged_range(g, cta, ncta, kbA, nkbA);
        named_sync(2, CT + 32);                          // the activation operand of this op is staged
        Unit u;
        for (int idx = 0; get_unit(g, cta, ncta, idx, u); ++idx) {
          for (int kb = u.kb0; kb < u.kb1; kb += G, ++q) {
            const int nb = min(G, u.kb1 - kb);
            const uint32_t slot = q & (NSLOT - 1);
            wait(&aready[slot], (q / NSLOT) & 1u);
            tc::fence_after_sync();
            if (lane == 0) {
              for (int j = 0; j < nb; ++j) {
                const uint64_t bdesc = tc::smem_desc_kmajor(b0 + (uint32_t)(kb + j - kbA) * 256u, 128, 256);
                tc::mma_i8_ts(tmem_d + slot * 64 + (uint32_t)j * 8, tmem_a + slot * 64 + (uint32_t)j * 8, bdesc, IDESC, 0u);
              }
              tc::mma_commit(&dfull[slot]);
            }
            __syncwarp();
          }
        }
      }
    }
  } else {
    // ================= compute threads =================
    const bool expander = t < 128;
    const int r = t & 127;
    const uint32_t lane_off = (uint32_t)(32 * (warp & 3)) << 16;
    uint32_t q = 0, gb = 0;
    bool dead = false;                                   // thread 0: a grid barrier timed out, stop waiting on the others
    int tri = 0;
    const int trace_cap = a.trace_stride < 0 ? -a.trace_stride : a.trace_stride;   // negative: also stamp inside the stages
    const bool fine = a.trace_stride < 0;
    // timeline entry: label in the top byte, %globaltimer (ns) below
    auto stamp = [&](unsigned label) {
      if (a.trace && t == 0 && tri < trace_cap) {
        unsigned long long gt;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
        a.trace[(size_t)cta * trace_cap + tri++] = ((unsigned long long)label << 56) | (gt & 0x00FFFFFFFFFFFFFFull);
      }
    };
    auto grid_barrier = [&]() {
      if (fine) stamp(20);
      __threadfence();
      named_sync(1, CT);
      if (fine) stamp(21);
      ++gb;
      if (t == 0) {
        red_release_add(a.sync);
        const uint32_t target = gb * (uint32_t)ncta;
        if (!dead) {
          uint32_t i = 0;
          while (ld_acquire_u32(a.sync) < target) {
            ++i;
            // give up on the limit, on a local pipeline time-out, or when another CTA has reported one
            if (i > GRID_WAIT_LIMIT || ((i & 63u) == 63u && (abort_s || *reinterpret_cast<volatile uint32_t*>(a.status)))) {
              dead = true;
              atomicCAS(a.status, 0u, 2u);
              break;
            }
          }
        }
      }
      named_sync(1, CT);
      stamp(1);
    };
    // fp16-valued floats xf[0 .. 32 nkb) -> digit columns of the B operand and block scales
    auto digits = [&](const float* xf, int nkb) {
      const int sub = t & 7;
      for (int kb0 = 0; kb0 < nkb; kb0 += CT / 8) {       // whole warps stay in the loop: the shuffles need every lane
        const int kbl = kb0 + (t >> 3);
        const bool valid = kbl < nkb;
        const float4 v = valid ? *reinterpret_cast<const float4*>(xf + kbl * 32 + sub * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float x[4] = {v.x, v.y, v.z, v.w};
        float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
        for (int o = 4; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const bool live = amax > 0.f && amax < INFINITY;
        int e = (__float_as_int(amax) >> 23) & 0xFF;
        e = max(e, 8 * NL);
        const float inv = __int_as_float((127 + (8 * NL - 3) - (e - 127)) << 23);
        int X[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) X[j] = live ? __float2int_rn(x[j] * inv) : 0;
        // elements 4 sub + {0, 2} are adjacent operand bytes, and so are 4 sub + {1, 3} (order of tc::expand_nibbles)
        if (!valid) continue;
        const int pos02 = 8 * (sub >> 1) + 2 * (sub & 1), pos13 = pos02 + 4;
        uint8_t* kbp = sB + (size_t)kbl * 256;
#pragma unroll
        for (int j = 0; j < NL; ++j) {
          int dg[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            dg[u] = (int)(int8_t)(X[u] & 0xFF);
            X[u] = (X[u] - dg[u]) >> 8;
          }
          *reinterpret_cast<uint16_t*>(kbp + (pos02 >> 4) * 128 + j * 16 + (pos02 & 15)) =
              (uint16_t)((dg[0] & 0xFF) | ((dg[2] & 0xFF) << 8));
          *reinterpret_cast<uint16_t*>(kbp + (pos13 >> 4) * 128 + j * 16 + (pos13 & 15)) =
              (uint16_t)((dg[1] & 0xFF) | ((dg[3] & 0xFF) << 8));
        }
        if (sub == 0) xs[kbl] = live ? __int_as_float((127 - (8 * NL - 3) + (e - 127)) << 23) : 0.f;
      }
    };
    // residual + split-K partials (slice order) -> hs (all of H), optional write-back, RMSNorm of the staged slice
    auto stage_norm = [&](const float* h_in, const float* parts, int nparts, float* h_out, bool writer, const float* nw,
                          int kbA, int nkbA) {
      if (nkbA == 0) return;                              // no unit of this op here (the writer always has one)
      float* hs = work;
      float* xf = work + a.H;
      const int H4 = a.H >> 2;
      float ss = 0.f;
      for (int i = t; i < H4; i += CT) {
        float4 v = __ldcg(reinterpret_cast<const float4*>(h_in) + i);
        float4 w[MAX_KSPLIT];                             // every partial is requested before the first add
#pragma unroll
        for (int p = 0; p < MAX_KSPLIT; ++p)
          w[p] = p < nparts ? __ldcg(reinterpret_cast<const float4*>(parts) + (size_t)p * H4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int p = 0; p < MAX_KSPLIT; ++p) {
          if (p < nparts) {
            v.x += w[p].x; v.y += w[p].y; v.z += w[p].z; v.w += w[p].w;
          }
        }
        reinterpret_cast<float4*>(hs)[i] = v;
        if (writer) reinterpret_cast<float4*>(h_out)[i] = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
      ss = warp_sum(ss);
      if (lane == 0) red[warp] = ss;
      if (fine) stamp(11);
      named_sync(1, CT);
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) tot += red[w];
      const float rnorm = rsqrtf(tot / (float)a.H + a.eps);
      for (int i = t; i < nkbA * 32; i += CT) {
        const int k = kbA * 32 + i;
        xf[i] = round16((hs[k] * __ldg(nw + k)) * rnorm);
      }
      named_sync(1, CT);
      if (fine) stamp(12);
      digits(xf, nkbA);
      if (fine) stamp(13);
    };
    // merge of the attention partials for the staged slice of the attention output vector
    auto stage_att = [&](int kbA, int nkbA) {
      float* xf = work;
      float* wtab = work + a.bkb * 32;                    // [head of the slice][chunk] = exp(m_c - M) / L
      if (nkbA > 0) {
        int p = (int)__ldcg(a.pos);
        p = p < 0 ? 0 : (p >= a.max_len ? a.max_len - 1 : p);
        int chunk, nch;
        attn_geometry(p, a.NKV, ncta, chunk, nch);
        const int hq0 = (kbA * 32) / HD, hq1 = ((kbA + nkbA) * 32 - 1) / HD;
        const int nheads = min(hq1 - hq0 + 1, MAX_WHEADS);
        for (int hh = warp; hh < nheads; hh += CT / 32) {
          const float* ap = a.att_part + (size_t)(hq0 + hh) * a.nch_max * (HD + 2);
          float M = -INFINITY;
          for (int c = lane; c < nch; c += 32) M = fmaxf(M, __ldcg(ap + (size_t)c * (HD + 2) + HD));
          M = warp_max(M);
          float L = 0.f;
          for (int c = lane; c < nch; c += 32)
            L += __ldcg(ap + (size_t)c * (HD + 2) + HD + 1) * __expf(__ldcg(ap + (size_t)c * (HD + 2) + HD) - M);
          L = warp_sum(L);
          const float invL = 1.f / L;
          for (int c = lane; c < nch; c += 32) wtab[hh * a.nch_max + c] = __expf(__ldcg(ap + (size_t)c * (HD + 2) + HD) - M) * invL;
        }
        if (fine) stamp(11);
        named_sync(1, CT);
        for (int i = t; i < nkbA * 32; i += CT) {
          const int k = kbA * 32 + i, hq = k / HD, d = k - hq * HD;
          const int hh = min(hq - hq0, MAX_WHEADS - 1);
          const float* ap = a.att_part + (size_t)hq * a.nch_max * (HD + 2) + d;
          float o = 0.f;
          for (int c0 = 0; c0 < nch; c0 += 8) {
            float pv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) pv[u] = c0 + u < nch ? __ldcg(ap + (size_t)(c0 + u) * (HD + 2)) : 0.f;
#pragma unroll
            for (int u = 0; u < 8; ++u)
              if (c0 + u < nch) o = fmaf(wtab[hh * a.nch_max + c0 + u], pv[u], o);
          }
          xf[i] = round16(o);
        }
        named_sync(1, CT);
        if (fine) stamp(12);
        digits(xf, nkbA);
        if (fine) stamp(13);
      }
    };
    auto stage_xm = [&](int kbA, int nkbA) {
      if (nkbA == 0) return;
      float* xf = work;
      const unsigned short* src = reinterpret_cast<const unsigned short*>(a.xm) + (size_t)kbA * 32;
      for (int i = t; i < nkbA * 32; i += CT) xf[i] = __half2float(__ushort_as_half(__ldcg(src + i)));
      named_sync(1, CT);
      digits(xf, nkbA);
    };

    // One linear over this CTA's units.  epi 0: fp32 partial [ks][N] to `out`; epi 1: SwiGLU of interleaved
    // (gate, up) rows to fp16 `out` (whole rows only).
    auto run_linear = [&](const PLinear& g, int kbA, int epi, void* out) {
      tc::fence_async_smem();                            // staged operand -> visible to the tensor core's reads
      named_sync(2, CT + 32);
      if (fine) stamp(10);
      Unit u;
      for (int idx = 0; get_unit(g, cta, ncta, idx, u); ++idx) {
        float acc = 0.f;
        for (int kb = u.kb0; kb < u.kb1; kb += G, ++q) {
          const int nb = min(G, u.kb1 - kb);
          const uint32_t s = q % (uint32_t)NST, slot = q & (NSLOT - 1);
          const uint8_t* st = ring + (size_t)s * STAGE_BYTES;
          wait(&full[s], (q / (uint32_t)NST) & 1u);
          if (expander) {
            if (q >= NSLOT) wait(&dempty[slot], ((q / NSLOT) - 1u) & 1u);
            tc::fence_after_sync();
#pragma unroll
            for (int j = 0; j < G; ++j) {
              if (j < nb) {
                const uint4 w = *reinterpret_cast<const uint4*>(st + (size_t)j * 2048 + r * 16);
                uint32_t ex[8];
                tc::expand_nibbles(w.x, ex[0], ex[1]);
                tc::expand_nibbles(w.y, ex[2], ex[3]);
                tc::expand_nibbles(w.z, ex[4], ex[5]);
                tc::expand_nibbles(w.w, ex[6], ex[7]);
                tc::tmem_st8(tmem_a + lane_off + slot * 64 + (uint32_t)j * 8, ex);
              }
            }
            tc::tmem_wait_st();
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              tc::mbar_arrive(&aready[slot]);
              tc::mbar_arrive(&empty[s]);
            }
          } else {
            wait(&dfull[slot], (q / NSLOT) & 1u);
            tc::fence_after_sync();
            uint32_t d[G][4];
#pragma unroll
            for (int j = 0; j < G; ++j)
              if (j < nb) tc::tmem_ld4(tmem_d + lane_off + slot * 64 + (uint32_t)j * 8, d[j]);
            tc::tmem_wait_ld();
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&dempty[slot]);
            const __half* sc = reinterpret_cast<const __half*>(st + STAGE_NIB) + r;
#pragma unroll
            for (int j = 0; j < G; ++j) {
              if (j < nb) {
                const float dw = __half2float(sc[j * 128]) * 0.0625f;     // 1/16 undoes the 16 (q - 8) operand scaling
                float f = fmaf(256.f, (float)(int32_t)d[j][1], (float)(int32_t)d[j][0]);
                f = fmaf(65536.f, (float)(int32_t)d[j][2], f);
                acc = fmaf(dw * xs[kb + j - kbA], f, acc);
              }
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&empty[s]);
          }
        }
        if (fine) stamp(14);
        if (!expander) {
          const int row = u.tile * 128 + r;
          if (epi == 0) {
            if (row < g.N) reinterpret_cast<float*>(out)[(size_t)u.ks * g.N + row] = acc;
          } else {
            const float partner = __shfl_xor_sync(0xffffffffu, acc, 1);
            if (row < g.N && (r & 1) == 0)
              reinterpret_cast<__half*>(out)[row >> 1] = __float2half_rn(acc / (1.f + __expf(-acc)) * partner);
          }
        }
      }
    };

    // Attention units: (KV head, chunk of positions).
    auto attention = [&](const PLayer& L, int ks_qkv) {
      const int GRP = a.NH / a.NKV, HALF = HD / 2, QR = (a.NH + 2 * a.NKV) * HD;
      constexpr int NG = CT / HD;                         // position groups of the P.V pass
      constexpr int PPG = 32 / NG;                        // positions per group and sub-chunk
      constexpr int DSEG = HD / 8;                        // dims per lane of a score row (8 lanes per position)
      float* raw = work;                                  // (GRP + 2) HD: fp16-valued q rows, k row, v row
      float* qs = raw + (MAX_GRP + 2) * HD;
      float* kn = qs + MAX_GRP * HD;
      float* vn = kn + HD;
      float* sc = vn + HD;                                // [MAX_GRP][32]
      float* stat = sc + MAX_GRP * 32;                    // [MAX_GRP][4]: max, sum, rescale of this sub-chunk
      float* redo = stat + MAX_GRP * 4;                   // [NG][MAX_GRP][HD]
      int p = (int)__ldcg(a.pos);
      p = p < 0 ? 0 : (p >= a.max_len ? a.max_len - 1 : p);
      int chunk, nch;
      attn_geometry(p, a.NKV, ncta, chunk, nch);
      const float* cs = a.cosT + (size_t)p * HALF;
      const float* sn = a.sinT + (size_t)p * HALF;
      for (int un = cta; un < a.NKV * nch; un += ncta) {
        const int kvh = un / nch, c = un - kvh * nch;
        const int base0 = c * chunk, end = min(base0 + chunk, p + 1);
        const bool has_new = p >= base0 && p < base0 + chunk;
        __half* kbase = L.kc + (size_t)kvh * a.max_len * HD;
        __half* vbase = L.vc + (size_t)kvh * a.max_len * HD;
        // a. the q rows of this KV head (and the new k, v rows): sum of the split-K partials + bias, rounded to fp16
        for (int i = t; i < (GRP + 2) * HD; i += CT) {
          const int hl = i / HD, d = i - hl * HD;
          if (hl >= GRP && !has_new) continue;
          const int row = hl < GRP ? (kvh * GRP + hl) * HD + d
                                   : (hl == GRP ? a.NH * HD + kvh * HD + d : (a.NH + a.NKV) * HD + kvh * HD + d);
          float w[MAX_KSPLIT];
#pragma unroll
          for (int ks = 0; ks < MAX_KSPLIT; ++ks) w[ks] = ks < ks_qkv ? __ldcg(a.part_qkv + (size_t)ks * QR + row) : 0.f;
          float v = 0.f;
#pragma unroll
          for (int ks = 0; ks < MAX_KSPLIT; ++ks)
            if (ks < ks_qkv) v += w[ks];
          raw[i] = round16(v + __ldg(L.bias + row));
        }
        named_sync(1, CT);
        if (fine) stamp(30);
        // b. RoPE (rotate-half pairs d, d + HD/2), fp16 rounding, append of the new row
        for (int i = t; i < (GRP + 1) * HD; i += CT) {
          const int hl = i / HD, d = i - hl * HD, dd = d % HALF;
          if (hl == GRP && !has_new) continue;
          const float* src = raw + hl * HD;
          const float x0 = src[d], x1 = src[d < HALF ? d + HALF : d - HALF];
          const float rr = round16(d < HALF ? x0 * cs[dd] - x1 * sn[dd] : x0 * cs[dd] + x1 * sn[dd]);
          if (hl < GRP) {
            qs[i] = rr;
          } else {
            kn[d] = rr;
            kbase[(size_t)p * HD + d] = __float2half_rn(rr);
          }
        }
        if (has_new) {
          for (int d = t; d < HD; d += CT) {
            const float v = raw[(GRP + 1) * HD + d];
            vn[d] = v;
            vbase[(size_t)p * HD + d] = __float2half_rn(v);
          }
        }
        if (t < MAX_GRP) {
          stat[t * 4] = -INFINITY;
          stat[t * 4 + 1] = 0.f;
        }
        named_sync(1, CT);
        if (fine) stamp(31);
        // c. sub-chunks of 32 positions with a running (max, sum)
        const int dv = t % HD, gv = t / HD;
        float acc[MAX_GRP];
#pragma unroll
        for (int h = 0; h < MAX_GRP; ++h) acc[h] = 0.f;
        for (int base = base0; base < end; base += 32) {
          const int j = base + (t >> 3), seg = t & 7;
          float kf[DSEG];
          if (j < p) {
            const uint4* kr = reinterpret_cast<const uint4*>(kbase + (size_t)j * HD + seg * DSEG);
#pragma unroll
            for (int i = 0; i < DSEG / 8; ++i) {
              const uint4 kq = kr[i];
              const uint32_t w[4] = {kq.x, kq.y, kq.z, kq.w};
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[u]));
                kf[8 * i + 2 * u] = f.x;
                kf[8 * i + 2 * u + 1] = f.y;
              }
            }
          } else {
#pragma unroll
            for (int e = 0; e < DSEG; ++e) kf[e] = j == p ? kn[seg * DSEG + e] : 0.f;
          }
          __half vraw[PPG];
#pragma unroll
          for (int i = 0; i < PPG; ++i) {
            const int jv = base + gv * PPG + i;
            vraw[i] = jv < p ? vbase[(size_t)jv * HD + dv] : __float2half_rn(0.f);
          }
          float s[MAX_GRP];
#pragma unroll
          for (int h = 0; h < MAX_GRP; ++h) {
            s[h] = 0.f;
            if (h < GRP) {
#pragma unroll
              for (int e = 0; e < DSEG; ++e) s[h] = fmaf(qs[h * HD + seg * DSEG + e], kf[e], s[h]);
            }
            s[h] += __shfl_xor_sync(0xffffffffu, s[h], 1);
            s[h] += __shfl_xor_sync(0xffffffffu, s[h], 2);
            s[h] += __shfl_xor_sync(0xffffffffu, s[h], 4);
          }
          if (seg == 0) {
#pragma unroll
            for (int h = 0; h < MAX_GRP; ++h) sc[h * 32 + (t >> 3)] = j <= p ? s[h] * a.scale : -INFINITY;
          }
          named_sync(1, CT);
          if (warp < GRP) {
            const float v = sc[warp * 32 + lane];
            const float m_old = stat[warp * 4];
            const float m_new = fmaxf(m_old, warp_max(v));           // finite: position base <= p is valid
            const float e = __expf(v - m_new);
            const float sum = warp_sum(e);
            sc[warp * 32 + lane] = e;
            if (lane == 0) {
              const float alpha = __expf(m_old - m_new);             // 0 on the first sub-chunk
              stat[warp * 4] = m_new;
              stat[warp * 4 + 1] = stat[warp * 4 + 1] * alpha + sum;
              stat[warp * 4 + 2] = alpha;
            }
          }
          named_sync(1, CT);
#pragma unroll
          for (int h = 0; h < MAX_GRP; ++h) {
            if (h < GRP) {
              float o = acc[h] * stat[h * 4 + 2];
#pragma unroll
              for (int i = 0; i < PPG; ++i) {
                const int jv = base + gv * PPG + i;
                const float vv = jv == p ? vn[dv] : __half2float(vraw[i]);
                o = fmaf(sc[h * 32 + gv * PPG + i], vv, o);
              }
              acc[h] = o;
            }
          }
          named_sync(1, CT);
        }
        if (fine) stamp(32);
        // d. position groups -> one partial per (head, chunk)
#pragma unroll
        for (int h = 0; h < MAX_GRP; ++h)
          if (h < GRP) redo[(gv * MAX_GRP + h) * HD + dv] = acc[h];
        named_sync(1, CT);
        for (int i = t; i < GRP * HD; i += CT) {
          const int h = i / HD, d = i - h * HD;
          float o = 0.f;
#pragma unroll
          for (int gq = 0; gq < NG; ++gq) o += redo[(gq * MAX_GRP + h) * HD + d];
          a.att_part[((size_t)(kvh * GRP + h) * a.nch_max + c) * (HD + 2) + d] = o;
        }
        if (t < GRP) {
          float* ap = a.att_part + ((size_t)(kvh * GRP + t) * a.nch_max + c) * (HD + 2) + HD;
          ap[0] = stat[t * 4];
          ap[1] = stat[t * 4 + 1];
        }
        named_sync(1, CT);
      }
    };

    stamp(0);
    int ks_down_prev = 0;
    for (int l = 0; l < a.layers; ++l) {
      const PLayer& L = a.layer[l];
      int kbA, nkbA;
      // ---- q/k/v projection of RMSNorm(residual)
      staged_range(L.lin[0], cta, ncta, kbA, nkbA);
      stage_norm(a.hA, a.part_down, ks_down_prev, a.hB, cta == L.lin[0].rot, L.ln1, kbA, nkbA);
      run_linear(L.lin[0], kbA, 0, a.part_qkv);
      grid_barrier();
      // ---- attention
      attention(L, L.lin[0].ksplit);
      grid_barrier();
      // ---- output projection
      staged_range(L.lin[1], cta, ncta, kbA, nkbA);
      stage_att(kbA, nkbA);
      run_linear(L.lin[1], kbA, 0, a.part_o);
      grid_barrier();
      // ---- gate/up projection of RMSNorm(residual + attention), SwiGLU
      staged_range(L.lin[2], cta, ncta, kbA, nkbA);
      stage_norm(a.hB, a.part_o, L.lin[1].ksplit, a.hA, cta == L.lin[2].rot, L.ln2, kbA, nkbA);
      run_linear(L.lin[2], kbA, 1, a.xm);
      grid_barrier();
      // ---- down projection
      staged_range(L.lin[3], cta, ncta, kbA, nkbA);
      stage_xm(kbA, nkbA);
      run_linear(L.lin[3], kbA, 0, a.part_down);
      grid_barrier();
      ks_down_prev = L.lin[3].ksplit;
    }
    // ---- the last residual add, spread over the CTAs (each element is read and written by one thread)
    for (int i = cta * CT + t; i < a.H; i += ncta * CT) {
      float v = __ldcg(a.hA + i);
      for (int p = 0; p < ks_down_prev; ++p) v += __ldcg(a.part_down + (size_t)p * a.H + i);
      a.hA[i] = v;
    }
    stamp(2);
  }

  if (!ok) atomicExch(a.status, 1u);
  tc::fence_before_sync();
  tc::drain_mmas_on_failure(ok, warp == WARP_MMA && lane == 0, &bar_drain);
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, 512);
  if (t == 0) {
    __threadfence();
    const uint32_t left = atomicAdd(a.sync + 1, 1u);
    if (left == (uint32_t)ncta - 1u) {                   // the last CTA out re-arms the counters for the next launch
      a.sync[0] = 0u;
      a.sync[1] = 0u;
      __threadfence();
    }
  }
}

unsigned long long* g_ptrace = nullptr;
int g_ptrace_stride = 0;

struct Plan {
  int ksplit[4];
  int rot[4];
  int nstage, bkb, nch_max, ncta;
  size_t smem;
  size_t off_layers, off_hB, off_pq, off_po, off_pd, off_att, off_sync, total;
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

void decode_persistent_trace(unsigned long long* buf, int stride) {
  g_ptrace = buf;
  g_ptrace_stride = stride;
}

namespace {

// Geometry for a model shape on this device.  Returns false when the shape does not fit the kernel.
bool make_plan(const q4b_decode_desc* d, Plan& p, const char** why) {
  const int ncta = sm_count();
  p.ncta = ncta;
  const int H = d->hidden, HD = d->head_dim, QR = d->n_heads * HD, QKV = (d->n_heads + 2 * d->n_kv_heads) * HD;
  if (HD != 64 && HD != 128) return *why = "head_dim must be 64 or 128", false;
  if (d->n_heads % d->n_kv_heads || d->n_heads / d->n_kv_heads > MAX_GRP) return *why = "more than 8 query heads per KV head", false;
  if (H % 256 || QR % 32 || d->ffn % 32) return *why = "hidden must be a multiple of 256, other K a multiple of 32", false;
  const int N[4] = {QKV, H, 2 * d->ffn, H};
  const int KB[4] = {H / 32, QR / 32, H / 32, d->ffn / 32};
  const char* env = getenv("Q4B_PERSISTENT_KSPLIT");     // "qkv,o,down" override for experiments
  int over[3] = {0, 0, 0};
  if (env) sscanf(env, "%d,%d,%d", &over[0], &over[1], &over[2]);
  int bkb = 0;
  for (int o = 0; o < 4; ++o) {
    const int tiles = (N[o] + 127) / 128;
    int ks = 1;
    if (o != 2 && tiles < ncta) {
      ks = ncta / tiles;
      ks = std::min(ks, std::max(1, KB[o] / 4));          // at least 4 k-blocks per slice
      ks = std::min(ks, 16);
      const int ov = o == 0 ? over[0] : (o == 1 ? over[1] : over[2]);
      if (ov > 0) ks = std::min(ov, KB[o]);
    }
    p.ksplit[o] = ks;
    p.rot[o] = 0;
    const int slice = ks == 1 ? KB[o] : (KB[o] + ks - 1) / ks + 1;
    bkb = std::max(bkb, slice);
  }
  // spread the ops with few units over different CTAs
  {
    const int u1 = ((N[1] + 127) / 128) * p.ksplit[1];
    if (u1 < ncta) p.rot[1] = ncta - u1;
    const int u3 = ((N[3] + 127) / 128) * p.ksplit[3];
    if (u3 < ncta) p.rot[3] = (ncta - u3) / 2;
  }
  p.bkb = (bkb + 3) & ~3;
  p.nch_max = ncta;
  const size_t work_gemv = (size_t)H + (size_t)p.bkb * 32 + (size_t)MAX_WHEADS * p.nch_max;
  const size_t work_attn = (size_t)(MAX_GRP + 2) * HD + (size_t)MAX_GRP * HD + 2 * HD + MAX_GRP * 32 + MAX_GRP * 4 +
                           (size_t)(CT / HD) * MAX_GRP * HD;
  const size_t misc = (size_t)p.bkb * 256 + (size_t)p.bkb * 4 + std::max(work_gemv, work_attn) * 4 + 256;
  if (misc + 4 * (size_t)STAGE_BYTES > MAX_DYN_SMEM) return *why = "activation staging does not fit shared memory", false;
  p.nstage = (int)std::min<size_t>(MAX_STAGES, (MAX_DYN_SMEM - misc) / STAGE_BYTES);
  p.smem = (size_t)p.nstage * STAGE_BYTES + misc;
  if ((QR / HD) > 0 && HD * MAX_WHEADS < ((KB[1] + p.ksplit[1] - 1) / p.ksplit[1] + 1) * 32 + HD)
    return *why = "o_proj K slice spans too many heads", false;
  size_t off = 0;
  p.off_layers = off; off = align_up(off + sizeof(PLayer) * (size_t)d->layers, 256);
  p.off_hB = off; off = align_up(off + (size_t)H * 4, 256);
  p.off_pq = off; off = align_up(off + (size_t)p.ksplit[0] * QKV * 4, 256);
  p.off_po = off; off = align_up(off + (size_t)p.ksplit[1] * H * 4, 256);
  p.off_pd = off; off = align_up(off + (size_t)p.ksplit[3] * H * 4, 256);
  p.off_att = off; off = align_up(off + (size_t)d->n_heads * p.nch_max * (HD + 2) * 4, 256);
  p.off_sync = off; off = align_up(off + 16, 256);
  p.total = off;
  return true;
}

bool packed_ok(const q4b_linear& L) { return L.Wt && L.St && aligned16(L.Wt) && aligned16(L.St); }

}  // namespace

size_t decode_persistent_workspace(const q4b_decode_desc* d) {
  Plan p;
  const char* why = "";
  if (!d || !make_plan(d, p, &why)) return 0;
  return p.total;
}

// One-time set-up: the device-side layer table and zeroed counters inside `ws`.  Synchronous.
int decode_persistent_prepare(const q4b_decode_desc* d, void* ws, size_t ws_bytes) {
  if (!d || !d->layer || !ws) return fail(Q4B_E_ARG, "decode_persistent_prepare: null argument");
  Plan p;
  const char* why = "";
  if (!make_plan(d, p, &why)) return fail(Q4B_E_SHAPE, why);
  if (ws_bytes < p.total || !aligned16(ws)) return fail(Q4B_E_WORKSPACE, "decode_persistent_prepare: workspace too small or unaligned");
  const int H = d->hidden, HD = d->head_dim, QR = d->n_heads * HD, QKV = (d->n_heads + 2 * d->n_kv_heads) * HD;
  const int N[4] = {QKV, H, 2 * d->ffn, H};
  const int KB[4] = {H / 32, QR / 32, H / 32, d->ffn / 32};
  std::vector<PLayer> tab((size_t)d->layers);
  for (int l = 0; l < d->layers; ++l) {
    const q4b_layer& L = d->layer[l];
    const q4b_linear* lin[4] = {&L.qkv, &L.o, &L.gu, &L.down};
    for (int o = 0; o < 4; ++o) {
      if (!packed_ok(*lin[o]) || lin[o]->N != N[o] || lin[o]->K != KB[o] * 32)
        return fail(Q4B_E_SHAPE, "decode_persistent_prepare: every layer matrix needs a tile-packed copy of the model's shape");
      PLinear& g = tab[l].lin[o];
      g.W = reinterpret_cast<const uint8_t*>(lin[o]->Wt);
      g.S = reinterpret_cast<const __half*>(lin[o]->St);
      g.N = N[o];
      g.KB = KB[o];
      g.tiles = (N[o] + 127) / 128;
      g.ksplit = p.ksplit[o];
      g.rot = p.rot[o];
    }
    if (!L.ln1 || !L.ln2 || !L.qkv_bias || !L.kc || !L.vc) return fail(Q4B_E_ARG, "decode_persistent_prepare: null layer pointer");
    tab[l].ln1 = L.ln1;
    tab[l].ln2 = L.ln2;
    tab[l].bias = L.qkv_bias;
    tab[l].kc = reinterpret_cast<__half*>(L.kc);
    tab[l].vc = reinterpret_cast<__half*>(L.vc);
  }
  char* base = reinterpret_cast<char*>(ws);
  cudaError_t e = cudaMemcpy(base + p.off_layers, tab.data(), sizeof(PLayer) * tab.size(), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemset(base + p.off_sync, 0, 16);
  if (e != cudaSuccess) {
    set_cuda_error(e, "decode_persistent_prepare");
    return Q4B_E_CUDA;
  }
  return Q4B_OK;
}

// All layers of one token.  On entry d->h holds the embedding row of the token, on exit the residual stream after the
// last layer.  `ws` must have been through decode_persistent_prepare for the same descriptor.
int decode_persistent_layers(const q4b_decode_desc* d, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (!d || !ws || !d->status) return fail(Q4B_E_ARG, "decode_persistent_layers: null argument");
  Plan p;
  const char* why = "";
  if (!make_plan(d, p, &why)) return fail(Q4B_E_SHAPE, why);
  if (ws_bytes < p.total) return fail(Q4B_E_WORKSPACE, "decode_persistent_layers: workspace too small");
  char* base = reinterpret_cast<char*>(ws);
  PArgs a;
  a.layer = reinterpret_cast<const PLayer*>(base + p.off_layers);
  a.layers = d->layers;
  a.H = d->hidden;
  a.FFN = d->ffn;
  a.NH = d->n_heads;
  a.NKV = d->n_kv_heads;
  a.HD = d->head_dim;
  a.max_len = d->max_len;
  a.eps = d->eps;
  a.scale = d->scale;
  a.cosT = d->cosT;
  a.sinT = d->sinT;
  a.pos = d->pos;
  a.hA = d->h;
  a.hB = reinterpret_cast<float*>(base + p.off_hB);
  a.part_qkv = reinterpret_cast<float*>(base + p.off_pq);
  a.part_o = reinterpret_cast<float*>(base + p.off_po);
  a.part_down = reinterpret_cast<float*>(base + p.off_pd);
  a.att_part = reinterpret_cast<float*>(base + p.off_att);
  a.xm = reinterpret_cast<__half*>(d->act);
  a.sync = reinterpret_cast<uint32_t*>(base + p.off_sync);
  a.status = d->status;
  a.trace = g_ptrace;
  a.trace_stride = g_ptrace_stride;
  a.nstage = p.nstage;
  a.bkb = p.bkb;
  a.nch_max = p.nch_max;
  auto kern = d->head_dim == 128 ? decode_persistent_kernel<128> : decode_persistent_kernel<64>;
  {
    cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), MAX_DYN_SMEM);
    if (e != cudaSuccess) {
      set_cuda_error(e, "decode_persistent: cudaFuncSetAttribute");
      return Q4B_E_CUDA;
    }
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, PT, p.smem);
    if (e != cudaSuccess || per_sm < 1) {
      if (e != cudaSuccess) set_cuda_error(e, "decode_persistent: occupancy query");
      return e != cudaSuccess ? Q4B_E_CUDA : fail(Q4B_E_SHAPE, "decode_persistent: the kernel does not fit one CTA per SM");
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.ncta, 1, 1);
  cfg.blockDim = dim3(PT, 1, 1);
  cfg.dynamicSmemBytes = p.smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;          // all CTAs co-resident: they wait on each other
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a);
  if (e != cudaSuccess) {
    set_cuda_error(e, "decode_persistent: launch");
    return Q4B_E_CUDA;
  }
  return Q4B_OK;
}

}  // namespace q4b
