// Decode attention: RoPE(q), RoPE(k_new), K/V append, GQA attention over an fp16 KV cache, split over the context.
//
// Reference arithmetic: ATTN4 (lab/qwen_kernels.py:517-605): NeoX pairs (d, d + HD/2) with fp32 cos/sin tables, q and
// the new k rounded to 16 bits after rotation, one writer per KV head for the cache append while readers take the new
// position from shared memory, s_j = (q . k_j) * scale, e_j = __expf(s_j - max), out = round16(sum e_j v_j / sum e_j).
// The split over the context follows the flash-decoding ATTN2 (:358-442): per-chunk (max, sum, partial output) go to
// a workspace and the last CTA to arrive combines them, here in chunk order so the result does not depend on timing.
//
// B200 shape: one CTA per (chunk of 128 positions, KV head, sequence) serves all NH/NKV query heads of that KV head,
// so every K/V row is read once.  Scores: one thread per position, its whole K row (HD * 2 bytes) in flight as
// 16-byte loads.  P.V: HD/8 lanes per row with 16-byte loads, 16 rows in flight per warp.
#include "q4b_internal.h"

namespace q4b {

namespace {

constexpr int CH = 128;        // positions per CTA
constexpr int AT = 128;        // threads per CTA
constexpr int NW = AT / 32;

template <int HD, int GRP>
__global__ void __launch_bounds__(AT) attn_decode_kernel(const __half* qkv, const float* __restrict__ cosT,
                                                         const float* __restrict__ sinT, const int64_t* posp,
                                                         __half* kc, __half* vc,
                                                         __half* out, int NH, int NKV, int max_len,
                                                         float scale, unsigned* cnt, float* part_ml, float* part_o, int NC) {
  constexpr int HALF = HD / 2;
  constexpr int LPR = HD / 8;          // lanes per K/V row in the P.V pass (16-byte loads)
  constexpr int PPI = 32 / LPR;        // rows per warp iteration
  __shared__ __align__(16) float qs[GRP][HD];
  __shared__ __align__(16) float kn[HD];
  __shared__ __align__(16) float vn[HD];
  __shared__ float sc[GRP][CH];
  __shared__ float redw[GRP][NW];
  __shared__ __align__(16) float red_o[NW][GRP][HD];
  __shared__ float stat[GRP][2];
  __shared__ bool last;

  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.z, kvh = blockIdx.y, chunk = blockIdx.x;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  int p = (int)posp[b];
  p = p < 0 ? 0 : (p >= max_len ? max_len - 1 : p);
  const int c0 = chunk * CH;
  if (c0 > p) return;                                            // chunk entirely in the future: nothing to do
  const int nact = p / CH + 1;                                   // active chunks of this sequence
  const bool has_new = p < c0 + CH;                              // this chunk holds the position being appended
  const int QKV = (NH + 2 * NKV) * HD;
  const __half* row = qkv + (size_t)b * QKV;
  const float* cs = cosT + (size_t)p * HALF;
  const float* sn = sinT + (size_t)p * HALF;
  __half* kbase = kc + ((size_t)b * NKV + kvh) * (size_t)max_len * HD;
  __half* vbase = vc + ((size_t)b * NKV + kvh) * (size_t)max_len * HD;

  for (int e = t; e < GRP * HD; e += AT) {
    const int hl = e / HD, d = e - hl * HD, dd = d % HALF;
    const __half* qh = row + (size_t)(kvh * GRP + hl) * HD;
    const float a = __half2float(qh[d]), o = __half2float(qh[d < HALF ? d + HALF : d - HALF]);
    const float r = d < HALF ? a * cs[dd] - o * sn[dd] : a * cs[dd] + o * sn[dd];
    qs[hl][d] = __half2float(__float2half_rn(r));
  }
  if (has_new) {
    for (int d = t; d < HD; d += AT) {
      const int dd = d % HALF;
      const __half* kh = row + (size_t)NH * HD + (size_t)kvh * HD;
      const float a = __half2float(kh[d]), o = __half2float(kh[d < HALF ? d + HALF : d - HALF]);
      const __half kr = __float2half_rn(d < HALF ? a * cs[dd] - o * sn[dd] : a * cs[dd] + o * sn[dd]);
      const __half vr = row[(size_t)(NH + NKV) * HD + (size_t)kvh * HD + d];
      kn[d] = __half2float(kr);
      vn[d] = __half2float(vr);
      kbase[(size_t)p * HD + d] = kr;                            // the only writer of (b, kvh, p)
      vbase[(size_t)p * HD + d] = vr;
    }
  }
  __syncthreads();

  // ---- scores: thread t <-> position c0 + t
  float s[GRP];
  {
    const int j = c0 + t;
    const bool valid = j <= p;
#pragma unroll
    for (int h = 0; h < GRP; ++h) s[h] = 0.f;
    if (valid) {
      if (j == p) {
#pragma unroll 4
        for (int d = 0; d < HD; ++d) {
          const float k = kn[d];
#pragma unroll
          for (int h = 0; h < GRP; ++h) s[h] = fmaf(qs[h][d], k, s[h]);
        }
      } else {
        const uint4* kr = reinterpret_cast<const uint4*>(kbase + (size_t)j * HD);
        uint4 kv[HD / 8];
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) kv[i] = kr[i];
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
          const uint32_t w[4] = {kv[i].x, kv[i].y, kv[i].z, kv[i].w};
          float kf[8];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[u]));
            kf[2 * u] = f.x;
            kf[2 * u + 1] = f.y;
          }
#pragma unroll
          for (int h = 0; h < GRP; ++h) {
            const float4 q0 = *reinterpret_cast<const float4*>(&qs[h][8 * i]);
            const float4 q1 = *reinterpret_cast<const float4*>(&qs[h][8 * i + 4]);
            float a = s[h];
            a = fmaf(q0.x, kf[0], a); a = fmaf(q0.y, kf[1], a); a = fmaf(q0.z, kf[2], a); a = fmaf(q0.w, kf[3], a);
            a = fmaf(q1.x, kf[4], a); a = fmaf(q1.y, kf[5], a); a = fmaf(q1.z, kf[6], a); a = fmaf(q1.w, kf[7], a);
            s[h] = a;
          }
        }
      }
    }
#pragma unroll
    for (int h = 0; h < GRP; ++h) s[h] = valid ? s[h] * scale : -INFINITY;
  }
  // chunk maximum per head
#pragma unroll
  for (int h = 0; h < GRP; ++h) {
    const float m = warp_max(s[h]);
    if (lane == 0) redw[h][warp] = m;
  }
  __syncthreads();
  float mx[GRP];
#pragma unroll
  for (int h = 0; h < GRP; ++h) {
    float m = redw[h][0];
#pragma unroll
    for (int w = 1; w < NW; ++w) m = fmaxf(m, redw[h][w]);
    mx[h] = m;                                                   // finite: position c0 <= p is always valid
  }
  __syncthreads();
#pragma unroll
  for (int h = 0; h < GRP; ++h) {
    const float e = __expf(s[h] - mx[h]);                        // 0 for masked positions
    sc[h][t] = e;
    const float l = warp_sum(e);
    if (lane == 0) redw[h][warp] = l;
  }
  __syncthreads();
  float ls[GRP];
#pragma unroll
  for (int h = 0; h < GRP; ++h) {
    float l = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) l += redw[h][w];
    ls[h] = l;
  }

  // ---- P.V: warp w <-> positions c0 + 32w .. +31; lane <-> (row in the iteration, 8 dims)
  const int psub = lane / LPR, d0 = (lane % LPR) * 8;
  float acc[GRP][8];
#pragma unroll
  for (int h = 0; h < GRP; ++h)
#pragma unroll
    for (int u = 0; u < 8; ++u) acc[h][u] = 0.f;
  constexpr int ITERS = 32 / PPI, UNR = ITERS < 8 ? ITERS : 8;
  for (int it0 = 0; it0 < ITERS; it0 += UNR) {
    uint4 vv[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int jl = 32 * warp + (it0 + u) * PPI + psub, j = c0 + jl;
      vv[u] = make_uint4(0u, 0u, 0u, 0u);
      if (j < p) vv[u] = *reinterpret_cast<const uint4*>(vbase + (size_t)j * HD + d0);
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int jl = 32 * warp + (it0 + u) * PPI + psub, j = c0 + jl;
      if (j > p) continue;
      float vf[8];
      if (j == p) {
#pragma unroll
        for (int k = 0; k < 8; ++k) vf[k] = vn[d0 + k];
      } else {
        const uint32_t w[4] = {vv[u].x, vv[u].y, vv[u].z, vv[u].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
          vf[2 * k] = f.x;
          vf[2 * k + 1] = f.y;
        }
      }
#pragma unroll
      for (int h = 0; h < GRP; ++h) {
        const float e = sc[h][jl];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[h][k] = fmaf(e, vf[k], acc[h][k]);
      }
    }
  }
#pragma unroll
  for (int h = 0; h < GRP; ++h)
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float a = acc[h][k];
#pragma unroll
      for (int o = 16; o >= LPR; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
      acc[h][k] = a;
    }
  if (psub == 0) {
#pragma unroll
    for (int h = 0; h < GRP; ++h)
#pragma unroll
      for (int k = 0; k < 8; ++k) red_o[warp][h][d0 + k] = acc[h][k];
  }
  __syncthreads();

  // ---- chunk result; a single active chunk writes the output directly
  const size_t head0 = (size_t)b * NH + (size_t)kvh * GRP;
  if (nact == 1) {
    for (int e = t; e < GRP * HD; e += AT) {
      const int hl = e / HD, d = e - hl * HD;
      float o = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) o += red_o[w][hl][d];
      float l = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) l += redw[hl][w];
      out[(head0 + hl) * HD + d] = __float2half_rn(o / l);
    }
    return;
  }
  for (int e = t; e < GRP * HD; e += AT) {
    const int hl = e / HD, d = e - hl * HD;
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) o += red_o[w][hl][d];
    part_o[((head0 + hl) * NC + chunk) * HD + d] = o;
  }
  if (t < GRP) {
    part_ml[((head0 + t) * NC + chunk) * 2] = mx[t];
    part_ml[((head0 + t) * NC + chunk) * 2 + 1] = ls[t];
  }
  __threadfence();
  __syncthreads();
  if (t == 0) last = atomicAdd(cnt + (size_t)b * NKV + kvh, 1u) == (unsigned)(nact - 1);
  __syncthreads();
  if (!last) return;
  __threadfence();
  if (t < GRP) {
    float M = -INFINITY;
    for (int c = 0; c < nact; ++c) M = fmaxf(M, __ldcg(part_ml + ((head0 + t) * NC + c) * 2));
    float L = 0.f;
    for (int c = 0; c < nact; ++c)
      L += __ldcg(part_ml + ((head0 + t) * NC + c) * 2 + 1) * __expf(__ldcg(part_ml + ((head0 + t) * NC + c) * 2) - M);
    stat[t][0] = M;
    stat[t][1] = L;
  }
  __syncthreads();
  for (int e = t; e < GRP * HD; e += AT) {
    const int hl = e / HD, d = e - hl * HD;
    const float M = stat[hl][0];
    float o = 0.f;
    for (int c = 0; c < nact; ++c)
      o += __ldcg(part_o + ((head0 + hl) * NC + c) * HD + d) * __expf(__ldcg(part_ml + ((head0 + hl) * NC + c) * 2) - M);
    out[(head0 + hl) * HD + d] = __float2half_rn(o / stat[hl][1]);
  }
  if (t == 0) cnt[(size_t)b * NKV + kvh] = 0u;
}


// ---- cluster variant ------------------------------------------------------------------------------------------------
// The context is cut into 8 chunks, one CTA each, and the 8 CTAs of a (sequence, KV head, head subgroup) form a
// thread-block cluster: partial (max, sum, output) stay in shared memory and the first CTA combines them through
// distributed shared memory in chunk order.  No workspace, no atomics, no second trip through global memory.  A query
// head group is split over CTAs (HSUB heads each) so that decode at batch 1 still spreads over several dozen SMs.
constexpr int NCL = 8;         // chunks = cluster size

template <int HD, int HSUB, int PASSES>
__global__ void __launch_bounds__(AT) attn_decode_cluster_kernel(const __half* qkv, const float* __restrict__ cosT,
                                                                 const float* __restrict__ sinT, const int64_t* posp,
                                                                 __half* kc, __half* vc, __half* out, int NH, int NKV, int GRP,
                                                                 int nsub, int max_len, float scale, int pre, unsigned long long* trace) {
  // pre != 0: the producer of `qkv` already rotated q and appended the rotated k / raw v at pos (the fused epilogue of
  // the QKV projection), so this kernel only reads: no tables, no writer, position pos comes from the cache like the rest
  constexpr int HALF = HD / 2;
  constexpr int LPR = HD / 8;          // lanes per K/V row in the P.V pass (16-byte loads)
  constexpr int PPI = 32 / LPR;        // rows per warp iteration
  constexpr int CHK = 128 * PASSES;    // positions per CTA
  __shared__ __align__(16) float qs[HSUB][HD];
  __shared__ __align__(16) float kn[HD];
  __shared__ __align__(16) float vn[HD];
  __shared__ float sc[HSUB][CHK];                // exp(score - warp maximum), read back only by the warp that wrote it
  __shared__ float wml[NW][HSUB][2];             // per warp: maximum, sum
  __shared__ __align__(16) float red_o[NW][HSUB][HD];
  // combiner (meaningful in the cluster's first CTA): every chunk PUSHES its partial output and (max, sum) here through
  // distributed shared memory, so after one cluster barrier the combine runs on local data only
  __shared__ __align__(16) float comb_o[NCL][HSUB][HD];
  __shared__ float comb_ml[NCL][HSUB][2];

  unsigned long long* tr = (trace && threadIdx.x == 0)
                               ? trace + (size_t)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 : nullptr;
  int tri = 0;
  auto stamp = [&]() {
    if (tr && tri < 15) {
      unsigned long long gt;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
      tr[tri++] = gt;
      tr[15] = (unsigned long long)tri;
    }
  };
  stamp();                                                          // 0: start
  pdl_launch_dependents();
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");      // "this CTA exists" (paired with the wait before the push)
  const int b = blockIdx.z, chunk = blockIdx.x;
  const int kvh = blockIdx.y / nsub, hs = blockIdx.y - kvh * nsub;
  const int h0 = hs * HSUB, nh = min(HSUB, GRP - h0);
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int c0 = chunk * CHK;
  __half* kbase = kc + ((size_t)b * NKV + kvh) * (size_t)max_len * HD;
  __half* vbase = vc + ((size_t)b * NKV + kvh) * (size_t)max_len * HD;
  const int psub = lane / LPR, d0 = (lane % LPR) * 8;     // P.V pass: lane <-> (row of the warp step, 8 dims)
  constexpr int IPP = 32 / PPI;                          // warp steps per pass
  constexpr bool VPRE = PASSES == 1;                     // V rows of the chunk held in registers from the start
  // Ahead of the dependency wait: ask for this chunk's K and V rows to be brought into L2.  Rows below the current
  // position were written by earlier tokens; a prefetch binds nothing, so a row that is still being appended by the
  // predecessor is simply read again after the wait.
  if (t < 2) {
    const int rows = min(CHK, max_len - c0);
    if (rows > 0) {
      const __half* src = (t == 0 ? kbase : vbase) + (size_t)c0 * HD;
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"((uint32_t)(rows * HD * 2)) : "memory");
    }
  }
  pdl_wait();
  stamp();                                                          // 1: predecessor complete
  const int64_t praw = posp[b];

  // ---- K (and, for one-pass chunks, V) rows are requested before the position is known, so that the position, the
  // cache rows and the new q/k/v row are one round trip to memory instead of two.  Rows at or beyond the current
  // position hold stale or concurrently appended data; they are loaded but never used.
  constexpr int PRE = PASSES * HD <= 256 ? PASSES : 256 / HD;       // passes whose K row is held in registers
  uint4 kv[PRE][HD / 8];
#pragma unroll
  for (int ps = 0; ps < PRE; ++ps) {
    const int j = min(c0 + 128 * ps + t, max_len - 1);
    const uint4* kr = reinterpret_cast<const uint4*>(kbase + (size_t)j * HD);
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) kv[ps][i] = kr[i];
  }
  uint4 vpre[VPRE ? IPP : 1];
  if (VPRE) {
#pragma unroll
    for (int it = 0; it < IPP; ++it) {
      const int j = min(c0 + 32 * warp + it * PPI + psub, max_len - 1);
      vpre[it] = *reinterpret_cast<const uint4*>(vbase + (size_t)j * HD + d0);
    }
  }
  int p = (int)praw;
  p = p < 0 ? 0 : (p >= max_len ? max_len - 1 : p);
  const bool active = c0 <= p;
  const int nact = p / CHK + 1;
  const size_t head0 = (size_t)b * NH + (size_t)kvh * GRP + h0;

  if (active) {
    const bool has_new = !pre && p < c0 + CHK;
    const int QKV = (NH + 2 * NKV) * HD;
    const __half* row = qkv + (size_t)b * QKV;
    const float* cs = cosT + (size_t)p * HALF;
    const float* sn = sinT + (size_t)p * HALF;
    for (int e = t; e < HSUB * HD; e += AT) {
      const int hl = e / HD, d = e - hl * HD, dd = d % HALF;
      float r = 0.f;
      if (hl < nh) {
        const __half* qh = row + (size_t)(kvh * GRP + h0 + hl) * HD;
        const float a = __half2float(qh[d]);
        if (pre) {
          r = a;
        } else {
          const float o = __half2float(qh[d < HALF ? d + HALF : d - HALF]);
          r = d < HALF ? a * cs[dd] - o * sn[dd] : a * cs[dd] + o * sn[dd];
        }
      }
      qs[hl][d] = __half2float(__float2half_rn(r));
    }
    if (has_new) {
      for (int d = t; d < HD; d += AT) {
        const int dd = d % HALF;
        const __half* kh = row + (size_t)NH * HD + (size_t)kvh * HD;
        const float a = __half2float(kh[d]), o = __half2float(kh[d < HALF ? d + HALF : d - HALF]);
        const __half kr = __float2half_rn(d < HALF ? a * cs[dd] - o * sn[dd] : a * cs[dd] + o * sn[dd]);
        const __half vr = row[(size_t)(NH + NKV) * HD + (size_t)kvh * HD + d];
        kn[d] = __half2float(kr);
        vn[d] = __half2float(vr);
        if (hs == 0) {                                              // the only writer of (b, kvh, p)
          kbase[(size_t)p * HD + d] = kr;
          vbase[(size_t)p * HD + d] = vr;
        }
      }
    }
    __syncthreads();

    // ---- scores; softmax statistics per WARP (shuffles only), so no block-wide barrier until the partial outputs
    float s[PASSES][HSUB];
#pragma unroll
    for (int ps = 0; ps < PASSES; ++ps) {
      const int j = c0 + 128 * ps + t;
      const bool valid = j <= p;
#pragma unroll
      for (int h = 0; h < HSUB; ++h) s[ps][h] = 0.f;
      if (!pre && j == p) {
#pragma unroll 4
        for (int d = 0; d < HD; ++d) {
          const float k = kn[d];
#pragma unroll
          for (int h = 0; h < HSUB; ++h) s[ps][h] = fmaf(qs[h][d], k, s[ps][h]);
        }
      } else if (valid) {
        const uint4* kr = reinterpret_cast<const uint4*>(kbase + (size_t)j * HD);
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
          const uint4 kq = ps < PRE ? kv[ps < PRE ? ps : 0][i] : kr[i];   // (registers hold rows below p exactly)
          const uint32_t w[4] = {kq.x, kq.y, kq.z, kq.w};
          float kf[8];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[u]));
            kf[2 * u] = f.x;
            kf[2 * u + 1] = f.y;
          }
#pragma unroll
          for (int h = 0; h < HSUB; ++h) {
            const float4 q0 = *reinterpret_cast<const float4*>(&qs[h][8 * i]);
            const float4 q1 = *reinterpret_cast<const float4*>(&qs[h][8 * i + 4]);
            float a = s[ps][h];
            a = fmaf(q0.x, kf[0], a); a = fmaf(q0.y, kf[1], a); a = fmaf(q0.z, kf[2], a); a = fmaf(q0.w, kf[3], a);
            a = fmaf(q1.x, kf[4], a); a = fmaf(q1.y, kf[5], a); a = fmaf(q1.z, kf[6], a); a = fmaf(q1.w, kf[7], a);
            s[ps][h] = a;
          }
        }
      }
#pragma unroll
      for (int h = 0; h < HSUB; ++h) s[ps][h] = valid ? s[ps][h] * scale : -INFINITY;
    }
    float wm[HSUB];                                                 // this warp's maximum (may be -inf: nothing valid)
#pragma unroll
    for (int h = 0; h < HSUB; ++h) {
      float m = s[0][h];
#pragma unroll
      for (int ps = 1; ps < PASSES; ++ps) m = fmaxf(m, s[ps][h]);
      wm[h] = warp_max(m);
      const float ref = wm[h] == -INFINITY ? 0.f : wm[h];
      float l = 0.f;
#pragma unroll
      for (int ps = 0; ps < PASSES; ++ps) {
        const float e = __expf(s[ps][h] - ref);                    // 0 for masked positions
        sc[h][128 * ps + t] = e;
        l += e;
      }
      l = warp_sum(l);
      if (lane == 0) {
        wml[warp][h][0] = wm[h];
        wml[warp][h][1] = l;
      }
    }
    __syncwarp();

    // ---- P.V over the positions this warp scored: c0 + 128 pass + 32 warp + (0..31)
    float acc[HSUB][8];
#pragma unroll
    for (int h = 0; h < HSUB; ++h)
#pragma unroll
      for (int u = 0; u < 8; ++u) acc[h][u] = 0.f;
    constexpr int UNR = IPP < 8 ? IPP : 8;
#pragma unroll
    for (int ps = 0; ps < PASSES; ++ps) {
#pragma unroll
      for (int it0 = 0; it0 < IPP; it0 += UNR) {
        uint4 vv[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const int j = c0 + 128 * ps + 32 * warp + (it0 + u) * PPI + psub;
          if (VPRE) {
            vv[u] = vpre[it0 + u];
          } else {
            vv[u] = make_uint4(0u, 0u, 0u, 0u);
            if (j < p || (pre && j == p)) vv[u] = *reinterpret_cast<const uint4*>(vbase + (size_t)j * HD + d0);
          }
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const int jl = 128 * ps + 32 * warp + (it0 + u) * PPI + psub, j = c0 + jl;
          if (j > p) continue;
          float vf[8];
          if (!pre && j == p) {
#pragma unroll
            for (int k = 0; k < 8; ++k) vf[k] = vn[d0 + k];
          } else {
            const uint32_t w[4] = {vv[u].x, vv[u].y, vv[u].z, vv[u].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
              vf[2 * k] = f.x;
              vf[2 * k + 1] = f.y;
            }
          }
#pragma unroll
          for (int h = 0; h < HSUB; ++h) {
            const float e = sc[h][jl];
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[h][k] = fmaf(e, vf[k], acc[h][k]);
          }
        }
      }
    }
#pragma unroll
    for (int h = 0; h < HSUB; ++h)
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float a = acc[h][k];
#pragma unroll
        for (int o = 16; o >= LPR; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        acc[h][k] = a;
      }
    if (psub == 0) {
#pragma unroll
      for (int h = 0; h < HSUB; ++h)
#pragma unroll
        for (int k = 0; k < 8; ++k) red_o[warp][h][d0 + k] = acc[h][k];
    }
    __syncthreads();
    stamp();                                                        // 2: scores and P.V of the chunk done
    // ---- the four warps' partials -> this chunk's partial (fixed warp order), pushed into the combiner CTA
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // pairs with the arrive at the top
    uint32_t r_o, r_ml;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r_o) : "r"((uint32_t)__cvta_generic_to_shared(&comb_o[chunk][0][0])), "r"(0));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r_ml) : "r"((uint32_t)__cvta_generic_to_shared(&comb_ml[chunk][0][0])), "r"(0));
    for (int e = t; e < HSUB * HD; e += AT) {
      const int hl = e / HD, d = e - hl * HD;
      float M = wml[0][hl][0];
#pragma unroll
      for (int w = 1; w < NW; ++w) M = fmaxf(M, wml[w][hl][0]);     // finite: position c0 <= p is valid
      float o = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const float f = __expf(wml[w][hl][0] - M);                  // -inf -> 0
        o += red_o[w][hl][d] * f;
        l += wml[w][hl][1] * f;
      }
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(r_o + (uint32_t)(e * 4)), "f"(o) : "memory");
      if (d == 0) {
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(r_ml + (uint32_t)(hl * 8)), "f"(M) : "memory");
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(r_ml + (uint32_t)(hl * 8 + 4)), "f"(l) : "memory");
      }
    }
  } else {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  cluster_sync_all();                                               // every active chunk's partials are in the combiner
  stamp();                                                          // 3: cluster barrier passed
  if (chunk != 0) return;
  // chunk order, so the result does not depend on timing; every thread derives the weights itself (a few exps) instead
  // of a second block-wide exchange
  for (int e = t; e < nh * HD; e += AT) {
    const int hl = e / HD, d = e - hl * HD;
    float M = -INFINITY;
    for (int c = 0; c < nact; ++c) M = fmaxf(M, comb_ml[c][hl][0]);
    float o = 0.f, L = 0.f;
    for (int c = 0; c < nact; ++c) {
      const float w = __expf(comb_ml[c][hl][0] - M);
      L += comb_ml[c][hl][1] * w;
      o += comb_o[c][hl][d] * w;
    }
    out[(head0 + hl) * HD + d] = __float2half_rn(o / L);
  }
  stamp();                                                          // 4: combined (first CTA of the cluster only)
}

template <int HD, int HSUB>
int launch_cluster_passes(int passes, dim3 grid, cudaStream_t st, const __half* qkv, const float* cosT, const float* sinT,
                          const int64_t* pos, __half* kc, __half* vc, __half* out, int NH, int NKV, int GRP, int nsub,
                          int max_len, float scale, int pre) {
  cudaError_t e;
  unsigned long long* trace = trace_slot(2, (int)(grid.x * grid.y * grid.z));
  if (passes == 1)
    e = launch_pdl_cluster(attn_decode_cluster_kernel<HD, HSUB, 1>, grid, dim3(AT), 0, st, NCL, 1, qkv, cosT, sinT, pos, kc, vc,
                           out, NH, NKV, GRP, nsub, max_len, scale, pre, trace);
  else if (passes == 2)
    e = launch_pdl_cluster(attn_decode_cluster_kernel<HD, HSUB, 2>, grid, dim3(AT), 0, st, NCL, 1, qkv, cosT, sinT, pos, kc, vc,
                           out, NH, NKV, GRP, nsub, max_len, scale, pre, trace);
  else
    e = launch_pdl_cluster(attn_decode_cluster_kernel<HD, HSUB, 4>, grid, dim3(AT), 0, st, NCL, 1, qkv, cosT, sinT, pos, kc, vc,
                           out, NH, NKV, GRP, nsub, max_len, scale, pre, trace);
  return check_launch(e, "attn_decode");
}

template <int HD>
int launch_cluster(int hsub, int passes, dim3 grid, cudaStream_t st, const __half* qkv, const float* cosT, const float* sinT,
                   const int64_t* pos, __half* kc, __half* vc, __half* out, int NH, int NKV, int GRP, int nsub, int max_len,
                   float scale, int pre) {
  switch (hsub) {
    case 1: return launch_cluster_passes<HD, 1>(passes, grid, st, qkv, cosT, sinT, pos, kc, vc, out, NH, NKV, GRP, nsub, max_len, scale, pre);
    case 2: return launch_cluster_passes<HD, 2>(passes, grid, st, qkv, cosT, sinT, pos, kc, vc, out, NH, NKV, GRP, nsub, max_len, scale, pre);
    case 3: return launch_cluster_passes<HD, 3>(passes, grid, st, qkv, cosT, sinT, pos, kc, vc, out, NH, NKV, GRP, nsub, max_len, scale, pre);
    default: return launch_cluster_passes<HD, 4>(passes, grid, st, qkv, cosT, sinT, pos, kc, vc, out, NH, NKV, GRP, nsub, max_len, scale, pre);
  }
}

size_t align16(size_t v) { return (v + 15) & ~(size_t)15; }

template <int HD>
int dispatch_grp(int grp, dim3 grid, cudaStream_t st, const __half* qkv, const float* cosT, const float* sinT,
                 const int64_t* pos, __half* kc, __half* vc, __half* out, int NH, int NKV, int max_len, float scale,
                 unsigned* cnt, float* ml, float* po, int NC) {
#define Q4B_ATTN_CASE(G)                                                                                         \
  case G:                                                                                                        \
    launch_pdl(attn_decode_kernel<HD, G>, grid, dim3(AT), 0, st, qkv, cosT, sinT, pos, kc, vc, out, NH, NKV, max_len, \
               scale, cnt, ml, po, NC);                                                                          \
    return Q4B_OK;
  switch (grp) {
    Q4B_ATTN_CASE(1) Q4B_ATTN_CASE(2) Q4B_ATTN_CASE(3) Q4B_ATTN_CASE(4) Q4B_ATTN_CASE(5) Q4B_ATTN_CASE(6)
    Q4B_ATTN_CASE(7) Q4B_ATTN_CASE(8)
    default: return Q4B_E_SHAPE;
  }
#undef Q4B_ATTN_CASE
}

}  // namespace

size_t attn_decode_workspace(int B, int NH, int HD, int max_len) {
  if (B <= 0 || NH <= 0 || HD <= 0 || max_len <= 0) return 0;
  const size_t NC = (size_t)(max_len + CH - 1) / CH;
  return align16((size_t)B * NH * 4) + align16((size_t)B * NH * NC * 2 * 4) + (size_t)B * NH * NC * HD * 4;
}

int attn_decode_mma(const void*, const float*, const float*, const int64_t*, void*, void*, void*, int, int, int, int, float,
                    cudaStream_t, void* xq = nullptr, void* xd = nullptr);
bool attn_cached_fits(int NH, int NKV, int HD, int max_len);
int attn_cached(const void*, const int64_t*, const void*, const void*, void*, int, int, int, float, cudaStream_t, int B = 1,
                const float* cosT = nullptr, const float* sinT = nullptr, void* xq = nullptr, void* xd = nullptr);

// which kernel serves several sequences: 0 = the shared-memory-resident cached form where the context fits it (default),
// 1 = always the streaming tensor-core kernel of attn_decode_mma.cu
static int g_batched_kernel = 0;
void attn_batched_kernel(int which) { g_batched_kernel = which; }

// pre != 0 (one sequence, max_len <= 4096 only): q arrives rotated and position pos is already in the cache (the fused
// epilogue of the QKV projection did both); cosT / sinT / ws may then be null.
int attn_decode(const void* qkv, const float* cosT, const float* sinT, const int64_t* pos, void* kc, void* vc, void* out,
                int B, int NH, int NKV, int HD, int max_len, float scale, void* ws, size_t ws_bytes, cudaStream_t st, int pre) {
  if (pre) {
    if (B != 1 || max_len > NCL * 128 * 4) return fail(Q4B_E_SHAPE, "attn_decode: the cached form serves one sequence with max_len <= 4096");
    if (NH <= 0 || NKV <= 0 || max_len <= 0 || (NH % NKV) || NH / NKV > 8 || (HD != 64 && HD != 128))
      return fail(Q4B_E_SHAPE, "attn_decode: need HD in {64,128}, NH a multiple of NKV, NH/NKV <= 8");
    if (!qkv || !pos || !kc || !vc || !out || !aligned16(kc) || !aligned16(vc)) return fail(Q4B_E_ALIGN, "attn_decode: null or misaligned pointer");
    // contexts up to 2048 with head_dim 128: the shared-memory-resident tensor-core kernel (attn_decode_cached.cu)
    if (attn_cached_fits(NH, NKV, HD, max_len) && aligned16(qkv)) return attn_cached(qkv, pos, kc, vc, out, NH, NKV, max_len, scale, st);
    static const int hsub_for[9] = {1, 1, 2, 3, 2, 3, 2, 4, 4};
    const int GRP = NH / NKV, hsub = hsub_for[GRP], nsub = (GRP + hsub - 1) / hsub;
    const int passes = max_len <= NCL * 128 ? 1 : (max_len <= NCL * 256 ? 2 : 4);
    dim3 grid(NCL, NKV * nsub, 1);
    if (HD == 128)
      return launch_cluster<128>(hsub, passes, grid, st, (const __half*)qkv, cosT, sinT, pos, (__half*)kc, (__half*)vc,
                                 (__half*)out, NH, NKV, GRP, nsub, max_len, scale, 1);
    return launch_cluster<64>(hsub, passes, grid, st, (const __half*)qkv, cosT, sinT, pos, (__half*)kc, (__half*)vc,
                              (__half*)out, NH, NKV, GRP, nsub, max_len, scale, 1);
  }
  if (B <= 0 || NH <= 0 || NKV <= 0 || max_len <= 0 || (NH % NKV) || NH / NKV > 8 || (HD != 64 && HD != 128))
    return fail(Q4B_E_SHAPE, "attn_decode: need HD in {64,128}, NH a multiple of NKV, NH/NKV <= 8");
  if (!qkv || !cosT || !sinT || !pos || !kc || !vc || !out || !ws || !aligned16(kc) || !aligned16(vc) || !aligned16(ws))
    return fail(Q4B_E_ALIGN, "attn_decode: null or misaligned pointer");
  if (ws_bytes < attn_decode_workspace(B, NH, HD, max_len)) return fail(Q4B_E_WORKSPACE, "attn_decode: workspace too small");
  // Several sequences: the tensor-core kernel that reads K/V once per KV group (throughput); one sequence keeps the
  // latency-oriented kernels below.
  if (B >= 2 && HD == 128 && aligned16(qkv)) {
    if (g_batched_kernel == 0 && attn_cached_fits(NH, NKV, HD, max_len))
      return attn_cached(qkv, pos, kc, vc, out, NH, NKV, max_len, scale, st, B, cosT, sinT);
    return attn_decode_mma(qkv, cosT, sinT, pos, kc, vc, out, B, NH, NKV, max_len, scale, st);
  }
  if (max_len <= NCL * 128 * 4) {
    // cluster path: 8 chunks of 128 / 256 / 512 positions; a head group is served by 1..4 CTAs
    static const int hsub_for[9] = {1, 1, 2, 3, 2, 3, 2, 4, 4};
    const int GRP = NH / NKV, hsub = hsub_for[GRP], nsub = (GRP + hsub - 1) / hsub;
    const int passes = max_len <= NCL * 128 ? 1 : (max_len <= NCL * 256 ? 2 : 4);
    dim3 grid(NCL, NKV * nsub, B);
    if (HD == 128)
      return launch_cluster<128>(hsub, passes, grid, st, (const __half*)qkv, cosT, sinT, pos, (__half*)kc, (__half*)vc,
                                 (__half*)out, NH, NKV, GRP, nsub, max_len, scale, 0);
    return launch_cluster<64>(hsub, passes, grid, st, (const __half*)qkv, cosT, sinT, pos, (__half*)kc, (__half*)vc,
                              (__half*)out, NH, NKV, GRP, nsub, max_len, scale, 0);
  }
  const int NC = (max_len + CH - 1) / CH;
  char* base = reinterpret_cast<char*>(ws);
  unsigned* cnt = reinterpret_cast<unsigned*>(base);
  float* ml = reinterpret_cast<float*>(base + align16((size_t)B * NH * 4));
  float* po = reinterpret_cast<float*>(base + align16((size_t)B * NH * 4) + align16((size_t)B * NH * NC * 2 * 4));
  dim3 grid(NC, NKV, B);
  int rc;
  if (HD == 128)
    rc = dispatch_grp<128>(NH / NKV, grid, st, (const __half*)qkv, cosT, sinT, pos, (__half*)kc, (__half*)vc, (__half*)out,
                           NH, NKV, max_len, scale, cnt, ml, po, NC);
  else
    rc = dispatch_grp<64>(NH / NKV, grid, st, (const __half*)qkv, cosT, sinT, pos, (__half*)kc, (__half*)vc, (__half*)out,
                          NH, NKV, max_len, scale, cnt, ml, po, NC);
  if (rc != Q4B_OK) return fail(rc, "attn_decode: unsupported head group");
  return check_launch("attn_decode");
}

// Decode attention whose output is also written as planar Q8_1.  Only the multi-sequence tensor-core kernel has the
// fused quantiser; other cases report Q4B_E_SHAPE and the caller quantises separately.
int attn_decode_q8(const void* qkv, const float* cosT, const float* sinT, const int64_t* pos, void* kc, void* vc, void* out,
                   void* xq, void* xd, int B, int NH, int NKV, int HD, int max_len, float scale, cudaStream_t st) {
  if (B < 2 || HD != 128 || NKV <= 0 || (NH % NKV) || NH / NKV > 8 || max_len <= 0) return Q4B_E_SHAPE;
  if (!qkv || !cosT || !sinT || !pos || !kc || !vc || !out || !xq || !xd || !aligned16(kc) || !aligned16(vc) || !aligned16(qkv))
    return fail(Q4B_E_ALIGN, "attn_decode_q8: null or misaligned pointer");
  // the shared-memory-resident kernel where the context fits it (its combine step quantises 32-dimension slices), else the
  // streaming kernel
  if (g_batched_kernel == 0 && attn_cached_fits(NH, NKV, HD, max_len))
    return attn_cached(qkv, pos, kc, vc, out, NH, NKV, max_len, scale, st, B, cosT, sinT, xq, xd);
  if (((NH / NKV) * HD) % 256) return Q4B_E_SHAPE;
  return attn_decode_mma(qkv, cosT, sinT, pos, kc, vc, out, B, NH, NKV, max_len, scale, st, xq, xd);
}

}  // namespace q4b
