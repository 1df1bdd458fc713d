// Decode attention of ONE sequence over an fp16 K/V cache that already holds the current position, with q already
// rotated: the attention half of ATTN4 (lab/qwen_kernels.py:548-603: s_j = (q . k_j) * scale, soft-max over j <= pos,
// out = round16(sum e_j v_j / sum e_j)); rotation and the cache append were done by the QKV projection's epilogue
// (gemv_mma.cu), as the reference's prefill path does it (lab/qwen_batched.py:1316-1362).
//
// Built for latency.  At batch 1 a layer's attention touches well under 1 MB; what costs is the chain of dependent
// round trips, so the kernel removes them one by one:
//   * the position and every cache row BELOW it were written by earlier decode steps, and the first launch of a decode
//     step (the embedding lookup) triggers its dependents only after its own dependency wait, so all work of earlier
//     steps is complete before any later launch of the step starts.  This kernel therefore reads the position and
//     copies its whole chunk of K and V rows into shared memory (cp.async, rows padded to 272 bytes) BEFORE its
//     dependency wait, while the QKV projection is still running;
//   * the context is cut into 8 equal chunks of the ACTUAL length (not of max_len), one CTA each, a thread-block
//     cluster per KV head; all query heads of the KV group form one 16-row MMA operand, so K and V are read once;
//   * after the wait only q (1.5 KB) and the row of the current position are fetched; S = Q K^T and O = P V run on
//     mma.sync.m16n8k16 (fp16 inputs, fp32 accumulation; P as two fp16 terms so the probabilities keep ~22 bits).
//     For S a warp owns 16 POSITIONS; the probabilities go through shared memory, and for O a warp owns 16 output
//     DIMENSIONS over all positions of the chunk, so the warps' outputs are disjoint and need no merge;
//   * chunks are combined by all eight CTAs at once: warp w PUSHES its 16 dimensions into CTA w's shared memory
//     (st.shared::cluster), every CTA pushes its (max, sum) pairs to all, and after ONE cluster barrier CTA j combines
//     dimensions 16 j .. 16 j + 15 of every head in chunk order: no workspace, no atomics, no remote loads, a sixteenth of
//     an output per thread.
#include "q4b_internal.h"

namespace q4b {

namespace {

constexpr int HD = 128;
constexpr int PITCH = HD * 2 + 16;             // bytes per staged row (conflict-free fragment reads)
constexpr int NCL = 8;                         // chunks = cluster size
constexpr int AT = 256, NW = AT / 32;
constexpr int MAXG = 8;                        // query heads per KV head
constexpr int MAX_CTX = 2048;                  // 8 chunks x 256 positions x 2 x 272 bytes of shared memory
constexpr int PPITCH = (256 + 8) * 2;          // bytes per row of the staged probabilities (conflict-free fragment reads)

__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
// 16 bytes global -> shared; `bytes` = 0 fills the destination with zeros instead (rows beyond the valid range)
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(bytes)
               : "memory");
}

// 8 fp16 values of a rotated head: `own` holds dimensions 8 cc .. 8 cc + 7, `other` the same offsets in the other half of
// the head (d +- 64); cs / sn are the 64 cosines / sines of the position.  NeoX pairs (d, d + 64), rounded to fp16.
__device__ __forceinline__ uint4 rotate8(uint4 own, uint4 other, int cc, const float* cs, const float* sn) {
  const __half2* a2 = reinterpret_cast<const __half2*>(&own);
  const __half2* b2 = reinterpret_cast<const __half2*>(&other);
  uint4 r;
  uint32_t* rw = reinterpret_cast<uint32_t*>(&r);
  const int d0 = (cc & 7) * 8;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = __half22float2(a2[i]), b = __half22float2(b2[i]);
    float lo0, hi0, lo1, hi1;
    if (cc < 8) {                                    // own = first half (d), other = second half (d + 64)
      rope_pair(a.x, b.x, cs[d0 + 2 * i], sn[d0 + 2 * i], lo0, hi0);
      rope_pair(a.y, b.y, cs[d0 + 2 * i + 1], sn[d0 + 2 * i + 1], lo1, hi1);
      rw[i] = pack_h2(lo0, lo1);
    } else {
      rope_pair(b.x, a.x, cs[d0 + 2 * i], sn[d0 + 2 * i], lo0, hi0);
      rope_pair(b.y, a.y, cs[d0 + 2 * i + 1], sn[d0 + 2 * i + 1], lo1, hi1);
      rw[i] = pack_h2(hi0, hi1);
    }
  }
  return r;
}

// ROPE = false: q arrives rotated and the cache already holds the current position (batch-1 chain).
// ROPE = true:  the whole of ATTN4 (lab/qwen_kernels.py:517-605) for gridDim.z sequences: q and the new k are rotated here
//               from the biased fp16 QKV row, the CTA that owns the current position appends k / v to the cache (single
//               writer) and uses them from shared memory; the rotation tables' row is fetched ahead of the wait.
template <bool ROPE>
__global__ void __launch_bounds__(AT, 2) attn_cached_kernel(const __half* qkv, const int64_t* posp, __half* kc, __half* vc,
                                                            __half* out, int NH, int NKV, int max_len, int cap, float scale_log2e,
                                                            unsigned long long* trace, const float* cosT, const float* sinT,
                                                            int8_t* xq, __half* xd) {
  extern __shared__ __align__(16) uint8_t sm[];
  __shared__ float s_cs[64], s_sn[64];
  {
    const size_t b = blockIdx.z;                     // sequence
    qkv += b * (size_t)(NH + 2 * NKV) * HD;
    posp += b;
    kc += b * (size_t)NKV * max_len * HD;
    vc += b * (size_t)NKV * max_len * HD;
    if (out) out += b * (size_t)NH * HD;
    if (xq) {
      xq += b * (size_t)NH * HD;
      xd += b * (size_t)NH * (HD / 32);
    }
  }
  const bool q8out = xq != nullptr;                  // combine in 32-dimension slices (CTAs 0..3) and quantise them
  uint8_t* sQ = sm;                                  // [16][PITCH]   q heads of the group (rows >= GRP zero)
  uint8_t* sK = sQ + 16 * PITCH;                     // [cap][PITCH]
  uint8_t* sV = sK + (size_t)cap * PITCH;            // [cap][PITCH]
  __shared__ float wmax[NW][MAXG], wsum[NW][MAXG];   // per warp and head: maximum score, sum of probabilities (base 2)
  // combiner: this CTA owns output dimensions 16 c .. 16 c + 15; every chunk pushes its share and its (max, sum) here
  __shared__ __align__(16) float comb_o[NCL][MAXG][32];   // [chunk][head][16 dims; 32 with the quantiser fused in]
  __shared__ float comb_ml[NCL][MAXG][2];

  const int t = threadIdx.x, warp = t >> 5, lane = t & 31, g = lane >> 2, tq = lane & 3;
  const int c = blockIdx.x, kvh = blockIdx.y;
  unsigned long long* tr = (trace && t == 0) ? trace + (size_t)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 : nullptr;
  int tri = 0;
  auto stamp = [&]() {
    if (tr && tri < 15) {
      unsigned long long gt;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
      tr[tri++] = gt;
      tr[15] = (unsigned long long)tri;
    }
  };
  stamp();                                           // 0: start
  pdl_launch_dependents();
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");   // "this CTA exists" (paired with the wait before the push)
  const int GRP = NH / NKV;
  // the position belongs to the state of earlier steps (see the header): readable ahead of the wait
  int p = (int)posp[0];
  p = p < 0 ? 0 : (p >= max_len ? max_len - 1 : p);
  const int n = p + 1;                               // positions 0 .. p
  int chunk = ((n + NCL - 1) / NCL + 15) & ~15;      // equal chunks of the actual context, whole 16-position warp tiles
  if (chunk > cap) chunk = cap;                      // (cannot happen while max_len <= 8 cap; keeps the copies in bounds)
  const int c0 = c * chunk, c1 = min(c0 + chunk, n); // this CTA: positions c0 .. c1 - 1
  const bool active = c0 < n;
  const int nact = (n + chunk - 1) / chunk;
  const int rows = active ? c1 - c0 : 0;
  const int rows16 = (rows + 15) & ~15;
  const __half* kbase = kc + (size_t)kvh * max_len * HD;
  const __half* vbase = vc + (size_t)kvh * max_len * HD;
  // ---- ahead of the wait: rows below the current position -> shared memory; the tail of the last warp tile is zeroed
  // (a masked probability times a stale NaN would still be a NaN)
  for (int e = t; e < rows16 * (HD / 8); e += AT) {
    const int r = e >> 4, cc = e & 15;
    const int j = c0 + r;
    const bool ld = j < p;                           // row p itself arrives after the wait
    const size_t off = (size_t)(ld ? j : 0) * HD + cc * 8;
    cp_async16(sK + (size_t)r * PITCH + cc * 16, kbase + off, ld ? 16 : 0);
    cp_async16(sV + (size_t)r * PITCH + cc * 16, vbase + off, ld ? 16 : 0);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  if (ROPE) {
    if (t < 64) {
      s_cs[t] = cosT[(size_t)p * 64 + t];
      s_sn[t] = sinT[(size_t)p * 64 + t];
    }
    __syncthreads();
  }
  stamp();                                           // 1: cache rows requested
  pdl_wait();
  stamp();                                           // 2: predecessor complete
  if (active) {
    // ---- q heads of the group (already rotated) and the row of the current position: both requested at once
    const bool mine = p >= c0 && p < c1 && t < 32;            // 16 threads carry the K row of position p, 16 its V row
    uint4 qv = make_uint4(0u, 0u, 0u, 0u), pv = make_uint4(0u, 0u, 0u, 0u);
    {
      const int hl = t >> 4, cc = t & 15;
      if (!ROPE) {
        if (hl < GRP) qv = *reinterpret_cast<const uint4*>(qkv + (size_t)(kvh * GRP + hl) * HD + cc * 8);
        if (mine) pv = *reinterpret_cast<const uint4*>((t < 16 ? kbase : vbase) + (size_t)p * HD + cc * 8);
      } else {
        uint4 qo = make_uint4(0u, 0u, 0u, 0u), po = make_uint4(0u, 0u, 0u, 0u);
        if (hl < GRP) {
          const __half* qh = qkv + (size_t)(kvh * GRP + hl) * HD;
          qv = *reinterpret_cast<const uint4*>(qh + cc * 8);
          qo = *reinterpret_cast<const uint4*>(qh + (cc ^ 8) * 8);
        }
        if (mine) {
          const __half* nh = qkv + (size_t)(t < 16 ? NH + kvh : NH + NKV + kvh) * HD;
          pv = *reinterpret_cast<const uint4*>(nh + cc * 8);
          if (t < 16) po = *reinterpret_cast<const uint4*>(nh + (cc ^ 8) * 8);
        }
        if (hl < GRP) qv = rotate8(qv, qo, cc, s_cs, s_sn);
        if (mine) {
          if (t < 16) pv = rotate8(pv, po, cc, s_cs, s_sn);
          *reinterpret_cast<uint4*>((t < 16 ? kc : vc) + ((size_t)kvh * max_len + p) * HD + cc * 8) = pv;   // the append
        }
      }
      *reinterpret_cast<uint4*>(sQ + hl * PITCH + cc * 16) = qv;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");      // this thread's copies have landed (zero-filled slot of row p too)
    __syncthreads();                                          // ... and everyone's; the plain stores below come after them
    if (mine) *reinterpret_cast<uint4*>((t < 16 ? sK : sV) + (size_t)(p - c0) * PITCH + (t & 15) * 16) = pv;
    __syncthreads();
    stamp();                                         // 3: operands staged
    uint32_t qa[8][2];                               // rows g of the A operand (rows g + 8 are zero)
    {
      const uint8_t* r0 = sQ + g * PITCH;
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        qa[s][0] = *reinterpret_cast<const uint32_t*>(r0 + (16 * s + 2 * tq) * 2);
        qa[s][1] = *reinterpret_cast<const uint32_t*>(r0 + (16 * s + 2 * tq + 8) * 2);
      }
    }
    // ---- S = Q K^T: warp w scores positions 16 w .. 16 w + 15 (and + 128 k for chunks beyond 128 rows)
    constexpr int MAXT = 2;                          // 16-position tiles per warp: chunks of up to 256 rows
    float sacc[MAXT][2][4];
    float mx = -INFINITY;                            // running maximum of head g over this warp's positions
#pragma unroll
    for (int it = 0; it < MAXT; ++it) {
      const int w0 = 16 * warp + 128 * it;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        sacc[it][j][0] = sacc[it][j][1] = sacc[it][j][2] = sacc[it][j][3] = 0.f;
        if (w0 < rows) {
          const uint8_t* kr = sK + (size_t)(w0 + 8 * j + g) * PITCH;
#pragma unroll
          for (int s = 0; s < 8; ++s) {
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kr + (16 * s + 2 * tq) * 2);
            const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kr + (16 * s + 2 * tq + 8) * 2);
            mma16816(sacc[it][j], qa[s][0], 0u, qa[s][1], 0u, b0, b1);
          }
        }
        const int key = w0 + 8 * j + 2 * tq;
        sacc[it][j][0] = key < rows ? sacc[it][j][0] * scale_log2e : -INFINITY;
        sacc[it][j][1] = key + 1 < rows ? sacc[it][j][1] * scale_log2e : -INFINITY;
        mx = fmaxf(mx, fmaxf(sacc[it][j][0], sacc[it][j][1]));
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    if (tq == 0) wmax[warp][g] = mx;                 // -inf for a warp without a valid position
    __syncthreads();
    // ---- chunk maximum of head g, probabilities as two fp16 terms into shared memory (the A operand of P V)
    float M = wmax[0][g];                            // finite: position 0 of the chunk is valid
#pragma unroll
    for (int w = 1; w < NW; ++w) M = fmaxf(M, wmax[w][g]);
    uint8_t* sPh = sK;                               // [8 heads][PPITCH] fp16, over the K tile (every warp is done with it)
    uint8_t* sPl = sK + 8 * PPITCH;
    float ps = 0.f;
#pragma unroll
    for (int it = 0; it < MAXT; ++it) {
      const int w0 = 16 * warp + 128 * it;
      if (w0 < rows16) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const float p0 = exp2f(sacc[it][j][0] - M), p1 = exp2f(sacc[it][j][1] - M);   // masked -> 0
          ps += p0 + p1;
          const __half2 h = __floats2half2_rn(p0, p1);
          const float2 hf = __half22float2(h);
          const int col = w0 + 8 * j + 2 * tq;
          *reinterpret_cast<uint32_t*>(sPh + g * PPITCH + col * 2) = *reinterpret_cast<const uint32_t*>(&h);
          *reinterpret_cast<uint32_t*>(sPl + g * PPITCH + col * 2) = pack_h2(p0 - hf.x, p1 - hf.y);   // P keeps ~22 bits
        }
      }
    }
    ps += __shfl_xor_sync(0xffffffffu, ps, 1);
    ps += __shfl_xor_sync(0xffffffffu, ps, 2);
    if (tq == 0) wsum[warp][g] = ps;
    __syncthreads();
    stamp();                                         // 4: chunk scored
    // ---- O = (P_hi + P_lo) V: warp w owns output dimensions 16 w .. 16 w + 15 of every head, over all positions
    float o[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    for (int k0 = 0; k0 < rows16; k0 += 16) {
      const int mtx = lane >> 3, r = lane & 7;       // matrices: (positions 0-7 | 8-15) x (dims +0 | +8)
      const uint8_t* addr = sV + (size_t)(k0 + (mtx & 1) * 8 + r) * PITCH + (16 * warp + 8 * (mtx >> 1)) * 2;
      uint32_t b0, b1, b2, b3;
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                   : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                   : "r"((uint32_t)__cvta_generic_to_shared(addr)));
      const uint32_t ph0 = *reinterpret_cast<const uint32_t*>(sPh + g * PPITCH + (k0 + 2 * tq) * 2);
      const uint32_t ph1 = *reinterpret_cast<const uint32_t*>(sPh + g * PPITCH + (k0 + 2 * tq + 8) * 2);
      const uint32_t pl0 = *reinterpret_cast<const uint32_t*>(sPl + g * PPITCH + (k0 + 2 * tq) * 2);
      const uint32_t pl1 = *reinterpret_cast<const uint32_t*>(sPl + g * PPITCH + (k0 + 2 * tq + 8) * 2);
      mma16816(o[0], ph0, 0u, ph1, 0u, b0, b1);
      mma16816(o[1], ph0, 0u, ph1, 0u, b2, b3);
      mma16816(o[0], pl0, 0u, pl1, 0u, b0, b1);
      mma16816(o[1], pl0, 0u, pl1, 0u, b2, b3);
    }
    // ---- push: this warp's 16 dimensions to CTA `warp`, the chunk's (max, sum) of every head to every CTA
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // pairs with the arrive at the top
    if (g < GRP) {
      uint32_t r_o;
      // owner of this warp's 16 dimensions: CTA `warp`, or with the quantiser fused in CTA warp / 2 (a Q8_1 block is 32)
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r_o)
                   : "r"((uint32_t)__cvta_generic_to_shared(&comb_o[c][g][q8out ? 16 * (warp & 1) : 0])), "r"(q8out ? warp >> 1 : warp));
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(r_o + (uint32_t)((8 * nt + 2 * tq) * 4)), "f"(o[nt][0]) : "memory");
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(r_o + (uint32_t)((8 * nt + 2 * tq + 1) * 4)), "f"(o[nt][1]) : "memory");
      }
    }
    if (t < NCL * MAXG) {                            // thread (target CTA, head)
      const int tgt = t >> 3, hl = t & 7;
      float Mh = wmax[0][hl], lh = 0.f;
#pragma unroll
      for (int w = 1; w < NW; ++w) Mh = fmaxf(Mh, wmax[w][hl]);
#pragma unroll
      for (int w = 0; w < NW; ++w) lh += wsum[w][hl];
      uint32_t r_ml;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r_ml) : "r"((uint32_t)__cvta_generic_to_shared(&comb_ml[c][hl][0])), "r"(tgt));
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(r_ml), "f"(Mh) : "memory");
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(r_ml + 4u), "f"(lh) : "memory");
    }
  } else {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  cluster_sync_all();                                // every active chunk's partials are in the combiners
  stamp();                                           // 5: cluster barrier passed
  if (q8out) {
    // CTAs 0..3 own dimensions 32 c .. 32 c + 31 of every head: warp = head, lane = dimension = one Q8_1 block.  Same sums in
    // the same chunk order as below, then the quantiser of quant_q8_1.cu on the rounded output.
    if (c < 4) {
      const int hl = t >> 5, dd = t & 31;
      if (hl < GRP) {
        float Mx = -INFINITY;
#pragma unroll
        for (int cc = 0; cc < NCL; ++cc) Mx = fmaxf(Mx, cc < nact ? comb_ml[cc][hl][0] : -INFINITY);
        float ov = 0.f, L = 0.f;
#pragma unroll
        for (int cc = 0; cc < NCL; ++cc) {
          const bool on = cc < nact;
          const float w = exp2f((on ? comb_ml[cc][hl][0] : -INFINITY) - Mx);
          L += (on ? comb_ml[cc][hl][1] : 0.f) * w;
          ov += (on ? comb_o[cc][hl][dd] : 0.f) * w;
        }
        const __half y16 = __float2half_rn(ov / L);
        const float y = __half2float(y16);
        const float d = warp_max(fabsf(y)) / 127.f;
        const int q = d > 0.f ? __float2int_rn(y / d) : 0;
        const size_t at = (size_t)(kvh * GRP + hl) * HD + 32 * c + dd;
        xq[at] = (int8_t)q;
        if (dd == 0) xd[at >> 5] = __float2half_rn(d);
        if (out) out[at] = y16;
      }
    }
    stamp();
    return;
  }
  // chunk order, so the result does not depend on timing; thread (head, dimension) of this CTA's 16 dimensions
  if (t < MAXG * 16) {
    const int hl = t >> 4, dd = t & 15;
    if (hl < GRP) {
      float mc[NCL], lc[NCL], oc[NCL];
#pragma unroll
      for (int cc = 0; cc < NCL; ++cc) {
        const bool on = cc < nact;
        mc[cc] = on ? comb_ml[cc][hl][0] : -INFINITY;
        lc[cc] = on ? comb_ml[cc][hl][1] : 0.f;
        oc[cc] = on ? comb_o[cc][hl][dd] : 0.f;
      }
      float Mx = mc[0];
#pragma unroll
      for (int cc = 1; cc < NCL; ++cc) Mx = fmaxf(Mx, mc[cc]);
      float ov = 0.f, L = 0.f;
#pragma unroll
      for (int cc = 0; cc < NCL; ++cc) {
        const float w = exp2f(mc[cc] - Mx);
        L += lc[cc] * w;
        ov += oc[cc] * w;
      }
      out[(size_t)(kvh * GRP + hl) * HD + 16 * c + dd] = __float2half_rn(ov / L);
    }
  }
  stamp();                                           // 6: combined
}

}  // namespace

// Largest context the shared-memory-resident form covers; longer caches use the chunked cluster kernel of attn_decode.cu.
bool attn_cached_fits(int NH, int NKV, int HD, int max_len) {
  return HD == 128 && NKV > 0 && NH % NKV == 0 && NH / NKV <= MAXG && max_len > 0 && max_len <= MAX_CTX;
}

// B = 1 with cosT == nullptr: the cached form (q rotated, row appended by the caller).  cosT / sinT given: RoPE and the
// append happen inside, for B sequences (qkv [B, (NH + 2 NKV) 128], pos [B], cache [B, NKV, max_len, 128], out [B, NH 128]).
int attn_cached(const void* qkv, const int64_t* pos, const void* kc, const void* vc, void* out, int NH, int NKV, int max_len,
                float scale, cudaStream_t st, int B, const float* cosT, const float* sinT, void* xq, void* xd) {
  if (!attn_cached_fits(NH, NKV, HD, max_len)) return fail(Q4B_E_SHAPE, "attn_decode_cached: needs head_dim 128, NH/NKV <= 8, max_len <= 2048");
  if (B < 1 || B > 65535 || (B > 1 && !cosT)) return fail(Q4B_E_SHAPE, "attn_decode_cached: 1 <= B, several sequences need the rotation tables");
  if (!qkv || !pos || !kc || !vc || (!out && !xq) || (xq && !xd) || !aligned16(qkv) || !aligned16(kc) || !aligned16(vc) || (cosT && !sinT))
    return fail(Q4B_E_ALIGN, "attn_decode_cached: null or misaligned pointer");
  int cap = ((max_len + NCL - 1) / NCL + 15) & ~15;  // positions per CTA at the longest context
  if (cap < 128) cap = 128;                          // the K tile's space later holds the per-warp partials (32 KB)
  const size_t smem = (size_t)(16 + 2 * cap) * PITCH;
  const void* kern = cosT ? reinterpret_cast<const void*>(&attn_cached_kernel<true>) : reinterpret_cast<const void*>(&attn_cached_kernel<false>);
  if (!cosT) prefer_max_shared(kern);                // the batch-1 chain shares one carve-out (see q4b_internal.h)
  if (cudaError_t e = ensure_dynamic_smem(kern, smem); e != cudaSuccess) {
    set_cuda_error(e, "attn_decode_cached");
    return Q4B_E_CUDA;
  }
  unsigned long long* trace = trace_slot(2, NCL * NKV * B);
  const float scale_log2e = scale * 1.4426950408889634f;
  __half* kcw = reinterpret_cast<__half*>(const_cast<void*>(kc));
  __half* vcw = reinterpret_cast<__half*>(const_cast<void*>(vc));
  cudaError_t e;
  if (cosT)
    e = launch_pdl_cluster(attn_cached_kernel<true>, dim3(NCL, NKV, B), dim3(AT), smem, st, NCL, 1, (const __half*)qkv, pos, kcw, vcw,
                           (__half*)out, NH, NKV, max_len, cap, scale_log2e, trace, cosT, sinT, (int8_t*)xq, (__half*)xd);
  else
    e = launch_pdl_cluster(attn_cached_kernel<false>, dim3(NCL, NKV, B), dim3(AT), smem, st, NCL, 1, (const __half*)qkv, pos, kcw, vcw,
                           (__half*)out, NH, NKV, max_len, cap, scale_log2e, trace, cosT, sinT, (int8_t*)xq, (__half*)xd);
  return check_launch(e, "attn_decode_cached");
}

}  // namespace q4b
