// Decode attention for batches of sequences: one new token per sequence against its fp16 K/V cache, on the fp16
// tensor cores.  Throughput-oriented sibling of attn_decode.cu (which is built for the latency of a single sequence).
//
// Reference arithmetic: ATTN4 (lab/qwen_kernels.py:517-605) as the batched engine launches it per sequence
// (`batchify`d, scripts/qwen_batched_decode.py:70-83, 116-121): q and the new k are rotated (rotate-half pairs d, d + 64) from the fp16 biased QKV
// row and rounded to fp16, k/v are appended at posp[b], scores = q.k * scale over positions 0..pos, fp32 soft-max,
// out = P.V rounded to fp16.
//
// Shape: grid (8 chunks, KV heads, sequences), the 8 chunk CTAs of one (sequence, KV head) form a thread-block
// cluster.  A CTA streams its chunk of the cache through shared memory in 64-position tiles (cp.async, two stages,
// rows padded to 272 bytes so that fragment reads are conflict-free).  All query heads of the KV group form ONE
// 16-row MMA operand (rows beyond the group are zero), so K and V are read once per group, not once per head:
//   S = Q K^T    mma.sync.m16n8k16, fp16 x fp16 -> fp32 (exact products of the fp16 inputs)
//   O += P V     P split as P_hi + P_lo (two fp16 terms, so the probabilities keep ~22 bits; with one term the output
//                moved by ~1e-4, enough to flip fp16 roundings downstream) x V via ldmatrix.trans
// with an fp32 online soft-max in base 2 per warp (a warp owns 16 positions of every tile).  Warps are merged in shared
// memory, chunks through distributed shared memory in chunk order, each CTA of the cluster writing an eighth of the outputs.
#include "q4b_internal.h"

namespace q4b {

namespace {

constexpr int HD = 128, HALF = 64;
constexpr int TILE = 64;                       // positions per tile (4 warps x 16)
constexpr int PITCH = HD * 2 + 16;             // bytes per staged row
constexpr int NCL = 8;                         // chunks per (sequence, KV head) = cluster size
constexpr int AT = 128, NW = 4;
constexpr int MAXG = 8;                        // query heads per KV head

__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

constexpr size_t STAGE = (size_t)TILE * PITCH;                 // one K or V tile
constexpr int NSTG = 1;                                        // tile buffers per CTA (other CTAs of the SM cover the load latency)
constexpr size_t DYN_SMEM = 16 * PITCH + 2 * NSTG * STAGE;     // Q rows, K tiles, V tiles

__global__ void __launch_bounds__(AT, 4) attn_decode_mma_kernel(const __half* qkv, const float* __restrict__ cosT,
                                                             const float* __restrict__ sinT, const int64_t* posp, __half* kc,
                                                             __half* vc, __half* out, int NH, int NKV, int max_len, int chunk,
                                                             float scale_log2e, unsigned long long* trace, int8_t* xq, __half* xd) {
  extern __shared__ __align__(16) uint8_t sm[];
  uint8_t* sQ = sm;                           // [16][PITCH]
  uint8_t* sK = sQ + 16 * PITCH;              // [2][TILE][PITCH]
  uint8_t* sV = sK + NSTG * STAGE;            // [NSTG][TILE][PITCH]
  __shared__ __align__(16) __half knew[HD], vnew[HD];
  __shared__ __align__(16) float part_o[MAXG][HD];   // this chunk: unnormalised output per head
  __shared__ float part_ml[MAXG][2];                 // (max, sum) in base-2 units
  __shared__ float wml[NW][MAXG][2];
  __shared__ float pml[MAXG][NCL][2];
  __shared__ float wgt[MAXG][NCL + 1];

  const int t = threadIdx.x, warp = t >> 5, lane = t & 31, g = lane >> 2, tq = lane & 3;
  const int c = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  // optional timeline: 16 %globaltimer stamps per CTA (thread 0), last entry = number of stamps
  unsigned long long* tr = (trace && t == 0) ? trace + (size_t)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 : nullptr;
  int tri = 0;
  auto stamp = [&]() {
    if (tr && tri < 15) {
      unsigned long long gt;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
      tr[tri++] = gt;
    }
  };
  stamp();                                     // 0: start
  pdl_launch_dependents();
  pdl_wait();
  stamp();                                     // 1: predecessor complete
  const int GRP = NH / NKV;
  int p = (int)posp[b];
  p = p < 0 ? 0 : (p >= max_len ? max_len - 1 : p);
  const int c0 = c * chunk;
  const bool active = c0 <= p;
  const int nact = p / chunk + 1;
  __half* kbase = kc + ((size_t)b * NKV + kvh) * (size_t)max_len * HD;
  __half* vbase = vc + ((size_t)b * NKV + kvh) * (size_t)max_len * HD;
  const int ntile = active ? (min(p, c0 + chunk - 1) - c0) / TILE + 1 : 0;

  auto issue_tile = [&](int i) {               // tile i of this chunk -> stage i & 1
    uint8_t* dk = sK + (size_t)(i % NSTG) * STAGE;
    uint8_t* dv = sV + (size_t)(i % NSTG) * STAGE;
    const int t0 = c0 + i * TILE;
    for (int e = t; e < TILE * (HD / 8); e += AT) {
      const int r = e >> 4, cc = e & 15;
      const int j = min(t0 + r, max_len - 1);  // rows beyond the position are masked later; keep the address valid
      cp_async16(dk + r * PITCH + cc * 16, kbase + (size_t)j * HD + cc * 8);
      cp_async16(dv + r * PITCH + cc * 16, vbase + (size_t)j * HD + cc * 8);
    }
    cp_async_commit();
  };
  if (ntile > 0) issue_tile(0);                // the cache rows below the position do not depend on this token

  float o[16][2];                              // rows g of the 16-row operand: 16 dim tiles x 2 columns
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;

  if (active) {
    // ---- q rows of the group (rotated, fp16) as the A operand; the new k/v row
    const int QKV = (NH + 2 * NKV) * HD;
    const __half* row = qkv + (size_t)b * QKV;
    const float* cs = cosT + (size_t)p * HALF;
    const float* sn = sinT + (size_t)p * HALF;
    const bool has_new = p < c0 + chunk;
    for (int e = t; e < 16 * HALF; e += AT) {
      const int hl = e / HALF, d = e - hl * HALF;
      float lo = 0.f, hi = 0.f;
      if (hl < GRP) {
        const __half* qh = row + (size_t)(kvh * GRP + hl) * HD;
        const float x0 = __half2float(qh[d]), x1 = __half2float(qh[d + HALF]);
        lo = x0 * cs[d] - x1 * sn[d];
        hi = x1 * cs[d] + x0 * sn[d];
      }
      *reinterpret_cast<__half*>(sQ + hl * PITCH + d * 2) = __float2half_rn(lo);
      *reinterpret_cast<__half*>(sQ + hl * PITCH + (d + HALF) * 2) = __float2half_rn(hi);
    }
    if (has_new && t < HALF) {
      const __half* kh = row + (size_t)NH * HD + (size_t)kvh * HD;
      const float x0 = __half2float(kh[t]), x1 = __half2float(kh[t + HALF]);
      const __half klo = __float2half_rn(x0 * cs[t] - x1 * sn[t]), khi = __float2half_rn(x1 * cs[t] + x0 * sn[t]);
      const __half v0 = row[(size_t)(NH + NKV) * HD + (size_t)kvh * HD + t];
      const __half v1 = row[(size_t)(NH + NKV) * HD + (size_t)kvh * HD + t + HALF];
      knew[t] = klo;
      knew[t + HALF] = khi;
      vnew[t] = v0;
      vnew[t + HALF] = v1;
      kbase[(size_t)p * HD + t] = klo;                           // the only writer of row p of (b, kvh)
      kbase[(size_t)p * HD + t + HALF] = khi;
      vbase[(size_t)p * HD + t] = v0;
      vbase[(size_t)p * HD + t + HALF] = v1;
    }
    __syncthreads();
    stamp();                                                     // 2: q / new row prepared
    uint32_t qa[8][2];                                           // rows g (rows g + 8 of the operand are zero)
    {
      const uint8_t* r0 = sQ + g * PITCH;
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        qa[s][0] = *reinterpret_cast<const uint32_t*>(r0 + (16 * s + 2 * tq) * 2);
        qa[s][1] = *reinterpret_cast<const uint32_t*>(r0 + (16 * s + 2 * tq + 8) * 2);
      }
    }

    for (int i = 0; i < ntile; ++i) {
      if (NSTG == 2 && i + 1 < ntile) {
        issue_tile(i + 1);
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      const int t0 = c0 + i * TILE;
      uint8_t* tk = sK + (size_t)(i % NSTG) * STAGE;
      uint8_t* tv = sV + (size_t)(i % NSTG) * STAGE;
      if (p >= t0 && p < t0 + TILE) {                            // the new row goes into the staged tile directly
        if (t < 16) reinterpret_cast<uint4*>(tk + (p - t0) * PITCH)[t] = reinterpret_cast<const uint4*>(knew)[t];
        else if (t < 32) reinterpret_cast<uint4*>(tv + (p - t0) * PITCH)[t - 16] = reinterpret_cast<const uint4*>(vnew)[t - 16];
        __syncthreads();
      }
      // ---- S = Q K^T for this warp's 16 positions
      float sacc[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f;
        const uint8_t* kr = tk + (16 * warp + 8 * j + g) * PITCH;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kr + (16 * s + 2 * tq) * 2);
          const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kr + (16 * s + 2 * tq + 8) * 2);
          mma16816(sacc[j], qa[s][0], 0u, qa[s][1], 0u, b0, b1);
        }
      }
      // ---- mask, online soft-max (base 2) for row g
      float mx = m_run;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int key = t0 + 16 * warp + 8 * j + 2 * tq;
        sacc[j][0] = key <= p ? sacc[j][0] * scale_log2e : -INFINITY;
        sacc[j][1] = key + 1 <= p ? sacc[j][1] * scale_log2e : -INFINITY;
        mx = fmaxf(mx, fmaxf(sacc[j][0], sacc[j][1]));
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float ref = mx == -INFINITY ? 0.f : mx;             // nothing valid yet: exp2(-inf - 0) = 0
      const float cor = exp2f(m_run - ref);
      m_run = mx;
      float ps = 0.f;
      uint32_t ph[2], pl[2];                                     // A fragments (row g): k 2tq.. and k 2tq + 8..
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float p0 = exp2f(sacc[j][0] - ref), p1 = exp2f(sacc[j][1] - ref);
        ps += p0 + p1;
        const __half2 h = __floats2half2_rn(p0, p1);
        const float2 hf = __half22float2(h);
        ph[j] = *reinterpret_cast<const uint32_t*>(&h);
        pl[j] = pack_h2(p0 - hf.x, p1 - hf.y);                   // second fp16 term: P keeps ~22 bits through the MMA
      }
      l_run = l_run * cor + ps;                                  // per-lane partial; reduced over the quad at the end
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        o[j][0] *= cor;
        o[j][1] *= cor;
      }
      // ---- O += (P_hi + P_lo) V over the warp's 16 positions
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        const int mtx = lane >> 3, r = lane & 7;
        const uint8_t* addr = tv + (16 * warp + (mtx & 1) * 8 + r) * PITCH + (8 * (j + (mtx >> 1))) * 2;
        uint32_t b0, b1, b2, b3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                     : "r"((uint32_t)__cvta_generic_to_shared(addr)));
        float a0[4] = {o[j][0], o[j][1], 0.f, 0.f}, a1[4] = {o[j + 1][0], o[j + 1][1], 0.f, 0.f};
        mma16816(a0, ph[0], 0u, ph[1], 0u, b0, b1);
        mma16816(a0, pl[0], 0u, pl[1], 0u, b0, b1);
        mma16816(a1, ph[0], 0u, ph[1], 0u, b2, b3);
        mma16816(a1, pl[0], 0u, pl[1], 0u, b2, b3);
        o[j][0] = a0[0];
        o[j][1] = a0[1];
        o[j + 1][0] = a1[0];
        o[j + 1][1] = a1[1];
      }
      __syncthreads();                                           // the tile buffer is free again
      if (NSTG == 1 && i + 1 < ntile) issue_tile(i + 1);
      stamp();                                                   // 3..: tile done
    }
    // ---- merge the four warps (each saw a quarter of every tile)
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    float* wo = reinterpret_cast<float*>(sK);                    // [NW][MAXG][HD], the tiles are dead
    if (g < GRP) {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        *reinterpret_cast<float2*>(wo + ((size_t)warp * MAXG + g) * HD + 8 * j + 2 * tq) = make_float2(o[j][0], o[j][1]);
      if (tq == 0) {
        wml[warp][g][0] = m_run;
        wml[warp][g][1] = l_run;
      }
    }
    __syncthreads();
    for (int e = t; e < GRP * HD; e += AT) {
      const int hl = e / HD, d = e - hl * HD;
      float M = wml[0][hl][0];
#pragma unroll
      for (int w = 1; w < NW; ++w) M = fmaxf(M, wml[w][hl][0]);
      const float Mr = M == -INFINITY ? 0.f : M;
      float ov = 0.f, lv = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const float f = exp2f(wml[w][hl][0] - Mr);
        ov += wo[((size_t)w * MAXG + hl) * HD + d] * f;
        lv += wml[w][hl][1] * f;
      }
      part_o[hl][d] = ov;
      if (d == 0) {
        part_ml[hl][0] = M;
        part_ml[hl][1] = lv;
      }
    }
    stamp();                                                     // warps merged
  }
  cluster_sync_all();                                            // every chunk's partials are in place
  stamp();                                                       // cluster barrier passed
  // ---- merge of the chunks, spread over the cluster: every CTA reads all (max, sum) pairs and writes 1/8 of the outputs
  {
    if (t < MAXG * NCL) {
      const int hl = t / NCL, cc = t - hl * NCL;
      if (hl < GRP && cc < nact) {
        pml[hl][cc][0] = ld_peer_f32(&part_ml[hl][0], (uint32_t)cc);
        pml[hl][cc][1] = ld_peer_f32(&part_ml[hl][1], (uint32_t)cc);
      }
    }
    __syncthreads();
    if (t < GRP) {
      float M = -INFINITY;
      for (int cc = 0; cc < nact; ++cc) M = fmaxf(M, pml[t][cc][0]);
      float L = 0.f;
      for (int cc = 0; cc < nact; ++cc) {
        const float w = exp2f(pml[t][cc][0] - M);
        wgt[t][cc] = w;
        L += pml[t][cc][1] * w;
      }
      wgt[t][NCL] = L;
    }
    __syncthreads();
    const size_t head0 = (size_t)b * NH + (size_t)kvh * GRP;
    const int per = (GRP * HD + NCL - 1) / NCL;                  // outputs per CTA
    for (int e = c * per + t; e < min((c + 1) * per, GRP * HD); e += AT) {
      const int hl = e / HD, d = e - hl * HD;
      float pv[NCL];
#pragma unroll
      for (int cc = 0; cc < NCL; ++cc) pv[cc] = cc < nact ? ld_peer_f32(&part_o[hl][d], (uint32_t)cc) : 0.f;
      float ov = 0.f;
#pragma unroll
      for (int cc = 0; cc < NCL; ++cc) ov += cc < nact ? pv[cc] * wgt[hl][cc] : 0.f;
      const __half hv = __float2half_rn(ov / wgt[hl][NCL]);
      out[(head0 + hl) * HD + d] = hv;
      if (xq) {
        // Fused Q8_1 quantiser of the rounded output (arithmetic of quant_q8_1.cu / the reference's QUANT_Q8,
        // lab/qwen_batched.py:1030-1039).  The host passes xq only when a CTA's share is a whole number of 32-blocks
        // and at most one per thread, so a warp holds exactly one block of one head here.
        const float v = __half2float(hv);
        const float amax = warp_max(fabsf(v));
        const float dq = amax / 127.f;
        const int q = dq > 0.f ? __float2int_rn(v / dq) : 0;
        const size_t col = (head0 + hl) * HD + d;
        xq[col] = (int8_t)q;
        if (lane == 0) xd[col >> 5] = __float2half_rn(dq);
      }
    }
  }
  cluster_sync_all();                                            // peers stay resident until their partials are read
  stamp();                                                       // end
  if (tr) tr[15] = (unsigned long long)tri;
}

unsigned long long* g_attn_trace = nullptr;

}  // namespace

// Device buffer for the optional timeline of the next launches (16 x uint64 per CTA, up to 4096 CTAs); null = off.
void attn_decode_mma_trace(unsigned long long* buf) { g_attn_trace = buf; }

// Same contract as attn_decode (head_dim 128 only); needs no workspace.
// xq / xd (optional): also write the output as planar Q8_1 (int8 [B, NH*128], fp16 [B, NH*128/32]), saving the separate
// quantiser launch in front of o_proj; needs (NH / NKV) * 128 to be a multiple of 256 (a CTA's eighth of a KV group is
// then whole 32-blocks).  Returns Q4B_E_SHAPE without launching when that does not hold.
int attn_decode_mma(const void* qkv, const float* cosT, const float* sinT, const int64_t* pos, void* kc, void* vc, void* out, int B,
                    int NH, int NKV, int max_len, float scale, cudaStream_t st, void* xq, void* xd) {
  if (xq && (!xd || ((NH / NKV) * HD) % (NCL * 32) != 0)) return Q4B_E_SHAPE;
  if (cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(&attn_decode_mma_kernel), DYN_SMEM); e != cudaSuccess) {
    set_cuda_error(e, "attn_decode_mma: cudaFuncSetAttribute");
    return Q4B_E_CUDA;
  }
  const int chunk = ((max_len + NCL - 1) / NCL + TILE - 1) / TILE * TILE;
  const float scale_log2e = scale * 1.4426950408889634f;
  return check_launch(launch_pdl_cluster(attn_decode_mma_kernel, dim3(NCL, NKV, B), dim3(AT), DYN_SMEM, st, NCL, 1,
                                         (const __half*)qkv, cosT, sinT, pos, (__half*)kc, (__half*)vc, (__half*)out, NH, NKV,
                                         max_len, chunk, scale_log2e, g_attn_trace, (int8_t*)xq, (__half*)xd),
                      "attn_decode_mma");
}

}  // namespace q4b
