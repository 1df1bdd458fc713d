// Prefill attention: RoPE + K/V append for a chunk of P prompt tokens, then causal GQA flash attention.
//
// Reference: the K/V write of the QKV GEMM epilogue `biasf_kv` (lab/qwen_batched.py:1316-1362: K rotated from the
// rounded biased values and stored 16-bit at posp[token], V copied) and flash_prefill_source / _v3
// (lab/qwen_batched.py:1563-1714, 1795-2037): Q rotated and rounded to 16 bits, S = Q K^T on tensor cores, fp32 online
// softmax in base 2 (scale * log2 e, exp2f), masked scores = -inf, probabilities rounded to 16 bits for the P.V MMA
// while the normaliser keeps the unrounded sum, out = round16(O / l).  fp16 here where the reference has bf16.
//
// Shape: one CTA = 64 query rows of one head (4 warps x 16 rows), key/value tiles of 64 positions staged in shared
// memory (rows padded to 272 bytes: conflict-free fragment reads), mma.sync.m16n8k16 for both products, ldmatrix.trans
// for the V operand.  Heaviest query tiles (longest key range) are scheduled first.  Attention is ~6 % of the prefill
// arithmetic at 2048 tokens; the int8 MMQ dominates.
#include "q4b_internal.h"

namespace q4b {

namespace {

constexpr int HD = 128, HALF = 64;
constexpr int BQ = 64, BK = 64;                 // query rows / keys per tile
constexpr int PITCH = HD * 2 + 16;              // bytes per staged row
constexpr int FT = 128;

__global__ void __launch_bounds__(128) rope_kv_append_kernel(const __half* qkv, const float* __restrict__ cosT,
                                                             const float* __restrict__ sinT, __half* kc, __half* vc, int P,
                                                             int NH, int NKV, int max_len, int pos0) {
  pdl_launch_dependents();
  pdl_wait();
  const int p = blockIdx.x, kvh = blockIdx.y, d = threadIdx.x;
  const int pos = pos0 + p;
  if (pos >= max_len) return;
  const __half* row = qkv + (size_t)p * (NH + 2 * NKV) * HD;
  const __half* kh = row + (size_t)NH * HD + (size_t)kvh * HD;
  const int dd = d % HALF;
  const float c = cosT[(size_t)pos * HALF + dd], s = sinT[(size_t)pos * HALF + dd];
  const float a = __half2float(kh[d]), o = __half2float(kh[d < HALF ? d + HALF : d - HALF]);
  float lo, hi;
  if (d < HALF) rope_pair(a, o, c, s, lo, hi);
  else rope_pair(o, a, c, s, lo, hi);
  kc[((size_t)kvh * max_len + pos) * HD + d] = __float2half_rn(d < HALF ? lo : hi);
  vc[((size_t)kvh * max_len + pos) * HD + d] = row[(size_t)(NH + NKV) * HD + (size_t)kvh * HD + d];
}

__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

__global__ void __launch_bounds__(FT) flash_prefill_kernel(const __half* qkv, const float* __restrict__ cosT,
                                                           const float* __restrict__ sinT, const __half* kc,
                                                           const __half* vc, __half* out, int P, int NH, int NKV,
                                                           int max_len, int pos0, float scale_log2e, int pre, uint8_t* xt) {
  extern __shared__ __align__(16) uint8_t sm[];
  uint8_t* sQ = sm;                      // [BQ][PITCH]
  uint8_t* sKV = sQ + BQ * PITCH;        // [2 stages][K, V][BK][PITCH]: the next key tile lands while this one is used
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31, g = lane >> 2, tq = lane & 3;
  const int h = blockIdx.y, kvh = h / (NH / NKV);
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;           // longest key ranges first
  const int q0 = qt * BQ;
  const int QKV = (NH + 2 * NKV) * HD;
  pdl_launch_dependents();
  pdl_wait();

  // ---- Q tile: rotate pairs (d, d + 64), round to fp16, stage
  for (int i = t; i < BQ * HALF; i += FT) {
    const int r = i / HALF, d = i - r * HALF;
    const int p = q0 + r;
    float lo = 0.f, hi = 0.f;
    if (p < P) {
      const __half* qh = qkv + (size_t)p * QKV + (size_t)h * HD;
      const float a = __half2float(qh[d]), b = __half2float(qh[d + HALF]);
      if (pre) {                                                 // q arrives rotated (QKV GEMM with the rope/kv epilogue)
        lo = a;
        hi = b;
      } else {
        const float c = cosT[(size_t)(pos0 + p) * HALF + d], s = sinT[(size_t)(pos0 + p) * HALF + d];
        rope_pair(a, b, c, s, lo, hi);
      }
    }
    *reinterpret_cast<__half*>(sQ + r * PITCH + d * 2) = __float2half_rn(lo);
    *reinterpret_cast<__half*>(sQ + r * PITCH + (d + HALF) * 2) = __float2half_rn(hi);
  }
  __syncthreads();
  // A fragments of this warp's 16 query rows, all 8 k-steps of the head dimension
  uint32_t qa[8][4];
  {
    const uint8_t* r0 = sQ + (warp * 16 + g) * PITCH, *r1 = r0 + 8 * PITCH;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      qa[s][0] = *reinterpret_cast<const uint32_t*>(r0 + (16 * s + 2 * tq) * 2);
      qa[s][1] = *reinterpret_cast<const uint32_t*>(r1 + (16 * s + 2 * tq) * 2);
      qa[s][2] = *reinterpret_cast<const uint32_t*>(r0 + (16 * s + 2 * tq + 8) * 2);
      qa[s][3] = *reinterpret_cast<const uint32_t*>(r1 + (16 * s + 2 * tq + 8) * 2);
    }
  }
  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;     // rows g and g + 8 of this warp
  const int row0 = q0 + warp * 16 + g, row1 = row0 + 8;          // query indices inside the chunk
  const int qpos0 = pos0 + row0, qpos1 = pos0 + row1;            // absolute positions
  const int last_key = min(pos0 + min(q0 + BQ, P), max_len) - 1; // last key any row of this tile may see
  const __half* kbase = kc + (size_t)kvh * max_len * HD;
  const __half* vbase = vc + (size_t)kvh * max_len * HD;

  // key tile -> stage: 16-byte asynchronous copies, rows past the last visible key zero-filled (source size 0)
  auto issue = [&](int k0, int stg) {
    uint8_t* dK = sKV + (size_t)stg * 2 * BK * PITCH;
    uint8_t* dV = dK + BK * PITCH;
    for (int i = t; i < BK * (HD / 8); i += FT) {
      const int r = i / (HD / 8), c = i - r * (HD / 8);
      const bool live = k0 + r <= last_key;
      const size_t src = (size_t)(live ? k0 + r : 0) * HD + c * 8;
      const uint32_t n = live ? 16u : 0u;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dK + r * PITCH + c * 16)),
                   "l"(kbase + src), "r"(n)
                   : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dV + r * PITCH + c * 16)),
                   "l"(vbase + src), "r"(n)
                   : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  issue(0, 0);
  for (int k0 = 0, it = 0; k0 <= last_key; k0 += BK, ++it) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");          // this thread's part of tile `it` has landed
    __syncthreads();                                             // ... everyone's; and tile it - 1 is fully consumed
    if (k0 + BK <= last_key) issue(k0 + BK, (it + 1) & 1);
    const uint8_t* sK = sKV + (size_t)(it & 1) * 2 * BK * PITCH;
    const uint8_t* sV = sK + BK * PITCH;

    // ---- S = Q K^T for 16 rows x 64 keys
    float sacc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f;
      // K fragments of two 16-dimension steps per ldmatrix.x4 (8 keys x 8 dims each: step 2 sp low / high, step 2 sp + 1
      // low / high) instead of eight 4-byte loads
      const int mi = lane >> 3;
      const uint8_t* kr = sK + (8 * j + (lane & 7)) * PITCH + (16 * (mi >> 1) + 8 * (mi & 1)) * 2;
#pragma unroll
      for (int sp = 0; sp < 4; ++sp) {
        uint32_t b0, b1, b2, b3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                     : "r"((uint32_t)__cvta_generic_to_shared(kr + 64 * sp)));
        mma16816(sacc[j], qa[2 * sp][0], qa[2 * sp][1], qa[2 * sp][2], qa[2 * sp][3], b0, b1);
        mma16816(sacc[j], qa[2 * sp + 1][0], qa[2 * sp + 1][1], qa[2 * sp + 1][2], qa[2 * sp + 1][3], b2, b3);
      }
    }
    // ---- scale, causal mask, online softmax (base 2)
    float mx0 = m0, mx1 = m1;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int key = k0 + 8 * j + 2 * tq;
      sacc[j][0] = key <= qpos0 ? sacc[j][0] * scale_log2e : -INFINITY;
      sacc[j][1] = key + 1 <= qpos0 ? sacc[j][1] * scale_log2e : -INFINITY;
      sacc[j][2] = key <= qpos1 ? sacc[j][2] * scale_log2e : -INFINITY;
      sacc[j][3] = key + 1 <= qpos1 ? sacc[j][3] * scale_log2e : -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(sacc[j][0], sacc[j][1]));
      mx1 = fmaxf(mx1, fmaxf(sacc[j][2], sacc[j][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    // a row that has seen no key yet keeps max = -inf; use 0 as its reference so that exp2(-inf - 0) = 0
    const float ref0 = mx0 == -INFINITY ? 0.f : mx0, ref1 = mx1 == -INFINITY ? 0.f : mx1;
    const float cor0 = exp2f(m0 - ref0), cor1 = exp2f(m1 - ref1);   // m = -inf -> 0
    m0 = mx0;
    m1 = mx1;
    float ps0 = 0.f, ps1 = 0.f;
    uint32_t pa[4][4];                                            // P as A fragments: 4 k-steps of 16 keys
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float p0 = exp2f(sacc[j][0] - ref0), p1 = exp2f(sacc[j][1] - ref0);
      const float p2 = exp2f(sacc[j][2] - ref1), p3 = exp2f(sacc[j][3] - ref1);
      ps0 += p0 + p1;
      ps1 += p2 + p3;
      pa[j >> 1][(j & 1) * 2 + 0] = pack_h2(p0, p1);              // row g
      pa[j >> 1][(j & 1) * 2 + 1] = pack_h2(p2, p3);              // row g + 8
    }
    l0 = l0 * cor0 + ps0;                                         // per-lane partial sums; reduced over the quad at the end
    l1 = l1 * cor1 + ps1;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      o[j][0] *= cor0;
      o[j][1] *= cor0;
      o[j][2] *= cor1;
      o[j][3] *= cor1;
    }
    // ---- O += P V : k = keys (4 steps of 16), n = head dims (16 tiles of 8); V fragments through ldmatrix.trans
#pragma unroll
    for (int s = 0; s < 4; ++s) {
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        const int mtx = lane >> 3, r = lane & 7;
        const uint8_t* addr = sV + (16 * s + (mtx & 1) * 8 + r) * PITCH + (8 * (j + (mtx >> 1))) * 2;
        uint32_t b0, b1, b2, b3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                     : "r"((uint32_t)__cvta_generic_to_shared(addr)));
        mma16816(o[j], pa[s][0], pa[s][1], pa[s][2], pa[s][3], b0, b1);
        mma16816(o[j + 1], pa[s][0], pa[s][1], pa[s][2], pa[s][3], b2, b3);
      }
    }
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const int NQ = NH * HD;
  if (out) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int d = 8 * j + 2 * tq;
      if (row0 < P) *reinterpret_cast<uint32_t*>(out + (size_t)row0 * NQ + (size_t)h * HD + d) = pack_h2(o[j][0] * inv0, o[j][1] * inv0);
      if (row1 < P) *reinterpret_cast<uint32_t*>(out + (size_t)row1 * NQ + (size_t)h * HD + d) = pack_h2(o[j][2] * inv1, o[j][3] * inv1);
    }
  }
  if (xt) {
    // The `q8` output of the reference's flash kernel (lab/qwen_batched.py:1812-1848): the rounded output quantised per
    // 32 head dimensions with the arithmetic of quant_q8_1.cu and written in the tiled operand format of the o-projection
    // GEMM (k-block 4 h + b of the [P, NH * 128] activation).  A row's 32-value block lives in the four lanes of a quad.
    const int KBO = NQ >> 5;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      float y0[8], y1[8];
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          y0[2 * jj + e] = __half2float(__float2half_rn(o[4 * b + jj][e] * inv0));
          y1[2 * jj + e] = __half2float(__float2half_rn(o[4 * b + jj][2 + e] * inv1));
          a0 = fmaxf(a0, fabsf(y0[2 * jj + e]));
          a1 = fmaxf(a1, fabsf(y1[2 * jj + e]));
        }
      }
      a0 = fmaxf(a0, __shfl_xor_sync(0xffffffffu, a0, 1));
      a0 = fmaxf(a0, __shfl_xor_sync(0xffffffffu, a0, 2));
      a1 = fmaxf(a1, __shfl_xor_sync(0xffffffffu, a1, 1));
      a1 = fmaxf(a1, __shfl_xor_sync(0xffffffffu, a1, 2));
      const float d0 = a0 / 127.f, d1 = a1 / 127.f;
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const int prow = rr ? row1 : row0;
        if (prow >= P) continue;
        const float dq = rr ? d1 : d0;
        uint8_t* rec = xt + ((size_t)(prow >> 7) * KBO + (size_t)h * 4 + b) * 4608;
        const int n = prow & 127;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float y = rr ? y1[2 * jj + e] : y0[2 * jj + e];
            const int q = dq > 0.f ? __float2int_rn(y / dq) : 0;
            rec[q8_tiled_offset(n, 8 * jj + 2 * tq + e)] = (uint8_t)(q & 0xFF);
          }
        if (tq == 0) reinterpret_cast<float*>(rec + 4096)[n] = __half2float(__float2half_rn(dq));
      }
    }
  }
}

constexpr size_t FLASH_SMEM = (size_t)(BQ + 4 * BK) * PITCH;

}  // namespace

// pre = 0: qkv un-rotated, K/V appended here (two launches).  pre = 1: q and the cache rows were rotated / written by
// the QKV GEMM's rope/kv epilogue; one launch.  out and / or xt (tiled Q8_1 of the output) receive the result.
int attn_prefill(const void* qkv, const float* cosT, const float* sinT, void* kc, void* vc, void* out, int P, int NH, int NKV,
                 int HDim, int max_len, int pos0, float scale, cudaStream_t st, int pre, void* xt) {
  if (P <= 0 || NH <= 0 || NKV <= 0 || (NH % NKV) || HDim != HD || max_len <= 0 || pos0 < 0 || pos0 + P > max_len)
    return fail(Q4B_E_SHAPE, "attn_prefill: need head_dim 128, NH a multiple of NKV, pos0 + P <= max_len");
  if (!qkv || (!pre && (!cosT || !sinT)) || !kc || !vc || (!out && !xt) || !aligned16(kc) || !aligned16(vc) || !aligned16(qkv) ||
      !aligned16(out) || !aligned16(xt))
    return fail(Q4B_E_ALIGN, "attn_prefill: null or misaligned pointer");
  if (cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(&flash_prefill_kernel), FLASH_SMEM); e != cudaSuccess) {
    set_cuda_error(e, "attn_prefill: cudaFuncSetAttribute");
    return Q4B_E_CUDA;
  }
  if (!pre) {
    int rc = check_launch(launch_pdl(rope_kv_append_kernel, dim3(P, NKV), dim3(HD), 0, st, (const __half*)qkv, cosT, sinT,
                                     (__half*)kc, (__half*)vc, P, NH, NKV, max_len, pos0),
                          "attn_prefill: kv append");
    if (rc != Q4B_OK) return rc;
  }
  const float scale_log2e = scale * 1.4426950408889634f;
  return check_launch(launch_pdl(flash_prefill_kernel, dim3((P + BQ - 1) / BQ, NH), dim3(FT), FLASH_SMEM, st,
                                 (const __half*)qkv, cosT, sinT, (const __half*)kc, (const __half*)vc, (__half*)out, P, NH, NKV,
                                 max_len, pos0, scale_log2e, pre, (uint8_t*)xt),
                      "attn_prefill");
}

}  // namespace q4b
