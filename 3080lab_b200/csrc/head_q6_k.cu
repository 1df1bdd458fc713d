// LM head stored as Q6_K (6.5625 bits per weight), one activation vector, greedy pick fused.
//
// logits[v] = sum_b sum_s (d[v, b] * sc[v, b, s]) * sum_{i<16} (q[v, b, s, i] - 32) * x[...] in fp32: the reference's
// Q6_K-exact head GEMV (gemv_q6_source, lab/qwen_kernels.py:608-678; host scripts/qwen_gguf.py:92-104, 133-139): the
// 6-bit code comes exactly out of the float magic constant, the partial sum of a 16-weight sub-block is formed first
// and scaled once by the fp32 product d * sc, as there.  Device layout: the reference's four planes,
//   L  uint32 [V, K/8]    low 4 bits of q + 32, nibble i of word w = weight 8 w + i
//   Hb uint32 [V, K/16]   high 2 bits of q + 32 of the 16 weights of a sub-block
//   SC int8   [V, K/16]   sub-block scales (16 weights each)
//   D  fp16   [V, K/256]  super-block scales
// (made from the file's bytes by gguf.q6_k_planes), with ONE change: inside an Hb word the two bits of weight i sit at
// bit 8 ((i % 8) / 2) + 2 ((i % 2) + 2 (i / 8)) instead of 2 i, so that a shift and a mask put the high bits of weights
// (0,2,4,6), (1,3,5,7), (8,10,12,14), (9,11,13,15) at bits 4-5 of the very bytes where (L & 0x0F0F0F0F) and
// ((L >> 4) & 0x0F0F0F0F) hold their low nibbles: four 6-bit codes per three instructions, then one byte-permute per
// weight drops a code into the mantissa of the magic constant.  For the 151 936 x 1536 head of a llama.cpp Q4_0 export that is
// 191 MB per token instead of the 467 MB of an fp16 table.
//
// Shape of the kernel as head_f16.cu: persistent grid, a lane owns the same K/32 columns of every row (NS sub-blocks
// of 16 weights), so its slice of x lives in registers; 4 rows per warp step, all loads of a step issued before the
// first use; argmax fused (FINISH_MB, lab/qwen_kernels.py:250-282: lowest index among the maxima, pos += 1).
#include "q4b_internal.h"

namespace q4b {

namespace {

constexpr int HT = 256, HW = HT / 32, RW = 4;
constexpr int MAX_CTAS = 1024;

__device__ __forceinline__ void arg_merge(float& v, int& idx, float ov, int oi) {
  if (ov > v || (ov == v && oi < idx)) {
    v = ov;
    idx = oi;
  }
}
__device__ __forceinline__ void arg_warp(float& v, int& idx) {
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    arg_merge(v, idx, ov, oi);
  }
}

template <int NS>   // sub-blocks of 16 weights per lane: K = 512 NS
__global__ void __launch_bounds__(HT, 1) head_q6_k_kernel(const uint32_t* __restrict__ L, const uint32_t* __restrict__ Hb,
                                                          const int8_t* __restrict__ SC, const __half* __restrict__ D,
                                                          const __half* x, float* __restrict__ logits, int V, int K, int64_t* tok,
                                                          int64_t* pos, float* partv, int* parti, unsigned* cnt) {
  __shared__ float bv[HW];
  __shared__ int bi[HW];
  __shared__ bool last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  pdl_wait();
  const int k0 = lane * 16 * NS;                          // first weight of this lane in a row
  float xf[NS][16];
#pragma unroll
  for (int s = 0; s < NS; ++s) {
    const uint4 a = *reinterpret_cast<const uint4*>(x + k0 + 16 * s), b = *reinterpret_cast<const uint4*>(x + k0 + 16 * s + 8);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      xf[s][2 * i] = f.x;
      xf[s][2 * i + 1] = f.y;
    }
  }
  const int KW8 = K >> 3, KW16 = K >> 4, KD = K >> 8;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  const int groups = (V + RW - 1) / RW;
  for (int g = blockIdx.x * HW + warp; g < groups; g += gridDim.x * HW) {
    const int r0 = g * RW;
    uint2 lo[RW][NS];
    uint32_t hi[RW][NS];
    float scale[RW][NS];
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      const size_t row = (size_t)min(r0 + r, V - 1);
#pragma unroll
      for (int s = 0; s < NS; ++s) {
        const int sb = lane * NS + s;                     // sub-block index in the row
        lo[r][s] = *reinterpret_cast<const uint2*>(L + row * KW8 + 2 * sb);
        hi[r][s] = Hb[row * KW16 + sb];
        scale[r][s] = __half2float(D[row * KD + (sb >> 4)]) * (float)SC[row * KW16 + sb];   // fp32 d * sc
      }
    }
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      float a = 0.f;
#pragma unroll
      for (int s = 0; s < NS; ++s) {
        const uint32_t l0 = lo[r][s].x, l1 = lo[r][s].y, hw = hi[r][s];
        // codes q + 32 (0..63) of weights (0,2,4,6), (1,3,5,7), (8,10,12,14), (9,11,13,15), one per byte
        const uint32_t qc[4] = {(l0 & 0x0F0F0F0Fu) | ((hw << 4) & 0x30303030u), ((l0 >> 4) & 0x0F0F0F0Fu) | ((hw << 2) & 0x30303030u),
                                (l1 & 0x0F0F0F0Fu) | (hw & 0x30303030u), ((l1 >> 4) & 0x0F0F0F0Fu) | ((hw >> 2) & 0x30303030u)};
        float p = 0.f;
#pragma unroll
        for (int gsel = 0; gsel < 4; ++gsel) {
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            const int i = 8 * (gsel >> 1) + 2 * b + (gsel & 1);              // weight index inside the sub-block
            // byte b of the code word into the low byte of 0x4B000000: the float 2^23 + q; minus (2^23 + 32) = q - 32, exactly
            const uint32_t bits = __byte_perm(qc[gsel], 0x4B000000u, 0x7440 + b);
            p = fmaf(__uint_as_float(bits) - 8388640.0f, xf[s][i], p);
          }
        }
        a = fmaf(scale[r][s], p, a);
      }
      a = warp_sum(a);
      const int row = r0 + r;
      if (row < V) {
        if (lane == 0) logits[row] = a;
        if (a > best) {                                   // rows ascend within a warp: strict > keeps the lowest index
          best = a;
          best_i = row;
        }
      }
    }
  }
  if (!tok && !pos) return;
  if (lane == 0) {
    bv[warp] = best;
    bi[warp] = best_i;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = lane < HW ? bv[lane] : -INFINITY;
    int idx = lane < HW ? bi[lane] : 0x7fffffff;
    arg_warp(v, idx);
    if (lane == 0) {
      partv[blockIdx.x] = v;
      parti[blockIdx.x] = idx;
      __threadfence();
      last = atomicAdd(cnt, 1u) == gridDim.x - 1;
    }
  }
  __syncthreads();
  if (!last || threadIdx.x >= 32) return;
  __threadfence();
  float v = -INFINITY;
  int idx = 0x7fffffff;
  for (int b = lane; b < (int)gridDim.x; b += 32) arg_merge(v, idx, __ldcg(partv + b), __ldcg(parti + b));
  arg_warp(v, idx);
  if (lane == 0) {
    if (tok) tok[0] = idx == 0x7fffffff ? 0 : idx;
    if (pos) pos[0] += 1;
    *cnt = 0u;
  }
}

}  // namespace

size_t head_workspace(int V);

int head_q6_k_argmax(const void* L, const void* Hb, const void* SC, const void* D, const void* x, float* logits, int V, int K,
                     int64_t* tok, int64_t* pos, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (V <= 0 || K <= 0 || (K % 512) || K > 2048) return fail(Q4B_E_SHAPE, "head_q6_k_argmax: need V > 0 and K in {512, 1024, 1536, 2048}");
  if (!L || !Hb || !SC || !D || !x || !logits || !ws || !aligned16(L) || !aligned16(x) || (reinterpret_cast<uintptr_t>(Hb) & 3u))
    return fail(Q4B_E_ALIGN, "head_q6_k_argmax: null or misaligned pointer");
  if (ws_bytes < head_workspace(V)) return fail(Q4B_E_WORKSPACE, "head_q6_k_argmax: workspace too small");
  unsigned* cnt = reinterpret_cast<unsigned*>(ws);
  float* partv = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + 16);
  int* parti = reinterpret_cast<int*>(partv + MAX_CTAS);
  int grid = sm_count();
  if (grid > MAX_CTAS) grid = MAX_CTAS;
  if (grid * HW * RW > V) grid = (V + HW * RW - 1) / (HW * RW);
#define Q4B_Q6_CASE(N)                                                                                                   \
  case N:                                                                                                                \
    return check_launch(launch_pdl(head_q6_k_kernel<N>, dim3(grid), dim3(HT), 0, st, (const uint32_t*)L, (const uint32_t*)Hb, \
                                   (const int8_t*)SC, (const __half*)D, (const __half*)x, logits, V, K, tok, pos, partv, parti, \
                                   cnt), "head_q6_k_argmax");
  switch (K / 512) {
    Q4B_Q6_CASE(1) Q4B_Q6_CASE(2) Q4B_Q6_CASE(3) Q4B_Q6_CASE(4)
    default: break;
  }
#undef Q4B_Q6_CASE
  return fail(Q4B_E_SHAPE, "head_q6_k_argmax: unsupported K");
}

}  // namespace q4b
