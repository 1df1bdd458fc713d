// LM head over a tied fp16 embedding table, one activation vector, greedy pick fused.
//
// logits[v] = sum_k float(E[v, k]) * float(x[k]) in fp32 — the reference's "logits" GEMV epilogue
// (lab/qwen_kernels.py:44) followed by FINISH_MB's argmax (lab/qwen_kernels.py:250-282: slices, last CTA combines,
// lowest index among the maxima, pos += 1, self-resetting counter), in one launch.
//
// This is the largest single stream of the decode step (V x H x 2 bytes).  Persistent grid: every warp walks groups of
// 4 rows with a grid-wide stride; a lane owns the same column chunks of every row, so its slice of x lives in
// registers for the whole kernel and each row costs only its own 16-byte loads, all issued before the first use.
#include "q4b_internal.h"

namespace q4b {

namespace {

constexpr int HT = 256, HW = HT / 32;

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

template <int NCH, int RW>   // NCH 16-byte column chunks per lane (>= ceil(H / 256)), RW rows per warp step
__global__ void __launch_bounds__(HT, 1) head_f16_kernel(const uint4* __restrict__ E, const uint4* x,
                                                         float* __restrict__ logits, int V, int H, int64_t* tok,
                                                         int64_t* pos, float* partv, int* parti, unsigned* cnt) {
  __shared__ float bv[HW];
  __shared__ int bi[HW];
  __shared__ bool last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int HC = H >> 3;                                  // 16-byte chunks per row
  pdl_launch_dependents();
  pdl_wait();
  float xf[NCH][8];
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int ci = lane + 32 * c;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (ci < HC) v = x[ci];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
      xf[c][2 * k] = f.x;
      xf[c][2 * k + 1] = f.y;
    }
  }
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  const int groups = (V + RW - 1) / RW;
  for (int g = blockIdx.x * HW + warp; g < groups; g += gridDim.x * HW) {
    const int r0 = g * RW;
    uint4 wv[RW][NCH];
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      const int row = min(r0 + r, V - 1);
      const uint4* rp = E + (size_t)row * HC;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int ci = lane + 32 * c;
        wv[r][c] = ci < HC ? ldg_stream16(rp + ci) : make_uint4(0u, 0u, 0u, 0u);
      }
    }
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      float a = 0.f;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const uint32_t w[4] = {wv[r][c].x, wv[r][c].y, wv[r][c].z, wv[r][c].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
          a = fmaf(f.x, xf[c][2 * k], a);
          a = fmaf(f.y, xf[c][2 * k + 1], a);
        }
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
  // warps hold interleaved row sets, so merge by (value, then lower index)
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

constexpr int MAX_HEAD_CTAS = 1024;

}  // namespace

size_t head_workspace(int V) {
  (void)V;
  return 16 + (size_t)MAX_HEAD_CTAS * 8;
}

int head_f16_argmax(const void* E, const void* x, float* logits, int V, int H, int64_t* tok, int64_t* pos, void* ws,
                    size_t ws_bytes, cudaStream_t st) {
  if (V <= 0 || H <= 0 || (H % 8) || H > 4096) return fail(Q4B_E_SHAPE, "head_f16_argmax: need V > 0, H a multiple of 8, H <= 4096");
  if (!E || !x || !logits || !ws || !aligned16(E) || !aligned16(x)) return fail(Q4B_E_ALIGN, "head_f16_argmax: null or misaligned pointer");
  if (ws_bytes < head_workspace(V)) return fail(Q4B_E_WORKSPACE, "head_f16_argmax: workspace too small");
  unsigned* cnt = reinterpret_cast<unsigned*>(ws);
  float* partv = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + 16);
  int* parti = reinterpret_cast<int*>(partv + MAX_HEAD_CTAS);
  int grid = sm_count();
  if (grid > MAX_HEAD_CTAS) grid = MAX_HEAD_CTAS;
  if (grid * HW * 4 > V) grid = (V + HW * 4 - 1) / (HW * 4);
  const uint4* e = reinterpret_cast<const uint4*>(E);
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  const int need = (H / 8 + 31) / 32;
#define Q4B_HEAD_CASE(C, RWS)                                                                         \
  if (need <= C) {                                                                                    \
    return check_launch(launch_pdl(head_f16_kernel<C, RWS>, dim3(grid), dim3(HT), 0, st, e, xv, logits, V, H, tok, pos,     \
                                   partv, parti, cnt), "head_f16_argmax");                                                 \
  }
  Q4B_HEAD_CASE(1, 4) Q4B_HEAD_CASE(2, 4) Q4B_HEAD_CASE(4, 4) Q4B_HEAD_CASE(6, 4) Q4B_HEAD_CASE(8, 4) Q4B_HEAD_CASE(16, 1)
#undef Q4B_HEAD_CASE
  return fail(Q4B_E_SHAPE, "head_f16_argmax: H too large");
}

}  // namespace q4b
