// Q4_0 GEMV for one activation vector, exact dequantise-and-dot on the CUDA cores.
//
// Arithmetic follows the reference's split-K GEMV (lab/qwen_kernels.py:14-113 with the inner loop of
// lab/experiments/gemv4.py:31-57 and the "magic" nibble conversion of lab/experiments/gemv3.py:38-40): per 32-weight
// block part = sum fmaf(q_i - 8, x_i) in weight order, then acc = fmaf(d, part, acc); block partials are combined by a
// shuffle tree and a fixed-order sum over the K splits, so results are bit-repeatable run to run.
//
// Work split: a "team" of KS x TW threads owns 4 consecutive rows.  TW (16 or 32) threads stride over the k-blocks of
// one K split, KS splits cover K.  The host picks (TW, KS) per K so that every thread gets the same number of blocks
// (K = 1536 -> 48 blocks = 16 lanes x 3; K = 8960 -> 280 blocks = 3 splits x 32 lanes x 3) and issues all of its
// loads (U = 3 blocks x 4 rows x 16 bytes) before the first use: one memory round trip per launch.
#include "q4b_internal.h"

namespace q4b {

namespace {

constexpr int R = 4;   // rows per team
constexpr int U = 3;   // k-blocks per thread in flight
constexpr int MAX_TEAMS = 8, MAX_KS = 8;

template <bool XF32>
struct XBlock {
  uint4 v[XF32 ? 8 : 4];
};

template <bool XF32>
__device__ __forceinline__ void load_x(XBlock<XF32>& xb, const void* X, int j) {
  if (XF32) {
    const uint4* p = reinterpret_cast<const uint4*>(X) + (size_t)j * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) xb.v[i] = p[i];
  } else {
    const uint4* p = reinterpret_cast<const uint4*>(X) + (size_t)j * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) xb.v[i] = p[i];
  }
}

template <bool XF32>
__device__ __forceinline__ void widen_x(const XBlock<XF32>& xb, float* xs) {
  if (XF32) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      xs[4 * i + 0] = __uint_as_float(xb.v[i].x);
      xs[4 * i + 1] = __uint_as_float(xb.v[i].y);
      xs[4 * i + 2] = __uint_as_float(xb.v[i].z);
      xs[4 * i + 3] = __uint_as_float(xb.v[i].w);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t w[4] = {xb.v[i].x, xb.v[i].y, xb.v[i].z, xb.v[i].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
        xs[8 * i + 2 * k] = f.x;
        xs[8 * i + 2 * k + 1] = f.y;
      }
    }
  }
}

template <int EPI, bool XF32, int TW>
__global__ void __launch_bounds__(256) gemv_q4_0_kernel(const uint4* __restrict__ W, const __half* __restrict__ S,
                                                        const void* X, void* Y,
                                                        const void* __restrict__ AUX, int N, int K, int KS, int teams) {
  __shared__ float red[MAX_TEAMS][MAX_KS][R];
  pdl_launch_dependents();
  pdl_wait();
  const int KB = K >> 5;
  const int per_team = KS * TW;
  const int team = threadIdx.x / per_team, r_in = threadIdx.x - team * per_team;
  const int ks = r_in / TW, lane_k = r_in - ks * TW;
  const int row0 = (blockIdx.x * teams + team) * R;
  const int chunk = (KB + KS - 1) / KS;
  const int kb = ks * chunk, ke = min(KB, kb + chunk);

  float acc[R] = {0.f, 0.f, 0.f, 0.f};
  if (row0 < N) {
    for (int j0 = kb + lane_k; j0 < ke; j0 += U * TW) {
      uint4 w[U][R];
      float d[U][R];
      XBlock<XF32> xb[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int j = j0 + u * TW;
        const bool ok = j < ke;
        const int jc = ok ? j : ke - 1;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const bool live = ok && (row0 + r < N);
          const size_t at = (size_t)(live ? row0 + r : row0) * KB + jc;
          w[u][r] = live ? ldg_stream16(W + at) : make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
          d[u][r] = live ? __half2float(__ldg(S + at)) : 0.f;
        }
        load_x<XF32>(xb[u], X, jc);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float xs[32];
        widen_x<XF32>(xb[u], xs);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const uint32_t q[4] = {w[u][r].x, w[u][r].y, w[u][r].z, w[u][r].w};
          float part = 0.f;
#pragma unroll
          for (int k = 0; k < 4; ++k)
#pragma unroll
            for (int i = 0; i < 8; ++i) part = fmaf(nib_f32(q[k], i), xs[8 * k + i], part);
          acc[r] = fmaf(d[u][r], part, acc[r]);   // d is 0 for blocks past the end of this thread's range
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float a = acc[r];
#pragma unroll
    for (int o = TW / 2; o; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    if (lane_k == 0) red[team][ks][r] = a;
  }
  __syncthreads();
  if (row0 >= N) return;
  if (EPI == Q4B_EPI_SWIGLU) {
    if (r_in < R / 2 && row0 + 2 * r_in + 1 < N) {
      float g = 0.f, u = 0.f;
      for (int s = 0; s < KS; ++s) {
        g += red[team][s][2 * r_in];
        u += red[team][s][2 * r_in + 1];
      }
      reinterpret_cast<__half*>(Y)[row0 / 2 + r_in] = __float2half_rn(g / (1.f + __expf(-g)) * u);
    }
  } else if (r_in < R && row0 + r_in < N) {
    float a = 0.f;
    for (int s = 0; s < KS; ++s) a += red[team][s][r_in];
    const int r = row0 + r_in;
    if (EPI == Q4B_EPI_STORE) reinterpret_cast<__half*>(Y)[r] = __float2half_rn(a);
    if (EPI == Q4B_EPI_BIASF) reinterpret_cast<__half*>(Y)[r] = __float2half_rn(a + reinterpret_cast<const float*>(AUX)[r]);
    if (EPI == Q4B_EPI_RESID) reinterpret_cast<float*>(Y)[r] += a;
    if (EPI == Q4B_EPI_LOGITS) reinterpret_cast<float*>(Y)[r] = a;
  }
}

struct Plan {
  int tw, ks, teams;
};

// Fewest load batches first (latency), then the best lane utilisation, then the fewest K splits.
Plan plan_for(int K) {
  const int KB = K / 32;
  Plan best{32, 1, 4};
  long best_batches = 1L << 40;
  double best_eff = -1.0;
  for (int tw : {16, 32})
    for (int ks = 1; ks <= MAX_KS; ++ks) {
      const int chunk = (KB + ks - 1) / ks;
      const int its = (chunk + tw - 1) / tw;
      const long batches = (its + U - 1) / U;
      const double eff = (double)KB / ((double)ks * tw * batches * U);
      if (batches < best_batches || (batches == best_batches && eff > best_eff + 1e-9)) {
        best_batches = batches;
        best_eff = eff;
        best = Plan{tw, ks, 1};
      }
    }
  int teams = 128 / (best.ks * best.tw);
  if (teams < 1) teams = 1;
  if (teams > MAX_TEAMS) teams = MAX_TEAMS;
  while ((teams * best.ks * best.tw) % 32) ++teams;      // whole warps only (TW = 16 with an odd KS)
  best.teams = teams;
  return best;
}

template <int EPI, bool XF32>
void launch_tw(const Plan& p, dim3 grid, dim3 block, cudaStream_t st, const uint4* W, const __half* S, const void* X,
               void* Y, const void* AUX, int N, int K) {
  if (p.tw == 16)
    launch_pdl(gemv_q4_0_kernel<EPI, XF32, 16>, grid, block, 0, st, W, S, X, Y, AUX, N, K, p.ks, p.teams);
  else
    launch_pdl(gemv_q4_0_kernel<EPI, XF32, 32>, grid, block, 0, st, W, S, X, Y, AUX, N, K, p.ks, p.teams);
}

template <int EPI>
void launch_x(bool xf32, const Plan& p, dim3 grid, dim3 block, cudaStream_t st, const uint4* W, const __half* S,
              const void* X, void* Y, const void* AUX, int N, int K) {
  if (xf32)
    launch_tw<EPI, true>(p, grid, block, st, W, S, X, Y, AUX, N, K);
  else
    launch_tw<EPI, false>(p, grid, block, st, W, S, X, Y, AUX, N, K);
}

}  // namespace

int gemv_q4_0(const void* W, const void* S, const void* X, void* Y, const void* AUX, int N, int K, int epilogue,
              int x_dtype, cudaStream_t st) {
  if (N <= 0 || K <= 0 || (K % 32)) return fail(Q4B_E_SHAPE, "gemv_q4_0: N > 0 and K a positive multiple of 32 required");
  if (epilogue == Q4B_EPI_SWIGLU && (N % 2)) return fail(Q4B_E_SHAPE, "gemv_q4_0: swiglu needs an even row count");
  if (x_dtype != Q4B_X_F16 && x_dtype != Q4B_X_F32) return fail(Q4B_E_ARG, "gemv_q4_0: unknown x_dtype");
  if (!W || !S || !X || !Y || !aligned16(W) || !aligned16(X)) return fail(Q4B_E_ALIGN, "gemv_q4_0: W, X must be 16-byte aligned, all pointers non-null");
  if ((reinterpret_cast<uintptr_t>(S) & 1u) || (reinterpret_cast<uintptr_t>(Y) & 3u)) return fail(Q4B_E_ALIGN, "gemv_q4_0: S/Y misaligned");
  if (epilogue == Q4B_EPI_BIASF && !AUX) return fail(Q4B_E_ALIGN, "gemv_q4_0: biasf needs AUX");
  const Plan p = plan_for(K);
  const int groups = (N + R - 1) / R;
  dim3 grid((groups + p.teams - 1) / p.teams), block(p.teams * p.ks * p.tw);
  const uint4* w = reinterpret_cast<const uint4*>(W);
  const __half* s = reinterpret_cast<const __half*>(S);
  const bool xf = x_dtype == Q4B_X_F32;
  switch (epilogue) {
    case Q4B_EPI_STORE: launch_x<Q4B_EPI_STORE>(xf, p, grid, block, st, w, s, X, Y, AUX, N, K); break;
    case Q4B_EPI_BIASF: launch_x<Q4B_EPI_BIASF>(xf, p, grid, block, st, w, s, X, Y, AUX, N, K); break;
    case Q4B_EPI_RESID: launch_x<Q4B_EPI_RESID>(xf, p, grid, block, st, w, s, X, Y, AUX, N, K); break;
    case Q4B_EPI_SWIGLU: launch_x<Q4B_EPI_SWIGLU>(xf, p, grid, block, st, w, s, X, Y, AUX, N, K); break;
    case Q4B_EPI_LOGITS: launch_x<Q4B_EPI_LOGITS>(xf, p, grid, block, st, w, s, X, Y, AUX, N, K); break;
    default: return fail(Q4B_E_ARG, "gemv_q4_0: unknown epilogue");
  }
  return check_launch("gemv_q4_0");
}

}  // namespace q4b
