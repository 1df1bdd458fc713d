// Embedding lookup, RMSNorm and the greedy pick (argmax + position advance).
#include "q4b_internal.h"

namespace q4b {

namespace {

// h[row] = float(E[tok[row]]), one CTA per row.  Reference: EMBED_F32 (lab/qwen_kernels.py:284-290) with an fp16 table.
// The lookup opens every decode step, and it is the step's fence: it lets its dependents start only AFTER its own
// dependency wait, i.e. after everything of the previous step has completed.  Later launches of the step may therefore
// read state that only earlier steps wrote (the position, cache rows below it) ahead of their own waits.
__global__ void __launch_bounds__(256) embed_kernel(const __half* __restrict__ E, const int64_t* tok, float* h, int H, int V) {
  pdl_wait();
  pdl_launch_dependents();
  long long t = tok[blockIdx.x];
  t = t < 0 ? 0 : (t >= V ? V - 1 : t);
  const __half2* src = reinterpret_cast<const __half2*>(E + (size_t)t * H);
  float2* dst = reinterpret_cast<float2*>(h + (size_t)blockIdx.x * H);
  for (int i = threadIdx.x; i < H / 2; i += blockDim.x) dst[i] = __half22float2(src[i]);
}

// out = round16(v * rsqrt(mean(v^2) + eps) * w), one CTA of 256 threads per row.
// Reference: RMSNORM_F32W_1P (lab/qwen_kernels.py:683-705): values stay in registers between the two passes,
// product order (v * r) * w, a single rounding at the store.
constexpr int RMS_T = 256, RMS_MAXV = 16;   // up to 4096 columns in registers; wider rows re-read h
__global__ void __launch_bounds__(RMS_T) rmsnorm_kernel(const float* h, const float* __restrict__ w, __half* out, int H,
                                                        float eps) {
  __shared__ float part[RMS_T / 32];
  pdl_launch_dependents();
  pdl_wait();
  const float* hr = h + (size_t)blockIdx.x * H;
  __half* o = out + (size_t)blockIdx.x * H;
  float v[RMS_MAXV];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < RMS_MAXV; ++u) {
    const int i = threadIdx.x + RMS_T * u;
    v[u] = i < H ? hr[i] : 0.f;
    ss += v[u] * v[u];
  }
  for (int i = threadIdx.x + RMS_T * RMS_MAXV; i < H; i += RMS_T) ss += hr[i] * hr[i];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int j = 0; j < RMS_T / 32; ++j) t += part[j];
  const float r = rsqrtf(t / (float)H + eps);
#pragma unroll
  for (int u = 0; u < RMS_MAXV; ++u) {
    const int i = threadIdx.x + RMS_T * u;
    if (i < H) o[i] = __float2half_rn(v[u] * r * w[i]);
  }
  for (int i = threadIdx.x + RMS_T * RMS_MAXV; i < H; i += RMS_T) o[i] = __float2half_rn(hr[i] * r * w[i]);
}

// Greedy pick.  Slices of one row go to ARG_SLICES CTAs; each writes (max, lowest index) and the last CTA of the row
// to arrive (threadfence + counter) combines them in slice order, writes tok, advances pos and re-zeroes the counter.
// Reference: FINISH_MB (lab/qwen_kernels.py:250-282); tie rule of FINISH (:227-240): lowest index among the maxima.
constexpr int ARG_SLICES = 64, ARG_T = 256;

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

__global__ void __launch_bounds__(ARG_T) argmax_kernel(const float* logits, int V, int64_t* tok,
                                                       int64_t* pos, float* partv, int* parti, unsigned* cnt) {
  __shared__ float bv[ARG_T / 32];
  __shared__ int bi[ARG_T / 32];
  __shared__ bool last;
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.y;
  const float* lr = logits + (size_t)row * V;
  const int per = (V + gridDim.x - 1) / gridDim.x;
  const int i0 = blockIdx.x * per, i1 = min(V, i0 + per);
  float v = -INFINITY;
  int idx = 0x7fffffff;
  for (int i = i0 + threadIdx.x; i < i1; i += ARG_T) {
    const float x = lr[i];
    if (x > v) {
      v = x;
      idx = i;
    }
  }
  arg_warp(v, idx);
  if ((threadIdx.x & 31) == 0) {
    bv[threadIdx.x >> 5] = v;
    bi[threadIdx.x >> 5] = idx;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    v = threadIdx.x < ARG_T / 32 ? bv[threadIdx.x] : -INFINITY;
    idx = threadIdx.x < ARG_T / 32 ? bi[threadIdx.x] : 0x7fffffff;
    arg_warp(v, idx);
    if (threadIdx.x == 0) {
      partv[row * gridDim.x + blockIdx.x] = v;
      parti[row * gridDim.x + blockIdx.x] = idx;
      __threadfence();
      last = atomicAdd(cnt + row, 1u) == gridDim.x - 1;
    }
  }
  __syncthreads();
  if (!last || threadIdx.x >= 32) return;
  __threadfence();
  v = -INFINITY;
  idx = 0x7fffffff;
  for (int b = threadIdx.x; b < (int)gridDim.x; b += 32)
    arg_merge(v, idx, __ldcg(partv + row * gridDim.x + b), __ldcg(parti + row * gridDim.x + b));
  arg_warp(v, idx);
  if (threadIdx.x == 0) {
    if (tok) tok[row] = idx == 0x7fffffff ? 0 : idx;
    if (pos) pos[row] += 1;
    cnt[row] = 0u;
  }
}

// Scratch of the allocation-free greedy pick: counters first, then per-slice maxima and indices, for up to
// STATIC_MAX_ROWS rows.  It lives in the library image: every GPU that loads the library carries these bytes until the
// process exits.
constexpr int STATIC_MAX_ROWS = 64;
constexpr size_t STATIC_SCRATCH_BYTES = 256 + (size_t)STATIC_MAX_ROWS * ARG_SLICES * 8;
static __device__ __align__(256) unsigned char g_argmax_scratch[STATIC_SCRATCH_BYTES];

}  // namespace

int embed(const void* E, const int64_t* tok, float* h, int rows, int H, int V, cudaStream_t st) {
  if (rows <= 0 || H <= 0 || (H % 2) || V <= 0) return fail(Q4B_E_SHAPE, "embed: rows, V > 0 and even H required");
  if (!E || !tok || !h || (reinterpret_cast<uintptr_t>(E) & 3u) || (reinterpret_cast<uintptr_t>(h) & 7u))
    return fail(Q4B_E_ALIGN, "embed: null or misaligned pointer");
  return check_launch(launch_pdl(embed_kernel, dim3(rows), dim3(256), 0, st, reinterpret_cast<const __half*>(E), tok, h, H, V), "embed");
}

int rmsnorm(const float* h, const float* w, void* out, int rows, int H, float eps, cudaStream_t st) {
  if (rows <= 0 || H <= 0) return fail(Q4B_E_SHAPE, "rmsnorm: rows, H > 0 required");
  if (!h || !w || !out) return fail(Q4B_E_ALIGN, "rmsnorm: null pointer");
  return check_launch(launch_pdl(rmsnorm_kernel, dim3(rows), dim3(RMS_T), 0, st, h, w, reinterpret_cast<__half*>(out), H, eps), "rmsnorm");
}

size_t argmax_workspace(int rows, int V) {
  (void)V;
  return (size_t)rows * (ARG_SLICES * 8 + 4) + 16;
}

int argmax_advance(const float* logits, int rows, int V, int64_t* tok, int64_t* pos, void* ws, size_t ws_bytes,
                   cudaStream_t st) {
  if (rows <= 0 || V <= 0) return fail(Q4B_E_SHAPE, "argmax_advance: rows, V > 0 required");
  if (!logits || !ws) return fail(Q4B_E_ALIGN, "argmax_advance: null pointer");
  if (ws_bytes < argmax_workspace(rows, V)) return fail(Q4B_E_WORKSPACE, "argmax_advance: workspace too small");
  // workspace: [rows] counters (kept zero between launches), then the per-slice maxima and indices
  unsigned* cnt = reinterpret_cast<unsigned*>(ws);
  float* partv = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + (((size_t)rows * 4 + 15) & ~(size_t)15));
  int* parti = reinterpret_cast<int*>(partv + (size_t)rows * ARG_SLICES);
  return check_launch(launch_pdl(argmax_kernel, dim3(ARG_SLICES, rows), dim3(ARG_T), 0, st, logits, V, tok, pos, partv, parti, cnt),
                      "argmax_advance");
}

// Greedy pick without caller-provided scratch.  In host code `g_argmax_scratch` is only a handle for the runtime, not a
// device address, so the address is looked up with cudaGetSymbolAddress: once per device, with that device current, and
// remembered.  No allocation of any kind happens here.
int argmax_advance_static(const float* logits, int rows, int V, int64_t* tok, int64_t* pos, cudaStream_t st) {
  if (rows <= 0 || V <= 0) return fail(Q4B_E_SHAPE, "argmax_advance_static: rows, V > 0 required");
  if (rows > STATIC_MAX_ROWS)
    return fail(Q4B_E_SHAPE, "argmax_advance_static: at most 64 rows fit the built-in scratch; use q4b_argmax_advance with a workspace");
  if (!logits) return fail(Q4B_E_ALIGN, "argmax_advance_static: null pointer");
  constexpr int MAX_DEV = 64;
  static unsigned char* base[MAX_DEV] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= MAX_DEV) {
    set_cuda_error(e != cudaSuccess ? e : cudaErrorInvalidDevice, "argmax_advance_static: cudaGetDevice");
    return Q4B_E_CUDA;
  }
  if (!base[dev]) {                                   // first call on this device: resolve the symbol's device address
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_argmax_scratch);
    if (e != cudaSuccess || !p) {
      set_cuda_error(e != cudaSuccess ? e : cudaErrorInvalidSymbol, "argmax_advance_static: cudaGetSymbolAddress");
      return Q4B_E_CUDA;
    }
    base[dev] = static_cast<unsigned char*>(p);
  }
  unsigned* cnt = reinterpret_cast<unsigned*>(base[dev]);
  float* partv = reinterpret_cast<float*>(base[dev] + 256);
  int* parti = reinterpret_cast<int*>(partv + (size_t)STATIC_MAX_ROWS * ARG_SLICES);
  // the array keeps whatever the previous call (or an interrupted one) left: the arrival counters must start at zero
  e = cudaMemsetAsync(cnt, 0, 256, st);
  if (e != cudaSuccess) {
    set_cuda_error(e, "argmax_advance_static: cudaMemsetAsync");
    return Q4B_E_CUDA;
  }
  argmax_kernel<<<dim3(ARG_SLICES, rows), ARG_T, 0, st>>>(logits, V, tok, pos, partv, parti, cnt);
  return check_launch("argmax_advance_static");
}

}  // namespace q4b
