// Tensor-parallel reduction of the row-parallel linears, fused with what follows it in the decode step:
//
//   h[b, :] += sum over ranks r (rank order) of part_r[b, :]        (the all-reduce after o_proj / down_proj)
//   xq, xd   = Q8_1( round16( RMSNorm(h[b, :]) * w ) )               (optional: the next linear's activation operand)
//
// one launch instead of NCCL all-reduce + residual add + RMSNorm/quantiser.  The reference is single-GPU; its launch
// sites for the pieces are the `resid` epilogue (lab/qwen_kernels.py:21-45) and rmsnorm_q8_source
// (lab/qwen_batched.py:1044-1091), whose arithmetic the second half repeats operation by operation.
//
// One-shot all-reduce over peer memory: every rank's partial [rows, H] fp32 lives in a buffer all ranks can address
// (symmetric memory, mapped over NVLink); every rank reads all partials with plain peer loads and computes the same sum
// in the same order, so the replicated residual stream stays bit-identical across ranks.  No multicast, no in-switch
// reduction: 0.9 MB per rank and call (7B shape, 64 rows) is latency-, not bandwidth-bound.
//
// Synchronisation: CTA b handles row b.  After the programmatic-dependency wait (its rank's GEMM is complete and
// flushed) it publishes `epoch` into slot [my rank][b] of every peer's flag array (release, system scope) and waits,
// with a bound, for slot [r][b] of its own array to reach `epoch` for every peer r (acquire, system scope).  Partials
// are double-buffered by the caller (consecutive calls alternate buffers) and epochs only grow: a rank can reach call
// k + 2, whose GEMM overwrites buffer k % 2, only after every peer has arrived at call k + 1, i.e. finished reading
// call k.  An expired wait sets the status word and the kernel finishes (garbage out, no hang).  The epoch is the
// sum of a launch argument and an optional device word, so a step captured once as a CUDA graph (arguments frozen) can be
// replayed: the word is advanced by the number of reductions per step at the end of every step.
#include "q4b_internal.h"

namespace q4b {

namespace {

constexpr int MAX_RANKS = 8;

struct ArArgs {
  const float* parts[MAX_RANKS];   // this call's partial of every rank (peer-mapped), [rows, H]
  uint32_t* flags[MAX_RANKS];      // every rank's flag array [world, rows]
  float* h;                        // [rows, H], replicated residual stream
  const float* nw;                 // RMSNorm weights [H], or null: no normalise / quantise
  int8_t* xq;
  __half* xd;
  uint32_t* status;
  const uint32_t* epoch_base;      // device word added to `epoch` (lets a captured graph replay with growing epochs), or null
  float eps;
  int rank, world, rows, H;
  uint32_t epoch, wait_limit;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// peer data: system-scope relaxed loads, never served from a stale line of this SM's L1
__device__ __forceinline__ float4 ld_peer4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(1024) tp_allreduce_kernel(const ArArgs a) {
  __shared__ float red[32];
  __shared__ int expired;
  const int row = blockIdx.x, t = threadIdx.x, i0 = 4 * t;
  pdl_launch_dependents();
  pdl_wait();                                             // this rank's partial is complete
  if (t == 0) expired = 0;
  const uint32_t epoch = a.epoch + (a.epoch_base ? *a.epoch_base : 0u);
  if (t < a.world && t != a.rank) {
    __threadfence_system();
    st_release_sys(a.flags[t] + (size_t)a.rank * a.rows + row, epoch);
    const uint32_t* mine = a.flags[a.rank] + (size_t)t * a.rows + row;
    bool ok = false;
    for (uint32_t i = 0; i < a.wait_limit; ++i) {
      if ((int32_t)(ld_acquire_sys(mine) - epoch) >= 0) {
        ok = true;
        break;
      }
      __nanosleep(64);
    }
    if (!ok) expired = 1;                                 // benign race: any writer stores 1
  }
  __syncthreads();
  if (expired && t == 0) atomicOr(a.status, 2u);

  const bool live = i0 < a.H;
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 hv = sum;
  if (live) {
    hv = *reinterpret_cast<const float4*>(a.h + (size_t)row * a.H + i0);
    float4 pv[MAX_RANKS];
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r)                   // all peer loads in flight together
      if (r < a.world) pv[r] = ld_peer4(a.parts[r] + (size_t)row * a.H + i0);
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r)
      if (r < a.world) {
        sum.x += pv[r].x; sum.y += pv[r].y; sum.z += pv[r].z; sum.w += pv[r].w;
      }
    hv.x += sum.x; hv.y += sum.y; hv.z += sum.z; hv.w += sum.w;
    *reinterpret_cast<float4*>(a.h + (size_t)row * a.H + i0) = hv;
  }
  if (!a.nw) return;
  // RMSNorm + Q8_1 of the updated row (rmsnorm_q8_1_kernel of quant_q8_1.cu, same operation order)
  float ss = live ? hv.x * hv.x + hv.y * hv.y + hv.z * hv.z + hv.w * hv.w : 0.f;
  ss = warp_sum(ss);
  if ((t & 31) == 0) red[t >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int j = 0; j < (int)(blockDim.x >> 5); ++j) tot += red[j];
  const float rn = rsqrtf(tot / (float)a.H + a.eps);
  float4 wv = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) wv = *reinterpret_cast<const float4*>(a.nw + i0);
  const __half2 p0 = __floats2half2_rn(hv.x * rn * wv.x, hv.y * rn * wv.y);
  const __half2 p1 = __floats2half2_rn(hv.z * rn * wv.z, hv.w * rn * wv.w);
  const float2 fa = __half22float2(p0), fb = __half22float2(p1);
  const float v[4] = {fa.x, fa.y, fb.x, fb.y};
  const size_t at = live ? (size_t)row * a.H + i0 : 0;
  quant_block4(v, a.xq + at, a.xd + (at >> 5), nullptr, t & 7, live);   // whole 8-lane groups are live or dead together
}

__global__ void tp_epoch_advance_kernel(uint32_t* base, uint32_t by) {
  pdl_launch_dependents();
  pdl_wait();                                             // every reduction of the step has read the old value
  if (threadIdx.x == 0) *base += by;
}

}  // namespace

int tp_epoch_advance(uint32_t* base, uint32_t by, cudaStream_t st) {
  if (!base) return fail(Q4B_E_ALIGN, "tp_epoch_advance: null pointer");
  return check_launch(launch_pdl(tp_epoch_advance_kernel, dim3(1), dim3(32), 0, st, base, by), "tp_epoch_advance");
}

int tp_allreduce(const void* const* parts, void* const* flags, int rank, int world, uint32_t epoch, const uint32_t* epoch_base,
                 float* h, int rows, int H,
                 const float* norm_w, float eps, void* xq, void* xd, uint32_t* status, uint32_t wait_limit, cudaStream_t st) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return fail(Q4B_E_ARG, "tp_allreduce: 1 <= world <= 8, 0 <= rank < world");
  if (rows <= 0 || H <= 0 || (H % 32) || H > 4096) return fail(Q4B_E_SHAPE, "tp_allreduce: rows > 0, H a multiple of 32, at most 4096");
  if (!parts || !flags || !h || !status || !aligned16(h)) return fail(Q4B_E_ALIGN, "tp_allreduce: null or misaligned pointer");
  if (norm_w && (!xq || !xd || !aligned16(norm_w) || (reinterpret_cast<uintptr_t>(xq) & 3u)))
    return fail(Q4B_E_ALIGN, "tp_allreduce: the fused RMSNorm + Q8_1 needs norm weights, xq and xd");
  ArArgs a{};
  for (int r = 0; r < world; ++r) {
    if (!parts[r] || !aligned16(parts[r]) || (world > 1 && !flags[r])) return fail(Q4B_E_ALIGN, "tp_allreduce: null or misaligned peer pointer");
    a.parts[r] = reinterpret_cast<const float*>(parts[r]);
    a.flags[r] = reinterpret_cast<uint32_t*>(flags[r]);
  }
  a.h = h;
  a.nw = norm_w;
  a.xq = reinterpret_cast<int8_t*>(xq);
  a.xd = reinterpret_cast<__half*>(xd);
  a.status = status;
  a.epoch_base = epoch_base;
  a.eps = eps;
  a.rank = rank; a.world = world; a.rows = rows; a.H = H;
  a.epoch = epoch;
  a.wait_limit = wait_limit ? wait_limit : (1u << 24);   // polls with a 64 ns sleep each: several seconds at most
  const int threads = ((H / 4 + 31) / 32) * 32;
  return check_launch(launch_pdl(tp_allreduce_kernel, dim3(rows), dim3(threads), 0, st, a), "tp_allreduce");
}

}  // namespace q4b
