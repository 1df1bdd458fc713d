// Internal declarations shared by the .cu files of libq4b200.  Not installed; the public C-ABI is include/q4b200.h.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <set>
#include <utility>

#include "../../include/q4b200.h"

namespace q4b {

// Last CUDA error text seen by a launcher on this thread (read through q4b_last_error()).
void set_cuda_error(cudaError_t e, const char* where);
int fail(int code, const char* msg);

inline int check_launch(const char* where) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_cuda_error(e, where);
    return Q4B_E_CUDA;
  }
  return Q4B_OK;
}

inline int check_launch(cudaError_t e, const char* where) {
  if (e != cudaSuccess) {
    set_cuda_error(e, where);
    return Q4B_E_CUDA;
  }
  return check_launch(where);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int sm_count();

// The kernels of the batch-1 decode chain (streaming GEMV, one-sequence attention) ask for the largest shared-memory
// carve-out.  An SM can change its L1 / shared-memory split only while it is idle, so a kernel that wants a different
// split than the one running cannot place a CTA beside it; with one split along the chain the CTAs of a
// programmatically dependent launch can move in while their predecessor is still running, which is what lets their
// weight prefetch overlap it.  Kernels that lean on L1 (the fp16 heads, the batched paths) keep the default: with the
// preference applied to every kernel the batch-1 head lost 6 % and the 8-sequence step 16 %.  Once per (kernel, device).
inline void prefer_max_shared(const void* kern) {
  static std::mutex mu;
  static std::set<std::pair<const void*, int>> done;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  std::lock_guard<std::mutex> lock(mu);
  if (done.insert({kern, dev}).second)
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) is per device: raise the limit of `kern` to `bytes` once per (kernel,
// device), so that a process that drives several GPUs configures each of them.  Returns a cudaError_t.
inline cudaError_t ensure_dynamic_smem(const void* kern, size_t bytes) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, size_t> done;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  size_t& have = done[{kern, dev}];
  if (bytes <= have) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess) have = bytes;
  return e;
}

// Ranges a batch-1 GEMV launch asks to be brought into L2 for launches further down the chain (see gemv_mma.cu).
struct GemvLookahead {
  const void* ptr[4];
  size_t bytes[4];
};

// Chain timeline (q4b_trace_chain): while a buffer is set, every traced launch gets its own region of 16 stamps per CTA
// and a host-side record (kernel id, CTAs, offset), so a captured graph keeps writing the same regions on every replay.
unsigned long long* trace_slot(int kernel_id, int ctas);

// Launch with the programmatic-dependent-launch attribute: the kernel may start while its predecessor in the stream is
// still running, so it must call pdl_wait() before it touches anything the predecessor writes (every kernel in this
// library does so before its first dependent access).  Captured into CUDA graphs as a programmatic edge.
// Consequence for loads: a buffer written by an earlier kernel of the chain is NOT read-only for the lifetime of this
// grid (the grid may have been resident before the write), so it must never be read through the non-coherent path
// (__ldg / ld.global.nc, or a const __restrict__ pointer the compiler may route there).  Only weights and tables are.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Same, with the CTAs grouped into thread-block clusters of (cx, cy, 1).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, unsigned cx,
                                      unsigned cy, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cx;
  attr[1].val.clusterDim.y = cy;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ---- device helpers -------------------------------------------------------------------------------------------
#ifdef __CUDACC__
// Exact nibble -> fp32: bits (0x4B000000 | q) are the float 2^23 + q, so subtracting 2^23 + 8 leaves q - 8.
__device__ __forceinline__ float nib_f32(uint32_t w, int i) {
  return __int_as_float(((w >> (4 * i)) & 15u) | 0x4B000000u) - 8388616.0f;
}

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Thread-block cluster helpers: full barrier (release/acquire) and a 4-byte read of a peer CTA's shared memory at the
// address `local` has in this CTA.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_peer_f32(const float* local, uint32_t rank) {
  uint32_t a;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
  return v;
}

// NeoX rotation of the pair (a, b) = (x[d], x[d + HD/2]) by the angle whose cosine / sine are c / s, with the operation
// order pinned so that every kernel that rotates the same values produces the same bits.
__device__ __forceinline__ void rope_pair(float a, float b, float c, float s, float& lo, float& hi) {
  lo = __fmaf_rn(a, c, -__fmul_rn(b, s));
  hi = __fmaf_rn(b, c, __fmul_rn(a, s));
}

// Byte offset, inside a 4608-byte record of the tiled Q8_1 format (one 128-row tile x one 32-value block), of element i
// of row n: 8-row x 16-byte core matrices, the 32 bytes of a block permuted as the nibble expansion permutes the weights.
__device__ __forceinline__ uint32_t q8_tiled_offset(int n, int i) {
  const int pos = 4 * (2 * (i >> 3) + (i & 1)) + ((i & 7) >> 1);
  return (uint32_t)((n >> 3) * 256 + (n & 7) * 16 + (pos >> 4) * 128 + (pos & 15));
}

// Q8_1 quantiser of one 32-value block (QUANT_Q8, lab/qwen_batched.py:1030-1039), planar output.
// 8 lanes per block, 4 consecutive values per lane: each lane reads 8 bytes and writes 4.
__device__ __forceinline__ void quant_block4(const float x[4], int8_t* q_out, __half* d_out, __half* s_out, int lane_in_blk,
                                             bool live) {
  float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
  for (int o = 4; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float d = amax / 127.f;
  int q[4], sq = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    q[i] = d > 0.f ? __float2int_rn(x[i] / d) : 0;
    sq += q[i];
  }
  if (live) {
    const uint32_t packed = (uint32_t)(q[0] & 0xFF) | ((uint32_t)(q[1] & 0xFF) << 8) | ((uint32_t)(q[2] & 0xFF) << 16) |
                            ((uint32_t)(q[3] & 0xFF) << 24);
    *reinterpret_cast<uint32_t*>(q_out) = packed;
  }
#pragma unroll
  for (int o = 4; o; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  if (live && lane_in_blk == 0) {
    *d_out = __float2half_rn(d);
    if (s_out) *s_out = __float2half_rn(d * (float)sq);
  }
}

// Tiled output for the prefill MMQ: per (tile of 128 rows, k-block) 4096 bytes in the UMMA K-major core-matrix order
// (8-row x 16-byte core matrices, the 32 bytes of a block permuted as the nibble expansion permutes the weights:
// position 4 (2 (i / 8) + (i & 1)) + (i & 7) / 2 for element i) followed by the 128 block scales as fp32.  Lane `sub`
// holds elements 4 sub .. 4 sub + 3: elements {0, 2} and {1, 3} land on adjacent bytes, two 16-bit stores.
__device__ __forceinline__ void quant_block4_tiled(const float x[4], uint8_t* tile, int n, int sub) {
  float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
  for (int o = 4; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float d = amax / 127.f;
  int q[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) q[i] = d > 0.f ? __float2int_rn(x[i] / d) : 0;
  const int pos02 = 8 * (sub >> 1) + 2 * (sub & 1), pos13 = pos02 + 4;
  uint8_t* rowp = tile + (n >> 3) * 256 + (n & 7) * 16;
  *reinterpret_cast<uint16_t*>(rowp + (pos02 >> 4) * 128 + (pos02 & 15)) = (uint16_t)((q[0] & 0xFF) | ((q[2] & 0xFF) << 8));
  *reinterpret_cast<uint16_t*>(rowp + (pos13 >> 4) * 128 + (pos13 & 15)) = (uint16_t)((q[1] & 0xFF) | ((q[3] & 0xFF) << 8));
  if (sub == 0) reinterpret_cast<float*>(tile + 4096)[n] = __half2float(__float2half_rn(d));
}

// Programmatic dependent launch: wait for the kernels this one depends on / let dependents start their prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

}  // namespace q4b
