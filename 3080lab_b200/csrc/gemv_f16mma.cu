// Batched-decode Q4_0 GEMV on fp16 tensor-core MMAs: up to 32 activation rows against weights dequantised to fp16.
//
//   Y[b, m] = epilogue( sum_k w16[m, k] * X[b, k] ),    w16[m, k] = round_fp16( (q4[m, k] - 8) * d[m, k / 32] )
//
// This is the arithmetic of the reference's batched-decode linears (gemv_v2_source, lab/qwen_batched.py:467-641):
// nibbles become exact fp16 integers through the 0x6400 exponent trick, are multiplied by the fp16 block scale with ONE
// rounding to fp16, and meet the fp16 activations in mma.sync.m16n8k16 with fp32 accumulation; epilogues as
// lab/qwen_batched.py:251-267.  The rounding of d * (q - 8) to fp16 is what separates this mode from the exact block-dot
// kernels; tests compare against an oracle that rounds the weights the same way.
//
// Shape of the kernel (B200), shared with the batch-1 GEMV of gemv_mma.cu:
//   * one CTA = one 128-row tile x one K slice of the tile-packed layout (pack.cu): its weights are ONE contiguous range,
//     fetched by a few 1-D bulk copies BEFORE the programmatic-dependency wait; after the wait one bulk copy per
//     activation row brings the K slice of X into a padded (conflict-free) shared-memory image;
//   * 16 warps = 4 row groups (two m16 tiles each) x 4 k groups; a lane reads 4 bytes of nibbles per row and k-block
//     and keeps that natural byte order: logical k slots of the MMA are a permutation of the block's 32 weights, and the
//     activation fragment is permuted to match with two byte-permutes, so no repacked weight copy is needed;
//   * the k groups are added in a fixed order through shared memory, K slices through the thread-block cluster
//     (every CTA pulls the partial sums of its share of the rows from its peers in rank order): bit-repeatable.
// Every wait is bounded (status word + fall through).
#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>

#include "q4b_internal.h"
#include "tc05.cuh"

namespace q4b {

namespace {

constexpr int GT = 512;
constexpr int ROWS = 128;
constexpr int CHK = 8;                  // k-blocks per weight bulk copy
constexpr int MAX_CHUNKS = 12;
constexpr int PSTR = ROWS + 4;          // row pitch of the partial-sum tile (floats): fragment stores hit 32 banks
constexpr size_t MAX_DYN_SMEM = 226 * 1024;

struct F16Args {
  const uint8_t* W;      // tile-packed nibbles [T, K/32, 128, 16 bytes]
  const __half* S;       // tile-packed scales [T, K/32, 128]
  const __half* X;       // [B, K]
  void* Y;               // [B, ldy]
  const void* AUX;
  uint32_t* status;
  int N, K, KB, B, epi, ldy, ksplit, cap;
  uint32_t wait_limit;
};

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   tc::smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(tc::smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }

// Two nibbles of `w` (bit positions 0-3 and 16-19, or 4-7 and 20-23) -> fp16 pair round((q - 8) * d).
// low form: (q | 0x6400) is the fp16 1024 + q, minus 1032 is q - 8 exactly; high form (nibble at bits 4-7 / 20-23):
// 1024 + 16 q, times 1/16 minus 72 is q - 8 exactly as well (one fused multiply-add, no rounding: the result is an integer
// of at most 4 bits).  The product with d rounds once, as the reference's __hmul2 does.
__device__ __forceinline__ uint32_t deq_lo(uint32_t w, __half2 d2) {
  const uint32_t h = (w & 0x000F000Fu) | 0x64006400u;
  return h2_as_u32(__hmul2(__hsub2(u32_as_h2(h), __float2half2_rn(1032.f)), d2));
}
__device__ __forceinline__ uint32_t deq_hi(uint32_t w, __half2 d2) {
  const uint32_t h = (w & 0x00F000F0u) | 0x64006400u;
  return h2_as_u32(__hmul2(__hfma2(u32_as_h2(h), __float2half2_rn(0.0625f), __float2half2_rn(-72.f)), d2));
}

__device__ __forceinline__ bool mbar_wait_n(uint64_t* bar, uint32_t parity, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i)
    if (tc::mbar_try(bar, parity)) return true;
  return false;
}

// 8-byte read of a peer CTA's shared memory at the address `local` has in this CTA
__device__ __forceinline__ float2 ld_peer_f32x2(const float* local, uint32_t rank) {
  uint32_t addr;
  float2 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(tc::smem_u32(local)), "r"(rank));
  asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr) : "memory");
  return v;
}

// bytes per staged activation row: an odd multiple of 64, so that the 16-byte fragment reads of a quarter warp (two
// rows x 64 bytes) fall into distinct banks
__host__ __device__ __forceinline__ size_t x_pitch(int cap) { return (size_t)(cap | 1) * 64; }

template <int NT>
__global__ void __launch_bounds__(GT, NT <= 2 ? 2 : 1) gemv_f16mma_kernel(const F16Args a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bar_load[MAX_CHUNKS];
  __shared__ __align__(8) uint64_t bar_x;

  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int rg = warp & 3, kg = warp >> 2;
  const int g = lane >> 2, tq = lane & 3;
  const int tile = blockIdx.x, ks = blockIdx.y;
  pdl_launch_dependents();
  const int kb0 = (int)(((long long)a.KB * ks) / a.ksplit), kb1 = (int)(((long long)a.KB * (ks + 1)) / a.ksplit);
  const int nkb = kb1 - kb0;
  const int cap = a.cap;                                  // k-blocks per window of the slab (nkb <= cap except for very long K)
  const size_t xp = x_pitch(cap);
  uint8_t* slabW = smem;                                  // [k-block][128 rows][16 bytes]
  uint8_t* slabS = slabW + (size_t)cap * 2048;            // [k-block][128 rows] fp16
  uint8_t* xs = slabS + (size_t)cap * 256;                // [8 NT rows][pitch] fp16: the K window of X
  float* P = reinterpret_cast<float*>(xs + (size_t)NT * 8 * xp);   // [8 NT columns][PSTR]: this CTA's partial sums

  // window `win` covers k-blocks kb0 + win cap .. of this CTA's slice; lane c of warp 0 owns weight chunk c
  auto issue_weights = [&](int win) {
    const int wkb = min(cap, nkb - win * cap), c = t;
    if (c * CHK < wkb) {
      const size_t kbg = (size_t)tile * a.KB + kb0 + (size_t)win * cap;
      const int n = min(CHK, wkb - c * CHK);
      tc::mbar_expect_tx(&bar_load[c], (uint32_t)n * (2048 + 256));
      bulk_g2s(slabW + (size_t)c * CHK * 2048, a.W + (kbg + (size_t)c * CHK) * 2048, (uint32_t)n * 2048, &bar_load[c]);
      bulk_g2s(slabS + (size_t)c * CHK * 256, a.S + (kbg + (size_t)c * CHK) * 128, (uint32_t)n * 256, &bar_load[c]);
    }
  };
  auto issue_x = [&](int win) {                           // warp 1: one bulk copy per activation row
    const int wkb = min(cap, nkb - win * cap);
    if (lane == 0) tc::mbar_expect_tx(&bar_x, (uint32_t)a.B * (uint32_t)wkb * 64u);
    __syncwarp();
    if (lane < a.B)
      bulk_g2s(xs + (size_t)lane * xp, a.X + (size_t)lane * a.K + ((size_t)kb0 + (size_t)win * cap) * 32, (uint32_t)wkb * 64u, &bar_x);
  };

  if (t < MAX_CHUNKS) {
    tc::mbar_init(&bar_load[t], 1);
    tc::mbar_fence_init();
    issue_weights(0);                                     // weights do not depend on the previous kernel
  }
  if (t == 32) {
    tc::mbar_init(&bar_x, 1);
    tc::mbar_fence_init();
  }
  // activation rows B .. 8 NT - 1 do not exist: their MMA columns read zeros
  for (int i = t; i < (NT * 8 - a.B) * (int)(xp / 16); i += GT)
    reinterpret_cast<uint4*>(xs + (size_t)a.B * xp)[i] = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();
  pdl_wait();                                             // X comes from the previous kernel
  if (warp == 1) issue_x(0);

  // ---- main loop: rows rg * 32 + {g, g + 8, g + 16, g + 24}, k-blocks kg, kg + 4, ... of each window
  // A lane holds word tq of each row's 16 bytes (nibble i = weight 8 tq + i).  Logical k slot -> weight of the block:
  // MMA 0 (nibbles 0, 4, 2, 6) slot 2 tq + {0, 1, 8, 9} = weight 8 tq + {0, 4, 2, 6}; MMA 1 (nibbles 1, 5, 3, 7) the same + 1.
  float c[2][NT][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int n = 0; n < NT; ++n) c[m][n][0] = c[m][n][1] = c[m][n][2] = c[m][n][3] = 0.f;
  const uint8_t* wp0 = slabW + (size_t)(rg * 32 + g) * 16 + 4 * tq;
  const __half* sp0 = reinterpret_cast<const __half*>(slabS) + rg * 32 + g;
  const uint8_t* xp0 = xs + (size_t)g * xp + tq * 16;
  bool ok = true;
  const int nwin = (nkb + cap - 1) / cap;
#pragma unroll 1
  for (int win = 0; win < nwin; ++win) {
    const int wkb = min(cap, nkb - win * cap);
    const uint32_t parity = (uint32_t)win & 1u;
    if (win > 0) {
      // every warp is done reading the previous window (the barrier closing the loop body); order those generic-proxy
      // reads before the bulk copies that overwrite the slab
      tc::fence_async_smem();
      if (t < MAX_CHUNKS) issue_weights(win);
      if (warp == 1) issue_x(win);
    }
    // warp w polls weight chunk w, the last warp the activations; the block barrier publishes the bulk-copied bytes to
    // everyone.  (Polling each chunk inside the loop instead, to start the MMAs while later chunks are in flight, was
    // measured slower: gate/up at 8 rows 7.9 us against 7.0.)
    if (lane == 0) {
      for (int ch = warp; ch * CHK < wkb; ch += GT / 32) ok = mbar_wait_n(&bar_load[ch], parity, a.wait_limit) && ok;
      if (warp == GT / 32 - 1) ok = mbar_wait_n(&bar_x, parity, a.wait_limit) && ok;
    }
    __syncthreads();
#pragma unroll 1
    for (int kb = kg; kb < wkb; kb += 4) {
      uint32_t w[4];
      __half2 d2[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        w[r] = *reinterpret_cast<const uint32_t*>(wp0 + (size_t)kb * 2048 + r * 8 * 16);
        d2[r] = __half2half2(sp0[kb * 128 + r * 8]);
      }
      uint32_t b[NT][4];                                  // {MMA 0 b0, MMA 0 b1, MMA 1 b0, MMA 1 b1}
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const uint4 x = *reinterpret_cast<const uint4*>(xp0 + (size_t)n * 8 * xp + (size_t)kb * 64);   // x[8 tq .. 8 tq + 7]
        b[n][0] = __byte_perm(x.x, x.z, 0x5410);          // x[8 tq + 0], x[8 tq + 4]
        b[n][1] = __byte_perm(x.y, x.w, 0x5410);          // x[8 tq + 2], x[8 tq + 6]
        b[n][2] = __byte_perm(x.x, x.z, 0x7632);          // x[8 tq + 1], x[8 tq + 5]
        b[n][3] = __byte_perm(x.y, x.w, 0x7632);          // x[8 tq + 3], x[8 tq + 7]
      }
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        const uint32_t wA = w[2 * m], wB = w[2 * m + 1];
        const uint32_t wA8 = wA >> 8, wB8 = wB >> 8;
        {
          const uint32_t a0 = deq_lo(wA, d2[2 * m]), a1 = deq_lo(wB, d2[2 * m + 1]);
          const uint32_t a2 = deq_lo(wA8, d2[2 * m]), a3 = deq_lo(wB8, d2[2 * m + 1]);
#pragma unroll
          for (int n = 0; n < NT; ++n) mma_f16(c[m][n], a0, a1, a2, a3, b[n][0], b[n][1]);
        }
        {
          const uint32_t a0 = deq_hi(wA, d2[2 * m]), a1 = deq_hi(wB, d2[2 * m + 1]);
          const uint32_t a2 = deq_hi(wA8, d2[2 * m]), a3 = deq_hi(wB8, d2[2 * m + 1]);
#pragma unroll
          for (int n = 0; n < NT; ++n) mma_f16(c[m][n], a0, a1, a2, a3, b[n][2], b[n][3]);
        }
      }
    }
    __syncthreads();
  }

  // ---- k groups added in order 0, 1, 2, 3 into P[column][row]
#pragma unroll 1
  for (int s = 0; s < 4; ++s) {
    if (kg == s) {
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          float* p0 = P + (size_t)(n * 8 + 2 * tq) * PSTR + rg * 32 + 16 * m + g;
          if (s == 0) {
            p0[0] = c[m][n][0]; p0[PSTR] = c[m][n][1]; p0[8] = c[m][n][2]; p0[PSTR + 8] = c[m][n][3];
          } else {
            p0[0] += c[m][n][0]; p0[PSTR] += c[m][n][1]; p0[8] += c[m][n][2]; p0[PSTR + 8] += c[m][n][3];
          }
        }
    }
    __syncthreads();
  }

  // ---- K slices: CTA `ks` of the cluster finishes row pairs [64 ks / ksplit, 64 (ks + 1) / ksplit) of the tile
  int pr0 = 0, pr1 = ROWS / 2;
  if (a.ksplit > 1) {
    cluster_sync_all();                                                     // every peer's P is complete and visible
    pr0 = (ROWS / 2 * ks) / a.ksplit;
    pr1 = (ROWS / 2 * (ks + 1)) / a.ksplit;
  }
  const int npr = pr1 - pr0;
  for (int i = t; i < npr * a.B; i += GT) {
    const int col = i / npr, pr = pr0 + (i - col * npr);
    const float* src = P + (size_t)col * PSTR + 2 * pr;
    float v0 = 0.f, v1 = 0.f;
    if (a.ksplit > 1) {
      for (int r = 0; r < a.ksplit; ++r) {                                  // rank order, whoever does the adding
        const float2 pv = ld_peer_f32x2(src, (uint32_t)r);
        v0 += pv.x;
        v1 += pv.y;
      }
    } else {
      v0 = src[0];
      v1 = src[1];
    }
    const int row = tile * ROWS + 2 * pr;
    if (row >= a.N) continue;
    const bool two = row + 1 < a.N;
    const size_t o = (size_t)col * a.ldy + row;
    switch (a.epi) {
      case Q4B_EPI_STORE: {
        __half* Y = reinterpret_cast<__half*>(a.Y);
        Y[o] = __float2half_rn(v0);
        if (two) Y[o + 1] = __float2half_rn(v1);
        break;
      }
      case Q4B_EPI_BIASF: {
        __half* Y = reinterpret_cast<__half*>(a.Y);
        const float* bias = reinterpret_cast<const float*>(a.AUX);
        Y[o] = __float2half_rn(v0 + bias[row]);
        if (two) Y[o + 1] = __float2half_rn(v1 + bias[row + 1]);
        break;
      }
      case Q4B_EPI_RESID: {
        float* Y = reinterpret_cast<float*>(a.Y);
        Y[o] += v0;
        if (two) Y[o + 1] += v1;
        break;
      }
      case Q4B_EPI_LOGITS: {
        float* Y = reinterpret_cast<float*>(a.Y);
        Y[o] = v0;
        if (two) Y[o + 1] = v1;
        break;
      }
      case Q4B_EPI_SWIGLU:                                                  // rows interleaved gate, up
        if (two) reinterpret_cast<__half*>(a.Y)[(size_t)col * a.ldy + (row >> 1)] = __float2half_rn(v0 / (1.f + __expf(-v0)) * v1);
        break;
      default: break;
    }
  }
  if (!ok) atomicOr(a.status, 1u);
  if (a.ksplit > 1) cluster_sync_all();                   // nobody leaves while a peer may still read its partial sums
}

size_t smem_for(int cap, int nt) {
  return (size_t)cap * (2048 + 256) + (size_t)nt * 8 * x_pitch(cap) + (size_t)nt * 8 * PSTR * sizeof(float);
}

template <int NT>
int prepare(size_t smem) {
  static size_t configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(Q4B_E_CUDA, "gemv_q4_0_f16mma: no current device");
  if (smem > configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_f16mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_DYN_SMEM);
    if (e != cudaSuccess) {
      set_cuda_error(e, "gemv_q4_0_f16mma");
      return Q4B_E_CUDA;
    }
    configured[dev] = MAX_DYN_SMEM;
  }
  return Q4B_OK;
}

// How many clusters of `ks` CTAs with `smem` bytes each can be resident at once (cached per device and configuration):
// a grid of T clusters that does not fit runs in two waves, which a smaller split avoids.
template <int NT>
int resident_clusters(int ks, size_t smem) {
  static std::mutex mu;
  static std::map<std::tuple<int, int, size_t>, int> cache;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  const auto key = std::make_tuple(dev, ks, smem);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(1, ks);
  cfg.blockDim = dim3(GT);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = ks;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemv_f16mma_kernel<NT>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    n = 1 << 30;                                          // unknown: do not constrain the split
  }
  cache[key] = n;
  return n;
}

template <int NT>
int launch(F16Args& a, int T, cudaStream_t st) {
  // K slices: fill the SMs when there are fewer row tiles than SMs; the slab holds `cap` k-blocks of one slice (longer
  // slices run as several windows); prefer a split whose clusters are all resident at once
  int cap_max = CHK * MAX_CHUNKS;
  while (cap_max > 1 && smem_for(cap_max, NT) > MAX_DYN_SMEM) --cap_max;
  int rc = prepare<NT>(MAX_DYN_SMEM);
  if (rc != Q4B_OK) return rc;
  int ks = sm_count() / T;
  ks = ks < 1 ? 1 : (ks > 8 ? 8 : ks);
  if (ks > a.KB) ks = a.KB;
  for (; ks > 1; --ks) {
    const int cap = std::min(cap_max, (a.KB + ks - 1) / ks);
    if (resident_clusters<NT>(ks, smem_for(cap, NT)) >= T) break;
  }
  a.ksplit = ks;
  a.cap = std::min(cap_max, (a.KB + ks - 1) / ks);
  dim3 grid(T, ks), block(GT);
  return check_launch(launch_pdl_cluster(gemv_f16mma_kernel<NT>, grid, block, smem_for(a.cap, NT), st, 1, ks, a), "gemv_q4_0_f16mma");
}

}  // namespace

int gemv_f16mma(const void* W, const void* S, const void* X, void* Y, const void* AUX, int N, int K, int B, int epi, int ldy,
                uint32_t* status, cudaStream_t st) {
  if (N <= 0 || K <= 0 || (K % 32)) return fail(Q4B_E_SHAPE, "gemv_q4_0_f16mma: N > 0 and K a positive multiple of 32 required");
  if (B < 1 || B > 32) return fail(Q4B_E_SHAPE, "gemv_q4_0_f16mma: 1 <= B <= 32 activation rows");
  if (!W || !S || !X || !Y || !status || !aligned16(W) || !aligned16(S) || !aligned16(X))
    return fail(Q4B_E_ALIGN, "gemv_q4_0_f16mma: null or misaligned pointer");
  if (epi < Q4B_EPI_STORE || epi > Q4B_EPI_LOGITS) return fail(Q4B_E_ARG, "gemv_q4_0_f16mma: unknown epilogue");
  if (epi == Q4B_EPI_BIASF && !AUX) return fail(Q4B_E_ALIGN, "gemv_q4_0_f16mma: biasf needs AUX");
  if (epi == Q4B_EPI_SWIGLU && (N % 2)) return fail(Q4B_E_SHAPE, "gemv_q4_0_f16mma: swiglu needs an even row count");
  if (ldy < (epi == Q4B_EPI_SWIGLU ? N / 2 : N)) return fail(Q4B_E_SHAPE, "gemv_q4_0_f16mma: ldy shorter than an output row");
  const int T = (N + ROWS - 1) / ROWS, KB = K / 32, nt = (B + 7) / 8;
  F16Args a{};
  a.W = reinterpret_cast<const uint8_t*>(W);
  a.S = reinterpret_cast<const __half*>(S);
  a.X = reinterpret_cast<const __half*>(X);
  a.Y = Y;
  a.AUX = AUX;
  a.status = status;
  a.N = N; a.K = K; a.KB = KB; a.B = B; a.epi = epi; a.ldy = ldy;
  a.wait_limit = tc::WAIT_LIMIT;
  switch (nt) {
    case 1: return launch<1>(a, T, st);
    case 2: return launch<2>(a, T, st);
    case 3: return launch<3>(a, T, st);
    default: return launch<4>(a, T, st);
  }
}

}  // namespace q4b
