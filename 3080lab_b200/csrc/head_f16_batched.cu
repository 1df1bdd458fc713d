// LM head over the tied fp16 embedding table for B = 1..32 sequences: logits[b, v] = sum_k E[v, k] * x[b, k], fp32
// accumulation.  The reference's batched engines use a tensor-core head over their own packed table
// (head_v2_source, lab/qwen_batched.py:681-833) or cuBLAS fp16 (scripts/qwen_batched_decode.py:183-185); with a tied
// fp16 table the same job is a plain fp16 stream.
//
// HBM-bound (V x H x 2 bytes once per step), so the job of the tensor cores here is only to keep the instruction count
// per byte low: mma.sync.m16n8k16 (fp16 in, fp32 out), 16 vocabulary rows per warp step, 8 sequences per n-tile.  The
// k order inside an MMA is free as long as both operands agree, which lets every lane read plain 16-byte chunks:
// lane (g, t) takes halves [32 s + 8 t, +8) of rows g and g + 8 (two MMAs' worth of A) and the same 16 bytes of
// x row 8 j + g for n-tile j (both B registers of both MMAs).  x lives in shared memory for the whole kernel.
#include "q4b_internal.h"

namespace q4b {

namespace {


__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NB n-tiles of 8 sequences; HBT threads.  A warp keeps 4 spans x 2 rows x 16 bytes per lane in flight: 16 warps = 64 KB per SM,
// what the HBM latency asks for (8 warps: 114 us for the 1.5B table at 8 sequences, 179 us at 32; 16 warps: 82 and 94 us).
// Up to 8 sequences keep 8 warps all the same: inside the Q8_1 decode step the 16-warp form made the STEP 39 us slower
// although the kernel itself was 31 us faster (measured repeatedly; the cause was not isolated).
template <int NB, int HBT>
__global__ void __launch_bounds__(HBT, 1) head_f16_batched_kernel(const uint4* __restrict__ E, const __half* x,
                                                                  float* logits, int V, int H, int B) {
  extern __shared__ __align__(16) uint8_t xs[];         // [8 NB][pitch] fp16, pitch = 2 H + 64 bytes (conflict-free)
  constexpr int HBW = HBT / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int HC = H >> 3;                                 // 16-byte chunks per row
  const uint32_t pitch = (uint32_t)H * 2 + 64;
  pdl_launch_dependents();
  pdl_wait();
  for (int i = threadIdx.x; i < 8 * NB * HC; i += HBT) {
    const int n = i / HC, c = i - n * HC;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (n < B) v = *reinterpret_cast<const uint4*>(x + (size_t)n * H + (size_t)c * 8);
    *reinterpret_cast<uint4*>(xs + n * pitch + c * 16) = v;
  }
  __syncthreads();
  const int spans = H >> 5;                              // 32 k per step (two MMAs)
  const int groups = (V + 15) >> 4;
  for (int grp = blockIdx.x * HBW + warp; grp < groups; grp += gridDim.x * HBW) {
    const int r0 = grp * 16;
    const int ra = min(r0 + g, V - 1), rb = min(r0 + g + 8, V - 1);
    const uint4* pa = E + (size_t)ra * HC + t;
    const uint4* pb = E + (size_t)rb * HC + t;
    float acc[NB][4];
#pragma unroll
    for (int j = 0; j < NB; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    constexpr int UN = HBT == 256 ? 8 : 4;               // spans in flight: 64 KB per SM either way
    for (int s0 = 0; s0 < spans; s0 += UN) {
      uint4 wa[UN], wb[UN];
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const int s = min(s0 + u, spans - 1);
        wa[u] = ldg_stream16(pa + 4 * s);
        wb[u] = ldg_stream16(pb + 4 * s);
      }
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        if (s0 + u < spans) {
#pragma unroll
          for (int j = 0; j < NB; ++j) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xs + (8 * j + g) * pitch + ((s0 + u) * 4 + t) * 16);
            mma16816(acc[j], wa[u].x, wb[u].x, wa[u].y, wb[u].y, xv.x, xv.y);
            mma16816(acc[j], wa[u].z, wb[u].z, wa[u].w, wb[u].w, xv.z, xv.w);
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      const int n0 = 8 * j + 2 * t;
      if (r0 + g < V) {
        if (n0 < B) logits[(size_t)n0 * V + r0 + g] = acc[j][0];
        if (n0 + 1 < B) logits[(size_t)(n0 + 1) * V + r0 + g] = acc[j][1];
      }
      if (r0 + g + 8 < V) {
        if (n0 < B) logits[(size_t)n0 * V + r0 + g + 8] = acc[j][2];
        if (n0 + 1 < B) logits[(size_t)(n0 + 1) * V + r0 + g + 8] = acc[j][3];
      }
    }
  }
}

template <int NB, int HBT>
int launch_hb(const void* E, const void* x, float* logits, int V, int H, int B, cudaStream_t st) {
  constexpr int HBW = HBT / 32;
  const size_t smem = (size_t)8 * NB * ((size_t)H * 2 + 64);
  auto kern = head_f16_batched_kernel<NB, HBT>;
  if (smem > 48 * 1024) {
    if (cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), 200 * 1024); e != cudaSuccess) {
      set_cuda_error(e, "head_f16_batched: cudaFuncSetAttribute");
      return Q4B_E_CUDA;
    }
  }
  int grid = sm_count();
  const int groups = (V + 15) / 16;
  if (grid * HBW > groups) grid = (groups + HBW - 1) / HBW;
  return check_launch(launch_pdl(kern, dim3(grid), dim3(HBT), smem, st, reinterpret_cast<const uint4*>(E),
                                 reinterpret_cast<const __half*>(x), logits, V, H, B),
                      "head_f16_batched");
}

}  // namespace

int head_f16_batched(const void* E, const void* x, float* logits, int V, int H, int B, cudaStream_t st) {
  if (V <= 0 || H <= 0 || (H % 32) || B < 1 || B > 32) return fail(Q4B_E_SHAPE, "head_f16_batched: need V > 0, H a multiple of 32, 1 <= B <= 32");
  if ((size_t)32 * ((size_t)H * 2 + 64) > 200 * 1024 && B > 16) return fail(Q4B_E_SHAPE, "head_f16_batched: H too large for 32 sequences");
  if (!E || !x || !logits || !aligned16(E) || !aligned16(x)) return fail(Q4B_E_ALIGN, "head_f16_batched: null or misaligned pointer");
  if (B <= 8) return launch_hb<1, 256>(E, x, logits, V, H, B, st);
  if (B <= 16) return launch_hb<2, 512>(E, x, logits, V, H, B, st);
  return launch_hb<4, 512>(E, x, logits, V, H, B, st);
}

}  // namespace q4b
