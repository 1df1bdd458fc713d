// Repack canonical Q4_0 (W int32 [N, K/8], S fp16 [N, K/32]) into the tile-packed streaming layout of the tensor-core
// kernels: rows in tiles of 128, and inside a tile k-block-major:
//   Wt int32 [T, K/32, 128, 4]   the 16 bytes of (row r of the tile, k-block b) at ((tile * KB + b) * 128 + r) * 16
//   St fp16  [T, K/32, 128]
// Same bytes as Q4_0 (plus zero padding of the last tile: nibbles 8 = weight 0, scale 0).  A CTA that owns one row
// tile and a run of k-blocks then reads ONE contiguous range, which a single bulk (TMA) copy moves, and thread r finds
// its row's block at a 16-byte stride from its neighbours' (no shared-memory bank conflicts).  The reference repacks
// for its tensor-core kernels in the same spirit (pack_q4_mma / pack_q4_i8, lab/qwen_batched.py:394-436, 987-1013).
#include "q4b_internal.h"

namespace q4b {

namespace {

__global__ void __launch_bounds__(256) pack_q4_0_kernel(const uint4* __restrict__ W, const __half* __restrict__ S,
                                                        uint4* __restrict__ Wt, __half* __restrict__ St, int N, int KB, size_t total) {
  const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;     // index into Wt as uint4: ((tile * KB + b) * 128 + r)
  if (i >= total) return;
  const int r = (int)(i & 127);
  const size_t tb = i >> 7;
  const int b = (int)(tb % KB);
  const size_t tile = tb / KB;
  const size_t row = tile * 128 + r;
  uint4 w = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
  __half s = __float2half_rn(0.f);
  if (row < (size_t)N) {
    w = W[row * KB + b];
    s = S[row * KB + b];
  }
  Wt[i] = w;
  St[i] = s;
}

}  // namespace

int pack_q4_0(const void* W, const void* S, void* Wt, void* St, int N, int K, cudaStream_t st) {
  if (N <= 0 || K <= 0 || (K % 32)) return fail(Q4B_E_SHAPE, "pack_q4_0: N > 0 and K a positive multiple of 32 required");
  if (!W || !S || !Wt || !St || !aligned16(W) || !aligned16(Wt) || !aligned16(St)) return fail(Q4B_E_ALIGN, "pack_q4_0: null or misaligned pointer");
  const int KB = K / 32;
  const size_t total = (size_t)((N + 127) / 128) * KB * 128;
  pack_q4_0_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const uint4*)W, (const __half*)S, (uint4*)Wt, (__half*)St, N, KB, total);
  return check_launch("pack_q4_0");
}

}  // namespace q4b
