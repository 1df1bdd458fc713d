// Measured peak of the int8 tensor-core path this library uses: tcgen05.mma.kind::i8, M = 128, N = 256, K = 32, issued
// back to back by one thread per SM onto ONE accumulator tile (so nothing but the tensor pipe limits it), operands in
// shared memory.  The benchmark reports the prefill MMQ against this number as well as against the nominal figure.
// (Reference: the lab measures its own peaks the same way, lab/experiments/tensor.py.)
#include "q4b_internal.h"
#include "tc05.cuh"

namespace q4b {

namespace {

constexpr int PK_N = 256;

__global__ void __launch_bounds__(128, 1) peak_i8_kernel(int iters, uint32_t* status) {
  extern __shared__ __align__(128) uint8_t smem[];       // A: 128 x 32 bytes, B: 256 x 32 bytes, K-major core matrices
  __shared__ __align__(8) uint64_t done;
  __shared__ uint32_t tmem_base_s;
  const int t = threadIdx.x, warp = t >> 5;
  for (int i = t; i < (128 + PK_N) * 32 / 4; i += 128) reinterpret_cast<uint32_t*>(smem)[i] = 0x01010101u;
  if (warp == 0) {
    tc::tmem_alloc(&tmem_base_s, 256);
    tc::tmem_relinquish();
  }
  if (t == 0) {
    tc::mbar_init(&done, 1);
    tc::mbar_fence_init();
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  if (t == 0) {
    const uint32_t tmem = tmem_base_s;
    const uint64_t adesc = tc::smem_desc_kmajor(tc::smem_u32(smem), 128, 256);
    const uint64_t bdesc = tc::smem_desc_kmajor(tc::smem_u32(smem + 128 * 32), 128, 256);
    constexpr uint32_t IDESC = tc::idesc_i8(128, PK_N);
    for (int i = 0; i < iters; ++i) tc::mma_i8_ss(tmem, adesc, bdesc, IDESC, i > 0 ? 1u : 0u);
    tc::mma_commit(&done);
    if (!tc::mbar_wait(&done, 0)) atomicExch(status, 1u);
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base_s, 256);
}

}  // namespace

// -> int8 operations (2 per multiply-accumulate) executed by one launch; 0 on a launch error (text in q4b_last_error)
double peak_i8_launch(int iters, uint32_t* status, cudaStream_t st) {
  if (iters <= 0 || !status) return 0.0;
  const int sms = sm_count();
  const size_t smem = (size_t)(128 + PK_N) * 32;
  peak_i8_kernel<<<sms, 128, smem, st>>>(iters, status);
  if (check_launch("peak_i8") != Q4B_OK) return 0.0;
  return 2.0 * 128.0 * PK_N * 32.0 * (double)iters * (double)sms;
}

}  // namespace q4b
