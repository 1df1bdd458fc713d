// Q8_1 activation quantiser and the fused RMSNorm + quantise kernel.
//
// Per 32 values: amax = max|x|, d = amax / 127 (fp32 division), q = d > 0 ? rint(x / d) : 0 (fp32 division, round to
// nearest even), exactly the arithmetic of the reference's QUANT_Q8 (lab/qwen_batched.py:1030-1039), so the int8
// values equal the reference's.  Stored per block: the 32 int8 values, d rounded to fp16, and optionally the Q8_1 sum
// term d * sum(q) as fp16.  Layout is planar: xq int8 [P, K], xd fp16 [P, K/32], xsum fp16 [P, K/32].
// The fused form follows rmsnorm_q8_source (lab/qwen_batched.py:1044-1091): the normalised value is rounded to 16 bits
// first, so the result is identical to RMSNorm followed by the quantiser.
#include "q4b_internal.h"

namespace q4b {

namespace {

__global__ void __launch_bounds__(256) quant_q8_1_tiled_kernel(const __half* x, uint8_t* xt, int P, int KB) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t gid = (size_t)blockIdx.x * 256 + threadIdx.x;
  const size_t blk = gid >> 3;
  const int sub = (int)(gid & 7);
  if (blk >= (size_t)P * KB) return;                 // whole 8-lane groups leave together
  const int p = (int)(blk / KB), kb = (int)(blk - (size_t)p * KB);
  const uint2 raw = *reinterpret_cast<const uint2*>(x + blk * 32 + sub * 4);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
  const float v[4] = {a.x, a.y, b.x, b.y};
  quant_block4_tiled(v, xt + ((size_t)(p >> 7) * KB + kb) * 4608, p & 127, sub);
}

// h_add != nullptr: the row is first completed, h[row] += h_add[0][row] + .. (written back), e.g. with the further parts of a
// linear whose launch was split along K; then normalised and quantised as usual.
__global__ void __launch_bounds__(1024) rmsnorm_q8_1_tiled_kernel(const float* h, const float* __restrict__ w, uint8_t* xt,
                                                                  int H, float eps, float* h_add, int n_add) {
  __shared__ float part[32];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, t = threadIdx.x, i0 = 4 * t;
  float4 hv = *reinterpret_cast<const float4*>(h + (size_t)row * H + i0);
  if (h_add) {
    for (int j = 0; j < n_add; ++j) {                    // the addends [n_add][rows, H], in order
      const float4 av = *reinterpret_cast<const float4*>(h_add + ((size_t)j * gridDim.x + row) * H + i0);
      hv.x += av.x; hv.y += av.y; hv.z += av.z; hv.w += av.w;
    }
    *reinterpret_cast<float4*>(const_cast<float*>(h) + (size_t)row * H + i0) = hv;
  }
  const float4 wv = *reinterpret_cast<const float4*>(w + i0);
  float ss = hv.x * hv.x + hv.y * hv.y + hv.z * hv.z + hv.w * hv.w;
  ss = warp_sum(ss);
  if ((t & 31) == 0) part[t >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int j = 0; j < (int)(blockDim.x >> 5); ++j) tot += part[j];
  const float r = rsqrtf(tot / (float)H + eps);
  const float v[4] = {__half2float(__float2half_rn(hv.x * r * wv.x)), __half2float(__float2half_rn(hv.y * r * wv.y)),
                      __half2float(__float2half_rn(hv.z * r * wv.z)), __half2float(__float2half_rn(hv.w * r * wv.w))};
  const int KB = H >> 5;
  quant_block4_tiled(v, xt + ((size_t)(row >> 7) * KB + (i0 >> 5)) * 4608, row & 127, t & 7);
}

// The same row pass with fp16 output in the operand order of the fp16-mode prefill GEMM (per 128-token tile and k-block
// 8192 bytes, [8-token group][8-value chunk][token][16 bytes], a chunk's values as (0,4,1,5,2,6,3,7)).  Two neighbouring
// threads hold the two halves of a chunk and trade one pair of values.
__global__ void __launch_bounds__(1024) rmsnorm_f16_tiled_kernel(const float* h, const float* __restrict__ w, uint8_t* xt, int H,
                                                                 float eps, float* h_add, int n_add) {
  __shared__ float part[32];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, t = threadIdx.x, i0 = 4 * t;
  float4 hv = *reinterpret_cast<const float4*>(h + (size_t)row * H + i0);
  if (h_add) {
    for (int j = 0; j < n_add; ++j) {                    // the addends [n_add][rows, H], in order
      const float4 av = *reinterpret_cast<const float4*>(h_add + ((size_t)j * gridDim.x + row) * H + i0);
      hv.x += av.x; hv.y += av.y; hv.z += av.z; hv.w += av.w;
    }
    *reinterpret_cast<float4*>(const_cast<float*>(h) + (size_t)row * H + i0) = hv;
  }
  const float4 wv = *reinterpret_cast<const float4*>(w + i0);
  float ss = hv.x * hv.x + hv.y * hv.y + hv.z * hv.z + hv.w * hv.w;
  ss = warp_sum(ss);
  if ((t & 31) == 0) part[t >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int j = 0; j < (int)(blockDim.x >> 5); ++j) tot += part[j];
  const float r = rsqrtf(tot / (float)H + eps);
  const __half2 a2 = __floats2half2_rn(hv.x * r * wv.x, hv.y * r * wv.y), b2 = __floats2half2_rn(hv.z * r * wv.z, hv.w * r * wv.w);
  const uint32_t A = *reinterpret_cast<const uint32_t*>(&a2), B = *reinterpret_cast<const uint32_t*>(&b2);
  const bool upper = t & 1;                                // values 4 .. 7 of the chunk
  const uint32_t R = __shfl_xor_sync(0xffffffffu, upper ? A : B, 1);
  uint2 o;                                                 // lower: (0,4,1,5) from A = (0,1), R = (4,5); upper: (2,6,3,7) from R = (2,3), B = (6,7)
  o.x = upper ? __byte_perm(R, B, 0x5410) : __byte_perm(A, R, 0x5410);
  o.y = upper ? __byte_perm(R, B, 0x7632) : __byte_perm(A, R, 0x7632);
  const int wi = i0 >> 3, KB = H >> 5, tk = row & 127;
  uint8_t* rec = xt + ((size_t)(row >> 7) * KB + (wi >> 2)) * 8192;
  *reinterpret_cast<uint2*>(rec + (tk >> 3) * 512 + (wi & 3) * 128 + (tk & 7) * 16 + (upper ? 8 : 0)) = o;
}

__global__ void __launch_bounds__(256) quant_q8_1_kernel(const __half* x, int8_t* xq, __half* xd, __half* xsum, size_t nblk) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t gid = (size_t)blockIdx.x * 256 + threadIdx.x;
  const size_t blk = gid >> 3;
  const int l = (int)(gid & 7);
  const bool live = blk < nblk;                      // whole 8-lane groups are live or dead together
  const size_t at = (live ? blk : 0) * 32 + l * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(x + at);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
  const float v[4] = {a.x, a.y, b.x, b.y};
  quant_block4(v, xq + at, xd + (live ? blk : 0), xsum ? xsum + (live ? blk : 0) : nullptr, l, live);
}

// One CTA of H/4 threads (<= 1024) per row: RMSNorm in registers, round to fp16, quantise.
__global__ void __launch_bounds__(1024) rmsnorm_q8_1_kernel(const float* h, const float* __restrict__ w, int8_t* xq,
                                                            __half* xd, __half* xsum, __half* x16, int H, float eps) {
  __shared__ float part[32];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, t = threadIdx.x, i0 = 4 * t;
  const float4 hv = *reinterpret_cast<const float4*>(h + (size_t)row * H + i0);
  const float4 wv = *reinterpret_cast<const float4*>(w + i0);
  float ss = hv.x * hv.x + hv.y * hv.y + hv.z * hv.z + hv.w * hv.w;
  ss = warp_sum(ss);
  if ((t & 31) == 0) part[t >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int j = 0; j < (int)(blockDim.x >> 5); ++j) tot += part[j];
  const float r = rsqrtf(tot / (float)H + eps);
  const __half2 p0 = __floats2half2_rn(hv.x * r * wv.x, hv.y * r * wv.y);
  const __half2 p1 = __floats2half2_rn(hv.z * r * wv.z, hv.w * r * wv.w);
  if (x16) {
    uint2 st;
    st.x = *reinterpret_cast<const uint32_t*>(&p0);
    st.y = *reinterpret_cast<const uint32_t*>(&p1);
    *reinterpret_cast<uint2*>(x16 + (size_t)row * H + i0) = st;
  }
  const float2 a = __half22float2(p0), b = __half22float2(p1);
  const float v[4] = {a.x, a.y, b.x, b.y};
  const size_t blk = ((size_t)row * H + i0) >> 5;
  quant_block4(v, xq + (size_t)row * H + i0, xd + blk, xsum ? xsum + blk : nullptr, t & 7, true);
}

}  // namespace

int quant_q8_1(const void* x, void* xq, void* xd, void* xsum, int rows, int K, cudaStream_t st) {
  if (rows <= 0 || K <= 0 || (K % 32)) return fail(Q4B_E_SHAPE, "quant_q8_1: rows > 0 and K a positive multiple of 32 required");
  if (!x || !xq || !xd || (reinterpret_cast<uintptr_t>(x) & 7u) || (reinterpret_cast<uintptr_t>(xq) & 3u))
    return fail(Q4B_E_ALIGN, "quant_q8_1: null or misaligned pointer");
  const size_t nblk = (size_t)rows * (K / 32);
  const size_t threads = nblk * 8;
  return check_launch(launch_pdl(quant_q8_1_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, st, (const __half*)x,
                                 (int8_t*)xq, (__half*)xd, (__half*)xsum, nblk), "quant_q8_1");
}

int quant_q8_1_tiled(const void* x, void* xt, int rows, int K, cudaStream_t st) {
  if (rows <= 0 || K <= 0 || (K % 32)) return fail(Q4B_E_SHAPE, "quant_q8_1_tiled: rows > 0 and K a positive multiple of 32 required");
  if (!x || !xt || (reinterpret_cast<uintptr_t>(x) & 7u) || !aligned16(xt)) return fail(Q4B_E_ALIGN, "quant_q8_1_tiled: null or misaligned pointer");
  const size_t threads = (size_t)rows * (K / 32) * 8;
  return check_launch(launch_pdl(quant_q8_1_tiled_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, st,
                                 (const __half*)x, (uint8_t*)xt, rows, K / 32), "quant_q8_1_tiled");
}

int rmsnorm_q8_1_tiled(const float* h, const float* w, void* xt, int rows, int H, float eps, cudaStream_t st, float* h_add, int n_add) {
  if (rows <= 0 || H <= 0 || (H % 128) || H > 4096) return fail(Q4B_E_SHAPE, "rmsnorm_q8_1_tiled: H must be a multiple of 128, at most 4096");
  if (!h || !w || !xt || !aligned16(h) || !aligned16(w) || !aligned16(xt) || !aligned16(h_add))
    return fail(Q4B_E_ALIGN, "rmsnorm_q8_1_tiled: null or misaligned pointer");
  return check_launch(launch_pdl(rmsnorm_q8_1_tiled_kernel, dim3(rows), dim3(H / 4), 0, st, h, w, (uint8_t*)xt, H, eps, h_add, n_add),
                      "rmsnorm_q8_1_tiled");
}

int rmsnorm_f16_tiled(const float* h, const float* w, void* xt, int rows, int H, float eps, cudaStream_t st, float* h_add, int n_add) {
  if (rows <= 0 || H <= 0 || (H % 128) || H > 4096) return fail(Q4B_E_SHAPE, "rmsnorm_f16_tiled: H must be a multiple of 128, at most 4096");
  if (!h || !w || !xt || !aligned16(h) || !aligned16(w) || !aligned16(xt) || !aligned16(h_add))
    return fail(Q4B_E_ALIGN, "rmsnorm_f16_tiled: null or misaligned pointer");
  return check_launch(launch_pdl(rmsnorm_f16_tiled_kernel, dim3(rows), dim3(H / 4), 0, st, h, w, (uint8_t*)xt, H, eps, h_add, n_add),
                      "rmsnorm_f16_tiled");
}

namespace {
__global__ void __launch_bounds__(256) add_rows_kernel(float* h, const float* h_add, size_t n4, int n_add) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n4) return;
  float4 a = reinterpret_cast<float4*>(h)[i];
  for (int j = 0; j < n_add; ++j) {
    const float4 b = reinterpret_cast<const float4*>(h_add)[(size_t)j * n4 + i];
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
  }
  reinterpret_cast<float4*>(h)[i] = a;
}
}  // namespace

// h[0 .. n) += h_add[0][0 .. n) + h_add[1][0 .. n) + .., n a multiple of 4 (completes rows whose further K parts were stored apart)
int add_rows(float* h, const float* h_add, size_t n, int n_add, cudaStream_t st) {
  if (!h || !h_add || !aligned16(h) || !aligned16(h_add) || (n % 4) || n == 0 || n_add < 1) return fail(Q4B_E_ALIGN, "add_rows: null, misaligned or ragged");
  return check_launch(launch_pdl(add_rows_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, st, h, h_add, n / 4, n_add), "add_rows");
}

int rmsnorm_q8_1(const float* h, const float* w, void* xq, void* xd, void* xsum, void* x16, int rows, int H, float eps,
                 cudaStream_t st) {
  if (rows <= 0 || H <= 0 || (H % 128) || H > 4096) return fail(Q4B_E_SHAPE, "rmsnorm_q8_1: H must be a multiple of 128, at most 4096");
  if (!h || !w || !xq || !xd || !aligned16(h) || !aligned16(w) || (reinterpret_cast<uintptr_t>(xq) & 3u))
    return fail(Q4B_E_ALIGN, "rmsnorm_q8_1: null or misaligned pointer");
  return check_launch(launch_pdl(rmsnorm_q8_1_kernel, dim3(rows), dim3(H / 4), 0, st, h, w, (int8_t*)xq, (__half*)xd,
                                 (__half*)xsum, (__half*)x16, H, eps), "rmsnorm_q8_1");
}

}  // namespace q4b
