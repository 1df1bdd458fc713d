// extern "C" surface of libq4b200: argument checks live in the per-op launchers, this file only forwards and keeps
// the per-thread error text.
#include <stdio.h>
#include <string.h>

#include "q4b_internal.h"

namespace q4b {

static thread_local char g_err[256] = "";
static int g_sm_count = 0;

void set_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_err, sizeof(g_err), "%s: CUDA error %d (%s)", where, (int)e, cudaGetErrorString(e));
}

int fail(int code, const char* msg) {
  snprintf(g_err, sizeof(g_err), "%s", msg);
  return code;
}

// ---- chain timeline state (host side; profiling runs only, not thread-safe)
static unsigned long long* g_chain_buf = nullptr;
static size_t g_chain_entries = 0, g_chain_next = 0;
static constexpr int MAX_CHAIN_RECORDS = 4096;
static long long g_chain_log[MAX_CHAIN_RECORDS][3];
static int g_chain_records = 0;

unsigned long long* trace_slot(int kernel_id, int ctas) {
  if (!g_chain_buf || ctas <= 0 || g_chain_records >= MAX_CHAIN_RECORDS) return nullptr;
  const size_t need = (size_t)ctas * 16;
  if (g_chain_next + need > g_chain_entries) return nullptr;
  unsigned long long* p = g_chain_buf + g_chain_next;
  g_chain_log[g_chain_records][0] = kernel_id;
  g_chain_log[g_chain_records][1] = ctas;
  g_chain_log[g_chain_records][2] = (long long)g_chain_next;
  ++g_chain_records;
  g_chain_next += need;
  return p;
}

// SM count of the CURRENT device (cached per device ordinal; grids are sized from it)
int sm_count() {
  static int per_dev[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return g_sm_count > 0 ? g_sm_count : 148;
  if (per_dev[dev] <= 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) per_dev[dev] = n;
    else return g_sm_count > 0 ? g_sm_count : 148;
  }
  return per_dev[dev];
}

// per-op launchers (defined next to their kernels)
int gemv_q4_0(const void*, const void*, const void*, void*, const void*, int, int, int, int, cudaStream_t);
int embed(const void*, const int64_t*, float*, int, int, int, cudaStream_t);
int rmsnorm(const float*, const float*, void*, int, int, float, cudaStream_t);
size_t argmax_workspace(int, int);
int argmax_advance(const float*, int, int, int64_t*, int64_t*, void*, size_t, cudaStream_t);
int argmax_advance_static(const float*, int, int, int64_t*, int64_t*, cudaStream_t);
size_t attn_decode_workspace(int, int, int, int);
int attn_decode(const void*, const float*, const float*, const int64_t*, void*, void*, void*, int, int, int, int, int, float,
                void*, size_t, cudaStream_t, int pre = 0);
int gemv_mma(const void*, const void*, const void*, void*, const void*, int, int, int, int, uint32_t*, cudaStream_t,
             const float* norm_w = nullptr, float eps = 0.f, const float* cosT = nullptr, const float* sinT = nullptr,
             const int64_t* pos = nullptr, void* kc = nullptr, void* vc = nullptr, int NH = 0, int NKV = 0, int HD = 0,
             int max_len = 0, int withhold_chunk = -1, const GemvLookahead* look = nullptr);
int gemv_mma_ksplit(int, int);
void mmq_prefill_trace(long long*);
void mmq_prefill_debug_no_copy(bool);
void attn_batched_kernel(int);
int tp_allreduce(const void* const*, void* const*, int, int, uint32_t, const uint32_t*, float*, int, int, const float*, float, void*,
                 void*, uint32_t*, uint32_t, cudaStream_t);
int tp_epoch_advance(uint32_t*, uint32_t, cudaStream_t);
int gemv_f16mma(const void*, const void*, const void*, void*, const void*, int, int, int, int, int, uint32_t*, cudaStream_t);
int gemv_q8mma(const void*, const void*, const void*, const void*, void*, const void*, int, int, int, int, int, uint32_t*, cudaStream_t);
double peak_i8_launch(int, uint32_t*, cudaStream_t);
int head_q6_k_argmax(const void*, const void*, const void*, const void*, const void*, float*, int, int, int64_t*, int64_t*, void*, size_t,
                     cudaStream_t);
void gemv_mma_trace(unsigned long long*);
size_t head_workspace(int);
int head_f16_argmax(const void*, const void*, float*, int, int, int64_t*, int64_t*, void*, size_t, cudaStream_t);
int head_f16_batched(const void*, const void*, float*, int, int, int, cudaStream_t);
int blockdot(const void*, const void*, int32_t*, int, int, int, int, uint32_t*, cudaStream_t);
int mmq_stream(const void*, const void*, const void*, const void*, void*, const void*, int, int, int, int, int, int, uint32_t*,
               cudaStream_t, const float* norm_w = nullptr, float eps = 0.f);
void mmq_stream_trace(unsigned long long*);
void attn_decode_mma_trace(unsigned long long*);
int attn_decode_q8(const void*, const float*, const float*, const int64_t*, void*, void*, void*, void*, void*, int, int, int, int, int,
                   float, cudaStream_t);
size_t decode_persistent_workspace(const q4b_decode_desc*);
int decode_persistent_prepare(const q4b_decode_desc*, void*, size_t);
int decode_persistent_layers(const q4b_decode_desc*, void*, size_t, cudaStream_t);
void decode_persistent_trace(unsigned long long*, int);
int attn_prefill(const void*, const float*, const float*, void*, void*, void*, int, int, int, int, int, int, float, cudaStream_t,
                 int pre = 0, void* xt = nullptr);
size_t q8_tiled_bytes(int, int);
int mmq_prefill(const void*, const void*, const void*, void*, const void*, int, int, int, int, int, uint32_t*, cudaStream_t,
                const float* cosT = nullptr, const float* sinT = nullptr, void* kc = nullptr, void* vc = nullptr, int NH = 0,
                int NKV = 0, int max_len = 0, int pos0 = 0, float* Y2 = nullptr, int parts = 1, int f16 = 0);
size_t f16_tiled_bytes(int, int);
int rmsnorm_f16_tiled(const float*, const float*, void*, int, int, float, cudaStream_t, float* h_add = nullptr, int n_add = 0);
int f16_tiled(const void*, void*, int, int, cudaStream_t);
int add_rows(float*, const float*, size_t, int, cudaStream_t);
int quant_q8_1_tiled(const void*, void*, int, int, cudaStream_t);
int rmsnorm_q8_1_tiled(const float*, const float*, void*, int, int, float, cudaStream_t, float* h_add = nullptr, int n_add = 1);
int pack_q4_0(const void*, const void*, void*, void*, int, int, cudaStream_t);
int quant_q8_1(const void*, void*, void*, void*, int, int, cudaStream_t);
int rmsnorm_q8_1(const float*, const float*, void*, void*, void*, void*, int, int, float, cudaStream_t);

}  // namespace q4b

using namespace q4b;

static inline cudaStream_t S(q4b_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

extern "C" {

int q4b_version(void) { return 1000; }

const char* q4b_last_error(void) { return g_err; }

int q4b_init(int device) {
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) {
    set_cuda_error(e, "q4b_init");
    return Q4B_E_CUDA;
  }
  int n = 0;
  e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device);
  if (e != cudaSuccess) {
    set_cuda_error(e, "q4b_init");
    return Q4B_E_CUDA;
  }
  g_sm_count = n;
  g_err[0] = 0;
  return Q4B_OK;
}

int q4b_gemv_q4_0(const void* W, const void* Sc, const void* X, void* Y, const void* AUX, int N, int K, int epilogue,
                  int x_dtype, q4b_stream_t stream) {
  return gemv_q4_0(W, Sc, X, Y, AUX, N, K, epilogue, x_dtype, S(stream));
}

int q4b_rmsnorm(const float* h, const float* w, void* out, int rows, int H, float eps, q4b_stream_t stream) {
  return rmsnorm(h, w, out, rows, H, eps, S(stream));
}

int q4b_embed(const void* E, const int64_t* tok, float* h, int rows, int H, int V, q4b_stream_t stream) {
  return embed(E, tok, h, rows, H, V, S(stream));
}

size_t q4b_attn_decode_workspace(int B, int NH, int HD, int max_len) { return attn_decode_workspace(B, NH, HD, max_len); }

int q4b_attn_decode_q8_1(const void* qkv, const float* cosT, const float* sinT, const int64_t* pos, void* kc, void* vc,
                         void* out, void* xq, void* xd, int B, int NH, int NKV, int HD, int max_len, float scale,
                         q4b_stream_t stream) {
  return attn_decode_q8(qkv, cosT, sinT, pos, kc, vc, out, xq, xd, B, NH, NKV, HD, max_len, scale, S(stream));
}

int q4b_attn_decode(const void* qkv, const float* cosT, const float* sinT, const int64_t* pos, void* kc, void* vc,
                    void* out, int B, int NH, int NKV, int HD, int max_len, float scale, void* workspace,
                    size_t workspace_bytes, q4b_stream_t stream) {
  return attn_decode(qkv, cosT, sinT, pos, kc, vc, out, B, NH, NKV, HD, max_len, scale, workspace, workspace_bytes, S(stream));
}

size_t q4b_head_workspace(int V) { return head_workspace(V); }

int q4b_head_f16_argmax(const void* E, const void* x, float* logits, int V, int H, int64_t* tok, int64_t* pos,
                        void* workspace, size_t workspace_bytes, q4b_stream_t stream) {
  return head_f16_argmax(E, x, logits, V, H, tok, pos, workspace, workspace_bytes, S(stream));
}

int q4b_head_q6_k_argmax(const void* L, const void* Hb, const void* SC, const void* D, const void* x, float* logits, int V, int K,
                         int64_t* tok, int64_t* pos, void* workspace, size_t workspace_bytes, q4b_stream_t stream) {
  return head_q6_k_argmax(L, Hb, SC, D, x, logits, V, K, tok, pos, workspace, workspace_bytes, S(stream));
}

int q4b_argmax_advance_static(const float* logits, int rows, int V, int64_t* tok, int64_t* pos, q4b_stream_t stream) {
  return argmax_advance_static(logits, rows, V, tok, pos, S(stream));
}

int q4b_head_f16_batched(const void* E, const void* x, float* logits, int V, int H, int B, q4b_stream_t stream) {
  return head_f16_batched(E, x, logits, V, H, B, S(stream));
}

size_t q4b_argmax_workspace(int rows, int V) { return argmax_workspace(rows, V); }

int q4b_argmax_advance(const float* logits, int rows, int V, int64_t* tok, int64_t* pos, void* workspace,
                       size_t workspace_bytes, q4b_stream_t stream) {
  return argmax_advance(logits, rows, V, tok, pos, workspace, workspace_bytes, S(stream));
}

int q4b_blockdot_q4_0_q8_1(const void* W, const void* xq, int32_t* out, int M, int K, int P, int mode, uint32_t* status,
                           q4b_stream_t stream) {
  return blockdot(W, xq, out, M, K, P, mode, status, S(stream));
}

int q4b_gemv_q4_0_tc(const void* W, const void* Sc, const void* X, void* Y, const void* AUX, int N, int K, int epilogue,
                     int x_dtype, uint32_t* status, q4b_stream_t stream) {
  if (x_dtype != Q4B_X_F16 && x_dtype != Q4B_X_F32) return fail(Q4B_E_ARG, "gemv_q4_0_tc: unknown x_dtype");
  const int ldy = epilogue == Q4B_EPI_SWIGLU ? N / 2 : N;
  return mmq_stream(W, Sc, X, nullptr, Y, AUX, N, K, 1, x_dtype == Q4B_X_F16 ? 0 : 1, epilogue, ldy, status, S(stream));
}

int q4b_gemv_q4_0_mma(const void* W, const void* Sc, const void* X, void* Y, const void* AUX, int N, int K, int epilogue,
                      int x_dtype, uint32_t* status, q4b_stream_t stream) {
  if (x_dtype != Q4B_X_F16 && x_dtype != Q4B_X_F32) return fail(Q4B_E_ARG, "gemv_q4_0_mma: unknown x_dtype");
  if (epilogue == Q4B_EPI_BIASF_ROPE_KV) return fail(Q4B_E_ARG, "gemv_q4_0_mma: use q4b_rmsnorm_qkv_rope_kv for the fused RoPE epilogue");
  return gemv_mma(W, Sc, X, Y, AUX, N, K, x_dtype == Q4B_X_F16 ? 0 : 1, epilogue, status, S(stream));
}

int q4b_rmsnorm_gemv_q4_0_mma(const void* W, const void* Sc, const float* h, const float* norm_w, float eps, void* Y,
                              const void* AUX, int N, int K, int epilogue, uint32_t* status, q4b_stream_t stream) {
  if (epilogue == Q4B_EPI_BIASF_ROPE_KV) return fail(Q4B_E_ARG, "rmsnorm_gemv_q4_0_mma: use q4b_rmsnorm_qkv_rope_kv for the fused RoPE epilogue");
  return gemv_mma(W, Sc, h, Y, AUX, N, K, 3, epilogue, status, S(stream), norm_w, eps);
}

int q4b_rmsnorm_qkv_rope_kv(const void* W, const void* Sc, const float* h, const float* norm_w, float eps, void* qkv,
                            const float* bias, int K, const float* cosT, const float* sinT, const int64_t* pos, void* kc,
                            void* vc, int NH, int NKV, int HD, int max_len, uint32_t* status, q4b_stream_t stream) {
  return gemv_mma(W, Sc, h, qkv, bias, (NH + 2 * NKV) * HD, K, 3, Q4B_EPI_BIASF_ROPE_KV, status, S(stream), norm_w, eps, cosT,
                  sinT, pos, kc, vc, NH, NKV, HD, max_len);
}

int q4b_gemv_q4_0_f16mma(const void* W, const void* Sc, const void* X, void* Y, const void* AUX, int N, int K, int B,
                         int epilogue, int ldy, uint32_t* status, q4b_stream_t stream) {
  return gemv_f16mma(W, Sc, X, Y, AUX, N, K, B, epilogue, ldy, status, S(stream));
}

int q4b_tp_allreduce_resid_rmsnorm_q8(const void* const* parts, void* const* flags, int rank, int world, uint32_t epoch,
                                      const uint32_t* epoch_base, float* h, int rows, int H, const float* norm_w, float eps,
                                      void* xq, void* xd, uint32_t* status, q4b_stream_t stream) {
  return tp_allreduce(parts, flags, rank, world, epoch, epoch_base, h, rows, H, norm_w, eps, xq, xd, status, 0u, S(stream));
}

int q4b_tp_epoch_advance(uint32_t* epoch_base, uint32_t by, q4b_stream_t stream) { return tp_epoch_advance(epoch_base, by, S(stream)); }

int q4b_debug_tp_allreduce_expired_wait(const void* const* parts, void* const* flags, int rank, int world, uint32_t epoch,
                                        float* h, int rows, int H, uint32_t* status, q4b_stream_t stream) {
  return tp_allreduce(parts, flags, rank, world, epoch, nullptr, h, rows, H, nullptr, 0.f, nullptr, nullptr, status, 4096u, S(stream));
}

int q4b_attn_batched_kernel(int which) {
  if (which != 0 && which != 1) return fail(Q4B_E_ARG, "attn_batched_kernel: 0 (cached form where it fits) or 1 (streaming kernel)");
  attn_batched_kernel(which);
  return Q4B_OK;
}

int q4b_mmq_q4_0_q8_1_mma(const void* W, const void* Sc, const void* xq, const void* xd, void* Y, const void* AUX, int N, int K,
                          int P, int epilogue, int ldy, uint32_t* status, q4b_stream_t stream) {
  return gemv_q8mma(W, Sc, xq, xd, Y, AUX, N, K, P, epilogue, ldy, status, S(stream));
}

int q4b_quant_mmq_q4_0_q8_1_mma(const void* W, const void* Sc, const void* x16, void* Y, const void* AUX, int N, int K, int P,
                                int epilogue, int ldy, uint32_t* status, q4b_stream_t stream) {
  return gemv_q8mma(W, Sc, nullptr, x16, Y, AUX, N, K, P, epilogue, ldy, status, S(stream));
}

size_t q4b_f16_tiled_bytes(int rows, int K) { return (rows > 0 && K > 0) ? f16_tiled_bytes(rows, K) : 0; }

int q4b_f16_tiled(const void* x, void* xt, int rows, int K, q4b_stream_t stream) { return f16_tiled(x, xt, rows, K, S(stream)); }

int q4b_mm_prefill_q4_0_f16(const void* Wt, const void* St, const void* xt, void* Y, const void* AUX, int N, int K, int P,
                            int epilogue, int ldy, uint32_t* status, q4b_stream_t stream) {
  return mmq_prefill(Wt, St, xt, Y, AUX, N, K, P, epilogue, ldy, status, S(stream), nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0,
                     nullptr, 1, 1);
}

int q4b_mm_prefill_f16_resid_ksplit(const void* Wt, const void* St, const void* xt, float* Y, float* Y2, int parts, int N, int K, int P,
                                    int ldy, uint32_t* status, q4b_stream_t stream) {
  if (parts < 2 || !Y2) return fail(Q4B_E_ARG, "mm_prefill_f16_resid_ksplit: parts >= 2 and Y2 required");
  return mmq_prefill(Wt, St, xt, Y, nullptr, N, K, P, Q4B_EPI_RESID, ldy, status, S(stream), nullptr, nullptr, nullptr, nullptr, 0, 0,
                     0, 0, Y2, parts, 1);
}

int q4b_rmsnorm_f16_tiled_add(float* h, const float* h_add, int n_add, const float* w, void* xt, int rows, int H, float eps,
                              q4b_stream_t stream) {
  if (n_add < 0 || n_add > 3 || (n_add > 0 && !h_add)) return fail(Q4B_E_ARG, "rmsnorm_f16_tiled_add: 0 .. 3 addends");
  return rmsnorm_f16_tiled(h, w, xt, rows, H, eps, S(stream), n_add ? const_cast<float*>(h_add) : nullptr, n_add);
}

int q4b_debug_mmq_prefill_expired_wait(const void* Wt, const void* St, const void* xt, void* Y, int N, int K, int P, uint32_t* status,
                                       q4b_stream_t stream) {
  mmq_prefill_debug_no_copy(true);
  const int rc = mmq_prefill(Wt, St, xt, Y, nullptr, N, K, P, Q4B_EPI_LOGITS, N, status, S(stream));
  mmq_prefill_debug_no_copy(false);
  return rc;
}

int q4b_mmq_prefill_trace(int64_t* device_buffer, size_t entries) {
  if (device_buffer && entries < 11 * 64) return fail(Q4B_E_WORKSPACE, "mmq_prefill_trace: need 11 x 64 entries");
  mmq_prefill_trace(reinterpret_cast<long long*>(device_buffer));
  return Q4B_OK;
}

int q4b_debug_gemv_mma_expired_wait(const void* W, const void* Sc, const void* X, void* Y, int N, int K, uint32_t* status,
                                    q4b_stream_t stream) {
  return gemv_mma(W, Sc, X, Y, nullptr, N, K, 0, Q4B_EPI_LOGITS, status, S(stream), nullptr, 0.f, nullptr, nullptr, nullptr,
                  nullptr, nullptr, 0, 0, 0, 0, 0);
}

int q4b_attn_decode_cached(const void* qkv, const int64_t* pos, const void* kc, const void* vc, void* out, int NH, int NKV,
                           int HD, int max_len, float scale, q4b_stream_t stream) {
  return attn_decode(qkv, nullptr, nullptr, pos, const_cast<void*>(kc), const_cast<void*>(vc), out, 1, NH, NKV, HD, max_len,
                     scale, nullptr, 0, S(stream), 1);
}

int q4b_pack_q4_0(const void* W, const void* Sc, void* Wt, void* St, int N, int K, q4b_stream_t stream) {
  return pack_q4_0(W, Sc, Wt, St, N, K, S(stream));
}

size_t q4b_q8_tiled_bytes(int rows, int K) { return (rows > 0 && K > 0) ? q8_tiled_bytes(rows, K) : 0; }

int q4b_quant_q8_1_tiled(const void* x, void* xt, int rows, int K, q4b_stream_t stream) {
  return quant_q8_1_tiled(x, xt, rows, K, S(stream));
}

int q4b_rmsnorm_q8_1_tiled(const float* h, const float* w, void* xt, int rows, int H, float eps, q4b_stream_t stream) {
  return rmsnorm_q8_1_tiled(h, w, xt, rows, H, eps, S(stream));
}

int q4b_mmq_prefill_q4_0_q8_1(const void* Wt, const void* St, const void* xt, void* Y, const void* AUX, int N, int K, int P,
                              int epilogue, int ldy, uint32_t* status, q4b_stream_t stream) {
  return mmq_prefill(Wt, St, xt, Y, AUX, N, K, P, epilogue, ldy, status, S(stream));
}

int q4b_mmq_prefill_qkv_rope_kv(const void* Wt, const void* St, const void* xt, void* qkv, const float* bias, int K, int P,
                                const float* cosT, const float* sinT, int pos0, void* kc, void* vc, int NH, int NKV, int HD,
                                int max_len, uint32_t* status, q4b_stream_t stream) {
  if (HD != 128) return fail(Q4B_E_SHAPE, "mmq_prefill_qkv_rope_kv: head_dim must be 128 (one row tile per head)");
  const int N = (NH + 2 * NKV) * HD;
  return mmq_prefill(Wt, St, xt, qkv, bias, N, K, P, Q4B_EPI_BIASF_ROPE_KV, N, status, S(stream), cosT, sinT, kc, vc, NH, NKV,
                     max_len, pos0);
}

int q4b_attn_prefill_cached(const void* qkv, const void* kc, const void* vc, void* out, void* xt, int P, int NH, int NKV, int HD,
                            int max_len, int pos0, float scale, q4b_stream_t stream) {
  return attn_prefill(qkv, nullptr, nullptr, const_cast<void*>(kc), const_cast<void*>(vc), out, P, NH, NKV, HD, max_len, pos0,
                      scale, S(stream), 1, xt);
}

int q4b_mmq_prefill_resid_ksplit(const void* Wt, const void* St, const void* xt, float* Y, float* Y2, int parts, int N, int K, int P,
                                 int ldy, uint32_t* status, q4b_stream_t stream) {
  if (!Y2) return fail(Q4B_E_ALIGN, "mmq_prefill_resid_ksplit: Y2 missing");
  return mmq_prefill(Wt, St, xt, Y, nullptr, N, K, P, Q4B_EPI_RESID, ldy, status, S(stream), nullptr, nullptr, nullptr, nullptr, 0, 0,
                     0, 0, Y2, parts);
}

int q4b_rmsnorm_q8_1_tiled_add(float* h, const float* h_add, int n_add, const float* w, void* xt, int rows, int H, float eps,
                               q4b_stream_t stream) {
  return rmsnorm_q8_1_tiled(h, w, xt, rows, H, eps, S(stream), const_cast<float*>(h_add), n_add);
}

int q4b_add_rows(float* h, const float* h_add, int n_add, size_t n, q4b_stream_t stream) { return add_rows(h, h_add, n, n_add, S(stream)); }

int q4b_attn_prefill(const void* qkv, const float* cosT, const float* sinT, void* kc, void* vc, void* out, int P, int NH,
                     int NKV, int HD, int max_len, int pos0, float scale, q4b_stream_t stream) {
  return attn_prefill(qkv, cosT, sinT, kc, vc, out, P, NH, NKV, HD, max_len, pos0, scale, S(stream));
}

int q4b_trace_buffer(uint64_t* device_buffer, size_t entries) {
  if (device_buffer && entries < (size_t)4096 * 16) return fail(Q4B_E_WORKSPACE, "trace_buffer: need 4096 x 16 entries");
  mmq_stream_trace(reinterpret_cast<unsigned long long*>(device_buffer));
  gemv_mma_trace(reinterpret_cast<unsigned long long*>(device_buffer));
  attn_decode_mma_trace(reinterpret_cast<unsigned long long*>(device_buffer));
  return Q4B_OK;
}

double q4b_peak_i8_launch(int iters, uint32_t* status, q4b_stream_t stream) { return peak_i8_launch(iters, status, S(stream)); }

int q4b_trace_chain(uint64_t* device_buffer, size_t entries) {
  g_chain_buf = reinterpret_cast<unsigned long long*>(device_buffer);
  g_chain_entries = device_buffer ? entries : 0;
  g_chain_next = 0;
  if (device_buffer) g_chain_records = 0;
  return Q4B_OK;
}

int q4b_trace_chain_log(int64_t* records, int max_records) {
  const int n = g_chain_records < max_records ? g_chain_records : max_records;
  for (int i = 0; i < n && records; ++i)
    for (int j = 0; j < 3; ++j) records[3 * i + j] = g_chain_log[i][j];
  return g_chain_records;
}

int q4b_rmsnorm_gemv_q4_0_tc(const void* W, const void* Sc, const float* h, const float* norm_w, float eps, void* Y,
                             const void* AUX, int N, int K, int epilogue, uint32_t* status, q4b_stream_t stream) {
  const int ldy = epilogue == Q4B_EPI_SWIGLU ? N / 2 : N;
  return mmq_stream(W, Sc, h, nullptr, Y, AUX, N, K, 1, 3, epilogue, ldy, status, S(stream), norm_w, eps);
}

int q4b_mmq_q4_0_q8_1(const void* W, const void* Sc, const void* xq, const void* xd, void* Y, const void* AUX, int N, int K,
                      int P, int epilogue, int ldy, uint32_t* status, q4b_stream_t stream) {
  if (P < 1 || P > 32) return fail(Q4B_E_SHAPE, "mmq_q4_0_q8_1: 1..32 activation rows supported by the streaming kernel");
  return mmq_stream(W, Sc, xq, xd, Y, AUX, N, K, P, 2, epilogue, ldy, status, S(stream));
}

int q4b_quant_q8_1(const void* x, void* xq, void* xd, void* xsum, int rows, int K, q4b_stream_t stream) {
  return quant_q8_1(x, xq, xd, xsum, rows, K, S(stream));
}

int q4b_rmsnorm_q8_1(const float* h, const float* w, void* xq, void* xd, void* xsum, void* x16, int rows, int H, float eps,
                     q4b_stream_t stream) {
  return rmsnorm_q8_1(h, w, xq, xd, xsum, x16, rows, H, eps, S(stream));
}

int q4b_decode_step(const q4b_decode_desc* d, q4b_stream_t stream) {
  if (!d || !d->layer) return fail(Q4B_E_ARG, "decode_step: null descriptor");
  cudaStream_t st = S(stream);
  const int H = d->hidden, QR = d->n_heads * d->head_dim;
  const bool tcp = (d->flags & Q4B_STEP_TENSOR_CORE) && d->status;
  const bool mmap = (d->flags & Q4B_STEP_MMA_GEMV) && d->status;
  auto mma_ok = [&](const q4b_linear& L) { return mmap && L.Wt && (L.K % 32) == 0 && gemv_mma_ksplit(L.N, L.K) > 0; };
  // the QKV projection can rotate q / k and append k, v itself when one 128-row tile holds whole heads
  const bool fused_kv = mmap && d->head_dim > 0 && (128 % d->head_dim) == 0 && d->max_len <= 4096 &&
                        d->n_heads % d->n_kv_heads == 0 && d->n_heads / d->n_kv_heads <= 8 && (d->head_dim == 64 || d->head_dim == 128);
  // one linear: the mma.sync streaming GEMV or the tcgen05 kernel when its shape allows, the CUDA-core GEMV otherwise
  // L2 look-ahead: a launch asks for the packed weights of launches two to three places down the chain, so that their
  // own bulk copies (issued one launch ahead, when their CTAs move in) find the lines in L2 instead of waiting on HBM
  // Measured on the 1.5B step: with the look-ahead ON the step is 1.2 % SLOWER (736.6 against 727.8 us): the prefetch
  // bursts compete in L2 with the latency-critical activation loads of the launch that is running.  It stays available
  // (Q4B_STEP_LOOKAHEAD) for shapes whose slabs do not fit beside their predecessors, and is off by default.
  const bool look_on = (d->flags & Q4B_STEP_LOOKAHEAD) != 0;
  auto look_at = [&](GemvLookahead& g, int slot, const q4b_linear* L) {
    if (!L || !L->Wt || !mma_ok(*L) || !look_on) return;
    const size_t tiles = (size_t)(L->N + 127) / 128, kb = (size_t)L->K / 32;
    g.ptr[2 * slot] = L->Wt;
    g.bytes[2 * slot] = tiles * kb * 2048;
    g.ptr[2 * slot + 1] = L->St;
    g.bytes[2 * slot + 1] = tiles * kb * 256;
  };
  auto lin = [&](const q4b_linear& L, const void* X, void* Y, const void* AUX, int epi, const q4b_linear* ahead0 = nullptr,
                 const q4b_linear* ahead1 = nullptr) -> int {
    if (mma_ok(L)) {
      GemvLookahead g{};
      look_at(g, 0, ahead0);
      look_at(g, 1, ahead1);
      return gemv_mma(L.Wt, L.St, X, Y, AUX, L.N, L.K, 0, epi, d->status, st, nullptr, 0.f, nullptr, nullptr, nullptr, nullptr, nullptr,
                      0, 0, 0, 0, -1, &g);
    }
    if (tcp && L.Wt && (L.K % 256) == 0)
      return mmq_stream(L.Wt, L.St, X, nullptr, Y, AUX, L.N, L.K, 1, 0, epi, epi == Q4B_EPI_SWIGLU ? L.N / 2 : L.N, d->status, st);
    return gemv_q4_0(L.W, L.S, X, Y, AUX, L.N, L.K, epi, Q4B_X_F16, st);
  };
  // RMSNorm followed by a linear: one launch on the tensor-core path (the norm is computed while staging the operand)
  auto norm_lin = [&](const float* nw, const q4b_linear& L, void* Y, const void* AUX, int epi, const q4b_linear* ahead0 = nullptr,
                      const q4b_linear* ahead1 = nullptr) -> int {
    if (mma_ok(L)) {
      GemvLookahead g{};
      look_at(g, 0, ahead0);
      look_at(g, 1, ahead1);
      return gemv_mma(L.Wt, L.St, d->h, Y, AUX, L.N, L.K, 3, epi, d->status, st, nw, d->eps, nullptr, nullptr, nullptr, nullptr, nullptr,
                      0, 0, 0, 0, -1, &g);
    }
    if (tcp && L.Wt && (L.K % 256) == 0)
      return mmq_stream(L.Wt, L.St, d->h, nullptr, Y, AUX, L.N, L.K, 1, 3, epi, epi == Q4B_EPI_SWIGLU ? L.N / 2 : L.N, d->status,
                        st, nw, d->eps);
    int rc = rmsnorm(d->h, nw, d->x, 1, H, d->eps, st);
    return rc != Q4B_OK ? rc : gemv_q4_0(L.W, L.S, d->x, Y, AUX, L.N, L.K, epi, Q4B_X_F16, st);
  };
#define Q4B_TRY(call)            \
  do {                           \
    int rc_ = (call);            \
    if (rc_ != Q4B_OK) return rc_; \
  } while (0)
  Q4B_TRY(embed(d->embed, d->tok, d->h, 1, H, d->vocab, st));
  const bool persistent = (d->flags & Q4B_STEP_PERSISTENT) && d->persistent_ws && d->status;
  if (persistent) Q4B_TRY(decode_persistent_layers(d, d->persistent_ws, d->persistent_ws_bytes, st));
  for (int i = 0; i < d->layers && !persistent; ++i) {
    const q4b_layer& L = d->layer[i];
    const q4b_layer* Ln = i + 1 < d->layers ? &d->layer[i + 1] : nullptr;
    // look-ahead plan: qkv asks for gate/up, o for down, gate/up for the next layer's qkv and o
    if (fused_kv && mma_ok(L.qkv)) {
      GemvLookahead g{};
      look_at(g, 0, &L.gu);
      Q4B_TRY(gemv_mma(L.qkv.Wt, L.qkv.St, d->h, d->qkv, L.qkv_bias, L.qkv.N, L.qkv.K, 3, Q4B_EPI_BIASF_ROPE_KV, d->status, st, L.ln1,
                       d->eps, d->cosT, d->sinT, d->pos, L.kc, L.vc, d->n_heads, d->n_kv_heads, d->head_dim, d->max_len, -1, &g));
      Q4B_TRY(attn_decode(d->qkv, nullptr, nullptr, d->pos, L.kc, L.vc, d->att, 1, d->n_heads, d->n_kv_heads, d->head_dim,
                          d->max_len, d->scale, nullptr, 0, st, 1));
    } else {
      Q4B_TRY(norm_lin(L.ln1, L.qkv, d->qkv, L.qkv_bias, Q4B_EPI_BIASF, &L.gu));
      Q4B_TRY(attn_decode(d->qkv, d->cosT, d->sinT, d->pos, L.kc, L.vc, d->att, 1, d->n_heads, d->n_kv_heads, d->head_dim,
                          d->max_len, d->scale, d->attn_ws, d->attn_ws_bytes, st));
    }
    Q4B_TRY(lin(L.o, d->att, d->h, nullptr, Q4B_EPI_RESID, &L.down));
    Q4B_TRY(norm_lin(L.ln2, L.gu, d->act, nullptr, Q4B_EPI_SWIGLU, Ln ? &Ln->qkv : nullptr, Ln ? &Ln->o : nullptr));
    Q4B_TRY(lin(L.down, d->act, d->h, nullptr, Q4B_EPI_RESID));
  }
  (void)QR;
  if (d->head.W) {
    Q4B_TRY(norm_lin(d->norm, d->head, d->logits, nullptr, Q4B_EPI_LOGITS));
    Q4B_TRY(argmax_advance(d->logits, 1, d->vocab, d->tok, d->pos, d->head_ws, d->head_ws_bytes, st));
  } else if (d->head_q6_L && d->head_q6_H && d->head_q6_SC && d->head_q6_D && (H % 512) == 0 && H <= 2048) {
    Q4B_TRY(rmsnorm(d->h, d->norm, d->x, 1, H, d->eps, st));
    Q4B_TRY(head_q6_k_argmax(d->head_q6_L, d->head_q6_H, d->head_q6_SC, d->head_q6_D, d->x, d->logits, d->vocab, H, d->tok, d->pos,
                             d->head_ws, d->head_ws_bytes, st));
  } else {
    Q4B_TRY(rmsnorm(d->h, d->norm, d->x, 1, H, d->eps, st));
    Q4B_TRY(head_f16_argmax(d->head16 ? d->head16 : d->embed, d->x, d->logits, d->vocab, H, d->tok, d->pos, d->head_ws,
                            d->head_ws_bytes, st));
  }
#undef Q4B_TRY
  return Q4B_OK;
}

size_t q4b_decode_persistent_workspace(const q4b_decode_desc* desc) { return decode_persistent_workspace(desc); }
int q4b_decode_persistent_prepare(const q4b_decode_desc* desc, void* ws, size_t ws_bytes) {
  return decode_persistent_prepare(desc, ws, ws_bytes);
}
int q4b_decode_persistent_layers(const q4b_decode_desc* desc, void* ws, size_t ws_bytes, q4b_stream_t stream) {
  return decode_persistent_layers(desc, ws, ws_bytes, S(stream));
}
int q4b_decode_persistent_trace(uint64_t* device_buffer, int stride) {
  decode_persistent_trace(reinterpret_cast<unsigned long long*>(device_buffer), device_buffer ? stride : 0);   // stride < 0: |stride| stamps per CTA, stages subdivided
  return Q4B_OK;
}

}  // extern "C"
