/* libq4b200 — C-ABI of the B200 (sm_100a) Qwen2.5 Q4_0 inference hot path.
 *
 * The reference launches every kernel through `Kern(src).launch(grid, block, args)` (scripts/qwen_fused.py:30-42;
 * 2-D grid + dynamic shared memory variant scripts/qwen_batched_decode.py:51-67): raw device pointers as 64-bit
 * integers, int32/float scalars, the launch on torch's current stream, buffers owned by the caller, no allocation
 * and no synchronisation inside.  Each function below replaces one such launch site (the kernel source it stands in
 * for is cited per function); grid/block/shared-memory choices move inside the library.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the comment says "host";
 *   - `stream` is a cudaStream_t passed as void* (0 = legacy default stream); launches are capturable in CUDA graphs;
 *   - return value: Q4B_OK or a negative Q4B_E_* code; shapes, alignment and workspace sizes are validated on the
 *     host before anything is launched; q4b_last_error() returns a text for the last failure on the calling thread;
 *   - nothing here allocates or frees device memory, and nothing synchronises;
 *   - workspaces and counters are caller-allocated, must be zero-filled once before first use, and are left zeroed
 *     again by each kernel that uses them (self-resetting, as the reference's `cnt` / `fin_cnt` words,
 *     lab/qwen_batched.py:659-661, lab/qwen_kernels.py:280).
 *
 * Layouts
 *   Q4_0 tile-packed (tensor-core kernels): Wt int32 [T, K/32, 128, 4], St fp16 [T, K/32, 128] with T = ceil(N/128):
 *   the 16 bytes of (row r of tile t, k-block b) sit at ((t * K/32 + b) * 128 + r) * 16; made by q4b_pack_q4_0.
 *   Q4_0 canonical: W int32 [N, K/8], nibble i of word w = weight 8w+i, value (nibble-8)*d; S fp16 [N, K/32]
 *   (scripts/qwen_gguf.py:44-60).  K must be a multiple of 32; W and S 16-byte aligned.
 *   Activations fp16, residual stream and logits fp32, KV cache fp16 [B, NKV, max_len, HD] per layer,
 *   RoPE tables fp32 [max_len, HD/2], token ids and positions int64 on the device.
 */
#ifndef Q4B200_H
#define Q4B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define Q4B_OK 0
#define Q4B_E_SHAPE (-1)      /* a dimension is zero, negative, or not a multiple the kernel needs */
#define Q4B_E_ALIGN (-2)      /* a pointer is null or not 16-byte aligned */
#define Q4B_E_WORKSPACE (-3)  /* workspace_bytes is smaller than the matching *_workspace() query */
#define Q4B_E_CUDA (-4)       /* the CUDA runtime reported an error; text in q4b_last_error() */
#define Q4B_E_ARG (-5)        /* unknown epilogue / dtype / mode id */
#define Q4B_E_TIMEOUT (-6)    /* a bounded device-side wait gave up (reported through a status word) */

/* GEMV / MMQ epilogues, named as the reference's (lab/qwen_kernels.py:21-45). */
#define Q4B_EPI_STORE 0   /* Y fp16 [N]        = acc */
#define Q4B_EPI_BIASF 1   /* Y fp16 [N]        = acc + AUX fp32 [N] */
#define Q4B_EPI_RESID 2   /* Y fp32 [N]       += acc */
#define Q4B_EPI_SWIGLU 3  /* Y fp16 [N/2]      = silu(acc[2o]) * acc[2o+1]  (rows interleaved gate, up) */
#define Q4B_EPI_LOGITS 4  /* Y fp32 [N]        = acc */
#define Q4B_EPI_SWIGLU_Q8 5 /* Q8_1 MMQ only: the SwiGLU product rounded to fp16 and quantised in the epilogue:
                               Y int8 [cols, N/2], AUX (written) fp16 [cols, N/64]; N a multiple of 64 */

#define Q4B_EPI_SWIGLU_F16T 7 /* q4b_mm_prefill_q4_0_f16 only: the SwiGLU product rounded to fp16 and written in the operand
                               order of the next fp16 GEMM (Y = a q4b_f16_tiled_bytes(P, N / 2) buffer; N a multiple of 128) */
#define Q4B_EPI_BIASF_ROPE_KV 6 /* q4b_rmsnorm_qkv_rope_kv only: bias, round, RoPE of q and k, K/V append (see there) */

#define Q4B_X_F16 0
#define Q4B_X_F32 1

typedef void* q4b_stream_t;

/* Library version (major * 1000 + minor). */
int q4b_version(void);
/* Text of the last error on the calling thread ("" if none).  Host pointer, valid until the next call. */
const char* q4b_last_error(void);
/* One-time per-device set-up (function attributes, SM count).  Replaces the module load + cuFuncSetAttribute of
 * Kern.__init__ (scripts/qwen_batched_decode.py:51-58).  Idempotent. */
int q4b_init(int device);

/* Q4_0 GEMV, one activation vector.  Replaces the launch of `gemv_source(S, epi, "g32f16", G)`
 * (lab/qwen_kernels.py:14-113; host call FusedQwen.gemv scripts/qwen_fused.py:104-107).
 * X: fp16 [K] (Q4B_X_F16) or fp32 [K] (Q4B_X_F32).  Y/AUX per epilogue (see Q4B_EPI_*). */
int q4b_gemv_q4_0(const void* W, const void* S, const void* X, void* Y, const void* AUX, int N, int K, int epilogue,
                  int x_dtype, q4b_stream_t stream);

/* RMSNorm over `rows` rows: out fp16 [rows, H] = h fp32 [rows, H] * rsqrt(mean(h^2) + eps) * w fp32 [H].
 * Replaces RMSNORM_F32W_1P (lab/qwen_kernels.py:683-705; host call FusedQwen.rms scripts/qwen_fused.py:109-111). */
int q4b_rmsnorm(const float* h, const float* w, void* out, int rows, int H, float eps, q4b_stream_t stream);

/* Embedding lookup: h fp32 [rows, H] = float(E fp16 [V, H][tok[row]]).  Replaces EMBED_F32
 * (lab/qwen_kernels.py:284-290).  Token ids outside [0, V) are clamped into range. */
int q4b_embed(const void* E, const int64_t* tok, float* h, int rows, int H, int V, q4b_stream_t stream);

/* Decode attention for B sequences, one new token each: RoPE(q), RoPE(k_new), K/V append at pos[b], GQA attention
 * over positions 0..pos[b], split over the context in fixed-size chunks with a deterministic combine.
 * Replaces ATTN4 (lab/qwen_kernels.py:517-605) and the flash-decoding ATTN2 (:358-442).
 * qkv fp16 [B, (NH + 2 NKV) HD]; cosT/sinT fp32 [max_len, HD/2]; pos int64 [B]; kc/vc fp16 [B, NKV, max_len, HD];
 * out fp16 [B, NH HD].  HD must be 64 or 128, NH a multiple of NKV with NH/NKV <= 8, pos[b] < max_len.
 * workspace: q4b_attn_decode_workspace(B, NH, HD, max_len) bytes, zero-filled once. */
size_t q4b_attn_decode_workspace(int B, int NH, int HD, int max_len);
int q4b_attn_decode(const void* qkv, const float* cosT, const float* sinT, const int64_t* pos, void* kc, void* vc,
                    void* out, int B, int NH, int NKV, int HD, int max_len, float scale, void* workspace,
                    size_t workspace_bytes, q4b_stream_t stream);

/* The same attention with the Q8_1 quantiser of its output fused in: besides `out` it writes xq int8 [B, NH*HD] and
 * xd fp16 [B, NH*HD/32], exactly what q4b_quant_q8_1(out, ...) would produce, so the quantiser launch in front of
 * o_proj (QUANT_Q8, lab/qwen_batched.py:1016-1041) disappears.  Only for B >= 2, head_dim 128 and (NH / NKV) * 128 a
 * multiple of 256; otherwise it returns Q4B_E_SHAPE without launching and the caller uses the two separate calls. */
int q4b_attn_decode_q8_1(const void* qkv, const float* cosT, const float* sinT, const int64_t* pos, void* kc, void* vc,
                         void* out, void* xq, void* xd, int B, int NH, int NKV, int HD, int max_len, float scale,
                         q4b_stream_t stream);

/* LM head for a tied fp16 embedding table with the greedy pick fused: logits fp32 [V] = E fp16 [V, H] . x fp16 [H];
 * tok[0] = lowest index among the maxima; pos[0] += 1.  Replaces gemv_source(..., "logits") + FINISH_MB
 * (lab/qwen_kernels.py:14-113, 250-282; host scripts/qwen_fused.py:133-142).  tok/pos may be null (logits only).
 * workspace: q4b_head_workspace(V) bytes, zero-filled once. */
size_t q4b_head_workspace(int V);
int q4b_head_f16_argmax(const void* E, const void* x, float* logits, int V, int H, int64_t* tok, int64_t* pos,
                        void* workspace, size_t workspace_bytes, q4b_stream_t stream);

/* LM head stored as Q6_K (the `output.weight` of llama.cpp's Q4_0 exports), 6.5625 bits per weight, greedy pick fused:
 * logits fp32 [V] = sum over 16-weight sub-blocks of (d * sc) * sum (q - 32) * x, fp32.  Replaces gemv_q6_source + FINISH_MB
 * (lab/qwen_kernels.py:608-678, 250-282; host scripts/qwen_gguf.py:92-104, 133-144).  Planes as the reference lays them
 * out: L uint32 [V, K/8] (low nibbles of q + 32, nibble i of word w = weight 8w+i), Hb uint32 [V, K/16] (high two bits of
 * the 16 weights of a sub-block; weight i at bit 8 ((i % 8) / 2) + 2 ((i % 2) + 2 (i / 8)), the reference uses bit 2 i),
 * SC int8 [V, K/16], D fp16 [V, K/256].  x fp16 [K].  K in {512, 1024, 1536, 2048}.
 * tok/pos may be null (logits only).  workspace: q4b_head_workspace(V) bytes, zero-filled once. */
int q4b_head_q6_k_argmax(const void* L, const void* Hb, const void* SC, const void* D, const void* x, float* logits, int V, int K,
                         int64_t* tok, int64_t* pos, void* workspace, size_t workspace_bytes, q4b_stream_t stream);

/* The same greedy pick for callers that may not allocate device memory.  (No counterpart in the reference: there the
 * caller always owns a torch-allocated workspace.)  Some hosts give a library nothing but the input and output
 * buffers and keep every allocation to themselves: a serving runtime whose device-memory budget is fixed at start-up,
 * or a binding from a language whose foreign-function layer can pass pointers but cannot create device buffers.  For
 * them the scratch (arrival counters and per-slice maxima) lives in a fixed array inside the library image, about
 * 33 KB per GPU for as long as the library is loaded.
 *   - at most 64 rows; more is rejected with Q4B_E_SHAPE (use q4b_argmax_advance with a workspace instead);
 *   - nothing is allocated or freed, by this function or by anything it calls;
 *   - the first call on each device looks up the array's device address (that device must be current); make that
 *     first call before any stream capture begins;
 *   - all calls on a device share the one array: two calls whose kernels can overlap on the GPU (different streams,
 *     no ordering between them) race on it and give wrong results.  Calls ordered on one stream are fine; the counters
 *     are cleared at the start of every call;
 *   - the looked-up address is kept for as long as the device's primary context lives (after a cudaDeviceReset or a
 *     context teardown it is stale: reload the library), and `stream` must belong to the device that is current. */
int q4b_argmax_advance_static(const float* logits, int rows, int V, int64_t* tok, int64_t* pos, q4b_stream_t stream);

/* LM head over the tied fp16 table for B = 1..32 sequences: logits fp32 [B, V] = x fp16 [B, H] . E fp16 [V, H]^T.
 * Replaces head_v2_source / the cuBLAS fp16 head of the batched engine (lab/qwen_batched.py:681-833,
 * scripts/qwen_batched_decode.py:172-185).  H a multiple of 32.  Follow with q4b_argmax_advance for the greedy pick. */
int q4b_head_f16_batched(const void* E, const void* x, float* logits, int V, int H, int B, q4b_stream_t stream);

/* Greedy pick over fp32 logits [rows, V]: tok[r] = lowest index among the maxima of row r; pos[r] += 1.
 * Replaces FINISH / FINISH_MB (lab/qwen_kernels.py:222-282) and the torch.argmax of the batched engine
 * (scripts/qwen_batched_decode.py:186-187).  workspace: q4b_argmax_workspace(rows, V) bytes, zero-filled once. */
size_t q4b_argmax_workspace(int rows, int V);
int q4b_argmax_advance(const float* logits, int rows, int V, int64_t* tok, int64_t* pos, void* workspace,
                       size_t workspace_bytes, q4b_stream_t stream);

/* ---- tensor-core block dots (verification entry) ----------------------------------------------------------------
 * out int32 [P, M, K/32]: out[n, m, b] = sum_{i<32} (q4[m, 32b+i] - 8) * xq[n, 32b+i], exact, computed with
 * tcgen05.mma.kind::i8.  The reference obtains the same integers from mma.m16n8k32.u8.s8 with the -8*sum(q8)
 * correction in the C operand (lab/qwen_batched.py:1237-1243); its tensor-core known-answer check demands exact
 * equality (lab/experiments/tensor.py:122-200).  W canonical Q4_0 words [M, K/8]; xq int8 [P, K].
 * mode bit 0: 0 = A operand staged in shared memory, 1 = A operand written to tensor memory; mode >> 1: tile width
 * (8, 16, 32; 0 = pick from P).  status: one uint32 the kernel sets to 1 if a bounded wait expired (zero it first). */
int q4b_blockdot_q4_0_q8_1(const void* W, const void* xq, int32_t* out, int M, int K, int P, int mode,
                           uint32_t* status, q4b_stream_t stream);

/* Repack canonical Q4_0 into the tile-packed layout (same bytes, last tile zero-padded).  Wt needs
 * ceil(N/128) * 128 * K/2 bytes, St ceil(N/128) * 128 * K/32 * 2 bytes.  Counterpart of the reference's repackers
 * pack_q4_mma / pack_q4_i8 (lab/qwen_batched.py:394-436, 987-1013). */
int q4b_pack_q4_0(const void* W, const void* S, void* Wt, void* St, int N, int K, q4b_stream_t stream);

/* ---- tensor-core path for decode --------------------------------------------------------------------------------
 * Q4_0 GEMV for one activation vector on the tcgen05 int8 tensor cores, exact: each 32-value block of x is split
 * into signed base-256 digits of a block-fixed-point integer, the digits are the columns of an int8 MMA, and the
 * integer block dots are recombined and scaled in fp32.  Same contract and epilogues as q4b_gemv_q4_0 (it replaces
 * the same launch site, lab/qwen_kernels.py:14-113) except that the weights are passed TILE-PACKED (Wt, St from
 * q4b_pack_q4_0); K must be a multiple of 256.  Launched with programmatic
 * dependent launch: the weight prefetch overlaps the kernel that precedes it in the stream.
 * status: one uint32, set to 1 if a bounded device-side wait expired (zero it once; check when convenient). */
int q4b_gemv_q4_0_tc(const void* Wt, const void* St, const void* X, void* Y, const void* AUX, int N, int K, int epilogue,
                     int x_dtype, uint32_t* status, q4b_stream_t stream);

/* ---- streaming GEMV for decode at batch 1 ----------------------------------------------------------------------------
 * Q4_0 GEMV for one activation vector, exact (four signed base-256 digit planes of a 30-bit block-fixed-point x, int32
 * block dots by mma.sync.m16n8k32.s8 with register accumulators, fp32 scale-and-add per block).  Same contract,
 * epilogues and tile-packed weights as q4b_gemv_q4_0_tc; it replaces the same launch site (gemv_source,
 * lab/qwen_kernels.py:14-113; host FusedQwen.gemv scripts/qwen_fused.py:104-107).  K a multiple of 32.  The CTA's whole
 * weight slab is bulk-copied into shared memory ahead of the programmatic-dependency wait, so in a chain of launches
 * the HBM stream of one kernel overlaps the computation of the one before it.
 * status: one uint32, set non-zero if a bounded device-side wait expired (zero it once; check when convenient). */
int q4b_gemv_q4_0_mma(const void* Wt, const void* St, const void* X, void* Y, const void* AUX, int N, int K, int epilogue,
                      int x_dtype, uint32_t* status, q4b_stream_t stream);

/* RMSNorm fused in front of q4b_gemv_q4_0_mma (see q4b_rmsnorm_gemv_q4_0_tc).  h, norm_w fp32 [K]. */
int q4b_rmsnorm_gemv_q4_0_mma(const void* Wt, const void* St, const float* h, const float* norm_w, float eps, void* Y,
                              const void* AUX, int N, int K, int epilogue, uint32_t* status, q4b_stream_t stream);

/* Which kernel q4b_attn_decode uses for B >= 2 sequences (head_dim 128): 0 (default) = the shared-memory-resident form
 * (whole chunk of K / V requested ahead of the dependency wait, RoPE and append inside) where max_len <= 2048, else the
 * streaming tensor-core kernel; 1 = always the streaming kernel.  Process-wide; meant for A/B measurements. */
int q4b_attn_batched_kernel(int which);

/* The QKV projection of one decode token with everything up to the cache write fused in: RMSNorm(h) -> Q4_0 GEMV ->
 * + bias, round to fp16 -> NeoX rotation of the q and k heads at position pos[0] from the ROUNDED values, rounded
 * again -> rotated k and raw v stored into the cache row pos[0].  This is the `biasf_kv` epilogue of the reference's
 * prefill GEMM (lab/qwen_batched.py:1316-1362) applied to the decode step, where the reference rotates inside the
 * attention kernel instead (ATTN4, lab/qwen_kernels.py:533-547); the values are the same.
 * qkv fp16 [(NH + 2 NKV) HD] receives rotated q, rotated k, v.  bias fp32 [(NH + 2 NKV) HD].  kc / vc fp16
 * [NKV, max_len, HD] (one sequence).  HD must divide 128 (a row tile holds whole heads).  Follow with
 * q4b_attn_decode_cached. */
int q4b_rmsnorm_qkv_rope_kv(const void* Wt, const void* St, const float* h, const float* norm_w, float eps, void* qkv,
                            const float* bias, int K, const float* cosT, const float* sinT, const int64_t* pos, void* kc,
                            void* vc, int NH, int NKV, int HD, int max_len, uint32_t* status, q4b_stream_t stream);

/* ---- batched-decode GEMV on fp16 tensor-core MMAs (the reference's own batched-decode arithmetic) ---------------------
 * Y[b, :] = epilogue(X[b, :] . W^T) for B = 1 .. 32 activation rows, with the weights dequantised to fp16 the way the
 * reference's batched-decode kernel does it (gemv_v2_source, lab/qwen_batched.py:467-641, nibble -> half2 through the
 * 0x6400 trick, times the fp16 block scale ROUNDED to fp16, `dq` :493-498) and multiplied by the fp16 activations in
 * mma.sync.m16n8k16 with fp32 accumulation.  It replaces the launch site Batched.step uses for qkv / o / gate_up / down
 * (scripts/qwen_batched_decode.py:156-187, `self.g[name]`), reading the tile-packed weights of q4b_pack_q4_0 instead
 * of a fragment-ordered copy (pack_q4_mma, lab/qwen_batched.py:394-436).  The result differs from the exact block-dot
 * kernels by the fp16 rounding of d * (q - 8): 2e-4 .. 5e-3 relative, as the reference documents for this path.
 * X fp16 [B, K]; Y [B, ldy]: fp16 for STORE / BIASF / SWIGLU (ldy >= N, or N / 2 for SWIGLU), fp32 for RESID (Y += result)
 * and LOGITS.  AUX: fp32 bias [N] for BIASF.  K a multiple of 32.
 * status: one uint32, set non-zero if a bounded device-side wait expired. */
int q4b_gemv_q4_0_f16mma(const void* Wt, const void* St, const void* X, void* Y, const void* AUX, int N, int K, int B,
                         int epilogue, int ldy, uint32_t* status, q4b_stream_t stream);

/* Q8_1 x Q4_0 for 1 .. 32 activation rows with register accumulators: the contract of q4b_mmq_q4_0_q8_1 (same launch
 * site: the linears of Batched.step, scripts/qwen_batched_decode.py:156-187, with the block arithmetic of the
 * reference's int8 MMQ, lab/qwen_batched.py:1237-1243: exact int32 dot per 32-weight block by mma.sync.m16n8k32.s8 with
 * the magic constant planted in the accumulator, then acc += d_w * d_x * float(dot) in fp32, blocks in ascending k
 * within a k group).  Epilogues STORE / BIASF / RESID / SWIGLU / SWIGLU_Q8 (unsplit launches) / LOGITS; K a multiple of 32; xq int8 [P, K] 16-byte
 * aligned, xd fp16 [P, K / 32].  Results equal q4b_mmq_q4_0_q8_1 up to the fp32 summation order over k groups. */
int q4b_mmq_q4_0_q8_1_mma(const void* Wt, const void* St, const void* xq, const void* xd, void* Y, const void* AUX, int N, int K,
                          int P, int epilogue, int ldy, uint32_t* status, q4b_stream_t stream);

/* q4b_quant_q8_1 + q4b_mmq_q4_0_q8_1_mma in one launch: x16 fp16 [P, K] is quantised to Q8_1 inside the kernel (each CTA its
 * own K window; QUANT_Q8 arithmetic, lab/qwen_batched.py:1030-1039) and multiplied as above.  Same results, bit for bit,
 * as the two launches.  Replaces the reference's `QUANT_Q8` + `gemm8` pair (scripts/qwen_prefill.py:208-246) for <= 32 rows. */
int q4b_quant_mmq_q4_0_q8_1_mma(const void* Wt, const void* St, const void* x16, void* Y, const void* AUX, int N, int K, int P,
                                int epilogue, int ldy, uint32_t* status, q4b_stream_t stream);

/* Exercise of the failure path of the bounded device-side waits, in a form that always returns: q4b_gemv_q4_0_mma
 * (fp16 x, logits epilogue) with the bulk copies of its first weight chunk withheld and the wait cut to a few thousand
 * polls.  The wait gives up, the kernel sets *status non-zero and finishes normally; Y is meaningless.  The reference's
 * persistent kernel reports expired waits the same way (capped waits + err word, lab/qwen_mega.py:75-83, 153-161). */
int q4b_debug_gemv_mma_expired_wait(const void* Wt, const void* St, const void* X, void* Y, int N, int K, uint32_t* status,
                                    q4b_stream_t stream);

/* Decode attention of one sequence when q is already rotated and position pos[0] is already in the cache
 * (q4b_rmsnorm_qkv_rope_kv did both): attention over positions 0 .. pos[0] only, no tables, no cache write.  Same
 * arithmetic as q4b_attn_decode (ATTN4, lab/qwen_kernels.py:548-603).  max_len <= 4096.
 * The kernel reads pos[0] and the cache rows BELOW it ahead of its programmatic-dependency wait, so those must come from
 * work that completed before the chain of programmatically dependent launches it sits in began: earlier decode steps
 * (q4b_embed, which opens a step, releases its dependents only after everything before it has completed), a prefill, or
 * a copy.  Only qkv and cache row pos[0] may come from the launch directly in front of it. */
int q4b_attn_decode_cached(const void* qkv, const int64_t* pos, const void* kc, const void* vc, void* out, int NH, int NKV,
                           int HD, int max_len, float scale, q4b_stream_t stream);

/* ---- prefill: Q8_1 x Q4_0 for many activation rows ------------------------------------------------------------------
 * Tiled Q8_1 activations for the prefill MMQ: for each (tile of 128 rows, 32-value block) 4096 bytes of int8 values
 * already in the tensor-core operand order, then the 128 block scales as fp32 (fp16-rounded values).  The quantisers
 * below write this format directly; rows beyond `rows` inside the last tile must be zero (zero-fill the buffer once).
 * q4b_q8_tiled_bytes(rows, K) = ceil(rows/128) * K/32 * 4608. */
size_t q4b_q8_tiled_bytes(int rows, int K);
/* QUANT_Q8 (lab/qwen_batched.py:1016-1041) / rmsnorm_q8_source (:1044-1091) with tiled output. */
int q4b_quant_q8_1_tiled(const void* x, void* xt, int rows, int K, q4b_stream_t stream);
int q4b_rmsnorm_q8_1_tiled(const float* h, const float* w, void* xt, int rows, int H, float eps, q4b_stream_t stream);
/* Y[P, :] = epilogue(Xt x Q4_0(Wt, St)^T): the prefill GEMM (gemm_q4i8_ms_source, lab/qwen_batched.py:1271-1561;
 * host Prefill.gemm8, scripts/qwen_prefill.py:176-190) on tcgen05 int8 tensor cores with TMEM accumulators, 128 x 128
 * tiles, exact int32 block dots rescaled per k-block in fp32.  Weights tile-packed, activations tiled Q8_1, any P;
 * K a multiple of 256; Y pitch ldy elements as in q4b_mmq_q4_0_q8_1.
 * Q4B_EPI_SWIGLU_Q8 (lab/qwen_batched.py:1363-1396): Y is a tiled Q8_1 buffer of q4b_q8_tiled_bytes(P, N / 2) bytes that
 * receives the SwiGLU product rounded to fp16 and quantised (the operand of the `down` GEMM); N a multiple of 128; AUX
 * and ldy unused. */
int q4b_mmq_prefill_q4_0_q8_1(const void* Wt, const void* St, const void* xt, void* Y, const void* AUX, int N, int K,
                              int P, int epilogue, int ldy, uint32_t* status, q4b_stream_t stream);

/* The prefill QKV projection with the reference's `biasf_kv` epilogue (lab/qwen_batched.py:1316-1362; launch site
 * Prefill.chunk, scripts/qwen_prefill.py:200-207): Q8_1 x Q4_0 GEMM + bias, rounded to fp16; the q and k heads rotated
 * (NeoX pairs) at positions pos0 + row from the ROUNDED values and rounded again; rotated k and raw v written into the
 * cache rows pos0 .. pos0 + P - 1 of ONE sequence.  qkv fp16 [P, (NH + 2 NKV) 128] receives rotated q, rotated k, v
 * (the reference leaves q un-rotated for its flash kernel; here the rotation happens once, in this epilogue).
 * bias fp32 [(NH + 2 NKV) 128]; cosT / sinT fp32 [max_len, 64]; kc / vc fp16 [NKV, max_len, 128].  HD must be 128.
 * Follow with q4b_attn_prefill_cached. */
int q4b_mmq_prefill_qkv_rope_kv(const void* Wt, const void* St, const void* xt, void* qkv, const float* bias, int K, int P,
                                const float* cosT, const float* sinT, int pos0, void* kc, void* vc, int NH, int NKV, int HD,
                                int max_len, uint32_t* status, q4b_stream_t stream);

/* Causal GQA flash attention of P prompt tokens whose q rows are already rotated and whose K/V rows are already in the
 * cache (q4b_mmq_prefill_qkv_rope_kv), flash_prefill_v3_source (lab/qwen_batched.py:1795-2037) in one launch.  Outputs,
 * either or both: out fp16 [P, NH 128]; xt = the same values as tiled Q8_1 (K = NH 128), the `q8` output of the
 * reference's kernel (:1812-1848) that feeds the o-projection GEMM without a separate quantiser launch. */
int q4b_attn_prefill_cached(const void* qkv, const void* kc, const void* vc, void* out, void* xt, int P, int NH, int NKV,
                            int HD, int max_len, int pos0, float scale, q4b_stream_t stream);

/* The prefill GEMM in the arithmetic of the reference's `cublas` prefill mode (scripts/qwen_prefill.py:37-53 DEQ kernel,
 * :156-160 fp16 matmul; the same `dq` as its fp16 batched GEMV, lab/qwen_batched.py:493-498): weights dequantised to fp16
 * ((q - 8) exact, times the block scale, rounded once), fp16 activations, fp32 accumulation over all of K - here inside one
 * kernel: the expander warps write the fp16 A operand into tensor memory, tcgen05.mma.kind::f16 accumulates, no dense fp16
 * copy of the matrix and no per-block rescale; the epilogue works on the fp32 sums (the reference's matmul rounds them to
 * fp16 first), and its SwiGLU forms the quotient with the approximate reciprocal (2 ulp of fp32, below the fp16 rounding of
 * the product).  About 3.7 times the speed of the int8 MMQ above on B200 and free of the activations' int8 rounding.  xt = q4b_f16_tiled(x): q4b_f16_tiled_bytes(rows, K) = ceil(rows/128) *
 * K/32 * 8192 bytes, zero-filled once by the caller.  Epilogues store, biasf, resid, swiglu, swiglu_f16t, logits. */
size_t q4b_f16_tiled_bytes(int rows, int K);
int q4b_f16_tiled(const void* x, void* xt, int rows, int K, q4b_stream_t stream);
int q4b_mm_prefill_q4_0_f16(const void* Wt, const void* St, const void* xt, void* Y, const void* AUX, int N, int K, int P,
                            int epilogue, int ldy, uint32_t* status, q4b_stream_t stream);

/* fp16 mode of q4b_mmq_prefill_resid_ksplit (same contract: Y += part 0, Y2[z - 1] = part z), and the RMSNorm that completes
 * h with n_add (0 .. 3) such parts and writes its fp16 result straight into the fp16 operand order (q4b_f16_tiled's). */
int q4b_mm_prefill_f16_resid_ksplit(const void* Wt, const void* St, const void* xt, float* Y, float* Y2, int parts, int N, int K, int P,
                                    int ldy, uint32_t* status, q4b_stream_t stream);
int q4b_rmsnorm_f16_tiled_add(float* h, const float* h_add, int n_add, const float* w, void* xt, int rows, int H, float eps,
                              q4b_stream_t stream);

/* The failure path of the prefill GEMM's bounded waits, in a form that always returns: q4b_mmq_prefill_q4_0_q8_1 (logits
 * epilogue, ldy = N) with its copy thread issuing nothing, so that every wait of the pipeline runs into its limit (about a
 * second by the SM clock).  The threads stop waiting, the kernel sets *status non-zero, frees its tensor memory and ends;
 * Y is meaningless. */
int q4b_debug_mmq_prefill_expired_wait(const void* Wt, const void* St, const void* xt, void* Y, int N, int K, int P, uint32_t* status,
                                       q4b_stream_t stream);

/* Pipeline timeline of the prefill GEMM: while a device buffer of 11 x 64 int64 is set, every q4b_mmq_prefill_* launch
 * runs a second instance of the kernel whose CTA (0, 0, 0) writes SM-clock stamps for its first 64 k-blocks, one row per
 * event: 0 activation stage requested, 1 A operand written (first expander warp), 2 MMA issued and committed, 3 accumulator
 * seen complete by the first rescale warp, 4 that warp has read it out (slot handed back), 5 that warp has folded it,
 * 6 .. 9 the MMA issuer before its waits for the A operand, the activation stage, a free accumulator slot, and after them;
 * row 10 holds the CTA's phases: entry, set-up done, main loop left, epilogue written, tensor memory released.
 * Null switches back to the plain instance (the default).  Used by `3080lab_b200/timeline.py prefill`. */
int q4b_mmq_prefill_trace(int64_t* device_buffer, size_t entries);

/* The residual-adding prefill GEMM with its launch split along K into `parts` (2 .. 4) CTAs per output tile: Y += part 0,
 * Y2[z - 1] = part z (fp32 [parts - 1][P, ldy], overwritten).  o_proj and down_proj have 12 row tiles x P / 128 token
 * tiles = 192 CTAs on 148 SMs at P = 2048; as 384 half-length CTAs they fill the machine in 1.5 instead of 2 rounds, as 576
 * third-length ones in 1.33.  The next reader of Y must add the parts: q4b_rmsnorm_q8_1_tiled_add does (h += h_add[0] + ..,
 * written back, then RMSNorm + tiled Q8_1), and q4b_add_rows after the last layer.  The order of the additions is fixed,
 * so results are bit-repeatable. */
int q4b_mmq_prefill_resid_ksplit(const void* Wt, const void* St, const void* xt, float* Y, float* Y2, int parts, int N, int K, int P,
                                 int ldy, uint32_t* status, q4b_stream_t stream);
int q4b_rmsnorm_q8_1_tiled_add(float* h, const float* h_add, int n_add, const float* w, void* xt, int rows, int H, float eps,
                               q4b_stream_t stream);
int q4b_add_rows(float* h, const float* h_add, int n_add, size_t n, q4b_stream_t stream);

/* Prefill attention for one sequence: rotate K (NeoX pairs) and append K/V of P prompt tokens at positions
 * pos0 .. pos0+P-1, then causal GQA flash attention of the P queries (rotated inside) over positions 0 .. pos0+P-1.
 * Replaces the K/V write of the `biasf_kv` epilogue (lab/qwen_batched.py:1316-1362) and flash_prefill_v3_source
 * (:1795-2037; host Prefill.chunk scripts/qwen_prefill.py:196-246).  qkv fp16 [P, (NH + 2 NKV) HD] (bias added,
 * un-rotated); kc/vc fp16 [NKV, max_len, HD]; out fp16 [P, NH HD].  HD = 128. */
int q4b_attn_prefill(const void* qkv, const float* cosT, const float* sinT, void* kc, void* vc, void* out, int P, int NH,
                     int NKV, int HD, int max_len, int pos0, float scale, q4b_stream_t stream);

/* Optional in-kernel timeline of the tensor-core kernels: while a buffer is set, thread 0 of every CTA writes up to 15
 * %globaltimer stamps (ns) at its phase boundaries into buffer[cta * 16 ..], and the count into entry 15.  The
 * reference has the same facility (`timed=True`, lab/qwen_kernels.py:46-53).  entries >= 4096 * 16; null switches it
 * off.  Host-side global state: not thread-safe, meant for profiling runs. */
int q4b_trace_buffer(uint64_t* device_buffer, size_t entries);

/* Peak of the int8 tensor-core path on this device, for roofline denominators: one launch of `iters` back-to-back
 * tcgen05.mma.kind::i8 (M 128, N 256, K 32) per SM onto one accumulator tile.  Returns the number of int8 operations the
 * launch executes (0.0 on error); the caller times the launch with events and divides.  status: one uint32, set
 * non-zero if the bounded completion wait expired.  (The reference measures its tensor peaks with a microbenchmark of
 * the same kind, lab/experiments/tensor.py.) */
double q4b_peak_i8_launch(int iters, uint32_t* status, q4b_stream_t stream);

/* Timeline of a whole chain of launches (for example one captured decode step): while a buffer is set, every launch of
 * the batch-1 GEMV (kernel id 1) and of the one-sequence attention (id 2) takes the next free region of the buffer,
 * 16 stamps per CTA as above, and the library keeps a host-side record per launch.  Because the region is fixed at
 * launch (capture) time, replays of a captured graph rewrite the same regions.  q4b_trace_chain(null, 0) stops handing
 * out regions (already captured launches keep theirs: keep the buffer alive while such a graph can run).
 * q4b_trace_chain_log copies up to max_records records of three int64 (kernel id, CTAs, offset of the region in
 * entries) to HOST memory and returns how many launches were recorded.  No reference counterpart beyond `timed=True`
 * (lab/qwen_kernels.py:46-53).  Host-side global state: not thread-safe, meant for profiling runs. */
int q4b_trace_chain(uint64_t* device_buffer, size_t entries);
int q4b_trace_chain_log(int64_t* records, int max_records);

/* RMSNorm fused in front of q4b_gemv_q4_0_tc: x = round16(h * rsqrt(mean(h^2) + eps) * norm_w) is formed while the
 * activation operand is staged, so the norm costs no launch (the reference tried the opposite fusion, norm in the
 * tail of the producing GEMV, lab/qwen_kernels.py:54-85, and measured it slower).  h, norm_w fp32 [K]. */
int q4b_rmsnorm_gemv_q4_0_tc(const void* Wt, const void* St, const float* h, const float* norm_w, float eps, void* Y,
                             const void* AUX, int N, int K, int epilogue, uint32_t* status, q4b_stream_t stream);

/* Q8_1 x Q4_0 matrix product ("MMQ") for P <= 32 activation rows (batched decode): Y[p, n] = epilogue(sum over
 * k-blocks of dw[n, b] * dx[p, b] * dot(p, n, b)) with exact int32 block dots.  Replaces the launch of
 * gemm_q4i8_ms_source (lab/qwen_batched.py:1271-1561; host Prefill.gemm8 scripts/qwen_prefill.py:176-190) and, for
 * batched decode, of gemv_v2_source (lab/qwen_batched.py:467-641; host Batched.gemv
 * scripts/qwen_batched_decode.py:138-154).  Weights tile-packed; xq int8 [P, K], xd fp16 [P, K/32]; Y rows have pitch
 * ldy elements:
 * store/biasf fp16 [P, ldy], resid/logits fp32 [P, ldy], swiglu fp16 [P, ldy] with N/2 outputs per row. */
int q4b_mmq_q4_0_q8_1(const void* Wt, const void* St, const void* xq, const void* xd, void* Y, const void* AUX, int N,
                      int K, int P, int epilogue, int ldy, uint32_t* status, q4b_stream_t stream);

/* Q8_1 quantiser: xq int8 [rows, K], xd fp16 [rows, K/32] (= amax/127 rounded to fp16), xsum fp16 [rows, K/32]
 * (= d * sum(q), may be null) from x fp16 [rows, K].  Replaces QUANT_Q8 (lab/qwen_batched.py:1016-1041). */
int q4b_quant_q8_1(const void* x, void* xq, void* xd, void* xsum, int rows, int K, q4b_stream_t stream);

/* RMSNorm fused with the Q8_1 quantiser (rmsnorm_q8_source, lab/qwen_batched.py:1044-1091): the normalised row is
 * rounded to fp16, then quantised.  x16 (fp16 [rows, H], may be null) also receives the rounded row.
 * H a multiple of 128, at most 4096. */
int q4b_rmsnorm_q8_1(const float* h, const float* w, void* xq, void* xd, void* xsum, void* x16, int rows, int H,
                     float eps, q4b_stream_t stream);

/* ---- whole decode step, batch 1 -------------------------------------------------------------------------------
 * One greedy decode token through every layer, launched back to back on `stream` (capturable as one CUDA graph).
 * Replaces the launch sequence of FusedQwen.step (scripts/qwen_fused.py:113-145): embed, then per layer
 * rmsnorm -> qkv GEMV(+bias) -> attention -> o GEMV(+residual) -> rmsnorm -> gate/up GEMV(+SwiGLU) -> down
 * GEMV(+residual), then final rmsnorm -> LM head -> argmax, pos += 1.  The descriptor is a HOST struct of device
 * pointers; the caller owns every buffer.  `layer` points to a host array of `layers` entries. */
typedef struct {
  const void* W;   /* canonical: int32 [N, K/8] */
  const void* S;   /* canonical: fp16  [N, K/32] */
  int N, K;
  const void* Wt;  /* tile-packed copy for the tensor-core path, or null */
  const void* St;
} q4b_linear;

typedef struct {
  const float* ln1;       /* fp32 [hidden] */
  const float* ln2;
  const float* qkv_bias;  /* fp32 [qkv rows] */
  q4b_linear qkv, o, gu, down;
  void* kc;               /* fp16 [batch, n_kv_heads, max_len, head_dim] */
  void* vc;
} q4b_layer;

typedef struct {
  int layers, hidden, ffn, n_heads, n_kv_heads, head_dim, vocab, max_len;
  float eps, scale;
  const void* embed;      /* fp16 [vocab, hidden]; also the LM head when head.W is null */
  const q4b_layer* layer; /* host array */
  const float* norm;      /* fp32 [hidden] */
  q4b_linear head;        /* Q4_0 head, or W = S = null for the tied fp16 head */
  const float* cosT;      /* fp32 [max_len, head_dim/2] */
  const float* sinT;
  int64_t* tok;           /* [1] in: token to feed, out: greedy pick */
  int64_t* pos;           /* [1] in: its position, out: +1 */
  float* h;               /* fp32 [hidden] residual stream */
  void* x;                /* fp16 [hidden] */
  void* qkv;              /* fp16 [qkv rows] */
  void* att;              /* fp16 [n_heads * head_dim] */
  void* act;              /* fp16 [ffn] */
  float* logits;          /* fp32 [vocab] */
  void* attn_ws;  size_t attn_ws_bytes;   /* q4b_attn_decode_workspace(1, ...) */
  void* head_ws;  size_t head_ws_bytes;   /* max(q4b_head_workspace, q4b_argmax_workspace(1, vocab)) */
  uint32_t* status;       /* [1] set non-zero when a bounded device-side wait expired (tensor-core paths); zero it once */
  int flags;              /* Q4B_STEP_* */
  void* persistent_ws;    /* Q4B_STEP_PERSISTENT: q4b_decode_persistent_workspace bytes, prepared once */
  size_t persistent_ws_bytes;
  const void* head16;     /* untied fp16 LM head [vocab, hidden] (a GGUF `output.weight` kept in fp16), or null: with
                             head.W null the head is then `embed` (tied) */
  const void* head_q6_L;  /* Q6_K LM head planes (see q4b_head_q6_k_argmax), or all null; taken when head.W is null and */
  const void* head_q6_H;  /* hidden is 512 .. 2048 in steps of 512 */
  const void* head_q6_SC;
  const void* head_q6_D;
} q4b_decode_desc;

#define Q4B_STEP_TENSOR_CORE 1  /* linears through q4b_gemv_q4_0_tc where K is a multiple of 256 */
#define Q4B_STEP_PERSISTENT 2   /* all layers in one cooperative kernel (q4b_decode_persistent_layers) */
#define Q4B_STEP_MMA_GEMV 4     /* linears through q4b_gemv_q4_0_mma, QKV through q4b_rmsnorm_qkv_rope_kv + q4b_attn_decode_cached */
#define Q4B_STEP_LOOKAHEAD 8    /* with Q4B_STEP_MMA_GEMV: each GEMV launch also asks for the weights of launches two to three
                                   places down the chain to be brought into L2 (cp.async.bulk.prefetch.L2); off by default */

/* ---- tensor-parallel reduction fused with the residual add and the next RMSNorm + Q8_1 quantiser ---------------------
 * h[b, :] += sum over ranks r = 0 .. world - 1 (in that order) of parts[r][b, :];  then, when norm_w is given,
 * (xq, xd) = Q8_1(round16(RMSNorm(h[b, :]) * norm_w)) exactly as q4b_rmsnorm_q8_1 would produce them.  One launch in
 * place of an NCCL all-reduce, the residual add and the quantiser (the reference is single-GPU: its pieces are the
 * `resid` epilogue, lab/qwen_kernels.py:21-45, and rmsnorm_q8_source, lab/qwen_batched.py:1044-1091).
 * parts / flags are HOST arrays of `world` device pointers valid on this GPU: parts[r] = rank r's partial [rows, H] fp32
 * for THIS call, flags[r] = rank r's flag array of world * rows uint32 (zeroed once, before the first call, on every
 * rank).  Peer memory is read with plain loads over NVLink (no multicast).  Contract: every rank calls with the same,
 * strictly increasing `epoch` (1, 2, ...), and alternates between two sets of partial buffers from call to call, so
 * that a rank's next-but-one GEMM cannot overwrite a partial a peer is still reading.  world = 1 degenerates to
 * h += parts[0] (flags unused).  H a multiple of 32, at most 4096; one CTA per row.
 * status: bit 1 is set when the bounded wait for a peer's arrival expired (the kernel then finishes on whatever it
 * reads; no hang). */
int q4b_tp_allreduce_resid_rmsnorm_q8(const void* const* parts, void* const* flags, int rank, int world, uint32_t epoch,
                                      const uint32_t* epoch_base, float* h, int rows, int H, const float* norm_w, float eps,
                                      void* xq, void* xd, uint32_t* status, q4b_stream_t stream);
/* *epoch_base += by, ordered after the launches before it on the stream (see above). */
int q4b_tp_epoch_advance(uint32_t* epoch_base, uint32_t by, q4b_stream_t stream);

/* Exercise of that kernel's failure path in a form that always returns: the same call with the wait cut to a few
 * thousand polls.  With flags nobody raises (a peer that never arrives) the wait gives up, *status gets bit 1, the
 * kernel finishes. */
int q4b_debug_tp_allreduce_expired_wait(const void* const* parts, void* const* flags, int rank, int world, uint32_t epoch,
                                        float* h, int rows, int H, uint32_t* status, q4b_stream_t stream);

int q4b_decode_step(const q4b_decode_desc* desc, q4b_stream_t stream);

/* ---- persistent decode: every layer of one batch-1 token in ONE cooperative kernel, one CTA per SM -------------
 * Same arithmetic and rounding points as the launch sequence above (scripts/qwen_fused.py:113-145: rmsnorm, qkv
 * GEMV + bias, RoPE / KV append / attention, o GEMV + residual, rmsnorm, gate/up GEMV + SwiGLU, down GEMV +
 * residual, per layer), but the ops are separated by grid barriers instead of kernel boundaries and the Q4_0 weights
 * stream through a shared-memory ring that never waits for activations.  Every layer matrix needs its tile-packed
 * copy (q4b_pack_q4_0); hidden a multiple of 256, head_dim 64 or 128, at most 8 query heads per KV head.
 *   workspace: bytes of device scratch for this model shape (0 if the shape is not supported).
 *   prepare:   one-time, synchronous: writes the device-side layer table into the workspace and zeroes its counters.
 *   layers:    in: desc->h = embedding row of the token, desc->pos = its position; out: desc->h = residual stream
 *              after the last layer, K/V rows appended.  desc->act is used as scratch.  Launches must not overlap
 *              on one workspace.  A bounded wait that expires sets *desc->status (2: grid barrier, 1: pipeline). */
size_t q4b_decode_persistent_workspace(const q4b_decode_desc* desc);
int q4b_decode_persistent_prepare(const q4b_decode_desc* desc, void* ws, size_t ws_bytes);
int q4b_decode_persistent_layers(const q4b_decode_desc* desc, void* ws, size_t ws_bytes, q4b_stream_t stream);
/* Optional timeline of the next persistent launches: `stride` %globaltimer stamps per CTA (start, after each grid
 * barrier, end) into a device buffer of (SM count) x stride uint64; null switches it off.  No reference counterpart. */
int q4b_decode_persistent_trace(uint64_t* device_buffer, int stride);

#ifdef __cplusplus
}
#endif
#endif /* Q4B200_H */
