/* lc0b200 — C ABI of the sm_100a kernels for the Lc0 BT4 transformer forward pass.
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer unless its name ends in _host.
 *  - "bf16" buffers hold __nv_bfloat16; the reference stores the same tensors as fp16.
 *  - Argument order follows the reference's kernel ABI: output pointers first, then
 *    inputs, then weights, then the integers the reference bakes into each op's
 *    specialization dataclass (same names), then the CUDA stream (a cudaStream_t
 *    passed as void*; NULL is the legacy default stream).
 *  - Every entry point returns an LC0B200_* status, never throws, never allocates,
 *    never synchronises (lc0b200_device_status is the one exception: it synchronises
 *    the device to read the flag word).  In-place use (out == in) is allowed wherever
 *    the reference graph does it.
 *  - Every call works on the CUDA device that is current in the calling thread; what the
 *    library keeps between calls (device addresses of its own symbols, kernel attributes,
 *    SM counts) is kept per device behind a mutex, so one process may drive several GPUs
 *    from several threads.  A failed kernel launch is reported by the call that made it
 *    and cleared; composite entry points (fused_qkv_projection, linear_int8*, net_forward)
 *    may have launched part of their kernels when they return an error.
 *  - Stream order is kept: results of a call are visible to whatever follows it on the same
 *    stream.  Kernels are launched with programmatic stream serialisation (their set-up may
 *    overlap the tail of the kernel before them on the stream; they wait for that kernel to
 *    complete before they touch global memory), which a caller's own kernels, copies and
 *    events on the stream need not know about.
 *  - Citations "K/x.py" are packages/lczero-triton/src/lczero_triton/bt4/kernels/x.py,
 *    "N" is packages/lczero-triton/src/lczero_triton/bt4/network.py and "T/x.py" is
 *    packages/lczero-triton/tests/x.py of the reference.
 */
#ifndef LC0B200_H_
#define LC0B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define LC0B200_API __attribute__((visibility("default")))
#else
#define LC0B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum {
  LC0B200_OK = 0,
  LC0B200_ERR_NULL_POINTER = 1,
  LC0B200_ERR_BAD_SHAPE = 2,
  LC0B200_ERR_UNSUPPORTED = 3,
  LC0B200_ERR_MISALIGNED = 4,
  LC0B200_ERR_CUDA = 5,
  LC0B200_ERR_DEVICE_TIMEOUT = 6,
  LC0B200_ERR_SCRATCH_LIMIT = 7
};

/* Activation codes (K/add_vectors.py:19-26 has none/mish/relu, K/layer_norm.py:18-25 has
 * none/mish/swish; one numbering serves both here). */
enum { LC0B200_ACT_NONE = 0, LC0B200_ACT_MISH = 1, LC0B200_ACT_RELU = 2, LC0B200_ACT_SWISH = 3 };

/* Batched-matmul operation codes, K/batched_matmul.py:19-23. */
enum { LC0B200_BMM_BODY_QK = 0, LC0B200_BMM_BODY_ATTENTION_V = 1, LC0B200_BMM_POLICY_QK = 2 };

/* GEMM element types and output kinds for lc0b200_gemm. */
enum { LC0B200_IN_BF16 = 0, LC0B200_IN_INT8 = 1 };
enum { LC0B200_OUT_BF16 = 0, LC0B200_OUT_F32 = 1, LC0B200_OUT_S32 = 2 };
/* Layout of the weight operand: [K,N] row-major as the reference stores it (ONNX
 * layout, N:1619-1639) or [N,K] row-major (pre-transposed at upload time). */
enum { LC0B200_W_KN = 0, LC0B200_W_NK = 1 };

LC0B200_API const char* lc0b200_version(void);
LC0B200_API const char* lc0b200_status_string(int status);
/* Synchronises the current device and returns LC0B200_ERR_DEVICE_TIMEOUT if any kernel on that device
 * gave up since the last call (detail_host[0..3] receives the flag words, may be NULL); clears the flag.
 * Word 0 says why: 1 = a bounded wait ran out (word 1 = which wait, word 2 = CTA), 2 = a kernel
 * found its shared-memory window not 1024-byte aligned and did nothing (word 1 = the address). */
LC0B200_API int lc0b200_device_status(unsigned int* detail_host);

/* ---- layout and element-wise ops ------------------------------------------------------ */

/* K/expand_planes.py:26-42: out[p*64+sq] = bit sq of masks[p] ? bf16(values[p]) : 0. */
LC0B200_API int lc0b200_expand_planes(void* out_bf16, const uint64_t* masks, const float* values,
                          long long plane_count, void* stream);
/* K/nchw_to_nhwc.py:26-44: first output_channels planes of [B,C,H*W] -> [B,H*W,output_channels]. */
LC0B200_API int lc0b200_nchw_to_nhwc(void* out_bf16, const void* in_bf16, int batch_size, int input_channels,
                         int output_channels, int height, int width, void* stream);
/* K/preprocess_attention_body.py:26-61: out[b,sq,:] = cat(planes[b,:,sq], encoding[b,sq,:]). */
LC0B200_API int lc0b200_preprocess_attention_body(void* out_bf16, const void* planes_bf16, const void* encoding_bf16,
                                      int batch_size, int input_channels, int encoding_channels,
                                      void* stream);
/* K/input_gating.py:26-51: out = in * mult[sq,c] + add[sq,c], gates broadcast over the batch. */
LC0B200_API int lc0b200_input_gating(void* out_bf16, const void* in_bf16, const void* mult_bf16, const void* add_bf16,
                         int batch_size, int square_count, int channel_count, void* stream);
/* K/add_vectors.py:37-66: out[i] = act(in[i] + bias[i mod bias_element_count]). */
LC0B200_API int lc0b200_add_vectors(void* out_bf16, const void* in_bf16, const void* bias_bf16, long long element_count,
                        int bias_element_count, int activation, void* stream);
/* K/add_bias_batched.py:35-66: out[bt,row,c] = act(in[bt,row,c] + bias[bt,c]). */
LC0B200_API int lc0b200_add_bias_batched(void* out_bf16, const void* in_bf16, const void* bias_bf16, int batch_count,
                             long long row_count, int channel_count, int activation, void* stream);
/* K/copy_type_converted.py:26-34: widen the final outputs to f32. */
LC0B200_API int lc0b200_copy_type_converted(float* out_f32, const void* in_bf16, long long element_count, void* stream);
/* K/policy_map.py:28-49: out[b,o] = in[b, table[o]], 0 when table[o] is out of range. */
LC0B200_API int lc0b200_policy_map(void* out_bf16, const void* in_bf16, const int32_t* table, int batch_size,
                       int input_element_count, int output_element_count, void* stream);

/* ---- dense contractions ------------------------------------------------------------------ */

/* K/matmul.py:57-116: C[m,n] = A[m,k] @ W[k,n], all row-major bf16, fp32 accumulation. */
LC0B200_API int lc0b200_matmul(void* out_bf16, const void* a_bf16, const void* w_kn_bf16, long long m, int n, int k,
                   void* stream);
/* K/fused_qkv.py:30-123: three projections sharing A, separate weights and outputs. */
LC0B200_API int lc0b200_fused_qkv_projection(void* q_bf16, void* k_bf16, void* v_bf16, const void* a_bf16,
                                 const void* wq_kn_bf16, const void* wk_kn_bf16, const void* wv_kn_bf16,
                                 long long m, int query_width, int key_width, int value_width, int k,
                                 void* stream);
/* K/fused_qkv.py:132-183: three row-broadcast bias adds in one launch (in place allowed). */
LC0B200_API int lc0b200_fused_qkv_bias(void* q_out, const void* q_in, const void* q_bias, void* k_out, const void* k_in,
                           const void* k_bias, void* v_out, const void* v_in, const void* v_bias,
                           long long row_count, int query_width, int key_width, int value_width,
                           void* stream);
/* K/batched_matmul.py:68-210.  operation BODY_QK: out[B*H,64,64] = scale * Q_h K_h^T with heads
 * interleaved in the channel dimension; POLICY_QK: out record stride 4288, contiguous operands;
 * BODY_ATTENTION_V: out[B,64,H*n] = P[b,h] @ V[b,:,h] (scale ignored, may be NULL).
 * scale points at one bf16 element on the device. */
LC0B200_API int lc0b200_batched_matmul(void* out_bf16, const void* a_bf16, const void* b_bf16, const void* scale_bf16,
                           int operation, long long batch_count, int m, int n, int k, int heads_per_sample,
                           void* stream);

/* General tensor-core GEMM with a fused epilogue (no counterpart as ONE reference kernel: it
 * stands for K/matmul.py followed by K/add_bias_batched.py / K/add_vectors.py):
 *   acc = A[m,k] @ W           (bf16 -> f32 accumulate, or int8 -> s32 accumulate)
 *   y   = acc                  (bf16 inputs)
 *       = acc * row_scale[m] * col_scale[n]   (int8 inputs; both scales f32, may be NULL = 1)
 *   out = act(y + bias[n])     (bias bf16, may be NULL), stored as bf16 / f32,
 *   or the raw s32 accumulator when out_kind == LC0B200_OUT_S32 (no scale, bias or activation).
 * lda / ldw / ldc are row pitches in elements.
 * Two projections of the same A as one product: with out_tail_bf16 set, output columns [0, n_main) go to
 * `out` (pitch ldc >= n_main) and columns [n_main, n) to out_tail_bf16 (pitch ldc_tail >= n - n_main); W, bias
 * and the ln_in vectors cover all n columns.  bf16 output only, n_main a multiple of 256, not with the residual
 * epilogue; the tensor-core kernel only (operands it cannot take are refused, not sent to the CUDA-core one).
 * A ragged last tile costs tensor-core time for its own width (rounded up to 32), not for a whole tile, so a
 * 32-wide projection rides on a 3072-wide one for about one per cent of its time. */
typedef struct lc0b200_gemm_args {
  void* out;
  const void* a;
  const void* w;
  const void* bias_bf16;
  const float* row_scale;
  const float* col_scale;
  long long m;
  int n;
  int k;
  long long lda;
  long long ldw;
  long long ldc;
  int in_type;   /* LC0B200_IN_*  */
  int out_kind;  /* LC0B200_OUT_* */
  int w_layout;  /* LC0B200_W_*   */
  int activation;
  /* ---- deferred LayerNorm (all zero = off).  The residual stream can be kept as the PRE-normalisation
   * rows z plus per-row partial sums, so that the stand-alone LayerNorm launches
   * (K/layer_norm.py:37-161, two per encoder layer) disappear:
   *   producer ("res"):  y = res_alpha * (acc + bias[n]) + skip[m,n], stored as bf16, and
   *     stats_out[part][m] = (sum, sum of squares) of the stored values over output columns
   *     [64*part, 64*part+64), part < ceil(n/64).  skip is plain bf16, or, when res_stats is given,
   *     itself deferred: skip = (z[m,n] - mean[m]) * rstd[m] * res_gamma[n] + res_beta[n] with mean /
   *     rstd from res_stats ([res_parts][m] partials over a width of n).
   *   consumer ("ln_in"): A holds deferred rows; with W' = diag(gamma) W staged as the weight,
   *     ln_in_c[n] = sum_k W'[k,n] and ln_in_d[n] = sum_k beta[k] W[k,n] + bias[n]:
   *     y = rstd[m] * (acc - mean[m] * ln_in_c[n]) + ln_in_d[n]   (bias_bf16 is ignored), then the
   *     activation.  mean / rstd come from ln_in_stats ([ln_in_parts][m] partials over a width of k).
   * Both need a bf16 output with a 16-byte aligned base and pitch and n > 64. */
  const float* ln_in_stats;
  const float* ln_in_c;
  const float* ln_in_d;
  int ln_in_parts;
  float ln_eps;
  const void* res_skip_bf16;
  long long ld_skip;
  const float* res_stats;
  const void* res_gamma_bf16;
  const void* res_beta_bf16;
  int res_parts;
  float res_alpha;
  float* stats_out;
  /* ---- second output for the trailing columns (all zero = off) */
  void* out_tail_bf16;
  long long ldc_tail;
  int n_main;
} lc0b200_gemm_args;
LC0B200_API int lc0b200_gemm(const lc0b200_gemm_args* args_host, void* stream);
/* Same contract on the plain CUDA-core kernel (any shape / alignment; used for the tiny head
 * layers and as an independent cross-check of the tensor-core kernel). */
LC0B200_API int lc0b200_gemm_simt(const lc0b200_gemm_args* args_host, void* stream);
/* Upload-time helper: dst[n,k] = src[k,n] (element_size 1 or 2). */
LC0B200_API int lc0b200_transpose(void* dst, const void* src, int rows, int cols, int element_size, void* stream);

/* ---- normalisation, softmax, attention -------------------------------------------------- */

/* K/layer_norm.py:37-161 (argument order out,in,bias,skip,gamma,beta,alpha as
 * T/test_layer_norm.py:412-415): v = act(in + bias); if has_skip v = alpha*v + skip;
 * out = (v - mean) / sqrt(var + epsilon) * gamma + beta, population variance, fp32 math.
 * alpha points at one bf16 element.  skip / alpha may be NULL when has_skip == 0.
 * If q_out_int8 and q_scale_f32 are non-NULL the normalised row (as rounded to bf16) is additionally
 * quantised per row (the multiply-by-reciprocal rule of lc0b200_quantize_rows) — no reference counterpart; out_bf16 may then be
 * NULL to store the quantised form only. */
LC0B200_API int lc0b200_layer_norm(void* out_bf16, const void* in_bf16, const void* bias_bf16, const void* skip_bf16,
                       const void* gamma_bf16, const void* beta_bf16, const void* alpha_bf16,
                       long long row_count, int width, int activation, int has_skip, float epsilon,
                       void* q_out_int8, float* q_scale_f32, void* stream);
/* K/softmax_64.py:45-71: out = softmax over 64 of clamp(qk + smolgen, +-131008), NaN kept. */
LC0B200_API int lc0b200_softmax_64(void* out_bf16, const void* scaled_qk_bf16, const void* smolgen_bf16,
                       long long row_count, void* stream);
/* Fused edge-biased attention for the 64-token board: N:1004-1047 (K/batched_matmul.py body_qk,
 * K/softmax_64.py, K/batched_matmul.py body_attention_v) in one kernel, scores never leave the SM.
 * q/k/v rows are tokens with heads interleaved in the channel dimension; ld* are row pitches in
 * elements; bias is [B, H, 64, 64] bf16 (may be NULL); depth (per-head width) must be 32.
 * Non-finite scores behave as in K/softmax_64.py (clamp, NaN kept in its row).  One deviation for
 * non-finite V: with an even head count heads 2j and 2j+1 share one 128-row tensor-core product, and
 * an Inf or NaN in V of one of them also turns the other's outputs for that position into NaN
 * (0 x Inf); the reference keeps it inside the head, as the odd-head-count kernel here does. */
LC0B200_API int lc0b200_attention(void* out_bf16, const void* q_bf16, const void* k_bf16, const void* v_bf16,
                      const void* bias_bf16, float scale, long long batch_size, int heads, int depth,
                      long long ldq, long long ldk, long long ldv, long long ldo, void* stream);
/* Symmetric per-row int8 quantisation (no reference counterpart; the reference has no int8 path):
 * scale s = max|x| / 127 (1 if the row is all zero) is what is stored, and the rounding uses ONE
 * reciprocal per row: inv = 127 / max|x| (IEEE division, fp32), q = rint(fp32(x * inv)), round-half-even,
 * saturated to [-127, 127].  This is not the same as rint(x / s) in last-bit ties; a caller that wants to
 * reproduce the bytes must use the multiply form.  (Weights, quantised once at upload, use IEEE
 * division by the per-channel scale: q = rint(w / s).) */
LC0B200_API int lc0b200_quantize_rows(void* out_int8, float* scale_f32, const void* in_bf16, long long row_count,
                          int width, long long ld_in, void* stream);
/* Rows of a deferred LayerNorm straight to per-row int8 (no reference counterpart): with mean / rstd of
 * row m from the partial sums stats[parts][row_count][2] that lc0b200_gemm wrote (stats_out) over a width
 * of `width`, y = bf16((z - mean) * rstd * gamma + beta), then quantised as lc0b200_quantize_rows does.
 * width a multiple of 8, at most 2048; pointers 16-byte aligned. */
LC0B200_API int lc0b200_normalize_quantize_rows(void* out_int8, float* scale_f32, const void* z_bf16,
                                                const float* stats, int parts, const void* gamma_bf16,
                                                const void* beta_bf16, long long row_count, int width, float epsilon,
                                                void* stream);
/* One int8 dense layer on bf16 activations (no reference counterpart): quantise the rows of a
 * (lc0b200_quantize_rows) into caller-provided scratch, then out = act(dequant(Aq @ Wq) + bias)
 * (lc0b200_gemm with int8 inputs).  w_nk_int8 is [n,k] row-major, col_scale the per-output-channel
 * weight scales.  scratch_q holds m*k bytes, scratch_scale m floats; both must be 16-byte aligned
 * and may be reused as soon as the call's kernels have run. */
LC0B200_API int lc0b200_linear_int8(void* out_bf16, const void* a_bf16, const void* w_nk_int8, const float* col_scale,
                        const void* bias_bf16, void* scratch_q, float* scratch_scale, long long m, int n, int k,
                        int activation, void* stream);

/* The same layer for callers that cannot allocate device memory at all (no counterpart in the
 * reference, whose kernels never need temporaries).  Think of an executor that runs a buffer plan
 * fixed at link time, or a search thread that must not call cudaMalloc because it stalls the whole
 * device: they pass only the input, the weights and the output, and the quantised activations and
 * row scales live in an array that is part of the library image.
 *  - Limits: m <= LC0B200_STATIC_MAX_ROWS and m * k <= LC0B200_STATIC_MAX_ACT_BYTES; anything larger
 *    is refused with LC0B200_ERR_SCRATCH_LIMIT and nothing is launched.  Every GPU that loads the
 *    library holds the array (about 8.06 MiB) until the process exits.
 *  - The first call on each device looks up the array's device address (no allocation); make that
 *    first call before any stream capture begins on that device.
 *  - All calls share the one array and it keeps what the last call wrote.  Nothing in it needs
 *    clearing between calls, but two calls whose kernels overlap on the GPU (different streams,
 *    or different host threads on the same device) race on it: keep them on one stream.
 *  - No cudaMalloc, cudaFree or other allocating routine is called, here or below. */
#define LC0B200_STATIC_MAX_ROWS 16384
#define LC0B200_STATIC_MAX_ACT_BYTES (8 * 1024 * 1024)
LC0B200_API int lc0b200_linear_int8_static(void* out_bf16, const void* a_bf16, const void* w_nk_int8,
                               const float* col_scale, const void* bias_bf16, long long m, int n, int k,
                               int activation, void* stream);

/* ---- heads -------------------------------------------------------------------------------- */

/* K/promotion_logits.py:67-145 (argument order records,keys,weights as the reference ABI):
 * records[b,4096+s*24+t*3+c] = records[b,(48+s)*64+56+t] + keys[b,56+t,:].(W[:,c] + W[:,3]). */
LC0B200_API int lc0b200_promotion_logits(void* records_bf16, const void* keys_bf16, const void* w_bf16, int batch_size,
                             int width, void* stream);
/* Input embedding front end, N:458-533 in two kernels instead of four:
 * pos_in[b, sq*12 + c] = plane c of position b at square sq (c < 12)           (k1+k2)
 * emb_in[b*64+sq, :]   = cat(112 plane values at sq, position[b, sq, :E])      (k1+k3) */
LC0B200_API int lc0b200_embed_position_input(void* pos_in_bf16, const uint64_t* masks, const float* values,
                                 int batch_size, void* stream);
LC0B200_API int lc0b200_embed_concat(void* emb_in_bf16, const uint64_t* masks, const float* values,
                         const void* position_bf16, int batch_size, int encoding_channels, void* stream);
/* Policy tail, N:1307-1356 in one kernel: promotion logits + gather + f32 store.
 * out[b,o] = f32(record value at table[o]) where record slots >= 4096 are computed on the fly. */
LC0B200_API int lc0b200_policy_tail(float* out_f32, const void* records_bf16, const void* keys_bf16, const void* w_bf16,
                        const int32_t* table, int batch_size, int width, void* stream);

/* The step right after the path in lc0 (BT4_PLAN.md:42-43: the graph emits raw WDL logits and the
 * runtime applies the softmax on the host): wdl_probs = softmax(wdl_logits) over 3, policy_probs =
 * softmax of the policy logits over the legal moves only (legal_mask[b,o] != 0; NULL = all legal;
 * illegal entries get 0; a position without legal moves gets all zeros), and the search's value pair
 * (BT4_PLAN.md:753 "Host WDL softmax and Q/D conversion"): q_d[b] = (Q, D) = (W - L, D) of those
 * probabilities, Q in [-1, 1] from the side to move.  Any output may be NULL, but not all three. */
LC0B200_API int lc0b200_output_probabilities(float* policy_probs, float* wdl_probs, float* q_d,
                                 const float* policy_logits, const float* wdl_logits, const uint8_t* legal_mask,
                                 int batch_size, int policy_size, void* stream);

/* ---- the whole forward pass as one object -------------------------------------------------
 *
 * What an engine written in C or C++ binds instead of the per-operator entry points: the role of the
 * reference's runtime (LC0EX_BACKEND_BENCHMARK.md:125-139: persistent buffers kept by name, one kernel
 * launch per graph node) for the graph of N:343-1550.  Shapes are the reference's layer sizes; weights
 * go in under the reference's canonical buffer names (every `name=` of N:343-1466, e.g.
 * "/encoder0/mha/Q/w/w") as bf16 in its input-major [K,N] layout, one-element constants
 * ("/encoder0/alpha*input/w", "/policy/scale/w", ...) included.  bf16 arithmetic with the encoder
 * LayerNorms folded into the GEMM epilogues, or int8 GEMMs (config.int8_gemms).  head depth
 * (embedding / heads) must be 32.
 *
 * All device memory is ONE caller-provided arena of lc0b200_net_arena_bytes() bytes (256-byte aligned):
 * weights as uploaded, the operands derived from them and the workspace for max_batch positions.
 * create / destroy allocate and free only a small host structure.  set_weight copies host memory to the
 * arena on `stream`; finalize derives the GEMM operands (transposes, LayerNorm folding) and synchronises
 * `stream` once; forward only launches (about 170 kernels at 15 layers) and neither allocates nor
 * synchronises, so it can be captured into a CUDA graph.  One forward at a time per network object. */
typedef struct lc0b200_net lc0b200_net;
typedef struct lc0b200_net_config {
  int embedding, layers, heads, ffn;
  int pos_enc;                                        /* positional-encoding channels per square */
  int smolgen_compress, smolgen_hidden, smolgen_gen;  /* channels per token, dense1 width, per-head width */
  int policy, policy_model;                           /* policy embedding and query/key widths */
  int value_embed, value_hidden, mlh_embed, mlh_hidden;
  float ln_eps;
  int int8_gemms;  /* 0: bf16 throughout.  1: QKV, attention output and both FFN GEMMs of every encoder layer on
                    * int8 operands (per-channel weight scales, per-token activation scales, s32 accumulation;
                    * weights are quantised on the device in finalize) - no reference counterpart */
} lc0b200_net_config;
LC0B200_API size_t lc0b200_net_arena_bytes(const lc0b200_net_config* config, int max_batch); /* 0 = bad config */
LC0B200_API int lc0b200_net_create(lc0b200_net** out, const lc0b200_net_config* config, int max_batch,
                                   void* device_arena, size_t arena_bytes);
LC0B200_API void lc0b200_net_destroy(lc0b200_net* net);
/* The buffers the network expects: index < lc0b200_net_weight_count(); *name stays valid while net lives. */
LC0B200_API int lc0b200_net_weight_count(const lc0b200_net* net);
LC0B200_API int lc0b200_net_weight_info(const lc0b200_net* net, int index, const char** name, long long* elements);
/* LC0B200_ERR_UNSUPPORTED: no such buffer; LC0B200_ERR_BAD_SHAPE: wrong element count. */
LC0B200_API int lc0b200_net_set_weight(lc0b200_net* net, const char* name, const void* host_bf16, long long elements,
                                       void* stream);
/* LC0B200_ERR_NULL_POINTER while any buffer is still missing. */
LC0B200_API int lc0b200_net_finalize(lc0b200_net* net, void* stream);
/* masks u64[batch,112], values f32[batch,112] (N:328-340) -> policy f32[batch,1858], raw WDL logits
 * f32[batch,3], moves left f32[batch,1]; all device pointers; batch <= max_batch. */
LC0B200_API int lc0b200_net_forward(lc0b200_net* net, const uint64_t* masks, const float* values, int batch,
                                    float* policy_f32, float* wdl_f32, float* mlh_f32, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* LC0B200_H_ */
