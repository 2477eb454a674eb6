// extern "C" entry points: argument validation, then dispatch to the kernel launchers.
// Nothing here allocates, synchronises (except lc0b200_device_status) or throws.
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>

#include "common.cuh"
#include "gemm.h"
#include "kernels.h"

namespace lc0b200 {

static __device__ unsigned int g_device_status[4] = {0u, 0u, 0u, 0u};

namespace {
std::mutex g_device_mutex;
DeviceInfo g_device_info[kMaxDevices];
std::atomic<bool> g_device_known[kMaxDevices];
}  // namespace

// In host code `g_device_status` is a handle, not an address: the address a kernel can use differs
// from device to device and is asked for once per device, with that device current.
const DeviceInfo* device_info() {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return nullptr;
  if (g_device_known[device].load(std::memory_order_acquire)) return &g_device_info[device];
  std::lock_guard<std::mutex> lock(g_device_mutex);
  if (!g_device_known[device].load(std::memory_order_relaxed)) {
    void* status = nullptr;
    int sms = 0;
    if (cudaGetSymbolAddress(&status, g_device_status) != cudaSuccess || status == nullptr) return nullptr;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) return nullptr;
    g_device_info[device].index = device;
    g_device_info[device].sm_count = sms;
    g_device_info[device].status = static_cast<unsigned int*>(status);
    g_device_known[device].store(true, std::memory_order_release);
  }
  return &g_device_info[device];
}

}  // namespace lc0b200

namespace lc0b200 {

int linear_int8(void* out, const void* a, const void* w_nk, const float* col_scale, const void* bias,
                void* scratch_q, float* scratch_scale, long long m, int n, int k, int activation,
                cudaStream_t stream) {
  int st = quantize_rows(scratch_q, scratch_scale, a, m, k, k, stream);
  if (st != LC0B200_OK) return st;
  lc0b200_gemm_args g = {};
  g.out = out; g.a = scratch_q; g.w = w_nk; g.bias_bf16 = bias;
  g.row_scale = scratch_scale; g.col_scale = col_scale;
  g.m = m; g.n = n; g.k = k;
  g.lda = k; g.ldw = k; g.ldc = n;
  g.in_type = LC0B200_IN_INT8; g.out_kind = LC0B200_OUT_BF16; g.w_layout = LC0B200_W_NK;
  g.activation = activation;
  return gemm_tcgen05_supported(g) ? gemm_tcgen05(g, stream) : gemm_simt(g, stream);
}

}  // namespace lc0b200

using namespace lc0b200;

#define REQUIRE_PTR(p) \
  do {                 \
    if ((p) == nullptr) return LC0B200_ERR_NULL_POINTER; \
  } while (0)
#define REQUIRE_SHAPE(cond) \
  do {                      \
    if (!(cond)) return LC0B200_ERR_BAD_SHAPE; \
  } while (0)
#define REQUIRE_ALIGNED(p, bytes) \
  do {                            \
    if ((reinterpret_cast<uintptr_t>(p) % (bytes)) != 0) return LC0B200_ERR_MISALIGNED; \
  } while (0)

static inline cudaStream_t S(void* stream) { return reinterpret_cast<cudaStream_t>(stream); }

static bool valid_activation(int a) { return a >= LC0B200_ACT_NONE && a <= LC0B200_ACT_SWISH; }

extern "C" {

LC0B200_API const char* lc0b200_version(void) { return "lc0b200 0.1 (sm_100a)"; }

LC0B200_API const char* lc0b200_status_string(int status) {
  switch (status) {
    case LC0B200_OK: return "ok";
    case LC0B200_ERR_NULL_POINTER: return "null pointer";
    case LC0B200_ERR_BAD_SHAPE: return "bad shape";
    case LC0B200_ERR_UNSUPPORTED: return "unsupported configuration";
    case LC0B200_ERR_MISALIGNED: return "misaligned pointer or pitch";
    case LC0B200_ERR_CUDA: return "CUDA error";
    case LC0B200_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
    case LC0B200_ERR_SCRATCH_LIMIT: return "problem exceeds the built-in scratch array";
    default: return "unknown status";
  }
}

LC0B200_API int lc0b200_device_status(unsigned int* detail_host) {
  if (cudaDeviceSynchronize() != cudaSuccess) return LC0B200_ERR_CUDA;
  unsigned int words[4] = {0u, 0u, 0u, 0u};
  if (cudaMemcpyFromSymbol(words, g_device_status, sizeof(words)) != cudaSuccess) return LC0B200_ERR_CUDA;
  if (detail_host != nullptr) {
    for (int i = 0; i < 4; ++i) detail_host[i] = words[i];
  }
  if (words[0] != 0u) {
    const unsigned int zero[4] = {0u, 0u, 0u, 0u};
    if (cudaMemcpyToSymbol(g_device_status, zero, sizeof(zero)) != cudaSuccess) return LC0B200_ERR_CUDA;
    return LC0B200_ERR_DEVICE_TIMEOUT;
  }
  return LC0B200_OK;
}

LC0B200_API int lc0b200_expand_planes(void* out, const uint64_t* masks, const float* values, long long plane_count,
                          void* stream) {
  REQUIRE_PTR(out); REQUIRE_PTR(masks); REQUIRE_PTR(values);
  REQUIRE_SHAPE(plane_count >= 0);
  if (plane_count == 0) return LC0B200_OK;
  return expand_planes(out, masks, values, plane_count, S(stream));
}

LC0B200_API int lc0b200_nchw_to_nhwc(void* out, const void* in, int batch_size, int input_channels, int output_channels,
                         int height, int width, void* stream) {
  REQUIRE_PTR(out); REQUIRE_PTR(in);
  REQUIRE_SHAPE(batch_size >= 0 && input_channels > 0 && output_channels > 0 && output_channels <= input_channels &&
                height > 0 && width > 0);
  if (batch_size == 0) return LC0B200_OK;
  return nchw_to_nhwc(out, in, batch_size, input_channels, output_channels, height * width, S(stream));
}

LC0B200_API int lc0b200_preprocess_attention_body(void* out, const void* planes, const void* encoding, int batch_size,
                                      int input_channels, int encoding_channels, void* stream) {
  REQUIRE_PTR(out); REQUIRE_PTR(planes); REQUIRE_PTR(encoding);
  REQUIRE_SHAPE(batch_size >= 0 && input_channels > 0 && encoding_channels >= 0);
  if (batch_size == 0) return LC0B200_OK;
  return preprocess_attention_body(out, planes, encoding, batch_size, input_channels, encoding_channels, S(stream));
}

LC0B200_API int lc0b200_input_gating(void* out, const void* in, const void* mult, const void* add, int batch_size,
                         int square_count, int channel_count, void* stream) {
  REQUIRE_PTR(out); REQUIRE_PTR(in); REQUIRE_PTR(mult); REQUIRE_PTR(add);
  REQUIRE_SHAPE(batch_size >= 0 && square_count > 0 && channel_count > 0);
  if (batch_size == 0) return LC0B200_OK;
  return input_gating(out, in, mult, add, batch_size, square_count, channel_count, S(stream));
}

LC0B200_API int lc0b200_add_vectors(void* out, const void* in, const void* bias, long long element_count, int bias_element_count,
                        int activation, void* stream) {
  REQUIRE_PTR(out); REQUIRE_PTR(in); REQUIRE_PTR(bias);
  REQUIRE_SHAPE(element_count >= 0 && bias_element_count > 0 && valid_activation(activation) &&
                activation != LC0B200_ACT_SWISH);
  if (element_count == 0) return LC0B200_OK;
  // One "batch" covering everything: bias index is i mod bias_element_count.
  return add_bias(out, in, bias, element_count, bias_element_count, element_count, activation, S(stream));
}

LC0B200_API int lc0b200_add_bias_batched(void* out, const void* in, const void* bias, int batch_count, long long row_count,
                             int channel_count, int activation, void* stream) {
  REQUIRE_PTR(out); REQUIRE_PTR(in); REQUIRE_PTR(bias);
  REQUIRE_SHAPE(batch_count >= 0 && row_count >= 0 && channel_count > 0 &&
                (activation == LC0B200_ACT_NONE || activation == LC0B200_ACT_MISH));
  const long long per_batch = row_count * channel_count;
  if (batch_count == 0 || per_batch == 0) return LC0B200_OK;
  return add_bias(out, in, bias, per_batch * batch_count, channel_count, per_batch, activation, S(stream));
}

LC0B200_API int lc0b200_copy_type_converted(float* out, const void* in, long long element_count, void* stream) {
  REQUIRE_PTR(out); REQUIRE_PTR(in);
  REQUIRE_SHAPE(element_count >= 0);
  if (element_count == 0) return LC0B200_OK;
  return widen(out, in, element_count, S(stream));
}

LC0B200_API int lc0b200_policy_map(void* out, const void* in, const int32_t* table, int batch_size, int input_element_count,
                       int output_element_count, void* stream) {
  REQUIRE_PTR(out); REQUIRE_PTR(in); REQUIRE_PTR(table);
  REQUIRE_SHAPE(batch_size >= 0 && input_element_count > 0 && output_element_count > 0);
  if (batch_size == 0) return LC0B200_OK;
  return policy_map(out, in, table, batch_size, input_element_count, output_element_count, S(stream));
}

static int check_gemm(const lc0b200_gemm_args* g) {
  REQUIRE_PTR(g);
  REQUIRE_PTR(g->out); REQUIRE_PTR(g->a); REQUIRE_PTR(g->w);
  REQUIRE_SHAPE(g->m >= 0 && g->n > 0 && g->k > 0);
  const bool has_tail = g->out_tail_bf16 != nullptr;
  if (has_tail) {
    REQUIRE_SHAPE(g->n_main > 0 && g->n_main < g->n && g->n_main % 256 == 0 && g->ldc_tail >= g->n - g->n_main);
    if (g->out_kind != LC0B200_OUT_BF16 || g->res_skip_bf16 != nullptr || g->stats_out != nullptr) return LC0B200_ERR_UNSUPPORTED;
  }
  REQUIRE_SHAPE(g->lda >= g->k && g->ldc >= (has_tail ? g->n_main : g->n));
  REQUIRE_SHAPE(g->ldw >= (g->w_layout == LC0B200_W_KN ? g->n : g->k));
  if (g->in_type != LC0B200_IN_BF16 && g->in_type != LC0B200_IN_INT8) return LC0B200_ERR_UNSUPPORTED;
  if (g->out_kind < LC0B200_OUT_BF16 || g->out_kind > LC0B200_OUT_S32) return LC0B200_ERR_UNSUPPORTED;
  if (g->w_layout != LC0B200_W_KN && g->w_layout != LC0B200_W_NK) return LC0B200_ERR_UNSUPPORTED;
  if (!valid_activation(g->activation)) return LC0B200_ERR_UNSUPPORTED;
  if (g->out_kind == LC0B200_OUT_S32 && g->in_type != LC0B200_IN_INT8) return LC0B200_ERR_UNSUPPORTED;
  if (g->ln_in_stats != nullptr) {
    REQUIRE_PTR(g->ln_in_c); REQUIRE_PTR(g->ln_in_d);
    REQUIRE_SHAPE(g->ln_in_parts > 0);
  }
  if (g->res_stats != nullptr) {
    REQUIRE_PTR(g->res_skip_bf16); REQUIRE_PTR(g->res_gamma_bf16); REQUIRE_PTR(g->res_beta_bf16);
    REQUIRE_SHAPE(g->res_parts > 0);
  }
  if (g->res_skip_bf16 != nullptr) REQUIRE_SHAPE(g->ld_skip >= g->n);
  return LC0B200_OK;
}

static bool has_deferred_layer_norm(const lc0b200_gemm_args* g) {
  return g->ln_in_stats != nullptr || g->res_skip_bf16 != nullptr || g->stats_out != nullptr;
}

LC0B200_API int lc0b200_gemm(const lc0b200_gemm_args* g, void* stream) {
  const int st = check_gemm(g);
  if (st != LC0B200_OK) return st;
  if (g->m == 0) return LC0B200_OK;
  if (gemm_tcgen05_supported(*g)) return gemm_tcgen05(*g, S(stream));
  if (has_deferred_layer_norm(g) || g->out_tail_bf16 != nullptr) return LC0B200_ERR_UNSUPPORTED;
  return gemm_simt(*g, S(stream));
}

LC0B200_API int lc0b200_gemm_simt(const lc0b200_gemm_args* g, void* stream) {
  const int st = check_gemm(g);
  if (st != LC0B200_OK) return st;
  if (g->m == 0) return LC0B200_OK;
  if (has_deferred_layer_norm(g) || g->out_tail_bf16 != nullptr) return LC0B200_ERR_UNSUPPORTED;
  return gemm_simt(*g, S(stream));
}

LC0B200_API int lc0b200_matmul(void* out, const void* a, const void* w, long long m, int n, int k, void* stream) {
  lc0b200_gemm_args g = {};
  g.out = out; g.a = a; g.w = w;
  g.m = m; g.n = n; g.k = k;
  g.lda = k; g.ldw = n; g.ldc = n;
  g.in_type = LC0B200_IN_BF16; g.out_kind = LC0B200_OUT_BF16; g.w_layout = LC0B200_W_KN;
  g.activation = LC0B200_ACT_NONE;
  return lc0b200_gemm(&g, stream);
}

LC0B200_API int lc0b200_fused_qkv_projection(void* q, void* k_out, void* v, const void* a, const void* wq, const void* wk,
                                 const void* wv, long long m, int query_width, int key_width, int value_width,
                                 int k, void* stream) {
  int st = lc0b200_matmul(q, a, wq, m, query_width, k, stream);
  if (st != LC0B200_OK) return st;
  st = lc0b200_matmul(k_out, a, wk, m, key_width, k, stream);
  if (st != LC0B200_OK) return st;
  return lc0b200_matmul(v, a, wv, m, value_width, k, stream);
}

LC0B200_API int lc0b200_fused_qkv_bias(void* q_out, const void* q_in, const void* q_bias, void* k_out, const void* k_in,
                           const void* k_bias, void* v_out, const void* v_in, const void* v_bias, long long row_count,
                           int query_width, int key_width, int value_width, void* stream) {
  REQUIRE_PTR(q_out); REQUIRE_PTR(q_in); REQUIRE_PTR(q_bias);
  REQUIRE_PTR(k_out); REQUIRE_PTR(k_in); REQUIRE_PTR(k_bias);
  REQUIRE_PTR(v_out); REQUIRE_PTR(v_in); REQUIRE_PTR(v_bias);
  REQUIRE_SHAPE(row_count >= 0 && query_width > 0 && key_width > 0 && value_width > 0);
  if (row_count == 0) return LC0B200_OK;
  void* const out[3] = {q_out, k_out, v_out};
  const void* const in[3] = {q_in, k_in, v_in};
  const void* const bias[3] = {q_bias, k_bias, v_bias};
  const int width[3] = {query_width, key_width, value_width};
  return fused_qkv_bias(out, in, bias, width, row_count, S(stream));
}

LC0B200_API int lc0b200_batched_matmul(void* out, const void* a, const void* b, const void* scale, int operation,
                           long long batch_count, int m, int n, int k, int heads_per_sample, void* stream) {
  REQUIRE_PTR(out); REQUIRE_PTR(a); REQUIRE_PTR(b);
  if (operation < LC0B200_BMM_BODY_QK || operation > LC0B200_BMM_POLICY_QK) return LC0B200_ERR_UNSUPPORTED;
  if (operation != LC0B200_BMM_BODY_ATTENTION_V) REQUIRE_PTR(scale);
  REQUIRE_SHAPE(batch_count >= 0 && m > 0 && n > 0 && k > 0 && heads_per_sample > 0);
  REQUIRE_SHAPE(batch_count % heads_per_sample == 0);
  if (operation == LC0B200_BMM_POLICY_QK) REQUIRE_SHAPE(m * n <= 4288);
  if (batch_count == 0) return LC0B200_OK;
  return batched_matmul(out, a, b, scale, operation, batch_count, m, n, k, heads_per_sample, S(stream));
}

LC0B200_API int lc0b200_transpose(void* dst, const void* src, int rows, int cols, int element_size, void* stream) {
  REQUIRE_PTR(dst); REQUIRE_PTR(src);
  REQUIRE_SHAPE(rows > 0 && cols > 0);
  if (element_size != 1 && element_size != 2) return LC0B200_ERR_UNSUPPORTED;
  return transpose(dst, src, rows, cols, element_size, S(stream));
}

LC0B200_API int lc0b200_layer_norm(void* out, const void* in, const void* bias, const void* skip, const void* gamma,
                       const void* beta, const void* alpha, long long row_count, int width, int activation,
                       int has_skip, float epsilon, void* q_out, float* q_scale, void* stream) {
  REQUIRE_PTR(in); REQUIRE_PTR(bias); REQUIRE_PTR(gamma); REQUIRE_PTR(beta);
  if (has_skip) { REQUIRE_PTR(skip); REQUIRE_PTR(alpha); }
  if ((q_out == nullptr) != (q_scale == nullptr)) return LC0B200_ERR_NULL_POINTER;
  if (out == nullptr && q_out == nullptr) return LC0B200_ERR_NULL_POINTER;  // out may be NULL only with q_out
  REQUIRE_SHAPE(row_count >= 0 && row_count <= 0x7FFFFFFFLL && width > 0 && epsilon >= 0.0f);
  if (activation != LC0B200_ACT_NONE && activation != LC0B200_ACT_MISH && activation != LC0B200_ACT_SWISH) {
    return LC0B200_ERR_UNSUPPORTED;
  }
  if (row_count == 0) return LC0B200_OK;
  return layer_norm(out, in, bias, skip, gamma, beta, alpha, row_count, width, activation, has_skip ? 1 : 0, epsilon,
                    q_out, q_scale, S(stream));
}

LC0B200_API int lc0b200_softmax_64(void* out, const void* qk, const void* smolgen, long long row_count, void* stream) {
  REQUIRE_PTR(out); REQUIRE_PTR(qk); REQUIRE_PTR(smolgen);
  REQUIRE_SHAPE(row_count >= 0 && row_count <= 8LL * 0x7FFFFFFF);
  REQUIRE_ALIGNED(out, 4); REQUIRE_ALIGNED(qk, 4); REQUIRE_ALIGNED(smolgen, 4);
  if (row_count == 0) return LC0B200_OK;
  return softmax_64(out, qk, smolgen, row_count, S(stream));
}

LC0B200_API int lc0b200_attention(void* out, const void* q, const void* k, const void* v, const void* bias, float scale,
                      long long batch_size, int heads, int depth, long long ldq, long long ldk, long long ldv,
                      long long ldo, void* stream) {
  REQUIRE_PTR(out); REQUIRE_PTR(q); REQUIRE_PTR(k); REQUIRE_PTR(v);
  REQUIRE_SHAPE(batch_size >= 0 && heads > 0);
  if (depth != 32) return LC0B200_ERR_UNSUPPORTED;
  const long long width = static_cast<long long>(heads) * depth;
  REQUIRE_SHAPE(ldq >= width && ldk >= width && ldv >= width && ldo >= width);
  REQUIRE_ALIGNED(out, 16); REQUIRE_ALIGNED(q, 16); REQUIRE_ALIGNED(k, 16); REQUIRE_ALIGNED(v, 16);
  if (bias != nullptr) REQUIRE_ALIGNED(bias, 16);
  if ((ldq | ldk | ldv | ldo) % 8 != 0) return LC0B200_ERR_MISALIGNED;
  if (batch_size == 0) return LC0B200_OK;
  return attention(out, q, k, v, bias, scale, batch_size, heads, ldq, ldk, ldv, ldo, S(stream));
}

LC0B200_API int lc0b200_quantize_rows(void* out, float* scale, const void* in, long long row_count, int width, long long ld_in,
                          void* stream) {
  REQUIRE_PTR(out); REQUIRE_PTR(scale); REQUIRE_PTR(in);
  REQUIRE_SHAPE(row_count >= 0 && width > 0 && ld_in >= width && row_count <= 8LL * 0x7FFFFFFF);
  if (row_count == 0) return LC0B200_OK;
  return quantize_rows(out, scale, in, row_count, width, ld_in, S(stream));
}

LC0B200_API int lc0b200_normalize_quantize_rows(void* out, float* scale, const void* z, const float* stats, int parts,
                                                const void* gamma, const void* beta, long long row_count, int width,
                                                float epsilon, void* stream) {
  REQUIRE_PTR(out); REQUIRE_PTR(scale); REQUIRE_PTR(z); REQUIRE_PTR(stats); REQUIRE_PTR(gamma); REQUIRE_PTR(beta);
  REQUIRE_SHAPE(row_count >= 0 && width > 0 && parts > 0 && epsilon > 0.0f && row_count <= 0x7FFFFFFFLL);
  return normalize_quantize_rows(out, scale, z, stats, parts, gamma, beta, row_count, width, epsilon, S(stream));
}

LC0B200_API int lc0b200_linear_int8(void* out, const void* a, const void* w_nk, const float* col_scale,
                                    const void* bias, void* scratch_q, float* scratch_scale, long long m, int n,
                                    int k, int activation, void* stream) {
  REQUIRE_PTR(out); REQUIRE_PTR(a); REQUIRE_PTR(w_nk); REQUIRE_PTR(col_scale);
  REQUIRE_PTR(scratch_q); REQUIRE_PTR(scratch_scale);
  REQUIRE_SHAPE(m >= 0 && n > 0 && k > 0 && m <= 8LL * 0x7FFFFFFF);
  REQUIRE_ALIGNED(scratch_q, 16); REQUIRE_ALIGNED(scratch_scale, 16);
  if (!valid_activation(activation)) return LC0B200_ERR_UNSUPPORTED;
  if (m == 0) return LC0B200_OK;
  return linear_int8(out, a, w_nk, col_scale, bias, scratch_q, scratch_scale, m, n, k, activation, S(stream));
}

LC0B200_API int lc0b200_promotion_logits(void* records, const void* keys, const void* w, int batch_size, int width,
                             void* stream) {
  REQUIRE_PTR(records); REQUIRE_PTR(keys); REQUIRE_PTR(w);
  REQUIRE_SHAPE(batch_size >= 0 && width > 0);
  if (batch_size == 0) return LC0B200_OK;
  return promotion_logits(records, keys, w, batch_size, width, S(stream));
}

LC0B200_API int lc0b200_embed_position_input(void* pos_in, const uint64_t* masks, const float* values, int batch_size,
                                 void* stream) {
  REQUIRE_PTR(pos_in); REQUIRE_PTR(masks); REQUIRE_PTR(values);
  REQUIRE_SHAPE(batch_size >= 0);
  if (batch_size == 0) return LC0B200_OK;
  return embed_position_input(pos_in, masks, values, batch_size, S(stream));
}

LC0B200_API int lc0b200_embed_concat(void* emb_in, const uint64_t* masks, const float* values, const void* position,
                         int batch_size, int encoding_channels, void* stream) {
  REQUIRE_PTR(emb_in); REQUIRE_PTR(masks); REQUIRE_PTR(values); REQUIRE_PTR(position);
  REQUIRE_SHAPE(batch_size >= 0 && encoding_channels >= 0);
  if (encoding_channels % 8 == 0) { REQUIRE_ALIGNED(emb_in, 16); REQUIRE_ALIGNED(position, 16); }
  if (batch_size == 0) return LC0B200_OK;
  return embed_concat(emb_in, masks, values, position, batch_size, encoding_channels, S(stream));
}

LC0B200_API int lc0b200_policy_tail(float* out, const void* records, const void* keys, const void* w, const int32_t* table,
                        int batch_size, int width, void* stream) {
  REQUIRE_PTR(out); REQUIRE_PTR(records); REQUIRE_PTR(keys); REQUIRE_PTR(w); REQUIRE_PTR(table);
  REQUIRE_SHAPE(batch_size >= 0 && width > 0);
  if (batch_size == 0) return LC0B200_OK;
  return policy_tail(out, records, keys, w, table, batch_size, width, S(stream));
}

LC0B200_API int lc0b200_output_probabilities(float* policy_probs, float* wdl_probs, float* q_d,
                                             const float* policy_logits, const float* wdl_logits,
                                             const uint8_t* legal_mask, int batch_size, int policy_size, void* stream) {
  if (policy_probs == nullptr && wdl_probs == nullptr && q_d == nullptr) return LC0B200_ERR_NULL_POINTER;
  if (policy_probs != nullptr) REQUIRE_PTR(policy_logits);
  if (wdl_probs != nullptr || q_d != nullptr) REQUIRE_PTR(wdl_logits);
  REQUIRE_SHAPE(batch_size >= 0 && policy_size > 0);
  if (batch_size == 0) return LC0B200_OK;
  return output_probabilities(policy_probs, wdl_probs, q_d, policy_logits, wdl_logits, legal_mask, batch_size,
                              policy_size, S(stream));
}

}  // extern "C"
