// Internal: host launchers of the non-GEMM kernels (validated arguments only; the C ABI in
// api.cu does the checking).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace lc0b200 {

// elementwise.cu
int expand_planes(void* out, const uint64_t* masks, const float* values, long long plane_count, cudaStream_t st);
int nchw_to_nhwc(void* out, const void* in, int batch, int in_ch, int out_ch, int hw, cudaStream_t st);
int preprocess_attention_body(void* out, const void* planes, const void* enc, int batch, int in_ch, int enc_ch,
                              cudaStream_t st);
int input_gating(void* out, const void* in, const void* mult, const void* add, int batch, int squares, int channels,
                 cudaStream_t st);
int add_bias(void* out, const void* in, const void* bias, long long total, int channels, long long per_batch,
             int activation, cudaStream_t st);
int fused_qkv_bias(void* const out[3], const void* const in[3], const void* const bias[3], const int width[3],
                   long long rows, cudaStream_t st);
int widen(float* out, const void* in, long long total, cudaStream_t st);
int policy_map(void* out, const void* in, const int32_t* table, int batch, int in_count, int out_count,
               cudaStream_t st);
int transpose(void* dst, const void* src, int rows, int cols, int element_size, cudaStream_t st);
int embed_position_input(void* out, const uint64_t* masks, const float* values, int batch, cudaStream_t st);
int embed_concat(void* out, const uint64_t* masks, const float* values, const void* position, int batch, int enc,
                 cudaStream_t st);
int quantize_rows(void* out, float* scale, const void* in, long long rows, int width, long long ld_in,
                  cudaStream_t st);

// api.cu: quantise rows into scratch, then the int8 GEMM with the dequantising epilogue.
int linear_int8(void* out, const void* a, const void* w_nk, const float* col_scale, const void* bias,
                void* scratch_q, float* scratch_scale, long long m, int n, int k, int activation,
                cudaStream_t stream);

// layernorm.cu
int normalize_quantize_rows(void* q_out, float* q_scale, const void* z, const float* stats, int parts, const void* gamma,
                            const void* beta, long long rows, int width, float epsilon, cudaStream_t st);
int layer_norm(void* out, const void* in, const void* bias, const void* skip, const void* gamma, const void* beta,
               const void* alpha, long long rows, int width, int activation, int has_skip, float epsilon,
               void* q_out, float* q_scale, cudaStream_t st);

// attention.cu
int softmax_64(void* out, const void* qk, const void* smolgen, long long rows, cudaStream_t st);
int attention(void* out, const void* q, const void* k, const void* v, const void* bias, float scale,
              long long batch, int heads, long long ldq, long long ldk, long long ldv, long long ldo,
              cudaStream_t st);
int batched_matmul(void* out, const void* a, const void* b, const void* scale, int operation, long long batch_count,
                   int m, int n, int k, int heads, cudaStream_t st);

// attention_tc.cu: the same operator on tcgen05 / TMEM (pairs of heads; needs an even head count)
bool attention_tc_supported(const void* out, const void* q, const void* k, const void* v, const void* bias,
                            long long batch, int heads, long long ldq, long long ldk, long long ldv, long long ldo);
int attention_tc(void* out, const void* q, const void* k, const void* v, const void* bias, float scale,
                 long long batch, int heads, long long ldq, long long ldk, long long ldv, long long ldo,
                 cudaStream_t st);

// policy.cu
int promotion_logits(void* records, const void* keys, const void* w, int batch, int width, cudaStream_t st);
int output_probabilities(float* policy_probs, float* wdl_probs, float* q_d, const float* policy_logits,
                         const float* wdl_logits,
                         const uint8_t* legal, int batch, int policy_size, cudaStream_t st);
int policy_tail(float* out, const void* records, const void* keys, const void* w, const int32_t* table, int batch,
                int width, cudaStream_t st);

}  // namespace lc0b200
