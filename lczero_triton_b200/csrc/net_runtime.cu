// The whole forward pass behind the C ABI: a network object that owns nothing but a plan.
//
// The reference's runtime (an lc0 backend written in C++) keeps persistent buffers by name, uploads
// the weights under the graph's canonical names and then launches the graph's kernels in order
// (LC0EX_BACKEND_BENCHMARK.md:125-139; names and [K,N] shapes: bt4/network.py:343-1466).  This file
// gives a C or C++ engine the same thing without Python: create a network for a shape, hand over the
// weights by name, finalise (transposes, LayerNorm folding), then call forward on device-resident
// packed planes.  All device memory is one caller-provided arena; the object itself is a small host
// structure.  The operator order is that of bt4/network.py (embedding :458-642, smolgen :778-849,
// attention :1004-1076, FFN :1089-1186, policy :1261-1356, value / moves-left :1475-1550) with the
// encoder LayerNorms deferred into the GEMM epilogues (see lc0b200_gemm_args) in bf16 mode, or with the four
// large GEMMs of every encoder layer on int8 operands and stand-alone LayerNorm kernels that also emit the
// quantised rows (config.int8_gemms; no reference counterpart for that mode).
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <new>
#include <string>
#include <vector>

#include "../../include/lc0b200.h"
#include "common.cuh"

namespace {

constexpr int kSquares = 64;
constexpr int kInputPlanes = 112;
constexpr int kPositionPlanes = 12;
constexpr int kPolicyRecord = 4288;
constexpr int kPolicySize = 1858;
constexpr int kPromotionStart = 4096;

struct Slot {
  void* dev = nullptr;
  long long count = 0;
  bool set = false;
  float first = 0.0f;  // value of element 0 (what a one-element constant buffer holds)
};

struct Dense {
  const void* w = nullptr;  // bf16 [n, k]
  int n = 0, k = 0;
  const void* bias = nullptr;
  const float* fold_c = nullptr;  // deferred LayerNorm: column sums of diag(gamma) W
  const float* fold_d = nullptr;  // beta^T W + bias
  const float* col_scale = nullptr;  // int8 weights: per-output-channel scale (w then holds int8 [n, k])
};

struct Layer {
  // bf16 mode (LayerNorms folded into *_f).  When 3 * embedding is a multiple of 256, qkv_f also holds smolgen's
  // compression as its trailing columns (one GEMM, second output: lc0b200_gemm_args::out_tail_bf16) and
  // compress_f is unused.
  Dense compress_f, sg1, sg2, qkv_f, out, ffn1_f, ffn2;
  Dense compress, qkv, ffn1;                             // int8 mode (stand-alone LayerNorms); out / ffn2 shared
  void* qkv_bias = nullptr;                              // int8 mode: Q, K, V biases back to back
};

// Bump allocator over the caller's arena; with base == nullptr it only measures.
struct Arena {
  char* base = nullptr;
  size_t used = 0;
  void* take(size_t bytes) {
    used = (used + 255) & ~static_cast<size_t>(255);
    void* p = base != nullptr ? base + used : nullptr;
    used += bytes;
    return p;
  }
};

float bf16_bits_to_float(uint16_t bits) {
  uint32_t u = static_cast<uint32_t>(bits) << 16;
  float f;
  std::memcpy(&f, &u, sizeof(f));
  return f;
}

// packed[n, k] = bf16(src[k, n] * gamma[k]);  c[n] = sum_k packed[n, k];  d[n] = sum_k beta[k] src[k, n] (+ bias[n]).
// One thread per output column; upload-time only.
__global__ void fold_layer_norm_kernel(__nv_bfloat16* __restrict__ packed, float* __restrict__ c, float* __restrict__ d,
                                       const __nv_bfloat16* __restrict__ src, const __nv_bfloat16* __restrict__ gamma,
                                       const __nv_bfloat16* __restrict__ beta, const __nv_bfloat16* __restrict__ bias,
                                       int k, int n) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= n) return;
  float sum_c = 0.0f, sum_d = 0.0f;
  for (int row = 0; row < k; ++row) {
    const float w = __bfloat162float(src[static_cast<long long>(row) * n + col]);
    const __nv_bfloat16 scaled = __float2bfloat16_rn(w * __bfloat162float(gamma[row]));
    packed[static_cast<long long>(col) * k + row] = scaled;
    sum_c += __bfloat162float(scaled);
    sum_d = fmaf(__bfloat162float(beta[row]), w, sum_d);
  }
  c[col] = sum_c;
  d[col] = sum_d + (bias != nullptr ? __bfloat162float(bias[col]) : 0.0f);
}

// Symmetric per-output-channel int8 (the quantiser of the int8 GEMM path): s[n] = max_k |W[k,n]| / 127
// (1 for an all-zero column), Wq[n,k] = clamp(rint(W[k,n] / s[n]), -127, 127), round-half-even, IEEE
// division.  One thread per output column; upload-time only.
__global__ void quantize_weight_kernel(int8_t* __restrict__ packed, float* __restrict__ scale,
                                       const __nv_bfloat16* __restrict__ src, int k, int n) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= n) return;
  float amax = 0.0f;
  for (int row = 0; row < k; ++row) amax = fmaxf(amax, fabsf(__bfloat162float(src[static_cast<long long>(row) * n + col])));
  const float s = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
  scale[col] = s;
  for (int row = 0; row < k; ++row) {
    const float w = __bfloat162float(src[static_cast<long long>(row) * n + col]);
    const int q = max(-127, min(127, __float2int_rn(__fdiv_rn(w, s))));
    packed[static_cast<long long>(col) * k + row] = static_cast<int8_t>(q);
  }
}

}  // namespace

struct lc0b200_net {
  lc0b200_net_config cfg;
  int max_batch = 0;
  Arena arena;
  size_t arena_bytes = 0;
  bool finalized = false;
  std::map<std::string, Slot> weights;
  // prepared operands
  Dense pe, emb, emb_ffn1, emb_ffn2, sg_shared, pol1, pol_q, pol_k, value[3], mlh[3];
  std::vector<Layer> layers;
  void* zero_bias = nullptr;
  int32_t* table = nullptr;
  // workspace
  void *pos_in, *position, *emb_in, *x[3], *branch, *hidden, *qkv, *merged, *compressed, *sg_hidden, *sg_gen, *sg_bias;
  void *pol_emb, *pol_q_buf, *pol_k_buf, *records, *val_emb, *val_hid, *mlh_emb, *mlh_hid;
  float* stats[3];
  void *q_d = nullptr, *q_f = nullptr;  // int8 mode: quantised activations [t, embedding] and [t, ffn]
  float* q_scale = nullptr;             // ... and their per-row scales
};

namespace {

std::string enc(int i, const char* tail) { return "/encoder" + std::to_string(i) + tail; }

// Every learned buffer of the forward pass, name -> element count (the reference's persistent
// buffers, bt4/network.py:349-449, 715-774, 868-936, 1089-1132, 1198-1251, 1427-1466).
std::vector<std::pair<std::string, long long>> weight_table(const lc0b200_net_config& c) {
  const long long d = c.embedding, f = c.ffn, e = c.pos_enc, cc = c.smolgen_compress, s1 = c.smolgen_hidden,
                  g = c.smolgen_gen, h = c.heads, p = c.policy, pm = c.policy_model;
  std::vector<std::pair<std::string, long long>> t = {
      {"/attn_body/embedding/preprocess/matmul/w", kSquares * kPositionPlanes * kSquares * e},
      {"/attn_body/embedding/preprocess/add/w", kSquares * e},
      {"/attn_body/matmul/w", (kInputPlanes + e) * d},
      {"/attn_body/add/w", d},
      {"/attn_body/ln/w/scale", d},
      {"/attn_body/ln/w/bias", d},
      {"/ip_mul_gate/w", kSquares * d},
      {"/ip_add_gate/w", kSquares * d},
      {"/attn_body/ffn/dense1/w/w", d * f},
      {"/attn_body/ffn/dense1/b/w", f},
      {"/attn_body/ffn/dense2/w/w", f * d},
      {"/attn_body/ffn/dense2/b/w", d},
      {"/attn_body/ln2/w/scale", d},
      {"/attn_body/ln2/w/bias", d},
      {"/const/smolgen_w", g * kSquares * kSquares},
      {"/attn_body/ffn/alpha/w", 1},
      {"/policy/scale/w", 1},
  };
  for (int i = 0; i < c.layers; ++i) {
    const std::pair<const char*, long long> per_layer[] = {
        {"/smolgen/compress/w", d * cc},      {"/smolgen/dense1/w/w", kSquares * cc * s1},
        {"/smolgen/dense1/b/w", s1},          {"/smolgen/ln1/w/scale", s1},
        {"/smolgen/ln1/w/bias", s1},          {"/smolgen/dense2/w/w", s1 * h * g},
        {"/smolgen/dense2/b/w", h * g},       {"/smolgen/ln2/w/scale", h * g},
        {"/smolgen/ln2/w/bias", h * g},       {"/mha/Q/w/w", d * d},
        {"/mha/Q/b/w", d},                    {"/mha/K/w/w", d * d},
        {"/mha/K/b/w", d},                    {"/mha/V/w/w", d * d},
        {"/mha/V/b/w", d},                    {"/mha/out/dense/w/w", d * d},
        {"/mha/out/dense/b/w", d},            {"/ln1/w/scale", d},
        {"/ln1/w/bias", d},                   {"/ffn/dense1/w/w", d * f},
        {"/ffn/dense1/b/w", f},               {"/ffn/dense2/w/w", f * d},
        {"/ffn/dense2/b/w", d},               {"/ln2/w/scale", d},
        {"/ln2/w/bias", d},                   {"/mha/QK/scale/w", 1},
        {"/alpha*input/w", 1},                {"/ffn/alpha/w", 1},
    };
    for (const auto& it : per_layer) t.emplace_back(enc(i, it.first), it.second);
  }
  const std::pair<const char*, long long> heads[] = {
      {"/policy/dense1/matmul/w", d * p},
      {"/policy/dense1/add/w", p},
      {"/policy/Q/matmul/w", p * pm},
      {"/policy/Q/add/w", pm},
      {"/policy/K/matmul/w", p * pm},
      {"/policy/K/add/w", pm},
      {"/policy/promotion/matmul/w", pm * 4},
      {"/value/embed/matmul/w", d * c.value_embed},
      {"/value/embed/add/w", c.value_embed},
      {"/value/dense1/matmul/w", static_cast<long long>(kSquares) * c.value_embed * c.value_hidden},
      {"/value/dense1/add/w", c.value_hidden},
      {"/value/dense2/matmul/w", c.value_hidden * 3LL},
      {"/value/dense2/add/w", 3},
      {"/mlh/embed/matmul/w", d * c.mlh_embed},
      {"/mlh/embed/add/w", c.mlh_embed},
      {"/mlh/dense1/matmul/w", static_cast<long long>(kSquares) * c.mlh_embed * c.mlh_hidden},
      {"/mlh/dense1/add/w", c.mlh_hidden},
      {"/mlh/dense2/matmul/w", c.mlh_hidden * 1LL},
      {"/mlh/dense2/add/w", 1},
  };
  for (const auto& it : heads) t.emplace_back(it.first, it.second);
  return t;
}

// Q, K, V and smolgen's compression read the same rows; they run as one GEMM when its second output can
// start at a multiple of 256 columns.
bool fuse_compress(const lc0b200_net_config& c) { return !c.int8_gemms && (3 * c.embedding) % 256 == 0; }

bool config_ok(const lc0b200_net_config& c) {
  return c.embedding > 0 && c.layers > 0 && c.heads > 0 && c.embedding % c.heads == 0 && c.embedding / c.heads == 32 &&
         c.ffn > 0 && c.pos_enc > 0 && c.smolgen_compress > 0 && c.smolgen_hidden > 0 && c.smolgen_gen > 0 &&
         c.policy > 0 && c.policy_model > 0 && c.value_embed > 0 && c.value_hidden > 0 && c.mlh_embed > 0 &&
         c.mlh_hidden > 0 && c.ln_eps > 0.0f && c.embedding % 64 == 0;
}

// Lays every device buffer out in the arena (or just measures, when the arena has no base).
void plan(lc0b200_net& net) {
  const lc0b200_net_config& c = net.cfg;
  Arena& a = net.arena;
  a.used = 0;
  for (const auto& it : weight_table(c)) {
    Slot& slot = net.weights[it.first];
    slot.count = it.second;
    slot.dev = a.take(static_cast<size_t>(it.second) * 2);
  }
  const size_t d = c.embedding, f = c.ffn;
  auto packed = [&](Dense& dense, size_t n, size_t k) {
    dense.n = static_cast<int>(n);
    dense.k = static_cast<int>(k);
    dense.w = a.take(n * k * 2);
  };
  auto folded = [&](Dense& dense, size_t n, size_t k) {
    packed(dense, n, k);
    dense.fold_c = static_cast<float*>(a.take(n * 4));
    dense.fold_d = static_cast<float*>(a.take(n * 4));
  };
  packed(net.pe, static_cast<size_t>(kSquares) * c.pos_enc, kSquares * kPositionPlanes);
  packed(net.emb, d, kInputPlanes + c.pos_enc);
  packed(net.emb_ffn1, f, d);
  packed(net.emb_ffn2, d, f);
  packed(net.sg_shared, kSquares * kSquares, c.smolgen_gen);
  net.layers.assign(c.layers, Layer());
  auto quantised = [&](Dense& dense, size_t n, size_t k) {
    dense.n = static_cast<int>(n);
    dense.k = static_cast<int>(k);
    dense.w = a.take(n * k);
    dense.col_scale = static_cast<float*>(a.take(n * 4));
  };
  for (Layer& l : net.layers) {
    packed(l.sg1, c.smolgen_hidden, static_cast<size_t>(kSquares) * c.smolgen_compress);
    packed(l.sg2, static_cast<size_t>(c.heads) * c.smolgen_gen, c.smolgen_hidden);
    if (c.int8_gemms) {
      packed(l.compress, c.smolgen_compress, d);
      quantised(l.qkv, 3 * d, d);
      l.qkv_bias = a.take(3 * d * 2);
      quantised(l.out, d, d);
      quantised(l.ffn1, f, d);
      quantised(l.ffn2, d, f);
    } else {
      if (fuse_compress(c)) {
        folded(l.qkv_f, 3 * d + c.smolgen_compress, d);
      } else {
        folded(l.compress_f, c.smolgen_compress, d);
        folded(l.qkv_f, 3 * d, d);
      }
      packed(l.out, d, d);
      folded(l.ffn1_f, f, d);
      packed(l.ffn2, d, f);
    }
  }
  packed(net.pol1, c.policy, d);
  packed(net.pol_q, c.policy_model, c.policy);
  packed(net.pol_k, c.policy_model, c.policy);
  packed(net.value[0], c.value_embed, d);
  packed(net.value[1], c.value_hidden, static_cast<size_t>(kSquares) * c.value_embed);
  packed(net.value[2], 3, c.value_hidden);
  packed(net.mlh[0], c.mlh_embed, d);
  packed(net.mlh[1], c.mlh_hidden, static_cast<size_t>(kSquares) * c.mlh_embed);
  packed(net.mlh[2], 1, c.mlh_hidden);
  net.zero_bias = a.take(d * 2);
  net.table = static_cast<int32_t*>(a.take(kPolicySize * 4));
  // workspace for max_batch positions
  const size_t b = net.max_batch, t = b * kSquares;
  net.pos_in = a.take(b * kSquares * kPositionPlanes * 2);
  net.position = a.take(b * kSquares * c.pos_enc * 2);
  net.emb_in = a.take(t * (kInputPlanes + c.pos_enc) * 2);
  for (auto& x : net.x) x = a.take(t * d * 2);
  net.branch = a.take(t * d * 2);
  net.hidden = a.take(t * f * 2);
  net.qkv = a.take(t * 3 * d * 2);
  net.merged = a.take(t * d * 2);
  net.compressed = a.take(t * c.smolgen_compress * 2);
  net.sg_hidden = a.take(b * c.smolgen_hidden * 2);
  net.sg_gen = a.take(b * c.heads * c.smolgen_gen * 2);
  net.sg_bias = a.take(b * c.heads * kSquares * kSquares * 2);
  net.pol_emb = a.take(t * c.policy * 2);
  net.pol_q_buf = a.take(t * c.policy_model * 2);
  net.pol_k_buf = a.take(t * c.policy_model * 2);
  net.records = a.take(b * kPolicyRecord * 2);
  net.val_emb = a.take(t * c.value_embed * 2);
  net.val_hid = a.take(b * c.value_hidden * 2);
  net.mlh_emb = a.take(t * c.mlh_embed * 2);
  net.mlh_hid = a.take(b * c.mlh_hidden * 2);
  if (c.int8_gemms) {
    net.q_d = a.take(t * d);
    net.q_f = a.take(t * f);
    net.q_scale = static_cast<float*>(a.take(t * 4));
  } else {
    const size_t parts = (d + 63) / 64;
    for (auto& s : net.stats) s = static_cast<float*>(a.take(parts * t * 2 * 4));
  }
  a.take(0);
}

const Slot* find(const lc0b200_net& net, const std::string& name) {
  auto it = net.weights.find(name);
  return it == net.weights.end() ? nullptr : &it->second;
}

// One GEMM through the public entry point (so that every argument check applies here too).
int run_gemm(void* out, const void* a, const Dense& w, long long m, int activation, int out_kind, void* stream,
             const void* bias_override = nullptr, bool use_bias = true, const float* row_scale = nullptr) {
  lc0b200_gemm_args g;
  std::memset(&g, 0, sizeof(g));
  g.out = out;
  g.a = a;
  g.w = w.w;
  g.bias_bf16 = bias_override != nullptr ? bias_override : (use_bias ? w.bias : nullptr);
  g.row_scale = row_scale;
  g.col_scale = w.col_scale;
  g.m = m;
  g.n = w.n;
  g.k = w.k;
  g.lda = w.k;
  g.ldw = w.k;
  g.ldc = w.n;
  g.in_type = w.col_scale != nullptr ? LC0B200_IN_INT8 : LC0B200_IN_BF16;
  g.out_kind = out_kind;
  g.w_layout = LC0B200_W_NK;
  g.activation = activation;
  g.ln_eps = 1e-3f;
  return lc0b200_gemm(&g, stream);
}

int run_gemm_folded(const lc0b200_net& net, void* out, const void* z, const Dense& w, long long m, const float* stats,
                    int activation, void* stream, void* out_tail = nullptr, int n_main = 0) {
  lc0b200_gemm_args g;
  std::memset(&g, 0, sizeof(g));
  g.out = out;
  g.a = z;
  g.w = w.w;
  g.m = m;
  g.n = w.n;
  g.k = w.k;
  g.lda = w.k;
  g.ldw = w.k;
  g.ldc = w.n;
  g.in_type = LC0B200_IN_BF16;
  g.out_kind = LC0B200_OUT_BF16;
  g.w_layout = LC0B200_W_NK;
  g.activation = activation;
  g.ln_in_stats = stats;
  g.ln_in_c = w.fold_c;
  g.ln_in_d = w.fold_d;
  g.ln_in_parts = (w.k + 63) / 64;
  g.ln_eps = net.cfg.ln_eps;
  if (out_tail != nullptr) {  // columns [n_main, n) to a matrix of their own
    g.out_tail_bf16 = out_tail;
    g.n_main = n_main;
    g.ldc = n_main;
    g.ldc_tail = w.n - n_main;
  }
  return lc0b200_gemm(&g, stream);
}

// z_out = alpha * (a W + bias) + skip, skip plain or a deferred LayerNorm (stats / gamma / beta); row sums out.
int run_gemm_residual(const lc0b200_net& net, void* z_out, const void* a, const Dense& w, const void* bias, long long m,
                      const void* skip, const float* skip_stats, const void* gamma, const void* beta, float alpha,
                      float* stats_out, void* stream) {
  lc0b200_gemm_args g;
  std::memset(&g, 0, sizeof(g));
  g.out = z_out;
  g.a = a;
  g.w = w.w;
  g.bias_bf16 = bias;
  g.m = m;
  g.n = w.n;
  g.k = w.k;
  g.lda = w.k;
  g.ldw = w.k;
  g.ldc = w.n;
  g.in_type = LC0B200_IN_BF16;
  g.out_kind = LC0B200_OUT_BF16;
  g.w_layout = LC0B200_W_NK;
  g.activation = LC0B200_ACT_NONE;
  g.ln_eps = net.cfg.ln_eps;
  g.res_skip_bf16 = skip;
  g.ld_skip = w.n;
  g.res_alpha = alpha;
  if (skip_stats != nullptr) {
    g.res_stats = skip_stats;
    g.res_gamma_bf16 = gamma;
    g.res_beta_bf16 = beta;
    g.res_parts = (w.n + 63) / 64;
  }
  g.stats_out = stats_out;
  return lc0b200_gemm(&g, stream);
}

#define NET_TRY(expr)                    \
  do {                                   \
    const int status_ = (expr);          \
    if (status_ != LC0B200_OK) return status_; \
  } while (0)

}  // namespace

extern "C" {

LC0B200_API size_t lc0b200_net_arena_bytes(const lc0b200_net_config* config, int max_batch) {
  if (config == nullptr || max_batch <= 0 || !config_ok(*config)) return 0;
  lc0b200_net probe;
  probe.cfg = *config;
  probe.max_batch = max_batch;
  plan(probe);
  return probe.arena.used + 256;
}

LC0B200_API int lc0b200_net_create(lc0b200_net** out, const lc0b200_net_config* config, int max_batch,
                                   void* device_arena, size_t arena_bytes) {
  if (out == nullptr || config == nullptr || device_arena == nullptr) return LC0B200_ERR_NULL_POINTER;
  if (max_batch <= 0 || !config_ok(*config)) return LC0B200_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(device_arena) & 255u) != 0) return LC0B200_ERR_MISALIGNED;
  if (arena_bytes < lc0b200_net_arena_bytes(config, max_batch)) return LC0B200_ERR_SCRATCH_LIMIT;
  lc0b200_net* net = new (std::nothrow) lc0b200_net();
  if (net == nullptr) return LC0B200_ERR_CUDA;
  net->cfg = *config;
  net->max_batch = max_batch;
  net->arena.base = static_cast<char*>(device_arena);
  net->arena_bytes = arena_bytes;
  plan(*net);
  *out = net;
  return LC0B200_OK;
}

LC0B200_API void lc0b200_net_destroy(lc0b200_net* net) { delete net; }

LC0B200_API int lc0b200_net_weight_count(const lc0b200_net* net) {
  return net == nullptr ? 0 : static_cast<int>(net->weights.size());
}

LC0B200_API int lc0b200_net_weight_info(const lc0b200_net* net, int index, const char** name, long long* elements) {
  if (net == nullptr) return LC0B200_ERR_NULL_POINTER;
  if (index < 0 || index >= static_cast<int>(net->weights.size())) return LC0B200_ERR_BAD_SHAPE;
  auto it = net->weights.begin();
  std::advance(it, index);
  if (name != nullptr) *name = it->first.c_str();
  if (elements != nullptr) *elements = it->second.count;
  return LC0B200_OK;
}

LC0B200_API int lc0b200_net_set_weight(lc0b200_net* net, const char* name, const void* host_bf16, long long elements,
                                       void* stream) {
  if (net == nullptr || name == nullptr || host_bf16 == nullptr) return LC0B200_ERR_NULL_POINTER;
  auto it = net->weights.find(name);
  if (it == net->weights.end()) return LC0B200_ERR_UNSUPPORTED;
  Slot& slot = it->second;
  if (elements != slot.count) return LC0B200_ERR_BAD_SHAPE;
  if (cudaMemcpyAsync(slot.dev, host_bf16, static_cast<size_t>(elements) * 2, cudaMemcpyHostToDevice,
                      reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess) {
    return LC0B200_ERR_CUDA;
  }
  slot.first = bf16_bits_to_float(*static_cast<const uint16_t*>(host_bf16));
  slot.set = true;
  net->finalized = false;
  return LC0B200_OK;
}

LC0B200_API int lc0b200_net_finalize(lc0b200_net* net, void* stream) {
  if (net == nullptr) return LC0B200_ERR_NULL_POINTER;
  for (const auto& it : net->weights) {
    if (!it.second.set) return LC0B200_ERR_NULL_POINTER;  // a weight was never handed over
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const lc0b200_net_config& c = net->cfg;
  auto dev = [&](const std::string& name) -> const void* { return find(*net, name)->dev; };
  // [K,N] as uploaded -> [N,K] for the tensor core.
  auto pack = [&](Dense& dense, const std::string& weight, const char* bias) -> int {
    dense.bias = bias != nullptr ? dev(bias) : nullptr;
    return lc0b200_transpose(const_cast<void*>(dense.w), dev(weight), dense.k, dense.n, 2, stream);
  };
  // Deferred LayerNorm: fold gamma / beta of `ln` into the (possibly concatenated) weight.
  // The parts are laid side by side along N, each as wide as its weight says; an empty bias name is a part
  // without bias.
  auto fold = [&](Dense& dense, const std::vector<std::string>& parts, const std::vector<std::string>& biases,
                  const std::string& ln) -> int {
    size_t off = 0;
    for (size_t i = 0; i < parts.size(); ++i) {
      const int width = static_cast<int>(find(*net, parts[i])->count / dense.k);
      const bool has_bias = !biases.empty() && !biases[i].empty();
      fold_layer_norm_kernel<<<(width + 127) / 128, 128, 0, st>>>(
          reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(dense.w)) + off * dense.k,
          const_cast<float*>(dense.fold_c) + off, const_cast<float*>(dense.fold_d) + off,
          static_cast<const __nv_bfloat16*>(dev(parts[i])), static_cast<const __nv_bfloat16*>(dev(ln + "/w/scale")),
          static_cast<const __nv_bfloat16*>(dev(ln + "/w/bias")),
          has_bias ? static_cast<const __nv_bfloat16*>(dev(biases[i])) : nullptr, dense.k, width);
      off += static_cast<size_t>(width);
    }
    if (off != static_cast<size_t>(dense.n)) return LC0B200_ERR_BAD_SHAPE;
    return cudaGetLastError() == cudaSuccess ? LC0B200_OK : LC0B200_ERR_CUDA;
  };
  // int8 mode: `count` output channels of `weight` ([K, count] as uploaded) into rows [first, first + count)
  // of the packed int8 operand, with their scales.
  auto quantise = [&](Dense& dense, const std::string& weight, size_t first, size_t count) -> int {
    quantize_weight_kernel<<<static_cast<unsigned>((count + 127) / 128), 128, 0, st>>>(
        static_cast<int8_t*>(const_cast<void*>(dense.w)) + first * dense.k, const_cast<float*>(dense.col_scale) + first,
        static_cast<const __nv_bfloat16*>(dev(weight)), dense.k, static_cast<int>(count));
    return cudaGetLastError() == cudaSuccess ? LC0B200_OK : LC0B200_ERR_CUDA;
  };
  NET_TRY(pack(net->pe, "/attn_body/embedding/preprocess/matmul/w", "/attn_body/embedding/preprocess/add/w"));
  NET_TRY(pack(net->emb, "/attn_body/matmul/w", nullptr));
  NET_TRY(pack(net->emb_ffn1, "/attn_body/ffn/dense1/w/w", "/attn_body/ffn/dense1/b/w"));
  NET_TRY(pack(net->emb_ffn2, "/attn_body/ffn/dense2/w/w", nullptr));
  NET_TRY(pack(net->sg_shared, "/const/smolgen_w", nullptr));
  for (int i = 0; i < c.layers; ++i) {
    Layer& l = net->layers[i];
    const std::string prev = i == 0 ? std::string("/attn_body/ln2") : enc(i - 1, "/ln2");
    NET_TRY(pack(l.sg1, enc(i, "/smolgen/dense1/w/w"), nullptr));
    NET_TRY(pack(l.sg2, enc(i, "/smolgen/dense2/w/w"), nullptr));
    if (c.int8_gemms) {
      NET_TRY(pack(l.compress, enc(i, "/smolgen/compress/w"), nullptr));
      const char* qkv_w[3] = {"/mha/Q/w/w", "/mha/K/w/w", "/mha/V/w/w"};
      const char* qkv_b[3] = {"/mha/Q/b/w", "/mha/K/b/w", "/mha/V/b/w"};
      const size_t d = c.embedding;
      for (int part = 0; part < 3; ++part) {
        NET_TRY(quantise(l.qkv, enc(i, qkv_w[part]), part * d, d));
        if (cudaMemcpyAsync(static_cast<char*>(l.qkv_bias) + part * d * 2, dev(enc(i, qkv_b[part])), d * 2,
                            cudaMemcpyDeviceToDevice, st) != cudaSuccess) {
          return LC0B200_ERR_CUDA;
        }
      }
      l.qkv.bias = l.qkv_bias;
      NET_TRY(quantise(l.out, enc(i, "/mha/out/dense/w/w"), 0, l.out.n));
      NET_TRY(quantise(l.ffn1, enc(i, "/ffn/dense1/w/w"), 0, l.ffn1.n));
      l.ffn1.bias = dev(enc(i, "/ffn/dense1/b/w"));
      NET_TRY(quantise(l.ffn2, enc(i, "/ffn/dense2/w/w"), 0, l.ffn2.n));
    } else {
      if (fuse_compress(c)) {
        NET_TRY(fold(l.qkv_f, {enc(i, "/mha/Q/w/w"), enc(i, "/mha/K/w/w"), enc(i, "/mha/V/w/w"), enc(i, "/smolgen/compress/w")},
                     {enc(i, "/mha/Q/b/w"), enc(i, "/mha/K/b/w"), enc(i, "/mha/V/b/w"), ""}, prev));
      } else {
        NET_TRY(fold(l.compress_f, {enc(i, "/smolgen/compress/w")}, {}, prev));
        NET_TRY(fold(l.qkv_f, {enc(i, "/mha/Q/w/w"), enc(i, "/mha/K/w/w"), enc(i, "/mha/V/w/w")},
                     {enc(i, "/mha/Q/b/w"), enc(i, "/mha/K/b/w"), enc(i, "/mha/V/b/w")}, prev));
      }
      NET_TRY(pack(l.out, enc(i, "/mha/out/dense/w/w"), nullptr));
      NET_TRY(fold(l.ffn1_f, {enc(i, "/ffn/dense1/w/w")}, {enc(i, "/ffn/dense1/b/w")}, enc(i, "/ln1")));
      NET_TRY(pack(l.ffn2, enc(i, "/ffn/dense2/w/w"), nullptr));
    }
  }
  NET_TRY(pack(net->pol1, "/policy/dense1/matmul/w", "/policy/dense1/add/w"));
  NET_TRY(pack(net->pol_q, "/policy/Q/matmul/w", "/policy/Q/add/w"));
  NET_TRY(pack(net->pol_k, "/policy/K/matmul/w", "/policy/K/add/w"));
  const char* head_names[2] = {"/value", "/mlh"};
  Dense* head_dense[2] = {net->value, net->mlh};
  for (int hd = 0; hd < 2; ++hd) {
    const std::string p = head_names[hd];
    NET_TRY(pack(head_dense[hd][0], p + "/embed/matmul/w", (p + "/embed/add/w").c_str()));
    NET_TRY(pack(head_dense[hd][1], p + "/dense1/matmul/w", (p + "/dense1/add/w").c_str()));
    NET_TRY(pack(head_dense[hd][2], p + "/dense2/matmul/w", (p + "/dense2/add/w").c_str()));
  }
  if (cudaMemsetAsync(net->zero_bias, 0, static_cast<size_t>(c.embedding) * 2, st) != cudaSuccess) return LC0B200_ERR_CUDA;
  // Attention-policy gather table from move geometry: plain moves (queen lines and knight jumps) by
  // from-square then to-square, then the 66 under-promotions by from-file, to-file, piece.
  std::vector<int32_t> table;
  table.reserve(kPolicySize);
  for (int src = 0; src < 64; ++src) {
    for (int dst = 0; dst < 64; ++dst) {
      if (src == dst) continue;
      const int dr = std::abs(dst / 8 - src / 8), df = std::abs(dst % 8 - src % 8);
      const bool queen_line = dr == 0 || df == 0 || dr == df;
      const bool knight = (dr == 1 && df == 2) || (dr == 2 && df == 1);
      if (queen_line || knight) table.push_back(src * 64 + dst);
    }
  }
  for (int sf = 0; sf < 8; ++sf) {
    for (int df = 0; df < 8; ++df) {
      if (std::abs(sf - df) > 1) continue;
      for (int piece = 0; piece < 3; ++piece) table.push_back(kPromotionStart + sf * 24 + df * 3 + piece);
    }
  }
  if (static_cast<int>(table.size()) != kPolicySize) return LC0B200_ERR_BAD_SHAPE;
  // (pageable source: the copy has completed with respect to the host buffer when the call returns)
  if (cudaMemcpyAsync(net->table, table.data(), table.size() * 4, cudaMemcpyHostToDevice, st) != cudaSuccess) {
    return LC0B200_ERR_CUDA;
  }
  if (cudaStreamSynchronize(st) != cudaSuccess) return LC0B200_ERR_CUDA;
  net->finalized = true;
  return LC0B200_OK;
}

LC0B200_API int lc0b200_net_forward(lc0b200_net* net, const uint64_t* masks, const float* values, int batch,
                                    float* policy_f32, float* wdl_f32, float* mlh_f32, void* stream) {
  if (net == nullptr || masks == nullptr || values == nullptr || policy_f32 == nullptr || wdl_f32 == nullptr ||
      mlh_f32 == nullptr) {
    return LC0B200_ERR_NULL_POINTER;
  }
  if (!net->finalized) return LC0B200_ERR_UNSUPPORTED;
  if (batch <= 0 || batch > net->max_batch) return LC0B200_ERR_BAD_SHAPE;
  const lc0b200_net_config& c = net->cfg;
  const long long b = batch, t = b * kSquares;
  const int d = c.embedding, h = c.heads;
  const float eps = c.ln_eps;
  auto dev = [&](const std::string& name) -> const void* { return find(*net, name)->dev; };
  auto scalar = [&](const std::string& name) -> float { return find(*net, name)->first; };
  auto bf = [](void* base, long long elements) -> void* { return static_cast<char*>(base) + elements * 2; };

  // ---- input embedding (network.py:458-642)
  NET_TRY(lc0b200_embed_position_input(net->pos_in, masks, values, batch, stream));
  NET_TRY(run_gemm(net->position, net->pos_in, net->pe, b, LC0B200_ACT_NONE, LC0B200_OUT_BF16, stream));
  NET_TRY(lc0b200_embed_concat(net->emb_in, masks, values, net->position, batch, c.pos_enc, stream));
  NET_TRY(run_gemm(net->branch, net->emb_in, net->emb, t, LC0B200_ACT_NONE, LC0B200_OUT_BF16, stream));
  void* skip = net->x[0];
  NET_TRY(lc0b200_layer_norm(skip, net->branch, dev("/attn_body/add/w"), nullptr, dev("/attn_body/ln/w/scale"),
                             dev("/attn_body/ln/w/bias"), nullptr, t, d, LC0B200_ACT_MISH, 0, eps, nullptr, nullptr,
                             stream));
  NET_TRY(lc0b200_input_gating(skip, skip, dev("/ip_mul_gate/w"), dev("/ip_add_gate/w"), batch, kSquares, d, stream));
  NET_TRY(run_gemm(net->hidden, skip, net->emb_ffn1, t, LC0B200_ACT_MISH, LC0B200_OUT_BF16, stream));

  void* body = nullptr;
  if (c.int8_gemms) {
    // ---- encoder tower, int8 GEMMs: stand-alone LayerNorm kernels that also emit the quantised rows
    const float* qs = net->q_scale;
    auto layer_norm_q = [&](void* out, const std::string& bias, const std::string& lnp, const void* skip_rows,
                            const std::string& alpha) -> int {
      return lc0b200_layer_norm(out, net->branch, dev(bias), skip_rows, dev(lnp + "/w/scale"), dev(lnp + "/w/bias"),
                                dev(alpha), t, d, LC0B200_ACT_NONE, 1, eps, net->q_d, net->q_scale, stream);
    };
    NET_TRY(run_gemm(net->branch, net->hidden, net->emb_ffn2, t, LC0B200_ACT_NONE, LC0B200_OUT_BF16, stream));
    body = net->x[1];
    NET_TRY(layer_norm_q(body, "/attn_body/ffn/dense2/b/w", "/attn_body/ln2", skip, "/attn_body/ffn/alpha/w"));
    void* spare[2] = {net->x[0], net->x[2]};
    for (int i = 0; i < c.layers; ++i) {
      const Layer& l = net->layers[i];
      NET_TRY(run_gemm(net->qkv, net->q_d, l.qkv, t, LC0B200_ACT_NONE, LC0B200_OUT_BF16, stream, nullptr, true, qs));
      NET_TRY(run_gemm(net->compressed, body, l.compress, t, LC0B200_ACT_NONE, LC0B200_OUT_BF16, stream));
      NET_TRY(run_gemm(net->sg_hidden, net->compressed, l.sg1, b, LC0B200_ACT_NONE, LC0B200_OUT_BF16, stream));
      NET_TRY(lc0b200_layer_norm(net->sg_hidden, net->sg_hidden, dev(enc(i, "/smolgen/dense1/b/w")), nullptr,
                                 dev(enc(i, "/smolgen/ln1/w/scale")), dev(enc(i, "/smolgen/ln1/w/bias")), nullptr, b,
                                 c.smolgen_hidden, LC0B200_ACT_SWISH, 0, eps, nullptr, nullptr, stream));
      NET_TRY(run_gemm(net->sg_gen, net->sg_hidden, l.sg2, b, LC0B200_ACT_NONE, LC0B200_OUT_BF16, stream));
      NET_TRY(lc0b200_layer_norm(net->sg_gen, net->sg_gen, dev(enc(i, "/smolgen/dense2/b/w")), nullptr,
                                 dev(enc(i, "/smolgen/ln2/w/scale")), dev(enc(i, "/smolgen/ln2/w/bias")), nullptr, b,
                                 h * c.smolgen_gen, LC0B200_ACT_SWISH, 0, eps, nullptr, nullptr, stream));
      NET_TRY(run_gemm(net->sg_bias, net->sg_gen, net->sg_shared, b * h, LC0B200_ACT_NONE, LC0B200_OUT_BF16, stream));
      NET_TRY(lc0b200_attention(net->merged, net->qkv, bf(net->qkv, d), bf(net->qkv, 2 * d), net->sg_bias,
                                scalar(enc(i, "/mha/QK/scale/w")), b, h, 32, 3LL * d, 3LL * d, 3LL * d, d, stream));
      NET_TRY(lc0b200_quantize_rows(net->q_d, net->q_scale, net->merged, t, d, d, stream));
      NET_TRY(run_gemm(net->branch, net->q_d, l.out, t, LC0B200_ACT_NONE, LC0B200_OUT_BF16, stream, nullptr, false, qs));
      void* attended = spare[0];
      NET_TRY(layer_norm_q(attended, enc(i, "/mha/out/dense/b/w"), enc(i, "/ln1"), body, enc(i, "/alpha*input/w")));
      NET_TRY(run_gemm(net->hidden, net->q_d, l.ffn1, t, LC0B200_ACT_MISH, LC0B200_OUT_BF16, stream, nullptr, true, qs));
      NET_TRY(lc0b200_quantize_rows(net->q_f, net->q_scale, net->hidden, t, c.ffn, c.ffn, stream));
      NET_TRY(run_gemm(net->branch, net->q_f, l.ffn2, t, LC0B200_ACT_NONE, LC0B200_OUT_BF16, stream, nullptr, false, qs));
      void* next = spare[1];
      NET_TRY(layer_norm_q(next, enc(i, "/ffn/dense2/b/w"), enc(i, "/ln2"), attended, enc(i, "/ffn/alpha/w")));
      spare[0] = body;
      spare[1] = attended;
      body = next;
    }
  } else {
  // ---- encoder tower with the LayerNorms deferred into the GEMM epilogues
  void* z = net->x[1];
  float* stats = net->stats[0];
  std::string ln = "/attn_body/ln2";
  NET_TRY(run_gemm_residual(*net, z, net->hidden, net->emb_ffn2, dev("/attn_body/ffn/dense2/b/w"), t, skip, nullptr,
                            nullptr, nullptr, scalar("/attn_body/ffn/alpha/w"), stats, stream));
  void* free_z[2] = {net->x[0], net->x[2]};
  float* free_s[2] = {net->stats[1], net->stats[2]};
  for (int i = 0; i < c.layers; ++i) {
    const Layer& l = net->layers[i];
    if (fuse_compress(c)) {
      NET_TRY(run_gemm_folded(*net, net->qkv, z, l.qkv_f, t, stats, LC0B200_ACT_NONE, stream, net->compressed, 3 * d));
    } else {
      NET_TRY(run_gemm_folded(*net, net->qkv, z, l.qkv_f, t, stats, LC0B200_ACT_NONE, stream));
      NET_TRY(run_gemm_folded(*net, net->compressed, z, l.compress_f, t, stats, LC0B200_ACT_NONE, stream));
    }
    // smolgen: per-position 64 x 64 logit bias for every head (network.py:778-849, 943-955)
    NET_TRY(run_gemm(net->sg_hidden, net->compressed, l.sg1, b, LC0B200_ACT_NONE, LC0B200_OUT_BF16, stream));
    NET_TRY(lc0b200_layer_norm(net->sg_hidden, net->sg_hidden, dev(enc(i, "/smolgen/dense1/b/w")), nullptr,
                               dev(enc(i, "/smolgen/ln1/w/scale")), dev(enc(i, "/smolgen/ln1/w/bias")), nullptr, b,
                               c.smolgen_hidden, LC0B200_ACT_SWISH, 0, eps, nullptr, nullptr, stream));
    NET_TRY(run_gemm(net->sg_gen, net->sg_hidden, l.sg2, b, LC0B200_ACT_NONE, LC0B200_OUT_BF16, stream));
    NET_TRY(lc0b200_layer_norm(net->sg_gen, net->sg_gen, dev(enc(i, "/smolgen/dense2/b/w")), nullptr,
                               dev(enc(i, "/smolgen/ln2/w/scale")), dev(enc(i, "/smolgen/ln2/w/bias")), nullptr, b,
                               h * c.smolgen_gen, LC0B200_ACT_SWISH, 0, eps, nullptr, nullptr, stream));
    NET_TRY(run_gemm(net->sg_bias, net->sg_gen, net->sg_shared, b * h, LC0B200_ACT_NONE, LC0B200_OUT_BF16, stream));
    // fused attention (network.py:1004-1047)
    NET_TRY(lc0b200_attention(net->merged, net->qkv, bf(net->qkv, d), bf(net->qkv, 2 * d), net->sg_bias,
                              scalar(enc(i, "/mha/QK/scale/w")), b, h, 32, 3LL * d, 3LL * d, 3LL * d, d, stream));
    void* z1 = free_z[0];
    float* stats1 = free_s[0];
    NET_TRY(run_gemm_residual(*net, z1, net->merged, l.out, dev(enc(i, "/mha/out/dense/b/w")), t, z, stats,
                              dev(ln + "/w/scale"), dev(ln + "/w/bias"), scalar(enc(i, "/alpha*input/w")), stats1,
                              stream));
    NET_TRY(run_gemm_folded(*net, net->hidden, z1, l.ffn1_f, t, stats1, LC0B200_ACT_MISH, stream));
    void* z2 = free_z[1];
    float* stats2 = free_s[1];
    NET_TRY(run_gemm_residual(*net, z2, net->hidden, l.ffn2, dev(enc(i, "/ffn/dense2/b/w")), t, z1, stats1,
                              dev(enc(i, "/ln1/w/scale")), dev(enc(i, "/ln1/w/bias")), scalar(enc(i, "/ffn/alpha/w")),
                              stats2, stream));
    free_z[0] = z;
    free_z[1] = z1;
    free_s[0] = stats;
    free_s[1] = stats1;
    z = z2;
    stats = stats2;
    ln = enc(i, "/ln2");
  }
  body = free_z[0];
  NET_TRY(lc0b200_layer_norm(body, z, net->zero_bias, nullptr, dev(ln + "/w/scale"), dev(ln + "/w/bias"), nullptr, t, d,
                             LC0B200_ACT_NONE, 0, eps, nullptr, nullptr, stream));
  }

  // ---- policy head (network.py:1261-1356)
  NET_TRY(run_gemm(net->pol_emb, body, net->pol1, t, LC0B200_ACT_MISH, LC0B200_OUT_BF16, stream));
  NET_TRY(run_gemm(net->pol_q_buf, net->pol_emb, net->pol_q, t, LC0B200_ACT_NONE, LC0B200_OUT_BF16, stream));
  NET_TRY(run_gemm(net->pol_k_buf, net->pol_emb, net->pol_k, t, LC0B200_ACT_NONE, LC0B200_OUT_BF16, stream));
  NET_TRY(lc0b200_batched_matmul(net->records, net->pol_q_buf, net->pol_k_buf, dev("/policy/scale/w"),
                                 LC0B200_BMM_POLICY_QK, b, kSquares, kSquares, c.policy_model, 1, stream));
  NET_TRY(lc0b200_policy_tail(policy_f32, net->records, net->pol_k_buf, dev("/policy/promotion/matmul/w"), net->table,
                              batch, c.policy_model, stream));
  // ---- value and moves-left heads (network.py:1475-1550)
  NET_TRY(run_gemm(net->val_emb, body, net->value[0], t, LC0B200_ACT_MISH, LC0B200_OUT_BF16, stream));
  NET_TRY(run_gemm(net->val_hid, net->val_emb, net->value[1], b, LC0B200_ACT_MISH, LC0B200_OUT_BF16, stream));
  NET_TRY(run_gemm(wdl_f32, net->val_hid, net->value[2], b, LC0B200_ACT_NONE, LC0B200_OUT_F32, stream));
  NET_TRY(run_gemm(net->mlh_emb, body, net->mlh[0], t, LC0B200_ACT_MISH, LC0B200_OUT_BF16, stream));
  NET_TRY(run_gemm(net->mlh_hid, net->mlh_emb, net->mlh[1], b, LC0B200_ACT_MISH, LC0B200_OUT_BF16, stream));
  NET_TRY(run_gemm(mlh_f32, net->mlh_hid, net->mlh[2], b, LC0B200_ACT_RELU, LC0B200_OUT_F32, stream));
  return LC0B200_OK;
}

}  // extern "C"
