// TEST INFRASTRUCTURE — never linked into the product library.
//
// C-ABI shim around the UNMODIFIED reference CPU sources (compiled in place from
// the reference tree by oracle/Makefile; outputs go to oracle/_ref/ only). It lets
// the tests and the CPU-baseline leg of bench.py call the reference's own
// functions through ctypes:
//   dequantizers          quantization.cpp:171-266, 1047-1052
//   fp16_to_fp32          quantization.cpp:47-90
//   Kahan FP32 matvec     utils.cpp:349-397
//   rmsnorm / softmax /   utils.cpp:648-698, 700-707, 428-489
//   silu / rope
//   TinyLlamaModel        model.cpp:154 (ctor), 536-807 (forward),
//                         2117 (forward_cpu_batch), 1094-1156 (logits batch)
//   KVCache               kv_cache.cpp:10
// The generation loop restated here (prefill through forward_cpu_batch when the
// prompt has >= 32 tokens, otherwise token by token; greedy = first maximum)
// follows api.cpp:596-700 and api.cpp:134-136 with the tokenizer left out.
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>
#include <algorithm>
#include <exception>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "logger.h"
#include "model.h"
#include "quantization.h"
#include "utils.h"
#include "ggml_types.h"

namespace {
struct RefModel {
  std::unique_ptr<TinyLlamaModel> model;
  KVCache kv;
  ModelConfig cfg;
};
thread_local std::string g_err;
}  // namespace

extern "C" {

const char* ref_last_error() { return g_err.c_str(); }

void ref_logger_off() { Logger::set_level(Logger::Level::OFF); }

// OpenMP threads of the reference's loops (a launcher may have set OMP_NUM_THREADS=1 for the whole process).
void ref_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#endif
}

float ref_fp16_to_fp32(uint16_t h, int is_scale_field) {
  return fp16_to_fp32(h, is_scale_field != 0);
}

// ggml_type: 8 = Q8_0, 12 = Q4_K, 14 = Q6_K (ggml_types.h:21-42)
int ref_dequant(int ggml_type, const void* blocks, size_t n_blocks, float* out) {
  switch (ggml_type) {
    case 8: {
      const block_q8_0* b = static_cast<const block_q8_0*>(blocks);
      for (size_t i = 0; i < n_blocks; ++i) dequantize_q8_0_block(&b[i], out + i * 32);
      return 0;
    }
    case 12: {
      const block_q4_K* b = static_cast<const block_q4_K*>(blocks);
      for (size_t i = 0; i < n_blocks; ++i) dequantize_q4_k_m(&b[i], out + i * 256, 256, false);
      return 0;
    }
    case 14: {
      const block_q6_K* b = static_cast<const block_q6_K*>(blocks);
      for (size_t i = 0; i < n_blocks; ++i) dequantize_q6_k(&b[i], out + i * 256, 256, false);
      return 0;
    }
    default:
      g_err = "ref_dequant: unsupported ggml type";
      return 1;
  }
}

int ref_matvec_f32(const float* w, const float* x, float* y, int rows, int cols) {
  std::vector<float> W(w, w + (size_t)rows * cols), X(x, x + cols), Y;
  matvec_f32_f32_vector_cpu(W, X, Y, rows, cols);
  std::memcpy(y, Y.data(), sizeof(float) * rows);
  return 0;
}

int ref_rmsnorm_vector(const float* x, const float* w, float* out, int n, float eps) {
  std::vector<float> X(x, x + n), W(w, w + n), O;
  rmsnorm_vector_cpu(X, W, O, eps);
  std::memcpy(out, O.data(), sizeof(float) * n);
  return 0;
}

int ref_rmsnorm_batch(const float* x, const float* w, float* out, int tokens, int n, float eps) {
  std::vector<float> X(x, x + (size_t)tokens * n), W(w, w + n), O;
  rmsnorm_batch_cpu(X, W, O, tokens, n, eps);
  std::memcpy(out, O.data(), sizeof(float) * (size_t)tokens * n);
  return 0;
}

int ref_softmax(const float* x, float* out, int n) {
  std::vector<float> X(x, x + n), O;
  softmax_vector_cpu(X, O);
  std::memcpy(out, O.data(), sizeof(float) * n);
  return 0;
}

int ref_silu(const float* x, float* out, int n) {
  std::vector<float> X(x, x + n), O(n);
  silu_cpu(X, O);
  std::memcpy(out, O.data(), sizeof(float) * n);
  return 0;
}

// freqs: [max_pos][head_dim/2][2] (cos, sin) as floats
int ref_rope_vector(float* x, int n_heads, int head_dim, int pos, const float* freqs,
                    int max_pos, int adjacent) {
  std::vector<std::pair<float, float>> f((size_t)max_pos * head_dim / 2);
  for (size_t i = 0; i < f.size(); ++i) f[i] = {freqs[2 * i], freqs[2 * i + 1]};
  std::vector<float> X(x, x + (size_t)n_heads * head_dim);
  apply_rope_vector(X, n_heads, head_dim, pos, f, max_pos, adjacent != 0);
  std::memcpy(x, X.data(), sizeof(float) * X.size());
  return 0;
}

void* ref_model_open(const char* gguf_path, int max_batch) {
  try {
    Logger::set_level(Logger::Level::OFF);
    ModelConfig init{};
    init.num_cpu_offload_layers = 0;  // CLI hint 0 = every layer on the CPU (model.cpp:187-189)
    init.use_mmap_for_gguf = true;
    auto rm = std::make_unique<RefModel>();
    rm->model = std::make_unique<TinyLlamaModel>(init, std::string(gguf_path));
    rm->cfg = rm->model->get_config();
    const ModelConfig& c = rm->cfg;
    int head_dim = c.hidden_size / c.num_attention_heads;
    rm->kv.initialize(c, c.num_hidden_layers, 0, c.max_position_embeddings,
                      c.num_key_value_heads, head_dim, max_batch > 0 ? max_batch : 1);
    return rm.release();
  } catch (const std::exception& e) {
    g_err = e.what();
    return nullptr;
  }
}

void ref_model_close(void* h) { delete static_cast<RefModel*>(h); }

// out[0..9] = hidden, ffn, n_heads, n_kv_heads, layers, vocab, max_pos, cpu_layers, eps bits, theta bits
int ref_model_config(void* h, int32_t* out) {
  const ModelConfig& c = static_cast<RefModel*>(h)->cfg;
  out[0] = c.hidden_size; out[1] = c.intermediate_size; out[2] = c.num_attention_heads;
  out[3] = c.num_key_value_heads; out[4] = c.num_hidden_layers; out[5] = c.vocab_size;
  out[6] = c.max_position_embeddings; out[7] = c.num_cpu_offload_layers;
  std::memcpy(&out[8], &c.rms_norm_eps, 4);
  std::memcpy(&out[9], &c.rope_theta, 4);
  return 0;
}

int ref_model_reset(void* h) {
  static_cast<RefModel*>(h)->kv.clear_data();
  return 0;
}

int ref_model_embedding(void* h, int token, float* out) {
  RefModel* rm = static_cast<RefModel*>(h);
  std::vector<float> e = rm->model->lookup_embedding(token);
  if (e.empty()) { g_err = "lookup_embedding returned empty"; return 1; }
  std::memcpy(out, e.data(), sizeof(float) * e.size());
  return 0;
}

// One decode step exactly as the session's loop does it (api.cpp:727, 763):
// host embedding lookup, forward(x, pos, &kv, nullptr) -> logits[V].
int ref_model_decode(void* h, int token, int pos, float* logits) {
  RefModel* rm = static_cast<RefModel*>(h);
  try {
    std::vector<float> x = rm->model->lookup_embedding(token);
    if (x.empty()) { g_err = "lookup_embedding returned empty"; return 1; }
    std::vector<float> out = rm->model->forward(x, pos, &rm->kv, nullptr);
    if ((int)out.size() != rm->cfg.vocab_size) { g_err = "forward returned wrong size"; return 2; }
    std::memcpy(logits, out.data(), sizeof(float) * out.size());
    rm->kv.seq_len = pos + 1;
    return 0;
  } catch (const std::exception& e) { g_err = e.what(); return 3; }
}

// Batched prefill as the session does it for prompts of >= 32 tokens
// (api.cpp:603-641): forward_cpu_batch over all tokens from position 0, then
// forward_cpu_logits_batch; the last row is returned. all_logits (optional)
// receives every row [n][V].
int ref_model_prefill(void* h, const int32_t* ids, int n, float* logits_last, float* all_logits) {
  RefModel* rm = static_cast<RefModel*>(h);
  try {
    const int H = rm->cfg.hidden_size, V = rm->cfg.vocab_size;
    std::vector<float> emb((size_t)n * H);
    for (int i = 0; i < n; ++i) {
      std::vector<float> e = rm->model->lookup_embedding(ids[i]);
      if (e.empty()) { g_err = "lookup_embedding returned empty"; return 1; }
      std::copy(e.begin(), e.end(), emb.begin() + (size_t)i * H);
    }
    std::vector<float> act = rm->model->forward_cpu_batch(emb, n, rm->cfg.num_cpu_offload_layers, 0, &rm->kv);
    if (act.empty()) { g_err = "forward_cpu_batch returned empty"; return 2; }
    std::vector<float> lg = rm->model->forward_cpu_logits_batch(act, n);
    if (lg.size() != (size_t)n * V) { g_err = "forward_cpu_logits_batch returned wrong size"; return 3; }
    if (logits_last) std::memcpy(logits_last, lg.data() + (size_t)(n - 1) * V, sizeof(float) * V);
    if (all_logits) std::memcpy(all_logits, lg.data(), sizeof(float) * lg.size());
    rm->kv.seq_len = n;
    return 0;
  } catch (const std::exception& e) { g_err = e.what(); return 4; }
}

// Copies the host FP32 K (which=0) or V (which=1) rows [0, n_pos) of a layer:
// layout [pos][n_kv][head_dim] (model.cpp:622-625).
int ref_model_kv(void* h, int layer, int which, int n_pos, float* out) {
  RefModel* rm = static_cast<RefModel*>(h);
  int hd = rm->cfg.hidden_size / rm->cfg.num_attention_heads;
  size_t n = (size_t)n_pos * rm->cfg.num_key_value_heads * hd;
  const std::vector<float>& src = which ? rm->kv.layers[layer].v : rm->kv.layers[layer].k;
  std::memcpy(out, src.data(), sizeof(float) * n);
  return 0;
}

}  // extern "C"
