// TEST INFRASTRUCTURE. Compile-and-link check of the reference-side adapter shown in INTEGRATION.md: the member
// functions a maintainer would add to TinyLlamaModel / KVCache (reference model.h:324-399, model.h:153-230), written
// against include/b200llama.h only. The reference's own headers are not needed: ModelConfig and the two classes are
// reduced here to the members the adapter touches. Built by tests/test_abi_cpu.py with g++ and linked against
// libb200llama.so; running it without a GPU must end in status 3 ("no CUDA device"), never in a crash.
#include <cstdio>
#include <stdexcept>
#include <string>
#include <vector>

#include "b200llama.h"

struct ModelConfig {
  int hidden_size = 0, vocab_size = 0;
  bool use_kvcache_quantization = false;
};

struct KVCache {
  int seq_len = 0;
  b200_engine* engine = nullptr;
  void clear_data() {
    seq_len = 0;
    if (engine) b200_kv_reset(engine, 0);
  }
};

class TinyLlamaModel {
 public:
  explicit TinyLlamaModel(const ModelConfig& c) : config_(c) {}
  ~TinyLlamaModel() { b200_engine_destroy(e_); }

  // TinyLlamaModel(const ModelConfig&, const std::string& gguf_path), model.cpp:154
  void b200_init(const std::string& path, bool int8_kv, int max_batch) {
    b200_model_desc ov{};
    ov.kv_dtype = int8_kv ? B200_KV_I8 : B200_KV_F32;
    ov.max_seqs = max_batch;
    ov.act_planes = 3;
    ov.tp_size = 1;
    if (b200_engine_load_gguf(path.c_str(), &ov, &e_)) throw std::runtime_error(b200_last_error());
    b200_model_desc d{};
    b200_engine_get_desc(e_, &d);
    config_.hidden_size = d.hidden_size;
    config_.vocab_size = d.vocab_size;
  }

  // std::vector<float> forward(std::vector<float>& input, int n_tokens, KVCache*, const std::vector<int>*), model.cpp:536
  std::vector<float> forward(std::vector<float>& input, int n_tokens, KVCache*, const std::vector<int>*) {
    std::vector<float> logits(config_.vocab_size);
    if (b200_forward(e_, 0, input.data(), n_tokens, logits.data())) return {};
    return logits;
  }

  // std::vector<float> lookup_embedding(int token_id), model_utils.cpp:11
  std::vector<float> lookup_embedding(int token_id) {
    std::vector<float> v(config_.hidden_size);
    if (b200_lookup_embedding(e_, token_id, v.data())) return {};
    return v;
  }

  // forward_device_batch_prefill(d_in, T, start_pos, cache, stream), model.cpp:1526 (token ids instead of embeddings)
  std::vector<float> prefill_tokens(const std::vector<int>& ids, int start_pos, int slot) {
    std::vector<float> logits(config_.vocab_size);
    if (b200_prefill(e_, slot, ids.data(), (int)ids.size(), start_pos, logits.data())) return {};
    return logits;
  }

  // forward_device_batch_generation(d_in, token_positions, original_sequence_indices, B, cache, stream), model.cpp:1863
  std::vector<std::vector<float>> decode_tokens(const std::vector<int>& toks, const std::vector<int>& token_positions,
                                                const std::vector<int>& original_sequence_indices) {
    const int B = (int)toks.size();
    std::vector<float> flat((size_t)B * config_.vocab_size);
    if (b200_decode(e_, B, toks.data(), token_positions.data(), original_sequence_indices.data(), flat.data(), nullptr)) return {};
    std::vector<std::vector<float>> out(B);
    for (int b = 0; b < B; ++b)
      out[b].assign(flat.begin() + (size_t)b * config_.vocab_size, flat.begin() + (size_t)(b + 1) * config_.vocab_size);
    return out;
  }

  b200_engine* engine() { return e_; }

 private:
  ModelConfig config_;
  b200_engine* e_ = nullptr;
};

int main(int argc, char** argv) {
  int n = -1;
  if (b200_device_count(&n)) return 10;
  ModelConfig cfg;
  TinyLlamaModel m(cfg);
  try {
    m.b200_init(argc > 1 ? argv[1] : "/nonexistent/model.gguf", true, 1);
  } catch (const std::exception& ex) {
    std::printf("init failed as expected without a model or a GPU: %s\n", ex.what());
    return n == 0 ? 0 : 1;
  }
  KVCache kv;
  kv.engine = m.engine();
  std::vector<float> x = m.lookup_embedding(1);
  std::vector<float> logits = m.forward(x, 0, &kv, nullptr);
  kv.clear_data();
  std::printf("devices %d, logits %zu\n", n, logits.size());
  return logits.empty() ? 2 : 0;
}
