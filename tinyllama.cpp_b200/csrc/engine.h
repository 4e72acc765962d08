// Engine state behind the C ABI: device-resident packed weights, KV cache, step buffers and the
// captured launch graphs of one decode step.
#pragma once
#include <map>
#include <string>
#include <vector>

#include "../../include/b200llama.h"
#include "common.cuh"

namespace b200 {

struct DevTensor {
  int type = -1;
  int64_t rows = 0, cols = 0;  // logical shape
  uint8_t* base = nullptr;     // packed types: stage images (see gemv.cuh); F32: the data
  size_t bytes = 0;            // packed bytes as in the file (the algorithmic byte count)
  int64_t img_rows = 0;        // rows the image holds data for (2 x rows for the gate+up image)
  int tiles = 0;               // image tiles of 16*R rows
  int halves = 0;              // gate+up image: which halves have arrived (bit 0 gate, bit 1 up)
  bool present() const { return base != nullptr; }
  const float* f32() const { return reinterpret_cast<const float*>(base); }
};

struct LayerW {
  DevTensor attn_norm, wq, wk, wv, wo, ffn_norm, wgu /* gate and up, interleaved by 8 rows */, wdown;
  void* k_cache = nullptr;
  void* v_cache = nullptr;
  float* k_scale = nullptr;
  float* v_scale = nullptr;
};

struct StepGraph {
  cudaGraphExec_t exec = nullptr;
  int nsplit = 1;
  int head_ctas = 0;
  int launches = 0;
};

}  // namespace b200

struct b200_engine {
  b200_model_desc desc{};
  // H and V are the full model widths; Hq, nq, nkv, KVD, F and Vl are this rank's shares under
  // tensor parallelism (equal to the full values on a single GPU)
  int H = 0, F = 0, nq = 0, nkv = 0, L = 0, V = 0, hd = 0, KVD = 0, max_ctx = 0, max_seqs = 0, P = 3;
  int Hq = 0, Vl = 0, F_full = 0;
  int tp_rank = 0, tp_size = 1;
  int f_blk0 = 0, f_blk1 = 0;  // this rank's range of 256-element blocks of the FFN dimension
  void* nccl_comm = nullptr;
  float* d_partial = nullptr;   // [max_seqs][H] partial sums awaiting the all-reduce
  float* d_logits_local = nullptr;
  int num_sms = 148;
  bool use_pdl = true;
  int* d_error = nullptr;       // device alias of h_error
  int* h_error = nullptr;       // host-mapped word a kernel sets when a bounded wait gives up
  // one-shot all-reduce over peer memory (tensor parallelism): an IPC-shared region per rank holding the
  // exchange slots [2][tp][max_seqs][H] of 8-byte packets {value, exchange number}
  bool use_peer = false;
  void* xregion = nullptr;
  void* peer_region[8] = {nullptr};  // the same region of every rank, mapped here (own rank: xregion)
  unsigned* d_epoch = nullptr;
  float* d_h2 = nullptr;             // second residual-stream buffer (the consumer of an exchange writes the other one)
  unsigned long long* d_trace = nullptr;  // B200_TRACE=1: one 8-slot timestamp record per launch of a step
  int trace_cap = 0;
  int last_launches = 0;
  bool finalized = false;
  cudaStream_t stream = nullptr;
  std::vector<b200::LayerW> layers;
  b200::DevTensor tok_embd, out_norm, out_w;
  float* rope = nullptr;
  // step buffers
  int* d_tokens = nullptr;
  int* d_positions = nullptr;
  int* d_slots = nullptr;
  int* d_argmax = nullptr;
  int* d_step = nullptr;
  int* d_forced = nullptr;
  int* d_forced_steps = nullptr;
  int forced_cap = 0;
  int* d_log = nullptr;
  int log_cap = 0;
  // repetition penalty of the device-resident greedy loop: window ring, running count, occurrence counts, value
  int* d_pen_ring = nullptr;
  int* d_pen_count = nullptr;
  uint8_t* d_pen_counts = nullptr;  // [max_seqs][pen_stride]: occurrences of each vocabulary index in the window
  float* d_pen_value = nullptr;
  int pen_stride = 0;
  float* d_h = nullptr;
  float* d_q = nullptr;
  float* d_kvnew = nullptr;
  float* d_attn = nullptr;
  float* d_act = nullptr;
  void* d_x16 = nullptr;        // fp16 activations of the tensor-core path, [max_seqs][max(H, F)]
  // prompt ingestion through the tensor-core matmul: buffers for one chunk of tokens, allocated at the first use
  int pf_cap = 0;
  int* pf_ints = nullptr;       // tokens | positions | slots, pf_cap each
  float* pf_h = nullptr;
  float* pf_q = nullptr;
  float* pf_kvnew = nullptr;
  float* pf_attn = nullptr;
  float* pf_act = nullptr;
  void* pf_x16 = nullptr;
  float* pf_partial = nullptr;   // tensor parallel: partial [chunk][H] outputs awaiting the all-reduce
  float* pf_part_o = nullptr;
  float* pf_part_ml = nullptr;
  int* pf_tickets = nullptr;
  float* d_tc_part = nullptr;   // split-K partial outputs of the tensor-core matmul, [8][512][H], allocated when the engine is finalized
  int gemm_min_batch = 16;      // batches at least this large take the tensor-core matmul (B200_GEMM_MIN_BATCH)
  float* d_logits = nullptr;
  float* d_amax_val = nullptr;
  int* d_amax_idx = nullptr;
  int amax_cap = 0;
  float* d_part_o = nullptr;
  float* d_part_ml = nullptr;
  int* d_tickets = nullptr;
  size_t part_cap = 0;  // floats in d_part_o
  float* h_logits_pinned = nullptr;
  int* h_ints_pinned = nullptr;
  std::map<int, b200::StepGraph> graphs;
  int64_t weight_bytes = 0;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  std::vector<void*> allocations;
  // Load-time staging: host bytes reach the device through two pinned buffers (the copy of one chunk
  // overlaps the host-side memcpy of the next) into device scratch that is reused from tensor to tensor;
  // everything here is released when the engine is finalized.
  struct Staging {
    uint8_t* pinned[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    size_t chunk = 0;
    int next = 0;
    uint8_t* scratch[3] = {nullptr, nullptr, nullptr};  // raw blocks, regrouped units, fp16 scale plane
    size_t scratch_cap[3] = {0, 0, 0};
  } stage;
};
