/* b200llama — C ABI of the B200 (sm_100a) decode engine for Llama-family models stored as
 * GGUF Q8_0 / Q4_K / Q6_K blocks.
 *
 * The reference (tinyllama.cpp) has no FFI boundary for its forward pass; the closest seam is
 * the C++ member-function surface of TinyLlamaModel / KVCache (model.h:324-399, model.h:153-230)
 * and the raw-pointer op layer below it (cuda_kernels.h:104-643). Every entry point here names
 * the reference interface it stands in for. All functions return 0 on success and a non-zero
 * status otherwise; nothing throws across this boundary (the reference throws
 * std::runtime_error from gpuErrchk, cuda_kernels.h:66-82, or returns an empty vector,
 * model.cpp:828-839); the text of the last failure on the calling thread is available from
 * b200_last_error(). Host pointers are plain memory owned by the caller. One engine is bound to
 * one CUDA device and must be driven from one host thread at a time, like the reference's model.
 */
#ifndef B200LLAMA_H
#define B200LLAMA_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* ggml tensor types accepted (ggml_types.h:21-42) */
enum { B200_TYPE_F32 = 0, B200_TYPE_Q8_0 = 8, B200_TYPE_Q4_K = 12, B200_TYPE_Q6_K = 14 };
/* KV cache element types: FP32 (KVCacheLayer::k_dev_fp32, model.h:137-138) or INT8 with one FP32
 * scale per (position, kv head) (k_dev_quantized / k_dev_scales, model.h:140-143). */
enum { B200_KV_F32 = 0, B200_KV_I8 = 1 };

typedef struct b200_engine b200_engine;

/* Mirrors the fields of ModelConfig (model.h:80-120) the forward pass reads, plus engine options. */
typedef struct b200_model_desc {
  int32_t hidden_size;
  int32_t intermediate_size;
  int32_t num_attention_heads;
  int32_t num_key_value_heads;
  int32_t num_hidden_layers;
  int32_t vocab_size;
  int32_t max_position_embeddings; /* RoPE table length (gpu_initialization.cpp:48-58) */
  float rms_norm_eps;
  float rope_theta;
  int32_t kv_dtype;   /* B200_KV_F32 | B200_KV_I8 (ModelConfig::use_kvcache_quantization) */
  int32_t max_seqs;   /* KV slots = KVCache::max_batch_size (model.h:168) */
  int32_t max_ctx;    /* positions held per slot; 0 = max_position_embeddings */
  int32_t act_planes; /* integer byte-planes the activations are split into for the GEMV: 2 or 3 (0 = 3) */
  int32_t device;     /* CUDA device ordinal */
  int32_t tp_rank;    /* tensor-parallel rank and world size (1 = single GPU) */
  int32_t tp_size;
  uint8_t nccl_id[128]; /* ncclUniqueId shared by all ranks when tp_size > 1 (see b200_nccl_unique_id) */
} b200_model_desc;

const char* b200_last_error(void);
int b200_device_count(int* count);

/* ---- engine life cycle: replaces TinyLlamaModel(config, gguf_path) (model.cpp:154),
 * map_gguf_weights (weight_management.cpp:677), initialize_gpu_and_rope
 * (gpu_initialization.cpp:15) and KVCache::initialize (kv_cache.cpp:10). Linear weights stay in
 * their packed block form on the device; nothing is expanded to FP32. ---- */
int b200_engine_create(const b200_model_desc* desc, b200_engine** out);
/* One GGUF tensor by its GGUF name ("blk.3.attn_q.weight", "token_embd.weight", ...). rows x cols
 * with cols = the input dimension (GGUF ne0). host_data holds the tensor exactly as stored in the file. */
int b200_engine_upload_tensor(b200_engine* e, const char* gguf_name, int ggml_type, const void* host_data,
                              size_t bytes, int64_t rows, int64_t cols);
/* Checks that every tensor arrived, builds the RoPE table and the launch graphs. */
int b200_engine_finalize(b200_engine* e);
/* Parses a GGUF file (gguf_parser.cpp:123) and does create + upload + finalize. desc_overrides may be
 * NULL; when given, only kv_dtype, max_seqs, max_ctx, act_planes, device and the tp_* fields are read. */
int b200_engine_load_gguf(const char* path, const b200_model_desc* desc_overrides, b200_engine** out);
int b200_engine_get_desc(const b200_engine* e, b200_model_desc* out);
int b200_engine_destroy(b200_engine* e);

/* KVCache::clear_data (model.h:188-203) for one sequence slot. */
int b200_kv_reset(b200_engine* e, int seq_slot);

/* TinyLlamaModel::lookup_embedding (model_utils.cpp:11-182): one row of token_embd as FP32. */
int b200_lookup_embedding(b200_engine* e, int token_id, float* host_out /* [hidden] */);

/* TinyLlamaModel::forward(input, n_tokens, kv_cache, mask) (model.cpp:536-807) and
 * forward_device(x_input_dev, pos, cache) (model.cpp:810-1090): one hidden-state vector in, the
 * logits of the token at position pos of slot seq_slot out. host_x [hidden] is overwritten with
 * the final residual stream like the reference's in-place `input`. */
int b200_forward(b200_engine* e, int seq_slot, float* host_x, int pos, float* host_logits /* [vocab] */);

/* Prompt ingestion: forward_cpu_batch + forward_cpu_logits_batch as driven by
 * TinyLlamaSession::generate (api.cpp:603-641) / forward_device_batch_prefill (model.cpp:1526).
 * Tokens occupy positions start_pos .. start_pos+n-1 of the slot. host_logits_last may be NULL. */
int b200_prefill(b200_engine* e, int seq_slot, const int32_t* token_ids, int n, int start_pos,
                 float* host_logits_last /* [vocab] */);

/* Sequence-aware prompt ingestion of several sequences in one call (the batch prefill of
 * TinyLlamaSession::generate_batch, api.cpp:1144-1421, with attention_batch_cpu_sequence_aware,
 * cpu_attention.cpp:203-325): the prompts are laid end to end (token_ids holds lens[0] + lens[1] + ... ids) and cut
 * into chunks of 512 tokens, so that short prompts share a chunk and its weight traffic; every token carries its own
 * position and KV slot, and each token attends only to its own sequence's rows. Always the tensor-core path.
 * Sequence s occupies positions start_pos[s] .. start_pos[s]+lens[s]-1 of slot slots[s] (slots distinct).
 * host_logits_last [n_seqs][vocab] (logits after each prompt's last token) may be NULL. Same kernels and the same
 * per-token arithmetic as one b200_prefill call per sequence on the tensor-core path (n >= 16). */
int b200_prefill_batch(b200_engine* e, int n_seqs, const int32_t* slots, const int32_t* token_ids, const int32_t* lens,
                       const int32_t* start_pos, float* host_logits_last);
/* The chunk plan b200_prefill_batch follows for prompts of these lengths (host arithmetic only, no GPU needed): one
 * record per run of tokens, out[i] = {chunk, first row in the chunk, tokens, position of the first token, index of the
 * sequence whose prompt ends with this run or -1}. chunk = tokens per chunk (the engine uses 512). */
int b200_prefill_plan(int n_seqs, const int32_t* lens, int chunk, int32_t* out /* [max_runs][5] */, int max_runs, int* n_runs);

/* One decode step for `batch` independent sequences: forward_device_batch_generation
 * (model.cpp:1863) with the embedding lookup of the session loop (api.cpp:727) folded in.
 * host_logits [batch][vocab] and argmax_out [batch] are each optional (NULL). argmax follows
 * the greedy rule of the sampler: first maximum (api.cpp:134-136). */
int b200_decode(b200_engine* e, int batch, const int32_t* token_ids, const int32_t* positions,
                const int32_t* seq_slots, float* host_logits, int32_t* argmax_out);

/* Greedy generation loop kept on the device (the session loop api.cpp:696-803 with temperature 0
 * and no repetition penalty): `steps` decode steps for `batch` sequences starting from
 * first_tokens at start_positions; each step's argmax feeds the next step without leaving HBM.
 * out_tokens [steps][batch] receives the sampled ids; elapsed_ms (optional) the CUDA-event time
 * of the loop. */
int b200_generate_greedy(b200_engine* e, int batch, const int32_t* first_tokens,
                         const int32_t* start_positions, const int32_t* seq_slots, int steps,
                         int32_t* out_tokens, float* elapsed_ms);

/* The same loop with the reference's repetition penalty applied on the device before every argmax
 * (apply_repetition_penalty, api.cpp:86-97, called from TinyLlamaSession::generate, api.cpp:678, 768; default 1.3):
 * every occurrence of a token id among the last 64 GENERATED ids turns its logit l into l / penalty when l > 0 and
 * l * penalty otherwise (an id that occurs twice is penalised twice); each chosen id then joins that window.
 * history holds the ids each sequence has generated so far, end to end (history_lens[b] of them for sequence b;
 * normally just first_tokens[b], the id sampled after the prompt, which the reference has already pushed);
 * both may be NULL for an empty history. Batches below the tensor-core switch point (16) only. */
int b200_generate_greedy_penalized(b200_engine* e, int batch, const int32_t* first_tokens, const int32_t* start_positions,
                                   const int32_t* seq_slots, int steps, float repetition_penalty, const int32_t* history,
                                   const int32_t* history_lens, int32_t* out_tokens, float* elapsed_ms);

/* ---- op level, for parity tests (cuda_kernels.h op layer) ---- */
/* Exact dequantizers: dequantize_q8_0_block / dequantize_q4_k_m / dequantize_q6_k
 * (quantization.cpp:1047-1052, 171-221, 223-266); bit-exact, no fused multiply-add. */
int b200_dequant(int ggml_type, const void* host_blocks, size_t n_blocks, float* host_out);
/* y[b][r] = dot(W[r,:], x[b,:]) on the packed blocks: the fused kernel that replaces
 * matvec_f32_f32_cuda (cuda_kernels.cu:291-314) / matvec_*_f32_vector_cpu (utils.cpp:293-397). */
int b200_matvec(int ggml_type, const void* host_blocks, int64_t rows, int64_t cols, const float* host_x,
                int batch, int act_planes, float* host_y);
/* Y[t][r] = dot(W[r,:], X[t,:]) for n_tokens rows of X on the tensor cores (tcgen05, fp16 operands, FP32
 * accumulation in tensor memory): the batch >= 16 / prompt path that replaces matmul_*_f32_batch_cpu
 * (utils.cpp:730-782, 890-1044) and smart_gemm_batch_cuda (model.cpp:2141-2249). host_x [n_tokens][cols],
 * host_y [n_tokens][rows]. Agrees with the FP32 dot to about 1e-3 of the largest output. */
int b200_matmul(int ggml_type, const void* host_blocks, int64_t rows, int64_t cols, const float* host_x, int n_tokens,
                float* host_y);
/* rmsnorm_vector_cpu (utils.cpp:648-673) / rmsnorm_vector_cuda (cuda_kernels.cu:209-253, 2499) as the decode path
 * computes it: the prologue of the matvec kernel (FP32 sum of squares, f = 1/sqrt(mean + max(eps, 1e-5)), out =
 * x*f*w) followed by its 24-bit block quantisation; host_out is the vector the matvec then multiplies
 * (within 2^-23 of the block's largest magnitude of the exact normalised value). n a multiple of 256. */
int b200_rmsnorm(const float* host_x, const float* host_w, int n, float eps, float* host_out);
/* rmsnorm_batch_cpu (utils.cpp:613-646: eps as given) as the prompt / batch >= 16 path computes it: one block per
 * token, output rounded to fp16 (the operand type of the tensor-core matmul), returned as floats. */
int b200_rmsnorm_batch(const float* host_x, const float* host_w, int n_tokens, int n, float eps, float* host_out);
/* One decode-step launch of the attention input, as TinyLlamaModel::forward does it (model.cpp:589-631): RMSNorm of
 * x, the q / k / v projections (packed blocks of the given types, [hidden][hidden] and [n_kv*hd][hidden]) and RoPE
 * on q and k at position pos (apply_rope_vector, utils.cpp:428-489, adjacent pairs; table as
 * gpu_initialization.cpp:48-58). host_norm_w may be NULL (no normalisation). Outputs q [hidden], k, v [n_kv*hd]. */
int b200_fused_qkv_rope(int type_q, const void* wq, int type_k, const void* wk, int type_v, const void* wv, int hidden,
                        int n_heads, int n_kv_heads, const float* host_x, const float* host_norm_w, float eps, int pos,
                        float rope_theta, int planes, float* q_out, float* k_out, float* v_out);
/* One decode-step launch of the MLP input (model.cpp:716-735): RMSNorm, gate and up projections ([ffn][hidden] each,
 * same block type) and SwiGLU, out[i] = (g * 1/(1+exp(-g))) * u (silu_cpu, utils.cpp:700-707). */
int b200_fused_gate_up_swiglu(int ggml_type, const void* wgate, const void* wup, int ffn, int hidden,
                              const float* host_x, const float* host_norm_w, float eps, int planes, float* host_out);
/* Decode attention of one new token over a cache of n_ctx earlier positions (attention_cuda,
 * cuda_kernels.cu:1078 / 2523; INT8 form: quantizer of cuda_kernels.cu:1535-1606 with a softmax
 * attention). q [n_heads][hd]; k_new, v_new [n_kv][hd] (already rotated); k_cache, v_cache
 * [n_ctx][n_kv][hd] FP32 (quantized on upload when kv_dtype is I8). out [n_heads][hd]. */
int b200_attention_decode(const float* q, const float* k_new, const float* v_new, const float* k_cache,
                          const float* v_cache, int n_ctx, int n_heads, int n_kv_heads, int head_dim,
                          int kv_dtype, int n_splits, float* out);

/* Causal attention of the last n_tokens positions of one sequence of n_ctx positions: the prompt form
 * (attention_batch_cpu, cpu_attention.cpp:91-201; attention_batch_prefill_cuda, cuda_kernels.cu:1710, 2055).
 * q [n_tokens][n_heads][hd] (rotated); k_rows, v_rows [n_ctx][n_kv][hd] FP32, rows of the n_tokens
 * included (quantized on upload when kv_dtype is I8); out [n_tokens][n_heads][hd]. head_dim 64 or 128.
 * fp16 tensor-core products with FP32 accumulation: agrees with the FP32 form to about 1e-3. */
int b200_attention_prefill(const float* q, const float* k_rows, const float* v_rows, int n_ctx, int n_tokens,
                           int n_heads, int n_kv_heads, int head_dim, int kv_dtype, float* out);

/* No counterpart in the reference. Decode attention for callers that must not allocate device
 * memory at the moment of the call (memory handed out once at start-up by an external pool the library
 * does not know, allocator frozen after initialisation, a latency budget that excludes cudaMalloc). All pointers are DEVICE pointers owned by the
 * caller: q [n_heads][hd]; kv_new = new K rows then new V rows [2][n_kv][hd] (already rotated);
 * k_cache / v_cache [n_kv][max_ctx][hd] (FP32, or int8 with k_scale / v_scale [n_kv][max_ctx]);
 * position = one int, the index of the new token (rows 0..position-1 of the caches are read, row
 * `position` is written); out [n_heads][hd]. The split-K scratch is a fixed array inside the library
 * (about 1 MiB per GPU, held until the process exits): n_heads * n_splits <= 2048, n_heads <= 512,
 * n_splits <= 64, head_dim in {16, 32, 64, 128}, anything larger is refused with status 2 and a message. The
 * host cannot see *position: the kernel checks it, and a value outside [0, max_ctx) makes the call read and
 * append nothing and fill `out` with NaN. The first call on each device looks up that array's address and
 * raises the kernel's shared-memory limit (both once per device ordinal); make that call outside any stream
 * capture. Calls share the scratch, so two calls whose kernels overlap on the GPU
 * (different streams) race; calls on one stream are safe. The launch is asynchronous on `stream`
 * (a cudaStream_t, may be NULL). */
int b200_attention_decode_noalloc(const float* d_q, const float* d_kv_new, void* d_k_cache, void* d_v_cache,
                                  float* d_k_scale, float* d_v_scale, const int* d_position, int n_heads,
                                  int n_kv_heads, int head_dim, int max_ctx, int kv_dtype, int n_splits,
                                  float* d_out, void* stream);

/* Timing and counters for the benchmark harness. */
int b200_engine_stats(const b200_engine* e, int64_t* kernel_launches_per_step, int64_t* weight_bytes,
                      int64_t* kv_bytes_per_position);
/* Repeats one kernel of the decode step alone (0 = the largest GEMV of a layer) `iters` times over
 * distinct layers' weights and returns its mean CUDA-event duration and algorithmic bytes. */
int b200_engine_time_kernel(b200_engine* e, int which, int iters, float* mean_us, int64_t* bytes_per_launch);

/* Step trace (no counterpart in the reference, which has no timers besides total wall time, api.cpp:825-831).
 * An engine created while B200_TRACE=1 is set in the environment gives every matvec and attention launch
 * of a step a record of eight device timestamps (GPU global timer, ns), written by the first thread of the
 * launch's first CTA: 0 kernel entry, 1 dependency wait over, 2 attention items done, 3 grid barrier passed,
 * 4 input vector held, 5 prologue done, 6 first tile computed, 7 that CTA's end (launches without an attention
 * phase stamp 1-3 together). This call waits for the engine's stream and returns the records of the most recent
 * step in launch order ([n][8]; launches that do not stamp, e.g. the embedding gather, stay zero). */
int b200_engine_read_trace(b200_engine* e, uint64_t* out, int max_records, int* n_records);

/* ---- tensor parallelism inside one node (no counterpart in the reference, whose MPI coordinator,
 * distributed_coordinator.cpp, only routes whole requests). One engine per GPU/process with
 * tp_rank/tp_size set and the same nccl_id; every rank uploads the WHOLE tensors (or loads the same
 * file) and keeps its shard: attn_q/k/v, ffn_gate/up and output by rows, attn_output and ffn_down by
 * 256-element blocks of the input dimension; two all-reduces per layer plus a gather of the logits.
 * All ranks must make the same calls with the same arguments. ---- */
/* Self-test of the failure path (no counterpart in the reference): launches a matvec as the consumer of a two-rank
 * exchange whose packets are never sent, with a probe limit of 64 instead of about a second. Every poll runs out, the
 * kernel raises the error word and returns; the call then answers status 4 (what b200_decode and the other engine
 * calls answer when a peer has gone away). No GPU fault is involved and the context stays usable. Status 1 means
 * that the kernel failed to report the missing exchange. */
int b200_selftest_exchange_timeout(void);
/* Fills 128 bytes with a fresh ncclUniqueId (rank 0 calls it and shares the bytes). */
int b200_nccl_unique_id(uint8_t* out128);
/* The contiguous share [begin, end) of `units` that rank tp_rank of tp_size owns (used for the FFN blocks). */
int b200_tp_share(int64_t units, int tp_size, int tp_rank, int64_t* begin, int64_t* end);

#ifdef __cplusplus
}
#endif
#endif
