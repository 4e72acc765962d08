/* TEST INFRASTRUCTURE — CPU restatement of the reference algorithm for the per-token
 * transformer forward over GGUF K-quant weights. Only tests, the smoke check and the
 * CPU-baseline leg of the benchmark may load this; the product library never does.
 *
 * Parity pin: every function here is checked against the reference's own CPU code
 * (compiled unmodified into oracle/_ref/libref_cpu.so) by tests/test_oracle_pin.py and
 * against the committed fixtures in tests/golden/ that were generated from it.
 * The INT8 KV-cache mode has no CPU counterpart in the reference; it is a restatement
 * of the reference's GPU quantizer arithmetic combined with its CPU softmax attention
 * ("restated oracle"), and is pinned only on the quantizer arithmetic.
 */
#ifndef B200_ORACLE_H
#define B200_ORACLE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

enum { ORC_F32 = 0, ORC_Q8_0 = 8, ORC_Q4_K = 12, ORC_Q6_K = 14 };

float orc_fp16_to_fp32(uint16_t h, int is_scale_field);
int orc_dequant(int ggml_type, const void* blocks, size_t n_blocks, float* out);
void orc_matvec_f32(const float* w, const float* x, float* y, int64_t rows, int64_t cols);
void orc_rmsnorm_vector(const float* x, const float* w, float* out, int n, float eps);
void orc_rmsnorm_batch(const float* x, const float* w, float* out, int tokens, int n, float eps);
void orc_softmax(const float* x, float* out, int n);
void orc_silu(const float* x, float* out, int n);
void orc_rope_table(float theta, int head_dim, int max_pos, float* table /* [max_pos][hd/2][2] */);
void orc_rope_vector(float* x, int n_heads, int head_dim, int pos, const float* table, int max_pos);
void orc_kv_quantize_i8(const float* x, int n, int8_t* q, float* scale);
void orc_attention_decode(const float* q, const float* kc, const float* vc, int T, int nq, int nkv, int hd,
                          int kv_int8, float* out);

typedef struct orc_model orc_model;
orc_model* orc_model_create(int hidden, int ffn, int n_heads, int n_kv_heads, int n_layers, int vocab,
                            int max_pos, float eps, float theta, int kv_int8, int max_seqs);
void orc_model_destroy(orc_model* m);
/* Dequantizes (or copies, for F32) one GGUF tensor into the model. rows x cols, cols = input dim. */
int orc_model_set_tensor(orc_model* m, const char* gguf_name, int ggml_type, const void* data,
                         int64_t rows, int64_t cols);
void orc_model_reset(orc_model* m, int seq);
/* One token through every layer at position pos of sequence slot seq; logits[V]. */
int orc_model_decode(orc_model* m, int seq, int token, int pos, float* logits);
/* n prompt tokens from position 0 with the batch expressions; logits of the last token. */
int orc_model_prefill(orc_model* m, int seq, const int32_t* ids, int n, float* logits_last);
/* Debug taps of the last decode call: hidden state after each layer [L][H]. */
const float* orc_model_layer_trace(orc_model* m);

#ifdef __cplusplus
}
#endif
#endif
