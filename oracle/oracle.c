/* TEST INFRASTRUCTURE — see oracle.h. Plain-C restatement of the reference CPU path.
 * Compile with -ffp-contract=off and without -march=native / fast-math (oracle/Makefile)
 * so that every float expression rounds exactly as the reference's x86-64 build does.
 * Each function cites the reference file:line it follows.
 */
#include "oracle.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

/* quantization.cpp:47-90 — IEEE half -> float, subnormals normalised; when the value is a
 * GGUF scale field (Q8_0 only, quantization.cpp:1048) a finite negative becomes positive. */
float orc_fp16_to_fp32(uint16_t h, int is_scale_field) {
  uint32_t sign = (h >> 15) & 1u, e = (h >> 10) & 0x1fu, m = h & 0x3ffu, x;
  if (e == 0) {
    if (m == 0) {
      x = sign << 31;
    } else {
      e = 1;
      while ((m & 0x400u) == 0) { m <<= 1; e--; }
      m &= ~0x400u;
      x = (sign << 31) | ((e - 15 + 127) << 23) | (m << 13);
    }
  } else if (e == 0x1f) {
    x = (sign << 31) | (0xffu << 23) | (m << 13);
  } else {
    x = (sign << 31) | ((e - 15 + 127) << 23) | (m << 13);
  }
  float f;
  memcpy(&f, &x, 4);
  if (is_scale_field && f < 0.0f && !(isnan(f) || isinf(f))) f = fabsf(f);
  return f;
}

/* quantization.cpp:1047-1052 */
static void dequant_q8_0(const uint8_t* b, float* out) {
  uint16_t dh;
  memcpy(&dh, b, 2);
  const float d = orc_fp16_to_fp32(dh, 1);
  const int8_t* qs = (const int8_t*)(b + 2);
  for (int i = 0; i < 32; ++i) out[i] = d * (float)qs[i];
}

/* quantization.cpp:145-155 */
static void scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* mn) {
  if (j < 4) {
    *sc = q[j] & 63;
    *mn = q[j + 4] & 63;
  } else {
    *sc = (uint8_t)((q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4));
    *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

/* quantization.cpp:171-221 — y = (d*sc)*q - (dmin*m), each operation rounded separately */
static void dequant_q4_k(const uint8_t* b, float* out) {
  uint16_t dh, mh;
  memcpy(&dh, b, 2);
  memcpy(&mh, b + 2, 2);
  const float d = orc_fp16_to_fp32(dh, 0), dmin = orc_fp16_to_fp32(mh, 0);
  const uint8_t* scales = b + 4;
  const uint8_t* qs = b + 16;
  for (int c = 0; c < 4; ++c) {
    uint8_t sc1, m1, sc2, m2;
    scale_min_k4(2 * c, scales, &sc1, &m1);
    scale_min_k4(2 * c + 1, scales, &sc2, &m2);
    const float d1 = d * (float)sc1, mf1 = dmin * (float)m1;
    const float d2 = d * (float)sc2, mf2 = dmin * (float)m2;
    for (int l = 0; l < 32; ++l) out[64 * c + l] = d1 * (float)(qs[32 * c + l] & 0x0F) - mf1;
    for (int l = 0; l < 32; ++l) out[64 * c + 32 + l] = d2 * (float)(qs[32 * c + l] >> 4) - mf2;
  }
}

/* quantization.cpp:223-266 — y = (d*sc)*q with q in [-32, 31] */
static void dequant_q6_k(const uint8_t* b, float* out) {
  uint16_t dh;
  memcpy(&dh, b + 208, 2);
  const float d = orc_fp16_to_fp32(dh, 0);
  for (int h = 0; h < 2; ++h) {
    const uint8_t* ql = b + 64 * h;
    const uint8_t* qh = b + 128 + 32 * h;
    const int8_t* sc = (const int8_t*)(b + 192) + 8 * h;
    float* y = out + 128 * h;
    for (int l = 0; l < 32; ++l) {
      const int is = l / 16;
      const int8_t q1 = (int8_t)((ql[l] & 0x0F) | (((qh[l] >> 0) & 3) << 4)) - 32;
      const int8_t q2 = (int8_t)((ql[l + 32] & 0x0F) | (((qh[l] >> 2) & 3) << 4)) - 32;
      const int8_t q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
      const int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
      y[l] = d * sc[is + 0] * q1;
      y[l + 32] = d * sc[is + 2] * q2;
      y[l + 64] = d * sc[is + 4] * q3;
      y[l + 96] = d * sc[is + 6] * q4;
    }
  }
}

/* quantization.cpp:1054-1223 (the whole-tensor loops; single pass over blocks) */
int orc_dequant(int t, const void* blocks, size_t n, float* out) {
  const uint8_t* b = (const uint8_t*)blocks;
  if (t == ORC_Q8_0) {
    for (size_t i = 0; i < n; ++i) dequant_q8_0(b + i * 34, out + i * 32);
  } else if (t == ORC_Q4_K) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) dequant_q4_k(b + i * 144, out + i * 256);
  } else if (t == ORC_Q6_K) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) dequant_q6_k(b + i * 210, out + i * 256);
  } else {
    return 1;
  }
  return 0;
}

/* utils.cpp:349-397 — Kahan-compensated double accumulation, cast to float at the end.
 * matmul_f32_f32_batch_cpu (utils.cpp:730-782) is the same dot per (token, row). */
void orc_matvec_f32(const float* w, const float* x, float* y, int64_t rows, int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* wr = w + r * cols;
    double sum = 0.0, comp = 0.0;
    for (int64_t c = 0; c < cols; ++c) {
      double term = (double)wr[c] * (double)x[c];
      double yk = term - comp;
      double t = sum + yk;
      comp = (t - sum) - yk;
      sum = t;
    }
    y[r] = (float)sum;
  }
}

/* utils.cpp:648-673 — eps is max(eps, 1e-5) in the vector form */
void orc_rmsnorm_vector(const float* x, const float* w, float* out, int n, float eps) {
  double ssq = 0.0;
  for (int i = 0; i < n; ++i) ssq += (double)x[i] * (double)x[i];
  ssq /= n;
  const float e = eps > 1e-5f ? eps : 1e-5f;
  const float f = 1.0f / sqrtf((float)ssq + e);
  for (int i = 0; i < n; ++i) out[i] = x[i] * f * w[i];
}

/* utils.cpp:613-646 — plain eps in the batch form */
void orc_rmsnorm_batch(const float* x, const float* w, float* out, int tokens, int n, float eps) {
  for (int t = 0; t < tokens; ++t) {
    const float* xt = x + (size_t)t * n;
    float* ot = out + (size_t)t * n;
    double ssq = 0.0;
    for (int i = 0; i < n; ++i) ssq += (double)xt[i] * (double)xt[i];
    const double mean = ssq / n;
    const float f = 1.0f / sqrtf((float)mean + eps);
    for (int i = 0; i < n; ++i) ot[i] = xt[i] * f * w[i];
  }
}

/* utils.cpp:675-698 */
void orc_softmax(const float* x, float* out, int n) {
  if (n <= 0) return;
  float mx = x[0];
  for (int i = 1; i < n; ++i)
    if (x[i] > mx) mx = x[i];
  float sum = 0.0f;
  for (int i = 0; i < n; ++i) {
    out[i] = expf(x[i] - mx);
    sum += out[i];
  }
  const float inv = 1.0f / (sum + 1e-9f);
  for (int i = 0; i < n; ++i) out[i] *= inv;
}

/* utils.cpp:700-707 */
void orc_silu(const float* x, float* out, int n) {
  for (int i = 0; i < n; ++i) {
    float s = 1.0f / (1.0f + expf(-x[i]));
    out[i] = x[i] * s;
  }
}

/* gpu_initialization.cpp:48-58 */
void orc_rope_table(float theta, int head_dim, int max_pos, float* table) {
  for (int pos = 0; pos < max_pos; ++pos)
    for (int i = 0; i < head_dim; i += 2) {
      float freq = powf(theta, -((float)i) / head_dim);
      float angle = pos * freq;
      size_t idx = ((size_t)pos * head_dim / 2) + (size_t)(i / 2);
      table[2 * idx] = cosf(angle);
      table[2 * idx + 1] = sinf(angle);
    }
}

/* utils.cpp:428-489 with adjacent pairing (the GGUF case, model.cpp:609) */
void orc_rope_vector(float* x, int n_heads, int head_dim, int pos, const float* table, int max_pos) {
  if (pos < 0 || pos >= max_pos) return;
  const int half = head_dim / 2;
  for (int h = 0; h < n_heads; ++h)
    for (int i = 0; i < half; ++i) {
      const float c = table[2 * ((size_t)pos * half + i)], s = table[2 * ((size_t)pos * half + i) + 1];
      float* p = x + (size_t)h * head_dim + 2 * i;
      const float x0 = p[0], x1 = p[1];
      p[0] = x0 * c - x1 * s;
      p[1] = x0 * s + x1 * c;
    }
}

/* cuda_kernels.cu:1494-1549, 1596-1599 — absmax over the vector, scale = absmax/127 (1.0
 * when absmax <= 1e-8), q = clamp(roundf(x / scale), -127, 127). */
void orc_kv_quantize_i8(const float* x, int n, int8_t* q, float* scale) {
  float amax = 0.0f;
  for (int i = 0; i < n; ++i) amax = fmaxf(amax, fabsf(x[i]));
  const float s = (amax > 1e-8) ? (amax / 127.0f) : 1.0f;
  *scale = s;
  for (int i = 0; i < n; ++i) {
    float v = roundf(x[i] / s);
    q[i] = (int8_t)fmaxf(-127.0f, fminf(127.0f, v));
  }
}


/* Standalone form of the attention step of forward_token (model.cpp:632-663): one new token
 * attending to rows 0..T-1 of kc / vc ([T][n_kv][hd], the last row being the new token).
 * With kv_int8 every row goes through orc_kv_quantize_i8 and back first ("restated oracle"). */
void orc_attention_decode(const float* q, const float* kc, const float* vc, int T, int nq, int nkv, int hd,
                          int kv_int8, float* out) {
  const int KV = nkv * hd;
  float* k = (float*)malloc(sizeof(float) * (size_t)T * KV);
  float* v = (float*)malloc(sizeof(float) * (size_t)T * KV);
  memcpy(k, kc, sizeof(float) * (size_t)T * KV);
  memcpy(v, vc, sizeof(float) * (size_t)T * KV);
  if (kv_int8) {
    int8_t* tmp = (int8_t*)malloc((size_t)hd);
    for (size_t r = 0; r < (size_t)T * nkv; ++r) {
      float sc;
      orc_kv_quantize_i8(k + r * hd, hd, tmp, &sc);
      for (int d = 0; d < hd; ++d) k[r * hd + d] = (float)tmp[d] * sc;
      orc_kv_quantize_i8(v + r * hd, hd, tmp, &sc);
      for (int d = 0; d < hd; ++d) v[r * hd + d] = (float)tmp[d] * sc;
    }
    free(tmp);
  }
  float* scores = (float*)malloc(sizeof(float) * (size_t)T);
  const float att_scale = 1.0f / sqrtf((float)hd);
  for (int h = 0; h < nq; ++h) {
    const float* qh = q + h * hd;
    const int kvh = h / (nq / nkv);
    for (int t = 0; t < T; ++t) {
      const float* kr = k + ((size_t)t * nkv + kvh) * hd;
      float s = 0.0f;
      for (int d = 0; d < hd; ++d) s += qh[d] * kr[d];
      scores[t] = s * att_scale;
    }
    orc_softmax(scores, scores, T);
    float* o = out + h * hd;
    for (int d = 0; d < hd; ++d) o[d] = 0.0f;
    for (int t = 0; t < T; ++t) {
      const float* vr = v + ((size_t)t * nkv + kvh) * hd;
      for (int d = 0; d < hd; ++d) o[d] += scores[t] * vr[d];
    }
  }
  free(k); free(v); free(scores);
}

/* ------------------------------------------------------------------------------------ */
typedef struct {
  float *attn_norm, *ffn_norm, *wq, *wk, *wv, *wo, *wgate, *wup, *wdown;
} orc_layer;

struct orc_model {
  int H, F, nq, nkv, L, V, max_pos, hd, kv_int8, max_seqs;
  float eps, theta;
  float* embd;
  float* out_norm;
  float* out_w;
  orc_layer* layers;
  float* rope;
  /* KV cache (model.h:132-144): [seq][pos][n_kv][hd] per layer */
  float** k;
  float** v;
  int8_t** kq;
  int8_t** vq;
  float** ks;
  float** vs;
  float* trace;
};

orc_model* orc_model_create(int hidden, int ffn, int n_heads, int n_kv_heads, int n_layers, int vocab,
                            int max_pos, float eps, float theta, int kv_int8, int max_seqs) {
  orc_model* m = (orc_model*)calloc(1, sizeof(orc_model));
  m->H = hidden; m->F = ffn; m->nq = n_heads; m->nkv = n_kv_heads; m->L = n_layers; m->V = vocab;
  m->max_pos = max_pos; m->eps = eps; m->theta = theta; m->hd = hidden / n_heads;
  m->kv_int8 = kv_int8; m->max_seqs = max_seqs > 0 ? max_seqs : 1;
  m->layers = (orc_layer*)calloc((size_t)n_layers, sizeof(orc_layer));
  m->rope = (float*)malloc(sizeof(float) * (size_t)max_pos * m->hd);
  orc_rope_table(theta, m->hd, max_pos, m->rope);
  const size_t per = (size_t)m->max_seqs * max_pos * n_kv_heads * m->hd;
  const size_t per_s = (size_t)m->max_seqs * max_pos * n_kv_heads;
  m->k = (float**)calloc((size_t)n_layers, sizeof(float*));
  m->v = (float**)calloc((size_t)n_layers, sizeof(float*));
  m->kq = (int8_t**)calloc((size_t)n_layers, sizeof(int8_t*));
  m->vq = (int8_t**)calloc((size_t)n_layers, sizeof(int8_t*));
  m->ks = (float**)calloc((size_t)n_layers, sizeof(float*));
  m->vs = (float**)calloc((size_t)n_layers, sizeof(float*));
  for (int l = 0; l < n_layers; ++l) {
    if (kv_int8) {
      m->kq[l] = (int8_t*)calloc(per, 1);
      m->vq[l] = (int8_t*)calloc(per, 1);
      m->ks[l] = (float*)calloc(per_s, sizeof(float));
      m->vs[l] = (float*)calloc(per_s, sizeof(float));
    } else {
      m->k[l] = (float*)calloc(per, sizeof(float));
      m->v[l] = (float*)calloc(per, sizeof(float));
    }
  }
  m->trace = (float*)calloc((size_t)n_layers * hidden, sizeof(float));
  return m;
}

void orc_model_destroy(orc_model* m) {
  if (!m) return;
  for (int l = 0; l < m->L; ++l) {
    orc_layer* w = &m->layers[l];
    free(w->attn_norm); free(w->ffn_norm); free(w->wq); free(w->wk); free(w->wv); free(w->wo);
    free(w->wgate); free(w->wup); free(w->wdown);
    free(m->k[l]); free(m->v[l]); free(m->kq[l]); free(m->vq[l]); free(m->ks[l]); free(m->vs[l]);
  }
  free(m->k); free(m->v); free(m->kq); free(m->vq); free(m->ks); free(m->vs);
  free(m->layers); free(m->rope); free(m->embd); free(m->out_norm); free(m->out_w); free(m->trace);
  free(m);
}

/* weight_management.cpp:677-973 (tensor names) + the lazy dequantization of
 * weight_management.cpp:27-196, done once here: the values are the same every time. */
int orc_model_set_tensor(orc_model* m, const char* name, int type, const void* data, int64_t rows, int64_t cols) {
  const size_t n = (size_t)rows * (size_t)cols;
  float* f = (float*)malloc(n * sizeof(float));
  if (!f) return 2;
  if (type == ORC_F32) memcpy(f, data, n * sizeof(float));
  else {
    const int be = type == ORC_Q8_0 ? 32 : 256;
    if (orc_dequant(type, data, n / be, f)) { free(f); return 3; }
  }
  float** slot = NULL;
  int layer = -1;
  char field[64];
  if (!strcmp(name, "token_embd.weight")) slot = &m->embd;
  else if (!strcmp(name, "output_norm.weight")) slot = &m->out_norm;
  else if (!strcmp(name, "output.weight")) slot = &m->out_w;
  else if (sscanf(name, "blk.%d.%63s", &layer, field) == 2 && layer >= 0 && layer < m->L) {
    orc_layer* w = &m->layers[layer];
    if (!strcmp(field, "attn_norm.weight")) slot = &w->attn_norm;
    else if (!strcmp(field, "ffn_norm.weight")) slot = &w->ffn_norm;
    else if (!strcmp(field, "attn_q.weight")) slot = &w->wq;
    else if (!strcmp(field, "attn_k.weight")) slot = &w->wk;
    else if (!strcmp(field, "attn_v.weight")) slot = &w->wv;
    else if (!strcmp(field, "attn_output.weight")) slot = &w->wo;
    else if (!strcmp(field, "ffn_gate.weight")) slot = &w->wgate;
    else if (!strcmp(field, "ffn_up.weight")) slot = &w->wup;
    else if (!strcmp(field, "ffn_down.weight")) slot = &w->wdown;
  }
  if (!slot) { free(f); return 1; }
  free(*slot);
  *slot = f;
  return 0;
}

void orc_model_reset(orc_model* m, int seq) {
  const size_t per = (size_t)m->max_pos * m->nkv * m->hd, per_s = (size_t)m->max_pos * m->nkv;
  for (int l = 0; l < m->L; ++l) {
    if (m->kv_int8) {
      memset(m->kq[l] + seq * per, 0, per);
      memset(m->vq[l] + seq * per, 0, per);
      memset(m->ks[l] + seq * per_s, 0, per_s * sizeof(float));
      memset(m->vs[l] + seq * per_s, 0, per_s * sizeof(float));
    } else {
      memset(m->k[l] + seq * per, 0, per * sizeof(float));
      memset(m->v[l] + seq * per, 0, per * sizeof(float));
    }
  }
}

const float* orc_model_layer_trace(orc_model* m) { return m->trace; }

/* One token through all layers. batch_expr = 0 follows TinyLlamaModel::forward
 * (model.cpp:536-807); batch_expr = 1 follows CPUBatchProcessor::forward_cpu_batch
 * (cpu_batch_processor.cpp:11-281), which differs per token only in the RMSNorm epsilon
 * rule and the rounding of the SwiGLU expression; its attention
 * (cpu_attention.cpp:91-201) is the same causal softmax over cache rows 0..pos. */
static int forward_token(orc_model* m, int seq, float* x, int pos, int batch_expr, float* logits) {
  const int H = m->H, F = m->F, nq = m->nq, nkv = m->nkv, hd = m->hd, KV = nkv * hd;
  if (pos < 0 || pos >= m->max_pos) return 1;
  float* xn = (float*)malloc(sizeof(float) * H);
  float* q = (float*)malloc(sizeof(float) * H);
  float* kvec = (float*)malloc(sizeof(float) * KV);
  float* vvec = (float*)malloc(sizeof(float) * KV);
  float* att = (float*)malloc(sizeof(float) * H);
  float* proj = (float*)malloc(sizeof(float) * H);
  float* gate = (float*)malloc(sizeof(float) * F);
  float* up = (float*)malloc(sizeof(float) * F);
  float* act = (float*)malloc(sizeof(float) * F);
  float* scores = (float*)malloc(sizeof(float) * (pos + 1));
  float* kd = (float*)malloc(sizeof(float) * hd);
  const float att_scale = 1.0f / sqrtf((float)hd);
  const size_t seq_off = (size_t)seq * m->max_pos;

  for (int l = 0; l < m->L; ++l) {
    const orc_layer* w = &m->layers[l];
    if (batch_expr) orc_rmsnorm_batch(x, w->attn_norm, xn, 1, H, m->eps);
    else orc_rmsnorm_vector(x, w->attn_norm, xn, H, m->eps);
    orc_matvec_f32(w->wq, xn, q, H, H);
    orc_matvec_f32(w->wk, xn, kvec, KV, H);
    orc_matvec_f32(w->wv, xn, vvec, KV, H);
    orc_rope_vector(q, nq, hd, pos, m->rope, m->max_pos);
    orc_rope_vector(kvec, nkv, hd, pos, m->rope, m->max_pos);
    /* KV write at pos (model.cpp:622-625); INT8 mode quantizes per (pos, kv head) */
    if (m->kv_int8) {
      for (int h = 0; h < nkv; ++h) {
        size_t row = (seq_off + pos) * nkv + h;
        orc_kv_quantize_i8(kvec + h * hd, hd, m->kq[l] + row * hd, &m->ks[l][row]);
        orc_kv_quantize_i8(vvec + h * hd, hd, m->vq[l] + row * hd, &m->vs[l][row]);
      }
    } else {
      memcpy(m->k[l] + (seq_off + pos) * KV, kvec, sizeof(float) * KV);
      memcpy(m->v[l] + (seq_off + pos) * KV, vvec, sizeof(float) * KV);
    }
    /* attention (model.cpp:632-663): float dot in index order, scale, softmax, t-major PV */
    for (int h = 0; h < nq; ++h) {
      const float* qh = q + h * hd;
      const int kvh = h / (nq / nkv);
      for (int t = 0; t <= pos; ++t) {
        const size_t row = (seq_off + t) * nkv + kvh;
        float s = 0.0f;
        if (m->kv_int8) {
          const int8_t* kq = m->kq[l] + row * hd;
          const float sc = m->ks[l][row];
          for (int d = 0; d < hd; ++d) s += qh[d] * ((float)kq[d] * sc); /* cuda_kernels.cu:1560 */
        } else {
          const float* kr = m->k[l] + row * hd;
          for (int d = 0; d < hd; ++d) s += qh[d] * kr[d];
        }
        scores[t] = s * att_scale;
      }
      orc_softmax(scores, scores, pos + 1);
      float* o = att + h * hd;
      for (int d = 0; d < hd; ++d) o[d] = 0.0f;
      for (int t = 0; t <= pos; ++t) {
        const size_t row = (seq_off + t) * nkv + kvh;
        if (m->kv_int8) {
          const int8_t* vq = m->vq[l] + row * hd;
          const float sc = m->vs[l][row];
          for (int d = 0; d < hd; ++d) o[d] += scores[t] * ((float)vq[d] * sc);
        } else {
          const float* vr = m->v[l] + row * hd;
          for (int d = 0; d < hd; ++d) o[d] += scores[t] * vr[d];
        }
      }
    }
    orc_matvec_f32(w->wo, att, proj, H, H);
    for (int i = 0; i < H; ++i) x[i] = x[i] + proj[i]; /* model.cpp:678 */
    if (batch_expr) orc_rmsnorm_batch(x, w->ffn_norm, xn, 1, H, m->eps);
    else orc_rmsnorm_vector(x, w->ffn_norm, xn, H, m->eps);
    orc_matvec_f32(w->wgate, xn, gate, F, H);
    orc_matvec_f32(w->wup, xn, up, F, H);
    if (batch_expr) { /* cpu_batch_processor.cpp:252-256 */
      for (int i = 0; i < F; ++i) {
        float g = gate[i];
        float sg = g / (1.0f + expf(-g));
        act[i] = sg * up[i];
      }
    } else { /* model.cpp:734-735 */
      orc_silu(gate, act, F);
      for (int i = 0; i < F; ++i) act[i] = act[i] * up[i];
    }
    orc_matvec_f32(w->wdown, act, proj, H, F);
    for (int i = 0; i < H; ++i) x[i] = x[i] + proj[i]; /* model.cpp:751 */
    memcpy(m->trace + (size_t)l * H, x, sizeof(float) * H);
  }
  if (logits) { /* model.cpp:780-803 / model.cpp:1094-1156 */
    if (batch_expr) orc_rmsnorm_batch(x, m->out_norm, xn, 1, H, m->eps);
    else orc_rmsnorm_vector(x, m->out_norm, xn, H, m->eps);
    orc_matvec_f32(m->out_w, xn, logits, m->V, H);
  }
  free(xn); free(q); free(kvec); free(vvec); free(att); free(proj); free(gate); free(up); free(act);
  free(scores); free(kd);
  return 0;
}

int orc_model_decode(orc_model* m, int seq, int token, int pos, float* logits) {
  if (token < 0 || token >= m->V || seq < 0 || seq >= m->max_seqs) return 2;
  float* x = (float*)malloc(sizeof(float) * m->H);
  memcpy(x, m->embd + (size_t)token * m->H, sizeof(float) * m->H); /* model_utils.cpp:11-182, F32 table */
  int rc = forward_token(m, seq, x, pos, 0, logits);
  free(x);
  return rc;
}

int orc_model_prefill(orc_model* m, int seq, const int32_t* ids, int n, float* logits_last) {
  if (seq < 0 || seq >= m->max_seqs) return 2;
  float* x = (float*)malloc(sizeof(float) * m->H);
  int rc = 0;
  for (int i = 0; i < n && !rc; ++i) {
    if (ids[i] < 0 || ids[i] >= m->V) { rc = 2; break; }
    memcpy(x, m->embd + (size_t)ids[i] * m->H, sizeof(float) * m->H);
    rc = forward_token(m, seq, x, i, 1, (i == n - 1) ? logits_last : NULL);
  }
  free(x);
  return rc;
}
