// Synthetic GGUF model writer: seeded N(0, sigma) FP32 weights, quantized by this
// file's own quantizers into the block layouts the reference DEQUANTIZERS read
// (quantization.cpp:145-266 for Q4_K / Q6_K, quantization.cpp:1047-1052 for Q8_0).
// The reference's own quantize_* functions target a different bit layout than its
// dequantizers and are never called by its forward pass, so they are not followed.
//
// Built as libb200synth.so (host only, OpenMP). Used by the tests and bench.py to
// produce the model files both the engine and the reference CPU path load.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// ---- counter-based RNG: value i of stream s depends only on (seed, s, i) ----
inline uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// Inverse normal CDF (P. J. Acklam's rational approximation, rel. error 1.15e-9).
inline double inv_norm_cdf(double p) {
  static const double a[] = {-3.969683028665376e+01, 2.209460984245205e+02, -2.759285104469687e+02,
                             1.383577518672690e+02,  -3.066479806614716e+01, 2.506628277459239e+00};
  static const double b[] = {-5.447609879822406e+01, 1.615858368580409e+02, -1.556989798598866e+02,
                             6.680131188771972e+01,  -1.328068155288572e+01};
  static const double c[] = {-7.784894002430293e-03, -3.223964580411365e-01, -2.400758277161838e+00,
                             -2.549732539343734e+00, 4.374664141464968e+00,  2.938163982698783e+00};
  static const double d[] = {7.784695709041462e-03, 3.224671290700398e-01, 2.445134137142996e+00,
                             3.754408661907416e+00};
  const double plow = 0.02425;
  if (p < plow) {
    double q = std::sqrt(-2.0 * std::log(p));
    return (((((c[0] * q + c[1]) * q + c[2]) * q + c[3]) * q + c[4]) * q + c[5]) /
           ((((d[0] * q + d[1]) * q + d[2]) * q + d[3]) * q + 1.0);
  }
  if (p > 1.0 - plow) {
    double q = std::sqrt(-2.0 * std::log(1.0 - p));
    return -(((((c[0] * q + c[1]) * q + c[2]) * q + c[3]) * q + c[4]) * q + c[5]) /
           ((((d[0] * q + d[1]) * q + d[2]) * q + d[3]) * q + 1.0);
  }
  double q = p - 0.5, r = q * q;
  return (((((a[0] * r + a[1]) * r + a[2]) * r + a[3]) * r + a[4]) * r + a[5]) * q /
         (((((b[0] * r + b[1]) * r + b[2]) * r + b[3]) * r + b[4]) * r + 1.0);
}

inline float normal_at(uint64_t seed, uint64_t stream, uint64_t i, float sigma) {
  uint64_t h = splitmix64(splitmix64(seed ^ (stream * 0xD6E8FEB86659FD93ull)) + i);
  double u = ((double)(h >> 11) + 0.5) * (1.0 / 9007199254740992.0);  // (0,1)
  return (float)(inv_norm_cdf(u) * (double)sigma);
}

// ---- fp32 -> fp16 bits, round to nearest even ----
inline uint16_t f32_to_f16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  int32_t e = (int32_t)((x >> 23) & 0xff) - 127 + 15;
  uint32_t m = x & 0x7fffffu;
  if (((x >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00u | (m ? 0x200u : 0));
  if (e >= 31) return (uint16_t)(sign | 0x7c00u);
  if (e <= 0) {
    if (e < -10) return (uint16_t)sign;
    m |= 0x800000u;
    int shift = 14 - e;
    uint32_t half = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) half++;
    return (uint16_t)(sign | half);
  }
  uint32_t half = (uint32_t)(e << 10) | (m >> 13);
  uint32_t rem = m & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) half++;
  return (uint16_t)(sign | half);
}

inline float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1f, m = h & 0x3ffu, x;
  if (e == 0) {
    if (m == 0) x = sign;
    else {
      int s = 0;
      while (!(m & 0x400u)) { m <<= 1; ++s; }
      x = sign | ((uint32_t)(127 - 15 + 1 - s) << 23) | ((m & 0x3ffu) << 13);
    }
  } else if (e == 31) x = sign | 0x7f800000u | (m << 13);
  else x = sign | ((e - 15 + 127) << 23) | (m << 13);
  float f;
  std::memcpy(&f, &x, 4);
  return f;
}

inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// ---- quantizers (layouts: see the header comment) ----
void quant_q8_0(const float* x, uint8_t* out) {  // 34 B: fp16 d, int8 qs[32]
  float amax = 0.f;
  for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(x[i]));
  uint16_t dh = f32_to_f16(amax / 127.f);
  float d = f16_to_f32(dh);
  float id = d > 0.f ? 1.f / d : 0.f;
  std::memcpy(out, &dh, 2);
  for (int i = 0; i < 32; ++i) out[2 + i] = (uint8_t)(int8_t)clampi((int)std::lrintf(x[i] * id), -127, 127);
}

void quant_q4_k(const float* x, uint8_t* out) {  // 144 B: fp16 d, dmin; scales[12]; qs[128]
  float sc[8], mn[8];
  float max_sc = 0.f, max_mn = 0.f;
  for (int s = 0; s < 8; ++s) {
    float lo = x[32 * s], hi = x[32 * s];
    for (int i = 1; i < 32; ++i) { lo = std::min(lo, x[32 * s + i]); hi = std::max(hi, x[32 * s + i]); }
    if (lo > 0.f) lo = 0.f;  // the stored minimum is subtracted and unsigned
    sc[s] = (hi - lo) / 15.f;
    mn[s] = -lo;
    max_sc = std::max(max_sc, sc[s]);
    max_mn = std::max(max_mn, mn[s]);
  }
  uint16_t dh = f32_to_f16(max_sc / 63.f), dmh = f32_to_f16(max_mn / 63.f);
  float d = f16_to_f32(dh), dmin = f16_to_f32(dmh);
  uint8_t ls[8], lm[8];
  for (int s = 0; s < 8; ++s) {
    ls[s] = (uint8_t)clampi(d > 0.f ? (int)std::lrintf(sc[s] / d) : 0, 0, 63);
    lm[s] = (uint8_t)clampi(dmin > 0.f ? (int)std::lrintf(mn[s] / dmin) : 0, 0, 63);
  }
  std::memcpy(out, &dh, 2);
  std::memcpy(out + 2, &dmh, 2);
  uint8_t* scales = out + 4;
  std::memset(scales, 0, 12);
  for (int j = 0; j < 8; ++j) {  // inverse of get_scale_min_k4
    if (j < 4) {
      scales[j] |= ls[j] & 63;
      scales[j + 4] |= lm[j] & 63;
    } else {
      scales[j + 4] = (uint8_t)((ls[j] & 0x0F) | ((lm[j] & 0x0F) << 4));
      scales[j - 4] |= (uint8_t)((ls[j] >> 4) << 6);
      scales[j] |= (uint8_t)((lm[j] >> 4) << 6);
    }
  }
  uint8_t* qs = out + 16;
  for (int c = 0; c < 4; ++c) {
    float d1 = d * ls[2 * c], m1 = dmin * lm[2 * c], d2 = d * ls[2 * c + 1], m2 = dmin * lm[2 * c + 1];
    for (int l = 0; l < 32; ++l) {
      int q1 = d1 > 0.f ? clampi((int)std::lrintf((x[64 * c + l] + m1) / d1), 0, 15) : 0;
      int q2 = d2 > 0.f ? clampi((int)std::lrintf((x[64 * c + 32 + l] + m2) / d2), 0, 15) : 0;
      qs[32 * c + l] = (uint8_t)(q1 | (q2 << 4));
    }
  }
}

void quant_q6_k(const float* x, uint8_t* out) {  // 210 B: ql[128], qh[64], int8 scales[16], fp16 d
  float sub[16];
  float max_abs_scale = 0.f;
  for (int s = 0; s < 16; ++s) {
    float amax = 0.f;
    for (int i = 0; i < 16; ++i) amax = std::max(amax, std::fabs(x[16 * s + i]));
    sub[s] = amax / 31.f;
    max_abs_scale = std::max(max_abs_scale, sub[s]);
  }
  uint16_t dh = f32_to_f16(max_abs_scale / 127.f);
  float d = f16_to_f32(dh);
  int8_t sc[16];
  for (int s = 0; s < 16; ++s) sc[s] = (int8_t)clampi(d > 0.f ? (int)std::lrintf(sub[s] / d) : 0, -128, 127);
  uint8_t* ql = out;
  uint8_t* qh = out + 128;
  std::memset(out, 0, 192);
  std::memcpy(out + 192, sc, 16);
  std::memcpy(out + 208, &dh, 2);
  int q[256];
  for (int i = 0; i < 256; ++i) {
    float s = d * (float)sc[i / 16];
    q[i] = s != 0.f ? clampi((int)std::lrintf(x[i] / s), -32, 31) + 32 : 32;
  }
  for (int h = 0; h < 2; ++h)
    for (int l = 0; l < 32; ++l) {
      int q1 = q[128 * h + l], q2 = q[128 * h + 32 + l], q3 = q[128 * h + 64 + l], q4 = q[128 * h + 96 + l];
      ql[64 * h + l] = (uint8_t)((q1 & 15) | ((q3 & 15) << 4));
      ql[64 * h + 32 + l] = (uint8_t)((q2 & 15) | ((q4 & 15) << 4));
      qh[32 * h + l] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
    }
}

int block_elems(int t) { return t == 8 ? 32 : (t == 12 || t == 14) ? 256 : 1; }
int block_bytes(int t) { return t == 8 ? 34 : t == 12 ? 144 : t == 14 ? 210 : 4; }

void quantize_rows(int type, const float* src, int64_t n, uint8_t* dst) {
  const int be = block_elems(type), bb = block_bytes(type);
  const int64_t nb = n / be;
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < nb; ++b) {
    const float* x = src + b * be;
    uint8_t* o = dst + b * bb;
    if (type == 8) quant_q8_0(x, o);
    else if (type == 12) quant_q4_k(x, o);
    else if (type == 14) quant_q6_k(x, o);
    else std::memcpy(o, x, 4);
  }
}

struct TensorPlan {
  std::string name;
  int type;
  int64_t rows, cols;  // cols = input dim (ne0)
  int kind;            // 0 = normal weights, 1 = norm vector
  uint64_t offset, bytes;
};

void put_u32(std::vector<uint8_t>& v, uint32_t x) { v.insert(v.end(), (uint8_t*)&x, (uint8_t*)&x + 4); }
void put_u64(std::vector<uint8_t>& v, uint64_t x) { v.insert(v.end(), (uint8_t*)&x, (uint8_t*)&x + 8); }
void put_f32(std::vector<uint8_t>& v, float x) { v.insert(v.end(), (uint8_t*)&x, (uint8_t*)&x + 4); }
void put_str(std::vector<uint8_t>& v, const std::string& s) {
  put_u64(v, s.size());
  v.insert(v.end(), s.begin(), s.end());
}
void kv_u32(std::vector<uint8_t>& v, const char* k, uint32_t x) { put_str(v, k); put_u32(v, 4); put_u32(v, x); }
void kv_f32(std::vector<uint8_t>& v, const char* k, float x) { put_str(v, k); put_u32(v, 6); put_f32(v, x); }
void kv_str(std::vector<uint8_t>& v, const char* k, const char* s) { put_str(v, k); put_u32(v, 8); put_str(v, s); }

}  // namespace

extern "C" {

// Worker threads of the generator / quantizers (a launcher may have set OMP_NUM_THREADS=1 for the whole process).
void b200_synth_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

struct b200_synth_config {
  int32_t hidden, ffn, n_heads, n_kv_heads, n_layers, vocab, max_pos;
  float eps, theta;
  int32_t scheme;       // 0: every linear Q8_0; 1: Q4_K with Q6_K for attn_v, ffn_down, output; 2: every linear Q6_K; 3: every linear Q4_K
  int32_t norm_random;  // bit 0: norm weights 1 + 0.1*N(0,1) instead of 1.0 (exercises the norm-weight indexing in small tests);
                        // bit 1: token_embd is quantised like attn_q (as real checkpoints ship it) instead of F32
  uint64_t seed;
  float sigma;
};

void b200_synth_fill_normal(float* dst, int64_t n, uint64_t seed, uint64_t stream, float sigma) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) dst[i] = normal_at(seed, stream, (uint64_t)i, sigma);
}

// n must be a multiple of the type's block size; dst holds n/block_elems blocks.
int b200_synth_quantize(int ggml_type, const float* src, int64_t n, void* dst) {
  if (ggml_type != 8 && ggml_type != 12 && ggml_type != 14) return 1;
  if (n % block_elems(ggml_type)) return 2;
  quantize_rows(ggml_type, src, n, (uint8_t*)dst);
  return 0;
}

int64_t b200_synth_type_bytes(int ggml_type, int64_t n) {
  return n / block_elems(ggml_type) * block_bytes(ggml_type);
}

int b200_synth_write_gguf(const char* path, const b200_synth_config* c) {
  const int H = c->hidden, F = c->ffn, L = c->n_layers, V = c->vocab;
  const int hd = H / c->n_heads, KV = hd * c->n_kv_heads;
  int t_main, t_alt;
  switch (c->scheme) {
    case 0: t_main = t_alt = 8; break;
    case 1: t_main = 12; t_alt = 14; break;
    case 2: t_main = t_alt = 14; break;
    case 3: t_main = t_alt = 12; break;
    default: return 1;
  }
  if (H % block_elems(t_main) || F % block_elems(t_alt) || H % block_elems(t_alt)) return 2;

  std::vector<TensorPlan> plan;
  auto add = [&](const std::string& n, int type, int64_t rows, int64_t cols, int kind) {
    plan.push_back({n, type, rows, cols, kind, 0, 0});
  };
  add("token_embd.weight", (c->norm_random & 2) ? t_main : 0, V, H, 0);
  for (int l = 0; l < L; ++l) {
    std::string p = "blk." + std::to_string(l) + ".";
    add(p + "attn_norm.weight", 0, 1, H, 1);
    add(p + "attn_q.weight", t_main, H, H, 0);
    add(p + "attn_k.weight", t_main, KV, H, 0);
    add(p + "attn_v.weight", t_alt, KV, H, 0);
    add(p + "attn_output.weight", t_main, H, H, 0);
    add(p + "ffn_norm.weight", 0, 1, H, 1);
    add(p + "ffn_gate.weight", t_main, F, H, 0);
    add(p + "ffn_up.weight", t_main, F, H, 0);
    add(p + "ffn_down.weight", t_alt, H, F, 0);
  }
  add("output_norm.weight", 0, 1, H, 1);
  add("output.weight", t_alt, V, H, 0);

  uint64_t off = 0;
  for (auto& t : plan) {
    t.offset = off;
    t.bytes = (uint64_t)(t.rows * t.cols / block_elems(t.type)) * block_bytes(t.type);
    off += (t.bytes + 31) / 32 * 32;
  }

  std::vector<uint8_t> head;
  put_u32(head, 0x46554747u);  // "GGUF"
  put_u32(head, 3);
  put_u64(head, plan.size());
  put_u64(head, 11);
  kv_str(head, "general.architecture", "llama");
  kv_str(head, "general.name", "synthetic");
  kv_u32(head, "llama.embedding_length", H);
  kv_u32(head, "llama.feed_forward_length", F);
  kv_u32(head, "llama.attention.head_count", c->n_heads);
  kv_u32(head, "llama.attention.head_count_kv", c->n_kv_heads);
  kv_u32(head, "llama.block_count", L);
  kv_u32(head, "llama.context_length", c->max_pos);
  kv_f32(head, "llama.attention.layer_norm_rms_epsilon", c->eps);
  kv_f32(head, "llama.rope.freq_base", c->theta);
  kv_u32(head, "llama.vocab_size", V);
  for (auto& t : plan) {
    put_str(head, t.name);
    if (t.kind == 1) {
      put_u32(head, 1);
      put_u64(head, (uint64_t)t.cols);
    } else {
      put_u32(head, 2);
      put_u64(head, (uint64_t)t.cols);  // ne0 = input dimension
      put_u64(head, (uint64_t)t.rows);
    }
    put_u32(head, (uint32_t)t.type);
    put_u64(head, t.offset);
  }
  while (head.size() % 32) head.push_back(0);

  FILE* f = std::fopen(path, "wb");
  if (!f) return 3;
  if (std::fwrite(head.data(), 1, head.size(), f) != head.size()) { std::fclose(f); return 4; }

  const int64_t CHUNK_ELEMS = (int64_t)1 << 24;
  std::vector<float> fbuf;
  std::vector<uint8_t> qbuf;
  uint64_t written = 0;
  for (size_t ti = 0; ti < plan.size(); ++ti) {
    const TensorPlan& t = plan[ti];
    const int64_t n = t.rows * t.cols;
    const int be = block_elems(t.type), bb = block_bytes(t.type);
    for (int64_t start = 0; start < n; start += CHUNK_ELEMS) {
      const int64_t cnt = std::min(CHUNK_ELEMS, n - start);
      fbuf.resize((size_t)cnt);
      if (t.kind == 1) {
        for (int64_t i = 0; i < cnt; ++i)
          fbuf[i] = (c->norm_random & 1) ? 1.0f + normal_at(c->seed, ti + 1, (uint64_t)(start + i), 0.1f) : 1.0f;
      } else {
        const uint64_t seed = c->seed, stream = ti + 1;
        const float sigma = c->sigma;
        float* dst = fbuf.data();
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < cnt; ++i) dst[i] = normal_at(seed, stream, (uint64_t)(start + i), sigma);
      }
      const uint8_t* src_bytes;
      size_t nbytes;
      if (t.type == 0) {
        src_bytes = (const uint8_t*)fbuf.data();
        nbytes = (size_t)cnt * 4;
      } else {
        nbytes = (size_t)(cnt / be) * bb;
        qbuf.resize(nbytes);
        quantize_rows(t.type, fbuf.data(), cnt, qbuf.data());
        src_bytes = qbuf.data();
      }
      if (std::fwrite(src_bytes, 1, nbytes, f) != nbytes) { std::fclose(f); return 4; }
      written += nbytes;
    }
    static const uint8_t zeros[32] = {0};
    size_t pad = (size_t)((32 - written % 32) % 32);
    if (pad && std::fwrite(zeros, 1, pad, f) != pad) { std::fclose(f); return 4; }
    written += pad;
  }
  std::fclose(f);
  return 0;
}

}  // extern "C"
