// Decode attention over the on-device KV cache with split-K over context length.
//
// One CTA = (context split, query head, sequence). Every CTA appends nothing except the one that
// owns the newest position: the new token's K/V row arrives as FP32 (already rotated) from the QKV
// kernel, is quantised here when the cache is INT8 (per (position, kv head) absmax scale:
// scale = absmax/127, or 1 when absmax <= 1e-8; q = clamp(roundf(x/scale), -127, 127) — the
// arithmetic of the reference quantizer, cuda_kernels.cu:1535-1549 and 1596-1599) and written to
// the cache by the first query head of the group. Partial (max, sum, output) triples go to a
// scratch buffer; the last CTA of a head to finish (atomic ticket) merges them in split order,
// so the result does not depend on scheduling.
//
// Softmax follows the reference CPU code (model.cpp:632-663, utils.cpp:675-698):
//   s_t = (q . k_t) / sqrt(hd);  p_t = exp(s_t - max);  o = sum p_t v_t / (sum p_t + 1e-9).
//
// Cache layout (device-internal): K and V [slot][kv_head][position][head_dim], scales
// [slot][kv_head][position]. Algorithmic HBM bytes = K and V rows of positions 0..pos-1 of the
// heads read, plus their scales.
#pragma once
#include "common.cuh"

namespace b200 {

struct AttnParams {
  const float* q;        // [batch][q_stride]
  const float* kv_new;   // [batch][kvn_stride]: K rows (n_kv*hd) then V rows
  int q_stride, kvn_stride;
  void* k_cache;         // this layer's cache base
  void* v_cache;
  float* k_scale;
  float* v_scale;
  const int* positions;  // [batch] position of the new token
  const int* slots;      // [batch] KV slot of each sequence
  int nq, nkv, hd, max_ctx, nsplit;
  float* part_o;         // [batch][nq][nsplit][hd]
  float* part_ml;        // [batch][nq][nsplit][2]
  int* tickets;          // [batch][nq], zero between launches
  float* out;            // [batch][out_stride]
  int out_stride;
  float att_scale;
};

__device__ __forceinline__ float i8_at(uint32_t w, int i) { return (float)(int)(int8_t)((w >> (8 * i)) & 0xFF); }

// KV_I8: int8 rows, 16 elements per lane per load; else FP32 rows, 4 elements per lane.
template <bool KV_I8>
__global__ void __launch_bounds__(128) attn_decode_kernel(const AttnParams prm) {
  extern __shared__ __align__(16) float sm[];
  // lets a dependent launch that opted in start its independent prologue (weight prefetch) now;
  // it still waits for this grid to finish before touching anything produced here
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int hd = prm.hd, G = prm.nq / prm.nkv, kvh = h / G;
  const int pos = prm.positions[b], slot = prm.slots[b];
  const int T = pos + 1;
  int chunk = (T + prm.nsplit - 1) / prm.nsplit;
  chunk = (chunk + 31) & ~31;
  const int t0 = split * chunk, t1 = min(T, t0 + chunk);

  float* q_s = sm;               // [hd]
  float* kn_s = q_s + hd;        // [hd] new K row as the cache will hold it (dequantised when INT8)
  float* vn_s = kn_s + hd;       // [hd]
  float* o_s = vn_s + hd;        // [nwarps][hd]
  float* sc_s = o_s + nwarps * hd;  // [cap]
  __shared__ float red[8];
  __shared__ int last_flag;

  for (int d = tid; d < hd; d += blockDim.x) q_s[d] = prm.q[(size_t)b * prm.q_stride + h * hd + d];

  const size_t head_row0 = ((size_t)slot * prm.nkv + kvh) * prm.max_ctx;  // row index of position 0
  const bool owns_new = (pos >= t0 && pos < t1);
  if (owns_new && warp < 2) {  // warp 0: K row, warp 1: V row
    const float* src = prm.kv_new + (size_t)b * prm.kvn_stride + (warp == 0 ? 0 : prm.nkv * hd) + kvh * hd;
    float* dst_s = warp == 0 ? kn_s : vn_s;
    if (KV_I8) {
      float amax = 0.f;
      for (int d = lane; d < hd; d += 32) amax = fmaxf(amax, fabsf(src[d]));
      amax = warp_max(amax);
      const float scale = ((double)amax > 1e-8) ? __fdiv_rn(amax, 127.0f) : 1.0f;
      int8_t* crow = reinterpret_cast<int8_t*>(warp == 0 ? prm.k_cache : prm.v_cache) + (head_row0 + pos) * hd;
      for (int d = lane; d < hd; d += 32) {
        float r = roundf(__fdiv_rn(src[d], scale));
        r = fmaxf(-127.0f, fminf(127.0f, r));
        const int8_t qv = (int8_t)r;
        dst_s[d] = __fmul_rn((float)qv, scale);
        if (h % G == 0) crow[d] = qv;
      }
      if (h % G == 0 && lane == 0) (warp == 0 ? prm.k_scale : prm.v_scale)[head_row0 + pos] = scale;
    } else {
      float* crow = reinterpret_cast<float*>(warp == 0 ? prm.k_cache : prm.v_cache) + (head_row0 + pos) * hd;
      for (int d = lane; d < hd; d += 32) {
        const float v = src[d];
        dst_s[d] = v;
        if (h % G == 0) crow[d] = v;
      }
    }
  }
  __syncthreads();

  constexpr int EPL = KV_I8 ? 16 : 4;   // elements per lane per row
  const int lpp = hd / EPL;             // lanes per position (<= 32)
  const int ppw = 32 / lpp;             // positions per warp iteration
  const int gl = lane % lpp, gi = lane / lpp;
  float qr[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) qr[i] = q_s[gl * EPL + i];

  // ---- scores ----
  for (int tb = t0 + warp * ppw; tb < t1; tb += nwarps * ppw) {
    const int t = tb + gi;
    float dot = 0.f;
    if (t < t1) {
      if (t == pos) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) dot = fmaf(qr[i], kn_s[gl * EPL + i], dot);
      } else if (KV_I8) {
        const uint4 kw = ldg128(reinterpret_cast<const int8_t*>(prm.k_cache) + (head_row0 + t) * hd + gl * 16);
        const uint32_t w4[4] = {kw.x, kw.y, kw.z, kw.w};
#pragma unroll
        for (int i = 0; i < 16; ++i) dot = fmaf(qr[i], i8_at(w4[i >> 2], i & 3), dot);
      } else {
        const float4 kf = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(prm.k_cache) + (head_row0 + t) * hd + gl * 4));
        dot = fmaf(qr[0], kf.x, fmaf(qr[1], kf.y, fmaf(qr[2], kf.z, qr[3] * kf.w)));
      }
    }
    for (int o = lpp >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (t < t1 && gl == 0) {
      if (KV_I8 && t != pos) dot *= prm.k_scale[head_row0 + t];
      sc_s[t - t0] = dot * prm.att_scale;
    }
  }
  __syncthreads();

  // ---- max and exp-sum over this split ----
  const int n = max(t1 - t0, 0);
  float m = -INFINITY;
  for (int i = tid; i < n; i += blockDim.x) m = fmaxf(m, sc_s[i]);
  m = warp_max(m);
  if (lane == 0) red[warp] = m;
  __syncthreads();
  m = red[0];
  for (int w = 1; w < nwarps; ++w) m = fmaxf(m, red[w]);
  __syncthreads();
  float l = 0.f;
  for (int i = tid; i < n; i += blockDim.x) {
    const float p = expf(sc_s[i] - m);
    sc_s[i] = p;
    l += p;
  }
  l = warp_sum(l);
  if (lane == 0) red[warp] = l;
  __syncthreads();
  l = 0.f;
  for (int w = 0; w < nwarps; ++w) l += red[w];

  // ---- weighted sum of V ----
  float acc[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) acc[i] = 0.f;
  for (int tb = t0 + warp * ppw; tb < t1; tb += nwarps * ppw) {
    const int t = tb + gi;
    if (t < t1) {
      const float p = sc_s[t - t0];
      if (t == pos) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) acc[i] = fmaf(p, vn_s[gl * EPL + i], acc[i]);
      } else if (KV_I8) {
        const uint4 vw = ldg128(reinterpret_cast<const int8_t*>(prm.v_cache) + (head_row0 + t) * hd + gl * 16);
        const uint32_t w4[4] = {vw.x, vw.y, vw.z, vw.w};
        const float ps = p * prm.v_scale[head_row0 + t];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = fmaf(ps, i8_at(w4[i >> 2], i & 3), acc[i]);
      } else {
        const float4 vf = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(prm.v_cache) + (head_row0 + t) * hd + gl * 4));
        acc[0] = fmaf(p, vf.x, acc[0]); acc[1] = fmaf(p, vf.y, acc[1]);
        acc[2] = fmaf(p, vf.z, acc[2]); acc[3] = fmaf(p, vf.w, acc[3]);
      }
    }
  }
  // fold the position groups of a warp, then the warps
#pragma unroll
  for (int i = 0; i < EPL; ++i)
    for (int o = lpp; o < 32; o <<= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
  if (gi == 0) {
#pragma unroll
    for (int i = 0; i < EPL; ++i) o_s[warp * hd + gl * EPL + i] = acc[i];
  }
  __syncthreads();
  const size_t pbase = ((size_t)b * prm.nq + h) * prm.nsplit;
  for (int d = tid; d < hd; d += blockDim.x) {
    float o = 0.f;
    for (int w = 0; w < nwarps; ++w) o += o_s[w * hd + d];
    prm.part_o[(pbase + split) * hd + d] = o;
  }
  if (tid == 0) {
    prm.part_ml[(pbase + split) * 2 + 0] = m;
    prm.part_ml[(pbase + split) * 2 + 1] = l;
  }

  // ---- merge: the last CTA of this (sequence, head) combines all splits ----
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&prm.tickets[b * prm.nq + h], 1);
    last_flag = (old == prm.nsplit - 1);
  }
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  float M = -INFINITY;
  for (int s = 0; s < prm.nsplit; ++s) M = fmaxf(M, __ldcg(&prm.part_ml[(pbase + s) * 2]));
  float L = 0.f;
  for (int s = 0; s < prm.nsplit; ++s) {
    const float ms = __ldcg(&prm.part_ml[(pbase + s) * 2]), ls = __ldcg(&prm.part_ml[(pbase + s) * 2 + 1]);
    if (ls > 0.f) L += ls * expf(ms - M);
  }
  const float inv = 1.0f / (L + 1e-9f);
  for (int d = tid; d < hd; d += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < prm.nsplit; ++s) {
      const float ms = __ldcg(&prm.part_ml[(pbase + s) * 2]), ls = __ldcg(&prm.part_ml[(pbase + s) * 2 + 1]);
      if (ls > 0.f) o = fmaf(expf(ms - M), __ldcg(&prm.part_o[(pbase + s) * hd + d]), o);
    }
    prm.out[(size_t)b * prm.out_stride + h * hd + d] = o * inv;
  }
  if (tid == 0) prm.tickets[b * prm.nq + h] = 0;
}

inline size_t attn_smem_bytes(int hd, int max_ctx, int nsplit, int nwarps) {
  const int cap = ((max_ctx + nsplit - 1) / nsplit + 31) & ~31;
  return sizeof(float) * (size_t)(3 * hd + nwarps * hd + cap);
}

}  // namespace b200
