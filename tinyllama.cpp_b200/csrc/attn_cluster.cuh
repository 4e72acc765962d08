// Decode attention, low-latency form: the context splits of one (sequence, head) are the CTAs of
// one thread-block cluster and meet through distributed shared memory, so nothing goes through
// global scratch, fences or atomics. At batch 1 the kernel is a chain of dependent round trips, not
// a bandwidth problem (a 7B layer holds ~8 MB of INT8 K/V at 1k context), so the design removes
// round trips:
//   * every warp runs an online softmax over its own positions (running max, rescaled sum and
//     output), with the K and V rows of a batch of positions requested together up front; the
//     scores never pass through shared memory and there is no block-wide pass per phase;
//   * the warps of a CTA are merged once in shared memory, the CTAs of a cluster once through
//     DSMEM by the cluster's first CTA, both in a fixed order (deterministic).
// Arithmetic is that of attn.cuh (reference model.cpp:632-663, utils.cpp:675-698; INT8 quantizer
// cuda_kernels.cu:1535-1549, 1596-1599) up to the reassociation the online form implies:
//   o = sum_t exp(s_t - M) v_t / (sum_t exp(s_t - M) + 1e-9),  s_t = (q . k_t) / sqrt(hd).
// The split that owns the newest position appends it to the cache (first query head of a group).
#pragma once
#include <cooperative_groups.h>

#include "attn.cuh"

namespace b200 {

constexpr int ATTC_THREADS = 256;
constexpr int ATTC_WARPS = ATTC_THREADS / 32;
constexpr int ATTC_MAX_CLUSTER = 8;

// floats of dynamic shared memory: q, new K row, new V row, per-warp (o[hd], m, l), CTA (o[hd], m, l)
__host__ __device__ __forceinline__ size_t attc_smem_floats(int hd) { return (size_t)3 * hd + (size_t)(ATTC_WARPS + 1) * (hd + 2); }

template <bool KV_I8, int HD>
__global__ void __launch_bounds__(ATTC_THREADS, 2) attn_cluster_kernel(const AttnParams prm) {
  namespace cg = cooperative_groups;
  extern __shared__ __align__(16) float sm[];
  cg::cluster_group cluster = cg::this_cluster();
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  unsigned long long* rec = (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) ? prm.trace : nullptr;
  trace_stamp(rec, 0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x, nsplit = gridDim.x, h = blockIdx.y, b = blockIdx.z;
  const int hd = HD ? HD : prm.hd, G = prm.nq / prm.nkv, kvh = h / G;
  float* q_s = sm;
  float* kn_s = q_s + hd;
  float* vn_s = kn_s + hd;
  float* wres = vn_s + hd;                       // [ATTC_WARPS][hd + 2]
  float* cres = wres + ATTC_WARPS * (hd + 2);    // [hd + 2]

  // q and the new K/V rows belong to the previous kernel until here
  asm volatile("griddepcontrol.wait;" ::: "memory");
  trace_stamp(rec, 1);
  trace_stamp(rec, 5);
  trace_stamp(rec, 6);
  trace_stamp(rec, 7);
  trace_stamp(rec, 4);
  const int pos = prm.positions[b], slot = prm.slots[b];
  const int T = pos + 1;
  constexpr int EPL = KV_I8 ? 16 : 4;  // elements per lane per row (one 16-byte load)
  constexpr int U = ATTN_UNROLL;
  const int lpp = hd / EPL;            // lanes per position
  const int ppw = 32 / lpp;            // positions per warp per load
  const int PB = ppw * U;              // positions per warp per batch
  int chunk = (T + nsplit - 1) / nsplit;
  chunk = (chunk + PB - 1) / PB * PB;
  const int t0 = split * chunk, t1 = min(T, t0 + chunk);
  const int gl = lane % lpp, gi = lane / lpp;
  const size_t head_row0 = ((size_t)slot * prm.nkv + kvh) * prm.max_ctx;
  const size_t row_bytes = (size_t)hd * (KV_I8 ? 1 : 4);
  const uint8_t* kbase = reinterpret_cast<const uint8_t*>(prm.k_cache) + head_row0 * row_bytes + gl * 16;
  const uint8_t* vbase = reinterpret_cast<const uint8_t*>(prm.v_cache) + head_row0 * row_bytes + gl * 16;

  // first batch of this warp: K, V and their scales are requested before anything else is touched
  uint4 kw[U], vw[U];
  float ks[U], vs[U];
  auto request = [&](int tb) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = tb + u * ppw + gi;
      kw[u] = make_uint4(0u, 0u, 0u, 0u);
      vw[u] = make_uint4(0u, 0u, 0u, 0u);
      ks[u] = 1.f;
      vs[u] = 1.f;
      if (t < t1 && t != pos) {
        kw[u] = ldg128(kbase + (size_t)t * row_bytes);
        vw[u] = ldg128(vbase + (size_t)t * row_bytes);
        if (KV_I8) {
          ks[u] = __ldg(&prm.k_scale[head_row0 + t]);
          vs[u] = __ldg(&prm.v_scale[head_row0 + t]);
        }
      }
    }
  };
  int tb = t0 + warp * PB;
  if (tb < t1) request(tb);

  for (int d = tid; d < hd; d += ATTC_THREADS) q_s[d] = prm.q[(size_t)b * prm.q_stride + h * hd + d];
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
  float qr[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) qr[i] = q_s[gl * EPL + i];

  // ---- online softmax over this warp's positions ----
  float m_run = -INFINITY, l_run = 0.f;  // l_run and acc are this lane's share (its own positions, its own dims)
  float acc[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) acc[i] = 0.f;
  for (; tb < t1; tb += ATTC_WARPS * PB) {
    float sc[U];
    float bmax = -INFINITY;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = tb + u * ppw + gi;
      float dot = 0.f;
      if (t == pos) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) dot = fmaf(qr[i], kn_s[gl * EPL + i], dot);
      } else if (KV_I8) {
        const uint32_t w4[4] = {kw[u].x, kw[u].y, kw[u].z, kw[u].w};
#pragma unroll
        for (int i = 0; i < 16; ++i) dot = fmaf(qr[i & (EPL - 1)], i8_at(w4[i >> 2], i & 3), dot);
        dot *= ks[u];
      } else {
        dot = fmaf(qr[0], __uint_as_float(kw[u].x), fmaf(qr[1], __uint_as_float(kw[u].y),
                   fmaf(qr[2], __uint_as_float(kw[u].z), qr[3 & (EPL - 1)] * __uint_as_float(kw[u].w))));
      }
      for (int o = lpp >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      sc[u] = t < t1 ? dot * prm.att_scale : -INFINITY;
      bmax = fmaxf(bmax, sc[u]);
    }
    for (int o = lpp; o < 32; o <<= 1) bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, o));
    const float m_new = fmaxf(m_run, bmax);  // finite: the batch holds at least one position
    const float corr = expf(m_run - m_new);  // 0 on the first batch
    l_run *= corr;
#pragma unroll
    for (int i = 0; i < EPL; ++i) acc[i] *= corr;
    m_run = m_new;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = tb + u * ppw + gi;
      if (t >= t1) continue;
      const float p = expf(sc[u] - m_new);
      l_run += p;
      if (t == pos) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) acc[i] = fmaf(p, vn_s[gl * EPL + i], acc[i]);
      } else if (KV_I8) {
        const float pv = p * vs[u];
        const uint32_t w4[4] = {vw[u].x, vw[u].y, vw[u].z, vw[u].w};
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i & (EPL - 1)] = fmaf(pv, i8_at(w4[i >> 2], i & 3), acc[i & (EPL - 1)]);
      } else {
        acc[0] = fmaf(p, __uint_as_float(vw[u].x), acc[0]);
        acc[1] = fmaf(p, __uint_as_float(vw[u].y), acc[1]);
        acc[2] = fmaf(p, __uint_as_float(vw[u].z), acc[2]);
        acc[3 & (EPL - 1)] = fmaf(p, __uint_as_float(vw[u].w), acc[3 & (EPL - 1)]);
      }
    }
    if (tb + ATTC_WARPS * PB < t1) request(tb + ATTC_WARPS * PB);
  }
  // fold the position groups of the warp (l: every lane of a group counted the same positions, so
  // one lane per group contributes), then park the warp's result
  float l_w = gl == 0 ? l_run : 0.f;
  for (int o = 16; o > 0; o >>= 1) l_w += __shfl_xor_sync(0xffffffffu, l_w, o);
#pragma unroll
  for (int i = 0; i < EPL; ++i)
    for (int o = lpp; o < 32; o <<= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
  float* wr = wres + warp * (hd + 2);
  if (gi == 0) {
#pragma unroll
    for (int i = 0; i < EPL; ++i) wr[gl * EPL + i] = acc[i];
  }
  if (lane == 0) {
    wr[hd] = m_run;
    wr[hd + 1] = l_w;
  }
  __syncthreads();
  // ---- the warps of this CTA, in warp order ----
  {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATTC_WARPS; ++w) M = fmaxf(M, wres[w * (hd + 2) + hd]);
    float e[ATTC_WARPS];
    float Lc = 0.f;
#pragma unroll
    for (int w = 0; w < ATTC_WARPS; ++w) {
      const float mw = wres[w * (hd + 2) + hd];
      e[w] = mw > -INFINITY ? expf(mw - M) : 0.f;
      Lc = fmaf(wres[w * (hd + 2) + hd + 1], e[w], Lc);
    }
    for (int d = tid; d < hd; d += ATTC_THREADS) {
      float o = 0.f;
#pragma unroll
      for (int w = 0; w < ATTC_WARPS; ++w) o = fmaf(e[w], wres[w * (hd + 2) + d], o);
      cres[d] = o;
    }
    if (tid == 0) {
      cres[hd] = M;
      cres[hd + 1] = Lc;
    }
  }
  trace_stamp(rec, 5);
  trace_stamp(rec, 6);
  cluster.sync();
  // ---- the CTAs of the cluster, in split order, by the first one ----
  if (cluster.block_rank() == 0) {
    const int nr = (int)cluster.num_blocks();
    float M = -INFINITY;
    float mr[ATTC_MAX_CLUSTER], lr[ATTC_MAX_CLUSTER];
#pragma unroll
    for (int r = 0; r < ATTC_MAX_CLUSTER; ++r) {
      mr[r] = -INFINITY;
      lr[r] = 0.f;
      if (r < nr) {
        const float* rem = cluster.map_shared_rank(cres, r);
        mr[r] = rem[hd];
        lr[r] = rem[hd + 1];
      }
      M = fmaxf(M, mr[r]);
    }
    float L = 0.f;
#pragma unroll
    for (int r = 0; r < ATTC_MAX_CLUSTER; ++r) {
      mr[r] = mr[r] > -INFINITY ? expf(mr[r] - M) : 0.f;  // now the weight of rank r
      L = fmaf(lr[r], mr[r], L);
    }
    const float inv = 1.0f / (L + 1e-9f);
    float* dst = prm.out + (size_t)b * prm.out_stride + h * hd;
    for (int d = tid; d < hd; d += ATTC_THREADS) {
      float o = 0.f;
#pragma unroll
      for (int r = 0; r < ATTC_MAX_CLUSTER; ++r)
        if (r < nr) o = fmaf(mr[r], cluster.map_shared_rank(cres, r)[d], o);
      dst[d] = o * inv;
    }
  }
  trace_stamp(rec, 7);
  cluster.sync();  // remote shared memory stays alive until the first CTA has read it
}

}  // namespace b200
