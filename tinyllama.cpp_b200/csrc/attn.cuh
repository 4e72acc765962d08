// Decode attention over the on-device KV cache with split-K over context length.
//
// One work item = (context split, query head, sequence), handled by a group of four warps. The
// group that owns the newest position also appends it: the new token's K/V row arrives as FP32
// (already rotated) from the QKV kernel, is quantised here when the cache is INT8 (per (position,
// kv head) absmax scale: scale = absmax/127, or 1 when absmax <= 1e-8; q = clamp(roundf(x/scale),
// -127, 127) — the arithmetic of the reference quantizer, cuda_kernels.cu:1535-1549 and 1596-1599)
// and written to the cache by the first query head of the group. Partial (max, sum, output)
// triples go to a scratch buffer and are merged in split order by the last group of a head to
// finish (atomic ticket), so the result does not depend on scheduling.
//
// Softmax follows the reference CPU code (model.cpp:632-663, utils.cpp:675-698):
//   s_t = (q . k_t) / sqrt(hd);  p_t = exp(s_t - max);  o = sum p_t v_t / (sum p_t + 1e-9).
//
// Cache layout (device-internal): K and V [slot][kv_head][position][head_dim], scales
// [slot][kv_head][position]. Algorithmic HBM bytes = K and V rows of positions 0..pos-1 of the
// heads read, plus their scales. Loads are issued four rows ahead per lane so that a group keeps
// 16 (INT8) or 4 (FP32) cache rows per warp in flight.
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
  int* tickets;          // [batch][nq], zero between launches (ticket merge only)
  float* out;            // [batch][out_stride]
  int out_stride;
  float att_scale;
  unsigned long long* trace;  // optional step-trace record (slots 0, 1: entry, inputs ready; 5: this CTA's partials written; 7: end)
  int cached_new;        // 1: the row of the newest position is already in the cache (prompt ingestion): read it like any other row
  int* error_flag;       // optional: set to 3 when a position lies outside [0, max_ctx) (nothing is read or written for that sequence)
};

constexpr int ATTN_GROUP_THREADS = 128;
constexpr int ATTN_UNROLL = 4;

__device__ __forceinline__ float i8_at(uint32_t w, int i) { return (float)(int)(int8_t)((w >> (8 * i)) & 0xFF); }
__device__ __forceinline__ void group_sync(int bar_id) { asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(ATTN_GROUP_THREADS) : "memory"); }

__host__ __device__ __forceinline__ int attn_split_cap(int max_ctx, int nsplit) { return ((max_ctx + nsplit - 1) / nsplit + 31) & ~31; }
// floats of shared memory one group needs
__host__ __device__ __forceinline__ size_t attn_group_floats(int hd, int max_ctx, int nsplit) {
  return (size_t)(3 * hd + 4 * hd + attn_split_cap(max_ctx, nsplit) + 16);
}

constexpr int ATTN_MAX_SPLITS = 64;
constexpr int ATTN_MERGE_AHEAD = 32;  // partial outputs requested before the (max, sum) pairs are known

// Merges the per-split partials of (sequence b, head h) in split order. Everything the merge reads
// is requested in one go: the partial outputs of up to 32 splits go into registers while the
// (max, sum) pairs make their own trip, so the whole merge costs one L2 round trip instead of one
// per split. scratch: 3 * ATTN_MAX_SPLITS floats of shared memory; called by all nthr threads of
// the group, which synchronise on bar_id.
__device__ __forceinline__ void attn_merge_head(const AttnParams& prm, int b, int h, int gtid, int nthr, float* dst, float* scratch,
                                                int bar_id) {
  const size_t pbase = ((size_t)b * prm.nq + h) * prm.nsplit;
  float* m_s = scratch;
  float* l_s = scratch + ATTN_MAX_SPLITS;
  float* w_s = scratch + 2 * ATTN_MAX_SPLITS;
  float v[ATTN_MERGE_AHEAD];
  const int d0 = gtid;  // first output element of this thread
#pragma unroll
  for (int s = 0; s < ATTN_MERGE_AHEAD; ++s)
    v[s] = (s < prm.nsplit && d0 < prm.hd) ? __ldcg(&prm.part_o[(pbase + s) * prm.hd + d0]) : 0.f;
  if (gtid < prm.nsplit) {
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(&prm.part_ml[(pbase + gtid) * 2]));
    m_s[gtid] = ml.x;
    l_s[gtid] = ml.y;
  }
  group_sync(bar_id);
  float M = -INFINITY;
#pragma unroll 1
  for (int s = 0; s < prm.nsplit; ++s) M = fmaxf(M, m_s[s]);
  if (gtid < prm.nsplit) w_s[gtid] = l_s[gtid] > 0.f ? expf(m_s[gtid] - M) : 0.f;
  group_sync(bar_id);
  float L = 0.f;
#pragma unroll 1
  for (int s = 0; s < prm.nsplit; ++s)
    if (l_s[s] > 0.f) L += l_s[s] * w_s[s];
  const float inv = 1.0f / (L + 1e-9f);
#pragma unroll 1
  for (int d = d0; d < prm.hd; d += nthr) {
    float o = 0.f;
    if (d == d0) {
#pragma unroll
      for (int s = 0; s < ATTN_MERGE_AHEAD; ++s)
        if (s < prm.nsplit) o = fmaf(w_s[s], v[s], o);
    } else {
#pragma unroll 1
      for (int s = 0; s < prm.nsplit && s < ATTN_MERGE_AHEAD; ++s) o = fmaf(w_s[s], __ldcg(&prm.part_o[(pbase + s) * prm.hd + d]), o);
    }
#pragma unroll 1
    for (int s = ATTN_MERGE_AHEAD; s < prm.nsplit; ++s) o = fmaf(w_s[s], __ldcg(&prm.part_o[(pbase + s) * prm.hd + d]), o);
    dst[d] = o * inv;
  }
}

// One (split, head, sequence) item by a group of 128 threads. KV_I8: int8 rows, 16 elements per
// lane per row; else FP32 rows, 4 elements per lane. sm = this group's shared memory. HD: the head
// dimension when known at compile time (the lane-to-position mapping then folds to constants and
// the code shrinks, which matters: the kernel runs from a cold instruction cache), 0 = read prm.hd.
template <bool KV_I8, int HD>
__device__ void attn_item(const AttnParams& prm, int split, int h, int b, float* sm, int gtid, int bar_id) {
  const int lane = gtid & 31, warp = gtid >> 5;
  constexpr int nwarps = ATTN_GROUP_THREADS / 32;
  const int hd = HD ? HD : prm.hd, G = prm.nq / prm.nkv, kvh = h / G;
  const int pos_real = prm.positions[b], slot = prm.slots[b];
  const int T = pos_real + 1;
  const int pos = prm.cached_new ? -1 : pos_real;  // the position whose K/V row comes from kv_new rather than from the cache
  int chunk = (T + prm.nsplit - 1) / prm.nsplit;
  chunk = (chunk + 31) & ~31;
  const int t0 = split * chunk, t1 = min(T, t0 + chunk);

  float* q_s = sm;                  // [hd]
  float* kn_s = q_s + hd;           // [hd] new K row as the cache will hold it (dequantised when INT8)
  float* vn_s = kn_s + hd;          // [hd]
  float* o_s = vn_s + hd;           // [nwarps][hd]
  float* red = o_s + nwarps * hd;   // [16]
  float* sc_s = red + 16;           // [cap]

  for (int d = gtid; d < hd; d += ATTN_GROUP_THREADS) q_s[d] = prm.q[(size_t)b * prm.q_stride + h * hd + d];

  const size_t head_row0 = ((size_t)slot * prm.nkv + kvh) * prm.max_ctx;  // row index of position 0
  const bool owns_new = (pos >= t0 && pos < t1);
  if (owns_new && warp < 2) {  // warp 0: K row, warp 1: V row
    const float* src = prm.kv_new + (size_t)b * prm.kvn_stride + (warp == 0 ? 0 : prm.nkv * hd) + kvh * hd;
    float* dst_s = warp == 0 ? kn_s : vn_s;
    if (KV_I8) {
      float amax = 0.f;
#pragma unroll 1
      for (int d = lane; d < hd; d += 32) amax = fmaxf(amax, fabsf(src[d]));
      amax = warp_max(amax);
      const float scale = ((double)amax > 1e-8) ? __fdiv_rn(amax, 127.0f) : 1.0f;
      int8_t* crow = reinterpret_cast<int8_t*>(warp == 0 ? prm.k_cache : prm.v_cache) + (head_row0 + pos) * hd;
#pragma unroll 1
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
#pragma unroll 1
      for (int d = lane; d < hd; d += 32) {
        const float v = src[d];
        dst_s[d] = v;
        if (h % G == 0) crow[d] = v;
      }
    }
  }
  group_sync(bar_id);

  constexpr int EPL = KV_I8 ? 16 : 4;   // elements per lane per row
  constexpr int U = ATTN_UNROLL;
  const int lpp = hd / EPL;             // lanes per position (<= 32)
  const int ppw = 32 / lpp;             // positions per warp per load
  const int gl = lane % lpp, gi = lane / lpp;
  float qr[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) qr[i] = q_s[gl * EPL + i];
  const size_t row_bytes = (size_t)hd * (KV_I8 ? 1 : 4);
  const uint8_t* kbase = reinterpret_cast<const uint8_t*>(prm.k_cache) + head_row0 * row_bytes + gl * 16;
  const uint8_t* vbase = reinterpret_cast<const uint8_t*>(prm.v_cache) + head_row0 * row_bytes + gl * 16;

  // The V rows of this warp's first batch of positions do not depend on the scores: request them
  // now so their latency overlaps the whole score / softmax phase.
  const int tb_first = t0 + warp * ppw * U;
  uint4 vw0[U];
  float vs0[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int t = tb_first + u * ppw + gi;
    vw0[u] = make_uint4(0u, 0u, 0u, 0u);
    vs0[u] = 1.f;
    if (t < t1 && t != pos) {
      vw0[u] = ldg128(vbase + (size_t)t * row_bytes);
      if (KV_I8) vs0[u] = __ldg(&prm.v_scale[head_row0 + t]);
    }
  }

  // ---- scores: U rows per lane requested before any is used ----
#pragma unroll 1
  for (int tb = t0 + warp * ppw * U; tb < t1; tb += nwarps * ppw * U) {
    uint4 kw[U];
    float ks[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = tb + u * ppw + gi;
      kw[u] = make_uint4(0u, 0u, 0u, 0u);
      ks[u] = 1.f;
      if (t < t1 && t != pos) {
        kw[u] = ldg128(kbase + (size_t)t * row_bytes);
        if (KV_I8) ks[u] = __ldg(&prm.k_scale[head_row0 + t]);
      }
    }
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
      if (t < t1 && gl == 0) sc_s[t - t0] = dot * prm.att_scale;
    }
  }
  group_sync(bar_id);

  // ---- max and exp-sum over this split ----
  const int n = max(t1 - t0, 0);
  float m = -INFINITY;
#pragma unroll 1
  for (int i = gtid; i < n; i += ATTN_GROUP_THREADS) m = fmaxf(m, sc_s[i]);
  m = warp_max(m);
  if (lane == 0) red[warp] = m;
  group_sync(bar_id);
  m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  float l = 0.f;
#pragma unroll 1
  for (int i = gtid; i < n; i += ATTN_GROUP_THREADS) {
    const float p = expf(sc_s[i] - m);
    sc_s[i] = p;
    l += p;
  }
  l = warp_sum(l);
  if (lane == 0) red[4 + warp] = l;
  group_sync(bar_id);
  l = (red[4] + red[5]) + (red[6] + red[7]);

  // ---- weighted sum of V ----
  float acc[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) acc[i] = 0.f;
#pragma unroll 1
  for (int tb = t0 + warp * ppw * U; tb < t1; tb += nwarps * ppw * U) {
    uint4 vw[U];
    float ps[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = tb + u * ppw + gi;
      vw[u] = make_uint4(0u, 0u, 0u, 0u);
      ps[u] = 0.f;
      if (t < t1) {
        ps[u] = sc_s[t - t0];
        if (t != pos) {
          if (tb == tb_first) {
            vw[u] = vw0[u];
            if (KV_I8) ps[u] *= vs0[u];
          } else {
            vw[u] = ldg128(vbase + (size_t)t * row_bytes);
            if (KV_I8) ps[u] *= __ldg(&prm.v_scale[head_row0 + t]);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = tb + u * ppw + gi;
      if (t == pos) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) acc[i] = fmaf(ps[u], vn_s[gl * EPL + i], acc[i]);
      } else if (KV_I8) {
        const uint32_t w4[4] = {vw[u].x, vw[u].y, vw[u].z, vw[u].w};
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i & (EPL - 1)] = fmaf(ps[u], i8_at(w4[i >> 2], i & 3), acc[i & (EPL - 1)]);
      } else {
        acc[0] = fmaf(ps[u], __uint_as_float(vw[u].x), acc[0]);
        acc[1] = fmaf(ps[u], __uint_as_float(vw[u].y), acc[1]);
        acc[2] = fmaf(ps[u], __uint_as_float(vw[u].z), acc[2]);
        acc[3 & (EPL - 1)] = fmaf(ps[u], __uint_as_float(vw[u].w), acc[3 & (EPL - 1)]);
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
  group_sync(bar_id);
  const size_t pbase = ((size_t)b * prm.nq + h) * prm.nsplit;
  for (int d = gtid; d < hd; d += ATTN_GROUP_THREADS)
    prm.part_o[(pbase + split) * hd + d] = (o_s[d] + o_s[hd + d]) + (o_s[2 * hd + d] + o_s[3 * hd + d]);
  if (gtid == 0) {
    prm.part_ml[(pbase + split) * 2 + 0] = m;
    prm.part_ml[(pbase + split) * 2 + 1] = l;
  }
}

// Stand-alone kernel: one group per CTA, ticket merge by the last CTA of each (sequence, head).
template <bool KV_I8, int HD>
__global__ void __launch_bounds__(ATTN_GROUP_THREADS, 5) attn_decode_kernel(const AttnParams prm) {
  extern __shared__ __align__(16) float sm[];
  __shared__ int last_flag;
  // lets a dependent launch that opted in start its independent prologue (weight prefetch) now;
  // it still waits for this grid to finish before touching anything produced here
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  unsigned long long* rec = (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) ? prm.trace : nullptr;
  trace_stamp(rec, 0);
  // when launched as a programmatic dependent itself: q and the new K/V rows belong to the previous kernel until here
  asm volatile("griddepcontrol.wait;" ::: "memory");
  trace_stamp(rec, 1);
  trace_stamp(rec, 2);
  trace_stamp(rec, 3);
  trace_stamp(rec, 4);
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  {
    // A position outside the cache would be written past the end of the caller's buffers: such a
    // sequence is skipped by all of its CTAs (nothing read, nothing appended), its output is set to
    // NaN and the error word, when there is one, is raised.
    const int pchk = prm.positions[b];
    if (pchk < 0 || pchk >= prm.max_ctx) {
      if (split == 0)
        for (int d = threadIdx.x; d < prm.hd; d += ATTN_GROUP_THREADS) prm.out[(size_t)b * prm.out_stride + h * prm.hd + d] = __int_as_float(0x7fc00000);
      if (threadIdx.x == 0 && prm.error_flag) *reinterpret_cast<volatile int*>(prm.error_flag) = 3;
      return;
    }
  }
  attn_item<KV_I8, HD>(prm, split, h, b, sm, threadIdx.x, 1);
  __syncthreads();  // every thread's partials are written; one thread publishes them for the whole CTA
  trace_stamp(rec, 5);
  trace_stamp(rec, 6);
  if (threadIdx.x == 0) {
    __threadfence();
    const int old = atomicAdd(&prm.tickets[b * prm.nq + h], 1);
    last_flag = (old == prm.nsplit - 1);
    if (last_flag) __threadfence();
  }
  __syncthreads();
  if (!last_flag) {
    trace_stamp(rec, 7);
    return;
  }
  attn_merge_head(prm, b, h, threadIdx.x, ATTN_GROUP_THREADS, prm.out + (size_t)b * prm.out_stride + h * prm.hd, sm, 1);
  if (threadIdx.x == 0) prm.tickets[b * prm.nq + h] = 0;
  trace_stamp(rec, 7);
}

// Prompt ingestion: appends the K and V rows of n tokens to the cache before their attention runs
// (same arithmetic as the append inside attn_item). grid = (tokens, ceil(kv heads / 4), 2: K | V), 128 threads: one warp per row.
constexpr int KVA_WARPS = 4;
__global__ void __launch_bounds__(32 * KVA_WARPS) kv_append_kernel(const float* __restrict__ kv_new, int kvn_stride, const int* __restrict__ positions,
                                                                   const int* __restrict__ slots, int nkv, int hd, int max_ctx, int kv_i8, void* k_cache,
                                                                   void* v_cache, float* k_scale, float* v_scale) {
  const int t = blockIdx.x, kvh = blockIdx.y * KVA_WARPS + (threadIdx.x >> 5), which = blockIdx.z, lane = threadIdx.x & 31;
  if (kvh >= nkv) return;
  const float* src = kv_new + (size_t)t * kvn_stride + (which ? nkv * hd : 0) + kvh * hd;
  const size_t crow = ((size_t)slots[t] * nkv + kvh) * max_ctx + positions[t];
  void* cache = which ? v_cache : k_cache;
  if (kv_i8) {
    float amax = 0.f;
    for (int d = lane; d < hd; d += 32) amax = fmaxf(amax, fabsf(src[d]));
    amax = warp_max(amax);
    const float scale = ((double)amax > 1e-8) ? __fdiv_rn(amax, 127.0f) : 1.0f;
    for (int d = lane; d < hd; d += 32) {
      float r = roundf(__fdiv_rn(src[d], scale));
      r = fmaxf(-127.0f, fminf(127.0f, r));
      reinterpret_cast<int8_t*>(cache)[crow * hd + d] = (int8_t)r;
    }
    if (lane == 0) (which ? v_scale : k_scale)[crow] = scale;
  } else {
    for (int d = lane; d < hd; d += 32) reinterpret_cast<float*>(cache)[crow * hd + d] = src[d];
  }
}

// Dynamic shared memory of the kernel: one group's working set, and never less than the
// 3 * ATTN_MAX_SPLITS floats the merge of the last CTA uses as scratch.
inline size_t attn_smem_bytes(int hd, int max_ctx, int nsplit, int /*nwarps*/) {
  const size_t fl = attn_group_floats(hd, max_ctx, nsplit);
  return sizeof(float) * (fl > (size_t)3 * ATTN_MAX_SPLITS ? fl : (size_t)3 * ATTN_MAX_SPLITS);
}

}  // namespace b200
