// Prompt-ingestion attention: causal attention of a chunk of consecutive tokens of ONE sequence
// against that sequence's KV cache (the chunk's own rows are already appended), on the fp16
// tensor cores (mma.sync m16n8k16, FP32 accumulation).
//
// Same mathematics as the reference's batch attention (cpu_attention.cpp:91-201: the token at
// position p attends to 0..p, softmax with 1/(sum + 1e-9), scores scaled by 1/sqrt(head_dim)), but
// every K/V row is read once per 64 queries instead of once per query.
//
// One CTA = 64 consecutive queries of one head, four warps of 16 query rows each; the key loop
// walks 64-key tiles with an online softmax. K and V tiles are converted to fp16 in shared memory:
// INT8 rows exactly (their per-row scale is applied to the FP32 scores, respectively folded into
// the probabilities), FP32 rows by rounding. INT8 tiles arrive through a two-deep cp.async ring so
// the next tile's bytes are in flight while this one is multiplied.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "attn.cuh"

namespace b200 {

struct PrefillAttnParams {
  const float* q;  // [T][q_stride], after RoPE
  int q_stride;
  const void* k_cache;  // this layer's cache: [(slot*nkv + kvh)*max_ctx + pos][hd]
  const void* v_cache;
  const float* k_scale;  // [(slot*nkv + kvh)*max_ctx + pos] (INT8 cache only)
  const float* v_scale;
  int slot, start, T;  // tokens occupy positions start .. start+T-1
  int nq, nkv, max_ctx;
  float* out;  // [T][out_stride]
  int out_stride;
  float att_scale;
};

constexpr int PFA_Q = 64;        // queries per CTA
constexpr int PFA_K = 64;        // keys per tile
constexpr int PFA_THREADS = 128;

__host__ __device__ constexpr int pfa_stride(int hd) { return hd + 8; }  // halves; rows start 16 bytes apart modulo 128
__host__ __device__ constexpr size_t pfa_smem_bytes(bool kv_i8, int hd) {
  return (size_t)2 * PFA_K * pfa_stride(hd) * 2 + 2 * PFA_K * 4 + (kv_i8 ? (size_t)2 * 2 * PFA_K * hd : 0);
}

__device__ __forceinline__ void pfa_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void pfa_ldm4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void pfa_ldm4t(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ uint32_t pfa_pack(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
// four signed bytes -> four halves, exactly: 0x6400 | (b ^ 0x80) is 1024 + (b + 128)
__device__ __forceinline__ void pfa_cvt4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  w ^= 0x80808080u;
  const uint32_t p0 = __byte_perm(w, 0x64646464u, 0x4140);
  const uint32_t p1 = __byte_perm(w, 0x64646464u, 0x4342);
  const __half2 off = __floats2half2_rn(1152.f, 1152.f);
  const __half2 r0 = __hsub2(*reinterpret_cast<const __half2*>(&p0), off);
  const __half2 r1 = __hsub2(*reinterpret_cast<const __half2*>(&p1), off);
  lo = *reinterpret_cast<const uint32_t*>(&r0);
  hi = *reinterpret_cast<const uint32_t*>(&r1);
}
__device__ __forceinline__ void pfa_cp16(void* smem, const void* gmem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void pfa_cp_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <bool KV_I8, int HD>
__global__ void __launch_bounds__(PFA_THREADS, 2) attn_prefill_kernel(const PrefillAttnParams prm) {
  static_assert(HD == 64 || HD == 128, "head_dim 64 or 128");
  constexpr int STR = pfa_stride(HD);
  constexpr int KSTEPS = HD / 16;
  constexpr int NT_O = HD / 8;
  extern __shared__ __align__(16) unsigned char pfa_smem[];
  __half* Ks = reinterpret_cast<__half*>(pfa_smem);
  __half* Vs = Ks + PFA_K * STR;
  float* ks_s = reinterpret_cast<float*>(Vs + PFA_K * STR);
  float* vs_s = ks_s + PFA_K;
  unsigned char* raw = reinterpret_cast<unsigned char*>(vs_s + PFA_K);  // [2][K | V][PFA_K*HD] (INT8 cache)

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int q0 = blockIdx.x * PFA_Q, h = blockIdx.y;
  const int kvh = h / (prm.nq / prm.nkv);
  const size_t crow0 = ((size_t)prm.slot * prm.nkv + kvh) * prm.max_ctx;
  const int qend = min(q0 + PFA_Q, prm.T);       // queries of this CTA: q0 .. qend-1
  const int kmax = prm.start + qend - 1;         // last key any of them sees
  const int nkt = kmax / PFA_K + 1;

  // this thread's two query rows and their Q fragments
  const int r0 = q0 + warp * 16 + g, r1 = r0 + 8;
  const int qpos0 = prm.start + r0, qpos1 = prm.start + r1;
  uint32_t qa[KSTEPS][4];
  {
    const float* qr0 = prm.q + (size_t)min(r0, prm.T - 1) * prm.q_stride + h * HD;
    const float* qr1 = prm.q + (size_t)min(r1, prm.T - 1) * prm.q_stride + h * HD;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      const float2 a = *reinterpret_cast<const float2*>(qr0 + ks * 16 + 2 * t);
      const float2 b = *reinterpret_cast<const float2*>(qr1 + ks * 16 + 2 * t);
      const float2 c = *reinterpret_cast<const float2*>(qr0 + ks * 16 + 8 + 2 * t);
      const float2 d = *reinterpret_cast<const float2*>(qr1 + ks * 16 + 8 + 2 * t);
      qa[ks][0] = pfa_pack(a.x, a.y);
      qa[ks][1] = pfa_pack(b.x, b.y);
      qa[ks][2] = pfa_pack(c.x, c.y);
      qa[ks][3] = pfa_pack(d.x, d.y);
    }
  }

  float o[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const float sc2 = prm.att_scale * 1.4426950408889634f;  // scores are kept in the log2 domain

  // scale of key (tid & 63) of a tile: threads 0..63 fetch K scales, 64..127 V scales
  auto fetch_scale = [&](int kt) -> float {
    const int key = kt * PFA_K + (tid & 63);
    if (key > kmax) return 0.f;  // rows nobody may see: zero weight, whatever the cache holds there
    if (!KV_I8) return 1.f;
    return (tid < 64 ? prm.k_scale : prm.v_scale)[crow0 + key];
  };
  constexpr int RAW_TILE = PFA_K * HD;            // bytes of one INT8 K (or V) tile
  constexpr int CP_PER_THREAD = RAW_TILE / 16 / PFA_THREADS;
  auto issue_raw = [&](int kt) {
    unsigned char* dstk = raw + (size_t)(kt & 1) * 2 * RAW_TILE;
    unsigned char* dstv = dstk + RAW_TILE;
    const unsigned char* srck = reinterpret_cast<const unsigned char*>(prm.k_cache) + (crow0 + (size_t)kt * PFA_K) * HD;
    const unsigned char* srcv = reinterpret_cast<const unsigned char*>(prm.v_cache) + (crow0 + (size_t)kt * PFA_K) * HD;
#pragma unroll
    for (int r = 0; r < CP_PER_THREAD; ++r) {
      const int i = tid + r * PFA_THREADS;
      const int key = kt * PFA_K + i / (HD / 16);
      if (key <= kmax) {  // rows past the last visible key are not touched (they may lie outside the cache)
        pfa_cp16(dstk + (size_t)i * 16, srck + (size_t)i * 16);
        pfa_cp16(dstv + (size_t)i * 16, srcv + (size_t)i * 16);
      }
    }
  };

  float sreg = 0.f;
  if (KV_I8) issue_raw(0);
  sreg = fetch_scale(0);

  for (int kt = 0; kt < nkt; ++kt) {
    if (KV_I8) pfa_cp_wait_all();
    __syncthreads();  // this tile's bytes have landed; everybody is done with the previous fp16 tiles
    const float scur = sreg;
    if (kt + 1 < nkt) {
      if (KV_I8) issue_raw(kt + 1);
      sreg = fetch_scale(kt + 1);
    }
    if (KV_I8) {
      const unsigned char* srck = raw + (size_t)(kt & 1) * 2 * RAW_TILE;
      const unsigned char* srcv = srck + RAW_TILE;
#pragma unroll
      for (int r = 0; r < CP_PER_THREAD; ++r) {
        const int i = tid + r * PFA_THREADS;
        const int key = i / (HD / 16), part = i % (HD / 16);
        const uint4 wk = *reinterpret_cast<const uint4*>(srck + (size_t)i * 16);
        const uint4 wv = *reinterpret_cast<const uint4*>(srcv + (size_t)i * 16);
        uint4 a, b;
        pfa_cvt4(wk.x, a.x, a.y); pfa_cvt4(wk.y, a.z, a.w); pfa_cvt4(wk.z, b.x, b.y); pfa_cvt4(wk.w, b.z, b.w);
        uint4* dk = reinterpret_cast<uint4*>(Ks + key * STR + part * 16);
        dk[0] = a; dk[1] = b;
        pfa_cvt4(wv.x, a.x, a.y); pfa_cvt4(wv.y, a.z, a.w); pfa_cvt4(wv.z, b.x, b.y); pfa_cvt4(wv.w, b.z, b.w);
        uint4* dv = reinterpret_cast<uint4*>(Vs + key * STR + part * 16);
        dv[0] = a; dv[1] = b;
      }
    } else {
      const float* srck = reinterpret_cast<const float*>(prm.k_cache) + (crow0 + (size_t)kt * PFA_K) * HD;
      const float* srcv = reinterpret_cast<const float*>(prm.v_cache) + (crow0 + (size_t)kt * PFA_K) * HD;
      constexpr int F4 = PFA_K * HD / 4 / PFA_THREADS;
#pragma unroll 4
      for (int r = 0; r < F4; ++r) {
        const int i = tid + r * PFA_THREADS;
        const int key = i / (HD / 4), part = i % (HD / 4);
        float4 fk = make_float4(0.f, 0.f, 0.f, 0.f), fv = fk;
        if (kt * PFA_K + key <= kmax) {
          fk = *reinterpret_cast<const float4*>(srck + (size_t)i * 4);
          fv = *reinterpret_cast<const float4*>(srcv + (size_t)i * 4);
        }
        *reinterpret_cast<uint2*>(Ks + key * STR + part * 4) = make_uint2(pfa_pack(fk.x, fk.y), pfa_pack(fk.z, fk.w));
        *reinterpret_cast<uint2*>(Vs + key * STR + part * 4) = make_uint2(pfa_pack(fv.x, fv.y), pfa_pack(fv.z, fv.w));
      }
    }
    (tid < 64 ? ks_s : vs_s)[tid & 63] = scur;
    __syncthreads();

    // S = Q K^T for this warp's 16 rows x 64 keys
    float s[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ks += 2) {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        uint32_t b[4];
        pfa_ldm4(b, Ks + (nt * 8 + (lane & 7)) * STR + ks * 16 + (lane >> 3) * 8);
        pfa_mma(s[nt], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b[0], b[1]);
        pfa_mma(s[nt], qa[ks + 1][0], qa[ks + 1][1], qa[ks + 1][2], qa[ks + 1][3], b[2], b[3]);
      }
    }
    // scale, causal mask, running maximum
    const int kbase = kt * PFA_K + 2 * t;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float2 kk = *reinterpret_cast<const float2*>(ks_s + nt * 8 + 2 * t);
      const int key = kbase + nt * 8;
      s[nt][0] = key <= qpos0 ? s[nt][0] * (kk.x * sc2) : -INFINITY;
      s[nt][1] = key + 1 <= qpos0 ? s[nt][1] * (kk.y * sc2) : -INFINITY;
      s[nt][2] = key <= qpos1 ? s[nt][2] * (kk.x * sc2) : -INFINITY;
      s[nt][3] = key + 1 <= qpos1 ? s[nt][3] * (kk.y * sc2) : -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
      mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);  // finite from the first tile on: key 0 is visible to every query
    const float al0 = exp2f(m0 - mn0), al1 = exp2f(m1 - mn1);
    m0 = mn0; m1 = mn1;
    uint32_t pa[8][2];
    float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float2 vv = *reinterpret_cast<const float2*>(vs_s + nt * 8 + 2 * t);
      const float p0 = exp2f(s[nt][0] - mn0), p1 = exp2f(s[nt][1] - mn0);
      const float p2 = exp2f(s[nt][2] - mn1), p3 = exp2f(s[nt][3] - mn1);
      ls0 += p0 + p1;
      ls1 += p2 + p3;
      pa[nt][0] = pfa_pack(p0 * vv.x, p1 * vv.y);
      pa[nt][1] = pfa_pack(p2 * vv.x, p3 * vv.y);
    }
    l0 = l0 * al0 + ls0;
    l1 = l1 * al1 + ls1;
#pragma unroll
    for (int i = 0; i < NT_O; ++i) { o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1; }
    // O += P V
#pragma unroll
    for (int j = 0; j < PFA_K / 16; ++j) {
#pragma unroll
      for (int np = 0; np < HD / 16; ++np) {
        uint32_t b[4];
        pfa_ldm4t(b, Vs + (j * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * STR + np * 16 + (lane >> 4) * 8);
        pfa_mma(o[2 * np], pa[2 * j][0], pa[2 * j][1], pa[2 * j + 1][0], pa[2 * j + 1][1], b[0], b[1]);
        pfa_mma(o[2 * np + 1], pa[2 * j][0], pa[2 * j][1], pa[2 * j + 1][0], pa[2 * j + 1][1], b[2], b[3]);
      }
    }
  }

  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = 1.0f / (l0 + 1e-9f), inv1 = 1.0f / (l1 + 1e-9f);  // softmax_vector_cpu (utils.cpp:675-698)
  if (r0 < prm.T) {
    float* dst = prm.out + (size_t)r0 * prm.out_stride + h * HD + 2 * t;
#pragma unroll
    for (int i = 0; i < NT_O; ++i) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][0] * inv0, o[i][1] * inv0);
  }
  if (r1 < prm.T) {
    float* dst = prm.out + (size_t)r1 * prm.out_stride + h * HD + 2 * t;
#pragma unroll
    for (int i = 0; i < NT_O; ++i) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][2] * inv1, o[i][3] * inv1);
  }
}

// Batched decode attention for grouped-query models: one CTA per (sequence, KV head) serves all
// G = n_heads / n_kv_heads query heads of the group (G <= 8), so every K/V row of the sequence is
// read once per step instead of once per query head. Same tiles and conversions as the prompt
// kernel; the G heads are the rows of one 16-row MMA tile (the other rows are zero). The four warps
// split each 64-key tile into 16-key quarters, each with its own running softmax; their partial
// results are merged through shared memory at the end. The new token's K/V rows are already in
// the cache (kv_append_kernel). With nsplit > 1 the context of every sequence is cut into nsplit
// runs of whole tiles, one CTA each (grid.z): a CTA then writes its (max, sum, weighted V) partials in
// the decode kernel's format and the last CTA of the (sequence, KV head) to finish merges them
// (ticket, attn_merge_head), so that one long sequence does not hold a layer's attention back.
struct GqaAttnParams {
  const float* q;  // [batch][q_stride], after RoPE
  int q_stride;
  const void* k_cache;
  const void* v_cache;
  const float* k_scale;
  const float* v_scale;
  const int* positions;  // [batch] position of the new token: keys 0..position are visible
  const int* slots;      // [batch]
  int nq, nkv, max_ctx;
  float* out;  // [batch][out_stride]
  int out_stride;
  float att_scale;
  int nsplit;      // context runs per sequence (<= ATTN_MAX_SPLITS)
  float* part_o;   // [batch][nq][nsplit][hd]   (nsplit > 1)
  float* part_ml;  // [batch][nq][nsplit][2]
  int* tickets;    // [batch][nq], zero between launches; entry of the group's first head is used
};

template <bool KV_I8, int HD>
__global__ void __launch_bounds__(PFA_THREADS, 3) attn_decode_gqa_kernel(const GqaAttnParams prm) {
  static_assert(HD == 64 || HD == 128, "head_dim 64 or 128");
  constexpr int STR = pfa_stride(HD);
  constexpr int KSTEPS = HD / 16;
  constexpr int NT_O = HD / 8;
  extern __shared__ __align__(16) unsigned char pfa_smem[];
  __half* Ks = reinterpret_cast<__half*>(pfa_smem);
  __half* Vs = Ks + PFA_K * STR;
  float* ks_s = reinterpret_cast<float*>(Vs + PFA_K * STR);
  float* vs_s = ks_s + PFA_K;
  unsigned char* raw = reinterpret_cast<unsigned char*>(vs_s + PFA_K);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int kvh = blockIdx.x, b = blockIdx.y;
  const int G = prm.nq / prm.nkv;
  const int pos = prm.positions[b];
  const size_t crow0 = ((size_t)prm.slots[b] * prm.nkv + kvh) * prm.max_ctx;
  const int kmax = pos;
  const int nkt_all = kmax / PFA_K + 1;
  const int split = blockIdx.z;
  const int tiles_per_split = (nkt_all + prm.nsplit - 1) / prm.nsplit;
  const int kt0 = split * tiles_per_split, nkt = min(nkt_all, kt0 + tiles_per_split);  // this CTA's tiles: kt0 .. nkt-1 (possibly none)

  // row g of the tile = query head kvh*G + g (g < G); rows G..15 are zero
  uint32_t qa[KSTEPS][2];
  {
    const float* qr = prm.q + (size_t)b * prm.q_stride + (size_t)(kvh * G + min(g, G - 1)) * HD;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      const float2 a = *reinterpret_cast<const float2*>(qr + ks * 16 + 2 * t);
      const float2 c = *reinterpret_cast<const float2*>(qr + ks * 16 + 8 + 2 * t);
      qa[ks][0] = g < G ? pfa_pack(a.x, a.y) : 0u;
      qa[ks][1] = g < G ? pfa_pack(c.x, c.y) : 0u;
    }
  }
  float o[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, l0 = 0.f;
  const float sc2 = prm.att_scale * 1.4426950408889634f;

  auto fetch_scale = [&](int kt) -> float {
    const int key = kt * PFA_K + (tid & 63);
    if (key > kmax) return 0.f;
    if (!KV_I8) return 1.f;
    return (tid < 64 ? prm.k_scale : prm.v_scale)[crow0 + key];
  };
  constexpr int RAW_TILE = PFA_K * HD;
  constexpr int CP_PER_THREAD = RAW_TILE / 16 / PFA_THREADS;
  auto issue_raw = [&](int kt) {
    unsigned char* dstk = raw + (size_t)(kt & 1) * 2 * RAW_TILE;
    unsigned char* dstv = dstk + RAW_TILE;
    const unsigned char* srck = reinterpret_cast<const unsigned char*>(prm.k_cache) + (crow0 + (size_t)kt * PFA_K) * HD;
    const unsigned char* srcv = reinterpret_cast<const unsigned char*>(prm.v_cache) + (crow0 + (size_t)kt * PFA_K) * HD;
#pragma unroll
    for (int r = 0; r < CP_PER_THREAD; ++r) {
      const int i = tid + r * PFA_THREADS;
      const int key = kt * PFA_K + i / (HD / 16);
      if (key <= kmax) {
        pfa_cp16(dstk + (size_t)i * 16, srck + (size_t)i * 16);
        pfa_cp16(dstv + (size_t)i * 16, srcv + (size_t)i * 16);
      }
    }
  };

  float sreg = 0.f;
  if (kt0 < nkt) {
    if (KV_I8) issue_raw(kt0);
    sreg = fetch_scale(kt0);
  }
  const int kw = 16 * warp;  // this warp's keys within a tile

#pragma unroll 1
  for (int kt = kt0; kt < nkt; ++kt) {
    if (KV_I8) pfa_cp_wait_all();
    __syncthreads();
    const float scur = sreg;
    if (kt + 1 < nkt) {
      if (KV_I8) issue_raw(kt + 1);
      sreg = fetch_scale(kt + 1);
    }
    if (KV_I8) {
      const unsigned char* srck = raw + (size_t)(kt & 1) * 2 * RAW_TILE;
      const unsigned char* srcv = srck + RAW_TILE;
#pragma unroll
      for (int r = 0; r < CP_PER_THREAD; ++r) {
        const int i = tid + r * PFA_THREADS;
        const int key = i / (HD / 16), part = i % (HD / 16);
        const uint4 wk = *reinterpret_cast<const uint4*>(srck + (size_t)i * 16);
        const uint4 wv = *reinterpret_cast<const uint4*>(srcv + (size_t)i * 16);
        uint4 a, c;
        pfa_cvt4(wk.x, a.x, a.y); pfa_cvt4(wk.y, a.z, a.w); pfa_cvt4(wk.z, c.x, c.y); pfa_cvt4(wk.w, c.z, c.w);
        uint4* dk = reinterpret_cast<uint4*>(Ks + key * STR + part * 16);
        dk[0] = a; dk[1] = c;
        pfa_cvt4(wv.x, a.x, a.y); pfa_cvt4(wv.y, a.z, a.w); pfa_cvt4(wv.z, c.x, c.y); pfa_cvt4(wv.w, c.z, c.w);
        uint4* dv = reinterpret_cast<uint4*>(Vs + key * STR + part * 16);
        dv[0] = a; dv[1] = c;
      }
    } else {
      const float* srck = reinterpret_cast<const float*>(prm.k_cache) + (crow0 + (size_t)kt * PFA_K) * HD;
      const float* srcv = reinterpret_cast<const float*>(prm.v_cache) + (crow0 + (size_t)kt * PFA_K) * HD;
      constexpr int F4 = PFA_K * HD / 4 / PFA_THREADS;
#pragma unroll 4
      for (int r = 0; r < F4; ++r) {
        const int i = tid + r * PFA_THREADS;
        const int key = i / (HD / 4), part = i % (HD / 4);
        float4 fk = make_float4(0.f, 0.f, 0.f, 0.f), fv = fk;
        if (kt * PFA_K + key <= kmax) {
          fk = *reinterpret_cast<const float4*>(srck + (size_t)i * 4);
          fv = *reinterpret_cast<const float4*>(srcv + (size_t)i * 4);
        }
        *reinterpret_cast<uint2*>(Ks + key * STR + part * 4) = make_uint2(pfa_pack(fk.x, fk.y), pfa_pack(fk.z, fk.w));
        *reinterpret_cast<uint2*>(Vs + key * STR + part * 4) = make_uint2(pfa_pack(fv.x, fv.y), pfa_pack(fv.z, fv.w));
      }
    }
    (tid < 64 ? ks_s : vs_s)[tid & 63] = scur;
    __syncthreads();
    if (kt * PFA_K + kw > kmax) continue;  // this warp's quarter of the tile lies past the newest key (uniform per warp)

    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ks += 2) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        uint32_t bf[4];
        pfa_ldm4(bf, Ks + (kw + nt * 8 + (lane & 7)) * STR + ks * 16 + (lane >> 3) * 8);
        pfa_mma(s[nt], qa[ks][0], 0u, qa[ks][1], 0u, bf[0], bf[1]);
        pfa_mma(s[nt], qa[ks + 1][0], 0u, qa[ks + 1][1], 0u, bf[2], bf[3]);
      }
    }
    const int kbase = kt * PFA_K + kw + 2 * t;
    float mx0 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const float2 kk = *reinterpret_cast<const float2*>(ks_s + kw + nt * 8 + 2 * t);
      const int key = kbase + nt * 8;
      s[nt][0] = key <= pos ? s[nt][0] * (kk.x * sc2) : -INFINITY;
      s[nt][1] = key + 1 <= pos ? s[nt][1] * (kk.y * sc2) : -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    const float mn0 = fmaxf(m0, mx0);  // finite: the quarter's first key is visible (checked above)
    const float al0 = exp2f(m0 - mn0);
    m0 = mn0;
    uint32_t pa[2];
    float ls0 = 0.f;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const float2 vv = *reinterpret_cast<const float2*>(vs_s + kw + nt * 8 + 2 * t);
      const float p0 = exp2f(s[nt][0] - mn0), p1 = exp2f(s[nt][1] - mn0);
      ls0 += p0 + p1;
      pa[nt] = pfa_pack(p0 * vv.x, p1 * vv.y);
    }
    l0 = l0 * al0 + ls0;
#pragma unroll
    for (int i = 0; i < NT_O; ++i) { o[i][0] *= al0; o[i][1] *= al0; }
#pragma unroll
    for (int np = 0; np < HD / 16; ++np) {
      uint32_t bf[4];
      pfa_ldm4t(bf, Vs + (kw + (lane & 7) + ((lane >> 3) & 1) * 8) * STR + np * 16 + (lane >> 4) * 8);
      pfa_mma(o[2 * np], pa[0], 0u, pa[1], 0u, bf[0], bf[1]);
      pfa_mma(o[2 * np + 1], pa[0], 0u, pa[1], 0u, bf[2], bf[3]);
    }
  }

  // ---- merge the four warps' partial results: [warp][G][HD] outputs and [warp][G] (max, sum) pairs ----
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  __syncthreads();  // everybody is done with the K/V tiles
  float* po = reinterpret_cast<float*>(pfa_smem);                 // [4][8][HD]
  float* pml = po + 4 * 8 * HD;                                   // [4][8][2]
  if (g < G) {
#pragma unroll
    for (int i = 0; i < NT_O; ++i) *reinterpret_cast<float2*>(po + ((size_t)warp * 8 + g) * HD + i * 8 + 2 * t) = make_float2(o[i][0], o[i][1]);
    if (t == 0) { pml[(warp * 8 + g) * 2] = m0; pml[(warp * 8 + g) * 2 + 1] = l0; }
  }
  __syncthreads();
  for (int idx = tid; idx < G * HD; idx += PFA_THREADS) {
    const int gq = idx / HD, d = idx - gq * HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, pml[(w * 8 + gq) * 2]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = pml[(w * 8 + gq) * 2];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);  // a warp that saw no key contributes nothing
      L += pml[(w * 8 + gq) * 2 + 1] * f;
      O += po[((size_t)w * 8 + gq) * HD + d] * f;
    }
    const int h = kvh * G + gq;
    if (prm.nsplit == 1) {
      prm.out[(size_t)b * prm.out_stride + (size_t)h * HD + d] = O / (L + 1e-9f);
    } else {  // partials as the decode kernel writes them: maximum in natural-log units, sum and weighted V relative to it
      const size_t pi = ((size_t)b * prm.nq + h) * prm.nsplit + split;
      prm.part_o[pi * HD + d] = O;
      if (d == 0) {
        prm.part_ml[pi * 2] = M * 0.6931471805599453f;
        prm.part_ml[pi * 2 + 1] = L;
      }
    }
  }
  if (prm.nsplit == 1) return;
  __shared__ int last_flag;
  __syncthreads();  // every thread's partials are written; one thread publishes them for the whole CTA
  if (tid == 0) {
    __threadfence();
    const int old = atomicAdd(&prm.tickets[b * prm.nq + kvh * G], 1);
    last_flag = (old == prm.nsplit - 1);
    if (last_flag) __threadfence();
  }
  __syncthreads();
  if (!last_flag) return;
  AttnParams ap{};
  ap.nq = prm.nq; ap.hd = HD; ap.nsplit = prm.nsplit; ap.part_o = prm.part_o; ap.part_ml = prm.part_ml;
  float* scratch = reinterpret_cast<float*>(pfa_smem);
  for (int gq = 0; gq < G; ++gq) {
    const int h = kvh * G + gq;
    attn_merge_head(ap, b, h, tid, PFA_THREADS, prm.out + (size_t)b * prm.out_stride + (size_t)h * HD, scratch, 1);
    group_sync(1);  // the scratch is reused by the next head
  }
  if (tid == 0) prm.tickets[b * prm.nq + kvh * G] = 0;
}

}  // namespace b200
