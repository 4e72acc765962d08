// Fused dequant-matvec over packed Q8_0 / Q4_K / Q6_K blocks for batch-1 style decode.
//
// Arithmetic: the activation vector is quantised once per CTA into P signed byte-planes
// (x ~ sx[blk] * x_int, x_int a (8P)-bit integer per element, one scale per 256 elements;
// P = 3 gives 24-bit activations, i.e. FP32-grade). Weights stay integers: every dot product
// over a quantisation sub-block is an exact integer sum built from dp4a, the sub-block's
// integer scale is applied with an integer multiply-add, and only one float multiply per
// (row, 64..128 weights) touches the block's fp16 scale. Minimum/offset terms use per-sub-block
// sums of the activations prepared in shared memory. Rows are reduced with warp shuffles.
//
// HBM traffic per launch = the packed bytes of the rows (each read once with 128-bit loads)
// plus the activation vector; that is the kernel's algorithmic byte count.
#pragma once
#include "common.cuh"
#include "dequant.cuh"

namespace b200 {

enum : int { EPI_STORE = 0, EPI_RESID = 1, EPI_QKV_ROPE = 2, EPI_SWIGLU = 3 };

struct GemvSeg {
  const uint8_t* w;   // Q4_K: blocks as in the file; Q6_K: ql plane; Q8_0: qs plane
  const uint8_t* qh;  // Q6_K high-bit plane
  const uint8_t* sc;  // Q6_K sub-scale plane
  const uint8_t* d;   // Q6_K / Q8_0 fp16 scale plane
  int type;
  int rows;
};

struct GemvParams {
  GemvSeg seg[3];
  int nseg;
  int K;                // input dimension (multiple of 256; of 64 for Q8_0-only launches)
  const float* x;       // [batch][x_stride]
  int x_stride;
  const float* norm_w;  // RMSNorm weight fused into the prologue, or nullptr
  float eps;
  int epi;
  float* y;             // STORE/RESID/SWIGLU: [batch][y_stride]; QKV: q output [batch][y_stride]
  int y_stride;
  float* y2;            // QKV: new K then V rows of this token, [batch][y2_stride]
  int y2_stride;
  const float* rope;    // [max_pos][head_dim/2][2] (cos, sin)
  const int* positions; // [batch]
  int head_dim;
  int max_pos;
  float* amax_val;      // optional per-CTA argmax partials [batch][gridDim.x]
  int* amax_idx;
};

// ---- shared-memory activation image ------------------------------------------------------
// Each plane stores 64-element chunks as four 16-byte pieces. Piece j of chunk c lives at
//   ((c >> 5) * 4 + j) * 512 + slot(c & 31) * 16
// so that a warp whose lanes read the same piece of 32 consecutive chunks (Q4_K, Q8_0), or of
// every second chunk (Q6_K), touches every bank exactly once per quarter-warp.
__host__ __device__ __forceinline__ int act_slot(int s) { return (s & 24) | ((s + ((s >> 3) & 1)) & 7); }
__host__ __device__ __forceinline__ int act_plane_stride(int K) { return ((K / 64 + 31) / 32) * 2048; }
__host__ __device__ __forceinline__ int act_sx_floats(int K) { return (K / 256 + 3) / 4 * 4; }  // keeps xs32/xs16 16-byte aligned
__host__ __device__ __forceinline__ size_t act_smem_bytes(int K, int P) {
  return (size_t)P * act_plane_stride(K) + (size_t)(act_sx_floats(K) + K / 32 + K / 16) * 4;
}

struct ActImage {
  const uint8_t* planes;
  int plane_stride;
  const float* sx;    // [K/256] scale of each 256-element block
  const float* xs32;  // [K/32]  sum of the (quantised) activations per 32 elements
  const float* xs16;  // [K/16]  per 16 elements
};

__device__ __forceinline__ ActImage act_carve(uint8_t* smem, int K, int P) {
  ActImage a;
  a.plane_stride = act_plane_stride(K);
  a.planes = smem;
  float* f = reinterpret_cast<float*>(smem + (size_t)P * a.plane_stride);
  a.sx = f;
  a.xs32 = f + act_sx_floats(K);
  a.xs16 = a.xs32 + K / 32;
  return a;
}

__device__ __forceinline__ uint4 act_piece(const ActImage& a, int p, int chunk, int j) {
  const uint8_t* ptr = a.planes + (size_t)p * a.plane_stride + ((chunk >> 5) * 4 + j) * 512 + act_slot(chunk & 31) * 16;
  return *reinterpret_cast<const uint4*>(ptr);
}

// Whole-CTA prologue: optional RMSNorm (reference utils.cpp:648-673: double mean of squares,
// f = 1/sqrtf((float)mean + eps), out = x*f*w) then quantisation into the plane image.
template <int P>
__device__ void act_build(uint8_t* smem, const float* __restrict__ x, const float* __restrict__ norm_w, float eps,
                          int K, float* red /* 33 floats of shared scratch */) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  float f = 1.0f;
  if (norm_w) {
    float ss = 0.f;
    for (int i = tid * 4; i < K; i += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(x + i);
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    double ds = (double)ss;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ds += __shfl_xor_sync(0xffffffffu, ds, o);
    double* dred = reinterpret_cast<double*>(red);
    if (lane == 0) dred[warp] = ds;
    __syncthreads();
    if (warp == 0) {
      double t = lane < nwarps ? dred[lane] : 0.0;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      if (lane == 0) {
        float mean = (float)(t / (double)K);
        reinterpret_cast<float*>(dred + 32)[0] = 1.0f / sqrtf(mean + eps);
      }
    }
    __syncthreads();
    f = reinterpret_cast<float*>(dred + 32)[0];
  }
  ActImage a = act_carve(smem, K, P);
  uint8_t* planes = const_cast<uint8_t*>(a.planes);
  float* sx = const_cast<float*>(a.sx);
  float* xs32 = const_cast<float*>(a.xs32);
  float* xs16 = const_cast<float*>(a.xs16);
  constexpr int QMAX = (1 << (8 * P - 1)) - 1;
  const int nblk = K / 256;
  for (int b = warp; b < nblk; b += nwarps) {
    const int e0 = b * 256 + lane * 8;
    float4 v0 = *reinterpret_cast<const float4*>(x + e0), v1 = *reinterpret_cast<const float4*>(x + e0 + 4);
    float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    if (norm_w) {
      float4 w0 = *reinterpret_cast<const float4*>(norm_w + e0), w1 = *reinterpret_cast<const float4*>(norm_w + e0 + 4);
      float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = v[i] * f * w[i];
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = warp_max(amax);
    const float scale = amax / (float)QMAX;
    const float inv = amax > 0.f ? (float)QMAX / amax : 0.f;
    int xi[8];
    int s8 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int q = __float2int_rn(v[i] * inv);
      q = max(-QMAX, min(QMAX, q));
      xi[i] = q;
      s8 += q;
    }
    const int s16 = s8 + __shfl_xor_sync(0xffffffffu, s8, 1);
    const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 2);
    if ((lane & 1) == 0) xs16[b * 16 + (lane >> 1)] = scale * (float)s16;
    if ((lane & 3) == 0) xs32[b * 8 + (lane >> 2)] = scale * (float)s32;
    if (lane == 0) sx[b] = scale;
    const int chunk = b * 4 + (lane >> 3), j = (lane & 7) >> 1, off8 = (lane & 1) * 8;
#pragma unroll
    for (int p = 0; p < P; ++p) {
      uint32_t w0 = 0, w1 = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        w0 |= (uint32_t)((xi[i] >> (8 * p)) & 0xFF) << (8 * i);
        w1 |= (uint32_t)((xi[4 + i] >> (8 * p)) & 0xFF) << (8 * i);
      }
      uint8_t* dst = planes + (size_t)p * a.plane_stride + ((chunk >> 5) * 4 + j) * 512 + act_slot(chunk & 31) * 16 + off8;
      *reinterpret_cast<uint2*>(dst) = make_uint2(w0, w1);
    }
  }
  __syncthreads();
}

template <int P>
__device__ __forceinline__ float combine_planes(const int (&I)[P]) {
  if (P == 1) return (float)I[0];
  if (P == 2) return fmaf((float)I[1], 256.f, (float)I[0]);
  return fmaf((float)I[P - 1], 65536.f, fmaf((float)I[1], 256.f, (float)I[0]));
}

// dot of four weight bytes with plane p of the activations; WS = weights signed
template <int P, bool WS>
__device__ __forceinline__ int dotp(int p, uint32_t w, uint32_t x, int c) {
  if (p == P - 1) return WS ? dp4a_ss(w, x, c) : dp4a_us(w, x, c);
  return WS ? dp4a_su(w, x, c) : dp4a_uu(w, x, c);
}

struct RowPtr {
  const uint8_t* w;
  const uint8_t* qh;
  const uint8_t* sc;
  const uint8_t* d;
};

// ---- Q4_K: one task = 64 weights = 32 bytes of nibbles (two complete sub-blocks) ----------
template <int P, int NR>
__device__ __forceinline__ void dot_q4k(const RowPtr (&rows)[NR], const ActImage& a, int K, int lane, float (&acc)[NR]) {
  const int ntask = K / 64;
  const int c = lane & 3;
  for (int task = lane; task < ntask; task += 32) {
    const int blk = task >> 2;
    uint4 hdr[NR], qa[NR], qb[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const uint8_t* bp = rows[r].w + (size_t)blk * 144;
      hdr[r] = ldg128(bp);
      qa[r] = ldg128_stream(bp + 16 + 32 * c);
      qb[r] = ldg128_stream(bp + 32 + 32 * c);
    }
    int Slo[NR][P], Shi[NR][P];
#pragma unroll
    for (int r = 0; r < NR; ++r)
#pragma unroll
      for (int p = 0; p < P; ++p) Slo[r][p] = Shi[r][p] = 0;
#pragma unroll
    for (int p = 0; p < P; ++p) {
      const uint4 x0 = act_piece(a, p, task, 0), x1 = act_piece(a, p, task, 1);
      const uint4 x2 = act_piece(a, p, task, 2), x3 = act_piece(a, p, task, 3);
      const uint32_t xl[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
      const uint32_t xh[8] = {x2.x, x2.y, x2.z, x2.w, x3.x, x3.y, x3.z, x3.w};
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const uint32_t q[8] = {qa[r].x, qa[r].y, qa[r].z, qa[r].w, qb[r].x, qb[r].y, qb[r].z, qb[r].w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          Slo[r][p] = dotp<P, false>(p, q[j] & 0x0F0F0F0Fu, xl[j], Slo[r][p]);
          Shi[r][p] = dotp<P, false>(p, q[j] & 0xF0F0F0F0u, xh[j], Shi[r][p]);  // 16x the nibble sum
        }
      }
    }
    const float sxb = a.sx[blk];
    const float xs_lo = a.xs32[2 * task], xs_hi = a.xs32[2 * task + 1];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const uint32_t yb = (hdr[r].y >> (8 * (c & 1) * 2)) , zb = (hdr[r].z >> (8 * (c & 1) * 2)), wb = (hdr[r].w >> (8 * (c & 1) * 2));
      // sub-blocks j0 = 2c, j1 = 2c+1 -> byte indices (j & 3) = 2(c&1), 2(c&1)+1
      const uint32_t y0 = yb & 0xFF, y1 = (yb >> 8) & 0xFF, z0 = zb & 0xFF, z1 = (zb >> 8) & 0xFF;
      const uint32_t w0 = wb & 0xFF, w1 = (wb >> 8) & 0xFF;
      int sc0, sc1, m0, m1;
      if (c < 2) {
        sc0 = y0 & 63; m0 = z0 & 63; sc1 = y1 & 63; m1 = z1 & 63;
      } else {
        sc0 = (w0 & 0xF) | ((y0 >> 6) << 4); m0 = (w0 >> 4) | ((z0 >> 6) << 4);
        sc1 = (w1 & 0xF) | ((y1 >> 6) << 4); m1 = (w1 >> 4) | ((z1 >> 6) << 4);
      }
      int I[P];
#pragma unroll
      for (int p = 0; p < P; ++p) I[p] = sc0 * Slo[r][p] + sc1 * (Shi[r][p] >> 4);
      const float2 dm = __half22float2(*reinterpret_cast<const __half2*>(&hdr[r].x));
      const float fsum = combine_planes<P>(I);
      acc[r] = fmaf(dm.x * sxb, fsum, acc[r]);
      acc[r] = fmaf(-dm.y, fmaf((float)m0, xs_lo, (float)m1 * xs_hi), acc[r]);
    }
  }
}

// ---- Q6_K: one task = half a block = 128 weights in eight 16-element sub-blocks ----------
template <int P, int NR>
__device__ __forceinline__ void dot_q6k(const RowPtr (&rows)[NR], const ActImage& a, int K, int lane, float (&acc)[NR]) {
  const int ntask = K / 128;
  for (int task = lane; task < ntask; task += 32) {
    const int blk = task >> 1, h = task & 1;
    uint4 ql[NR][4], qh[NR][2];
    uint2 scw[NR];
    uint16_t dh[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const uint8_t* pl = rows[r].w + (size_t)blk * 128 + 64 * h;
      const uint8_t* ph = rows[r].qh + (size_t)blk * 64 + 32 * h;
#pragma unroll
      for (int i = 0; i < 4; ++i) ql[r][i] = ldg128_stream(pl + 16 * i);
      qh[r][0] = ldg128_stream(ph);
      qh[r][1] = ldg128_stream(ph + 16);
      scw[r] = ldg64(rows[r].sc + (size_t)blk * 16 + 8 * h);
      dh[r] = ldg16(rows[r].d + (size_t)blk * 2);
    }
    int I[NR][P];
#pragma unroll
    for (int r = 0; r < NR; ++r)
#pragma unroll
      for (int p = 0; p < P; ++p) I[r][p] = 0;
    // group g: 0 -> elements 0..31 (chunk A pieces 0,1), 1 -> 32..63 (A pieces 2,3),
    //          2 -> 64..95 (chunk B pieces 0,1), 3 -> 96..127 (B pieces 2,3)
#pragma unroll
    for (int g = 0; g < 4; ++g) {
#pragma unroll
      for (int is = 0; is < 2; ++is) {
        uint32_t qv[NR][4];
#pragma unroll
        for (int r = 0; r < NR; ++r) {
          const uint4 lw = ql[r][(g & 1) * 2 + is];  // ql bytes (g&1)*32 + 16*is ..
          const uint4 hw = qh[r][is];                // qh bytes 16*is ..
          const uint32_t l4[4] = {lw.x, lw.y, lw.z, lw.w}, h4[4] = {hw.x, hw.y, hw.z, hw.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t lo = (g < 2) ? (l4[j] & 0x0F0F0F0Fu) : ((l4[j] >> 4) & 0x0F0F0F0Fu);
            uint32_t hb;
            if (g == 0) hb = (h4[j] << 4);
            else if (g == 1) hb = (h4[j] << 2);
            else if (g == 2) hb = h4[j];
            else hb = (h4[j] >> 2);
            qv[r][j] = lo | (hb & 0x30303030u);
          }
        }
        int S[NR][P];
#pragma unroll
        for (int p = 0; p < P; ++p) {
          const uint4 xv = act_piece(a, p, 2 * task + (g >> 1), (g & 1) * 2 + is);
          const uint32_t x4[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
          for (int r = 0; r < NR; ++r) {
            int s = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) s = dotp<P, false>(p, qv[r][j], x4[j], s);
            S[r][p] = s;
          }
        }
#pragma unroll
        for (int r = 0; r < NR; ++r) {
          const int k = 2 * g + is;  // sub-scale index within the half
          const uint32_t word = k < 4 ? scw[r].x : scw[r].y;
          const int sc = (int)(int8_t)((word >> (8 * (k & 3))) & 0xFF);
#pragma unroll
          for (int p = 0; p < P; ++p) I[r][p] += sc * S[r][p];
        }
      }
    }
    const float sxb = a.sx[blk];
    const float4 xa = *reinterpret_cast<const float4*>(a.xs16 + 8 * task);
    const float4 xb = *reinterpret_cast<const float4*>(a.xs16 + 8 * task + 4);
    const float xs[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      float corr = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t word = k < 4 ? scw[r].x : scw[r].y;
        corr = fmaf((float)(int)(int8_t)((word >> (8 * (k & 3))) & 0xFF), xs[k], corr);
      }
      const float d = half_bits_to_float(dh[r]);
      acc[r] = fmaf(d, fmaf(sxb, combine_planes<P>(I[r]), -32.f * corr), acc[r]);
    }
  }
}

// ---- Q8_0: one task = two blocks = 64 signed bytes -----------------------------------------
template <int P, int NR>
__device__ __forceinline__ void dot_q80(const RowPtr (&rows)[NR], const ActImage& a, int K, int lane, float (&acc)[NR]) {
  const int ntask = K / 64;
  for (int task = lane; task < ntask; task += 32) {
    uint4 q[NR][4];
    uint32_t dd[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const uint8_t* pq = rows[r].w + (size_t)task * 64;
#pragma unroll
      for (int i = 0; i < 4; ++i) q[r][i] = ldg128_stream(pq + 16 * i);
      dd[r] = ldg32(rows[r].d + (size_t)task * 4);
    }
    int I0[NR][P], I1[NR][P];
#pragma unroll
    for (int r = 0; r < NR; ++r)
#pragma unroll
      for (int p = 0; p < P; ++p) I0[r][p] = I1[r][p] = 0;
#pragma unroll
    for (int p = 0; p < P; ++p) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 xv = act_piece(a, p, task, i);
        const uint32_t x4[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
        for (int r = 0; r < NR; ++r) {
          const uint32_t w4[4] = {q[r][i].x, q[r][i].y, q[r][i].z, q[r][i].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (i < 2) I0[r][p] = dotp<P, true>(p, w4[j], x4[j], I0[r][p]);
            else I1[r][p] = dotp<P, true>(p, w4[j], x4[j], I1[r][p]);
          }
        }
      }
    }
    const float sxb = a.sx[task >> 2];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const float d0 = scale_field_to_float((uint16_t)(dd[r] & 0xFFFF)), d1 = scale_field_to_float((uint16_t)(dd[r] >> 16));
      acc[r] = fmaf(d0 * sxb, combine_planes<P>(I0[r]), acc[r]);
      acc[r] = fmaf(d1 * sxb, combine_planes<P>(I1[r]), acc[r]);
    }
  }
}

__device__ __forceinline__ RowPtr row_ptr(const GemvSeg& s, int row, int K) {
  RowPtr r;
  const size_t nb = (size_t)(K / (s.type == T_Q8_0 ? 32 : 256));
  const size_t b0 = (size_t)row * nb;
  if (s.type == T_Q4_K) {
    r.w = s.w + b0 * 144; r.qh = r.sc = r.d = nullptr;
  } else if (s.type == T_Q6_K) {
    r.w = s.w + b0 * 128; r.qh = s.qh + b0 * 64; r.sc = s.sc + b0 * 16; r.d = s.d + b0 * 2;
  } else {
    r.w = s.w + b0 * 32; r.d = s.d + b0 * 2; r.qh = r.sc = nullptr;
  }
  return r;
}

// One CTA = 8 warps; blockIdx.y = batch element. Each warp walks over row pairs.
template <int P>
__global__ void __launch_bounds__(256, 2) gemv_kernel(const GemvParams prm) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ double red_scratch[34];
  const int b = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  act_build<P>(smem, prm.x + (size_t)b * prm.x_stride, prm.norm_w, prm.eps, prm.K, reinterpret_cast<float*>(red_scratch));
  const ActImage a = act_carve(smem, prm.K, P);

  int total_rows = 0;
  for (int s = 0; s < prm.nseg; ++s) total_rows += prm.seg[s].rows;
  const int npairs = prm.epi == EPI_SWIGLU ? prm.seg[0].rows : total_rows / 2;
  const int wpc = blockDim.x >> 5;
  float best_v = -INFINITY;
  int best_i = 0x7fffffff;

  for (int pair = blockIdx.x * wpc + warp; pair < npairs; pair += gridDim.x * wpc) {
    RowPtr rows[2];
    int type, seg_id = 0, row0;
    if (prm.epi == EPI_SWIGLU) {
      rows[0] = row_ptr(prm.seg[0], pair, prm.K);
      rows[1] = row_ptr(prm.seg[1], pair, prm.K);
      type = prm.seg[0].type;
      row0 = pair;
    } else {
      row0 = 2 * pair;
      while (seg_id + 1 < prm.nseg && row0 >= prm.seg[seg_id].rows) { row0 -= prm.seg[seg_id].rows; ++seg_id; }
      rows[0] = row_ptr(prm.seg[seg_id], row0, prm.K);
      rows[1] = row_ptr(prm.seg[seg_id], row0 + 1, prm.K);
      type = prm.seg[seg_id].type;
    }
    float acc[2] = {0.f, 0.f};
    if (type == T_Q4_K) dot_q4k<P, 2>(rows, a, prm.K, lane, acc);
    else if (type == T_Q6_K) dot_q6k<P, 2>(rows, a, prm.K, lane, acc);
    else dot_q80<P, 2>(rows, a, prm.K, lane, acc);
    acc[0] = warp_sum(acc[0]);
    acc[1] = warp_sum(acc[1]);
    if (lane == 0) {
      if (prm.epi == EPI_SWIGLU) {
        // reference model.cpp:734-735 with silu_cpu (utils.cpp:700-707): (g * 1/(1+exp(-g))) * u
        const float g = acc[0], u = acc[1];
        const float sig = 1.0f / (1.0f + expf(-g));
        prm.y[(size_t)b * prm.y_stride + row0] = (g * sig) * u;
      } else if (prm.epi == EPI_RESID) {
        float* y = prm.y + (size_t)b * prm.y_stride + row0;
        y[0] = y[0] + acc[0];
        y[1] = y[1] + acc[1];
      } else if (prm.epi == EPI_QKV_ROPE) {
        float v0 = acc[0], v1 = acc[1];
        if (seg_id < 2) {  // q and k are rotated in adjacent pairs (reference utils.cpp:428-489)
          const int pos = prm.positions[b];
          if (pos >= 0 && pos < prm.max_pos) {
            const int i = (row0 % prm.head_dim) >> 1;
            const float2 cs = *reinterpret_cast<const float2*>(prm.rope + ((size_t)pos * (prm.head_dim >> 1) + i) * 2);
            const float r0 = __fsub_rn(__fmul_rn(v0, cs.x), __fmul_rn(v1, cs.y));
            const float r1 = __fadd_rn(__fmul_rn(v0, cs.y), __fmul_rn(v1, cs.x));
            v0 = r0; v1 = r1;
          }
        }
        float* dst = seg_id == 0 ? prm.y + (size_t)b * prm.y_stride + row0
                                 : prm.y2 + (size_t)b * prm.y2_stride + (seg_id == 2 ? prm.seg[1].rows : 0) + row0;
        dst[0] = v0;
        dst[1] = v1;
      } else {
        const int row = 2 * pair;
        float* y = prm.y + (size_t)b * prm.y_stride + row;
        y[0] = acc[0];
        y[1] = acc[1];
        if (prm.amax_val) {
          if (acc[0] > best_v || (acc[0] == best_v && row < best_i)) { best_v = acc[0]; best_i = row; }
          if (acc[1] > best_v || (acc[1] == best_v && row + 1 < best_i)) { best_v = acc[1]; best_i = row + 1; }
        }
      }
    }
  }
  if (prm.amax_val) {  // per-CTA (value, first index) of the rows this CTA produced
    __shared__ float sv[8];
    __shared__ int si[8];
    if (lane == 0) { sv[warp] = best_v; si[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float bv = sv[0];
      int bi = si[0];
      for (int w = 1; w < wpc; ++w)
        if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
      prm.amax_val[(size_t)b * gridDim.x + blockIdx.x] = bv;
      prm.amax_idx[(size_t)b * gridDim.x + blockIdx.x] = bi;
    }
  }
}

}  // namespace b200
