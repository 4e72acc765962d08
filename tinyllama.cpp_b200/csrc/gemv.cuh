// Fused dequant-matvec over packed Q8_0 / Q4_K / Q6_K blocks for decode (one activation vector
// per launch column).
//
// Arithmetic. The activation vector is quantised once per CTA into P balanced base-256 digit
// planes (x ~ sx[blk] * x_int, x_int = sum_p digit_p * 256^p, every digit a signed byte, one scale
// per 256 elements; P = 3 gives 24-bit activations, i.e. FP32-grade). Weights stay the integers
// that are stored in the blocks. A warp owns a tile of 16 output rows and walks along K one
// 256-element block at a time; every 32 elements it issues one integer tensor-core instruction
// (mma.sync m16n8k32, u8/s8 x s8 -> s32) whose 16 x 32 A operand is built in registers from the
// packed nibbles / 6-bit fields with a couple of logic ops, and whose B operand is the digit
// planes (one column per plane) read from shared memory. The exact integer sub-block sums are
// multiplied by the integer sub-block scales (6-bit for Q4_K, int8 for Q6_K) with integer
// multiply-adds; one float multiply per (row, 256-block) applies the fp16 block scale. The
// Q4_K minimum term and the Q6_K "-32" offset use per-sub-block sums of the activations, also
// kept as digit bytes, and are evaluated with dp4a. Rows are finished with warp shuffles.
//
// Work split. One persistent CTA of 16 warps per SM takes a contiguous range of tiles; inside the
// CTA the (tile, block) sequence is cut into 16 equal contiguous pieces, one per warp, so that
// short matrices still keep every warp streaming. Partial row sums meet in shared memory in a
// fixed order (deterministic).
//
// HBM traffic per launch = the packed bytes of the rows (each read exactly once, 64-bit and
// 128-bit loads that bypass L1) plus the activation vector; that is the algorithmic byte count.
#pragma once
#include "common.cuh"
#include "dequant.cuh"

namespace b200 {

enum : int { EPI_STORE = 0, EPI_RESID = 1, EPI_QKV_ROPE = 2, EPI_SWIGLU = 3 };
constexpr int GEMV_WARPS = 16;
constexpr int GEMV_THREADS = GEMV_WARPS * 32;

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
  int K;                // input dimension, a multiple of 256
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
  int ntiles;           // 16-row tiles (SWIGLU: 8 gate rows + 8 up rows per tile)
};

// ---- shared-memory activation image ------------------------------------------------------
// planes  [P][plane_stride]   digit bytes, element e of plane p at p*plane_stride + e; the stride
//                             is = 32 (mod 128) so the planes read by one mma fall in distinct banks
// sx      [K/256]             float scale of each 256-element block
// xs32d   [4][K/32]           digit d of the sum of x_int over each 32 elements (Q4_K minimum term)
// xs16d   [4][K/16]           the same per 16 elements (Q6_K offset term)
__host__ __device__ __forceinline__ int act_plane_stride(int K) { return (K + 127) / 128 * 128 + 32; }
__host__ __device__ __forceinline__ int act_sx_floats(int K) { return (K / 256 + 3) / 4 * 4; }
__host__ __device__ __forceinline__ size_t act_smem_bytes(int K, int P) {
  return (size_t)P * act_plane_stride(K) + (size_t)act_sx_floats(K) * 4 + (size_t)4 * (K / 32) + (size_t)4 * (K / 16);
}

struct ActImage {
  const uint8_t* planes;
  int plane_stride;
  const float* sx;
  const uint8_t* xs32d;
  const uint8_t* xs16d;
  int n32, n16;
};

__device__ __forceinline__ ActImage act_carve(uint8_t* smem, int K, int P) {
  ActImage a;
  a.plane_stride = act_plane_stride(K);
  a.planes = smem;
  uint8_t* p = smem + (size_t)P * a.plane_stride;
  a.sx = reinterpret_cast<const float*>(p);
  p += act_sx_floats(K) * 4;
  a.xs32d = p;
  a.n32 = K / 32;
  p += 4 * a.n32;
  a.xs16d = p;
  a.n16 = K / 16;
  return a;
}

// balanced base-256 digits of v: v = d0 + 256 d1 + 65536 d2 + 2^24 d3, every d in [-128, 127]
__device__ __forceinline__ void balanced_digits4(int v, int (&d)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    d[i] = (int)(int8_t)(v & 0xFF);
    v = (v - d[i]) >> 8;
  }
}

// Whole-CTA prologue: optional RMSNorm (reference utils.cpp:648-673: double mean of squares,
// f = 1/sqrtf((float)mean + eps), out = x*f*w) then quantisation into the image above.
template <int P>
__device__ void act_build(uint8_t* smem, const float* __restrict__ x, const float* __restrict__ norm_w, float eps,
                          int K, double* red /* 33 doubles of shared scratch */) {
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
    if (lane == 0) red[warp] = ds;
    __syncthreads();
    if (warp == 0) {
      double t = lane < nwarps ? red[lane] : 0.0;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      if (lane == 0) {
        float mean = (float)(t / (double)K);
        reinterpret_cast<float*>(red + 32)[0] = 1.0f / sqrtf(mean + eps);
      }
    }
    __syncthreads();
    f = reinterpret_cast<float*>(red + 32)[0];
  }
  ActImage a = act_carve(smem, K, P);
  uint8_t* planes = const_cast<uint8_t*>(a.planes);
  float* sx = const_cast<float*>(a.sx);
  uint8_t* xs32d = const_cast<uint8_t*>(a.xs32d);
  uint8_t* xs16d = const_cast<uint8_t*>(a.xs16d);
  // largest magnitude P balanced digits can hold: 127 * (256^P - 1) / 255
  constexpr int QMAX = P == 3 ? 8355711 : (P == 2 ? 32639 : 127);
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
    int s8 = 0;
    uint32_t pw[P][2];
#pragma unroll
    for (int p = 0; p < P; ++p) pw[p][0] = pw[p][1] = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int q = __float2int_rn(v[i] * inv);
      q = max(-QMAX, min(QMAX, q));
      s8 += q;
#pragma unroll
      for (int p = 0; p < P; ++p) {
        const int dgt = (int)(int8_t)(q & 0xFF);
        q = (q - dgt) >> 8;
        pw[p][i >> 2] |= (uint32_t)(dgt & 0xFF) << (8 * (i & 3));
      }
    }
#pragma unroll
    for (int p = 0; p < P; ++p)
      *reinterpret_cast<uint2*>(planes + (size_t)p * a.plane_stride + e0) = make_uint2(pw[p][0], pw[p][1]);
    const int s16 = s8 + __shfl_xor_sync(0xffffffffu, s8, 1);
    const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 2);
    if ((lane & 1) == 0) {
      int dg[4];
      balanced_digits4(s16, dg);
#pragma unroll
      for (int i = 0; i < 4; ++i) xs16d[i * a.n16 + b * 16 + (lane >> 1)] = (uint8_t)dg[i];
    }
    if ((lane & 3) == 0) {
      int dg[4];
      balanced_digits4(s32, dg);
#pragma unroll
      for (int i = 0; i < 4; ++i) xs32d[i * a.n32 + b * 8 + (lane >> 2)] = (uint8_t)dg[i];
    }
    if (lane == 0) sx[b] = scale;
  }
  __syncthreads();
}

// D(16x8, s32) = A(16x32, u8 or s8) * B(32x8, s8); C = 0.
template <bool A_SIGNED>
__device__ __forceinline__ void imma_16x8x32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  if (A_SIGNED)
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
  else
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ uint2 ldg64_stream(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

// byte i (0..3) of w, zero-extended / sign-extended (i is a compile-time constant after unrolling)
__device__ __forceinline__ int byte_u(uint32_t w, int i) { return (int)__byte_perm(w, 0, 0x4440 | i); }
__device__ __forceinline__ int byte_s(uint32_t w, uint32_t i) {
  // prmt: a selector nibble with bit 3 set replicates the sign bit of the chosen byte
  int d;
  const uint32_t sel = i | ((8 | i) << 4) | ((8 | i) << 8) | ((8 | i) << 12);
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(w), "r"(0), "r"(sel));
  return d;
}

struct RowPtr {
  const uint8_t* w;
  const uint8_t* qh;
  const uint8_t* sc;
  const uint8_t* d;
};

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

// ---- per-format work on one 256-element block of a 16-row tile ----------------------------
// Lane (g = lane >> 2, t = lane & 3) feeds rows g and g + 8 of the tile and the four k-slices
// 8t .. 8t+7 of every 32-element group; it receives columns 2t and 2t+1 of the product.
struct LaneCtx {
  int g, t;
  float wa, wb;  // 256^plane of columns 2t, 2t+1 (0 for unused columns)
  float wd;      // 256^t: weight of digit t in the minimum / offset terms
};

template <int P>
__device__ __forceinline__ uint2 b_frag(const ActImage& a, int col, int elem) {
  if (col < P) return *reinterpret_cast<const uint2*>(a.planes + (size_t)col * a.plane_stride + elem);
  return make_uint2(0u, 0u);
}

struct RawQ4 {
  uint2 q[2][4];
  uint4 h[2];
};
__device__ __forceinline__ void load_q4(RawQ4& r, const RowPtr& ra, const RowPtr& rb, int blk, int t) {
  const uint8_t* pa = ra.w + (size_t)blk * 144;
  const uint8_t* pb = rb.w + (size_t)blk * 144;
  r.h[0] = ldg128_stream(pa);
  r.h[1] = ldg128_stream(pb);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    r.q[0][c] = ldg64_stream(pa + 16 + 32 * c + 8 * t);
    r.q[1][c] = ldg64_stream(pb + 16 + 32 * c + 8 * t);
  }
}

template <int P>
__device__ __forceinline__ void compute_q4(const RawQ4& r, const ActImage& a, int blk, const LaneCtx& L, float& acc0, float& acc1) {
  // eight 6-bit scales and minima per row, four to a word (get_scale_min_k4 of the reference,
  // quantization.cpp:145-155, applied to four sub-blocks at once)
  uint32_t scA[2], scB[2], mnA[2], mnB[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const uint32_t y = r.h[i].y, z = r.h[i].z, w = r.h[i].w;
    scA[i] = y & 0x3F3F3F3Fu;
    mnA[i] = z & 0x3F3F3F3Fu;
    scB[i] = (w & 0x0F0F0F0Fu) | ((y >> 2) & 0x30303030u);
    mnB[i] = ((w >> 4) & 0x0F0F0F0Fu) | ((z >> 2) & 0x30303030u);
  }
  int Jlo[4] = {0, 0, 0, 0}, Jhi[4] = {0, 0, 0, 0};
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int e = blk * 256 + 64 * c + 8 * L.t;
    const uint2 bl = b_frag<P>(a, L.g, e), bh = b_frag<P>(a, L.g, e + 32);
    int cl[4], ch[4];
    imma_16x8x32<false>(cl, r.q[0][c].x & 0x0F0F0F0Fu, r.q[1][c].x & 0x0F0F0F0Fu, r.q[0][c].y & 0x0F0F0F0Fu,
                        r.q[1][c].y & 0x0F0F0F0Fu, bl.x, bl.y);
    imma_16x8x32<false>(ch, r.q[0][c].x & 0xF0F0F0F0u, r.q[1][c].x & 0xF0F0F0F0u, r.q[0][c].y & 0xF0F0F0F0u,
                        r.q[1][c].y & 0xF0F0F0F0u, bh.x, bh.y);  // 16 x the high-nibble sums
    const int sl0 = byte_u(c < 2 ? scA[0] : scB[0], (2 * c) & 3), sh0 = byte_u(c < 2 ? scA[0] : scB[0], (2 * c + 1) & 3);
    const int sl1 = byte_u(c < 2 ? scA[1] : scB[1], (2 * c) & 3), sh1 = byte_u(c < 2 ? scA[1] : scB[1], (2 * c + 1) & 3);
    Jlo[0] += sl0 * cl[0]; Jlo[1] += sl0 * cl[1]; Jlo[2] += sl1 * cl[2]; Jlo[3] += sl1 * cl[3];
    Jhi[0] += sh0 * ch[0]; Jhi[1] += sh0 * ch[1]; Jhi[2] += sh1 * ch[2]; Jhi[3] += sh1 * ch[3];
  }
  const float f0 = L.wa * fmaf((float)Jhi[0], 0.0625f, (float)Jlo[0]) + L.wb * fmaf((float)Jhi[1], 0.0625f, (float)Jlo[1]);
  const float f1 = L.wa * fmaf((float)Jhi[2], 0.0625f, (float)Jlo[2]) + L.wb * fmaf((float)Jhi[3], 0.0625f, (float)Jlo[3]);
  // minimum term: sum_sub m_sub * X_sub, digit t of X handled by lane t
  const uint2 xw = *reinterpret_cast<const uint2*>(a.xs32d + (size_t)L.t * a.n32 + blk * 8);
  const int M0 = dp4a_us(mnB[0], xw.y, dp4a_us(mnA[0], xw.x, 0));
  const int M1 = dp4a_us(mnB[1], xw.y, dp4a_us(mnA[1], xw.x, 0));
  const float sxb = a.sx[blk];
  const float2 dm0 = __half22float2(*reinterpret_cast<const __half2*>(&r.h[0].x));
  const float2 dm1 = __half22float2(*reinterpret_cast<const __half2*>(&r.h[1].x));
  acc0 = fmaf(sxb, dm0.x * f0 - dm0.y * (L.wd * (float)M0), acc0);
  acc1 = fmaf(sxb, dm1.x * f1 - dm1.y * (L.wd * (float)M1), acc1);
}

struct RawQ6 {
  uint2 ql[2][4];  // [row][half*2 + (low|high 32 bytes)]
  uint2 qh[2][2];  // [row][half]
  uint4 sc[2];
  uint16_t d[2];
};
__device__ __forceinline__ void load_q6(RawQ6& r, const RowPtr& ra, const RowPtr& rb, int blk, int t) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const RowPtr& rp = i ? rb : ra;
#pragma unroll
    for (int j = 0; j < 4; ++j) r.ql[i][j] = ldg64_stream(rp.w + (size_t)blk * 128 + 32 * j + 8 * t);
#pragma unroll
    for (int h = 0; h < 2; ++h) r.qh[i][h] = ldg64_stream(rp.qh + (size_t)blk * 64 + 32 * h + 8 * t);
    r.sc[i] = ldg128_stream(rp.sc + (size_t)blk * 16);
    r.d[i] = ldg16(rp.d + (size_t)blk * 2);
  }
}

// Q6_K: a group of 32 consecutive elements holds two 16-element sub-blocks. Lanes t = 0,1 carry
// the first one, t = 2,3 the second; columns 0..P-1 see only the first (B is zero for t >= 2),
// columns P..2P-1 only the second, so one instruction yields both sub-block sums separately.
template <int P>
__device__ __forceinline__ void compute_q6(const RawQ6& r, const ActImage& a, int blk, const LaneCtx& L, float& acc0, float& acc1) {
  const int col = L.g, sub_of_col = col / P, plane = col - sub_of_col * P;
  const bool b_on = col < 2 * P && sub_of_col == (L.t >> 1);
  // which sub-block (0/1) columns 2t and 2t+1 belong to
  const uint32_t selA = (uint32_t)((2 * L.t) / P), selB = (uint32_t)((2 * L.t + 1) / P);
  int J[4] = {0, 0, 0, 0};
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t hf[2][2][4];  // [row][word][field] : 2-bit fields moved to bits 4-5 of every byte
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint32_t hw[2] = {r.qh[i][h].x, r.qh[i][h].y};
#pragma unroll
      for (int w = 0; w < 2; ++w) {
        hf[i][w][0] = (hw[w] << 4) & 0x30303030u;
        hf[i][w][1] = (hw[w] << 2) & 0x30303030u;
        hf[i][w][2] = hw[w] & 0x30303030u;
        hf[i][w][3] = (hw[w] >> 2) & 0x30303030u;
      }
    }
#pragma unroll
    for (int g4 = 0; g4 < 4; ++g4) {
      uint32_t av[2][2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const uint2 lw = r.ql[i][h * 2 + (g4 & 1)];
        const uint32_t l2[2] = {lw.x, lw.y};
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          const uint32_t nib = g4 < 2 ? (l2[w] & 0x0F0F0F0Fu) : ((l2[w] >> 4) & 0x0F0F0F0Fu);
          av[i][w] = nib | hf[i][w][g4];
        }
      }
      const int e = blk * 256 + 128 * h + 32 * g4 + 8 * L.t;
      uint2 bv = make_uint2(0u, 0u);
      if (b_on) bv = *reinterpret_cast<const uint2*>(a.planes + (size_t)plane * a.plane_stride + e);
      int c[4];
      imma_16x8x32<false>(c, av[0][0], av[1][0], av[0][1], av[1][1], bv.x, bv.y);
      // sub-scale index within the block: 8h + 2*g4 + (0|1) -> word (2h + g4/2), byte 2(g4&1) + sel
      const int wsel = 2 * h + (g4 >> 1);
      const uint32_t w0 = wsel == 0 ? r.sc[0].x : wsel == 1 ? r.sc[0].y : wsel == 2 ? r.sc[0].z : r.sc[0].w;
      const uint32_t w1 = wsel == 0 ? r.sc[1].x : wsel == 1 ? r.sc[1].y : wsel == 2 ? r.sc[1].z : r.sc[1].w;
      const uint32_t bA = 2 * (g4 & 1) + selA, bB = 2 * (g4 & 1) + selB;
      J[0] += byte_s(w0, bA) * c[0];
      J[1] += byte_s(w0, bB) * c[1];
      J[2] += byte_s(w1, bA) * c[2];
      J[3] += byte_s(w1, bB) * c[3];
    }
  }
  const float f0 = L.wa * (float)J[0] + L.wb * (float)J[1];
  const float f1 = L.wa * (float)J[2] + L.wb * (float)J[3];
  // offset term: the stored quants are q + 32, so subtract 32 * sum_sub sc_sub * X_sub (digit t per lane)
  const uint4 xw = *reinterpret_cast<const uint4*>(a.xs16d + (size_t)L.t * a.n16 + blk * 16);
  const int C0 = dp4a_ss(r.sc[0].w, xw.w, dp4a_ss(r.sc[0].z, xw.z, dp4a_ss(r.sc[0].y, xw.y, dp4a_ss(r.sc[0].x, xw.x, 0))));
  const int C1 = dp4a_ss(r.sc[1].w, xw.w, dp4a_ss(r.sc[1].z, xw.z, dp4a_ss(r.sc[1].y, xw.y, dp4a_ss(r.sc[1].x, xw.x, 0))));
  const float sxb = a.sx[blk];
  acc0 = fmaf(sxb * half_bits_to_float(r.d[0]), f0 - 32.f * (L.wd * (float)C0), acc0);
  acc1 = fmaf(sxb * half_bits_to_float(r.d[1]), f1 - 32.f * (L.wd * (float)C1), acc1);
}

struct RawQ8 {
  uint2 q[2][8];
  uint4 d[2];
};
__device__ __forceinline__ void load_q8(RawQ8& r, const RowPtr& ra, const RowPtr& rb, int blk, int t) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const RowPtr& rp = i ? rb : ra;
#pragma unroll
    for (int j = 0; j < 8; ++j) r.q[i][j] = ldg64_stream(rp.w + (size_t)blk * 256 + 32 * j + 8 * t);
    r.d[i] = ldg128_stream(rp.d + (size_t)blk * 16);
  }
}

template <int P>
__device__ __forceinline__ void compute_q8(const RawQ8& r, const ActImage& a, int blk, const LaneCtx& L, float& acc0, float& acc1) {
  const uint32_t dw0[4] = {r.d[0].x, r.d[0].y, r.d[0].z, r.d[0].w}, dw1[4] = {r.d[1].x, r.d[1].y, r.d[1].z, r.d[1].w};
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint2 bv = b_frag<P>(a, L.g, blk * 256 + 32 * j + 8 * L.t);
    int c[4];
    imma_16x8x32<true>(c, r.q[0][j].x, r.q[1][j].x, r.q[0][j].y, r.q[1][j].y, bv.x, bv.y);
    // the scale field of a Q8_0 block is used by magnitude (reference quantization.cpp:85-87)
    const float d0 = scale_field_to_float((uint16_t)((dw0[j >> 1] >> (16 * (j & 1))) & 0xFFFF));
    const float d1 = scale_field_to_float((uint16_t)((dw1[j >> 1] >> (16 * (j & 1))) & 0xFFFF));
    s0 = fmaf(d0, L.wa * (float)c[0] + L.wb * (float)c[1], s0);
    s1 = fmaf(d1, L.wa * (float)c[2] + L.wb * (float)c[3], s1);
  }
  const float sxb = a.sx[blk];
  acc0 = fmaf(sxb, s0, acc0);
  acc1 = fmaf(sxb, s1, acc1);
}

// blocks [blk0, blk1) of one tile for this warp; the next block's loads are in flight while the
// current one is multiplied (two register buffers used alternately)
#define B200_SEGMENT_LOOP(RAW, LOAD, COMPUTE)                   \
  {                                                             \
    RAW bufA, bufB;                                             \
    LOAD(bufA, ra, rb, blk0, L.t);                              \
    int b = blk0;                                               \
    while (true) {                                              \
      if (b + 1 < blk1) LOAD(bufB, ra, rb, b + 1, L.t);         \
      COMPUTE<P>(bufA, a, b, L, acc0, acc1);                    \
      if (++b >= blk1) break;                                   \
      if (b + 1 < blk1) LOAD(bufA, ra, rb, b + 1, L.t);         \
      COMPUTE<P>(bufB, a, b, L, acc0, acc1);                    \
      if (++b >= blk1) break;                                   \
    }                                                           \
  }

template <int P>
__device__ __forceinline__ void tile_segment(int type, const RowPtr& ra, const RowPtr& rb, const ActImage& a, int blk0, int blk1,
                                             LaneCtx L, float wa6, float wb6, float& acc0, float& acc1) {
  if (type == T_Q4_K) {
    B200_SEGMENT_LOOP(RawQ4, load_q4, compute_q4)
  } else if (type == T_Q6_K) {
    L.wa = wa6;
    L.wb = wb6;
    B200_SEGMENT_LOOP(RawQ6, load_q6, compute_q6)
  } else {
    B200_SEGMENT_LOOP(RawQ8, load_q8, compute_q8)
  }
}

// Maps (tile, row-in-tile 0..15) to a segment and a row of it. Ordinary launches: the segments'
// rows are concatenated and cut into 16-row tiles (every segment but the last has a multiple of
// 16 rows). SwiGLU launches: tile = 8 rows of seg 0 (gate) followed by the same 8 rows of seg 1 (up).
__device__ __forceinline__ void tile_row(const GemvParams& p, int tile, int r, int& seg, int& row, bool& valid) {
  if (p.epi == EPI_SWIGLU) {
    seg = r >> 3;
    row = tile * 8 + (r & 7);
    valid = row < p.seg[0].rows;
  } else {
    row = tile * 16 + r;
    seg = 0;
    while (seg + 1 < p.nseg && row >= p.seg[seg].rows) { row -= p.seg[seg].rows; ++seg; }
    valid = row < p.seg[seg].rows;
  }
  if (!valid) row = p.seg[seg].rows - 1;  // loads stay in bounds; the result is discarded
}

template <int P>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_kernel(const GemvParams prm) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ double red_scratch[34];
  __shared__ float part[GEMV_WARPS][2][16];
  __shared__ int part_tile[GEMV_WARPS][2];
  __shared__ float sv[GEMV_WARPS];
  __shared__ int si[GEMV_WARPS];
  const int bidx = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  act_build<P>(smem, prm.x + (size_t)bidx * prm.x_stride, prm.norm_w, prm.eps, prm.K, red_scratch);
  const ActImage a = act_carve(smem, prm.K, P);

  LaneCtx L;
  L.g = lane >> 2;
  L.t = lane & 3;
  const float pw[4] = {1.f, 256.f, 65536.f, 16777216.f};
  {
    const int c0 = 2 * L.t, c1 = 2 * L.t + 1;
    L.wa = c0 < P ? pw[c0] : 0.f;
    L.wb = c1 < P ? pw[c1] : 0.f;
    L.wd = pw[L.t];
  }
  float wa6, wb6;
  {
    const int c0 = 2 * L.t, c1 = 2 * L.t + 1;
    wa6 = c0 < 2 * P ? pw[c0 % P] : 0.f;
    wb6 = c1 < 2 * P ? pw[c1 % P] : 0.f;
  }

  const int nblk = prm.K / 256;
  const int tA = (int)((long long)blockIdx.x * prm.ntiles / gridDim.x);
  const int tB = (int)((long long)(blockIdx.x + 1) * prm.ntiles / gridDim.x);
  float best_v = -INFINITY;
  int best_i = 0x7fffffff;

  for (int tb = tA; tb < tB; tb += GEMV_WARPS) {
    const int nt = min(GEMV_WARPS, tB - tb);
    const int total = nt * nblk;
    const int i0 = (int)((long long)warp * total / GEMV_WARPS), i1 = (int)((long long)(warp + 1) * total / GEMV_WARPS);
    int nseg_used = 0;
    for (int i = i0; i < i1;) {
      const int tl = i / nblk, blk0 = i - tl * nblk;
      const int blk1 = min(nblk, blk0 + (i1 - i));
      int segA, rowA, segB, rowB;
      bool vA, vB;
      tile_row(prm, tb + tl, L.g, segA, rowA, vA);
      tile_row(prm, tb + tl, L.g + 8, segB, rowB, vB);
      const RowPtr ra = row_ptr(prm.seg[segA], rowA, prm.K), rb = row_ptr(prm.seg[segB], rowB, prm.K);
      float acc0 = 0.f, acc1 = 0.f;
      tile_segment<P>(prm.seg[segA].type, ra, rb, a, blk0, blk1, L, wa6, wb6, acc0, acc1);
      acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
      acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
      acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
      acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
      if (nseg_used < 2) {
        if (L.t == 0) {
          part[warp][nseg_used][L.g] = acc0;
          part[warp][nseg_used][L.g + 8] = acc1;
        }
        if (lane == 0) part_tile[warp][nseg_used] = tl;
      }
      ++nseg_used;
      i += blk1 - blk0;
    }
    if (lane == 0)
      for (int s = nseg_used; s < 2; ++s) part_tile[warp][s] = -1;
    __syncthreads();

    if (warp < nt) {  // warp j finishes tile j of this batch: lanes 0..15 own one row each
      const int r = lane & 15;
      float tot = 0.f;
      for (int w = 0; w < GEMV_WARPS; ++w)
#pragma unroll
        for (int s = 0; s < 2; ++s)
          if (part_tile[w][s] == warp) tot += part[w][s][r];
      const int tile = tb + warp;
      if (prm.epi == EPI_SWIGLU) {
        // reference model.cpp:734-735 with silu_cpu (utils.cpp:700-707): (g * 1/(1+exp(-g))) * u
        const float u = __shfl_sync(0xffffffffu, tot, (lane & 7) + 8);
        const int row = tile * 8 + (lane & 7);
        if (lane < 8 && row < prm.seg[0].rows) {
          const float sig = 1.0f / (1.0f + expf(-tot));
          prm.y[(size_t)bidx * prm.y_stride + row] = (tot * sig) * u;
        }
      } else {
        int seg, row;
        bool valid;
        tile_row(prm, tile, r, seg, row, valid);
        const float other = __shfl_xor_sync(0xffffffffu, tot, 1);
        if (lane < 16 && valid) {
          if (prm.epi == EPI_RESID) {
            float* y = prm.y + (size_t)bidx * prm.y_stride + row;
            *y = *y + tot;
          } else if (prm.epi == EPI_QKV_ROPE) {
            float v = tot;
            if (seg < 2) {  // q and k are rotated in adjacent pairs (reference utils.cpp:428-489)
              const int pos = prm.positions[bidx];
              if (pos >= 0 && pos < prm.max_pos) {
                const int i = (row % prm.head_dim) >> 1;
                const float2 cs = *reinterpret_cast<const float2*>(prm.rope + ((size_t)pos * (prm.head_dim >> 1) + i) * 2);
                v = (row & 1) ? __fadd_rn(__fmul_rn(other, cs.y), __fmul_rn(tot, cs.x))
                              : __fsub_rn(__fmul_rn(tot, cs.x), __fmul_rn(other, cs.y));
              }
            }
            float* dst = seg == 0 ? prm.y + (size_t)bidx * prm.y_stride + row
                                  : prm.y2 + (size_t)bidx * prm.y2_stride + (seg == 2 ? prm.seg[1].rows : 0) + row;
            *dst = v;
          } else {
            prm.y[(size_t)bidx * prm.y_stride + row] = tot;
            if (tot > best_v || (tot == best_v && row < best_i)) { best_v = tot; best_i = row; }
          }
        }
      }
    }
    __syncthreads();
  }
  if (prm.amax_val) {  // per-CTA (value, first index) of the rows this CTA produced
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best_v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best_v || (ov == best_v && oi < best_i)) { best_v = ov; best_i = oi; }
    }
    if (lane == 0) { sv[warp] = best_v; si[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float bv = sv[0];
      int bi = si[0];
      for (int w = 1; w < GEMV_WARPS; ++w)
        if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
      prm.amax_val[(size_t)bidx * gridDim.x + blockIdx.x] = bv;
      prm.amax_idx[(size_t)bidx * gridDim.x + blockIdx.x] = bi;
    }
  }
}

}  // namespace b200
