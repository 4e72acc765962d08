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
// Data movement. One persistent CTA per SM takes a contiguous range of 16-row tiles. A producer
// warp streams every tile into a ring of shared-memory stages with bulk asynchronous copies
// (cp.async.bulk, completion on an mbarrier): one copy per row of up to 16 consecutive blocks, so
// HBM sees long contiguous runs (a whole 16-row tile of a 4096-wide Q4_K matrix is 36 KB of
// consecutive addresses) and several stages are in flight without holding registers. The 16
// consumer warps each take one 256-element block column of the staged tile, build their mma
// operands from shared memory, and their partial row sums meet in a fixed order (deterministic).
// The first stages are requested before the activation prologue runs, and the kernel supports
// programmatic dependent launch: weights are prefetched while the previous kernel drains, and
// only then does it wait for that kernel's results.
//
// HBM traffic per launch = the packed bytes of the rows (each read exactly once) plus the
// activation vector; that is the algorithmic byte count.
#pragma once
#include "common.cuh"
#include "dequant.cuh"

namespace b200 {

enum : int { EPI_STORE = 0, EPI_RESID = 1, EPI_QKV_ROPE = 2, EPI_SWIGLU = 3 };
constexpr int GEMV_WARPS = 16;                       // consumer warps; one more warp produces
constexpr int GEMV_THREADS = (GEMV_WARPS + 1) * 32;
constexpr int GEMV_SLAB = 16;                        // 256-element blocks per row per stage
constexpr int GEMV_MAX_STAGES = 4;

// Device-resident form of a weight matrix, row-major, one "unit" per 256 elements of a row:
//   Q4_K  unit = the 144-byte block exactly as in the file
//   Q6_K  unit = 208 bytes: ql[128] | qh[64] | scales[16] of the block; the block's fp16 d lives
//         in a separate plane d[row][block] (a 210-byte block cannot sit on a 16-byte boundary)
//   Q8_0  unit = 272 bytes: the 8 x 32 quants of eight consecutive blocks, then their 8 fp16 d
// The byte count is that of the file in every case; nothing is expanded.
__host__ __device__ __forceinline__ int gemv_unit_bytes(int type) { return type == T_Q4_K ? 144 : type == T_Q6_K ? 208 : 272; }

struct GemvSeg {
  const uint8_t* w;  // units, [rows][K/256][unit]
  const uint8_t* d;  // Q6_K only: fp16 [rows][K/256]
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
  int nstages;          // ring depth
  int row_stride;       // bytes between rows of a stage in shared memory (= 32 mod 128)
  int* error_flag;      // set when a bounded wait gives up
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

__device__ __forceinline__ void consumer_sync();

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
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = GEMV_WARPS;  // consumer warps only
  float f = 1.0f;
  if (norm_w) {
    float ss = 0.f;
    for (int i = tid * 4; i < K; i += GEMV_WARPS * 32 * 4) {
      float4 v = *reinterpret_cast<const float4*>(x + i);
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    double ds = (double)ss;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ds += __shfl_xor_sync(0xffffffffu, ds, o);
    if (lane == 0) red[warp] = ds;
    consumer_sync();
    if (warp == 0) {
      double t = lane < nwarps ? red[lane] : 0.0;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      if (lane == 0) {
        float mean = (float)(t / (double)K);
        reinterpret_cast<float*>(red + 32)[0] = 1.0f / sqrtf(mean + eps);
      }
    }
    consumer_sync();
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
  consumer_sync();
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


// ---- mbarrier / bulk-copy / launch-dependency primitives -----------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(void* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(void* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait: gives up after a fixed number of probes and reports failure instead of spinning forever.
__device__ __forceinline__ bool mbar_wait(void* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (int i = 0; i < (1 << 20); ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
// global -> shared bulk copy (16-byte aligned addresses, size a multiple of 16); completion is
// signalled on the mbarrier as transferred bytes
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, void* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(GEMV_WARPS * 32) : "memory"); }

// ---- per-format work on one 256-element block of a staged 16-row tile ----------------------
// Lane (g = lane >> 2, t = lane & 3) feeds rows g and g + 8 of the tile and the k-slice
// 8t .. 8t+7 of every 32-element group; it receives columns 2t and 2t+1 of the product.
// pa / pb point at this block's unit in rows g / g + 8 of the stage; L.bplane already includes the lane's 8t offset.
struct LaneCtx {
  int g, t;
  float wa, wb;    // 256^plane of columns 2t, 2t+1 for Q4_K / Q8_0 (0 for unused columns)
  float wa6, wb6;  // the same for the Q6_K column layout
  float wd;        // 256^t: weight of digit t in the minimum / offset terms
  const uint8_t* bplane;  // digit plane this lane's B column reads (any valid plane for unused columns)
};

template <int P>
__device__ __forceinline__ void compute_q4(const uint8_t* pa, const uint8_t* pb, const ActImage& a, int blk, const LaneCtx& L,
                                           float& acc0, float& acc1) {
  const uint4 h0 = *reinterpret_cast<const uint4*>(pa), h1 = *reinterpret_cast<const uint4*>(pb);
  // eight 6-bit scales and minima per row, four to a word (get_scale_min_k4 of the reference,
  // quantization.cpp:145-155, applied to four sub-blocks at once)
  const uint32_t scA0 = h0.y & 0x3F3F3F3Fu, mnA0 = h0.z & 0x3F3F3F3Fu;
  const uint32_t scB0 = (h0.w & 0x0F0F0F0Fu) | ((h0.y >> 2) & 0x30303030u);
  const uint32_t mnB0 = ((h0.w >> 4) & 0x0F0F0F0Fu) | ((h0.z >> 2) & 0x30303030u);
  const uint32_t scA1 = h1.y & 0x3F3F3F3Fu, mnA1 = h1.z & 0x3F3F3F3Fu;
  const uint32_t scB1 = (h1.w & 0x0F0F0F0Fu) | ((h1.y >> 2) & 0x30303030u);
  const uint32_t mnB1 = ((h1.w >> 4) & 0x0F0F0F0Fu) | ((h1.z >> 2) & 0x30303030u);
  int Jlo[4] = {0, 0, 0, 0}, Jhi[4] = {0, 0, 0, 0};
  const uint8_t* bp = L.bplane + blk * 256;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint2 qa = *reinterpret_cast<const uint2*>(pa + 16 + 32 * c + 8 * L.t), qb = *reinterpret_cast<const uint2*>(pb + 16 + 32 * c + 8 * L.t);
    const uint2 bl = *reinterpret_cast<const uint2*>(bp + 64 * c), bh = *reinterpret_cast<const uint2*>(bp + 64 * c + 32);
    int cl[4], ch[4];
    imma_16x8x32<false>(cl, qa.x & 0x0F0F0F0Fu, qb.x & 0x0F0F0F0Fu, qa.y & 0x0F0F0F0Fu, qb.y & 0x0F0F0F0Fu, bl.x, bl.y);
    imma_16x8x32<false>(ch, qa.x & 0xF0F0F0F0u, qb.x & 0xF0F0F0F0u, qa.y & 0xF0F0F0F0u, qb.y & 0xF0F0F0F0u, bh.x, bh.y);  // 16 x
    const uint32_t s0 = c < 2 ? scA0 : scB0, s1 = c < 2 ? scA1 : scB1;
    const int sl0 = byte_u(s0, (2 * c) & 3), sh0 = byte_u(s0, (2 * c + 1) & 3);
    const int sl1 = byte_u(s1, (2 * c) & 3), sh1 = byte_u(s1, (2 * c + 1) & 3);
    Jlo[0] += sl0 * cl[0]; Jlo[1] += sl0 * cl[1]; Jlo[2] += sl1 * cl[2]; Jlo[3] += sl1 * cl[3];
    Jhi[0] += sh0 * ch[0]; Jhi[1] += sh0 * ch[1]; Jhi[2] += sh1 * ch[2]; Jhi[3] += sh1 * ch[3];
  }
  const float f0 = L.wa * fmaf((float)Jhi[0], 0.0625f, (float)Jlo[0]) + L.wb * fmaf((float)Jhi[1], 0.0625f, (float)Jlo[1]);
  const float f1 = L.wa * fmaf((float)Jhi[2], 0.0625f, (float)Jlo[2]) + L.wb * fmaf((float)Jhi[3], 0.0625f, (float)Jlo[3]);
  // minimum term: sum_sub m_sub * X_sub, digit t of X handled by lane t
  const uint2 xw = *reinterpret_cast<const uint2*>(a.xs32d + (size_t)L.t * a.n32 + blk * 8);
  const int M0 = dp4a_us(mnB0, xw.y, dp4a_us(mnA0, xw.x, 0));
  const int M1 = dp4a_us(mnB1, xw.y, dp4a_us(mnA1, xw.x, 0));
  const float sxb = a.sx[blk];
  const float2 dm0 = __half22float2(*reinterpret_cast<const __half2*>(&h0.x));
  const float2 dm1 = __half22float2(*reinterpret_cast<const __half2*>(&h1.x));
  acc0 = fmaf(sxb, dm0.x * f0 - dm0.y * (L.wd * (float)M0), acc0);
  acc1 = fmaf(sxb, dm1.x * f1 - dm1.y * (L.wd * (float)M1), acc1);
}

// Q6_K: a group of 32 consecutive elements holds two 16-element sub-blocks. Lanes t = 0,1 carry
// the first one, t = 2,3 the second; columns 0..P-1 see only the first (B is zero for t >= 2),
// columns P..2P-1 only the second, so one instruction yields both sub-block sums separately.
template <int P>
__device__ __forceinline__ void compute_q6(const uint8_t* pa, const uint8_t* pb, float d0, float d1, const ActImage& a, int blk,
                                           const LaneCtx& L, float& acc0, float& acc1) {
  const int col = L.g, sub_of_col = col / P, plane = col - sub_of_col * P;
  const bool b_on = col < 2 * P && sub_of_col == (L.t >> 1);
  const uint32_t selA = (uint32_t)((2 * L.t) / P), selB = (uint32_t)((2 * L.t + 1) / P);
  const uint8_t* bp = a.planes + (size_t)(b_on ? plane : 0) * a.plane_stride + blk * 256 + 8 * L.t;
  const uint4 sc0 = *reinterpret_cast<const uint4*>(pa + 192), sc1 = *reinterpret_cast<const uint4*>(pb + 192);
  int J[4] = {0, 0, 0, 0};
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint2 ha = *reinterpret_cast<const uint2*>(pa + 128 + 32 * h + 8 * L.t), hb = *reinterpret_cast<const uint2*>(pb + 128 + 32 * h + 8 * L.t);
    const uint32_t hw[2][2] = {{ha.x, ha.y}, {hb.x, hb.y}};
#pragma unroll
    for (int g4 = 0; g4 < 4; ++g4) {
      uint32_t av[2][2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const uint2 lw = *reinterpret_cast<const uint2*>((i ? pb : pa) + 64 * h + 32 * (g4 & 1) + 8 * L.t);
        const uint32_t l2[2] = {lw.x, lw.y};
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          const uint32_t nib = g4 < 2 ? (l2[w] & 0x0F0F0F0Fu) : ((l2[w] >> 4) & 0x0F0F0F0Fu);
          const uint32_t hi = g4 == 0 ? (hw[i][w] << 4) : g4 == 1 ? (hw[i][w] << 2) : g4 == 2 ? hw[i][w] : (hw[i][w] >> 2);
          av[i][w] = nib | (hi & 0x30303030u);
        }
      }
      uint2 bv = *reinterpret_cast<const uint2*>(bp + 128 * h + 32 * g4);
      if (!b_on) bv = make_uint2(0u, 0u);
      int c[4];
      imma_16x8x32<false>(c, av[0][0], av[1][0], av[0][1], av[1][1], bv.x, bv.y);
      // sub-scale index within the block: 8h + 2*g4 + (0|1) -> word (2h + g4/2), byte 2(g4&1) + sel
      const int wsel = 2 * h + (g4 >> 1);
      const uint32_t w0 = wsel == 0 ? sc0.x : wsel == 1 ? sc0.y : wsel == 2 ? sc0.z : sc0.w;
      const uint32_t w1 = wsel == 0 ? sc1.x : wsel == 1 ? sc1.y : wsel == 2 ? sc1.z : sc1.w;
      const uint32_t bA = 2 * (g4 & 1) + selA, bB = 2 * (g4 & 1) + selB;
      J[0] += byte_s(w0, bA) * c[0];
      J[1] += byte_s(w0, bB) * c[1];
      J[2] += byte_s(w1, bA) * c[2];
      J[3] += byte_s(w1, bB) * c[3];
    }
  }
  const float f0 = L.wa6 * (float)J[0] + L.wb6 * (float)J[1];
  const float f1 = L.wa6 * (float)J[2] + L.wb6 * (float)J[3];
  // offset term: the stored quants are q + 32, so subtract 32 * sum_sub sc_sub * X_sub (digit t per lane)
  const uint4 xw = *reinterpret_cast<const uint4*>(a.xs16d + (size_t)L.t * a.n16 + blk * 16);
  const int C0 = dp4a_ss(sc0.w, xw.w, dp4a_ss(sc0.z, xw.z, dp4a_ss(sc0.y, xw.y, dp4a_ss(sc0.x, xw.x, 0))));
  const int C1 = dp4a_ss(sc1.w, xw.w, dp4a_ss(sc1.z, xw.z, dp4a_ss(sc1.y, xw.y, dp4a_ss(sc1.x, xw.x, 0))));
  const float sxb = a.sx[blk];
  acc0 = fmaf(sxb * d0, f0 - 32.f * (L.wd * (float)C0), acc0);
  acc1 = fmaf(sxb * d1, f1 - 32.f * (L.wd * (float)C1), acc1);
}

template <int P>
__device__ __forceinline__ void compute_q8(const uint8_t* pa, const uint8_t* pb, const ActImage& a, int blk, const LaneCtx& L,
                                           float& acc0, float& acc1) {
  const uint4 da = *reinterpret_cast<const uint4*>(pa + 256), db = *reinterpret_cast<const uint4*>(pb + 256);
  const uint32_t dw0[4] = {da.x, da.y, da.z, da.w}, dw1[4] = {db.x, db.y, db.z, db.w};
  const uint8_t* bp = L.bplane + blk * 256;
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint2 qa = *reinterpret_cast<const uint2*>(pa + 32 * j + 8 * L.t), qb = *reinterpret_cast<const uint2*>(pb + 32 * j + 8 * L.t);
    const uint2 bv = *reinterpret_cast<const uint2*>(bp + 32 * j);
    int c[4];
    imma_16x8x32<true>(c, qa.x, qb.x, qa.y, qb.y, bv.x, bv.y);
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

__host__ __device__ __forceinline__ size_t gemv_ring_offset(int K, int P) { return (act_smem_bytes(K, P) + 127) / 128 * 128; }

template <int P>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_kernel(const GemvParams prm) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) unsigned long long full_bar[GEMV_MAX_STAGES];
  __shared__ __align__(8) unsigned long long empty_bar[GEMV_MAX_STAGES];
  __shared__ double red_scratch[34];
  __shared__ float part[2][GEMV_WARPS][16];
  __shared__ float sv[GEMV_WARPS];
  __shared__ int si[GEMV_WARPS];
  __shared__ int abort_flag;
  const int bidx = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int D = prm.nstages, RSS = prm.row_stride;
  uint8_t* ring = smem + gemv_ring_offset(prm.K, P);
  const size_t stage_bytes = (size_t)16 * RSS;

  const int nblk = prm.K / 256;
  const int nslab = (nblk + GEMV_SLAB - 1) / GEMV_SLAB;
  const int tA = (int)((long long)blockIdx.x * prm.ntiles / gridDim.x);
  const int tB = (int)((long long)(blockIdx.x + 1) * prm.ntiles / gridDim.x);
  const int nst_total = (tB - tA) * nslab;

  if (threadIdx.x == 0) {
    for (int s = 0; s < D; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], GEMV_WARPS);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == GEMV_WARPS) {
    // ---- producer: lanes 0..15 each copy one row of the tile slab; weights never depend on the
    // previous kernel, so this starts before the dependency wait of the consumers ----
    for (int s = 0; s < nst_total; ++s) {
      const int slot = s % D, use = s / D;
      if (use > 0) {
        bool ok = true;
        if (lane == 0 && !*(volatile int*)&abort_flag) ok = mbar_wait(&empty_bar[slot], (use - 1) & 1);
        if (!ok) { abort_flag = 1; if (prm.error_flag) atomicExch(prm.error_flag, 1); }
        __syncwarp();
      }
      const int tile = tA + s / nslab, slab = s - (s / nslab) * nslab;
      const int b0 = slab * GEMV_SLAB, nb = min(GEMV_SLAB, nblk - b0);
      int seg, row;
      bool valid;
      tile_row(prm, tile, lane & 15, seg, row, valid);
      const int ub = gemv_unit_bytes(prm.seg[seg].type);
      const uint32_t bytes = (uint32_t)(nb * ub);
      if (lane == 0) mbar_expect_tx(&full_bar[slot], bytes * 16);
      __syncwarp();
      if (lane < 16) {
        const uint8_t* src = prm.seg[seg].w + ((size_t)row * nblk + b0) * ub;
        bulk_g2s(ring + slot * stage_bytes + (size_t)lane * RSS, src, bytes, &full_bar[slot]);
      }
    }
    return;
  }

  // ---- consumers ----
  pdl_wait();  // the activation vector (and the buffers this kernel writes) belong to the previous kernel until here
  act_build<P>(smem, prm.x + (size_t)bidx * prm.x_stride, prm.norm_w, prm.eps, prm.K, red_scratch);
  const ActImage a = act_carve(smem, prm.K, P);

  LaneCtx L;
  L.g = lane >> 2;
  L.t = lane & 3;
  {
    const float pw[4] = {1.f, 256.f, 65536.f, 16777216.f};
    const int c0 = 2 * L.t, c1 = 2 * L.t + 1;
    L.wa = c0 < P ? pw[c0] : 0.f;
    L.wb = c1 < P ? pw[c1] : 0.f;
    L.wa6 = c0 < 2 * P ? pw[c0 % P] : 0.f;
    L.wb6 = c1 < 2 * P ? pw[c1 % P] : 0.f;
    L.wd = pw[L.t];
    L.bplane = a.planes + (size_t)(L.g < P ? L.g : 0) * a.plane_stride + 8 * L.t;
  }

  float best_v = -INFINITY;
  int best_i = 0x7fffffff;
  float acc0 = 0.f, acc1 = 0.f;
  for (int s = 0; s < nst_total; ++s) {
    const int slot = s % D, use = s / D;
    const int tl = s / nslab, slab = s - tl * nslab;
    const int tile = tA + tl;
    const int b0 = slab * GEMV_SLAB, nb = min(GEMV_SLAB, nblk - b0);
    int segA, rowA, segB, rowB;
    bool vA, vB;
    tile_row(prm, tile, L.g, segA, rowA, vA);
    tile_row(prm, tile, L.g + 8, segB, rowB, vB);
    const int type = prm.seg[segA].type;
    const int blk = b0 + warp;
    float d0 = 0.f, d1 = 0.f;
    if (type == T_Q6_K && warp < nb) {  // requested before the wait so its latency hides behind it
      d0 = half_bits_to_float(ldg16(prm.seg[segA].d + ((size_t)rowA * nblk + blk) * 2));
      d1 = half_bits_to_float(ldg16(prm.seg[segB].d + ((size_t)rowB * nblk + blk) * 2));
    }
    if (!*(volatile int*)&abort_flag) {
      if (!mbar_wait(&full_bar[slot], use & 1)) {
        abort_flag = 1;
        if (prm.error_flag) atomicExch(prm.error_flag, 1);
      }
    }
    if (warp < nb) {
      const int ub = gemv_unit_bytes(type);
      const uint8_t* pa = ring + slot * stage_bytes + (size_t)L.g * RSS + (size_t)warp * ub;
      const uint8_t* pb = pa + (size_t)8 * RSS;
      if (type == T_Q4_K) compute_q4<P>(pa, pb, a, blk, L, acc0, acc1);
      else if (type == T_Q6_K) compute_q6<P>(pa, pb, d0, d1, a, blk, L, acc0, acc1);
      else compute_q8<P>(pa, pb, a, blk, L, acc0, acc1);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[slot]);
    if (slab != nslab - 1) continue;

    // ---- tile finished: fold the four k-slices, meet the other warps, finish the rows ----
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
    const int pp = tl & 1;
    if (L.t == 0) {
      part[pp][warp][L.g] = acc0;
      part[pp][warp][L.g + 8] = acc1;
    }
    acc0 = acc1 = 0.f;
    consumer_sync();
    if (warp == (tl & (GEMV_WARPS - 1))) {  // lanes 0..15 own one row each
      const int r = lane & 15;
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < GEMV_WARPS; ++w) tot += part[pp][w][r];
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
  }
  if (prm.amax_val) {  // per-CTA (value, first index) of the rows this CTA produced
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best_v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best_v || (ov == best_v && oi < best_i)) { best_v = ov; best_i = oi; }
    }
    if (lane == 0) { sv[warp] = best_v; si[warp] = best_i; }
    consumer_sync();
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
