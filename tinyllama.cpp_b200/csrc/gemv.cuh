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
constexpr int GEMV_WARPS = 16;                       // consumer warps
constexpr int GEMV_PROD_WARPS = 4;                   // producer warps, four tile rows each
constexpr int GEMV_THREADS = (GEMV_WARPS + GEMV_PROD_WARPS) * 32;
constexpr int GEMV_SLAB = 16;                        // most 256-element blocks per row per stage (one per consumer warp)
constexpr int GEMV_MAX_STAGES = 6;
constexpr int GEMV_SLOT_BYTES = 54 * 1024;           // one ring stage: 16 rows x up to 16 Q6_K units (+ row padding)

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
  int amax_row_offset;  // added to the row index reported in amax_idx (vocabulary shard offset)
  const float* resid;   // RESID: y = resid + W x (nullptr: y itself)
  int ntiles;           // 16-row tiles (SWIGLU: 8 gate rows + 8 up rows per tile)
  int slab[3];          // 256-element blocks per row per stage (<= GEMV_SLAB), by format (see gemv_type_index)
  int row_stride[3];    // bytes between rows of a stage in shared memory (= 32 mod 128), by format
  int* error_flag;      // set when a bounded wait gives up
};

__host__ __device__ __forceinline__ int gemv_type_index(int type) { return type == T_Q4_K ? 0 : type == T_Q6_K ? 1 : 2; }
// Ring geometry per weight format: the widest slab whose 16 padded rows fit one ring slot.
__host__ __device__ __forceinline__ void gemv_ring_geometry(int K, GemvParams& p) {
  const int nblk = K / 256;
  const int ubs[3] = {144, 208, 272};
  for (int i = 0; i < 3; ++i) {
    int slab = nblk < GEMV_SLAB ? nblk : GEMV_SLAB;
    while (slab > 1 && 16 * ((slab * ubs[i] + 127) / 128 * 128 + 32) > GEMV_SLOT_BYTES) --slab;
    p.slab[i] = slab;
    p.row_stride[i] = (slab * ubs[i] + 127) / 128 * 128 + 32;
  }
}

// ---- shared-memory activation image ------------------------------------------------------
// planes  [P][plane_stride]   digit bytes, element e of plane p at p*plane_stride + e; the stride
//                             is = 32 (mod 128) so the planes read by one mma fall in distinct banks
// sx      [K/256]             float scale of each 256-element block
// xs32d   [4][K/32]           digit d of the sum of x_int over each 32 elements (Q4_K minimum term)
// xs16d   [4][K/16]           the same per 16 elements (Q6_K offset term)
__host__ __device__ __forceinline__ int act_plane_stride(int K) { return (K + 127) / 128 * 128 + 32; }
__host__ __device__ __forceinline__ int act_sx_floats(int K) { return (K / 256 + 3) / 4 * 4; }
__host__ __device__ __forceinline__ size_t act_smem_bytes(int K, int P) {
  return (size_t)P * act_plane_stride(K) + (size_t)act_sx_floats(K) * 4 + (size_t)4 * (K / 32 + 16) + (size_t)4 * (K / 16 + 16);
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
  a.n32 = K / 32 + 16;  // digit-plane strides are offset by 16 bytes so the four digits fall in different banks
  p += 4 * a.n32;
  a.xs16d = p;
  a.n16 = K / 16 + 16;
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

// Quantises the eight elements v[] this lane holds of 256-element block b (after the optional
// RMSNorm scaling) and writes the block's digit planes, digit sums and scale.
template <int P>
__device__ __forceinline__ void act_quantize_block(const ActImage& a, int b, int lane, const float (&vin)[8],
                                                   const float* __restrict__ norm_w, const float4 (&nw)[2], float f) {
  uint8_t* planes = const_cast<uint8_t*>(a.planes);
  float* sx = const_cast<float*>(a.sx);
  uint8_t* xs32d = const_cast<uint8_t*>(a.xs32d);
  uint8_t* xs16d = const_cast<uint8_t*>(a.xs16d);
  // largest magnitude P balanced digits can hold: 127 * (256^P - 1) / 255
  constexpr int QMAX = P == 3 ? 8355711 : (P == 2 ? 32639 : 127);
  const int e0 = b * 256 + lane * 8;
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = vin[i];
  if (norm_w) {
    const float w[8] = {nw[0].x, nw[0].y, nw[0].z, nw[0].w, nw[1].x, nw[1].y, nw[1].z, nw[1].w};
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

// Prologue run by the 16 consumer warps: optional RMSNorm (reference utils.cpp:648-673: mean of
// squares, f = 1/sqrtf(mean + eps), out = x*f*w) then quantisation into the image above. Each
// warp owns the 256-element blocks warp, warp+16, ...; the vector is read from global memory once
// (up to four blocks per warp stay in registers between the two passes).
// XFN(i) returns element i of the input vector.
template <int P, typename XFN>
__device__ void act_build(uint8_t* smem, XFN xfn, const float* __restrict__ norm_w, float eps, int K, float* red /* 18 floats */) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nblk = K / 256;
  constexpr int KEEP = 4;
  float xv[KEEP][8];
  float4 wv[KEEP][2];  // norm weights, requested together with x so the two latencies overlap
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < KEEP; ++k) {
    const int b = warp + k * GEMV_WARPS;
    if (b < nblk && norm_w) {
      wv[k][0] = __ldg(reinterpret_cast<const float4*>(norm_w + b * 256 + lane * 8));
      wv[k][1] = __ldg(reinterpret_cast<const float4*>(norm_w + b * 256 + lane * 8 + 4));
    }
  }
#pragma unroll
  for (int k = 0; k < KEEP; ++k) {
    const int b = warp + k * GEMV_WARPS;
    if (b < nblk) {
      xfn(b * 256 + lane * 8, xv[k]);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(xv[k][i], xv[k][i], ss);
    }
  }
  for (int b = warp + KEEP * GEMV_WARPS; b < nblk; b += GEMV_WARPS) {  // very long vectors: extra blocks are re-read later
    float t[8];
    xfn(b * 256 + lane * 8, t);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(t[i], t[i], ss);
  }
  float f = 1.0f;
  if (norm_w) {
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    consumer_sync();
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < GEMV_WARPS; ++w) t += (double)red[w];
    f = 1.0f / sqrtf((float)(t / (double)K) + eps);
  }
  const ActImage a = act_carve(smem, K, P);
#pragma unroll
  for (int k = 0; k < KEEP; ++k) {
    const int b = warp + k * GEMV_WARPS;
    if (b < nblk) act_quantize_block<P>(a, b, lane, xv[k], norm_w, wv[k], f);
  }
  for (int b = warp + KEEP * GEMV_WARPS; b < nblk; b += GEMV_WARPS) {
    float t[8];
    xfn(b * 256 + lane * 8, t);
    float4 w2[2];
    if (norm_w) {
      w2[0] = __ldg(reinterpret_cast<const float4*>(norm_w + b * 256 + lane * 8));
      w2[1] = __ldg(reinterpret_cast<const float4*>(norm_w + b * 256 + lane * 8 + 4));
    }
    act_quantize_block<P>(a, b, lane, t, norm_w, w2, f);
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
  for (int i = 0; i < (1 << 16); ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity), "r"(20000u)  // park up to ~20 us per probe: waiting warps must not steal issue slots
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
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 15, %0;" ::"n"(GEMV_WARPS * 32) : "memory"); }
// split-phase named barrier over the consumer warps: the warps that only contribute partial sums
// arrive and move on, the warp that finishes the tile waits for all of them
constexpr int GEMV_TILE_BARS = 8;  // tiles that may be in flight between the fastest and the slowest warp
__device__ __forceinline__ void tile_bar_arrive(int id) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "n"(GEMV_WARPS * 32) : "memory"); }
__device__ __forceinline__ void tile_bar_sync(int id) { asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(GEMV_WARPS * 32) : "memory"); }

// ---- per-format work on one 256-element block of a staged 16-row tile ----------------------
// Lane (g = lane >> 2, t = lane & 3) feeds rows g and g + 8 of the tile and the k-slice
// 8t .. 8t+7 of every 32-element group; it receives columns 2t and 2t+1 of the product.
// pa / pb point at this block's unit in rows g / g + 8 of the stage; L.bplane already includes the lane's 8t offset.
struct LaneCtx {
  int g, t;
  float wa, wb;    // 256^plane of columns 2t, 2t+1 for Q4_K / Q8_0 (0 for unused columns)
  float wa6, wb6;  // the same for the Q6_K column layout
  float wd;        // 256^t: weight of digit t in the minimum / offset terms (t = lane & 3)
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


// ---- the streaming pipeline ----------------------------------------------------------------
struct GemvShared {
  unsigned long long full_bar[GEMV_MAX_STAGES];
  unsigned long long empty_bar[GEMV_MAX_STAGES];
  float red[GEMV_WARPS + 2];
  float part[GEMV_TILE_BARS][GEMV_WARPS][16];
  float sv[GEMV_WARPS];
  int si[GEMV_WARPS];
  int abort_flag;
};

struct PipeCtx {
  GemvShared* sh;
  uint8_t* act;   // activation image
  uint8_t* ring;  // nstages slots of GEMV_SLOT_BYTES
  int nstages;
  int slot;       // ring slot of the next stage (producer and consumers count alike)
  int use;        // how many times the ring has wrapped
  int gt;         // tiles finished so far
  __device__ __forceinline__ void next_stage() {
    if (++slot == nstages) { slot = 0; ++use; }
  }
};

__device__ __forceinline__ void pipe_init(GemvShared* sh, int nstages) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < nstages; ++s) {
      mbar_init(&sh->full_bar[s], GEMV_PROD_WARPS);
      mbar_init(&sh->empty_bar[s], GEMV_WARPS);
    }
    sh->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
}

__device__ __forceinline__ void pipe_fail(const GemvParams& prm, GemvShared* sh) {
  sh->abort_flag = 1;
  if (prm.error_flag) atomicExch(prm.error_flag, 1);
}

// Producer warp pw (0..3): lanes 0..3 copy rows 4*pw .. 4*pw+3 of every stage of this CTA's tiles.
__device__ __forceinline__ void gemv_produce(const GemvParams& prm, PipeCtx& pc, int pw, int lane, int cta, int ncta) {
  GemvShared* sh = pc.sh;
  const int nblk = prm.K / 256;
  // tiles are dealt round-robin over the CTAs so that launches mixing formats of different cost
  // (Q6_K tiles take about twice as long as Q4_K ones) stay balanced
  for (int tile = cta; tile < prm.ntiles; tile += ncta) {
    int seg = 0, row = 0;
    bool valid;
    tile_row(prm, tile, 4 * pw + (lane & 3), seg, row, valid);
    const int type = prm.seg[seg].type, ti = gemv_type_index(type);
    const int ub = gemv_unit_bytes(type);
    const int slab_blocks = prm.slab[ti], RSS = prm.row_stride[ti];
    const int nslab = (nblk + slab_blocks - 1) / slab_blocks;
    const uint8_t* src_row = prm.seg[seg].w + (size_t)row * nblk * ub;
    for (int slab = 0; slab < nslab; ++slab, pc.next_stage()) {
      const int slot = pc.slot, use = pc.use;
      if (use > 0) {
        if (lane == 0 && !*(volatile int*)&sh->abort_flag && !mbar_wait(&sh->empty_bar[slot], (use - 1) & 1)) pipe_fail(prm, sh);
        __syncwarp();
      }
      const int b0 = slab * slab_blocks, nb = min(slab_blocks, nblk - b0);
      const uint32_t bytes = (uint32_t)(nb * ub);
      if (lane == 0) mbar_expect_tx(&sh->full_bar[slot], bytes * 4);
      __syncwarp();
      if (lane < 4)
        bulk_g2s(pc.ring + (size_t)slot * GEMV_SLOT_BYTES + (size_t)(4 * pw + lane) * RSS, src_row + (size_t)b0 * ub, bytes,
                 &sh->full_bar[slot]);
    }
  }
}

// The 16 consumer warps: prologue, then one block column per warp per stage, then the row epilogue.
template <int P, typename XFN>
__device__ __forceinline__ void gemv_consume(const GemvParams& prm, PipeCtx& pc, XFN xfn, int bidx, int cta, int ncta, float& best_v,
                                             int& best_i) {
  GemvShared* sh = pc.sh;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  act_build<P>(pc.act, xfn, prm.norm_w, prm.eps, prm.K, sh->red);
  const ActImage a = act_carve(pc.act, prm.K, P);

  LaneCtx L;
  L.g = lane >> 2;
  L.t = lane & 3;
  {
    const int c0 = 2 * L.t, c1 = 2 * L.t + 1;
    auto p256 = [](int e) { return __int_as_float((127 + 8 * e) << 23); };  // 256^e
    L.wa = c0 < P ? p256(c0) : 0.f;
    L.wb = c1 < P ? p256(c1) : 0.f;
    L.wa6 = c0 < 2 * P ? p256(c0 % P) : 0.f;
    L.wb6 = c1 < 2 * P ? p256(c1 % P) : 0.f;
    L.wd = p256(L.t);
    L.bplane = a.planes + (size_t)(L.g < P ? L.g : 0) * a.plane_stride + 8 * L.t;
  }
  const int nblk = prm.K / 256;

  for (int tile = cta; tile < prm.ntiles; tile += ncta, ++pc.gt) {
    int segA, rowA, segB, rowB;
    bool vA, vB;
    tile_row(prm, tile, L.g, segA, rowA, vA);
    tile_row(prm, tile, L.g + 8, segB, rowB, vB);
    const int type = prm.seg[segA].type, ti = gemv_type_index(type);
    const int ub = gemv_unit_bytes(type);
    const int slab_blocks = prm.slab[ti], RSS = prm.row_stride[ti];
    const int nslab = (nblk + slab_blocks - 1) / slab_blocks;
    float acc0 = 0.f, acc1 = 0.f;
    for (int slab = 0; slab < nslab; ++slab, pc.next_stage()) {
      const int slot = pc.slot, use = pc.use;
      const int b0 = slab * slab_blocks, nb = min(slab_blocks, nblk - b0);
      const int blk = b0 + warp;
      float d0 = 0.f, d1 = 0.f;
      if (type == T_Q6_K && warp < nb) {  // requested before the wait so its latency hides behind it
        d0 = half_bits_to_float(ldg16(prm.seg[segA].d + ((size_t)rowA * nblk + blk) * 2));
        d1 = half_bits_to_float(ldg16(prm.seg[segB].d + ((size_t)rowB * nblk + blk) * 2));
      }
      if (lane == 0 && !*(volatile int*)&sh->abort_flag && !mbar_wait(&sh->full_bar[slot], use & 1)) pipe_fail(prm, sh);
      __syncwarp();  // one lane probes; the rest of the warp parks here
      if (warp < nb) {
        const uint8_t* pa = pc.ring + (size_t)slot * GEMV_SLOT_BYTES + (size_t)L.g * RSS + (size_t)warp * ub;
        const uint8_t* pb = pa + (size_t)8 * RSS;
        if (type == T_Q4_K) compute_q4<P>(pa, pb, a, blk, L, acc0, acc1);
        else if (type == T_Q6_K) compute_q6<P>(pa, pb, d0, d1, a, blk, L, acc0, acc1);
        else compute_q8<P>(pa, pb, a, blk, L, acc0, acc1);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->empty_bar[slot]);
    }
    // ---- tile finished: fold the four k-slices, hand the partial sums to the finishing warp ----
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
    // A warp can run at most nstages (< GEMV_TILE_BARS) tiles ahead of the slowest one, so slot and
    // barrier gt % GEMV_TILE_BARS are free again when they come round.
    const int pp = pc.gt % GEMV_TILE_BARS;
    if (L.t == 0) {
      sh->part[pp][warp][L.g] = acc0;
      sh->part[pp][warp][L.g + 8] = acc1;
    }
    if (warp != (pc.gt & (GEMV_WARPS - 1))) {
      __syncwarp();
      tile_bar_arrive(1 + pp);
      continue;
    }
    tile_bar_sync(1 + pp);  // this warp finishes the tile; lanes 0..15 own one row each
    const int r = lane & 15;
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < GEMV_WARPS; ++w) tot += sh->part[pp][w][r];
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
          const float* rs = (prm.resid ? prm.resid : prm.y) + (size_t)bidx * prm.y_stride + row;
          prm.y[(size_t)bidx * prm.y_stride + row] = *rs + tot;
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
          const int grow = row + prm.amax_row_offset;
          if (tot > best_v || (tot == best_v && grow < best_i)) { best_v = tot; best_i = grow; }
        }
      }
    }
  }
}

// Per-CTA (value, first index) of the rows this CTA produced, from the per-lane running bests.
__device__ __forceinline__ void gemv_store_argmax(const GemvParams& prm, GemvShared* sh, float best_v, int best_i, int bidx, int cta,
                                                  int ncta) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best_v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best_v || (ov == best_v && oi < best_i)) { best_v = ov; best_i = oi; }
  }
  if (lane == 0) { sh->sv[warp] = best_v; sh->si[warp] = best_i; }
  consumer_sync();
  if (threadIdx.x == 0) {
    float bv = sh->sv[0];
    int bi = sh->si[0];
    for (int w = 1; w < GEMV_WARPS; ++w)
      if (sh->sv[w] > bv || (sh->sv[w] == bv && sh->si[w] < bi)) { bv = sh->sv[w]; bi = sh->si[w]; }
    prm.amax_val[(size_t)bidx * ncta + cta] = bv;
    prm.amax_idx[(size_t)bidx * ncta + cta] = bi;
  }
}

__host__ __device__ __forceinline__ size_t gemv_ring_offset(int K, int P) { return (act_smem_bytes(K, P) + 127) / 128 * 128; }

struct XFromGlobal {
  const float* x;
  __device__ __forceinline__ void operator()(int e, float (&v)[8]) const {
    const float4 a = *reinterpret_cast<const float4*>(x + e), b = *reinterpret_cast<const float4*>(x + e + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};

// One launch = one fused matvec for blockIdx.y's activation vector; one persistent CTA per SM.
template <int P>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_kernel(const GemvParams prm, int nstages) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ GemvShared sh;
  PipeCtx pc;
  pc.sh = &sh;
  pc.act = smem;
  pc.ring = smem + gemv_ring_offset(prm.K, P);
  pc.nstages = nstages;
  pc.slot = 0;
  pc.use = 0;
  pc.gt = 0;
  pipe_init(&sh, nstages);
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp >= GEMV_WARPS) {
    // weights never depend on the previous kernel, so the producers start before the consumers' dependency wait
    gemv_produce(prm, pc, warp - GEMV_WARPS, lane, blockIdx.x, gridDim.x);
    return;
  }
  pdl_wait();  // the activation vector (and the buffers this kernel writes) belong to the previous kernel until here
  float best_v = -INFINITY;
  int best_i = 0x7fffffff;
  XFromGlobal xfn{prm.x + (size_t)blockIdx.y * prm.x_stride};
  gemv_consume<P>(prm, pc, xfn, blockIdx.y, blockIdx.x, gridDim.x, best_v, best_i);
  if (prm.amax_val) gemv_store_argmax(prm, &sh, best_v, best_i, blockIdx.y, blockIdx.x, gridDim.x);
}

}  // namespace b200
