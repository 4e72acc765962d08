// Fused dequant-matvec over packed Q8_0 / Q4_K / Q6_K blocks for decode (one activation vector
// per launch column).
//
// Arithmetic. The activation vector is quantised once per CTA into P balanced base-256 digit
// planes (x ~ sx[blk] * x_int, x_int = sum_p digit_p * 256^p, every digit a signed byte, one scale
// per 256 elements; P = 3 gives 24-bit activations, i.e. FP32-grade). Weights stay the integers
// that are stored in the blocks. A warp owns one 256-element block column of a 16-row group;
// every 32 elements it issues one integer tensor-core instruction (mma.sync m16n8k32, u8/s8 x s8
// -> s32) whose 16 x 32 A operand is built in registers from the packed nibbles / 6-bit fields
// with a few logic ops, and whose B columns are the digit planes. The exact integer sub-block
// sums are multiplied by the integer sub-block scales (6-bit for Q4_K, int8 for Q6_K) with
// integer multiply-adds; one float multiply per (row, 256-block) applies the fp16 block scale.
// The Q4_K minimum term and the Q6_K "-32" offset use per-sub-block sums of the activations, also
// kept as digit bytes, and are evaluated with dp4a.
//
// Data movement. Weights live in HBM as "stage images": the matrix is cut into tiles of 16*R
// rows and slabs of S <= 16 blocks along K, and each (tile, slab) is stored as one contiguous
// run laid out exactly as it will sit in shared memory (rows padded to a stride = 32 mod 128 so
// the fragment loads are free of bank conflicts). One persistent CTA per SM walks its tiles:
// 16 consumer warps and one producer warp. One lane of the producer requests every stage with ONE
// bulk asynchronous copy (cp.async.bulk, completion counted on an mbarrier) into a ring of
// shared-memory slots as soon as the slot is empty (a second mbarrier per slot counts the consumer
// warps that are done with it), so HBM sees runs of 20-70 KB, several stages are in flight
// without holding registers, and the consumers contain no copy code at all. The 16 consumer warps
// each take one (row group, block) task of the staged slab. When a row has at most 16 blocks a
// warp meets the same block column in every tile, and its B fragments (the activation digits)
// stay in registers for the whole launch. Partial row sums are parked in shared memory and the
// rows of up to 16 tiles are finished together, in a fixed order (deterministic), by all threads.
// The kernel supports programmatic dependent launch: the producer never depends on the previous
// kernel and starts at once; only the consumers wait for that kernel's results.
//
// HBM traffic per launch = the packed bytes of the rows (each read exactly once, plus the row
// padding: 1.4 % for a 4096-wide Q4_K matrix) plus the activation vector.
#pragma once
#include "common.cuh"
#include "dequant.cuh"

namespace b200 {

enum : int { EPI_STORE = 0, EPI_RESID = 1, EPI_QKV_ROPE = 2, EPI_SWIGLU = 3, EPI_PEER = 4 };
constexpr int GEMV_MAX_TP = 8;
constexpr int GEMV_WARPS = 16;                        // consumer warps
constexpr int GEMV_CONSUMER_THREADS = GEMV_WARPS * 32;
constexpr int GEMV_THREADS = GEMV_CONSUMER_THREADS + 32;  // + one producer warp
constexpr int GEMV_MAX_STAGES = 8;
constexpr int GEMV_NTB = 16;                          // tiles whose partial sums are parked before their rows are finished
constexpr int GEMV_SMEM_BUDGET = 208 * 1024;          // dynamic shared memory (activation image + ring)

// One "unit" per 256 elements of a row:
//   Q4_K  unit = the 144-byte block exactly as in the file
//   Q6_K  unit = 208 bytes: ql[128] | qh[64] | scales[16] of the block; the fp16 d of the S blocks
//         of a stage row follow the row's units (a 210-byte block cannot sit on a 16-byte boundary)
//   Q8_0  unit = 272 bytes: the 8 x 32 quants of eight consecutive blocks, then their 8 fp16 d
// The byte count is that of the file in every case; nothing is expanded.
__host__ __device__ __forceinline__ int gemv_unit_bytes(int type) { return type == T_Q4_K ? 144 : type == T_Q6_K ? 208 : 272; }

// How a [rows][K] matrix of one block type is cut into ring stages. nblk, nslab, S, S_last and R
// depend on K only, so segments of different types in one launch share them.
struct GemvGeom {
  int nblk;      // 256-element blocks per row
  int nslab;     // stages per tile
  int S, S_last; // blocks per row in a full stage / in the last stage of a tile
  int R;         // 16-row groups per tile (> 1 only for short rows, so that all 16 warps have a task)
  int ub;        // unit bytes
  int RS, RS_last;        // bytes between rows of a stage (= 32 mod 128)
  int d_off, d_off_last;  // Q6_K: offset of the row's fp16 block scales within a stage row
  uint32_t stage_bytes, stage_bytes_last, tile_bytes;
};

__host__ __device__ __forceinline__ int gemv_pad_row(int bytes) { return (bytes + 95) / 128 * 128 + 32; }

__host__ __device__ inline GemvGeom gemv_geometry(int type, int K) {
  GemvGeom g;
  g.nblk = K / 256;
  g.ub = gemv_unit_bytes(type);
  g.nslab = (g.nblk + GEMV_WARPS - 1) / GEMV_WARPS;
  g.S = (g.nblk + g.nslab - 1) / g.nslab;
  g.S_last = g.nblk - (g.nslab - 1) * g.S;
  g.R = g.nslab == 1 ? (GEMV_WARPS / g.nblk > 0 ? GEMV_WARPS / g.nblk : 1) : 1;
  const int dfull = type == T_Q6_K ? (2 * g.S + 15) / 16 * 16 : 0, dlast = type == T_Q6_K ? (2 * g.S_last + 15) / 16 * 16 : 0;
  g.d_off = g.S * g.ub;
  g.d_off_last = g.S_last * g.ub;
  g.RS = gemv_pad_row(g.S * g.ub + dfull);
  g.RS_last = gemv_pad_row(g.S_last * g.ub + dlast);
  g.stage_bytes = (uint32_t)(g.R * 16 * g.RS);
  g.stage_bytes_last = (uint32_t)(g.R * 16 * g.RS_last);
  g.tile_bytes = (uint32_t)(g.nslab - 1) * g.stage_bytes + g.stage_bytes_last;
  return g;
}

// Image row of logical row r. Gate and up projections share one image: every 16-row group holds
// eight gate rows followed by the same eight up rows (half = 0 gate, 1 up); half < 0: plain.
__host__ __device__ __forceinline__ int64_t gemv_image_row(int64_t r, int half) {
  return half < 0 ? r : ((r >> 3) << 4) + (r & 7) + 8 * half;
}

// Scatters contiguous units [rows][nblk][ub] (and, for Q6_K, their fp16 scales [rows][nblk]) into
// the stage images. The image must have been zeroed (padding, rows beyond the matrix).
__global__ void stage_image_kernel(const uint8_t* __restrict__ units, const uint16_t* __restrict__ dsrc, int64_t rows, GemvGeom g,
                                   int half, uint8_t* __restrict__ img) {
  const int cpu = g.ub / 16;
  const int64_t total = rows * g.nblk * cpu;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t u = i / cpu;
    const int c = (int)(i - u * cpu);
    const int64_t r = u / g.nblk;
    const int b = (int)(u - r * g.nblk);
    const int64_t dr = gemv_image_row(r, half);
    const int64_t tile = dr / (16 * g.R);
    const int rr = (int)(dr - tile * 16 * g.R);
    const int slab = b / g.S, bb = b - slab * g.S;
    const bool last = slab == g.nslab - 1;
    uint8_t* dst = img + (size_t)tile * g.tile_bytes + (size_t)slab * g.stage_bytes + (size_t)rr * (last ? g.RS_last : g.RS) +
                   (size_t)bb * g.ub + (size_t)c * 16;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(units + (size_t)u * g.ub + (size_t)c * 16);
  }
  if (dsrc) {
    const int64_t nd = rows * g.nblk;
    for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < nd; u += stride) {
      const int64_t r = u / g.nblk;
      const int b = (int)(u - r * g.nblk);
      const int64_t dr = gemv_image_row(r, half);
      const int64_t tile = dr / (16 * g.R);
      const int rr = (int)(dr - tile * 16 * g.R);
      const int slab = b / g.S, bb = b - slab * g.S;
      const bool last = slab == g.nslab - 1;
      uint8_t* dst = img + (size_t)tile * g.tile_bytes + (size_t)slab * g.stage_bytes + (size_t)rr * (last ? g.RS_last : g.RS) +
                     (size_t)(last ? g.d_off_last : g.d_off) + (size_t)bb * 2;
      *reinterpret_cast<uint16_t*>(dst) = dsrc[u];
    }
  }
}

struct GemvSeg {
  const uint8_t* img;  // stage images, [tiles][tile_bytes]
  int type;
  int rows;            // image rows that hold data (SWIGLU: 2 x the projection's rows)
  int tiles;
  int RS, RS_last, d_off, d_off_last;
  uint32_t stage_bytes, stage_bytes_last, tile_bytes;
};

struct GemvParams {
  GemvSeg seg[3];
  int nseg;
  int K;                // input dimension, a multiple of 256
  int nblk, nslab, S, S_last, R;  // GemvGeom of K
  uint32_t slot_bytes;  // ring slot = the largest stage of the launch
  int early_stages;     // stages requested before the kernel holds its input vector (the rest of the ring right after)
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
  uint2* amax_peer[8];  // tensor parallel: where each rank receives this rank's argmax partials as packets
                        // {value, index | (exchange number & 0x7fff) << 17}, [batch][gridDim.x] each; nullptr: not sent
  unsigned amax_epoch_k; // number of that exchange within the step (added to *epoch_base)
  // repetition penalty on the logits (reference apply_repetition_penalty, api.cpp:86-97): a row is penalised once per
  // occurrence of its vocabulary index in the window of generated ids, l -> l / penalty when positive, l * penalty
  // otherwise; pen_counts [batch][pen_stride] holds the occurrence counts (index = global vocabulary index)
  const uint8_t* pen_counts;
  int pen_stride;
  const float* pen_value;
  const float* resid;   // RESID: y = resid + W x (nullptr: y itself)
  int ntiles;           // over all segments
  int* error_flag;      // set when a bounded wait gives up
  unsigned long long* trace;  // optional step-trace record, eight slots: 0 entry, 1-3 dependency wait over, 4 input vector held,
                              // 5 prologue done, 6 first tile computed, 7 end
  // ---- tensor-parallel exchange without a collective call (one-shot all-reduce over peer memory) ----
  // Every exchanged value travels as an 8-byte packet {value, exchange number}: one aligned 64-bit
  // store, so the number can never be seen without its value, and no flag word, ticket or
  // system-wide fence is needed.
  // Producer side (EPI_PEER): each partial output row is stored as a packet into this rank's slot of
  // the exchange buffer of every rank (peer_y[r]: [batch][y_stride] packets in rank r's memory).
  // Consumer side (x_parts != nullptr): the input vector is x + the tp slots of the local exchange
  // buffer, summed in rank order; each thread polls (bounded) the packets it needs until they carry
  // this exchange's number. The first CTA stores the sum to x_out.
  int tp, tp_rank;
  uint2* peer_y[GEMV_MAX_TP];
  const unsigned* epoch_base;   // device scalar: exchanges completed before this step
  unsigned epoch_k;             // 1 + index of this launch's exchange within the step
  const uint2* x_parts;         // [tp][parts_stride] local exchange slots (packets) to add to x
  size_t parts_stride;          // packets between the slots of consecutive ranks
  float* x_out;                 // [batch][x_stride] where CTA 0 stores the summed input
  int poll_limit;               // probes of a packet before the consumer gives up (0: the default, about a second)
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

// Balanced base-256 digits (every digit a signed byte in [-128, 127]) come from plain byte
// extraction after a bias: v + 0x80...80 has bytes digit + 128, and xor 0x80 turns them into the
// signed digits.

// Quantises the eight elements v[] this lane holds of 256-element block b, whose largest
// magnitude over the warp is amax, and writes the block's digit planes, digit sums and scale.
template <int P>
__device__ __forceinline__ void act_quantize_block(const ActImage& a, int b, int lane, const float (&v)[8], float amax) {
  uint8_t* planes = const_cast<uint8_t*>(a.planes);
  float* sx = const_cast<float*>(a.sx);
  uint8_t* xs32d = const_cast<uint8_t*>(a.xs32d);
  uint8_t* xs16d = const_cast<uint8_t*>(a.xs16d);
  // largest magnitude P balanced digits can hold: 127 * (256^P - 1) / 255
  constexpr int QMAX = P == 3 ? 8355711 : (P == 2 ? 32639 : 127);
  constexpr int BIAS = P == 3 ? 0x808080 : (P == 2 ? 0x8080 : 0x80);
  const int e0 = b * 256 + lane * 8;
  const float scale = amax * (1.0f / (float)QMAX);
  const float inv = amax > 0.f ? __fdividef((float)QMAX, amax) : 0.f;  // any consistent inverse works: q is clamped to +-QMAX
  int s8 = 0;
  uint32_t u[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int q = __float2int_rn(v[i] * inv);
    q = max(-QMAX, min(QMAX, q));
    s8 += q;
    u[i] = (uint32_t)(q + BIAS);
  }
#pragma unroll
  for (int p = 0; p < P; ++p) {
    const uint32_t sel = (uint32_t)p | ((uint32_t)(4 + p) << 4);  // byte p of the first word, byte p of the second
    const uint32_t w0 = __byte_perm(__byte_perm(u[0], u[1], sel), __byte_perm(u[2], u[3], sel), 0x5410) ^ 0x80808080u;
    const uint32_t w1 = __byte_perm(__byte_perm(u[4], u[5], sel), __byte_perm(u[6], u[7], sel), 0x5410) ^ 0x80808080u;
    *reinterpret_cast<uint2*>(planes + (size_t)p * a.plane_stride + e0) = make_uint2(w0, w1);
  }
  const int s16 = s8 + __shfl_xor_sync(0xffffffffu, s8, 1);
  const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 2);
  if ((lane & 1) == 0) {
    const uint32_t dg = ((uint32_t)s16 + 0x80808080u) ^ 0x80808080u;
#pragma unroll
    for (int i = 0; i < 4; ++i) xs16d[i * a.n16 + b * 16 + (lane >> 1)] = (uint8_t)(dg >> (8 * i));
  }
  if ((lane & 3) == 0) {
    const uint32_t dg = ((uint32_t)s32 + 0x80808080u) ^ 0x80808080u;
#pragma unroll
    for (int i = 0; i < 4; ++i) xs32d[i * a.n32 + b * 8 + (lane >> 2)] = (uint8_t)(dg >> (8 * i));
  }
  if (lane == 0) sx[b] = scale;
}

// Prologue run by the 16 consumer warps: optional RMSNorm (reference utils.cpp:648-673: mean of
// squares, f = 1/sqrtf(mean + eps), out = x*f*w) then quantisation into the image above. Each
// warp owns the 256-element blocks warp, warp+16, .... The norm weights do not
// depend on the previous kernel: they are requested first, and only then (before_x) does the
// kernel wait for the grid it depends on, so their trip to HBM overlaps that wait.
// XFN(e, v) loads elements e .. e+7 of the input vector; AFTERX(ss) is called by every thread
// right after its part of the vector has been requested and summed.
__device__ __forceinline__ void pdl_wait();
__device__ __forceinline__ uint32_t smem_u32(const void* p);

template <int P>
__device__ __forceinline__ void act_scale_block(float (&v)[8], const float* __restrict__ norm_w, const float4 (&nw)[2], float f,
                                                float& amax) {
  if (norm_w) {
    const float w[8] = {nw[0].x, nw[0].y, nw[0].z, nw[0].w, nw[1].x, nw[1].y, nw[1].z, nw[1].w};
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = v[i] * f * w[i];
  }
  amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
}

template <int P, typename XFN, typename BEFOREX, typename AFTERX>
__device__ void act_build(uint8_t* smem, XFN xfn, const float* __restrict__ norm_w, float eps, int K, float* red /* 18 floats */,
                          BEFOREX before_x, AFTERX after_x) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nblk = K / 256;
  // This code runs once per launch, from a cold instruction cache, so it is kept small. The warp's
  // first three blocks stay in registers between the two passes; further blocks (rows longer than
  // 12288) are read again.
  float xv[8];
  float4 wv[2];
  wv[0] = wv[1] = make_float4(1.f, 1.f, 1.f, 1.f);
  if (warp < nblk && norm_w) {
    wv[0] = __ldg(reinterpret_cast<const float4*>(norm_w + warp * 256 + lane * 8));
    wv[1] = __ldg(reinterpret_cast<const float4*>(norm_w + warp * 256 + lane * 8 + 4));
  }
  before_x();  // the activation vector (and the buffers this kernel writes) belong to the previous kernel until here
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) xv[i] = 0.f;
  if (warp < nblk) {
    xfn(warp * 256 + lane * 8, xv);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(xv[i], xv[i], ss);
  }
  // the warp's second and third block (rows of up to 12288 elements) are requested now as well and kept
  float x1[8], x2[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) x1[i] = x2[i] = 0.f;
  if (warp + GEMV_WARPS < nblk) xfn((warp + GEMV_WARPS) * 256 + lane * 8, x1);
  if (warp + 2 * GEMV_WARPS < nblk) xfn((warp + 2 * GEMV_WARPS) * 256 + lane * 8, x2);
#pragma unroll
  for (int i = 0; i < 8; ++i) ss = fmaf(x2[i], x2[i], fmaf(x1[i], x1[i], ss));
#pragma unroll 1
  for (int b = warp + 3 * GEMV_WARPS; b < nblk; b += GEMV_WARPS) {
    float t[8];
    xfn(b * 256 + lane * 8, t);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(t[i], t[i], ss);
  }
  after_x(ss);  // runs once the loads above have returned (it is handed a value computed from them)
  float f = 1.0f;
  if (norm_w) {
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    consumer_sync();
    // fixed-order pairwise sum of the 16 warp partials (the reference accumulates in double; the
    // difference is below 1e-7 relative and FP64 is slow on this part)
    float r[GEMV_WARPS];
#pragma unroll
    for (int w = 0; w < GEMV_WARPS; ++w) r[w] = red[w];
#pragma unroll
    for (int n = GEMV_WARPS / 2; n > 0; n >>= 1)
#pragma unroll
      for (int w = 0; w < n; ++w) r[w] = r[2 * w] + r[2 * w + 1];
    f = rsqrtf(r[0] * (1.0f / (float)K) + eps);  // 2 ulp; the exact form costs a few hundred cycles of dependent latency here
  }
  const ActImage a = act_carve(smem, K, P);
  {
    float amax;
    act_scale_block<P>(xv, norm_w, wv, f, amax);
    if (warp < nblk) act_quantize_block<P>(a, warp, lane, xv, warp_max(amax));
  }
  // rows longer than 4096: the remaining blocks two at a time, so that their shuffle chains overlap
#pragma unroll 1
  for (int b = warp + GEMV_WARPS; b < nblk; b += 2 * GEMV_WARPS) {
    const int b2 = b + GEMV_WARPS;
    const bool two = b2 < nblk;
    float4 w1[2], w2[2];
    w1[0] = w1[1] = w2[0] = w2[1] = make_float4(1.f, 1.f, 1.f, 1.f);
    if (b != warp + GEMV_WARPS) {  // beyond the blocks kept in registers: read again
      xfn(b * 256 + lane * 8, x1);
      if (two) xfn(b2 * 256 + lane * 8, x2);
    }
    if (norm_w) {
      w1[0] = __ldg(reinterpret_cast<const float4*>(norm_w + b * 256 + lane * 8));
      w1[1] = __ldg(reinterpret_cast<const float4*>(norm_w + b * 256 + lane * 8 + 4));
      if (two) {
        w2[0] = __ldg(reinterpret_cast<const float4*>(norm_w + b2 * 256 + lane * 8));
        w2[1] = __ldg(reinterpret_cast<const float4*>(norm_w + b2 * 256 + lane * 8 + 4));
      }
    }
    float a1, a2 = 0.f;
    act_scale_block<P>(x1, norm_w, w1, f, a1);
    if (two) act_scale_block<P>(x2, norm_w, w2, f, a2);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      a1 = fmaxf(a1, __shfl_xor_sync(0xffffffffu, a1, o));
      a2 = fmaxf(a2, __shfl_xor_sync(0xffffffffu, a2, o));
    }
    act_quantize_block<P>(a, b, lane, x1, a1);
    if (two) act_quantize_block<P>(a, b2, lane, x2, a2);
  }
  consumer_sync();
}

// Op-level probe of the decode prologue: one CTA of 16 warps runs act_build (RMSNorm when norm_w is
// given, then the digit-plane quantisation) exactly as the matvec kernel does and writes the vector the
// matvec will see, x_hat[e] = sx[block] * sum_p digit_p[e] * 256^p, so that a test can compare the
// normalisation (and the 24-bit quantisation) with the reference's rmsnorm_vector_cpu.
__global__ void __launch_bounds__(GEMV_CONSUMER_THREADS, 1) act_probe_kernel(const float* __restrict__ x, const float* __restrict__ norm_w, float eps,
                                                                             int K, float* __restrict__ out) {
  extern __shared__ __align__(128) uint8_t smem_probe[];
  __shared__ float red[GEMV_WARPS + 2];
  auto xfn = [&](int e, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(x + e), b = *reinterpret_cast<const float4*>(x + e + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  };
  act_build<3>(smem_probe, xfn, norm_w, eps, K, red, [] {}, [](float) {});
  const ActImage a = act_carve(smem_probe, K, 3);
  for (int e = threadIdx.x; e < K; e += blockDim.x) {
    int v = 0;
#pragma unroll
    for (int p = 2; p >= 0; --p) v = v * 256 + (int)(int8_t)a.planes[(size_t)p * a.plane_stride + e];
    out[e] = a.sx[e >> 8] * (float)v;
  }
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

// ---- per-format work on one 256-element block of a staged 16-row group ----------------------
// Lane (g = lane >> 2, t = lane & 3) feeds rows g and g + 8 of the group and the k-slice
// 8t .. 8t+7 of every 32 elements, and supplies column g of the B operand. Column layout:
//   Q4_K / Q8_0: digit plane p sits in column 2p, so lane t receives plane t in c[0] (row g) and
//                c[2] (row g + 8); odd columns are zero and c[1], c[3] are ignored;
//   Q6_K:        a group of 32 elements holds two 16-element sub-blocks; column 2p + s carries
//                plane p restricted to sub-block s (zero elsewhere), so lane t receives
//                (plane t, sub-block 0) in c[0] / c[2] and (plane t, sub-block 1) in c[1] / c[3].
struct LaneCtx {
  int g, t;
  float wt;  // 256^t when t < P, else 0: weight of the digit plane this lane receives
  float wd;  // 256^t: weight of digit t of the activation sums in the minimum / offset terms
};

// The B operand of one 256-element block for this lane, plus the block's activation sums and scale.
struct BFrag {
  uint2 b[8];      // per 32 elements: the two words of column g
  uint32_t xw[4];  // digit t of the 32-element sums (2 words, Q4_K) or of the 16-element sums (4 words, Q6_K)
  float sx;
};

template <int P>
__device__ __forceinline__ void load_bfrag(int type, const ActImage& a, int blk, const LaneCtx& L, BFrag& f) {
  bool on;
  int plane;
  if (type == T_Q6_K) {
    on = L.g < 2 * P && (L.t >> 1) == (L.g & 1);
    plane = L.g >> 1;
  } else {
    on = !(L.g & 1) && (L.g >> 1) < P;
    plane = L.g >> 1;
  }
  const uint8_t* bp = a.planes + (size_t)(on ? plane : 0) * a.plane_stride + blk * 256 + 8 * L.t;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint2 v = *reinterpret_cast<const uint2*>(bp + 32 * j);
    f.b[j] = on ? v : make_uint2(0u, 0u);
  }
  if (type == T_Q6_K) {
    const uint4 v = *reinterpret_cast<const uint4*>(a.xs16d + (size_t)L.t * a.n16 + blk * 16);
    f.xw[0] = v.x; f.xw[1] = v.y; f.xw[2] = v.z; f.xw[3] = v.w;
  } else {
    const uint2 v = *reinterpret_cast<const uint2*>(a.xs32d + (size_t)L.t * a.n32 + blk * 8);
    f.xw[0] = v.x; f.xw[1] = v.y; f.xw[2] = 0u; f.xw[3] = 0u;
  }
  f.sx = a.sx[blk];
}

// pa / pb point at this block's unit in rows g / g + 8 of the stage.
__device__ __forceinline__ void compute_q4(const uint8_t* pa, const uint8_t* pb, const BFrag& f, const LaneCtx& L, float& acc0,
                                           float& acc1) {
  const uint4 h0 = *reinterpret_cast<const uint4*>(pa), h1 = *reinterpret_cast<const uint4*>(pb);
  // eight 6-bit scales and minima per row, four to a word (get_scale_min_k4 of the reference,
  // quantization.cpp:145-155, applied to four sub-blocks at once)
  const uint32_t scA0 = h0.y & 0x3F3F3F3Fu, mnA0 = h0.z & 0x3F3F3F3Fu;
  const uint32_t scB0 = (h0.w & 0x0F0F0F0Fu) | ((h0.y >> 2) & 0x30303030u);
  const uint32_t mnB0 = ((h0.w >> 4) & 0x0F0F0F0Fu) | ((h0.z >> 2) & 0x30303030u);
  const uint32_t scA1 = h1.y & 0x3F3F3F3Fu, mnA1 = h1.z & 0x3F3F3F3Fu;
  const uint32_t scB1 = (h1.w & 0x0F0F0F0Fu) | ((h1.y >> 2) & 0x30303030u);
  const uint32_t mnB1 = ((h1.w >> 4) & 0x0F0F0F0Fu) | ((h1.z >> 2) & 0x30303030u);
  int Jlo0 = 0, Jlo1 = 0, Jhi0 = 0, Jhi1 = 0;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint2 qa = *reinterpret_cast<const uint2*>(pa + 16 + 32 * c + 8 * L.t), qb = *reinterpret_cast<const uint2*>(pb + 16 + 32 * c + 8 * L.t);
    int cl[4], ch[4];
    imma_16x8x32<false>(cl, qa.x & 0x0F0F0F0Fu, qb.x & 0x0F0F0F0Fu, qa.y & 0x0F0F0F0Fu, qb.y & 0x0F0F0F0Fu, f.b[2 * c].x, f.b[2 * c].y);
    imma_16x8x32<false>(ch, qa.x & 0xF0F0F0F0u, qb.x & 0xF0F0F0F0u, qa.y & 0xF0F0F0F0u, qb.y & 0xF0F0F0F0u, f.b[2 * c + 1].x,
                        f.b[2 * c + 1].y);  // 16 x the high nibbles
    const uint32_t s0 = c < 2 ? scA0 : scB0, s1 = c < 2 ? scA1 : scB1;
    Jlo0 += byte_u(s0, (2 * c) & 3) * cl[0];
    Jlo1 += byte_u(s1, (2 * c) & 3) * cl[2];
    Jhi0 += byte_u(s0, (2 * c + 1) & 3) * ch[0];
    Jhi1 += byte_u(s1, (2 * c + 1) & 3) * ch[2];
  }
  const float f0 = fmaf((float)Jhi0, 0.0625f, (float)Jlo0), f1 = fmaf((float)Jhi1, 0.0625f, (float)Jlo1);
  // minimum term: sum_sub m_sub * X_sub, digit t of X handled by lane t
  const int M0 = dp4a_us(mnB0, f.xw[1], dp4a_us(mnA0, f.xw[0], 0));
  const int M1 = dp4a_us(mnB1, f.xw[1], dp4a_us(mnA1, f.xw[0], 0));
  const float2 dm0 = __half22float2(*reinterpret_cast<const __half2*>(&h0.x));
  const float2 dm1 = __half22float2(*reinterpret_cast<const __half2*>(&h1.x));
  acc0 = fmaf(f.sx, dm0.x * (L.wt * f0) - dm0.y * (L.wd * (float)M0), acc0);
  acc1 = fmaf(f.sx, dm1.x * (L.wt * f1) - dm1.y * (L.wd * (float)M1), acc1);
}

__device__ __forceinline__ void compute_q6(const uint8_t* pa, const uint8_t* pb, float d0, float d1, const BFrag& f, const LaneCtx& L,
                                           float& acc0, float& acc1) {
  const uint4 sc0 = *reinterpret_cast<const uint4*>(pa + 192), sc1 = *reinterpret_cast<const uint4*>(pb + 192);
  const uint32_t sw0[4] = {sc0.x, sc0.y, sc0.z, sc0.w}, sw1[4] = {sc1.x, sc1.y, sc1.z, sc1.w};
  int J0 = 0, J1 = 0;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint2 ha = *reinterpret_cast<const uint2*>(pa + 128 + 32 * h + 8 * L.t), hb = *reinterpret_cast<const uint2*>(pb + 128 + 32 * h + 8 * L.t);
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const uint2 la = *reinterpret_cast<const uint2*>(pa + 64 * h + 32 * q + 8 * L.t), lb = *reinterpret_cast<const uint2*>(pb + 64 * h + 32 * q + 8 * L.t);
#pragma unroll
      for (int hi = 0; hi < 2; ++hi) {
        const int g4 = q + 2 * hi;  // 32-element group within the 128-element half (reference quantization.cpp:223-266)
        auto six = [&](uint32_t lw, uint32_t hw) -> uint32_t {
          const uint32_t nib = hi ? ((lw >> 4) & 0x0F0F0F0Fu) : (lw & 0x0F0F0F0Fu);
          const uint32_t top = g4 == 0 ? (hw << 4) : g4 == 1 ? (hw << 2) : g4 == 2 ? hw : (hw >> 2);
          return nib | (top & 0x30303030u);
        };
        int c[4];
        imma_16x8x32<false>(c, six(la.x, ha.x), six(lb.x, hb.x), six(la.y, ha.y), six(lb.y, hb.y), f.b[4 * h + g4].x, f.b[4 * h + g4].y);
        // sub-block 8h + 2*g4 + s: byte 2*(g4 & 1) + s of scale word 2h + g4/2
        const uint32_t w0 = sw0[2 * h + hi], w1 = sw1[2 * h + hi];
        J0 += byte_s(w0, 2 * q) * c[0];
        J0 += byte_s(w0, 2 * q + 1) * c[1];
        J1 += byte_s(w1, 2 * q) * c[2];
        J1 += byte_s(w1, 2 * q + 1) * c[3];
      }
    }
  }
  // offset term: the stored quants are q + 32, so subtract 32 * sum_sub sc_sub * X_sub (digit t per lane)
  const int C0 = dp4a_ss(sc0.w, f.xw[3], dp4a_ss(sc0.z, f.xw[2], dp4a_ss(sc0.y, f.xw[1], dp4a_ss(sc0.x, f.xw[0], 0))));
  const int C1 = dp4a_ss(sc1.w, f.xw[3], dp4a_ss(sc1.z, f.xw[2], dp4a_ss(sc1.y, f.xw[1], dp4a_ss(sc1.x, f.xw[0], 0))));
  acc0 = fmaf(f.sx * d0, L.wt * (float)J0 - 32.f * (L.wd * (float)C0), acc0);
  acc1 = fmaf(f.sx * d1, L.wt * (float)J1 - 32.f * (L.wd * (float)C1), acc1);
}

__device__ __forceinline__ void compute_q8(const uint8_t* pa, const uint8_t* pb, const BFrag& f, const LaneCtx& L, float& acc0,
                                           float& acc1) {
  const uint4 da = *reinterpret_cast<const uint4*>(pa + 256), db = *reinterpret_cast<const uint4*>(pb + 256);
  const uint32_t dw0[4] = {da.x, da.y, da.z, da.w}, dw1[4] = {db.x, db.y, db.z, db.w};
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint2 qa = *reinterpret_cast<const uint2*>(pa + 32 * j + 8 * L.t), qb = *reinterpret_cast<const uint2*>(pb + 32 * j + 8 * L.t);
    int c[4];
    imma_16x8x32<true>(c, qa.x, qb.x, qa.y, qb.y, f.b[j].x, f.b[j].y);
    // the scale field of a Q8_0 block is used by magnitude (reference quantization.cpp:85-87)
    const float d0 = scale_field_to_float((uint16_t)((dw0[j >> 1] >> (16 * (j & 1))) & 0xFFFF));
    const float d1 = scale_field_to_float((uint16_t)((dw1[j >> 1] >> (16 * (j & 1))) & 0xFFFF));
    s0 = fmaf(d0, (float)c[0], s0);
    s1 = fmaf(d1, (float)c[2], s1);
  }
  acc0 = fmaf(f.sx * L.wt, s0, acc0);
  acc1 = fmaf(f.sx * L.wt, s1, acc1);
}

// Segment and tile-within-segment of a launch-wide tile index (segments are laid end to end).
__device__ __forceinline__ void gemv_locate(const GemvParams& p, int tile, int& seg, int& tl) {
  seg = 0;
  tl = tile;
  while (seg + 1 < p.nseg && tl >= p.seg[seg].tiles) { tl -= p.seg[seg].tiles; ++seg; }
}

// ---- the streaming pipeline ----------------------------------------------------------------
// Ring of nstages shared-memory slots. full_bar[s] completes when the bulk copy of the stage in
// slot s has landed (transaction bytes); empty_bar[s] completes when all 16 consumer warps have
// finished with it. The producer warp (one lane) walks the CTA's (tile, slab) sequence and
// refills a slot as soon as it is empty; the consumers never touch the copy engine.
struct GemvShared {
  unsigned long long full_bar[GEMV_MAX_STAGES];
  unsigned long long empty_bar[GEMV_MAX_STAGES];
  unsigned long long xready_bar;  // the consumers hold their part of the input vector (16 arrivals)
  float red[GEMV_WARPS + 2];
  float part[GEMV_NTB][GEMV_WARPS][16];
  float sv[GEMV_WARPS];
  int si[GEMV_WARPS];
  int abort_flag;
  int xfail;  // a poll of the tensor-parallel exchange gave up
};

__device__ __forceinline__ void pipe_init(GemvShared* sh, int nstages) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < nstages; ++s) {
      mbar_init(&sh->full_bar[s], 1);
      mbar_init(&sh->empty_bar[s], GEMV_WARPS);
    }
    mbar_init(&sh->xready_bar, GEMV_WARPS);
    sh->abort_flag = 0;
    sh->xfail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
}

__device__ __forceinline__ void pipe_fail(const GemvParams& prm, GemvShared* sh, int code = 1) {
  sh->abort_flag = 1;
  if (prm.error_flag) *reinterpret_cast<volatile int*>(prm.error_flag) = code;  // host-mapped word: a plain store
}

__device__ __forceinline__ bool pipe_aborted(GemvShared* sh) { return *(volatile int*)&sh->abort_flag != 0; }

// The producer: one lane requests every stage of this CTA's tiles, in the order the consumers use
// them (tiles cta, cta + ncta, ...; slabs in order), each with ONE bulk copy. Weights never depend
// on the previous kernel, so the first `early_stages` stages are requested at once; the rest waits
// until the consumers hold their input vector (behind a full ring of weight traffic on this SM
// those loads would wait for microseconds).
__device__ __forceinline__ void gemv_produce(const GemvParams& prm, GemvShared* sh, uint8_t* ring, int nstages, int cta, int ncta) {
  int slot = 0, fills = 0, n = 0;
#pragma unroll 1
  for (int tile = cta; tile < prm.ntiles; tile += ncta) {
    int s, tl;
    gemv_locate(prm, tile, s, tl);
    const GemvSeg& sg = prm.seg[s];
    const uint8_t* src = sg.img + (size_t)tl * sg.tile_bytes;
#pragma unroll 1
    for (int slab = 0; slab < prm.nslab; ++slab, ++n) {
      if (n == prm.early_stages && !mbar_wait(&sh->xready_bar, 0)) pipe_fail(prm, sh);
      if (fills > 0 && !mbar_wait(&sh->empty_bar[slot], (fills - 1) & 1)) pipe_fail(prm, sh);
      if (pipe_aborted(sh)) return;
      const uint32_t bytes = slab == prm.nslab - 1 ? sg.stage_bytes_last : sg.stage_bytes;
      mbar_expect_tx(&sh->full_bar[slot], bytes);
      bulk_g2s(ring + (size_t)slot * prm.slot_bytes, src + (size_t)slab * sg.stage_bytes, bytes, &sh->full_bar[slot]);
      if (++slot == nstages) { slot = 0; ++fills; }
    }
  }
}

// Finishes the rows of the n tiles parked in sh->part (tiles first_i .. first_i+n-1 of this CTA's
// sequence): every thread sums the partials of one row in warp order and applies the epilogue.
__device__ __forceinline__ void gemv_flush(const GemvParams& prm, GemvShared* sh, int first_i, int n, int bidx, int cta, int ncta,
                                        unsigned peer_tag, float& best_v, int& best_i) {
  consumer_sync();
  const int tid = threadIdx.x, lane = tid & 31;
  const int R = prm.R, S = prm.S;
  const int total = n * R * 16;
#pragma unroll 1
  for (int base = (tid & ~31); base < total; base += GEMV_WARPS * 32) {
    const int idx = base + lane;
    const bool in = idx < total;
    const int slot = in ? idx / (16 * R) : 0;
    const int rgi = in ? (idx >> 4) - slot * R : 0;
    const int r = idx & 15;
    float tot = 0.f;
    if (in) {
      const float* pp = &sh->part[slot][rgi * S][r];
#pragma unroll 4
      for (int s = 0; s < S; ++s) tot += pp[s * 16];
    }
    int seg, tl;
    gemv_locate(prm, cta + (first_i + slot) * ncta, seg, tl);
    const int irow = (tl * R + rgi) * 16 + r;  // image row within the segment
    const bool valid = in && irow < prm.seg[seg].rows;
    if (prm.epi == EPI_SWIGLU) {
      // reference model.cpp:734-735 with silu_cpu (utils.cpp:700-707): (g * 1/(1+exp(-g))) * u
      const float u = __shfl_sync(0xffffffffu, tot, (lane & 23) + 8);
      if (valid && r < 8) {
        const float sig = 1.0f / (1.0f + expf(-tot));
        prm.y[(size_t)bidx * prm.y_stride + (irow >> 4) * 8 + r] = (tot * sig) * u;
      }
    } else {
      const float other = __shfl_xor_sync(0xffffffffu, tot, 1);
      if (valid) {
        const int row = irow;
        if (prm.epi == EPI_PEER) {
          const uint2 pkt = make_uint2(__float_as_uint(tot), peer_tag);
          for (int r = 0; r < prm.tp; ++r) prm.peer_y[r][(size_t)bidx * prm.y_stride + row] = pkt;
        } else if (prm.epi == EPI_RESID) {
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
          const int grow = row + prm.amax_row_offset;
          if (prm.pen_counts) {
            const int times = prm.pen_counts[(size_t)bidx * prm.pen_stride + grow];
            if (times) {
              const float pen = *prm.pen_value;
#pragma unroll 1
              for (int k = 0; k < times; ++k) tot = tot > 0.0f ? __fdiv_rn(tot, pen) : __fmul_rn(tot, pen);
            }
          }
          prm.y[(size_t)bidx * prm.y_stride + row] = tot;
          if (tot > best_v || (tot == best_v && grow < best_i)) { best_v = tot; best_i = grow; }
        }
      }
    }
  }
  consumer_sync();
}

// State of a consumer warp while it walks the CTA's tiles.
struct ConsumerCtx {
  GemvShared* sh;
  uint8_t* ring;
  int nstages;
  int slot, use;   // ring slot of the next stage and how often the ring has wrapped
  int tile, i;     // launch-wide tile index and its number in this CTA's sequence
  int cta, ncta, bidx;
  int rg, bi;      // this warp's row group and block within a stage
  bool rg_ok, breg;
  int cur_type;    // block type the register-held B fragments were built for
  unsigned peer_tag;  // exchange number carried by the packets of an EPI_PEER launch
  float best_v;
  int best_i;
};

// Tiles [.., seg_end) of one segment (all of block type TYPE), one (row group, block) task per
// warp per stage; partial row sums are parked per tile and finished GEMV_NTB tiles at a time.
template <int P, int TYPE>
__device__ __forceinline__ void gemv_tiles(const GemvParams& prm, const GemvSeg& sg, int seg_end, ConsumerCtx& c, const ActImage& a,
                                           const LaneCtx& L, BFrag& bf) {
  GemvShared* sh = c.sh;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int ub = TYPE == T_Q4_K ? 144 : TYPE == T_Q6_K ? 208 : 272;
  const int nslab = prm.nslab;
  // byte offset of this lane's first row (row g of the warp's row group) and block within a stage
  const uint32_t off_full = (uint32_t)(c.rg * 16 + L.g) * (uint32_t)sg.RS + (uint32_t)c.bi * ub;
  const uint32_t off_last = (uint32_t)(c.rg * 16 + L.g) * (uint32_t)sg.RS_last + (uint32_t)c.bi * ub;
#pragma unroll 1
  for (; c.tile < seg_end; c.tile += c.ncta, ++c.i) {
    float acc0 = 0.f, acc1 = 0.f;
#pragma unroll 1
    for (int slab = 0; slab < nslab; ++slab) {
      const bool last = slab == nslab - 1;
      const bool active = c.rg_ok && c.bi < (last ? prm.S_last : prm.S);
      // the activation digits are ready before the weights: fetch them ahead of the wait (with at
      // most 16 blocks per row the warp meets the same block every time and keeps them)
      if (active && (!c.breg || c.cur_type != TYPE)) {
        load_bfrag<P>(TYPE, a, slab * prm.S + c.bi, L, bf);
        c.cur_type = TYPE;
      }
      if (!pipe_aborted(sh) && !mbar_wait(&sh->full_bar[c.slot], c.use & 1)) pipe_fail(prm, sh);
      if (active) {
        const int RSt = last ? sg.RS_last : sg.RS;
        const uint8_t* pa = c.ring + (size_t)c.slot * prm.slot_bytes + (last ? off_last : off_full);
        const uint8_t* pb = pa + 8 * RSt;
        if (TYPE == T_Q4_K) {
          compute_q4(pa, pb, bf, L, acc0, acc1);
        } else if (TYPE == T_Q6_K) {
          const uint8_t* ra = pa - c.bi * ub;
          const int dof = (last ? sg.d_off_last : sg.d_off) + 2 * c.bi;
          const float d0 = half_bits_to_float(*reinterpret_cast<const uint16_t*>(ra + dof));
          const float d1 = half_bits_to_float(*reinterpret_cast<const uint16_t*>(ra + 8 * RSt + dof));
          compute_q6(pa, pb, d0, d1, bf, L, acc0, acc1);
        } else {
          compute_q8(pa, pb, bf, L, acc0, acc1);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->empty_bar[c.slot]);  // this warp is done with the slot
      if (++c.slot == c.nstages) { c.slot = 0; ++c.use; }
    }
    // ---- tile finished: fold the four k-slices and park the partial sums ----
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
    const int pp = c.i % GEMV_NTB;
    if (c.i == 0 && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) trace_stamp(prm.trace, 6);
    if (L.t == 0) {
      sh->part[pp][warp][L.g] = acc0;
      sh->part[pp][warp][L.g + 8] = acc1;
    }
    // rows are finished when GEMV_NTB tiles are parked or after the CTA's last tile
    if (pp == GEMV_NTB - 1 || c.tile + c.ncta >= prm.ntiles) gemv_flush(prm, sh, c.i - pp, pp + 1, c.bidx, c.cta, c.ncta, c.peer_tag, c.best_v, c.best_i);
  }
}

// Per-CTA (value, first index) of the rows this CTA produced, from the per-thread running bests.
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
    if (prm.amax_peer[0]) {
      const unsigned tag = (*prm.epoch_base + prm.amax_epoch_k) & 0x7fffu;
      const uint2 pkt = make_uint2(__float_as_uint(bv), ((unsigned)bi & 0x1ffffu) | (tag << 17));
      for (int r = 0; r < prm.tp; ++r) prm.amax_peer[r][(size_t)bidx * ncta + cta] = pkt;
    }
  }
}

__host__ __device__ __forceinline__ size_t gemv_ring_offset(int K, int P) { return (act_smem_bytes(K, P) + 127) / 128 * 128; }

// Loads eight elements of the input vector. Under tensor parallelism it adds the ranks' partial
// sums, in rank order (so every rank computes the same bits): the eight packets of each rank are
// polled until all carry this exchange's number (written by other GPUs: read past L1), bounded; the
// first CTA stores the total.
struct XLoad {
  const float* x;
  const uint2* parts;  // nullptr: plain load
  size_t parts_stride;
  int nparts;
  unsigned tag;
  int limit;           // probes before giving up
  float* out;          // nullptr: do not store
  int* fail;           // set when a poll gives up
  __device__ __forceinline__ void operator()(int e, float (&v)[8]) const {
    const float4 a = *reinterpret_cast<const float4*>(x + e), b = *reinterpret_cast<const float4*>(x + e + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    if (parts) {
#pragma unroll 1
      for (int r = 0; r < nparts; ++r) {
        const uint2* src = parts + (size_t)r * parts_stride + e;
        uint4 p[4];
        int it = 0;
        while (true) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(p[i].x), "=r"(p[i].y), "=r"(p[i].z), "=r"(p[i].w) : "l"(src + 2 * i));
          const bool ok = p[0].y == tag && p[0].w == tag && p[1].y == tag && p[1].w == tag && p[2].y == tag && p[2].w == tag && p[3].y == tag &&
                          p[3].w == tag;
          if (ok) break;
          if (++it > limit) {  // bounded (about a second by default): report instead of hanging when a rank has gone away
            *reinterpret_cast<volatile int*>(fail) = 1;
            break;
          }
          if (it > 16) __nanosleep(32);
        }
        v[0] += __uint_as_float(p[0].x); v[1] += __uint_as_float(p[0].z); v[2] += __uint_as_float(p[1].x); v[3] += __uint_as_float(p[1].z);
        v[4] += __uint_as_float(p[2].x); v[5] += __uint_as_float(p[2].z); v[6] += __uint_as_float(p[3].x); v[7] += __uint_as_float(p[3].z);
      }
      if (out) {
        *reinterpret_cast<float4*>(out + e) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(out + e + 4) = make_float4(v[4], v[5], v[6], v[7]);
      }
    }
  }
};

// The 16 consumer warps: prologue, then the tiles segment by segment.
template <int P>
__device__ __forceinline__ void gemv_consume(const GemvParams& prm, GemvShared* sh, uint8_t* smem, uint8_t* ring, int nstages) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int cta = blockIdx.x, ncta = gridDim.x, bidx = blockIdx.y;
  unsigned long long* rec = (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) ? prm.trace : nullptr;
  XLoad xfn{prm.x + (size_t)bidx * prm.x_stride, prm.x_parts ? prm.x_parts + (size_t)bidx * prm.x_stride : nullptr,
            prm.parts_stride, prm.tp, prm.x_parts ? *prm.epoch_base + prm.epoch_k : 0u, prm.poll_limit > 0 ? prm.poll_limit : (1 << 22),
            (prm.x_out && cta == 0) ? prm.x_out + (size_t)bidx * prm.x_stride : nullptr, &sh->xfail};
  auto after_x = [&](float ss) {
    uint32_t z;
    asm volatile("and.b32 %0, %1, 0;" : "=r"(z) : "r"(__float_as_int(ss)));  // issue order: after the loads have returned
    if (lane == (int)z) {
      if (threadIdx.x == 0) trace_stamp(rec, 4);
      mbar_arrive(&sh->xready_bar);
    }
  };
  auto before_x = [&]() {
    pdl_wait();
    trace_stamp(rec, 1);
    trace_stamp(rec, 2);
    trace_stamp(rec, 3);
  };
  act_build<P>(smem, xfn, prm.norm_w, prm.eps, prm.K, sh->red, before_x, after_x);
  // act_build ended with a barrier: every poll is over. A poll that gave up is reported through the error word; the
  // weight pipeline itself is intact, so the launch runs to its end (on a meaningless input vector) and returns.
  if (prm.x_parts && threadIdx.x == 0 && *(volatile int*)&sh->xfail && prm.error_flag) *reinterpret_cast<volatile int*>(prm.error_flag) = 1;
  trace_stamp(rec, 5);
  const ActImage a = act_carve(smem, prm.K, P);

  LaneCtx L;
  L.g = lane >> 2;
  L.t = lane & 3;
  L.wd = __int_as_float((127 + 8 * L.t) << 23);  // 256^t
  L.wt = L.t < P ? L.wd : 0.f;
  ConsumerCtx c;
  c.sh = sh; c.ring = ring; c.nstages = nstages; c.slot = 0; c.use = 0;
  c.tile = cta; c.i = 0; c.cta = cta; c.ncta = ncta; c.bidx = bidx;
  c.rg = warp / prm.S; c.bi = warp - c.rg * prm.S;
  c.rg_ok = c.rg < prm.R;
  // rows of at most 16 blocks: one stage per tile, the warp meets the same block column every
  // time and its B fragments stay in registers until the block type changes
  c.breg = prm.nslab == 1;
  c.cur_type = -1;
  c.best_v = -INFINITY; c.best_i = 0x7fffffff;
  c.peer_tag = prm.epi == EPI_PEER ? *prm.epoch_base + prm.epoch_k : 0u;
  BFrag bf;
  int seg_end = 0;
#pragma unroll 1
  for (int s = 0; s < prm.nseg; ++s) {
    const GemvSeg& sg = prm.seg[s];
    seg_end += sg.tiles;
    if (c.tile >= seg_end) continue;
    if (sg.type == T_Q4_K) gemv_tiles<P, T_Q4_K>(prm, sg, seg_end, c, a, L, bf);
    else if (sg.type == T_Q6_K) gemv_tiles<P, T_Q6_K>(prm, sg, seg_end, c, a, L, bf);
    else gemv_tiles<P, T_Q8_0>(prm, sg, seg_end, c, a, L, bf);
  }
  if (prm.amax_val) gemv_store_argmax(prm, sh, c.best_v, c.best_i, bidx, cta, ncta);
}

// One launch = one fused matvec for blockIdx.y's activation vector; one persistent CTA per SM:
// 16 consumer warps and one producer warp. There is one instantiation per activation width only: a
// decode step alternates between this kernel and the attention kernel 160 times, and their code
// should stay in the instruction caches.
template <int P>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_kernel(const __grid_constant__ GemvParams prm, int nstages) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ GemvShared sh;
  uint8_t* ring = smem + gemv_ring_offset(prm.K, P);
  pipe_init(&sh, nstages);
  pdl_launch_dependents();
  if (threadIdx.x >= GEMV_CONSUMER_THREADS) {
    if (threadIdx.x == GEMV_CONSUMER_THREADS) gemv_produce(prm, &sh, ring, nstages, blockIdx.x, gridDim.x);
    return;
  }
  unsigned long long* rec = (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) ? prm.trace : nullptr;
  trace_stamp(rec, 0);
  gemv_consume<P>(prm, &sh, smem, ring, nstages);
  trace_stamp(rec, 7);
}

}  // namespace b200
