// Batched matmul on the 5th-generation tensor cores for batch >= 16 decode and prompt ingestion:
//   Y[t][row] = sum_k W[row][k] * X[t][k]        (W packed Q8_0 / Q4_K / Q6_K, X fp16, fp32 accumulate)
// Replaces matmul_*_f32_batch_cpu (reference utils.cpp:730-782, 890-1044) / smart_gemm_batch_cuda
// (model.cpp:2141-2249). "Swap-AB": the weight rows are the M side of the MMA (128 per CTA tile),
// the tokens the N side (32..512 per tile; above 256 a K step issues two 256-token MMA halves that
// share the dequantised weight stage, so the accumulator fills all 512 tensor-memory columns).
//
// A CTA (608 threads) owns one tile of 128 rows x NT tokens and walks K in steps of 64 elements.
// Five roles meet only on mbarriers; there is no block-wide barrier inside the K loop:
//   * a weight-producer warp brings the packed units of the tile's 128 rows, one 256-element block
//     per tensor copy (cp.async.bulk.tensor.4d over the stage images), into a ring of 1-4 stages;
//   * sixteen warps dequantise: a thread owns (row, 16-element quarter of the step), copies its
//     share of a landed block from the ring into registers (which frees the stage), converts it to
//     fp16 and stores it into one of 4 or 8 weight stages (128 rows x 128 bytes) in the K-major
//     128-byte-swizzle layout the MMA unit reads from shared memory;
//   * one lane of an activation-producer warp moves the matching slices of the fp16 activations
//     with TMA (cp.async.bulk.tensor.2d, same swizzle, tokens beyond T read as zero) into 2-4
//     activation stages as soon as the MMAs that read a stage have completed;
//   * one lane of the MMA warp issues four tcgen05.mma (M=128, N=NT, K=16, kind::f16) per step that
//     accumulate into a 128-lane x NT-column fp32 tile in tensor memory, and does nothing else:
//     a single thread's dependent instruction stream is slow (measured: with the activation loads,
//     stage arithmetic and descriptor construction in this thread it needed 1 100 cycles per step and
//     everyone else waited for it); tcgen05.commit tells the other roles when a stage may be reused;
//   * after the last step the sixteen warps read their TMEM lanes back (tcgen05.ld 32x32b:
//     thread = weight row, registers = tokens) and run the same epilogues as the matvec kernel
//     (store, residual add, RoPE scatter, SwiGLU).
// Every wait is bounded; on a give-up the kernel sets the error word, frees its tensor memory and returns.
//
// fp16 operands: dequantised weights are rounded to fp16 (relative 2^-11) and activations likewise,
// so results agree with the FP32 reference dot to about 1e-3 of the largest output, not to 1e-3 of
// each element; the parity tests state that tolerance.
#pragma once
#include <cuda.h>  // CUtensorMap (types only; the encoder is fetched through cudaGetDriverEntryPoint)

#include "gemv.cuh"

namespace b200 {

constexpr int TC_M = 128;        // weight rows per CTA tile (the MMA's M)
constexpr int TC_KC = 64;        // elements along K per shared-memory stage: one 128-byte swizzled row of fp16
constexpr int TC_WORKERS = 512;   // sixteen dequantising warps: thread = (weight row, 16-element quarter of the 64-element step)
constexpr int TC_THREADS = TC_WORKERS + 96;  // + the MMA warp, the weight-producer warp and the activation-producer warp
constexpr int TC_MAX_N = 512;     // tokens per CTA tile (all 512 TMEM columns); above 256 the tile is two MMA halves

struct TcParams {
  GemvSeg seg[3];
  int nseg;
  int K;
  int nblk, nslab, S, S_last, R;  // GemvGeom of K (where a unit sits inside the stage images)
  const __half* x16;              // [T][K] activations (already normalised when the layer asks for it)
  int T;                          // tokens
  int NT;                         // tokens per CTA tile: a multiple of 32, <= 512 (a multiple of 64 above 256)
  int tmem_cols;                  // power of two >= max(32, NT)
  int epi;                        // EPI_STORE / EPI_RESID / EPI_QKV_ROPE / EPI_SWIGLU
  float* y;                       // [T][y_stride]
  int y_stride;
  float* y2;                      // QKV: new K then V rows, [T][y2_stride]
  int y2_stride;
  const float* resid;             // RESID: y = resid + W x (nullptr: y itself)
  const float* rope;
  const int* positions;           // [T]
  int head_dim, max_pos;
  int ntiles_m;                   // 128-row tiles over all segments
  int a_stages;                   // weight-tile stages: 4 or 8
  int b_stages;                   // activation stages (2 to 4)
  int w_stages, w_stage_bytes;    // packed-weight ring: stages of 128 rows x unit bytes
  int w_rowcopy;                  // 1: the producer copies row by row (geometries a tensor map cannot describe)
  int ksplit, kblocks;            // split-K: CTA z takes 256-element blocks [z*kblocks, (z+1)*kblocks) and stores to y + z*T*y_stride (EPI_STORE only)
  int* error_flag;
};

// ---- tcgen05 / TMEM primitives (inline PTX) ---------------------------------------------------
__device__ __forceinline__ void tc_alloc(uint32_t* smem_dst, int ncols) {  // one full warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, int ncols) {  // the same warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] (+)= A[smem] * B[smem]^T, M = 128, K = 16 fp16 per instruction
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// arrives on the mbarrier once every MMA issued so far by this thread has completed
__device__ __forceinline__ void tc_commit(void* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// this warp's 32 TMEM lanes, 8 consecutive columns: thread = lane, registers = columns
__device__ __forceinline__ void tc_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile in the 128-byte-swizzle layout: rows of 128
// bytes, 8-row groups 1024 bytes apart, 16-byte chunk c of row r stored at chunk c ^ (r & 7).
// Fields: start address >> 4 [0,14), leading byte offset >> 4 [16,30) (1: unused with this
// swizzle), stride byte offset >> 4 [32,46) (1024 >> 4), descriptor version 1 [46,48), layout
// type 2 = SWIZZLE_128B [61,64). A step of 16 elements along K advances the start by 32 bytes.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_addr) {
  const uint32_t lo = ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16);
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return ((uint64_t)hi << 32) | lo;
}
// Instruction descriptor, kind::f16: D = F32 [4,6) = 1, A and B = F16 (0) and K-major (0),
// N >> 3 at [17,23), M >> 4 at [24,29).
__host__ __device__ __forceinline__ uint32_t tc_idesc(int n) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TC_M >> 4) << 24); }

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// 16-byte chunk c (0..7) of row r in a swizzled tile
__device__ __forceinline__ uint32_t tc_swz(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

// Where a thread finds one unit (image row, block) in the packed-weight ring, and the block's
// Q6_K scale: the batched kernel reads the same stage images the matvec kernel streams (GemvGeom).
struct TcUnit {
  const uint8_t* unit;
  const uint8_t* d;  // Q6_K: this block's fp16 d
};

// The packed bytes of one 256-element block that one thread needs for the block's four K steps,
// fetched one block ahead of their use so that the loads overlap the previous block's work. A
// thread owns (row, half, sub): elements [64*kc + 32*half + 16*sub, +16) of every step kc.
//   Q4_K: r[0] = d, dmin, 12 scale bytes; r[1 + kc] = its 16 nibble bytes of step kc
//   Q6_K: r[hh] = its 16 ql bytes, r[2 + hh] = its 16 qh bytes of 128-element half hh; r[4] = scales; r[5].x = d
//   Q8_0: r[kc] = its 16 quants of step kc; r[4] = the eight fp16 d
struct TcRaw {
  uint4 r[6];
};

__device__ __forceinline__ void tc_fetch(int type, const TcUnit& u, int half, int sub, TcRaw& t) {
  if (type == T_Q4_K) {
    t.r[0] = *reinterpret_cast<const uint4*>(u.unit);
#pragma unroll
    for (int kc = 0; kc < 4; ++kc) t.r[1 + kc] = *reinterpret_cast<const uint4*>(u.unit + 16 + 32 * kc + 16 * sub);
  } else if (type == T_Q6_K) {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      t.r[hh] = *reinterpret_cast<const uint4*>(u.unit + 64 * hh + 32 * half + 16 * sub);
      t.r[2 + hh] = *reinterpret_cast<const uint4*>(u.unit + 128 + 32 * hh + 16 * sub);
    }
    t.r[4] = *reinterpret_cast<const uint4*>(u.unit + 192);
    t.r[5].x = *reinterpret_cast<const uint16_t*>(u.d);
  } else {
#pragma unroll
    for (int kc = 0; kc < 4; ++kc) t.r[kc] = *reinterpret_cast<const uint4*>(u.unit + 32 * (2 * kc + half) + 16 * sub);
    t.r[4] = *reinterpret_cast<const uint4*>(u.unit + 256);
  }
}

__device__ __forceinline__ uint32_t u4_word(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// Byte k of `v` (0..255) as a float, without an integer-to-float conversion: 0x4B0000bb is
// 8388608 + bb, and subtracting 8388608 (+ the format's own offset) is exact.
__device__ __forceinline__ float byte_to_float(uint32_t v, int k, float bias) {
  return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7440 | k)) - bias;
}

// Byte k of `v` (its top two bits clear, bit 7 pre-set by the caller: v = q | 0x80 per byte) as the
// float 1 + q / 128: the byte lands in mantissa bits 16..22 under the exponent of 1.0 (its bit 7 is
// the exponent's lowest bit). One PRMT, and the affine map back to q folds into the FMA that applies
// the scale: scale * (q - off) = (128 scale) * X - (128 + off) * scale, X = 1 + q/128.
__device__ __forceinline__ float byte_to_unit_float(uint32_t v, int k) {
  return __uint_as_float(__byte_perm(v, 0x3F000000u, 0x7044 | (k << 8)));
}

// Dequantises the thread's 16 elements of step kc (elements [64*kc + 32*half + 16*sub, +16) of the
// block held in `t`) to fp16: two 16-byte chunks w[0..1] (eight halves each). kc is a compile-time
// constant at every call site (the K steps of a block are unrolled). Each weight is computed in
// FP32 as the reference does and rounded to fp16 once (scaling in fp16 pairs was measured to triple
// the error of the products: the sub-block scale's rounding is shared by 16 or 32 weights and does
// not average out). Formulas: reference dequantize_q4_k_m / dequantize_q6_k /
// dequantize_q8_0_block (quantization.cpp:171-266, 1047-1052); the matmul contract is a tolerance.
__device__ __forceinline__ void tc_dequant16(int type, const TcRaw& t, int kc, int half, int sub, uint4 (&w)[2]) {
  float v[16];
  if (type == T_Q4_K) {
    const uint4 h = t.r[0];
    const float2 dm = __half22float2(*reinterpret_cast<const __half2*>(&h.x));
    const int sb = 2 * kc + half;  // 32-element sub-block
    // get_scale_min_k4 (quantization.cpp:145-155) on the 12 scale bytes h.y h.z h.w
    auto q = [&](int i) -> int {
      const uint32_t wv = i < 4 ? h.y : (i < 8 ? h.z : h.w);
      return (int)((wv >> (8 * (i & 3))) & 0xFF);
    };
    int sc, mn;
    if (sb < 4) {
      sc = q(sb) & 63;
      mn = q(sb + 4) & 63;
    } else {
      sc = (q(sb + 4) & 0xF) | ((q(sb - 4) >> 6) << 4);
      mn = (q(sb + 4) >> 4) | ((q(sb) >> 6) << 4);
    }
    const float d1 = dm.x * (float)sc, m1 = dm.y * (float)mn;
    // d1 * q - m1 = D * X - (D + m1), D = 128 d1 (exact), X = 1 + q/128: the constant's rounding is 2^-24 of
    // 128 d1, far below the fp16 rounding of the result
    const float D = 128.0f * d1, C = -(D + m1);
    const int shift = half ? 4 : 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // word i: its bytes 4i .. 4i+3 -> elements 4i .. 4i+3
      const uint32_t word = ((u4_word(t.r[1 + kc], i) >> shift) & 0x0F0F0F0Fu) | 0x80808080u;
#pragma unroll
      for (int k = 0; k < 4; ++k) v[4 * i + k] = fmaf(D, byte_to_unit_float(word, k), C);
    }
  } else if (type == T_Q6_K) {
    const int hh = kc >> 1, j = 2 * (kc & 1) + half;  // 128-element half, which of q1..q4
    const float d = half_bits_to_float((uint16_t)t.r[5].x);
    // sub-block scale 8hh + 2j + sub (signed byte)
    const uint32_t sw = u4_word(t.r[4], 2 * hh + (j >> 1));
    const float sc = d * (float)(int)(int8_t)((sw >> (16 * (j & 1) + 8 * sub)) & 0xFF);
    const float S = 128.0f * sc, C = -160.0f * sc;  // sc * (q - 32) = S * X - (128 + 32) sc, X = 1 + q/128 (both products exact scalings of sc)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t lword = u4_word(t.r[hh], i), hword = u4_word(t.r[2 + hh], i);
      // low nibbles from ql (its high nibbles for q3 / q4), bits 4-5 from the qh pair of this quarter: one variable
      // shift brings that pair to bits 4-5, one bitwise select joins the two, one more clears bits 6-7 and sets bit 7
      const uint32_t lo = (kc & 1) ? (lword >> 4) : lword;
      const uint32_t hi = (kc & 1) ? (hword >> (2 * half)) : (hword << (4 - 2 * half));
      const uint32_t six = (((lo ^ hi) & 0x0F0F0F0Fu) ^ hi) & 0x3F3F3F3Fu | 0x80808080u;
#pragma unroll
      for (int k = 0; k < 4; ++k) v[4 * i + k] = fmaf(S, byte_to_unit_float(six, k), C);  // sc * (q - 32)
    }
  } else {  // Q8_0 unit: 8 x 32 quants, then 8 fp16 d
    const int b32 = 2 * kc + half;
    const uint32_t dwv = u4_word(t.r[4], b32 >> 1);
    const float d = scale_field_to_float((uint16_t)((dwv >> (16 * (b32 & 1))) & 0xFFFF));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t word = u4_word(t.r[kc], i) ^ 0x80808080u;  // int8 + 128 as an unsigned byte
#pragma unroll
      for (int k = 0; k < 4; ++k) v[4 * i + k] = d * byte_to_float(word, k, 8388736.0f);  // 8388608 + 128
    }
  }
  w[0] = make_uint4(pack_h2(v[0], v[1]), pack_h2(v[2], v[3]), pack_h2(v[4], v[5]), pack_h2(v[6], v[7]));
  w[1] = make_uint4(pack_h2(v[8], v[9]), pack_h2(v[10], v[11]), pack_h2(v[12], v[13]), pack_h2(v[14], v[15]));
}

constexpr int TC_B_STAGES = 4;  // at most: activation tiles in flight (TMA)
constexpr int TC_A_STAGES = 8;  // at most: weight-tile stages (four per 256-element block; one or two blocks deep)
constexpr int TC_W_STAGES = 4;  // at most: packed-weight stages in flight (TMA)
constexpr int TC_D_BYTES = 2 * TC_M * 32;  // Q6_K block scales of a tile's rows for the current and the next slab

// Tensor maps of one launch: the fp16 activations and, per segment, the packed units of its stage
// images seen as a 4-D array (bytes of a stage row / rows of an image tile / slabs / image tiles) -
// one map for the full slabs and one for the last slab of every tile, whose rows are shorter.
struct alignas(64) TcMaps {
  CUtensorMap act;
  CUtensorMap w[3][2];
};

struct TcShared {
  unsigned long long a_full[TC_A_STAGES];  // all dequantising warps have stored their part of the weight tile
  unsigned long long b_full[TC_B_STAGES];  // the activation tile has landed (TMA transaction bytes)
  unsigned long long mma_done[TC_A_STAGES];  // the MMAs that read weight stage i (and its activation stage) have completed
  unsigned long long done_bar;             // all MMAs of the tile have completed
  unsigned long long w_full[TC_W_STAGES];  // the packed units of a block (and, at a slab start, the Q6_K scales) have landed
  unsigned long long w_empty[TC_W_STAGES]; // all dequantising warps have copied their part of the stage into registers
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void tc_fail(const TcParams& p, TcShared* sh) {
  sh->abort_flag = 1;
  if (p.error_flag) *reinterpret_cast<volatile int*>(p.error_flag) = 1;
}
__device__ __forceinline__ void tc_wait(const TcParams& p, TcShared* sh, void* bar, uint32_t parity) {
  if (!*(volatile int*)&sh->abort_flag && !mbar_wait(bar, parity)) tc_fail(p, sh);
}

// 2-D tiled TMA load of one activation tile (64 elements along K x NT tokens, 128-byte swizzle)
__device__ __forceinline__ void tc_tma_load_2d(void* dst, const void* tmap, int c0, int c1, void* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
               "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
               : "memory");
}

// grid = (128-row tiles over all segments, token tiles of NT, K splits); 608 threads: warps 0-15
// dequantise the weight tile (thread = row x 16-element quarter), warp 16 issues the MMAs, warp 17
// moves the packed weights, warp 18 the activation tiles. Dynamic shared memory (1024-byte aligned):
// 4 or 8 weight stages of 16 KB, 2-4 activation stages of NT x 128 bytes, the packed-weight ring,
// the Q6_K scale buffers.
// nslab: slabs per stage-image tile; rows that are one slab long need one Q6_K scale buffer, not two
__host__ __device__ __forceinline__ size_t tc_smem_bytes(int NT, int a_stages, int b_stages, int w_stages, int w_stage_bytes, int nslab) {
  return 1024 + a_stages * (size_t)TC_M * 128 + b_stages * (size_t)NT * 128 + (size_t)w_stages * w_stage_bytes + (nslab == 1 ? TC_D_BYTES / 2 : TC_D_BYTES);
}
constexpr int TC_SMEM_MAX = 226 * 1024;  // dynamic part; the barriers live in static shared memory

// 4-D tiled TMA load of the packed units of 128 rows of one block (no swizzle: rows land back to back)
__device__ __forceinline__ void tc_tma_load_4d(void* dst, const void* tmap, int c0, int c1, int c2, int c3, void* bar) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_u32(dst)),
               "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const TcParams p, const __grid_constant__ TcMaps maps) {
  extern __shared__ uint8_t tc_smem_raw[];
  __shared__ TcShared sh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* const Abase = smem;                                 // [4][128 rows][128 B]
  uint8_t* const Bbase = smem + p.a_stages * TC_M * 128;      // [b_stages][NT rows][128 B]
  const uint32_t b_stage_bytes = (uint32_t)p.NT * 128;
  uint8_t* const Wbase = Bbase + (size_t)p.b_stages * b_stage_bytes;       // [w_stages][128 rows][unit bytes]
  uint8_t* const Dbase = Wbase + (size_t)p.w_stages * p.w_stage_bytes;     // [2][128 rows][32 B]
  // ---- which rows, which tokens, which part of K ----
  int seg = 0, mt = blockIdx.x;
  while (seg + 1 < p.nseg && mt >= (p.seg[seg].rows + TC_M - 1) / TC_M) { mt -= (p.seg[seg].rows + TC_M - 1) / TC_M; ++seg; }
  const GemvSeg& sg = p.seg[seg];
  const int row0 = mt * TC_M;             // first image row of the tile within the segment
  const int t0 = blockIdx.y * p.NT;       // first token of the tile
  const int blk0 = blockIdx.z * p.kblocks;
  const int nblocks = min(p.K / 256 - blk0, p.kblocks), nsteps = 4 * nblocks;
  if (tid == 0) {
    for (int i = 0; i < TC_A_STAGES; ++i) { mbar_init(&sh.a_full[i], TC_WORKERS / 32); mbar_init(&sh.mma_done[i], 1); }
    for (int i = 0; i < TC_B_STAGES; ++i) mbar_init(&sh.b_full[i], 1);
    for (int i = 0; i < TC_W_STAGES; ++i) { mbar_init(&sh.w_full[i], 1); mbar_init(&sh.w_empty[i], TC_WORKERS / 32); }
    mbar_init(&sh.done_bar, 1);
    sh.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tc_alloc(&sh.tmem_base, p.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = sh.tmem_base;

  if (warp == TC_WORKERS / 32) {
    // ---- MMA warp: one lane waits for a weight stage and an activation stage and issues the step's
    //      four MMAs. Its instruction stream is the kernel's critical path (one thread, every
    //      instruction waits for the one before), so it is kept to the bare minimum: running stage
    //      counters instead of divisions, descriptors advanced by constants, loads left to others ----
    if (lane == 0) {
      const int nhalf = p.NT > 256 ? 2 : 1, nmma = p.NT / nhalf;  // one MMA covers at most 256 tokens
      const uint32_t idesc = tc_idesc(nmma);
      const uint64_t b_half = (uint64_t)((nmma * 128) >> 4);  // descriptor units between the two token halves of an activation stage
      const int nb = p.b_stages, na = p.a_stages;
      const uint64_t adesc0 = tc_smem_desc(smem_u32(Abase)), bdesc0 = tc_smem_desc(smem_u32(Bbase));
      const uint64_t a_step = (uint64_t)((TC_M * 128) >> 4), b_step = (uint64_t)(b_stage_bytes >> 4);
      int sa = 0, sb = 0;
      uint32_t pa = 0, pb = 0;
      uint64_t adesc = adesc0, bdesc = bdesc0;
      bool ok = !*(volatile int*)&sh.abort_flag;
#pragma unroll 1
      for (int s = 0; s < nsteps && ok; ++s) {
        ok = mbar_wait(&sh.a_full[sa], pa) && mbar_wait(&sh.b_full[sb], pb);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {  // 16 elements along K = 32 bytes = 2 descriptor units
          tc_mma_f16(tmem_d, adesc + 2 * k4, bdesc + 2 * k4, idesc, (s | k4) ? 1u : 0u);
          if (nhalf == 2) tc_mma_f16(tmem_d + (uint32_t)nmma, adesc + 2 * k4, bdesc + b_half + 2 * k4, idesc, (s | k4) ? 1u : 0u);
        }
        tc_commit(&sh.mma_done[sa]);
        adesc += a_step; bdesc += b_step;
        if (++sa == na) { sa = 0; pa ^= 1u; adesc = adesc0; }
        if (++sb == nb) { sb = 0; pb ^= 1u; bdesc = bdesc0; }
      }
      if (!ok) tc_fail(p, &sh);
      tc_commit(&sh.done_bar);
    }
    __syncwarp();
  } else if (warp == TC_WORKERS / 32 + 2) {
    // ---- activation producer: tile of step s into stage s % nb as soon as the MMAs of step s - nb have read it ----
    if (lane == 0) {
      const int nb = p.b_stages, na = p.a_stages;
#pragma unroll 1
      for (int s = 0; s < nsteps; ++s) {
        if (s >= nb) tc_wait(p, &sh, &sh.mma_done[(s - nb) % na], (uint32_t)(((s - nb) / na) & 1));
        void* bar = &sh.b_full[s % nb];
        mbar_expect_tx(bar, b_stage_bytes);
        uint8_t* dst = Bbase + (size_t)(s % nb) * b_stage_bytes;
        tc_tma_load_2d(dst, &maps.act, (4 * blk0 + s) * TC_KC, t0, bar);
        if (p.NT > 256) tc_tma_load_2d(dst + (size_t)(p.NT / 2) * 128, &maps.act, (4 * blk0 + s) * TC_KC, t0 + p.NT / 2, bar);  // a box holds at most 256 rows
      }
    }
    __syncwarp();
  } else if (warp == TC_WORKERS / 32 + 1) {
    // ---- weight producer: one tensor copy per 256-element block brings the packed units of the
    //      tile's 128 rows into the ring (rows beyond the images read as zero); at the start of a
    //      slab the lanes also copy the rows' Q6_K block scales ----
    const int ub = gemv_unit_bytes(sg.type), tr = 16 * p.R, nw = p.w_stages;
    const bool q6 = sg.type == T_Q6_K;
#pragma unroll 1
    for (int blk = 0; blk < nblocks; ++blk) {
      const int gb = blk0 + blk, slab = gb / p.S, bb = gb - slab * p.S;
      const bool last = slab == p.nslab - 1;
      const int stage = blk % nw;
      void* bar = &sh.w_full[stage];
      if (blk >= nw && lane == 0) tc_wait(p, &sh, &sh.w_empty[stage], (uint32_t)((blk / nw - 1) & 1));
      __syncwarp();
      const bool with_d = q6 && (bb == 0 || blk == 0);
      const uint32_t dbytes = (uint32_t)((2 * (last ? p.S_last : p.S) + 15) / 16 * 16);
      if (lane == 0) {
        mbar_expect_tx(bar, (uint32_t)(TC_M * ub) + (with_d ? TC_M * dbytes : 0u));
        if (!p.w_rowcopy)
          tc_tma_load_4d(Wbase + (size_t)stage * p.w_stage_bytes, &maps.w[seg][last ? 1 : 0], bb * ub / 4, row0 % tr, last ? 0 : slab, row0 / tr, bar);
      }
      if (with_d || p.w_rowcopy) {
        for (int r = lane; r < TC_M; r += 32) {
          const int irow = min(row0 + r, sg.rows - 1);  // rows past the segment repeat the last one; their results are dropped
          const int tile = irow / tr, rr = irow - tile * tr;
          const uint8_t* rowp = sg.img + (size_t)tile * sg.tile_bytes + (size_t)slab * sg.stage_bytes + (size_t)rr * (last ? sg.RS_last : sg.RS);
          if (p.w_rowcopy) bulk_g2s(Wbase + (size_t)stage * p.w_stage_bytes + (size_t)r * ub, rowp + (size_t)bb * ub, (uint32_t)ub, bar);
          if (with_d) bulk_g2s(Dbase + (size_t)(slab & 1) * (TC_M * 32) + (size_t)r * 32, rowp + (last ? sg.d_off_last : sg.d_off), dbytes, bar);
        }
      }
    }
    __syncwarp();
  } else {
    // ---- dequantising warps: thread = (weight row, 16-element quarter of the step) ----
    const int my_row = tid & (TC_M - 1), my_half = (tid >> 8) & 1, my_sub = (tid >> 7) & 1;
    const int ub = gemv_unit_bytes(sg.type), nw = p.w_stages;
    TcRaw cur;
#pragma unroll 1
    for (int blk = 0; blk < nblocks; ++blk) {
      {
        const int gb = blk0 + blk, slab = gb / p.S, bb = gb - slab * p.S;
        const int stage = blk % nw;
        tc_wait(p, &sh, &sh.w_full[stage], (uint32_t)((blk / nw) & 1));
        TcUnit u;
        u.unit = Wbase + (size_t)stage * p.w_stage_bytes + (size_t)my_row * ub;
        u.d = Dbase + (size_t)(slab & 1) * (TC_M * 32) + (size_t)my_row * 32 + 2 * bb;
        tc_fetch(sg.type, u, my_half, my_sub, cur);  // the thread's share of the block, into registers
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.w_empty[stage]);  // the stage may be refilled
      }
      const int adepth = p.a_stages >> 2;            // blocks the weight-tile ring holds
      const int abase = (blk % adepth) * 4, alap = blk / adepth;
#pragma unroll
      for (int kc = 0; kc < 4; ++kc) {
        uint8_t* A = Abase + (size_t)(abase + kc) * TC_M * 128;  // stage = step % a_stages
        uint4 w[2];
        tc_dequant16(sg.type, cur, kc, my_half, my_sub, w);
        // the MMAs that read this stage a ring lap ago must be done before it is overwritten
        if (alap >= 1) tc_wait(p, &sh, &sh.mma_done[abase + kc], (uint32_t)((alap - 1) & 1));
#pragma unroll
        for (int c = 0; c < 2; ++c) *reinterpret_cast<uint4*>(A + tc_swz(my_row, my_half * 4 + my_sub * 2 + c)) = w[c];
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.a_full[abase + kc]);  // one arrival per warp: 512 arrivals on one barrier word would serialise
      }
    }
  }
  // ---- epilogue: warp w reads TMEM lanes 32*(w & 3) .. +31 (= weight rows), the four warp groups split the tokens ----
  if (warp < TC_WORKERS / 32) tc_wait(p, &sh, &sh.done_bar, 0u);
  tc_fence_after();
  if (warp < TC_WORKERS / 32 && !*(volatile int*)&sh.abort_flag) {
    const int r_in_tile = 32 * (warp & 3) + lane;
    const int row_img = row0 + r_in_tile;
    const bool row_ok = row_img < sg.rows;
    const int ncol_q = p.NT / 4;  // the four warps that share a lane quarter split the tokens (NT is a multiple of 32)
    const int c_begin = (warp >> 2) * ncol_q;
    for (int c0 = c_begin; c0 < c_begin + ncol_q; c0 += 8) {
      float v[8];
      tc_ld8(tmem_d + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)c0, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int t = t0 + c0 + j;
        const bool ok = row_ok && t < p.T;
        const float tot = v[j];
        if (p.epi == EPI_SWIGLU) {
          // image rows: eight gate rows then the same eight up rows (reference model.cpp:734-735, batch form
          // cpu_batch_processor.cpp:252-256: (g / (1 + exp(-g))) * u)
          const float up = __shfl_sync(0xffffffffu, tot, (lane & 23) + 8);
          if (ok && (r_in_tile & 15) < 8) {
            const int orow = (row_img >> 4) * 8 + (r_in_tile & 7);
            p.y[(size_t)t * p.y_stride + orow] = (tot / (1.0f + expf(-tot))) * up;
          }
        } else {
          const float other = __shfl_xor_sync(0xffffffffu, tot, 1);
          if (ok) {
            if (p.epi == EPI_RESID) {
              const float* rs = (p.resid ? p.resid : p.y) + (size_t)t * p.y_stride + row_img;
              p.y[(size_t)t * p.y_stride + row_img] = *rs + tot;
            } else if (p.epi == EPI_QKV_ROPE) {
              float o = tot;
              if (seg < 2) {
                const int pos = p.positions[t];
                if (pos >= 0 && pos < p.max_pos) {
                  const int i = (row_img % p.head_dim) >> 1;
                  const float2 cs = *reinterpret_cast<const float2*>(p.rope + ((size_t)pos * (p.head_dim >> 1) + i) * 2);
                  o = (row_img & 1) ? __fadd_rn(__fmul_rn(other, cs.y), __fmul_rn(tot, cs.x))
                                    : __fsub_rn(__fmul_rn(tot, cs.x), __fmul_rn(other, cs.y));
                }
              }
              float* dst = seg == 0 ? p.y + (size_t)t * p.y_stride + row_img
                                    : p.y2 + (size_t)t * p.y2_stride + (seg == 2 ? p.seg[1].rows : 0) + row_img;
              *dst = o;
            } else {
              p.y[((size_t)blockIdx.z * p.T + t) * p.y_stride + row_img] = tot;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tc_dealloc(tmem_d, p.tmem_cols);
}

// Split-K epilogue: y[t][r] = base + sum_z part[z][t][r], z in order (deterministic); base = (resid ? resid : y)[t][r]
// when add_base is set, else 0.
// Four consecutive rows per thread (the launcher checks that rows and y_stride are multiples of 4).
__global__ void splitk_reduce_kernel(const float* __restrict__ part, int ksplit, int T, int rows, const float* __restrict__ resid, int add_base,
                                     float* __restrict__ y, int y_stride) {
  const size_t n = (size_t)T * rows, n4 = n / 4;
  const int rows4 = rows / 4;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / rows4, r = (i - t * rows4) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (add_base) acc = *reinterpret_cast<const float4*>((resid ? resid : y) + t * y_stride + r);
    for (int z = 0; z < ksplit; ++z) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(part + (size_t)z * n) + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4*>(y + t * y_stride + r) = acc;
  }
}

// x16[t][k] = fp16(x[t][k]) or, with norm weights, fp16(RMSNorm(x[t])[k]) (reference rmsnorm_batch_cpu,
// utils.cpp:613-646: f = 1/sqrtf(mean(x^2) + eps), out = x * f * w). One block of 512 threads per token;
// the row stays in registers between the two passes (rows of up to 16384 elements, else it is read again).
constexpr int TOH_THREADS = 512;
__global__ void __launch_bounds__(TOH_THREADS) to_half_kernel(const float* __restrict__ x, int x_stride, const float* __restrict__ norm_w, float eps, int K,
                                                              __half* __restrict__ out) {
  __shared__ float red[TOH_THREADS / 32 + 1];
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)t * x_stride);
  const int n4 = K / 4;  // K is a multiple of 256
  constexpr int KEEP = 8;
  float4 v[KEEP];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < KEEP; ++i) {
    const int j = tid + i * TOH_THREADS;
    v[i] = j < n4 ? xr[j] : make_float4(0.f, 0.f, 0.f, 0.f);
    ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  }
  for (int j = tid + KEEP * TOH_THREADS; j < n4; j += TOH_THREADS) {
    const float4 a = xr[j];
    ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  float f = 1.0f;
  if (norm_w) {
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (tid == 0) {
      float tot = 0.f;
      for (int w = 0; w < TOH_THREADS / 32; ++w) tot += red[w];
      red[TOH_THREADS / 32] = 1.0f / sqrtf(tot / (float)K + eps);
    }
    __syncthreads();
    f = red[TOH_THREADS / 32];
  }
  const float4* wr = reinterpret_cast<const float4*>(norm_w);
  uint2* orow = reinterpret_cast<uint2*>(out + (size_t)t * K);
  auto emit = [&](int j, float4 a) {
    if (norm_w) {
      const float4 w = __ldg(wr + j);
      a.x = a.x * f * w.x; a.y = a.y * f * w.y; a.z = a.z * f * w.z; a.w = a.w * f * w.w;
    }
    orow[j] = make_uint2(pack_h2(a.x, a.y), pack_h2(a.z, a.w));
  };
#pragma unroll
  for (int i = 0; i < KEEP; ++i) {
    const int j = tid + i * TOH_THREADS;
    if (j < n4) emit(j, v[i]);
  }
  for (int j = tid + KEEP * TOH_THREADS; j < n4; j += TOH_THREADS) emit(j, xr[j]);
}

}  // namespace b200
