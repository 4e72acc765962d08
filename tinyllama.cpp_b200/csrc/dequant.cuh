// Exact block dequantizers (parity tools) and the load-time plane split of Q6_K / Q8_0.
#pragma once
#include "common.cuh"

namespace b200 {

// fp16 -> fp32 of a GGUF scale field: finite negatives become positive
// (reference quantization.cpp:85-87; used for Q8_0 only, quantization.cpp:1048).
__device__ __forceinline__ float scale_field_to_float(uint16_t h) {
  float f = half_bits_to_float(h);
  if (f < 0.0f && !isnan(f) && !isinf(f)) f = fabsf(f);
  return f;
}

// 6-bit scale / min of sub-block j of a Q4_K block (reference quantization.cpp:145-155).
__device__ __forceinline__ void q4k_scale_min(int j, const uint8_t* q, int& sc, int& mn) {
  if (j < 4) {
    sc = q[j] & 63;
    mn = q[j + 4] & 63;
  } else {
    sc = (q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4);
    mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

// One thread per output element; every multiply and subtract is rounded separately
// (__fmul_rn / __fsub_rn are never contracted into an FMA), which is what makes the
// result bit-identical to the reference's x86-64 build.
__global__ void dequant_q8_0_kernel(const uint8_t* __restrict__ blocks, size_t n_elems, float* __restrict__ out) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_elems) return;
  const uint8_t* b = blocks + (i / 32) * 34;
  uint16_t dh = (uint16_t)b[0] | ((uint16_t)b[1] << 8);
  float d = scale_field_to_float(dh);
  out[i] = __fmul_rn(d, (float)(int8_t)b[2 + (i % 32)]);
}

__global__ void dequant_q4_k_kernel(const uint8_t* __restrict__ blocks, size_t n_elems, float* __restrict__ out) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_elems) return;
  const uint8_t* b = blocks + (i / 256) * 144;
  const int e = (int)(i % 256), c = e / 64, w = e % 64, l = w % 32, hi = w / 32;
  float d = half_bits_to_float((uint16_t)b[0] | ((uint16_t)b[1] << 8));
  float dmin = half_bits_to_float((uint16_t)b[2] | ((uint16_t)b[3] << 8));
  int sc, mn;
  q4k_scale_min(2 * c + hi, b + 4, sc, mn);
  float d1 = __fmul_rn(d, (float)sc), mf = __fmul_rn(dmin, (float)mn);
  int q = hi ? (b[16 + 32 * c + l] >> 4) : (b[16 + 32 * c + l] & 0x0F);
  out[i] = __fsub_rn(__fmul_rn(d1, (float)q), mf);
}

__global__ void dequant_q6_k_kernel(const uint8_t* __restrict__ blocks, size_t n_elems, float* __restrict__ out) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_elems) return;
  const uint8_t* b = blocks + (i / 256) * 210;
  const int e = (int)(i % 256), h = e / 128, r = e % 128, g = r / 32, l = r % 32, is = l / 16;
  const uint8_t* ql = b + 64 * h;
  const uint8_t qh = b[128 + 32 * h + l];
  const int8_t sc = (int8_t)b[192 + 8 * h + 2 * g + is];
  float d = half_bits_to_float((uint16_t)b[208] | ((uint16_t)b[209] << 8));
  int q;
  if (g == 0) q = (ql[l] & 0x0F) | (((qh >> 0) & 3) << 4);
  else if (g == 1) q = (ql[l + 32] & 0x0F) | (((qh >> 2) & 3) << 4);
  else if (g == 2) q = (ql[l] >> 4) | (((qh >> 4) & 3) << 4);
  else q = (ql[l + 32] >> 4) | (((qh >> 6) & 3) << 4);
  q -= 32;
  out[i] = __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
}

// ---- load-time regrouping ---------------------------------------------------------------
// A Q6_K block is 210 bytes and a Q8_0 block 34 bytes, so in a row of them nothing sits on the
// 16-byte boundaries that bulk copies and 128-bit loads need. On the device the same bytes are
// therefore kept as 16-byte-aligned units of 256 elements (see gemv_unit_bytes):
//   Q6_K: unit = first 208 bytes of the block (ql | qh | scales); the trailing fp16 d of every
//         block goes to a separate plane d[block]
//   Q8_0: unit = 272 bytes = the 32 quants of 8 consecutive blocks, then their 8 fp16 d
// The byte count is unchanged (210 / 34 per block); nothing is expanded. Q4_K blocks are
// 144 = 9 x 16 bytes and stay exactly as in the file.
__global__ void split_q6_k_kernel(const uint8_t* __restrict__ src, size_t n_blocks, uint8_t* __restrict__ units,
                                  uint8_t* __restrict__ dplane) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_blocks * 210) return;
  size_t blk = i / 210;
  int o = (int)(i % 210);
  if (o < 208) units[blk * 208 + o] = src[i];
  else dplane[blk * 2 + (o - 208)] = src[i];
}

__global__ void regroup_q8_0_kernel(const uint8_t* __restrict__ src, size_t n_blocks, uint8_t* __restrict__ units) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_blocks * 34) return;
  size_t blk = i / 34, grp = blk / 8;
  int j = (int)(blk % 8), o = (int)(i % 34);
  units[grp * 272 + (o < 2 ? 256 + 2 * j + o : 32 * j + (o - 2))] = src[i];
}

}  // namespace b200
