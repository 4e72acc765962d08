// Shared device/host helpers for the sm_100a decode engine.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>
#include <string>

namespace b200 {

// Step trace: when a launch is given a record (eight 64-bit slots), the first thread of its first
// CTA writes the GPU's global nanosecond timer there at fixed points of the kernel.
__device__ __forceinline__ void trace_stamp(unsigned long long* rec, int col) {
  if (rec) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    rec[col] = t;
  }
}


enum : int { T_F32 = 0, T_Q8_0 = 8, T_Q4_K = 12, T_Q6_K = 14 };

struct CudaError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

inline void cuda_check(cudaError_t e, const char* what, const char* file, int line) {
  if (e != cudaSuccess) {
    throw CudaError(std::string(what) + ": " + cudaGetErrorString(e) + " (" + file + ":" + std::to_string(line) + ")");
  }
}
#define CK(x) ::b200::cuda_check((x), #x, __FILE__, __LINE__)

inline int64_t type_block_elems(int t) { return t == T_Q8_0 ? 32 : (t == T_Q4_K || t == T_Q6_K) ? 256 : 1; }
inline int64_t type_block_bytes(int t) { return t == T_Q8_0 ? 34 : t == T_Q4_K ? 144 : t == T_Q6_K ? 210 : 4; }

// ---- device helpers ----
__device__ __forceinline__ uint4 ldg128(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

// 4-way byte dot products (weights a, activation digits b).
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

__device__ __forceinline__ float half_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace b200
