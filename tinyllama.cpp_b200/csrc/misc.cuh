// Small kernels around the layer loop: embedding gather and greedy token selection.
#pragma once
#include "common.cuh"

namespace b200 {

// TinyLlamaModel::lookup_embedding for an FP32 table (reference model_utils.cpp:11-182):
// h[b][:] = token_embd[tokens[b]][:]. grid.x = batch.
__global__ void embed_kernel(const int* __restrict__ tokens, const float* __restrict__ embd, float* __restrict__ h, int H, int vocab) {
  const int b = blockIdx.x;
  int tok = tokens[b];
  tok = min(max(tok, 0), vocab - 1);
  const float4* src = reinterpret_cast<const float4*>(embd + (size_t)tok * H);
  float4* dst = reinterpret_cast<float4*>(h + (size_t)b * H);
  for (int i = threadIdx.x; i < H / 4; i += blockDim.x) dst[i] = __ldg(src + i);
}

// Greedy sampling (reference api.cpp:134-136: first maximum) from the per-CTA partials the
// lm_head kernel left, then bookkeeping for the next step: tokens[b] <- chosen (or the forced
// token while a prompt is being replayed), positions[b] += 1, and the id is appended to the
// step log. One block; warp w handles sequences w, w+nwarps, ...
constexpr int PEN_WINDOW = 64;  // reference apply_repetition_penalty: window = 64 generated tokens

struct SelectParams {
  const float* amax_val;  // [ranks][batch][parts_per_rank]
  const int* amax_idx;
  int nparts;             // ranks * parts_per_rank
  int parts_per_rank;
  int batch;
  int* tokens;            // [batch] in: this step's token, out: next step's
  int* positions;         // [batch]
  int* argmax_out;        // [batch] argmax of this step's logits
  int* step_counter;      // steps done since the loop was armed
  const int* forced;      // [forced_steps][batch] tokens to feed instead of the argmax, or nullptr
  const int* forced_steps;// device scalar
  int* log;               // [log_cap][batch]
  int log_cap;
  unsigned* epoch;        // tensor-parallel exchange counter to advance at the end of the step, or nullptr
  unsigned epoch_inc;
  // tensor parallel over peer memory: the partials arrive as packets {value, index | (number & 0x7fff) << 17} in
  // amax_pkts (same [ranks][batch][parts_per_rank] order) and are polled (bounded) instead of read from amax_val / amax_idx
  const uint2* amax_pkts;
  unsigned epoch_k;       // this exchange's number = *epoch + epoch_k
  int* error_flag;
  // repetition penalty: the window of the last PEN_WINDOW generated ids of every sequence (a ring and its running
  // count) and the per-id occurrence counts the lm_head launch reads; nullptr: no penalty bookkeeping
  int* pen_ring;          // [batch][PEN_WINDOW]
  int* pen_count;         // [batch]
  uint8_t* pen_counts;    // [batch][pen_stride]
  int pen_stride;
};

__global__ void select_kernel(const SelectParams p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int step = *p.step_counter;
  const int fsteps = p.forced ? *p.forced_steps : 0;
  const unsigned want = p.amax_pkts ? ((*p.epoch + p.epoch_k) & 0x7fffu) : 0u;
#pragma unroll 1
  for (int b = warp; b < p.batch; b += nwarps) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll 1
    for (int i = lane; i < p.nparts; i += 32) {
      const size_t at = ((size_t)(i / p.parts_per_rank) * p.batch + b) * p.parts_per_rank + (i % p.parts_per_rank);
      float v;
      int idx;
      if (p.amax_pkts) {
        uint2 pk;
        int it = 0;
        while (true) {
          asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(pk.x), "=r"(pk.y) : "l"(p.amax_pkts + at));
          if ((pk.y >> 17) == want) break;
          if (++it > (1 << 22)) {  // bounded: a rank has gone away
            if (p.error_flag) *reinterpret_cast<volatile int*>(p.error_flag) = 1;
            break;
          }
          if (it > 16) __nanosleep(32);
        }
        v = __uint_as_float(pk.x);
        idx = (int)(pk.y & 0x1ffffu);
      } else {
        v = p.amax_val[at];
        idx = p.amax_idx[at];
      }
      if (v > bv || (v == bv && idx < bi)) { bv = v; bi = idx; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (p.pen_ring && lane == 0) {
      // the chosen id enters the window of generated tokens, the id generated PEN_WINDOW steps ago leaves it
      int* ring = p.pen_ring + (size_t)b * PEN_WINDOW;
      uint8_t* counts = p.pen_counts + (size_t)b * p.pen_stride;
      const int cnt = p.pen_count[b];
      const int at = cnt % PEN_WINDOW;
      if (cnt >= PEN_WINDOW) {
        const int old = ring[at];
        if (old >= 0) counts[old] -= 1;
      }
      ring[at] = bi;
      counts[bi] += 1;
      p.pen_count[b] = cnt + 1;
    }
    if (lane == 0) {
      p.argmax_out[b] = bi;
      int next = bi;
      if (step + 1 < fsteps) next = p.forced[(size_t)(step + 1) * p.batch + b];
      p.tokens[b] = next;
      p.positions[b] += 1;
      if (step < p.log_cap) p.log[(size_t)step * p.batch + b] = bi;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *p.step_counter = step + 1;
    if (p.epoch) *p.epoch += p.epoch_inc;
  }
}

// First maximum of each row of logits [batch][vocab] (reference api.cpp:134-136), in the partial
// format select_kernel merges (one part per sequence). One block per sequence.
__global__ void argmax_rows_kernel(const float* __restrict__ logits, int vocab, int index_offset, float* __restrict__ amax_val,
                                   int* __restrict__ amax_idx) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const float* row = logits + (size_t)b * vocab;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
#pragma unroll 1
  for (int i = tid; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (v > bv) { bv = v; bi = i; }  // increasing i per thread: the first maximum stays
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < nwarps; ++w)
      if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
    amax_val[b] = bv;
    amax_idx[b] = bi + index_offset;  // offset of this rank's share of the vocabulary
  }
}

// h[i] += partial[i]: the residual add after a tensor-parallel all-reduce.
__global__ void add_inplace_kernel(float* __restrict__ h, const float* __restrict__ partial, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) h[i] = h[i] + partial[i];
}

// fp16 -> fp32, element by element (op-level checks of the batch RMSNorm path).
__global__ void half_to_float_kernel(const __half* __restrict__ in, float* __restrict__ out, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __half2float(in[i]);
}

}  // namespace b200
