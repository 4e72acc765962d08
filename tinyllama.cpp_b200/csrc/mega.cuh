// One persistent kernel per decode step (batch 1): every phase of every layer runs inside a
// single cooperative launch of one CTA per SM.
//
// Why: at batch 1 a 7B layer moves 127 MB, i.e. about 17 us of HBM time, in five dependent
// steps. As separate kernels each step pays a launch/dependency gap and a cold pipeline (about
// 3.5 us measured), which is more than the data time of the smaller steps. Here the producer warps
// run through the weight tiles of ALL phases in order, limited only by the shared-memory ring, so
// the next phase's weights are already on chip while the consumers finish a phase, cross the grid
// barrier and rebuild their activation image; HBM never drains between phases.
//
// Phases per layer: [RMSNorm+QKV+RoPE] | [KV append + split-K attention + merge] | [O proj +
// residual] | [RMSNorm + gate/up + SwiGLU] | [down proj + residual]; then [RMSNorm + lm_head +
// argmax partials] and the greedy token selection. Phases are separated by a grid-wide barrier
// (arrival counter in global memory, bounded spin).
#pragma once
#include "attn.cuh"
#include "gemv.cuh"

namespace b200 {

struct MegaLayer {
  GemvSeg q, k, v, o, gate, up, down;
  const float* attn_norm;
  const float* ffn_norm;
  void* k_cache;
  void* v_cache;
  float* k_scale;
  float* v_scale;
};

struct MegaParams {
  const MegaLayer* layers;  // device array [L]
  int L, H, F, KVD, nq, nkv, hd, V, max_ctx, max_pos;
  float eps, att_scale;
  GemvSeg head;
  const float* out_norm;
  const float* embd;
  const float* rope;
  int embed_from_tokens;    // 1: layer 0 reads the embedding row of tokens[0]; 0: h already holds the input
  int* tokens;
  int* positions;
  int* slots;
  float* h;
  float* q;
  float* kvnew;
  float* attn;
  float* act;
  float* logits;
  float* part_o;
  float* part_ml;
  int* tickets;
  int nsplit;
  float* amax_val;
  int* amax_idx;
  int* argmax_out;
  int* step_counter;
  const int* forced;
  const int* forced_steps;
  int* log;
  int log_cap;
  unsigned* grid_bar;       // arrival counter, zero at launch
  int* error_flag;
  int nstages;
};

enum : int { PH_QKV = 0, PH_O = 1, PH_GATEUP = 2, PH_DOWN = 3, PH_HEAD = 4 };

__device__ __forceinline__ void mega_make_gemv(const MegaParams& mp, int l, int kind, const float* x0, GemvParams& g) {
  g = GemvParams{};
  g.eps = mp.eps;
  g.error_flag = mp.error_flag;
  g.positions = mp.positions;
  g.rope = mp.rope;
  g.head_dim = mp.hd;
  g.max_pos = mp.max_pos;
  int max_ub;
  if (kind == PH_HEAD) {
    g.seg[0] = mp.head; g.nseg = 1; g.K = mp.H; g.norm_w = mp.out_norm; g.epi = EPI_STORE;
    g.y = mp.logits; g.y_stride = mp.V; g.amax_val = mp.amax_val; g.amax_idx = mp.amax_idx;
    g.ntiles = (mp.V + 15) / 16;
    max_ub = gemv_unit_bytes(mp.head.type);
  } else {
    const MegaLayer& w = mp.layers[l];
    if (kind == PH_QKV) {
      g.seg[0] = w.q; g.seg[1] = w.k; g.seg[2] = w.v; g.nseg = 3; g.K = mp.H; g.norm_w = w.attn_norm; g.epi = EPI_QKV_ROPE;
      g.y = mp.q; g.y_stride = mp.H; g.y2 = mp.kvnew; g.y2_stride = 2 * mp.KVD;
      g.ntiles = (mp.H + 2 * mp.KVD) / 16;
      max_ub = max(gemv_unit_bytes(w.q.type), max(gemv_unit_bytes(w.k.type), gemv_unit_bytes(w.v.type)));
    } else if (kind == PH_O) {
      g.seg[0] = w.o; g.nseg = 1; g.K = mp.H; g.epi = EPI_RESID; g.y = mp.h; g.y_stride = mp.H;
      g.resid = (l == 0 && x0) ? x0 : nullptr;
      g.ntiles = mp.H / 16;
      max_ub = gemv_unit_bytes(w.o.type);
    } else if (kind == PH_GATEUP) {
      g.seg[0] = w.gate; g.seg[1] = w.up; g.nseg = 2; g.K = mp.H; g.norm_w = w.ffn_norm; g.epi = EPI_SWIGLU;
      g.y = mp.act; g.y_stride = mp.F;
      g.ntiles = (mp.F + 7) / 8;
      max_ub = gemv_unit_bytes(w.gate.type);
    } else {
      g.seg[0] = w.down; g.nseg = 1; g.K = mp.F; g.epi = EPI_RESID; g.y = mp.h; g.y_stride = mp.H;
      g.ntiles = mp.H / 16;
      max_ub = gemv_unit_bytes(w.down.type);
    }
  }
  gemv_ring_geometry(g.K, g);
  (void)max_ub;
}

// Grid-wide barrier over the consumer threads of all CTAs (all CTAs are co-resident: cooperative
// launch). Bounded: after ~1 s of polling it records an error and lets the kernel run to its end.
__device__ __forceinline__ void mega_grid_sync(const MegaParams& mp, GemvShared* sh, unsigned& target, int ncta) {
  consumer_sync();
  if (threadIdx.x == 0) {
    target += (unsigned)ncta;
    __threadfence();
    atomicAdd(mp.grid_bar, 1u);
    if (!*(volatile int*)&sh->abort_flag) {
      bool ok = false;
      for (int i = 0; i < (1 << 24); ++i) {
        unsigned v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(mp.grid_bar) : "memory");
        if ((int)(v - target) >= 0) { ok = true; break; }
        if (i > 64) __nanosleep(40);
      }
      if (!ok) {
        sh->abort_flag = 1;
        if (mp.error_flag) atomicExch(mp.error_flag, 2);
      }
    }
    __threadfence();
  }
  consumer_sync();
}

template <int P, bool KV_I8>
__global__ void __launch_bounds__(GEMV_THREADS, 1) mega_decode_kernel(const MegaParams mp) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ GemvShared sh;
  __shared__ GemvParams g_cons;                   // the phase the consumers are in
  __shared__ GemvParams g_prod[GEMV_PROD_WARPS];  // the phase each producer warp is streaming
  __shared__ int attn_last[4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, ncta = gridDim.x;
  PipeCtx pc;
  pc.sh = &sh;
  pc.act = smem;
  pc.ring = smem + gemv_ring_offset(mp.F > mp.H ? mp.F : mp.H, P);
  pc.nstages = mp.nstages;
  pc.slot = 0;
  pc.use = 0;
  pc.gt = 0;
  pipe_init(&sh, mp.nstages);
  const float* x0 = nullptr;
  if (mp.embed_from_tokens) {
    int tok = mp.tokens[0];
    tok = min(max(tok, 0), mp.V - 1);
    x0 = mp.embd + (size_t)tok * mp.H;
  }
  const int nphase = 4 * mp.L + 1;

  if (warp >= GEMV_WARPS) {
    // ---- producers: the weight tiles of every phase, in order ----
    const int pw = warp - GEMV_WARPS;
#pragma unroll 1
    for (int ph = 0; ph < nphase; ++ph) {
      if (lane == 0) mega_make_gemv(mp, ph >> 2, ph == nphase - 1 ? PH_HEAD : (ph & 3), x0, g_prod[pw]);
      __syncwarp();
      gemv_produce(g_prod[pw], pc, pw, lane, cta, ncta);
      __syncwarp();
    }
    return;
  }

  // ---- consumers ----
  unsigned bar_target = 0;
  float best_v = -INFINITY;
  int best_i = 0x7fffffff;
#pragma unroll 1
  for (int ph = 0; ph < nphase; ++ph) {
    const int l = ph >> 2, kind = ph == nphase - 1 ? PH_HEAD : (ph & 3);
    if (threadIdx.x == 0) mega_make_gemv(mp, l, kind, x0, g_cons);
    consumer_sync();
    const float* xsrc = kind == PH_QKV ? ((l == 0 && x0) ? x0 : mp.h) : kind == PH_O ? mp.attn : kind == PH_DOWN ? mp.act : mp.h;
    XFromGlobal xfn{xsrc};
    gemv_consume<P>(g_cons, pc, xfn, 0, cta, ncta, best_v, best_i);
    if (kind == PH_HEAD) gemv_store_argmax(g_cons, &sh, best_v, best_i, 0, cta, ncta);
    mega_grid_sync(mp, &sh, bar_target, ncta);
    if (kind != PH_QKV) continue;
    // attention: (head, split) items over 4-warp groups of all CTAs; the last group of a head merges
    {
      const MegaLayer& w = mp.layers[l];
      AttnParams a{};
      a.q = mp.q; a.kv_new = mp.kvnew; a.q_stride = mp.H; a.kvn_stride = 2 * mp.KVD;
      a.k_cache = w.k_cache; a.v_cache = w.v_cache; a.k_scale = w.k_scale; a.v_scale = w.v_scale;
      a.positions = mp.positions; a.slots = mp.slots;
      a.nq = mp.nq; a.nkv = mp.nkv; a.hd = mp.hd; a.max_ctx = mp.max_ctx; a.nsplit = mp.nsplit;
      a.part_o = mp.part_o; a.part_ml = mp.part_ml; a.tickets = mp.tickets;
      a.out = mp.attn; a.out_stride = mp.H; a.att_scale = mp.att_scale;
      const int grp = warp >> 2, gtid = threadIdx.x & (ATTN_GROUP_THREADS - 1);
      float* gsm = reinterpret_cast<float*>(smem) + (size_t)grp * attn_group_floats(mp.hd, mp.max_ctx, mp.nsplit);
      const int nitems = mp.nq * mp.nsplit;
      for (int item = cta * 4 + grp; item < nitems; item += ncta * 4) {
        const int hq = item / mp.nsplit, split = item - hq * mp.nsplit;
        attn_item<KV_I8>(a, split, hq, 0, gsm, gtid, 9 + grp);
        group_sync(9 + grp);
        if (gtid == 0) {
          __threadfence();
          attn_last[grp] = (atomicAdd(&mp.tickets[hq], 1) == mp.nsplit - 1);
          if (attn_last[grp]) __threadfence();
        }
        group_sync(9 + grp);
        if (attn_last[grp]) {
          attn_merge_head(a, 0, hq, gtid, ATTN_GROUP_THREADS, mp.attn + hq * mp.hd);
          if (gtid == 0) mp.tickets[hq] = 0;
        }
        group_sync(9 + grp);
      }
    }
    mega_grid_sync(mp, &sh, bar_target, ncta);
  }
  // greedy selection and bookkeeping for the next step (reference api.cpp:134-136: first maximum)
  if (cta == 0 && warp == 0) {
    const int step = *mp.step_counter;
    const int fsteps = mp.forced ? *mp.forced_steps : 0;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lane; i < ncta; i += 32) {
      const float v = __ldcg(&mp.amax_val[i]);
      const int idx = __ldcg(&mp.amax_idx[i]);
      if (v > bv || (v == bv && idx < bi)) { bv = v; bi = idx; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) {
      mp.argmax_out[0] = bi;
      int next = bi;
      if (step + 1 < fsteps) next = mp.forced[step + 1];
      mp.tokens[0] = next;
      mp.positions[0] += 1;
      if (step < mp.log_cap) mp.log[step] = bi;
      *mp.step_counter = step + 1;
    }
  }
}

}  // namespace b200
