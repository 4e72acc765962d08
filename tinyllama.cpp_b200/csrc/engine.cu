// Engine: weight residency, KV cache, the per-token launch sequence and its CUDA graph.
#include "engine.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>

#include "attn.cuh"
#include "dequant.cuh"
#include "gemv.cuh"
#include "gguf.h"
#include "mega.cuh"
#include "misc.cuh"
#include "tp.h"

namespace b200 {

thread_local std::string g_err;

template <typename T>
static T* dev_alloc(b200_engine* e, size_t n) {
  void* p = nullptr;
  CK(cudaMalloc(&p, std::max<size_t>(n * sizeof(T), 16)));
  if (e) e->allocations.push_back(p);
  return static_cast<T*>(p);
}

static void set_gemv_attrs() {
  static bool done = false;
  if (done) return;
  const int maxb = 216 * 1024;
  CK(cudaFuncSetAttribute(gemv_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, maxb));
  CK(cudaFuncSetAttribute(gemv_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, maxb));
  CK(cudaFuncSetAttribute((mega_decode_kernel<2, true>), cudaFuncAttributeMaxDynamicSharedMemorySize, maxb));
  CK(cudaFuncSetAttribute((mega_decode_kernel<2, false>), cudaFuncAttributeMaxDynamicSharedMemorySize, maxb));
  CK(cudaFuncSetAttribute((mega_decode_kernel<3, true>), cudaFuncAttributeMaxDynamicSharedMemorySize, maxb));
  CK(cudaFuncSetAttribute((mega_decode_kernel<3, false>), cudaFuncAttributeMaxDynamicSharedMemorySize, maxb));
  CK(cudaFuncSetAttribute(attn_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
  CK(cudaFuncSetAttribute(attn_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
  done = true;
}

// Uploads one packed tensor and regroups Q6_K / Q8_0 into aligned 256-element units on the device.
static void upload_packed(b200_engine* e, DevTensor& t, int type, const void* host, size_t bytes, int64_t rows, int64_t cols,
                          cudaStream_t stream) {
  const int64_t be = type_block_elems(type), bb = type_block_bytes(type);
  if (cols % 256) throw std::runtime_error("tensor columns must be a multiple of 256");
  const size_t nblk = (size_t)(rows * cols / be);
  if (bytes != nblk * (size_t)bb) throw std::runtime_error("tensor byte count does not match rows x cols for its type");
  t.type = type; t.rows = rows; t.cols = cols; t.bytes = bytes;
  t.base = dev_alloc<uint8_t>(e, bytes + 256);
  if (type == T_Q6_K || type == T_Q8_0) {
    uint8_t* stage = nullptr;
    CK(cudaMalloc((void**)&stage, bytes));
    CK(cudaMemcpyAsync(stage, host, bytes, cudaMemcpyHostToDevice, stream));
    const unsigned grid = (unsigned)((bytes + 255) / 256);
    if (type == T_Q6_K) {
      t.d = t.base + (nblk * 208 + 15) / 16 * 16;
      split_q6_k_kernel<<<grid, 256, 0, stream>>>(stage, nblk, t.base, t.d);
    } else {
      regroup_q8_0_kernel<<<grid, 256, 0, stream>>>(stage, nblk, t.base);
    }
    CK(cudaGetLastError());
    CK(cudaStreamSynchronize(stream));
    CK(cudaFree(stage));
  } else {
    CK(cudaMemcpyAsync(t.base, host, bytes, cudaMemcpyHostToDevice, stream));
    CK(cudaStreamSynchronize(stream));
  }
}

static GemvSeg seg_of(const DevTensor& t) {
  GemvSeg s;
  s.w = t.base; s.d = t.d; s.type = t.type; s.rows = (int)t.rows;
  return s;
}

// Fills in the tile count and ring geometry, checks the launch's shape rules and starts the
// kernel with one persistent CTA per SM (fewer when there are fewer tiles), as a programmatic
// dependent launch when the engine allows it. Returns the grid width.
static int launch_gemv(const b200_engine* e, GemvParams p, int batch, cudaStream_t st) {
  if (p.K % 256) throw std::runtime_error("gemv: K must be a multiple of 256");
  int max_ub = 0;
  for (int s = 0; s < p.nseg; ++s) max_ub = std::max(max_ub, gemv_unit_bytes(p.seg[s].type));
  if (p.epi == EPI_SWIGLU) {
    if (p.nseg != 2 || p.seg[0].rows != p.seg[1].rows || p.seg[0].type != p.seg[1].type)
      throw std::runtime_error("gemv: gate and up must have the same shape and block type");
    p.ntiles = (p.seg[0].rows + 7) / 8;
  } else {
    int rows = 0;
    for (int s = 0; s < p.nseg; ++s) {
      if (s + 1 < p.nseg && p.seg[s].rows % 16) throw std::runtime_error("gemv: segment rows must be a multiple of 16");
      rows += p.seg[s].rows;
    }
    p.ntiles = (rows + 15) / 16;
  }
  gemv_ring_geometry(p.K, p);
  (void)max_ub;
  const size_t ring_off = gemv_ring_offset(p.K, e->P);
  const size_t budget = 214 * 1024;
  if (ring_off + 2 * (size_t)GEMV_SLOT_BYTES > budget) throw std::runtime_error("gemv: input dimension too large for shared memory");
  const int nstages = (int)std::min<size_t>(GEMV_MAX_STAGES, (budget - ring_off) / GEMV_SLOT_BYTES);
  p.error_flag = e->d_error;
  const size_t smem = ring_off + (size_t)nstages * GEMV_SLOT_BYTES;
  const int gx = std::max(1, std::min(p.ntiles, e->num_sms));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(gx, batch);
  cfg.blockDim = dim3(GEMV_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = e->use_pdl ? 1 : 0;
  if (e->P == 2) CK(cudaLaunchKernelEx(&cfg, gemv_kernel<2>, p, nstages));
  else CK(cudaLaunchKernelEx(&cfg, gemv_kernel<3>, p, nstages));
  return gx;
}


static int attn_nsplit(const b200_engine* e, int batch) {
  int want = (4 * e->num_sms + e->nq * batch - 1) / (e->nq * batch);
  return std::max(1, std::min(want, 32));
}

// Ring depth the persistent kernel can afford for this model, or 0 when it does not fit.
static int mega_stage_count(const b200_engine* e) {
  const size_t ring_off = gemv_ring_offset(std::max(e->F, e->H), e->P);
  const size_t budget = 214 * 1024;
  if (ring_off + 2 * (size_t)GEMV_SLOT_BYTES > budget) return 0;
  if (4 * attn_group_floats(e->hd, e->max_ctx, attn_nsplit(e, 1)) * sizeof(float) > ring_off) return 0;
  return (int)std::min<size_t>(GEMV_MAX_STAGES, (budget - ring_off) / GEMV_SLOT_BYTES);
}

// One decode step of a single sequence as ONE cooperative launch (see mega.cuh).
static int enqueue_mega(b200_engine* e, cudaStream_t st, bool with_embed) {
  MegaParams mp{};
  mp.layers = static_cast<const MegaLayer*>(e->d_mega_layers);
  mp.L = e->L; mp.H = e->H; mp.F = e->F; mp.KVD = e->KVD; mp.nq = e->nq; mp.nkv = e->nkv; mp.hd = e->hd; mp.V = e->V;
  mp.max_ctx = e->max_ctx; mp.max_pos = e->desc.max_position_embeddings;
  mp.eps = std::max(e->desc.rms_norm_eps, 1e-5f);
  mp.att_scale = 1.0f / std::sqrt((float)e->hd);
  mp.head = seg_of(e->out_w); mp.out_norm = e->out_norm.f32(); mp.embd = e->tok_embd.f32(); mp.rope = e->rope;
  mp.embed_from_tokens = with_embed ? 1 : 0;
  mp.tokens = e->d_tokens; mp.positions = e->d_positions; mp.slots = e->d_slots;
  mp.h = e->d_h; mp.q = e->d_q; mp.kvnew = e->d_kvnew; mp.attn = e->d_attn; mp.act = e->d_act; mp.logits = e->d_logits;
  mp.part_o = e->d_part_o; mp.part_ml = e->d_part_ml; mp.tickets = e->d_tickets; mp.nsplit = attn_nsplit(e, 1);
  mp.amax_val = e->d_amax_val; mp.amax_idx = e->d_amax_idx; mp.argmax_out = e->d_argmax; mp.step_counter = e->d_step;
  mp.forced = e->d_forced; mp.forced_steps = e->d_forced_steps; mp.log = e->d_log; mp.log_cap = e->log_cap;
  mp.grid_bar = e->d_grid_bar; mp.error_flag = e->d_error; mp.nstages = e->mega_stages;
  CK(cudaMemsetAsync(e->d_grid_bar, 0, sizeof(unsigned), st));
  const size_t smem = gemv_ring_offset(std::max(e->F, e->H), e->P) + (size_t)e->mega_stages * GEMV_SLOT_BYTES;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(e->num_sms);
  cfg.blockDim = dim3(GEMV_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const bool i8 = e->desc.kv_dtype == B200_KV_I8;
  if (e->P == 2) {
    if (i8) CK(cudaLaunchKernelEx(&cfg, mega_decode_kernel<2, true>, mp));
    else CK(cudaLaunchKernelEx(&cfg, mega_decode_kernel<2, false>, mp));
  } else {
    if (i8) CK(cudaLaunchKernelEx(&cfg, mega_decode_kernel<3, true>, mp));
    else CK(cudaLaunchKernelEx(&cfg, mega_decode_kernel<3, false>, mp));
  }
  return 1;
}

// Tensor parallel: sum the partial [batch, H] outputs over the ranks, then add them to the residual stream.
static int tp_reduce_add(b200_engine* e, int batch, cudaStream_t st) {
  Nccl& n = Nccl::get();
  const size_t count = (size_t)batch * e->H;
  n.check(n.AllReduce(e->d_partial, e->d_partial, count, Nccl::kFloat32, Nccl::kSum, e->nccl_comm, st), "ncclAllReduce");
  add_inplace_kernel<<<(unsigned)((count + 255) / 256), 256, 0, st>>>(e->d_h, e->d_partial, (int)count);
  CK(cudaGetLastError());
  return 2;
}

// The launch sequence of one decode step for `batch` sequences (also what gets captured).
// Per layer: [RMSNorm + QKV + RoPE] -> [KV append + attention] -> [O proj + residual] ->
// [RMSNorm + gate/up + SwiGLU] -> [down proj + residual]; then [RMSNorm + lm_head + argmax
// partials] and token selection. Returns the number of kernel launches.
static int enqueue_step(b200_engine* e, int batch, int nsplit, cudaStream_t st, bool with_embed, int* head_ctas_out) {
  int launches = 0;
  const int H = e->H, F = e->F, KVD = e->KVD;
  const float eps = std::max(e->desc.rms_norm_eps, 1e-5f);  // reference utils.cpp:666-667
  const bool tp = e->tp_size > 1;
  if (batch == 1 && e->use_mega && e->mega_stages >= 2 && !tp) {
    if (head_ctas_out) *head_ctas_out = e->num_sms;
    return enqueue_mega(e, st, with_embed);
  }
  if (with_embed) {
    embed_kernel<<<batch, 256, 0, st>>>(e->d_tokens, e->tok_embd.f32(), e->d_h, H, e->V);
    CK(cudaGetLastError());
    ++launches;
  }
  for (int l = 0; l < e->L; ++l) {
    const LayerW& w = e->layers[l];
    {
      GemvParams p{};
      p.seg[0] = seg_of(w.wq); p.seg[1] = seg_of(w.wk); p.seg[2] = seg_of(w.wv); p.nseg = 3;
      p.K = H; p.x = e->d_h; p.x_stride = H; p.norm_w = w.attn_norm.f32(); p.eps = eps; p.epi = EPI_QKV_ROPE;
      p.y = e->d_q; p.y_stride = e->Hq; p.y2 = e->d_kvnew; p.y2_stride = 2 * KVD;
      p.rope = e->rope; p.positions = e->d_positions; p.head_dim = e->hd; p.max_pos = e->desc.max_position_embeddings;
      launch_gemv(e, p, batch, st);
      ++launches;
    }
    {
      AttnParams a{};
      a.q = e->d_q; a.kv_new = e->d_kvnew; a.q_stride = e->Hq; a.kvn_stride = 2 * KVD;
      a.k_cache = w.k_cache; a.v_cache = w.v_cache; a.k_scale = w.k_scale; a.v_scale = w.v_scale;
      a.positions = e->d_positions; a.slots = e->d_slots;
      a.nq = e->nq; a.nkv = e->nkv; a.hd = e->hd; a.max_ctx = e->max_ctx; a.nsplit = nsplit;
      a.part_o = e->d_part_o; a.part_ml = e->d_part_ml; a.tickets = e->d_tickets;
      a.out = e->d_attn; a.out_stride = e->Hq; a.att_scale = 1.0f / std::sqrt((float)e->hd);
      const size_t smem = attn_smem_bytes(e->hd, e->max_ctx, nsplit, 4);
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(nsplit, e->nq, batch);
      cfg.blockDim = dim3(ATTN_GROUP_THREADS);
      cfg.dynamicSmemBytes = smem;
      cfg.stream = st;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = e->use_pdl ? 1 : 0;
      if (e->desc.kv_dtype == B200_KV_I8) CK(cudaLaunchKernelEx(&cfg, attn_decode_kernel<true>, a));
      else CK(cudaLaunchKernelEx(&cfg, attn_decode_kernel<false>, a));
      ++launches;
    }
    {
      GemvParams p{};
      p.seg[0] = seg_of(w.wo); p.nseg = 1; p.K = e->Hq; p.x = e->d_attn; p.x_stride = e->Hq; p.epi = tp ? EPI_STORE : EPI_RESID;
      p.y = tp ? e->d_partial : e->d_h; p.y_stride = H;
      launch_gemv(e, p, batch, st);
      ++launches;
      if (tp) launches += tp_reduce_add(e, batch, st);
    }
    {
      GemvParams p{};
      p.seg[0] = seg_of(w.wgate); p.seg[1] = seg_of(w.wup); p.nseg = 2;
      p.K = H; p.x = e->d_h; p.x_stride = H; p.norm_w = w.ffn_norm.f32(); p.eps = eps; p.epi = EPI_SWIGLU;
      p.y = e->d_act; p.y_stride = F;
      launch_gemv(e, p, batch, st);
      ++launches;
    }
    {
      GemvParams p{};
      p.seg[0] = seg_of(w.wdown); p.nseg = 1; p.K = F; p.x = e->d_act; p.x_stride = F; p.epi = tp ? EPI_STORE : EPI_RESID;
      p.y = tp ? e->d_partial : e->d_h; p.y_stride = H;
      launch_gemv(e, p, batch, st);
      ++launches;
      if (tp) launches += tp_reduce_add(e, batch, st);
    }
  }
  {
    GemvParams p{};
    p.seg[0] = seg_of(e->out_w); p.nseg = 1; p.K = H; p.x = e->d_h; p.x_stride = H;
    p.norm_w = e->out_norm.f32(); p.eps = eps; p.epi = EPI_STORE;
    // each rank computes its share of the vocabulary; shares and argmax partials are then gathered
    const size_t half = (size_t)e->max_seqs * e->amax_cap * e->tp_size;
    p.y = tp ? e->d_logits_local : e->d_logits; p.y_stride = e->Vl;
    p.amax_val = tp ? e->d_amax_val + half : e->d_amax_val; p.amax_idx = tp ? e->d_amax_idx + half : e->d_amax_idx;
    p.amax_row_offset = e->tp_rank * e->Vl;
    const int grid = launch_gemv(e, p, batch, st);
    ++launches;
    if (tp) {
      Nccl& n = Nccl::get();
      n.check(n.AllGather(e->d_logits_local, e->d_logits, (size_t)batch * e->Vl, Nccl::kFloat32, e->nccl_comm, st), "ncclAllGather");
      n.check(n.AllGather(p.amax_val, e->d_amax_val, (size_t)batch * grid, Nccl::kFloat32, e->nccl_comm, st), "ncclAllGather");
      n.check(n.AllGather(p.amax_idx, e->d_amax_idx, (size_t)batch * grid, Nccl::kInt32, e->nccl_comm, st), "ncclAllGather");
      launches += 3;
    }
    if (head_ctas_out) *head_ctas_out = grid;
    SelectParams s{};
    s.amax_val = e->d_amax_val; s.amax_idx = e->d_amax_idx; s.nparts = grid * e->tp_size; s.parts_per_rank = grid; s.batch = batch;
    s.tokens = e->d_tokens; s.positions = e->d_positions; s.argmax_out = e->d_argmax; s.step_counter = e->d_step;
    s.forced = e->d_forced; s.forced_steps = e->d_forced_steps; s.log = e->d_log; s.log_cap = e->log_cap;
    select_kernel<<<1, 256, 0, st>>>(s);
    CK(cudaGetLastError());
    ++launches;
  }
  return launches;
}

static StepGraph& get_graph(b200_engine* e, int batch, bool with_embed = true) {
  const int key = batch * 2 + (with_embed ? 1 : 0);
  auto it = e->graphs.find(key);
  if (it != e->graphs.end()) return it->second;
  StepGraph g;
  g.nsplit = attn_nsplit(e, batch);
  cudaGraph_t graph = nullptr;
  CK(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
  try {
    g.launches = enqueue_step(e, batch, g.nsplit, e->stream, with_embed, &g.head_ctas);
  } catch (...) {
    cudaStreamEndCapture(e->stream, &graph);
    if (graph) cudaGraphDestroy(graph);
    throw;
  }
  CK(cudaStreamEndCapture(e->stream, &graph));
  CK(cudaGraphInstantiate(&g.exec, graph, 0));
  CK(cudaGraphDestroy(graph));
  return e->graphs.emplace(key, g).first->second;
}

}  // namespace b200

#include "engine_abi.inc"
#include "engine_noalloc.inc"
