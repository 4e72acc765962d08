// Engine: weight residency, KV cache, the per-token launch sequence and its CUDA graph.
#include "engine.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <thread>

#include "attn.cuh"
#include "attn_cluster.cuh"
#include "attn_prefill.cuh"
#include "dequant.cuh"
#include "gemv.cuh"
#include "gemm_tc.cuh"
#include "gguf.h"
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

// memcpy split over a few threads: one thread moves 5-8 GB/s out of the page cache, which is less than the link takes.
static void parallel_memcpy(void* dst, const void* src, size_t n) {
  const int nt = n >= ((size_t)8 << 20) ? 4 : 1;
  if (nt == 1) { std::memcpy(dst, src, n); return; }
  std::thread th[4];
  const size_t per = (n / nt + 4095) & ~(size_t)4095;
  for (int i = 0; i < nt; ++i) {
    const size_t off = std::min(n, per * i), len = std::min(per, n - off);
    th[i] = std::thread([=] { if (len) std::memcpy(static_cast<uint8_t*>(dst) + off, static_cast<const uint8_t*>(src) + off, len); });
  }
  for (int i = 0; i < nt; ++i) th[i].join();
}

// cuTensorMapEncodeTiled, fetched from the driver at run time (the library links only the runtime).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn tensor_map_encoder() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    if (!p || q != cudaDriverEntryPointSuccess) throw std::runtime_error("cuTensorMapEncodeTiled is not available from this driver");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Raises the kernels' dynamic shared-memory limits. The attribute belongs to the device that is
// current when it is set, so this runs once per device ordinal, not once per process.
static void set_gemv_attrs() {
  static bool done[64] = {false};
  int dev = 0;
  CK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) throw std::runtime_error("device ordinal out of range");
  if (done[dev]) return;
  const int maxb = GEMV_SMEM_BUDGET;
  CK(cudaFuncSetAttribute(gemv_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, maxb));
  CK(cudaFuncSetAttribute(gemv_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, maxb));
  CK(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_MAX));
  (void)tensor_map_encoder();
  CK(cudaFuncSetAttribute((attn_decode_kernel<true, 0>), cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
  CK(cudaFuncSetAttribute((attn_decode_kernel<false, 0>), cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
  CK(cudaFuncSetAttribute((attn_decode_kernel<true, 64>), cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
  CK(cudaFuncSetAttribute((attn_decode_kernel<false, 64>), cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
  CK(cudaFuncSetAttribute((attn_decode_kernel<true, 128>), cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
  CK(cudaFuncSetAttribute((attn_decode_kernel<false, 128>), cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
  CK(cudaFuncSetAttribute((attn_prefill_kernel<true, 64>), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pfa_smem_bytes(true, 64)));
  CK(cudaFuncSetAttribute((attn_prefill_kernel<true, 128>), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pfa_smem_bytes(true, 128)));
  CK(cudaFuncSetAttribute((attn_prefill_kernel<false, 64>), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pfa_smem_bytes(false, 64)));
  CK(cudaFuncSetAttribute((attn_prefill_kernel<false, 128>), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pfa_smem_bytes(false, 128)));
  CK(cudaFuncSetAttribute((attn_decode_gqa_kernel<true, 64>), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pfa_smem_bytes(true, 64)));
  CK(cudaFuncSetAttribute((attn_decode_gqa_kernel<true, 128>), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pfa_smem_bytes(true, 128)));
  CK(cudaFuncSetAttribute((attn_decode_gqa_kernel<false, 64>), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pfa_smem_bytes(false, 64)));
  CK(cudaFuncSetAttribute((attn_decode_gqa_kernel<false, 128>), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pfa_smem_bytes(false, 128)));
  done[dev] = true;
}

// Prompt attention on the tensor cores handles head sizes 64 and 128; B200_PREFILL_ATTN=0 sends
// prompts through the per-token decode kernel instead.
static bool prefill_attn_available(int hd) {
  static const bool on = [] { const char* v = std::getenv("B200_PREFILL_ATTN"); return !(v && v[0] == '0'); }();
  return on && (hd == 64 || hd == 128);
}

static void launch_prefill_attention(const PrefillAttnParams& a, bool kv_i8, int hd, cudaStream_t st) {
  const dim3 grid((a.T + PFA_Q - 1) / PFA_Q, a.nq);
  const size_t smem = pfa_smem_bytes(kv_i8, hd);
  if (hd == 128) {
    if (kv_i8) attn_prefill_kernel<true, 128><<<grid, PFA_THREADS, smem, st>>>(a);
    else attn_prefill_kernel<false, 128><<<grid, PFA_THREADS, smem, st>>>(a);
  } else if (hd == 64) {
    if (kv_i8) attn_prefill_kernel<true, 64><<<grid, PFA_THREADS, smem, st>>>(a);
    else attn_prefill_kernel<false, 64><<<grid, PFA_THREADS, smem, st>>>(a);
  } else {
    throw std::runtime_error("prompt attention kernel: head_dim must be 64 or 128");
  }
  CK(cudaGetLastError());
}

// Batched decode of grouped-query models: one CTA per (sequence, KV head) on the tensor cores.
// B200_GQA_ATTN=0 keeps the per-head decode kernel, =2 also uses this kernel when every query head
// has its own KV head.
static bool gqa_attn_available(int hd, int nq, int nkv) {
  static const int mode = [] { const char* v = std::getenv("B200_GQA_ATTN"); return v ? atoi(v) : 1; }();
  const int G = nq / nkv;
  return mode != 0 && (hd == 64 || hd == 128) && G <= 8 && (G >= 2 || mode == 2);
}

// Context runs per sequence for the grouped-query batch attention: about 1024 keys per CTA at the
// engine's maximum context (B200_GQA_SPLITS overrides), at most 8.
static int gqa_attn_splits(const b200_engine* e) {
  if (const char* v = std::getenv("B200_GQA_SPLITS")) return std::max(1, std::min(atoi(v), 8));
  return std::max(1, std::min((e->max_ctx + 1023) / 1024, 8));
}

static void launch_gqa_attention(const GqaAttnParams& a, int batch, bool kv_i8, int hd, cudaStream_t st) {
  const dim3 grid(a.nkv, batch, a.nsplit);
  const size_t smem = pfa_smem_bytes(kv_i8, hd);
  if (hd == 128) {
    if (kv_i8) attn_decode_gqa_kernel<true, 128><<<grid, PFA_THREADS, smem, st>>>(a);
    else attn_decode_gqa_kernel<false, 128><<<grid, PFA_THREADS, smem, st>>>(a);
  } else {
    if (kv_i8) attn_decode_gqa_kernel<true, 64><<<grid, PFA_THREADS, smem, st>>>(a);
    else attn_decode_gqa_kernel<false, 64><<<grid, PFA_THREADS, smem, st>>>(a);
  }
  CK(cudaGetLastError());
}

// Device scratch of the loader, grown on demand and reused from tensor to tensor (stream order keeps the reuse safe
// as long as every load-time kernel and copy runs on the same stream).
static uint8_t* stage_scratch(b200_engine* e, int which, size_t bytes) {
  auto& st = e->stage;
  if (st.scratch_cap[which] < bytes) {
    if (st.scratch[which]) {
      CK(cudaDeviceSynchronize());  // earlier tensors may still be reading the old buffer
      CK(cudaFree(st.scratch[which]));
      st.scratch[which] = nullptr;
      st.scratch_cap[which] = 0;
    }
    const size_t cap = std::max(bytes, (size_t)32 << 20);
    CK(cudaMalloc((void**)&st.scratch[which], cap));
    st.scratch_cap[which] = cap;
  }
  return st.scratch[which];
}

// Host (pageable, typically the mmap of the model file) -> device through two pinned buffers: while the copy engine
// moves one chunk, the host fills the other. Replaces the reference's per-tensor host copy + upload
// (weight_management.cpp:873-875).
static void h2d_staged(b200_engine* e, void* dst, const void* src, size_t bytes, cudaStream_t stream) {
  auto& st = e->stage;
  if (!st.pinned[0]) {
    st.chunk = (size_t)64 << 20;
    for (int i = 0; i < 2; ++i) {
      CK(cudaMallocHost((void**)&st.pinned[i], st.chunk));
      CK(cudaEventCreateWithFlags(&st.done[i], cudaEventDisableTiming));
    }
  }
  const uint8_t* s = static_cast<const uint8_t*>(src);
  uint8_t* d = static_cast<uint8_t*>(dst);
  for (size_t off = 0; off < bytes; off += st.chunk) {
    const size_t n = std::min(st.chunk, bytes - off);
    const int b = st.next;
    st.next ^= 1;
    CK(cudaEventSynchronize(st.done[b]));  // the copy that last used this buffer has finished (no-op the first time)
    parallel_memcpy(st.pinned[b], s + off, n);
    CK(cudaMemcpyAsync(d + off, st.pinned[b], n, cudaMemcpyHostToDevice, stream));
    CK(cudaEventRecord(st.done[b], stream));
  }
}

static void stage_release(b200_engine* e) {
  auto& st = e->stage;
  for (int i = 0; i < 2; ++i) {
    if (st.pinned[i]) cudaFreeHost(st.pinned[i]);
    if (st.done[i]) cudaEventDestroy(st.done[i]);
    st.pinned[i] = nullptr; st.done[i] = nullptr;
  }
  for (int i = 0; i < 3; ++i) {
    if (st.scratch[i]) cudaFree(st.scratch[i]);
    st.scratch[i] = nullptr; st.scratch_cap[i] = 0;
  }
}

// Uploads one packed tensor and lays it out on the device as the stage images the matvec kernel
// streams (Q6_K / Q8_0 are first regrouped into aligned 256-element units). half >= 0: the tensor
// is the gate (0) or up (1) projection and shares its image with the other one, every 16-row
// group holding eight gate rows and the same eight up rows.
static void upload_packed(b200_engine* e, DevTensor& t, int type, const void* host, size_t bytes, int64_t rows, int64_t cols,
                          cudaStream_t stream, int half = -1) {
  const int64_t be = type_block_elems(type), bb = type_block_bytes(type);
  if (cols % 256) throw std::runtime_error("tensor columns must be a multiple of 256");
  const size_t nblk = (size_t)(rows * cols / be);
  if (bytes != nblk * (size_t)bb) throw std::runtime_error("tensor byte count does not match rows x cols for its type");
  const GemvGeom g = gemv_geometry(type, (int)cols);
  if ((size_t)g.stage_bytes * 2 + gemv_ring_offset((int)cols, 3) > (size_t)GEMV_SMEM_BUDGET)
    throw std::runtime_error("tensor rows are too long for the matvec kernel's shared memory");
  if (half >= 0) {
    if (rows % 8) throw std::runtime_error("gate/up projections need a multiple of 8 rows");
    if (t.base && (t.type != type || t.rows != rows || t.cols != cols))
      throw std::runtime_error("ffn_gate and ffn_up must have the same shape and block type");
    if (t.halves & (1 << half)) throw std::runtime_error("tensor uploaded twice");
  } else if (t.base) {
    throw std::runtime_error("tensor uploaded twice");
  }
  const int64_t img_rows = half >= 0 ? 2 * rows : rows;
  const int tile_rows = 16 * g.R;
  if (!t.base) {
    t.type = type; t.rows = rows; t.cols = cols; t.bytes = 0; t.img_rows = img_rows;
    t.tiles = (int)((img_rows + tile_rows - 1) / tile_rows);
    const size_t img_bytes = (size_t)t.tiles * g.tile_bytes;
    t.base = dev_alloc<uint8_t>(e, img_bytes + 256);
    CK(cudaMemsetAsync(t.base, 0, img_bytes + 256, stream));
  }
  t.bytes += bytes;
  if (half >= 0) t.halves |= 1 << half;
  uint8_t* raw = stage_scratch(e, 0, bytes + 16);
  h2d_staged(e, raw, host, bytes, stream);
  const size_t n256 = (size_t)(rows * cols / 256);
  const uint8_t* usrc = raw;
  uint16_t* dsrc = nullptr;
  if (type == T_Q6_K || type == T_Q8_0) {
    uint8_t* units = stage_scratch(e, 1, n256 * g.ub + 16);
    const unsigned grid = (unsigned)((bytes + 255) / 256);
    if (type == T_Q6_K) {
      dsrc = reinterpret_cast<uint16_t*>(stage_scratch(e, 2, n256 * 2 + 16));
      split_q6_k_kernel<<<grid, 256, 0, stream>>>(raw, nblk, units, reinterpret_cast<uint8_t*>(dsrc));
    } else {
      regroup_q8_0_kernel<<<grid, 256, 0, stream>>>(raw, nblk, units);
    }
    CK(cudaGetLastError());
    usrc = units;
  }
  stage_image_kernel<<<1184, 256, 0, stream>>>(usrc, dsrc, rows, g, half, t.base);
  CK(cudaGetLastError());
  // no synchronisation here: the scratch buffers are reused by the next tensor on the same stream, in order
}

static GemvSeg seg_of(const DevTensor& t) {
  const GemvGeom g = gemv_geometry(t.type, (int)t.cols);
  GemvSeg s;
  s.img = t.base; s.type = t.type; s.rows = (int)t.img_rows; s.tiles = t.tiles;
  s.RS = g.RS; s.RS_last = g.RS_last; s.d_off = g.d_off; s.d_off_last = g.d_off_last;
  s.stage_bytes = g.stage_bytes; s.stage_bytes_last = g.stage_bytes_last; s.tile_bytes = g.tile_bytes;
  return s;
}

// Fills in the launch geometry (tiles, ring slot size and depth), and starts the kernel with one
// persistent CTA per SM (fewer when there are fewer tiles), as a programmatic dependent launch
// when the engine allows it. Returns the grid width.
static int launch_gemv(const b200_engine* e, GemvParams p, int batch, cudaStream_t st) {
  if (p.K % 256) throw std::runtime_error("gemv: K must be a multiple of 256");
  const GemvGeom g0 = gemv_geometry(p.seg[0].type, p.K);
  p.nblk = g0.nblk; p.nslab = g0.nslab; p.S = g0.S; p.S_last = g0.S_last; p.R = g0.R;
  p.ntiles = 0;
  uint32_t slot = 0;
  for (int s = 0; s < p.nseg; ++s) {
    p.ntiles += p.seg[s].tiles;
    slot = std::max(slot, std::max(p.seg[s].stage_bytes, p.seg[s].stage_bytes_last));
  }
  if (p.epi == EPI_SWIGLU && p.nseg != 1) throw std::runtime_error("gemv: SwiGLU takes the combined gate+up image");
  p.slot_bytes = (slot + 127) / 128 * 128;
  const int gx = std::max(1, std::min(p.ntiles, e->num_sms));
  const size_t ring_off = gemv_ring_offset(p.K, e->P);
  const size_t budget = GEMV_SMEM_BUDGET;
  if (ring_off + 2 * (size_t)p.slot_bytes > budget) throw std::runtime_error("gemv: input dimension too large for shared memory");
  // ring depth: what fits, but no more slots than this CTA will ever fill
  const int stages_per_cta = ((p.ntiles + gx - 1) / gx) * p.nslab;
  const int nstages = std::max(1, (int)std::min<size_t>(std::min(GEMV_MAX_STAGES, stages_per_cta), (budget - ring_off) / p.slot_bytes));
  // bytes the producer requests before the consumers hold their input vector (B200_GEMV_EARLY_KB, default 80)
  static const int early_kb = [] { const char* v = getenv("B200_GEMV_EARLY_KB"); return v && atoi(v) > 0 ? atoi(v) : 80; }();
  p.early_stages = std::max(1, std::min(nstages, (int)((size_t)early_kb * 1024 / p.slot_bytes)));
  p.error_flag = e->d_error;
  const size_t smem = ring_off + (size_t)nstages * p.slot_bytes;
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


// Starts the tensor-core matmul for T tokens (gemm_tc.cuh). x16: [T][K] fp16 activations.
static void encode_map(CUtensorMap* tm, CUtensorMapDataType dt, int rank, const void* base, const cuuint64_t* gdim, const cuuint64_t* gstr,
                       const cuuint32_t* box, CUtensorMapSwizzle swz) {
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult rc = tensor_map_encoder()(tm, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string((int)rc));
}

static void launch_gemm_tc(const b200_engine* e, TcParams p, cudaStream_t st) {
  set_gemv_attrs();
  const GemvGeom g0 = gemv_geometry(p.seg[0].type, p.K);
  p.nblk = g0.nblk; p.nslab = g0.nslab; p.S = g0.S; p.S_last = g0.S_last; p.R = g0.R;
  int ub_max0 = 0;
  for (int s = 0; s < p.nseg; ++s) ub_max0 = std::max(ub_max0, gemv_unit_bytes(p.seg[s].type));
  // token tile: the whole batch when it fits (two MMA halves above 256 tokens: the tile then needs a multiple of 64,
  // and its 64 KB activation stages leave room for one stage of packed units only if those are Q4_K), else tiles of 256
  int NT = (p.T + 31) / 32 * 32;
  if (NT > 256) {
    NT = (p.T + 63) / 64 * 64;
    if (NT > TC_MAX_N) NT = TC_MAX_N;
    if (tc_smem_bytes(NT, 4, 2, 1, (TC_M * ub_max0 + 127) / 128 * 128, p.nslab) > (size_t)TC_SMEM_MAX) NT = 256;
  }
  p.NT = NT;
  p.tmem_cols = 32;
  while (p.tmem_cols < NT) p.tmem_cols *= 2;
  p.ntiles_m = 0;
  int ub_max = 0;
  for (int s = 0; s < p.nseg; ++s) {
    p.ntiles_m += (p.seg[s].rows + TC_M - 1) / TC_M;
    ub_max = std::max(ub_max, gemv_unit_bytes(p.seg[s].type));
  }
  p.error_flag = e->d_error;
  if (p.ksplit < 1) { p.ksplit = 1; p.kblocks = p.K / 256; }
  // shared memory: a weight-tile ring two blocks deep when the token tile is narrow enough, fewer
  // activation stages for the widest token tiles, the rest for the packed-weight ring
  p.w_stage_bytes = (TC_M * ub_max + 127) / 128 * 128;
  static const int a_force = [] { const char* v = std::getenv("B200_TC_A_STAGES"); return v ? atoi(v) : 0; }();
  p.a_stages = NT <= 128 ? 8 : 4;
  if (a_force == 4 || a_force == 8) p.a_stages = a_force;
  p.b_stages = NT > 256 ? 2 : NT > 128 ? 3 : 4;
  auto fits = [&](int w) { return tc_smem_bytes(NT, p.a_stages, p.b_stages, w, p.w_stage_bytes, p.nslab) <= (size_t)TC_SMEM_MAX; };
  if (p.a_stages == 8 && !fits(2)) { p.b_stages = 2; if (!fits(1)) { p.a_stages = 4; p.b_stages = NT > 256 ? 2 : NT > 128 ? 3 : 4; } }
  p.w_stages = TC_W_STAGES;
  while (p.w_stages > 1 && !fits(p.w_stages)) --p.w_stages;
  if (!fits(p.w_stages)) throw std::runtime_error("tensor-core matmul: tile does not fit shared memory");
  static const bool force_rowcopy = [] { const char* v = std::getenv("B200_TC_ROWCOPY"); return v && v[0] == '1'; }();
  const int tr = 16 * p.R;
  p.w_rowcopy = (force_rowcopy || (tr < TC_M ? TC_M % tr : tr % TC_M)) ? 1 : 0;
  TcMaps maps;
  std::memset(&maps, 0, sizeof(maps));
  {  // activation tiles: 64 elements along K x NT tokens, written in the 128-byte-swizzle layout; tokens beyond T read as zero
    const cuuint64_t gdim[2] = {(cuuint64_t)p.K, (cuuint64_t)p.T};
    const cuuint64_t gstr[1] = {(cuuint64_t)p.K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)TC_KC, (cuuint32_t)(NT > 256 ? NT / 2 : NT)};
    encode_map(&maps.act, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p.x16, gdim, gstr, box, CU_TENSOR_MAP_SWIZZLE_128B);
  }
  if (!p.w_rowcopy) {
    // packed units: (32-bit words of a stage row, rows of an image tile, slabs, image tiles); box = one unit x 128 rows
    for (int s = 0; s < p.nseg; ++s) {
      const GemvSeg& sg = p.seg[s];
      const cuuint32_t ub = (cuuint32_t)gemv_unit_bytes(sg.type);
      const cuuint32_t box[4] = {ub / 4, (cuuint32_t)std::min(tr, TC_M), 1, (cuuint32_t)std::max(1, TC_M / tr)};
      for (int last = 0; last < 2; ++last) {
        if (!last && p.nslab == 1) continue;
        const cuuint64_t rs = (cuuint64_t)(last ? sg.RS_last : sg.RS);
        const cuuint64_t gdim[4] = {rs / 4, (cuuint64_t)tr, (cuuint64_t)(last ? 1 : p.nslab - 1), (cuuint64_t)sg.tiles};
        const cuuint64_t gstr[3] = {rs, (cuuint64_t)(last ? sg.stage_bytes_last : sg.stage_bytes), (cuuint64_t)sg.tile_bytes};
        const uint8_t* base = sg.img + (last ? (size_t)(p.nslab - 1) * sg.stage_bytes : 0);
        encode_map(&maps.w[s][last], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, base, gdim, gstr, box, CU_TENSOR_MAP_SWIZZLE_NONE);
      }
    }
  }
  dim3 grid(p.ntiles_m, (p.T + NT - 1) / NT, p.ksplit);
  gemm_tc_kernel<<<grid, TC_THREADS, tc_smem_bytes(NT, p.a_stages, p.b_stages, p.w_stages, p.w_stage_bytes, p.nslab), st>>>(p, maps);
  CK(cudaGetLastError());
}

// B200_ATTN_CLUSTER=1 runs the engine's attention as one thread-block cluster per head
// (attn_cluster.cuh) instead of the ticket kernel; measured slower inside the step graph so far.
static bool attn_use_cluster() {
  static const bool on = [] { const char* v = getenv("B200_ATTN_CLUSTER"); return v && atoi(v) != 0; }();
  return on;
}

// Context splits per (sequence, head): about four CTAs per SM for the ticket kernel; for the
// cluster kernel a power of two up to 8 (the portable cluster size), about two CTAs per SM.
static int attn_nsplit(const b200_engine* e, int batch) {
  if (!attn_use_cluster()) {
    static const int per_sm = [] { const char* v = getenv("B200_ATTN_CTAS_PER_SM"); return v && atoi(v) > 0 ? atoi(v) : 4; }();
    int want = (per_sm * e->num_sms + e->nq * batch - 1) / (e->nq * batch);
    return std::max(1, std::min(want, 32));
  }
  const int want = 2 * e->num_sms / std::max(1, e->nq * batch);
  int cl = 1;
  while (cl * 2 <= want && cl * 2 <= ATTC_MAX_CLUSTER) cl *= 2;
  return cl;
}

// Starts decode attention: the cluster kernel when the split count is 1, 2, 4 or 8 (and the
// ticket kernel is not forced), else the ticket kernel.
static void launch_attention(const AttnParams& a, int batch, bool kv_i8, bool use_pdl, bool force_ticket, cudaStream_t st) {
  const int ns = a.nsplit;
  const bool cluster = !force_ticket && (ns == 1 || ns == 2 || ns == 4 || ns == 8);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(ns, a.nq, batch);
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (use_pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (cluster) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = ns;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
    cfg.blockDim = dim3(ATTC_THREADS);
    cfg.dynamicSmemBytes = attc_smem_floats(a.hd) * sizeof(float);
    cfg.attrs = attr;
    cfg.numAttrs = na;
    if (a.hd == 128) {
      if (kv_i8) CK(cudaLaunchKernelEx(&cfg, attn_cluster_kernel<true, 128>, a));
      else CK(cudaLaunchKernelEx(&cfg, attn_cluster_kernel<false, 128>, a));
    } else if (a.hd == 64) {
      if (kv_i8) CK(cudaLaunchKernelEx(&cfg, attn_cluster_kernel<true, 64>, a));
      else CK(cudaLaunchKernelEx(&cfg, attn_cluster_kernel<false, 64>, a));
    } else {
      if (kv_i8) CK(cudaLaunchKernelEx(&cfg, attn_cluster_kernel<true, 0>, a));
      else CK(cudaLaunchKernelEx(&cfg, attn_cluster_kernel<false, 0>, a));
    }
    return;
  }
  const size_t smem = attn_smem_bytes(a.hd, a.max_ctx, ns, 4);
  if (smem > 160 * 1024) throw std::runtime_error("context too long for the requested split count");
  cfg.blockDim = dim3(ATTN_GROUP_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.attrs = attr;
  cfg.numAttrs = na;
  if (a.hd == 128) {
    if (kv_i8) CK(cudaLaunchKernelEx(&cfg, attn_decode_kernel<true, 128>, a));
    else CK(cudaLaunchKernelEx(&cfg, attn_decode_kernel<false, 128>, a));
  } else if (a.hd == 64) {
    if (kv_i8) CK(cudaLaunchKernelEx(&cfg, attn_decode_kernel<true, 64>, a));
    else CK(cudaLaunchKernelEx(&cfg, attn_decode_kernel<false, 64>, a));
  } else {
    if (kv_i8) CK(cudaLaunchKernelEx(&cfg, attn_decode_kernel<true, 0>, a));
    else CK(cudaLaunchKernelEx(&cfg, attn_decode_kernel<false, 0>, a));
  }
}

// Step-trace record of the launch with this index within the step (nullptr when tracing is off).
static unsigned long long* trace_rec(const b200_engine* e, int launch_index) {
  return e->d_trace && launch_index < e->trace_cap ? e->d_trace + 8 * (size_t)launch_index : nullptr;
}

// Tensor parallel: sum the partial [batch, H] outputs over the ranks, then add them to the residual stream.
static int tp_reduce_add(b200_engine* e, int batch, cudaStream_t st, float* h = nullptr, float* partial = nullptr) {
  Nccl& n = Nccl::get();
  const size_t count = (size_t)batch * e->H;
  if (!h) h = e->d_h;
  if (!partial) partial = e->d_partial;
  n.check(n.AllReduce(partial, partial, count, Nccl::kFloat32, Nccl::kSum, e->nccl_comm, st), "ncclAllReduce");
  add_inplace_kernel<<<(unsigned)std::min<size_t>((count + 255) / 256, 4096), 256, 0, st>>>(h, partial, count);
  CK(cudaGetLastError());
  return 2;
}

// One fused linear layer of the step: the matvec kernel (one launch column per sequence), or, for
// large batches on a single GPU, fp16 conversion (+RMSNorm) followed by the tensor-core matmul.
// Returns the number of launches; *grid_out = partial-argmax parts per sequence (lm_head only).
static int launch_linear(b200_engine* e, GemvParams p, int batch, cudaStream_t st, bool use_tc, int* grid_out = nullptr,
                         void* x16_buf = nullptr) {
  if (!use_tc) {
    const int g = launch_gemv(e, p, batch, st);
    if (grid_out) *grid_out = g;
    return 1;
  }
  __half* x16 = static_cast<__half*>(x16_buf ? x16_buf : e->d_x16);
  to_half_kernel<<<batch, TOH_THREADS, 0, st>>>(p.x, p.x_stride, p.norm_w, p.eps, p.K, x16);
  CK(cudaGetLastError());
  TcParams t{};
  for (int s = 0; s < p.nseg; ++s) t.seg[s] = p.seg[s];
  t.nseg = p.nseg; t.K = p.K; t.x16 = x16; t.T = batch; t.epi = p.epi; t.y = p.y; t.y_stride = p.y_stride; t.y2 = p.y2;
  t.y2_stride = p.y2_stride; t.resid = p.resid; t.rope = p.rope; t.positions = p.positions; t.head_dim = p.head_dim; t.max_pos = p.max_pos;
  int n = 2;
  // Few row tiles (O and down projections: 32 for a 4096-row matrix) leave most SMs idle: split K over
  // up to 8 CTAs per tile, partial outputs summed in order by a small kernel (with the residual).
  const int ctas = (int)((p.seg[0].rows + TC_M - 1) / TC_M) * ((batch + TC_MAX_N - 1) / TC_MAX_N);
  const int nblk = p.K / 256;
  int ks = 1;
  if ((p.epi == EPI_RESID || (p.epi == EPI_STORE && !p.amax_val)) && p.nseg == 1 && batch <= 512 && e->d_tc_part) ks = std::max(1, std::min({8, e->num_sms / std::max(1, ctas), nblk / 4}));
  if (ks > 1) {
    t.ksplit = ks; t.kblocks = (nblk + ks - 1) / ks;
    t.ksplit = (nblk + t.kblocks - 1) / t.kblocks;  // no empty split
    t.epi = EPI_STORE; t.y = e->d_tc_part; t.y_stride = p.seg[0].rows;
    launch_gemm_tc(e, t, st);
    const size_t nel = (size_t)batch * p.seg[0].rows;
    if (p.seg[0].rows % 4 || p.y_stride % 4) throw std::runtime_error("split-K matmul: rows must be a multiple of 4");
    splitk_reduce_kernel<<<(unsigned)std::min<size_t>((nel / 4 + 255) / 256, 1184), 256, 0, st>>>(e->d_tc_part, t.ksplit, batch, p.seg[0].rows, p.resid, p.epi == EPI_RESID ? 1 : 0, p.y,
                                                                                                   p.y_stride);
    CK(cudaGetLastError());
    ++n;
  } else {
    launch_gemm_tc(e, t, st);
  }
  if (p.amax_val) {  // lm_head: the matvec kernel leaves argmax partials; here a small kernel scans the logits
    argmax_rows_kernel<<<batch, 256, 0, st>>>(p.y, p.y_stride, p.amax_row_offset, p.amax_val, p.amax_idx);
    CK(cudaGetLastError());
    if (grid_out) *grid_out = 1;
    ++n;
  }
  return n;
}

// The launch sequence of one decode step for `batch` sequences (also what gets captured).
// Per layer: [RMSNorm + QKV + RoPE] -> [KV append + attention] -> [O proj + residual] ->
// [RMSNorm + gate/up + SwiGLU] -> [down proj + residual]; then [RMSNorm + lm_head + argmax
// partials] and token selection. Returns the number of kernel launches.
static int enqueue_step(b200_engine* e, int batch, int nsplit, cudaStream_t st, bool with_embed, int* head_ctas_out, bool penalized = false) {
  int launches = 0;
  const int H = e->H, F = e->F, KVD = e->KVD;
  const float eps = std::max(e->desc.rms_norm_eps, 1e-5f);  // reference utils.cpp:666-667
  const bool tp = e->tp_size > 1;
  // Tensor parallelism over peer memory (e->use_peer): the O and down projections store their
  // partial rows into every rank's exchange slots (exchange k of the step uses slot set k & 1),
  // and the next matvec adds the tp slots to the residual stream in its prologue and stores the
  // new stream to the other of two buffers. There are 2L exchanges per step, so the stream is back
  // in d_h when the step ends.
  const bool use_tc = batch >= e->gemm_min_batch;  // under tensor parallelism the partial [batch, H] tiles go through ncclAllReduce
  const bool peer = tp && e->use_peer && !use_tc;
  auto slot_of = [&](void* region, int k, int src) {
    return static_cast<uint2*>(region) + ((size_t)(k & 1) * e->tp_size + src) * e->max_seqs * H;
  };
  auto amax_of = [&](void* region) {  // argmax packets of the lm_head launch, behind the exchange slots: [rank][batch][parts]
    return static_cast<uint2*>(region) + (size_t)2 * e->tp_size * e->max_seqs * H;
  };
  float* hcur = e->d_h;
  float* hnext = e->d_h2;
  int pending = -1;  // exchange whose sum the next matvec has to pick up
  auto as_producer = [&](GemvParams& p, int k) {
    p.epi = EPI_PEER; p.tp = e->tp_size; p.tp_rank = e->tp_rank; p.y = nullptr; p.y_stride = H;
    for (int r = 0; r < e->tp_size; ++r) p.peer_y[r] = slot_of(e->peer_region[r], k, e->tp_rank);
    p.epoch_base = e->d_epoch; p.epoch_k = (unsigned)k + 1u;
    pending = k;
  };
  auto as_consumer = [&](GemvParams& p) {
    p.x = hcur;
    if (pending < 0) return;
    p.tp = e->tp_size; p.tp_rank = e->tp_rank;
    p.x_parts = slot_of(e->xregion, pending, 0); p.parts_stride = (size_t)e->max_seqs * H;
    p.epoch_base = e->d_epoch; p.epoch_k = (unsigned)pending + 1u;
    p.x_out = hnext;
    std::swap(hcur, hnext);
    pending = -1;
  };
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
      if (peer) as_consumer(p);
      p.y = e->d_q; p.y_stride = e->Hq; p.y2 = e->d_kvnew; p.y2_stride = 2 * KVD;
      p.rope = e->rope; p.positions = e->d_positions; p.head_dim = e->hd; p.max_pos = e->desc.max_position_embeddings;
      p.trace = trace_rec(e, launches);
      launches += launch_linear(e, p, batch, st, use_tc);
    }
    auto fill_attn = [&](AttnParams& a, int ns) {
      a.q = e->d_q; a.kv_new = e->d_kvnew; a.q_stride = e->Hq; a.kvn_stride = 2 * KVD;
      a.k_cache = w.k_cache; a.v_cache = w.v_cache; a.k_scale = w.k_scale; a.v_scale = w.v_scale;
      a.positions = e->d_positions; a.slots = e->d_slots;
      a.nq = e->nq; a.nkv = e->nkv; a.hd = e->hd; a.max_ctx = e->max_ctx; a.nsplit = ns;
      a.part_o = e->d_part_o; a.part_ml = e->d_part_ml; a.tickets = e->d_tickets;
      a.out = e->d_attn; a.out_stride = e->Hq; a.att_scale = 1.0f / std::sqrt((float)e->hd);
      a.error_flag = e->d_error;
    };
    if (use_tc && gqa_attn_available(e->hd, e->nq, e->nkv)) {
      const bool i8 = e->desc.kv_dtype == B200_KV_I8;
      kv_append_kernel<<<dim3(batch, (e->nkv + KVA_WARPS - 1) / KVA_WARPS, 2), 32 * KVA_WARPS, 0, st>>>(e->d_kvnew, 2 * KVD, e->d_positions, e->d_slots, e->nkv, e->hd, e->max_ctx, i8 ? 1 : 0,
                                                             w.k_cache, w.v_cache, w.k_scale, w.v_scale);
      CK(cudaGetLastError());
      GqaAttnParams a{};
      a.q = e->d_q; a.q_stride = e->Hq;
      a.k_cache = w.k_cache; a.v_cache = w.v_cache; a.k_scale = w.k_scale; a.v_scale = w.v_scale;
      a.positions = e->d_positions; a.slots = e->d_slots;
      a.nq = e->nq; a.nkv = e->nkv; a.max_ctx = e->max_ctx;
      a.out = e->d_attn; a.out_stride = e->Hq; a.att_scale = 1.0f / std::sqrt((float)e->hd);
      a.nsplit = gqa_attn_splits(e); a.part_o = e->d_part_o; a.part_ml = e->d_part_ml; a.tickets = e->d_tickets;
      launch_gqa_attention(a, batch, i8, e->hd, st);
      launches += 2;
    } else {
      AttnParams a{};
      fill_attn(a, nsplit);
      a.trace = trace_rec(e, launches);
      launch_attention(a, batch, e->desc.kv_dtype == B200_KV_I8, e->use_pdl, !attn_use_cluster(), st);
      ++launches;
    }
    {
      GemvParams p{};
      p.seg[0] = seg_of(w.wo); p.nseg = 1; p.K = e->Hq; p.x = e->d_attn; p.x_stride = e->Hq; p.epi = tp ? EPI_STORE : EPI_RESID;
      p.y = tp ? e->d_partial : e->d_h; p.y_stride = H;
      if (peer) as_producer(p, 2 * l);
      p.trace = trace_rec(e, launches);
      launches += launch_linear(e, p, batch, st, use_tc);
      if (tp && !peer) launches += tp_reduce_add(e, batch, st);
    }
    {
      GemvParams p{};
      p.seg[0] = seg_of(w.wgu); p.nseg = 1;
      p.K = H; p.x = e->d_h; p.x_stride = H; p.norm_w = w.ffn_norm.f32(); p.eps = eps; p.epi = EPI_SWIGLU;
      if (peer) as_consumer(p);
      p.y = e->d_act; p.y_stride = F;
      p.trace = trace_rec(e, launches);
      launches += launch_linear(e, p, batch, st, use_tc);
    }
    {
      GemvParams p{};
      p.seg[0] = seg_of(w.wdown); p.nseg = 1; p.K = F; p.x = e->d_act; p.x_stride = F; p.epi = tp ? EPI_STORE : EPI_RESID;
      p.y = tp ? e->d_partial : e->d_h; p.y_stride = H;
      if (peer) as_producer(p, 2 * l + 1);
      p.trace = trace_rec(e, launches);
      launches += launch_linear(e, p, batch, st, use_tc);
      if (tp && !peer) launches += tp_reduce_add(e, batch, st);
    }
  }
  {
    GemvParams p{};
    p.seg[0] = seg_of(e->out_w); p.nseg = 1; p.K = H; p.x = e->d_h; p.x_stride = H;
    p.norm_w = e->out_norm.f32(); p.eps = eps; p.epi = EPI_STORE;
    if (peer) as_consumer(p);
    // each rank computes its share of the vocabulary; shares and argmax partials are then gathered
    const size_t half = (size_t)e->max_seqs * e->amax_cap * e->tp_size;
    p.y = tp ? e->d_logits_local : e->d_logits; p.y_stride = e->Vl;
    p.amax_val = tp ? e->d_amax_val + half : e->d_amax_val; p.amax_idx = tp ? e->d_amax_idx + half : e->d_amax_idx;
    p.amax_row_offset = e->tp_rank * e->Vl;
    // Peer mode: the step graph holds no collective call at all. Every rank's argmax partials travel as packets
    // into every rank's exchange region (the matvec launch uses at most num_sms CTAs: parts_per_rank = its grid),
    // and the logits shares stay local; calls that hand logits to the host gather them after the graph.
    if (penalized) {
      if (use_tc) throw std::runtime_error("the repetition penalty of the device loop is built for the matvec path (batch < " + std::to_string(e->gemm_min_batch) + ")");
      p.pen_counts = e->d_pen_counts; p.pen_stride = e->pen_stride; p.pen_value = e->d_pen_value;
    }
    const int head_grid = std::max(1, std::min(e->out_w.tiles, e->num_sms));
    const unsigned head_epoch_k = 2u * (unsigned)e->L + 1u;
    if (peer) {
      for (int r = 0; r < e->tp_size; ++r) p.amax_peer[r] = amax_of(e->peer_region[r]) + (size_t)e->tp_rank * batch * head_grid;
      p.tp = e->tp_size; p.tp_rank = e->tp_rank;
      p.epoch_base = e->d_epoch;
      p.amax_epoch_k = head_epoch_k;
    }
    p.trace = trace_rec(e, launches);
    int grid = 0;
    launches += launch_linear(e, p, batch, st, use_tc, &grid);
    if (tp && !peer) {
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
    if (penalized) { s.pen_ring = e->d_pen_ring; s.pen_count = e->d_pen_count; s.pen_counts = e->d_pen_counts; s.pen_stride = e->pen_stride; }
    if (peer) {  // the next step's packets carry new numbers
      s.epoch = e->d_epoch; s.epoch_inc = 2u * (unsigned)e->L + 2u;
      s.amax_pkts = amax_of(e->xregion); s.epoch_k = head_epoch_k; s.error_flag = e->d_error;
    }
    select_kernel<<<1, 256, 0, st>>>(s);
    CK(cudaGetLastError());
    ++launches;
  }
  return launches;
}

// ---- prompt ingestion on the tensor cores -------------------------------------------------------
// forward_device_batch_prefill (reference model.cpp:1526-1862) / CPUBatchProcessor::forward_cpu_batch
// (cpu_batch_processor.cpp:11-281): all tokens of a chunk go through every layer together. Linear
// layers = fp16 conversion (+RMSNorm, batch form: eps as configured) + tcgen05 matmul; the chunk's
// K/V rows are appended to the cache first, then the prompt-attention kernel (64 queries per CTA on
// the fp16 tensor cores; head sizes other than 64 / 128: the decode-attention kernel per token) runs
// over the cache rows up to and including each token's own position (causal). Only the last token's logits are
// computed (the reference computes all rows and keeps the last, model.cpp:1094-1156).
constexpr int PF_CHUNK = 512;

static void ensure_prefill_buffers(b200_engine* e) {
  if (e->pf_cap) return;
  const int T = PF_CHUNK;
  e->pf_ints = dev_alloc<int>(e, (size_t)3 * T);
  e->pf_h = dev_alloc<float>(e, (size_t)T * e->H);
  e->pf_q = dev_alloc<float>(e, (size_t)T * e->H);
  e->pf_kvnew = dev_alloc<float>(e, (size_t)T * 2 * e->KVD);
  e->pf_attn = dev_alloc<float>(e, (size_t)T * e->H);
  e->pf_act = dev_alloc<float>(e, (size_t)T * e->F);
  e->pf_x16 = dev_alloc<uint16_t>(e, (size_t)T * std::max(e->H, e->F));
  if (e->tp_size > 1) e->pf_partial = dev_alloc<float>(e, (size_t)T * e->H);
  size_t items = 0;
  for (int t = 1; t <= T; ++t) items = std::max(items, (size_t)t * e->nq * attn_nsplit(e, t));
  e->pf_part_o = dev_alloc<float>(e, items * e->hd);
  e->pf_part_ml = dev_alloc<float>(e, items * 2);
  e->pf_tickets = dev_alloc<int>(e, (size_t)T * e->nq);
  CK(cudaMemset(e->pf_tickets, 0, (size_t)T * e->nq * 4));
  e->pf_cap = T;
}

// A run of consecutive tokens of one sequence inside a chunk: rows [row0, row0 + len) of the chunk's buffers hold the
// tokens at positions start .. start+len-1 of KV slot `slot`. logits_to >= 0: this run ends its sequence's prompt,
// and the logits of its last token go to row logits_to of the caller's host buffer.
struct PrefillRun {
  int row0, len, slot, start, logits_to;
};

// One chunk of T <= PF_CHUNK prompt tokens, possibly of several sequences (sequence-aware: every token carries its
// own position and KV slot through the RoPE epilogue and the cache append, and attention runs per run of tokens,
// each over its own sequence's cache rows; reference api.cpp:1144-1421 / cpu_attention.cpp:203-325).
// meta = token ids | positions | slots, T each. After the layers, the logits of the last token of every run with
// logits_to >= 0 are computed and copied to host_logits + logits_to * V (nullptr: left in e->d_logits only).
static void prefill_chunk(b200_engine* e, int T, const std::vector<int>& meta, const std::vector<PrefillRun>& runs, float* host_logits) {
  ensure_prefill_buffers(e);
  cudaStream_t st = e->stream;
  const int H = e->H, F = e->F, KVD = e->KVD;
  const bool tp = e->tp_size > 1;
  CK(cudaMemcpyAsync(e->pf_ints, meta.data(), meta.size() * 4, cudaMemcpyHostToDevice, st));
  CK(cudaStreamSynchronize(st));  // meta may not outlive this call
  const int* d_tok = e->pf_ints;
  const int* d_pos = e->pf_ints + T;
  const int* d_slot = e->pf_ints + 2 * T;
  const float eps = e->desc.rms_norm_eps;  // rmsnorm_batch_cpu form (utils.cpp:613-646)
  const bool i8 = e->desc.kv_dtype == B200_KV_I8;
  embed_kernel<<<T, 256, 0, st>>>(d_tok, e->tok_embd.f32(), e->pf_h, H, e->V);
  CK(cudaGetLastError());
  const int nsplit = attn_use_cluster() ? 1 : attn_nsplit(e, T);
  for (int l = 0; l < e->L; ++l) {
    const LayerW& w = e->layers[l];
    {
      GemvParams p{};
      p.seg[0] = seg_of(w.wq); p.seg[1] = seg_of(w.wk); p.seg[2] = seg_of(w.wv); p.nseg = 3;
      p.K = H; p.x = e->pf_h; p.x_stride = H; p.norm_w = w.attn_norm.f32(); p.eps = eps; p.epi = EPI_QKV_ROPE;
      p.y = e->pf_q; p.y_stride = e->Hq; p.y2 = e->pf_kvnew; p.y2_stride = 2 * KVD;
      p.rope = e->rope; p.positions = d_pos; p.head_dim = e->hd; p.max_pos = e->desc.max_position_embeddings;
      launch_linear(e, p, T, st, true, nullptr, e->pf_x16);
    }
    kv_append_kernel<<<dim3(T, (e->nkv + KVA_WARPS - 1) / KVA_WARPS, 2), 32 * KVA_WARPS, 0, st>>>(e->pf_kvnew, 2 * KVD, d_pos, d_slot, e->nkv, e->hd, e->max_ctx, i8 ? 1 : 0, w.k_cache,
                                                        w.v_cache, w.k_scale, w.v_scale);
    CK(cudaGetLastError());
    if (prefill_attn_available(e->hd)) {
      for (const PrefillRun& r : runs) {
        PrefillAttnParams a{};
        a.q = e->pf_q + (size_t)r.row0 * e->Hq; a.q_stride = e->Hq;
        a.k_cache = w.k_cache; a.v_cache = w.v_cache; a.k_scale = w.k_scale; a.v_scale = w.v_scale;
        a.slot = r.slot; a.start = r.start; a.T = r.len; a.nq = e->nq; a.nkv = e->nkv; a.max_ctx = e->max_ctx;
        a.out = e->pf_attn + (size_t)r.row0 * e->Hq; a.out_stride = e->Hq; a.att_scale = 1.0f / std::sqrt((float)e->hd);
        launch_prefill_attention(a, i8, e->hd, st);
      }
    } else {
      AttnParams a{};
      a.q = e->pf_q; a.kv_new = e->pf_kvnew; a.q_stride = e->Hq; a.kvn_stride = 2 * KVD;
      a.k_cache = w.k_cache; a.v_cache = w.v_cache; a.k_scale = w.k_scale; a.v_scale = w.v_scale;
      a.positions = d_pos; a.slots = d_slot;
      a.nq = e->nq; a.nkv = e->nkv; a.hd = e->hd; a.max_ctx = e->max_ctx; a.nsplit = nsplit;
      a.part_o = e->pf_part_o; a.part_ml = e->pf_part_ml; a.tickets = e->pf_tickets;
      a.out = e->pf_attn; a.out_stride = e->Hq; a.att_scale = 1.0f / std::sqrt((float)e->hd);
      a.cached_new = 1;
      launch_attention(a, T, i8, false, true, st);
    }
    {
      GemvParams p{};
      p.seg[0] = seg_of(w.wo); p.nseg = 1; p.K = e->Hq; p.x = e->pf_attn; p.x_stride = e->Hq; p.epi = tp ? EPI_STORE : EPI_RESID;
      p.y = tp ? e->pf_partial : e->pf_h; p.y_stride = H;
      launch_linear(e, p, T, st, true, nullptr, e->pf_x16);
      if (tp) tp_reduce_add(e, T, st, e->pf_h, e->pf_partial);
    }
    {
      GemvParams p{};
      p.seg[0] = seg_of(w.wgu); p.nseg = 1;
      p.K = H; p.x = e->pf_h; p.x_stride = H; p.norm_w = w.ffn_norm.f32(); p.eps = eps; p.epi = EPI_SWIGLU;
      p.y = e->pf_act; p.y_stride = F;
      launch_linear(e, p, T, st, true, nullptr, e->pf_x16);
    }
    {
      GemvParams p{};
      p.seg[0] = seg_of(w.wdown); p.nseg = 1; p.K = F; p.x = e->pf_act; p.x_stride = F; p.epi = tp ? EPI_STORE : EPI_RESID;
      p.y = tp ? e->pf_partial : e->pf_h; p.y_stride = H;
      launch_linear(e, p, T, st, true, nullptr, e->pf_x16);
      if (tp) tp_reduce_add(e, T, st, e->pf_h, e->pf_partial);
    }
  }
  for (const PrefillRun& r : runs) {  // final norm + lm_head for the last token of a prompt only, on the matvec kernel
    if (r.logits_to < 0) continue;
    GemvParams p{};
    p.seg[0] = seg_of(e->out_w); p.nseg = 1; p.K = H; p.x = e->pf_h + (size_t)(r.row0 + r.len - 1) * H; p.x_stride = H;
    p.norm_w = e->out_norm.f32(); p.eps = eps; p.epi = EPI_STORE; p.y = tp ? e->d_logits_local : e->d_logits; p.y_stride = e->Vl;
    launch_gemv(e, p, 1, st);
    if (tp) {  // every rank holds its share of the vocabulary: gather the shares (in rank order = vocabulary order for one row)
      Nccl& n = Nccl::get();
      n.check(n.AllGather(e->d_logits_local, e->d_logits, (size_t)e->Vl, Nccl::kFloat32, e->nccl_comm, st), "ncclAllGather");
    }
    if (host_logits) CK(cudaMemcpyAsync(host_logits + (size_t)r.logits_to * e->V, e->d_logits, (size_t)e->V * 4, cudaMemcpyDeviceToHost, st));
  }
}

// Prompt ingestion of one or several sequences through the tensor-core path: the tokens of all sequences are laid
// end to end and cut into chunks of PF_CHUNK, so that short prompts share a chunk (and its weight traffic).
// host_logits: [n_seqs][V] or nullptr.
// The chunk plan of a sequence-aware ingestion: the prompts laid end to end and cut every `chunk` tokens. Each run is
// a stretch of one sequence inside one chunk; runs are returned in order, `chunk_of[i]` = the chunk run i belongs to.
// Pure host arithmetic (exposed through b200_prefill_plan so that it can be checked without a GPU).
static void plan_prefill_runs(int n_seqs, const int32_t* slots, const int32_t* lens, const int32_t* start_pos, int chunk,
                              std::vector<PrefillRun>& runs, std::vector<int>& chunk_of) {
  int T = 0, c = 0;
  for (int s = 0; s < n_seqs; ++s) {
    int done = 0;
    while (done < lens[s]) {
      const int take = std::min(lens[s] - done, chunk - T);
      runs.push_back({T, take, slots ? slots[s] : s, (start_pos ? start_pos[s] : 0) + done, done + take == lens[s] ? s : -1});
      chunk_of.push_back(c);
      T += take;
      done += take;
      if (T == chunk) { T = 0; ++c; }
    }
  }
}

static void prefill_sequences(b200_engine* e, int n_seqs, const int32_t* slots, const int32_t* ids, const int32_t* lens, const int32_t* start_pos,
                              float* host_logits) {
  std::vector<PrefillRun> all;
  std::vector<int> chunk_of;
  plan_prefill_runs(n_seqs, slots, lens, start_pos, PF_CHUNK, all, chunk_of);
  std::vector<size_t> seq_off(n_seqs + 1, 0);
  for (int s = 0; s < n_seqs; ++s) seq_off[s + 1] = seq_off[s] + (size_t)lens[s];
  // which sequence a run belongs to: runs come in sequence order, a new sequence starts when the previous one's last run ended
  size_t i = 0;
  int seq = 0, done = 0;
  while (i < all.size()) {
    const int c = chunk_of[i];
    std::vector<PrefillRun> runs;
    std::vector<int> tok, pos, slot;
    for (; i < all.size() && chunk_of[i] == c; ++i) {
      const PrefillRun& r = all[i];
      runs.push_back(r);
      for (int t = 0; t < r.len; ++t) {
        tok.push_back(ids[seq_off[seq] + done + t]);
        pos.push_back(r.start + t);
        slot.push_back(r.slot);
      }
      done += r.len;
      if (done == lens[seq]) { ++seq; done = 0; }
    }
    const int T = (int)tok.size();
    std::vector<int> meta;
    meta.reserve((size_t)3 * T);
    meta.insert(meta.end(), tok.begin(), tok.end());
    meta.insert(meta.end(), pos.begin(), pos.end());
    meta.insert(meta.end(), slot.begin(), slot.end());
    prefill_chunk(e, T, meta, runs, host_logits);
  }
}

static StepGraph& get_graph(b200_engine* e, int batch, bool with_embed = true, bool penalized = false) {
  const int key = batch * 4 + (with_embed ? 1 : 0) + (penalized ? 2 : 0);
  auto it = e->graphs.find(key);
  if (it != e->graphs.end()) return it->second;
  StepGraph g;
  g.nsplit = attn_nsplit(e, batch);
  cudaGraph_t graph = nullptr;
  CK(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
  try {
    g.launches = enqueue_step(e, batch, g.nsplit, e->stream, with_embed, &g.head_ctas, penalized);
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
