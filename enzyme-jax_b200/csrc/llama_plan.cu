// Host side of the llama path: error plumbing, plan creation, packed weight
// layout, and the forward kernel sequence (test/llama.py:35-238 of the
// reference, applied to whole sequences).
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "attention.cuh"
#include "elementwise.cuh"
#include "gemm_epilogue.cuh"
#include "plan.cuh"

namespace b200 {

// ---- errors -------------------------------------------------------------------
static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int32_t fail(int32_t code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return (v && *v) ? atoi(v) : dflt;
}

bool pdl_enabled() {
  static const bool on = env_int("B200_PDL", 1) != 0;
  return on;
}

// ---- launch counter and event profiler -----------------------------------------
static std::atomic<long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

struct ProfSample { cudaEvent_t a, b; int cls; double work; };
static std::mutex g_prof_mu;
static std::vector<ProfSample> g_prof;
static size_t g_prof_used = 0;
static std::atomic<int> g_prof_on{0};

ProfScope::ProfScope(int cls, double work, cudaStream_t s) : stream(s) {
  if (!g_prof_on.load(std::memory_order_relaxed)) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (g_prof_used == g_prof.size()) {
    ProfSample ps;
    if (cudaEventCreate(&ps.a) != cudaSuccess || cudaEventCreate(&ps.b) != cudaSuccess) return;
    g_prof.push_back(ps);
  }
  slot = (int)g_prof_used++;
  g_prof[slot].cls = cls;
  g_prof[slot].work = work;
  cudaEventRecord(g_prof[slot].a, stream);
}
ProfScope::~ProfScope() {
  if (slot < 0) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  cudaEventRecord(g_prof[slot].b, stream);
}

// ---- per-device state ---------------------------------------------------------
static std::mutex g_mu;
static uint32_t* g_status[64] = {nullptr};
static int g_sms[64] = {0};

uint32_t* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status[dev]) {
    uint32_t* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    g_status[dev] = p;
  }
  return g_status[dev];
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!g_sms[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sms[dev] = n;
  }
  return g_sms[dev];
}

// ---- layouts --------------------------------------------------------------------
void build_layout(const B200Plan& p, size_t es, bool with_t, PackedLayout* out) {
  Arena a(nullptr);
  auto take = [&](size_t bytes) { size_t off = a.used; a.take(bytes); return off; };
  out->layer.assign(p.L, LayerOffsets{});
  out->g_att = take((size_t)p.L * p.d * 4);
  out->g_ffn = take((size_t)p.L * p.d * 4);
  out->g_final = take((size_t)p.d * 4);
  out->emb = take((size_t)p.V * p.d * es);
  for (int l = 0; l < p.L; ++l) {
    LayerOffsets& o = out->layer[l];
    o.wqkv = take((size_t)3 * p.d_loc * p.d * es);
    o.wo = take((size_t)p.d * p.d_loc * es);
    o.w13 = take((size_t)2 * p.h_loc * p.d * es);
    o.w2 = take((size_t)p.d * p.h_loc * es);
  }
  out->wcls = take((size_t)p.V_loc * p.d * es);
  if (with_t) {
    for (int l = 0; l < p.L; ++l) {
      LayerOffsets& o = out->layer[l];
      o.wqkv_t = take((size_t)3 * p.d_loc * p.d * es);
      o.wo_t = take((size_t)p.d * p.d_loc * es);
      o.w13_t = take((size_t)2 * p.h_loc * p.d * es);
      o.w2_t = take((size_t)p.d * p.h_loc * es);
    }
    out->wcls_t = take((size_t)p.V_loc * p.d * es);
  }
  out->total = a.used;
}

void carve_forward(const B200Plan& p, Arena& a, int B, int S, bool keep, FwdActs* out) {
  const size_t T = (size_t)B * S, es = p.esize;
  out->layer.assign(p.L, LayerActs{});
  auto carve_one = [&](LayerActs& la, float* x_in) {
    la.x_in = x_in ? x_in : a.take<float>(T * p.d * 4);
    la.xb = a.take(T * p.d * es);
    la.rinv1 = a.take<float>(T * 4);
    la.qkv = a.take(T * 3 * p.d_loc * es);
    la.o = a.take(T * p.d_loc * es);
    la.lse = a.take<float>((size_t)B * p.H_loc * S * 4);
    la.xb2 = a.take(T * p.d * es);
    la.rinv2 = a.take<float>(T * 4);
    la.hg = a.take(T * p.h_loc * es);
  };
  if (!keep) {
    LayerActs la;
    carve_one(la, nullptr);
    la.x_mid = la.x_in;
    la.x_out = la.x_in;
    la.xb2 = la.xb;  // the two normed buffers are never live together
    for (int l = 0; l < p.L; ++l) out->layer[l] = la;
    out->fin.x_last = la.x_in;
    out->fin.rinv_f = la.rinv1;
    out->fin.xf = la.xb;
    return;
  }
  float* x_next = nullptr;
  for (int l = 0; l < p.L; ++l) {
    LayerActs& la = out->layer[l];
    carve_one(la, x_next);
    la.x_mid = a.take<float>(T * p.d * 4);
    la.gate = a.take(T * p.h_loc * es);
    la.up = a.take(T * p.h_loc * es);
    la.x_out = a.take<float>(T * p.d * 4);
    x_next = la.x_out;
  }
  out->fin.x_last = x_next;
  out->fin.rinv_f = a.take<float>(T * 4);
  out->fin.xf = a.take(T * p.d * es);
}

// ---- forward ---------------------------------------------------------------------
static int32_t gemm(const B200Plan& p, const void* A, int lda, const void* B, int ldb, int M, int N, int K, int kind,
                    int out_dtype, const EpiParams& epi, cudaStream_t stream, const PeerBands* bands = nullptr) {
  GemmArgs g;
  g.A = A; g.B = B; g.M = M; g.N = N; g.K = K; g.lda = lda; g.ldb = ldb;
  g.in_dtype = p.dtype; g.out_dtype = out_dtype; g.kind = kind; g.epi = epi;
  if (bands && bands->flags) {  // A arrives band by band from the other ranks: the kernel waits for each band itself
    g.band_flags = bands->flags; g.band_epoch = bands->epoch; g.band_rows = bands->rows; g.band_first = bands->first;
    g.band_budget = bands->budget;
  }
  return launch_gemm(g, p.gemm_impl, stream);
}

// Row-parallel projection followed by the residual add: fused when the model is
// on one GPU; with tensor parallelism the partial products are summed over the
// ranks first (one all-reduce per block) and then added.
static int32_t proj_residual(const B200Plan& p, const void* A, int lda, const void* W, int ldw, int T, int K,
                             const float* x_in, float* x_out, void* tp_tmp, cudaStream_t stream) {
  EpiParams e;
  if (p.tp_size == 1) {
    e.out = x_out; e.ldo = p.d; e.resid_in = x_in;
    return gemm(p, A, lda, W, ldw, T, p.d, K, EPI_RESID, B200_F32, e, stream);
  }
  // Peer-memory path: the partial product goes straight into the buffer the other ranks map; two kernels
  // reduce it over NVLink and add the sum to the residual stream.
  if (void* pbuf = comm_peer_buffer(p.comm, (size_t)T * p.d * p.esize)) {
    e.out = pbuf; e.ldo = p.d;
    B200_TRY(gemm(p, A, lda, W, ldw, T, p.d, K, EPI_STORE, p.dtype, e, stream));
    return comm_peer_allreduce_add(p.comm, (size_t)T * p.d, p.dtype, x_in, x_out, stream);
  }
  // Token chunks: the projection of chunk c+1 computes while chunk c is summed over the ranks on the
  // communication stream (NCCL over NVLink); the compute stream joins all chunks before the add.
  int chunks = (T >= 512 * p.tp_chunks && T % (128 * p.tp_chunks) == 0) ? p.tp_chunks : 1;
  const int rows = T / chunks;
  const size_t es = p.esize;
  for (int c = 0; c < chunks; ++c) {
    GemmArgs g;
    g.A = reinterpret_cast<const uint8_t*>(A) + (size_t)c * rows * lda * es;
    g.B = W; g.M = rows; g.N = p.d; g.K = K; g.lda = lda; g.ldb = ldw;
    g.in_dtype = p.dtype; g.out_dtype = p.dtype; g.kind = EPI_STORE;
    g.epi.out = reinterpret_cast<uint8_t*>(tp_tmp) + (size_t)c * rows * p.d * es;
    g.epi.ldo = p.d;
    if (chunks > 1) g.max_ctas = sm_count() - p.reserve_sms;
    B200_TRY(launch_gemm(g, p.gemm_impl, stream));
    if (chunks == 1) {
      B200_TRY(comm_allreduce(p.comm, tp_tmp, (size_t)T * p.d, p.dtype, stream));
    } else {
      B200_CUDA_OK(cudaEventRecord(p.ev_fork[c], stream));
      B200_CUDA_OK(cudaStreamWaitEvent(p.comm_stream, p.ev_fork[c], 0));
      B200_TRY(comm_allreduce(p.comm, g.epi.out, (size_t)rows * p.d, p.dtype, p.comm_stream));
      B200_CUDA_OK(cudaEventRecord(p.ev_join[c], p.comm_stream));
    }
  }
  if (chunks > 1)
    for (int c = 0; c < chunks; ++c) B200_CUDA_OK(cudaStreamWaitEvent(stream, p.ev_join[c], 0));
  if (x_out != x_in)
    B200_CUDA_OK(cudaMemcpyAsync(x_out, x_in, (size_t)T * p.d * 4, cudaMemcpyDeviceToDevice, stream));
  return launch_add_to_f32(x_out, tp_tmp, p.dtype, (size_t)T * p.d, stream);
}

// Tensor-parallel forward with a row-sharded residual stream (peer memory up, T a multiple of the ranks).  This rank
// keeps the fp32 residual rows [rank * T/tp, (rank + 1) * T/tp) only.  The row-parallel projections (Wo, W2) leave
// their bf16 partial product, all T rows, in the exchange buffer; comm_peer_reduce_norm then sums every own row over
// the ranks, adds it to the residual row, norms it and deposits the normed row with every rank, so that the next
// column-parallel projection (QKV, W1|W3, logits) finds all T normed rows in local memory.  Per block: one kernel
// and one crossing of NVLink in each direction instead of all-reduce + add + norm over all T rows.
static int32_t forward_row_sharded(B200Plan* p, const int32_t* tokens, int B, int S, const uint8_t* w,
                                   const PackedLayout& wl, float* logits, void* kv_out, const LayerActs& a,
                                   void* part, void* xbg, cudaStream_t stream) {
  const int T = B * S, d = p->d, dl = p->d_loc, hl = p->h_loc;
  const int rows = T / p->tp_size, row0 = p->tp_rank * rows;
  const float* g_att = reinterpret_cast<const float*>(w + wl.g_att);
  const float* g_ffn = reinterpret_cast<const float*>(w + wl.g_ffn);
  const float* g_fin = reinterpret_cast<const float*>(w + wl.g_final);
  const float eps = p->cfg.rms_eps;
  float* x_own = a.x_in;  // [T, d] in the workspace; the first T/tp rows hold this rank's residual rows
  // Pushed partial products: the Wo / W2 GEMMs store every row band straight into the memory of the rank that owns
  // it (slot = this rank), tile by tile while they compute, so the reduce-scatter half of the exchange crosses NVLink
  // under the GEMM and the exchange kernel sums from local memory.  Needs the CTA-pair kernel for both shapes.
  void* push_base[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  bool push = p->tp_push && comm_peer_push_bases(p->comm, T, d, p->dtype, push_base);
  auto proj_args = [&](const void* A, int lda, const void* W, int ldw, int K) {
    GemmArgs g;
    g.A = A; g.B = W; g.M = T; g.N = d; g.K = K; g.lda = lda; g.ldb = ldw;
    g.in_dtype = p->dtype; g.out_dtype = p->dtype; g.kind = EPI_STORE;
    g.epi.out = part; g.epi.ldo = d;
    return g;
  };
  if (push) {
    for (int which = 0; which < 2 && push; ++which) {
      GemmArgs g = which ? proj_args(a.hg, hl, w, hl, hl) : proj_args(a.o, dl, w, dl, dl);
      g.push_rows = rows;
      push = gemm_push_supported(g, p->gemm_impl);
    }
  }
  p->tp_push_last = push ? 1 : 0;
  // Gathered rows consumed band by band: the exchange kernel returns once this rank's rows are delivered, and the
  // column-parallel GEMM that follows starts on the band that is already here and waits for every other band just
  // before it first loads rows of it, so the all-gather half of the exchange crosses NVLink under that GEMM.  Needs
  // the CTA-pair kernel for all three consumers.
  bool bands = p->tp_bands && rows % 256 == 0;
  if (bands) {
    const int ns[3] = {3 * dl, 2 * hl, p->V_loc};
    const int kinds[3] = {EPI_ROPE, EPI_SWIGLU, EPI_STORE};
    for (int i = 0; i < (logits ? 3 : 2) && bands; ++i) {
      GemmArgs g;
      g.A = xbg; g.B = w; g.M = T; g.N = ns[i]; g.K = d; g.lda = d; g.ldb = d;
      g.in_dtype = p->dtype; g.out_dtype = i == 2 ? B200_F32 : p->dtype; g.kind = kinds[i];
      g.epi.out = i == 0 ? a.qkv : i == 1 ? a.hg : (void*)logits;
      g.epi.ldo = i == 1 ? hl : ns[i];
      if (i == 0) { g.epi.rope_cos = p->rope_cos; g.epi.rope_sin = p->rope_sin; g.epi.head_size = p->hs; }
      g.band_rows = rows;
      bands = gemm_bands_supported(g, p->gemm_impl);
    }
  }
  p->tp_bands_last = bands ? 1 : 0;
  PeerBands pb;
  auto row_parallel = [&](const void* A, int lda, const void* W, int ldw, int K) -> int32_t {
    GemmArgs g = proj_args(A, lda, W, ldw, K);
    if (push) {
      g.push_rows = rows;
      for (int o = 0; o < p->tp_size; ++o) g.push_base[o] = push_base[o];
    }
    return launch_gemm(g, p->gemm_impl, stream);
  };
  B200_TRY(launch_embed(tokens + row0, w + wl.emb, p->dtype, x_own, rows, d, p->V, stream));
  B200_TRY(comm_peer_reduce_norm(p->comm, T, d, p->dtype, false, x_own, g_att, eps, stream, false, bands ? &pb : nullptr));
  for (int l = 0; l < p->L; ++l) {
    const LayerOffsets& o = wl.layer[l];
    {
      EpiParams e;
      e.out = a.qkv; e.ldo = 3 * dl;
      e.rope_cos = p->rope_cos; e.rope_sin = p->rope_sin;
      e.seq_len = S; e.pos_base = 0; e.head_size = p->hs; e.rope_cols = 2 * dl;
      B200_TRY(gemm(*p, xbg, d, w + o.wqkv, d, T, 3 * dl, d, EPI_ROPE, p->dtype, e, stream, &pb));
    }
    if (kv_out) {
      uint8_t* dst = reinterpret_cast<uint8_t*>(kv_out) + (size_t)l * 2 * T * dl * p->esize;
      const uint8_t* src = reinterpret_cast<const uint8_t*>(a.qkv);
      for (int part_i = 0; part_i < 2; ++part_i)
        B200_CUDA_OK(cudaMemcpy2DAsync(dst + (size_t)part_i * T * dl * p->esize, (size_t)dl * p->esize,
                                       src + (size_t)(1 + part_i) * dl * p->esize, (size_t)3 * dl * p->esize,
                                       (size_t)dl * p->esize, T, cudaMemcpyDeviceToDevice, stream));
    }
    {
      AttnArgs at;
      const uint8_t* base = reinterpret_cast<const uint8_t*>(a.qkv);
      at.q = base; at.k = base + (size_t)dl * p->esize; at.v = base + (size_t)2 * dl * p->esize;
      at.o = a.o; at.lse = a.lse;
      at.batch = B; at.seq = S; at.n_heads = p->H_loc; at.head_size = p->hs;
      at.ldq = 3 * dl; at.ldkv = 3 * dl; at.ldo = dl; at.dtype = p->dtype;
      B200_TRY(launch_attn_fwd(at, p->attn_impl, stream));
    }
    B200_TRY(row_parallel(a.o, dl, w + o.wo, dl, dl));
    B200_TRY(comm_peer_reduce_norm(p->comm, T, d, p->dtype, true, x_own, g_ffn + (size_t)l * d, eps, stream, push,
                                   bands ? &pb : nullptr));
    {
      EpiParams e;
      e.out = a.hg; e.ldo = hl;
      B200_TRY(gemm(*p, xbg, d, w + o.w13, d, T, 2 * hl, d, EPI_SWIGLU, p->dtype, e, stream, &pb));
    }
    B200_TRY(row_parallel(a.hg, hl, w + o.w2, hl, hl));
    const float* g_next = l + 1 < p->L ? g_att + (size_t)(l + 1) * d : g_fin;
    // the last exchange has a consumer only when logits are asked for; without one it waits for the peers itself
    const bool last = l + 1 == p->L;
    B200_TRY(comm_peer_reduce_norm(p->comm, T, d, p->dtype, true, x_own, g_next, eps, stream, push,
                                   bands && (!last || logits) ? &pb : nullptr));
    if (last && !logits) pb = PeerBands{};
  }
  if (logits) {
    EpiParams e;
    e.out = logits; e.ldo = p->V_loc;
    B200_TRY(gemm(*p, xbg, d, w + wl.wcls, d, T, p->V_loc, d, EPI_STORE, B200_F32, e, stream, &pb));
  }
  return B200_OK;
}

// The row-sharded forward over TWO halves of the batch whose exchanges overlap the other half's compute.  Half h
// holds the sequences [h B/2, (h+1) B/2); each half has its own partial-product and gathered-activation regions and
// its own T/(2 tp) residual rows per rank.  Compute kernels run on the caller's stream, the exchange kernels - in one
// fixed order on every rank, which is what their flag protocol needs - on the plan's communication stream in their
// lean form (one small CTA per SM, which fits beside a GEMM or attention CTA):
//   compute:  QKV_0 ATT_0 WO_0 | QKV_1 ATT_1 WO_1 | W13_0 W2_0 | W13_1 W2_1 | next layer ...
//   exchange:              EX1_0 ............ EX1_1 ....... EX2_0 ....... EX2_1 ...
// so every exchange crosses NVLink while the tensor cores work on the other half.  Events order the two streams:
// part_ready[h] (a projection left its partial product) and xb_ready[h] (the gathered rows of half h are whole).
static int32_t forward_row_sharded_pipelined(B200Plan* p, const int32_t* tokens, int B, int S, const uint8_t* w,
                                             const PackedLayout& wl, float* logits, void* kv_out, const LayerActs& a,
                                             void* part, void* xbg, cudaStream_t stream) {
  const int Bh = B / 2, Th = Bh * S, T = B * S, d = p->d, dl = p->d_loc, hl = p->h_loc;
  const int rows = Th / p->tp_size, row0 = p->tp_rank * rows;
  const size_t es = p->esize;
  const float* g_att = reinterpret_cast<const float*>(w + wl.g_att);
  const float* g_ffn = reinterpret_cast<const float*>(w + wl.g_ffn);
  const float* g_fin = reinterpret_cast<const float*>(w + wl.g_final);
  const float eps = p->cfg.rms_eps;
  cudaStream_t cs = p->comm_stream;
  const size_t half_bytes = align_up((size_t)Th * d * es, 256);
  const size_t each = align_up((size_t)T * d * es, 256);  // the gathered area starts where it does for the whole batch
  auto part_rel = [&](int h) { return (size_t)h * half_bytes; };
  auto xb_rel = [&](int h) { return each + (size_t)h * half_bytes; };
  auto part_h = [&](int h) { return reinterpret_cast<uint8_t*>(part) + part_rel(h); };
  auto xb_h = [&](int h) { return reinterpret_cast<uint8_t*>(part) + xb_rel(h); };
  (void)xbg;
  auto rowsz = [&](int cols) { return (size_t)Th * cols * es; };
  float* x_own[2] = {a.x_in, a.x_in + (size_t)rows * d};  // [rows, d] per half, inside the workspace's [T, d]
  cudaEvent_t* part_ready = p->ev_fork;  // [h]
  cudaEvent_t* xb_ready = p->ev_join;    // [h]
  auto exchange = [&](int h, bool reduce, const float* gain) -> int32_t {
    // on the communication stream, after the projection of half h has left its partial product
    if (reduce) {
      B200_CUDA_OK(cudaEventRecord(part_ready[h], stream));
      B200_CUDA_OK(cudaStreamWaitEvent(cs, part_ready[h], 0));
    }
    B200_TRY(comm_peer_reduce_norm_at(p->comm, Th, d, p->dtype, reduce, x_own[h], gain, eps, part_rel(h), xb_rel(h),
                                      /*lean=*/true, cs));
    B200_CUDA_OK(cudaEventRecord(xb_ready[h], cs));
    return B200_OK;
  };
  auto wait_xb = [&](int h) -> int32_t {
    B200_CUDA_OK(cudaStreamWaitEvent(stream, xb_ready[h], 0));
    return B200_OK;
  };
  // the communication stream starts behind everything the caller has queued (tokens, the previous call's readers)
  B200_CUDA_OK(cudaEventRecord(p->ev_fork[2], stream));
  B200_CUDA_OK(cudaStreamWaitEvent(cs, p->ev_fork[2], 0));
  for (int h = 0; h < 2; ++h) {
    // the embedding rows of this rank's share of half h; the first norm has no partial sums
    B200_TRY(launch_embed(tokens + (size_t)h * Th + row0, w + wl.emb, p->dtype, x_own[h], rows, d, p->V, cs));
    B200_TRY(exchange(h, false, g_att));
  }
  uint8_t* qkv = reinterpret_cast<uint8_t*>(a.qkv);
  uint8_t* o = reinterpret_cast<uint8_t*>(a.o);
  uint8_t* hg = reinterpret_cast<uint8_t*>(a.hg);
  for (int l = 0; l < p->L; ++l) {
    const LayerOffsets& lo = wl.layer[l];
    for (int h = 0; h < 2; ++h) {
      uint8_t* qkv_h = qkv + h * rowsz(3 * dl);
      uint8_t* o_h = o + h * rowsz(dl);
      B200_TRY(wait_xb(h));
      {
        EpiParams e;
        e.out = qkv_h; e.ldo = 3 * dl;
        e.rope_cos = p->rope_cos; e.rope_sin = p->rope_sin;
        e.seq_len = S; e.pos_base = 0; e.head_size = p->hs; e.rope_cols = 2 * dl;
        B200_TRY(gemm(*p, xb_h(h), d, w + lo.wqkv, d, Th, 3 * dl, d, EPI_ROPE, p->dtype, e, stream));
      }
      if (kv_out) {
        // kv_out [L, 2, B, S, d_loc]: rotated keys and values of this layer, rows of half h
        uint8_t* dst = reinterpret_cast<uint8_t*>(kv_out) + ((size_t)l * 2 * T + (size_t)h * Th) * dl * es;
        for (int part_i = 0; part_i < 2; ++part_i)
          B200_CUDA_OK(cudaMemcpy2DAsync(dst + (size_t)part_i * T * dl * es, (size_t)dl * es,
                                         qkv_h + (size_t)(1 + part_i) * dl * es, (size_t)3 * dl * es, (size_t)dl * es, Th,
                                         cudaMemcpyDeviceToDevice, stream));
      }
      {
        AttnArgs at;
        at.q = qkv_h; at.k = qkv_h + (size_t)dl * es; at.v = qkv_h + (size_t)2 * dl * es;
        at.o = o_h; at.lse = a.lse + (size_t)h * Bh * p->H_loc * S;
        at.batch = Bh; at.seq = S; at.n_heads = p->H_loc; at.head_size = p->hs;
        at.ldq = 3 * dl; at.ldkv = 3 * dl; at.ldo = dl; at.dtype = p->dtype;
        B200_TRY(launch_attn_fwd(at, p->attn_impl, stream));
      }
      {
        EpiParams e;
        e.out = part_h(h); e.ldo = d;
        B200_TRY(gemm(*p, o_h, dl, w + lo.wo, dl, Th, d, dl, EPI_STORE, p->dtype, e, stream));
      }
      B200_TRY(exchange(h, true, g_ffn + (size_t)l * d));
    }
    for (int h = 0; h < 2; ++h) {
      uint8_t* hg_h = hg + h * rowsz(hl);
      B200_TRY(wait_xb(h));
      {
        EpiParams e;
        e.out = hg_h; e.ldo = hl;
        B200_TRY(gemm(*p, xb_h(h), d, w + lo.w13, d, Th, 2 * hl, d, EPI_SWIGLU, p->dtype, e, stream));
      }
      {
        EpiParams e;
        e.out = part_h(h); e.ldo = d;
        B200_TRY(gemm(*p, hg_h, hl, w + lo.w2, hl, Th, d, hl, EPI_STORE, p->dtype, e, stream));
      }
      const float* g_next = l + 1 < p->L ? g_att + (size_t)(l + 1) * d : g_fin;
      B200_TRY(exchange(h, true, g_next));
    }
  }
  for (int h = 0; h < 2; ++h) {
    B200_TRY(wait_xb(h));
    if (logits) {
      EpiParams e;
      e.out = logits + (size_t)h * Th * p->V_loc; e.ldo = p->V_loc;
      B200_TRY(gemm(*p, xb_h(h), d, w + wl.wcls, d, Th, p->V_loc, d, EPI_STORE, B200_F32, e, stream));
    }
  }
  return B200_OK;
}

static int32_t forward_impl(B200Plan* p, const int32_t* tokens, int B, int S, const uint8_t* w, const PackedLayout& wl,
                            float* logits, void* saved, void* kv_out, void* ws, size_t ws_bytes,
                            cudaStream_t stream) {
  const int T = B * S;
  const bool keep = saved != nullptr;
  Arena wa(ws);
  FwdActs acts;
  if (keep) {
    Arena sa(saved);
    carve_forward(*p, sa, B, S, true, &acts);
  } else {
    carve_forward(*p, wa, B, S, false, &acts);
  }
  void* tp_tmp = p->tp_size > 1 ? wa.take((size_t)T * p->d * p->esize) : nullptr;
  if (wa.used > ws_bytes) return fail(B200_ERR_WORKSPACE, "forward needs %zu workspace bytes, got %zu", wa.used, ws_bytes);
  if (p->tp_size > 1 && !keep && T % p->tp_size == 0 && p->row_shard) {
    void *part = nullptr, *xbg = nullptr;
    if (comm_peer_rowshard_buffers(p->comm, (size_t)T * p->d * p->esize, &part, &xbg)) {
      // two halves of the batch in flight when the batch splits into two equal sets of sequences whose rows divide
      // over the ranks
      if (p->tp_pipeline && B % 2 == 0 && (B / 2 * S) % p->tp_size == 0 && ((size_t)(B / 2) * S * p->d * p->esize) % 256 == 0)
      {
        p->tp_push_last = 0;
        p->tp_bands_last = 0;
        return forward_row_sharded_pipelined(p, tokens, B, S, w, wl, logits, kv_out, acts.layer[0], part, xbg, stream);
      }
      return forward_row_sharded(p, tokens, B, S, w, wl, logits, kv_out, acts.layer[0], part, xbg, stream);
    }
  }

  const float* g_att = reinterpret_cast<const float*>(w + wl.g_att);
  const float* g_ffn = reinterpret_cast<const float*>(w + wl.g_ffn);
  const float* g_fin = reinterpret_cast<const float*>(w + wl.g_final);
  const float eps = p->cfg.rms_eps;
  const int d = p->d, dl = p->d_loc, hl = p->h_loc;

  B200_TRY(launch_embed(tokens, w + wl.emb, p->dtype, acts.layer[0].x_in, T, d, p->V, stream));
  for (int l = 0; l < p->L; ++l) {
    const LayerActs& a = acts.layer[l];
    const LayerOffsets& o = wl.layer[l];
    B200_TRY(launch_rmsnorm(a.x_in, g_att + (size_t)l * d, a.xb, a.rinv1, T, d, eps, p->dtype, stream));
    {  // q,k,v = xb Wqkv^T with the pair rotation of q and k fused (test/llama.py:149-168)
      EpiParams e;
      e.out = a.qkv; e.ldo = 3 * dl;
      e.rope_cos = p->rope_cos; e.rope_sin = p->rope_sin;
      e.seq_len = S; e.pos_base = 0; e.head_size = p->hs; e.rope_cols = 2 * dl;
      B200_TRY(gemm(*p, a.xb, d, w + o.wqkv, d, T, 3 * dl, d, EPI_ROPE, p->dtype, e, stream));
    }
    if (kv_out) {
      // kv_out [L, 2, B, S, d_loc]: rotated keys and values of this layer
      uint8_t* dst = reinterpret_cast<uint8_t*>(kv_out) + (size_t)l * 2 * T * dl * p->esize;
      const uint8_t* src = reinterpret_cast<const uint8_t*>(a.qkv);
      for (int part = 0; part < 2; ++part)
        B200_CUDA_OK(cudaMemcpy2DAsync(dst + (size_t)part * T * dl * p->esize, (size_t)dl * p->esize,
                                       src + (size_t)(1 + part) * dl * p->esize, (size_t)3 * dl * p->esize,
                                       (size_t)dl * p->esize, T, cudaMemcpyDeviceToDevice, stream));
    }
    {
      AttnArgs at;
      const uint8_t* base = reinterpret_cast<const uint8_t*>(a.qkv);
      at.q = base; at.k = base + (size_t)dl * p->esize; at.v = base + (size_t)2 * dl * p->esize;
      at.o = a.o; at.lse = a.lse;
      at.batch = B; at.seq = S; at.n_heads = p->H_loc; at.head_size = p->hs;
      at.ldq = 3 * dl; at.ldkv = 3 * dl; at.ldo = dl; at.dtype = p->dtype;
      B200_TRY(launch_attn_fwd(at, p->attn_impl, stream));
    }
    B200_TRY(proj_residual(*p, a.o, dl, w + o.wo, dl, T, dl, a.x_in, a.x_mid, tp_tmp, stream));
    B200_TRY(launch_rmsnorm(a.x_mid, g_ffn + (size_t)l * d, a.xb2, a.rinv2, T, d, eps, p->dtype, stream));
    {  // hg = silu(xb2 W1^T) * (xb2 W3^T) from the interleaved [W1;W3] product (test/llama.py:224-229)
      EpiParams e;
      e.out = a.hg; e.ldo = hl; e.out_gate = a.gate; e.out_up = a.up;
      B200_TRY(gemm(*p, a.xb2, d, w + o.w13, d, T, 2 * hl, d, EPI_SWIGLU, p->dtype, e, stream));
    }
    B200_TRY(proj_residual(*p, a.hg, hl, w + o.w2, hl, T, hl, a.x_mid, a.x_out, tp_tmp, stream));
  }
  B200_TRY(launch_rmsnorm(acts.fin.x_last, g_fin, acts.fin.xf, acts.fin.rinv_f, T, d, eps, p->dtype, stream));
  if (logits) {
    EpiParams e;
    e.out = logits; e.ldo = p->V_loc;
    B200_TRY(gemm(*p, acts.fin.xf, d, w + wl.wcls, d, T, p->V_loc, d, EPI_STORE, B200_F32, e, stream));
  }
  return B200_OK;
}

int32_t launch_attn_fwd(const AttnArgs& a, int impl, cudaStream_t stream) {
  // causal: half of the 4*S^2*hs flops per (batch, head)
  ProfScope prof(PROF_ATTN_FWD, 2.0 * a.batch * a.n_heads * (double)a.seq * a.seq * a.head_size, stream);
  if (impl == 2) return launch_attn_fwd_simt(a, stream);
  if (impl == 1) return launch_attn_fwd_mma(a, stream);
  if (attn_fwd_mma_supports(a)) return launch_attn_fwd_mma(a, stream);
  return launch_attn_fwd_simt(a, stream);
}

static int32_t check_plan_call(const B200Plan* p, int B, int S) {
  if (!p) return fail(B200_ERR_INVALID_ARG, "plan is null");
  if (B <= 0 || S <= 0) return fail(B200_ERR_BAD_SHAPE, "batch=%d seq=%d must be positive", B, S);
  if (S > p->cfg.seq_len) return fail(B200_ERR_BAD_SHAPE, "seq=%d exceeds the plan's seq_len=%d", S, p->cfg.seq_len);
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev != p->device)
    return fail(B200_ERR_INVALID_ARG, "plan was created on device %d, current device is %d", p->device, dev);
  return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" {

const char* b200_last_error(void) { return g_err; }
const char* b200_version(void) { return "0.1"; }
int64_t b200_launch_count(void) { return g_launches.load(); }

int32_t b200_profile_enable(int32_t on) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (on) g_prof_used = 0;
  g_prof_on.store(on ? 1 : 0);
  return B200_OK;
}

int32_t b200_profile_read(int32_t cls, double* total_ms, double* total_work, int64_t* launches) {
  if (cls < 0 || cls >= PROF_NUM) return fail(B200_ERR_INVALID_ARG, "unknown kernel class %d", cls);
  std::lock_guard<std::mutex> lk(g_prof_mu);
  double ms = 0, work = 0;
  int64_t n = 0;
  for (size_t i = 0; i < g_prof_used; ++i) {
    if (g_prof[i].cls != cls) continue;
    B200_CUDA_OK(cudaEventSynchronize(g_prof[i].b));
    float t = 0.f;
    B200_CUDA_OK(cudaEventElapsedTime(&t, g_prof[i].a, g_prof[i].b));
    ms += t; work += g_prof[i].work; ++n;
  }
  if (total_ms) *total_ms = ms;
  if (total_work) *total_work = work;
  if (launches) *launches = n;
  return B200_OK;
}

int32_t b200_device_status(b200_stream_t stream, uint32_t* code) {
  uint32_t* word = device_status_word();
  if (!word) return fail(B200_ERR_CUDA, "no device status word");
  uint32_t host = 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  B200_CUDA_OK(cudaMemcpyAsync(&host, word, 4, cudaMemcpyDeviceToHost, s));
  B200_CUDA_OK(cudaStreamSynchronize(s));
  if (host) {
    B200_CUDA_OK(cudaMemsetAsync(word, 0, 4, s));
    B200_CUDA_OK(cudaStreamSynchronize(s));
  }
  if (code) *code = host;
  if (host) return fail(B200_ERR_TIMEOUT, "a bounded device-side wait ran out (status word 0x%x)", host);
  return B200_OK;
}

int32_t b200_plan_create(const B200LlamaConfig* cfg, int32_t tp_rank, int32_t tp_size, void* comm, B200Plan** out) {
  if (!cfg || !out) return fail(B200_ERR_INVALID_ARG, "cfg and out must not be null");
  *out = nullptr;
  if (cfg->dim <= 0 || cfg->hidden_dim <= 0 || cfg->n_layers <= 0 || cfg->n_heads <= 0 || cfg->vocab_size <= 0 ||
      cfg->seq_len <= 0)
    return fail(B200_ERR_BAD_SHAPE, "config sizes must be positive");
  if (cfg->n_kv_heads != cfg->n_heads)
    return fail(B200_ERR_UNSUPPORTED, "n_kv_heads (%d) must equal n_heads (%d), as in the reference model",
                cfg->n_kv_heads, cfg->n_heads);
  if (cfg->dim % cfg->n_heads) return fail(B200_ERR_BAD_SHAPE, "dim %% n_heads != 0");
  if (cfg->dtype != B200_F32 && cfg->dtype != B200_BF16) return fail(B200_ERR_BAD_DTYPE, "dtype must be fp32 or bf16");
  if (tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size) return fail(B200_ERR_INVALID_ARG, "bad tensor-parallel rank %d of %d", tp_rank, tp_size);
  if (tp_size > 1 && !comm) return fail(B200_ERR_INVALID_ARG, "tensor parallelism needs a communicator");
  const int hs = cfg->dim / cfg->n_heads;
  if (hs != 16 && hs != 32 && hs != 48 && hs != 64 && hs != 128)
    return fail(B200_ERR_BAD_SHAPE, "head size %d is not one of 16/32/48/64/128", hs);
  if (cfg->n_heads % tp_size || cfg->hidden_dim % (16 * tp_size) || cfg->vocab_size % (16 * tp_size) ||
      (cfg->dim / tp_size) % 16 || cfg->dim % 16)
    return fail(B200_ERR_BAD_SHAPE, "dim, hidden_dim, vocab (per rank) must be multiples of 16 and heads divisible by tp_size");
  int dev = 0;
  B200_CUDA_OK(cudaGetDevice(&dev));
  int major = 0;
  B200_CUDA_OK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) return fail(B200_ERR_ARCH, "device %d has compute capability %d.x; this library is sm_100a only", dev, major);

  B200Plan* p = new B200Plan();
  p->cfg = *cfg;
  p->tp_rank = tp_rank; p->tp_size = tp_size; p->comm = comm;
  p->d = cfg->dim; p->h = cfg->hidden_dim; p->L = cfg->n_layers; p->H = cfg->n_heads; p->hs = hs; p->V = cfg->vocab_size;
  p->d_loc = p->d / tp_size; p->h_loc = p->h / tp_size; p->V_loc = p->V / tp_size; p->H_loc = p->H / tp_size;
  p->dtype = cfg->dtype;
  p->esize = cfg->dtype == B200_BF16 ? 2 : 4;
  p->device = dev;
  p->gemm_impl = env_int("B200_GEMM_IMPL", 0);
  p->attn_impl = env_int("B200_ATTN_IMPL", 0);
  build_layout(*p, p->esize, false, &p->wl);
  build_layout(*p, p->esize, true, &p->wlt);
  build_layout(*p, 4, false, &p->gl);
  const size_t tb = (size_t)cfg->seq_len * (hs / 2) * 4;
  if (cudaMalloc(&p->rope_cos, tb) != cudaSuccess || cudaMalloc(&p->rope_sin, tb) != cudaSuccess) {
    cudaFree(p->rope_cos);
    delete p;
    return fail(B200_ERR_CUDA, "cannot allocate the rotation tables");
  }
  int32_t st = launch_rope_table(p->rope_cos, p->rope_sin, cfg->seq_len, hs, cfg->rope_theta, 0);
  if (st == B200_OK && cudaStreamSynchronize(0) != cudaSuccess) st = fail(B200_ERR_CUDA, "rotation table kernel failed");
  if (st != B200_OK) {
    cudaFree(p->rope_cos); cudaFree(p->rope_sin);
    delete p;
    return st;
  }
  device_status_word();
  if (tp_size > 1) {
    // Chunked projections with the all-reduce of chunk c overlapping the GEMM of chunk c+1 measured SLOWER
    // than one all-reduce per block on 4 GPUs (45.3 ms vs 48.9 / 54.1 ms for 2 / 4 chunks), so the default is 1.
    p->row_shard = env_int("B200_TP_ROW_SHARD", 1) != 0;
    // Two halves in flight hide the exchange but halve the rows of every GEMM and put a second kernel on the SMs; at
    // the 7B shape that won on one 4-GPU box (30.1 against 34.0 ms per step) and lost on three others (36-37 against
    // 34-35 ms) and at two ranks (57-61 against 54.5 ms).  So it is off unless asked for (B200_TP_PIPELINE = 1) or
    // chosen by a caller that timed both (b200_plan_set_option).
    p->tp_pipeline = env_int("B200_TP_PIPELINE", 0) != 0;
    p->tp_push = env_int("B200_TP_PUSH", 1) != 0;  // 0: the exchange kernel pulls the partial products itself
    p->tp_bands = env_int("B200_TP_BANDS", 1) != 0;  // 0: the exchange kernel waits for all gathered rows itself
    p->reserve_sms = env_int("B200_TP_RESERVE_SMS", 0);
    p->tp_chunks = env_int("B200_TP_CHUNKS", 1);
    if (p->tp_chunks < 1) p->tp_chunks = 1;
    if (p->tp_chunks > 8) p->tp_chunks = 8;
    bool ok = cudaStreamCreateWithFlags(&p->comm_stream, cudaStreamNonBlocking) == cudaSuccess;
    for (int i = 0; i < 8 && ok; ++i)
      ok = cudaEventCreateWithFlags(&p->ev_fork[i], cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&p->ev_join[i], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) {
      b200_plan_destroy(p);
      return fail(B200_ERR_CUDA, "cannot create the communication stream and events");
    }
  }
  *out = p;
  return B200_OK;
}

int32_t b200_plan_destroy(B200Plan* p) {
  if (!p) return B200_OK;
  cudaFree(p->rope_cos);
  cudaFree(p->rope_sin);
  for (int i = 0; i < 8; ++i) {
    if (p->ev_fork[i]) cudaEventDestroy(p->ev_fork[i]);
    if (p->ev_join[i]) cudaEventDestroy(p->ev_join[i]);
  }
  if (p->comm_stream) cudaStreamDestroy(p->comm_stream);
  delete p;
  return B200_OK;
}

// Registry of plans for callers that cannot keep a handle (custom-call handlers): keyed by the config, the
// tensor-parallel placement, the communicator and the device; entries live until the process exits.
namespace {
struct PlanKey {
  B200LlamaConfig cfg;
  int tp_rank, tp_size, device;
  void* comm;
};
struct PlanEntry { PlanKey key; B200Plan* plan; };
std::mutex g_plans_mu;
std::vector<PlanEntry> g_plans;
bool same_key(const PlanKey& a, const PlanKey& b) {
  return a.cfg.dim == b.cfg.dim && a.cfg.hidden_dim == b.cfg.hidden_dim && a.cfg.n_layers == b.cfg.n_layers &&
         a.cfg.n_heads == b.cfg.n_heads && a.cfg.n_kv_heads == b.cfg.n_kv_heads && a.cfg.vocab_size == b.cfg.vocab_size &&
         a.cfg.seq_len == b.cfg.seq_len && a.cfg.dtype == b.cfg.dtype && a.cfg.rope_theta == b.cfg.rope_theta &&
         a.cfg.rms_eps == b.cfg.rms_eps && a.tp_rank == b.tp_rank && a.tp_size == b.tp_size && a.device == b.device &&
         a.comm == b.comm;
}
}  // namespace

int32_t b200_plan_cached(const B200LlamaConfig* cfg, int32_t tp_rank, int32_t tp_size, void* comm, B200Plan** out) {
  if (!cfg || !out) return fail(B200_ERR_INVALID_ARG, "cfg and out must not be null");
  PlanKey key;
  key.cfg = *cfg; key.tp_rank = tp_rank; key.tp_size = tp_size; key.comm = comm; key.device = -1;
  B200_CUDA_OK(cudaGetDevice(&key.device));
  std::lock_guard<std::mutex> lk(g_plans_mu);
  for (const PlanEntry& e : g_plans)
    if (same_key(e.key, key)) {
      *out = e.plan;
      return B200_OK;
    }
  B200Plan* p = nullptr;
  B200_TRY(b200_plan_create(cfg, tp_rank, tp_size, comm, &p));
  g_plans.push_back(PlanEntry{key, p});
  *out = p;
  return B200_OK;
}

// Run-time options of a plan.  "tp_pipeline": 1 = the tensor-parallel prefill runs two halves of the batch with
// the exchange of one beside the compute of the other, 0 = one batch with the exchange between the kernels.  Every
// rank of the communicator must hold the same value whenever b200_forward runs (the exchange kernels pair up in
// launch order); which of the two is faster depends on the rank count and on how busy the NVLink fabric is, so a
// caller may time both during warm-up and keep the faster one.  "tp_push": 1 (default) = the row-parallel projections
// of that prefill store their partial products straight into the memory of the ranks that own the rows, 0 = into
// local memory, from where the exchange kernel pulls them; same value on every rank.
int32_t b200_plan_set_option(B200Plan* p, const char* name, int32_t value) {
  if (!p || !name) return fail(B200_ERR_INVALID_ARG, "null argument");
  if (!strcmp(name, "tp_pipeline")) {
    p->tp_pipeline = value != 0;
    return B200_OK;
  }
  if (!strcmp(name, "tp_push")) {
    p->tp_push = value != 0;
    return B200_OK;
  }
  if (!strcmp(name, "tp_bands")) {
    p->tp_bands = value != 0;
    return B200_OK;
  }
  return fail(B200_ERR_INVALID_ARG, "unknown plan option '%s'", name);
}

int32_t b200_plan_get_option(const B200Plan* p, const char* name, int32_t* value) {
  if (!p || !name || !value) return fail(B200_ERR_INVALID_ARG, "null argument");
  if (!strcmp(name, "tp_pipeline")) {
    *value = p->tp_pipeline ? 1 : 0;
    return B200_OK;
  }
  if (!strcmp(name, "tp_push")) {
    *value = p->tp_push ? 1 : 0;
    return B200_OK;
  }
  if (!strcmp(name, "tp_bands")) {
    *value = p->tp_bands ? 1 : 0;
    return B200_OK;
  }
  if (!strcmp(name, "tp_bands_last")) {  // read-only
    *value = p->tp_bands_last;
    return B200_OK;
  }
  if (!strcmp(name, "tp_push_last")) {  // read-only: whether the last tensor-parallel forward pushed its partial products
    *value = p->tp_push_last;
    return B200_OK;
  }
  return fail(B200_ERR_INVALID_ARG, "unknown plan option '%s'", name);
}

int32_t b200_packed_weight_bytes(const B200Plan* p, int32_t with_t, size_t* bytes) {
  if (!p || !bytes) return fail(B200_ERR_INVALID_ARG, "null argument");
  *bytes = with_t ? p->wlt.total : p->wl.total;
  return B200_OK;
}

int32_t b200_packed_grad_bytes(const B200Plan* p, size_t* bytes) {
  if (!p || !bytes) return fail(B200_ERR_INVALID_ARG, "null argument");
  *bytes = p->gl.total;
  return B200_OK;
}

int32_t b200_pack_weights(const B200Plan* p, const void* const* leaves, int32_t ld, int32_t with_t, void* packed,
                          b200_stream_t stream_) {
  if (!p || !leaves || !packed) return fail(B200_ERR_INVALID_ARG, "null argument");
  for (int i = 0; i < B200_NUM_LEAVES; ++i) {
    if (!leaves[i]) return fail(B200_ERR_INVALID_ARG, "leaf %d is null", i);
    if (!aligned16(leaves[i])) return fail(B200_ERR_MISALIGNED, "leaf %d is not 16-byte aligned", i);
  }
  if (ld != B200_F32 && ld != B200_BF16) return fail(B200_ERR_BAD_DTYPE, "leaf dtype must be fp32 or bf16");
  if (!aligned16(packed)) return fail(B200_ERR_MISALIGNED, "packed buffer is not 16-byte aligned");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const PackedLayout& wl = with_t ? p->wlt : p->wl;
  uint8_t* w = reinterpret_cast<uint8_t*>(packed);
  const size_t les = ld == B200_BF16 ? 2 : 4;
  const int d = p->d, h = p->h, dl = p->d_loc, hl = p->h_loc, Vl = p->V_loc, L = p->L, r = p->tp_rank, dt = p->dtype;
  auto leaf = [&](int i, size_t elem_off) { return reinterpret_cast<const uint8_t*>(leaves[i]) + elem_off * les; };
  auto plain = [&](const void* src, int sld, void* dst, int dld, int rows, int cols, int ddt) {
    return launch_copy_rows(src, ld, sld, dst, ddt, dld, rows, cols, rows, rows, 0, s);
  };
  B200_TRY(plain(leaf(B200_LEAF_RMS_ATT, 0), d, w + wl.g_att, d, L, d, B200_F32));
  B200_TRY(plain(leaf(B200_LEAF_RMS_FFN, 0), d, w + wl.g_ffn, d, L, d, B200_F32));
  B200_TRY(plain(leaf(B200_LEAF_RMS_FINAL, 0), d, w + wl.g_final, d, 1, d, B200_F32));
  B200_TRY(plain(leaf(B200_LEAF_TOK_EMB, 0), d, w + wl.emb, d, p->V, d, dt));
  for (int l = 0; l < L; ++l) {
    const LayerOffsets& o = wl.layer[l];
    const size_t dd = (size_t)l * d * d, hd = (size_t)l * h * d;
    const int qkv_leaf[3] = {B200_LEAF_WQ, B200_LEAF_WK, B200_LEAF_WV};
    for (int j = 0; j < 3; ++j)  // head rows of this rank, q then k then v
      B200_TRY(plain(leaf(qkv_leaf[j], dd + (size_t)r * dl * d), d, w + o.wqkv + (size_t)j * dl * d * p->esize, d, dl,
                     d, dt));
    // wo [d, d]: columns of this rank's heads
    B200_TRY(plain(leaf(B200_LEAF_WO, dd + (size_t)r * dl), d, w + o.wo, dl, d, dl, dt));
    // w1/w3 rows of this rank, interleaved in groups of 8: [8 of w1 | 8 of w3 | ...]
    B200_TRY(launch_copy_rows(leaf(B200_LEAF_W1, hd + (size_t)r * hl * d), ld, d, w + o.w13, dt, d, hl, d, 8, 16, 0, s));
    B200_TRY(launch_copy_rows(leaf(B200_LEAF_W3, hd + (size_t)r * hl * d), ld, d, w + o.w13, dt, d, hl, d, 8, 16, 8, s));
    // w2 [d, h]: columns of this rank's hidden units
    B200_TRY(plain(leaf(B200_LEAF_W2, hd + (size_t)r * hl), h, w + o.w2, hl, d, hl, dt));
    if (with_t) {
      B200_TRY(launch_transpose(w + o.wqkv, dt, d, w + o.wqkv_t, dt, 3 * dl, 3 * dl, d, s));
      B200_TRY(launch_transpose(w + o.wo, dt, dl, w + o.wo_t, dt, d, d, dl, s));
      B200_TRY(launch_transpose(w + o.w13, dt, d, w + o.w13_t, dt, 2 * hl, 2 * hl, d, s));
      B200_TRY(launch_transpose(w + o.w2, dt, hl, w + o.w2_t, dt, d, d, hl, s));
    }
  }
  B200_TRY(plain(leaf(B200_LEAF_WCLS, (size_t)r * Vl * d), d, w + wl.wcls, d, Vl, d, dt));
  if (with_t) B200_TRY(launch_transpose(w + wl.wcls, dt, d, w + wl.wcls_t, dt, Vl, Vl, d, s));
  return B200_OK;
}

int32_t b200_saved_bytes(const B200Plan* p, int32_t B, int32_t S, size_t* bytes) {
  if (!p || !bytes) return fail(B200_ERR_INVALID_ARG, "null argument");
  if (B <= 0 || S <= 0) return fail(B200_ERR_BAD_SHAPE, "batch and seq must be positive");
  Arena a(nullptr);
  FwdActs acts;
  carve_forward(*p, a, B, S, true, &acts);
  *bytes = a.used;
  return B200_OK;
}

int32_t b200_forward(B200Plan* p, const int32_t* tokens, int32_t B, int32_t S, const void* packed_w, float* logits,
                     void* saved, void* kv_out, void* ws, size_t ws_bytes, b200_stream_t stream) {
  B200_TRY(check_plan_call(p, B, S));
  if (!tokens || !packed_w || !ws) return fail(B200_ERR_INVALID_ARG, "tokens, weights and workspace must not be null");
  if (!aligned16(ws) || !aligned16(packed_w) || (logits && !aligned16(logits)) || (saved && !aligned16(saved)))
    return fail(B200_ERR_MISALIGNED, "buffers must be 16-byte aligned");
  // The backward pass contracts against the transposed copies, which sit
  // behind the plain weights in both layouts, so either packing serves here.
  return forward_impl(p, tokens, B, S, reinterpret_cast<const uint8_t*>(packed_w), p->wl, logits, saved, kv_out, ws,
                      ws_bytes, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
