// One decode step over the paged KV cache, plus the workspace-size query and
// the single-kernel entry points of the C ABI.
#include "attention.cuh"
#include "elementwise.cuh"
#include "gemm_epilogue.cuh"
#include "plan.cuh"

namespace b200 {

size_t backward_workspace_bytes(const B200Plan& p, int B, int S);

namespace {

// Writes row `pos` of every sequence: the rotated key and the value just
// produced by the QKV projection (test/llama.py:170-175, append-last).  Pages
// are head-major: [page][head][row][head_size].
template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ qkv, T* __restrict__ kpages, T* __restrict__ vpages,
                                 const int32_t* __restrict__ page_table, int pos, int page_size, int max_pages,
                                 int d_local, int hs) {
  constexpr int E = 16 / sizeof(T);  // elements per 16-byte piece
  const int b = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();  // qkv comes from the projection before
  const int page = page_table[(size_t)b * max_pages + pos / page_size];
  const int n_heads = d_local / hs;
  const T* src = qkv + (size_t)b * 3 * d_local;
  for (int c = threadIdx.x * E; c < d_local; c += blockDim.x * E) {
    const int h = c / hs, e = c % hs;
    const size_t dst = (((size_t)page * n_heads + h) * page_size + pos % page_size) * hs + e;
    *reinterpret_cast<uint4*>(kpages + dst) = *reinterpret_cast<const uint4*>(src + d_local + c);
    *reinterpret_cast<uint4*>(vpages + dst) = *reinterpret_cast<const uint4*>(src + 2 * d_local + c);
  }
}

struct DecodeWs {
  float* x; void* xb; void* qkv; void* o; void* hg; void* tp_tmp; float* scratch;
  void* splitk; size_t splitk_bytes;
  int n_splits;
};

void carve_decode(const B200Plan& p, Arena& a, int B, int ctx, DecodeWs* w) {
  const size_t es = p.esize;
  w->x = a.take<float>((size_t)B * p.d * 4);
  w->xb = a.take((size_t)B * p.d * es);
  w->qkv = a.take((size_t)B * 3 * p.d_loc * es);
  w->o = a.take((size_t)B * p.d_loc * es);
  w->hg = a.take((size_t)B * p.h_loc * es);
  w->tp_tmp = p.tp_size > 1 ? a.take((size_t)B * p.d * es) : nullptr;
  w->n_splits = decode_pick_splits(B, p.H_loc, ctx);
  w->scratch = a.take<float>(decode_scratch_floats(B, p.H_loc, p.hs, w->n_splits) * 4);
  // K-split partials of the projections: up to 8 splits of the widest one (W1|W3)
  w->splitk_bytes = (size_t)8 * B * 2 * p.h_loc * 4;
  w->splitk = a.take(w->splitk_bytes);
}

int32_t gemm(const B200Plan& p, const DecodeWs& ws, const void* A, int lda, const void* Bm, int ldb, int M, int N, int K,
             int kind, int out_dtype, const EpiParams& epi, cudaStream_t stream) {
  GemmArgs g;
  g.splitk_scratch = ws.splitk; g.splitk_bytes = ws.splitk_bytes;
  g.A = A; g.B = Bm; g.M = M; g.N = N; g.K = K; g.lda = lda; g.ldb = ldb;
  g.in_dtype = p.dtype; g.out_dtype = out_dtype; g.kind = kind; g.epi = epi;
  return launch_gemm(g, p.gemm_impl, stream);
}

int32_t proj_residual(const B200Plan& p, const DecodeWs& ws, const void* A, int lda, const void* W, int ldw, int M, int K,
                      float* x, void* tp_tmp, cudaStream_t stream) {
  EpiParams e;
  if (p.tp_size == 1) {
    e.out = x; e.ldo = p.d; e.resid_in = x;
    return gemm(p, ws, A, lda, W, ldw, M, p.d, K, EPI_RESID, B200_F32, e, stream);
  }
  if (void* pbuf = comm_peer_buffer(p.comm, (size_t)M * p.d * p.esize)) {
    e.out = pbuf; e.ldo = p.d;
    B200_TRY(gemm(p, ws, A, lda, W, ldw, M, p.d, K, EPI_STORE, p.dtype, e, stream));
    return comm_peer_allreduce_add(p.comm, (size_t)M * p.d, p.dtype, x, x, stream);
  }
  e.out = tp_tmp; e.ldo = p.d;
  B200_TRY(gemm(p, ws, A, lda, W, ldw, M, p.d, K, EPI_STORE, p.dtype, e, stream));
  B200_TRY(comm_allreduce(p.comm, tp_tmp, (size_t)M * p.d, p.dtype, stream));
  return launch_add_to_f32(x, tp_tmp, p.dtype, (size_t)M * p.d, stream);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int32_t b200_workspace_bytes(const B200Plan* p, int32_t mode, int32_t B, int32_t S, size_t* bytes) {
  if (!p || !bytes) return fail(B200_ERR_INVALID_ARG, "null argument");
  if (B <= 0 || S <= 0) return fail(B200_ERR_BAD_SHAPE, "batch and seq must be positive");
  Arena a(nullptr);
  const size_t tp = p->tp_size > 1 ? align_up((size_t)B * S * p->d * p->esize, 256) : 0;
  switch (mode) {
    case 0: {
      FwdActs acts;
      carve_forward(*p, a, B, S, false, &acts);
      *bytes = a.used + tp + 256;
      return B200_OK;
    }
    case 1: *bytes = tp + 256; return B200_OK;
    case 2: *bytes = backward_workspace_bytes(*p, B, S) + 256; return B200_OK;
    case 3: {
      DecodeWs w;
      carve_decode(*p, a, B, S, &w);  // S = context length after the step
      *bytes = a.used + 256;
      return B200_OK;
    }
  }
  return fail(B200_ERR_INVALID_ARG, "unknown workspace mode %d", mode);
}

int32_t b200_decode_step(B200Plan* p, const int32_t* tokens, const float* x_in, int32_t B, int32_t pos,
                         const void* packed_w, void* kv_pages, const int32_t* page_table, int32_t n_pages,
                         int32_t page_size, int32_t max_pages, float* hidden_out, float* logits, void* ws,
                         size_t ws_bytes, b200_stream_t stream_) {
  if (!p) return fail(B200_ERR_INVALID_ARG, "plan is null");
  if (B <= 0 || pos < 0) return fail(B200_ERR_BAD_SHAPE, "batch=%d pos=%d", B, pos);
  if (pos >= p->cfg.seq_len) return fail(B200_ERR_BAD_SHAPE, "pos=%d exceeds the plan's seq_len=%d", pos, p->cfg.seq_len);
  if ((!tokens && !x_in) || !packed_w || !kv_pages || !page_table || !ws)
    return fail(B200_ERR_INVALID_ARG, "null argument");
  if (n_pages <= 0 || page_size <= 0 || max_pages <= 0 || (pos / page_size) >= max_pages)
    return fail(B200_ERR_BAD_SHAPE, "page geometry does not hold position %d", pos);
  if (!aligned16(packed_w) || !aligned16(kv_pages) || !aligned16(ws) || (x_in && !aligned16(x_in)))
    return fail(B200_ERR_MISALIGNED, "buffers must be 16-byte aligned");
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev != p->device) return fail(B200_ERR_INVALID_ARG, "wrong current device");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const int ctx = pos + 1;
  Arena wa(ws);
  DecodeWs w;
  carve_decode(*p, wa, B, ctx, &w);
  if (wa.used > ws_bytes) return fail(B200_ERR_WORKSPACE, "decode needs %zu workspace bytes, got %zu", wa.used, ws_bytes);

  const uint8_t* wt = reinterpret_cast<const uint8_t*>(packed_w);
  const PackedLayout& wl = p->wl;
  const float* g_att = reinterpret_cast<const float*>(wt + wl.g_att);
  const float* g_ffn = reinterpret_cast<const float*>(wt + wl.g_ffn);
  const float* g_fin = reinterpret_cast<const float*>(wt + wl.g_final);
  const int d = p->d, dl = p->d_loc, hl = p->h_loc, es = p->esize;
  const float eps = p->cfg.rms_eps;

  if (x_in)
    B200_CUDA_OK(cudaMemcpyAsync(w.x, x_in, (size_t)B * d * 4, cudaMemcpyDeviceToDevice, stream));
  else
    B200_TRY(launch_embed(tokens, wt + wl.emb, p->dtype, w.x, B, d, p->V, stream));

  const size_t layer_bytes = (size_t)2 * n_pages * page_size * dl * es;
  for (int l = 0; l < p->L; ++l) {
    const LayerOffsets& o = wl.layer[l];
    uint8_t* kv = reinterpret_cast<uint8_t*>(kv_pages) + (size_t)l * layer_bytes;
    B200_TRY(launch_rmsnorm(w.x, g_att + (size_t)l * d, w.xb, nullptr, B, d, eps, p->dtype, stream));
    {
      EpiParams e;
      e.out = w.qkv; e.ldo = 3 * dl;
      e.rope_cos = p->rope_cos; e.rope_sin = p->rope_sin;
      e.seq_len = 1; e.pos_base = pos; e.head_size = p->hs; e.rope_cols = 2 * dl;
      B200_TRY(gemm(*p, w, w.xb, d, wt + o.wqkv, d, B, 3 * dl, d, EPI_ROPE, p->dtype, e, stream));
    }
    if (p->dtype == B200_BF16)
      B200_CUDA_OK(launch_pdl(kv_append_kernel<bf16>, dim3(B), dim3(128), 0, stream, (const bf16*)w.qkv, (bf16*)kv,
                              (bf16*)(kv + layer_bytes / 2), page_table, pos, page_size, max_pages, dl, p->hs));
    else
      B200_CUDA_OK(launch_pdl(kv_append_kernel<float>, dim3(B), dim3(128), 0, stream, (const float*)w.qkv, (float*)kv,
                              (float*)(kv + layer_bytes / 2), page_table, pos, page_size, max_pages, dl, p->hs));
    B200_LAUNCH_OK("kv_append_kernel");
    {
      AttnDecodeArgs a;
      a.q = w.qkv; a.kv_pages = kv; a.page_table = page_table; a.o = w.o; a.scratch = w.scratch;
      a.batch = B; a.ctx = ctx; a.n_heads = p->H_loc; a.head_size = p->hs;
      a.ldq = 3 * dl; a.ldo = dl; a.n_pages = n_pages; a.page_size = page_size; a.max_pages = max_pages;
      a.d_local = dl; a.dtype = p->dtype; a.n_splits = w.n_splits;
      B200_TRY(launch_attn_decode(a, stream));
    }
    B200_TRY(proj_residual(*p, w, w.o, dl, wt + o.wo, dl, B, dl, w.x, w.tp_tmp, stream));
    B200_TRY(launch_rmsnorm(w.x, g_ffn + (size_t)l * d, w.xb, nullptr, B, d, eps, p->dtype, stream));
    {
      EpiParams e;
      e.out = w.hg; e.ldo = hl;
      B200_TRY(gemm(*p, w, w.xb, d, wt + o.w13, d, B, 2 * hl, d, EPI_SWIGLU, p->dtype, e, stream));
    }
    B200_TRY(proj_residual(*p, w, w.hg, hl, wt + o.w2, hl, B, hl, w.x, w.tp_tmp, stream));
  }
  if (hidden_out) B200_TRY(launch_rmsnorm(w.x, g_fin, hidden_out, nullptr, B, d, eps, B200_F32, stream));
  if (logits) {
    B200_TRY(launch_rmsnorm(w.x, g_fin, w.xb, nullptr, B, d, eps, p->dtype, stream));
    EpiParams e;
    e.out = logits; e.ldo = p->V_loc;
    B200_TRY(gemm(*p, w, w.xb, d, wt + wl.wcls, d, B, p->V_loc, d, EPI_STORE, B200_F32, e, stream));
  }
  return B200_OK;
}

int32_t b200_gemm(const void* A, const void* Bm, void* Y, int32_t M, int32_t N, int32_t K, int32_t lda, int32_t ldb,
                  int32_t ldy, int32_t ta, int32_t tb, int32_t in_dtype, int32_t out_dtype, int32_t accumulate,
                  int32_t impl, b200_stream_t stream) {
  if (!A || !Bm || !Y) return fail(B200_ERR_INVALID_ARG, "null operand");
  GemmArgs g;
  g.A = A; g.B = Bm; g.M = M; g.N = N; g.K = K; g.lda = lda; g.ldb = ldb; g.ta = ta; g.tb = tb;
  g.in_dtype = in_dtype; g.out_dtype = out_dtype; g.kind = EPI_STORE;
  g.epi.out = Y; g.epi.ldo = ldy; g.epi.accumulate = accumulate;
  return launch_gemm(g, impl, reinterpret_cast<cudaStream_t>(stream));
}

int32_t b200_rmsnorm(const float* x, const float* gain, void* y, float* rinv, int32_t rows, int32_t dim, float eps,
                     int32_t out_dtype, b200_stream_t stream) {
  if (!x || !gain || !y) return fail(B200_ERR_INVALID_ARG, "null operand");
  if (!aligned16(x) || !aligned16(gain) || !aligned16(y)) return fail(B200_ERR_MISALIGNED, "operands must be 16-byte aligned");
  return launch_rmsnorm(x, gain, y, rinv, rows, dim, eps, out_dtype, reinterpret_cast<cudaStream_t>(stream));
}

int32_t b200_attention(const void* q, const void* k, const void* v, void* o, float* lse, int32_t batch, int32_t seq,
                       int32_t n_heads, int32_t head_size, int32_t ldq, int32_t ldkv, int32_t ldo, int32_t dtype,
                       int32_t impl, b200_stream_t stream) {
  if (!q || !k || !v || !o) return fail(B200_ERR_INVALID_ARG, "null operand");
  AttnArgs a;
  a.q = q; a.k = k; a.v = v; a.o = o; a.lse = lse;
  a.batch = batch; a.seq = seq; a.n_heads = n_heads; a.head_size = head_size;
  a.ldq = ldq; a.ldkv = ldkv; a.ldo = ldo; a.dtype = dtype;
  return launch_attn_fwd(a, impl, reinterpret_cast<cudaStream_t>(stream));
}

int32_t b200_attention_backward(const void* q, const void* k, const void* v, const void* o, const float* lse,
                                const void* d_o, void* dq, void* dk, void* dv, float* delta_scratch, int32_t batch,
                                int32_t seq, int32_t n_heads, int32_t head_size, int32_t ldq, int32_t ldkv, int32_t ldo,
                                int32_t dtype, int32_t impl, b200_stream_t stream) {
  if (!q || !k || !v || !o || !lse || !d_o || !dq || !dk || !dv || !delta_scratch)
    return fail(B200_ERR_INVALID_ARG, "null operand");
  AttnBwdArgs a;
  a.f.q = q; a.f.k = k; a.f.v = v; a.f.o = const_cast<void*>(o); a.f.lse = const_cast<float*>(lse);
  a.f.batch = batch; a.f.seq = seq; a.f.n_heads = n_heads; a.f.head_size = head_size;
  a.f.ldq = ldq; a.f.ldkv = ldkv; a.f.ldo = ldo; a.f.dtype = dtype;
  a.d_o = d_o; a.lddo = ldo; a.dq = dq; a.dk = dk; a.dv = dv; a.lddq = ldq; a.lddkv = ldkv;
  a.delta = delta_scratch;
  return launch_attn_bwd(a, impl, reinterpret_cast<cudaStream_t>(stream));
}

int32_t b200_argmax(const float* logits, int32_t rows, int32_t cols, int32_t ld, int32_t* out_tokens,
                    b200_stream_t stream) {
  if (!logits || !out_tokens) return fail(B200_ERR_INVALID_ARG, "null argument");
  return launch_argmax_rows(logits, rows, cols, ld, out_tokens, reinterpret_cast<cudaStream_t>(stream));
}

int32_t b200_selftest_bounded_wait(int64_t budget_cycles, uint32_t* reached_end_device, b200_stream_t stream) {
  if (!reached_end_device) return fail(B200_ERR_INVALID_ARG, "null argument");
  if (budget_cycles <= 0 || budget_cycles > 4000000000LL) return fail(B200_ERR_INVALID_ARG, "budget out of range");
  return launch_bounded_wait_selftest(budget_cycles, reached_end_device, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
