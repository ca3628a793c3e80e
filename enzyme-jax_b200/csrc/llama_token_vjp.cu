// Reverse mode of the reference's own call shape: one residual vector against a
// cache of `pos` rows per layer (test/llama.py:35-238), differentiated with
// respect to EVERY input as the reference's test does (test/llama.py:315-317 and
// test/test_utils.py:505-514: x, every weight leaf, key_cache and value_cache).
//
// The step is run as a sequence of pos + 1 attention rows of which only the
// last is live: rows 0..pos-1 of K and V are the cache rows (inputs, taken as
// they are: the reference appends the new row after the rotation, :161-175), their
// query rows are zero and their output cotangent is zero, so the attention
// forward / backward kernels of the sequence path give exactly o, dq, dk_new,
// dv_new of the new token and dK, dV of the cache rows.  Everything else works on
// one row with the kernels and rules of the sequence backward
// (Implementations/HLODerivatives.td:964-1339 composed per block).
//
// The returned hidden state does not depend on wcls (the logits projection is
// commented out in the reference, test/llama.py:236) nor on an embedding table, so
// their gradients are identically zero - what the reference materialises for
// arguments JAX drops as dead (primitives.py:733-744, :1550-1569).
#include "attention.cuh"
#include "elementwise.cuh"
#include "gemm_epilogue.cuh"
#include "plan.cuh"
#include "token_path.cuh"

namespace b200 {

void carve_token(const B200Plan& p, Arena& a, int S, TokWs* w) {
  const size_t es = p.esize, d = p.d, h = p.h;
  w->layer.assign(p.L, TokLayer{});
  float* x_next = nullptr;
  for (int l = 0; l < p.L; ++l) {
    TokLayer& t = w->layer[l];
    t.x_in = x_next ? x_next : a.take<float>(d * 4);
    t.xb = a.take(d * es);
    t.rinv1 = a.take<float>(4);
    t.qkv = a.take((size_t)S * 3 * d * es);
    t.o = a.take((size_t)S * d * es);
    t.lse = a.take<float>((size_t)p.H * S * 4);
    t.x_mid = a.take<float>(d * 4);
    t.xb2 = a.take(d * es);
    t.rinv2 = a.take<float>(4);
    t.gate = a.take(h * es);
    t.up = a.take(h * es);
    t.hg = a.take(h * es);
    x_next = a.take<float>(d * 4);
  }
  w->x_last = x_next;
  w->rinv_f = a.take<float>(4);
  w->dx = a.take<float>(d * 4);
  w->dxb = a.take(d * es);
  w->dhg = a.take(h * es);
  w->dgu = a.take(2 * h * es);
  w->d_o = a.take((size_t)S * d * es);
  w->dqkv = a.take((size_t)S * 3 * d * es);
  w->delta = a.take<float>((size_t)p.H * S * 4);
  w->n_parts = rmsnorm_bwd_parts(1);
  w->dg_part = a.take<float>((size_t)w->n_parts * d * 4);
  w->splitk_bytes = (size_t)4 << 20;
  w->splitk = a.take(w->splitk_bytes);
}

namespace {

int32_t gemm_epi(const B200Plan& p, const TokWs& ws, const void* A, int lda, const void* W, int ldw, int N, int K,
                 int kind, int out_dtype, const EpiParams& epi, cudaStream_t stream) {
  GemmArgs g;
  g.splitk_scratch = ws.splitk; g.splitk_bytes = ws.splitk_bytes;
  g.A = A; g.B = W; g.M = 1; g.N = N; g.K = K; g.lda = lda; g.ldb = ldw;
  g.in_dtype = p.dtype; g.out_dtype = out_dtype; g.kind = kind; g.epi = epi;
  return launch_gemm(g, p.gemm_impl, stream);
}

// Y[M,N] = op(A) op(B)^T, plain store
int32_t gemm_plain(const B200Plan& p, const TokWs& ws, const void* A, int lda, int ta, const void* Bm, int ldb, int tb,
                   int M, int N, int K, void* out, int ldo, int out_dtype, cudaStream_t stream) {
  GemmArgs g;
  g.splitk_scratch = ws.splitk; g.splitk_bytes = ws.splitk_bytes;
  g.A = A; g.B = Bm; g.M = M; g.N = N; g.K = K; g.lda = lda; g.ldb = ldb; g.ta = ta; g.tb = tb;
  g.in_dtype = p.dtype; g.out_dtype = out_dtype; g.kind = EPI_STORE;
  g.epi.out = out; g.epi.ldo = ldo;
  return launch_gemm(g, p.gemm_impl, stream);
}

}  // namespace

size_t token_vjp_workspace_bytes(const B200Plan& p, int pos) {
  Arena a(nullptr);
  TokWs w;
  carve_token(p, a, pos + 1, &w);
  return a.used;
}

// Forward of the reference call shape, keeping in `t` what the backward needs.  `hidden` receives the final-normed
// hidden state (fp32 [d]).
int32_t token_forward_run(B200Plan* p, const TokWs& t, const float* x, const void* key_cache,
                                 const void* value_cache, int pos, const uint8_t* w, const PackedLayout& wl,
                                 float* hidden, cudaStream_t stream) {
  const int d = p->d, h = p->h, dt = p->dtype, S = pos + 1;
  const size_t es = p->esize;
  const float* g_att = reinterpret_cast<const float*>(w + wl.g_att);
  const float* g_ffn = reinterpret_cast<const float*>(w + wl.g_ffn);
  const float* g_fin = reinterpret_cast<const float*>(w + wl.g_final);
  const float eps = p->cfg.rms_eps;
  B200_CUDA_OK(cudaMemcpyAsync(t.layer[0].x_in, x, (size_t)d * 4, cudaMemcpyDeviceToDevice, stream));
  for (int l = 0; l < p->L; ++l) {
    const TokLayer& a = t.layer[l];
    const LayerOffsets& o = wl.layer[l];
    float* x_out = l + 1 < p->L ? t.layer[l + 1].x_in : t.x_last;
    uint8_t* qkv = reinterpret_cast<uint8_t*>(a.qkv);
    uint8_t* row_new = qkv + (size_t)pos * 3 * d * es;
    B200_TRY(launch_rmsnorm(a.x_in, g_att + (size_t)l * d, a.xb, a.rinv1, 1, d, eps, dt, stream));
    {
      EpiParams e;
      e.out = row_new; e.ldo = 3 * d;
      e.rope_cos = p->rope_cos; e.rope_sin = p->rope_sin;
      e.seq_len = 1; e.pos_base = pos; e.head_size = p->hs; e.rope_cols = 2 * d;
      B200_TRY(gemm_epi(*p, t, a.xb, d, w + o.wqkv, d, 3 * d, d, EPI_ROPE, dt, e, stream));
    }
    if (pos > 0) {
      // rows 0..pos-1: zero queries, the cache rows as keys and values
      B200_CUDA_OK(cudaMemset2DAsync(qkv, (size_t)3 * d * es, 0, (size_t)d * es, pos, stream));
      const uint8_t* kc = reinterpret_cast<const uint8_t*>(key_cache) + (size_t)l * pos * d * es;
      const uint8_t* vc = reinterpret_cast<const uint8_t*>(value_cache) + (size_t)l * pos * d * es;
      B200_CUDA_OK(cudaMemcpy2DAsync(qkv + (size_t)d * es, (size_t)3 * d * es, kc, (size_t)d * es, (size_t)d * es, pos,
                                     cudaMemcpyDeviceToDevice, stream));
      B200_CUDA_OK(cudaMemcpy2DAsync(qkv + (size_t)2 * d * es, (size_t)3 * d * es, vc, (size_t)d * es, (size_t)d * es, pos,
                                     cudaMemcpyDeviceToDevice, stream));
    }
    {
      AttnArgs at;
      at.q = qkv; at.k = qkv + (size_t)d * es; at.v = qkv + (size_t)2 * d * es;
      at.o = a.o; at.lse = a.lse;
      at.batch = 1; at.seq = S; at.n_heads = p->H; at.head_size = p->hs;
      at.ldq = 3 * d; at.ldkv = 3 * d; at.ldo = d; at.dtype = dt;
      B200_TRY(launch_attn_fwd(at, p->attn_impl, stream));
    }
    {
      EpiParams e;
      e.out = a.x_mid; e.ldo = d; e.resid_in = a.x_in;
      B200_TRY(gemm_epi(*p, t, reinterpret_cast<uint8_t*>(a.o) + (size_t)pos * d * es, d, w + o.wo, d, d, d, EPI_RESID,
                        B200_F32, e, stream));
    }
    B200_TRY(launch_rmsnorm(a.x_mid, g_ffn + (size_t)l * d, a.xb2, a.rinv2, 1, d, eps, dt, stream));
    {
      EpiParams e;
      e.out = a.hg; e.ldo = h; e.out_gate = a.gate; e.out_up = a.up;
      B200_TRY(gemm_epi(*p, t, a.xb2, d, w + o.w13, d, 2 * h, d, EPI_SWIGLU, dt, e, stream));
    }
    {
      EpiParams e;
      e.out = x_out; e.ldo = d; e.resid_in = a.x_mid;
      B200_TRY(gemm_epi(*p, t, a.hg, h, w + o.w2, h, d, h, EPI_RESID, B200_F32, e, stream));
    }
  }
  return launch_rmsnorm(t.x_last, g_fin, hidden, t.rinv_f, 1, d, eps, B200_F32, stream);
}

int32_t token_forward_impl(B200Plan* p, const float* x, const void* key_cache, const void* value_cache, int pos,
                           const uint8_t* w, float* hidden_out, void* ws, size_t ws_bytes, cudaStream_t stream) {
  Arena wa(ws);
  TokWs t;
  carve_token(*p, wa, pos + 1, &t);
  if (wa.used > ws_bytes) return fail(B200_ERR_WORKSPACE, "token forward needs %zu workspace bytes, got %zu", wa.used, ws_bytes);
  return token_forward_run(p, t, x, key_cache, value_cache, pos, w, p->wl, hidden_out, stream);
}

int32_t token_vjp_impl(B200Plan* p, const float* x, const void* key_cache, const void* value_cache, int pos,
                       const uint8_t* w, const float* d_hidden, float* hidden_out, float* dx_out, float* grads,
                       float* dkc, float* dvc, void* ws, size_t ws_bytes, cudaStream_t stream) {
  const int d = p->d, h = p->h, dt = p->dtype, S = pos + 1;
  const size_t es = p->esize;
  const PackedLayout& wl = p->wlt;
  const PackedLayout& gl = p->gl;
  Arena wa(ws);
  TokWs t;
  carve_token(*p, wa, S, &t);
  if (wa.used > ws_bytes) return fail(B200_ERR_WORKSPACE, "token VJP needs %zu workspace bytes, got %zu", wa.used, ws_bytes);
  const float* g_att = reinterpret_cast<const float*>(w + wl.g_att);
  const float* g_ffn = reinterpret_cast<const float*>(w + wl.g_ffn);
  const float* g_fin = reinterpret_cast<const float*>(w + wl.g_final);
  const float* cos_p = p->rope_cos + (size_t)pos * (p->hs / 2);
  const float* sin_p = p->rope_sin + (size_t)pos * (p->hs / 2);

  // ---- forward, keeping what the backward needs; when the caller does not want the hidden state it goes to scratch
  B200_TRY(token_forward_run(p, t, x, key_cache, value_cache, pos, w, wl, hidden_out ? hidden_out : t.dx, stream));

  // ---- backward ----
  uint8_t* g = reinterpret_cast<uint8_t*>(grads);
  auto gf = [&](size_t off) { return reinterpret_cast<float*>(g + off); };
  B200_TRY(launch_zero_f32(grads, gl.total / 4, stream));  // embedding and wcls stay zero: dead arguments
  B200_TRY(launch_convert(d_hidden, B200_F32, t.dxb, dt, (size_t)d, stream));
  B200_TRY(launch_rmsnorm_bwd(t.x_last, g_fin, t.rinv_f, t.dxb, dt, t.dx, 0, t.dxb, t.dg_part, t.n_parts, 1, d, stream));
  B200_TRY(launch_colsum_parts(t.dg_part, t.n_parts, d, gf(gl.g_final), 0, stream));
  for (int l = p->L - 1; l >= 0; --l) {
    const TokLayer& a = t.layer[l];
    const LayerOffsets& o = wl.layer[l];
    const LayerOffsets& go = gl.layer[l];
    // feed-forward block
    B200_TRY(gemm_plain(*p, t, t.dxb, d, 1, a.hg, h, 1, d, h, 1, gf(go.w2), h, B200_F32, stream));
    B200_TRY(gemm_plain(*p, t, t.dxb, d, 0, w + o.w2_t, d, 0, 1, h, d, t.dhg, h, dt, stream));
    B200_TRY(launch_swiglu_bwd(a.gate, a.up, t.dhg, t.dgu, dt, 1, h, stream));
    B200_TRY(gemm_plain(*p, t, t.dgu, 2 * h, 1, a.xb2, d, 1, 2 * h, d, 1, gf(go.w13), d, B200_F32, stream));
    B200_TRY(gemm_plain(*p, t, t.dgu, 2 * h, 0, w + o.w13_t, 2 * h, 0, 1, d, 2 * h, t.dxb, d, dt, stream));
    B200_TRY(launch_rmsnorm_bwd(a.x_mid, g_ffn + (size_t)l * d, a.rinv2, t.dxb, dt, t.dx, 1, t.dxb, t.dg_part, t.n_parts,
                                1, d, stream));
    B200_TRY(launch_colsum_parts(t.dg_part, t.n_parts, d, gf(gl.g_ffn) + (size_t)l * d, 0, stream));
    // attention block: only the last row of the output carries a cotangent
    uint8_t* d_o = reinterpret_cast<uint8_t*>(t.d_o);
    uint8_t* dqkv = reinterpret_cast<uint8_t*>(t.dqkv);
    uint8_t* qkv = reinterpret_cast<uint8_t*>(a.qkv);
    const uint8_t* o_new = reinterpret_cast<const uint8_t*>(a.o) + (size_t)pos * d * es;
    B200_TRY(gemm_plain(*p, t, t.dxb, d, 1, o_new, d, 1, d, d, 1, gf(go.wo), d, B200_F32, stream));
    B200_CUDA_OK(cudaMemsetAsync(d_o, 0, (size_t)S * d * es, stream));
    B200_TRY(gemm_plain(*p, t, t.dxb, d, 0, w + o.wo_t, d, 0, 1, d, d, d_o + (size_t)pos * d * es, d, dt, stream));
    {
      AttnBwdArgs ab;
      ab.f.q = qkv; ab.f.k = qkv + (size_t)d * es; ab.f.v = qkv + (size_t)2 * d * es;
      ab.f.o = a.o; ab.f.lse = a.lse;
      ab.f.batch = 1; ab.f.seq = S; ab.f.n_heads = p->H; ab.f.head_size = p->hs;
      ab.f.ldq = 3 * d; ab.f.ldkv = 3 * d; ab.f.ldo = d; ab.f.dtype = dt;
      ab.d_o = d_o; ab.lddo = d;
      ab.dq = dqkv; ab.dk = dqkv + (size_t)d * es; ab.dv = dqkv + (size_t)2 * d * es;
      ab.lddq = 3 * d; ab.lddkv = 3 * d;
      ab.delta = t.delta;
      B200_TRY(launch_attn_bwd(ab, p->attn_impl, stream));
    }
    if (pos > 0) {  // cotangents of the cache rows (they entered after the rotation: no inverse rotation)
      B200_TRY(launch_copy_rows(dqkv + (size_t)d * es, dt, 3 * d, dkc + (size_t)l * pos * d, B200_F32, d, pos, d, pos,
                                pos, 0, stream));
      B200_TRY(launch_copy_rows(dqkv + (size_t)2 * d * es, dt, 3 * d, dvc + (size_t)l * pos * d, B200_F32, d, pos, d,
                                pos, pos, 0, stream));
    }
    uint8_t* drow = dqkv + (size_t)pos * 3 * d * es;
    B200_TRY(launch_rope_bwd(drow, dt, 3 * d, 1, 2 * d, p->hs, 1, cos_p, sin_p, stream));
    B200_TRY(gemm_plain(*p, t, drow, 3 * d, 1, a.xb, d, 1, 3 * d, d, 1, gf(go.wqkv), d, B200_F32, stream));
    B200_TRY(gemm_plain(*p, t, drow, 3 * d, 0, w + o.wqkv_t, 3 * d, 0, 1, d, 3 * d, t.dxb, d, dt, stream));
    B200_TRY(launch_rmsnorm_bwd(a.x_in, g_att + (size_t)l * d, a.rinv1, t.dxb, dt, t.dx, 1, t.dxb, t.dg_part, t.n_parts,
                                1, d, stream));
    B200_TRY(launch_colsum_parts(t.dg_part, t.n_parts, d, gf(gl.g_att) + (size_t)l * d, 0, stream));
  }
  B200_CUDA_OK(cudaMemcpyAsync(dx_out, t.dx, (size_t)d * 4, cudaMemcpyDeviceToDevice, stream));
  return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" {

int32_t b200_token_vjp_workspace_bytes(const B200Plan* p, int32_t pos, size_t* bytes) {
  if (!p || !bytes) return fail(B200_ERR_INVALID_ARG, "null argument");
  if (pos < 0 || pos >= p->cfg.seq_len) return fail(B200_ERR_BAD_SHAPE, "pos=%d outside the plan's seq_len=%d", pos, p->cfg.seq_len);
  *bytes = token_vjp_workspace_bytes(*p, pos) + 256;
  return B200_OK;
}

// Sizes a compiler pass needs before any device exists (the types of the custom call's packed-weight operand and
// scratch result): the layout arithmetic of the plan without creating one.
int32_t b200_static_sizes(const B200LlamaConfig* cfg, int32_t with_transposed, int32_t pos, size_t* packed_bytes,
                          size_t* grad_bytes, size_t* token_workspace_bytes) {
  if (!cfg) return fail(B200_ERR_INVALID_ARG, "cfg is null");
  if (cfg->dim <= 0 || cfg->hidden_dim <= 0 || cfg->n_layers <= 0 || cfg->n_heads <= 0 || cfg->vocab_size <= 0 ||
      cfg->dim % cfg->n_heads || pos < 0)
    return fail(B200_ERR_BAD_SHAPE, "bad config");
  B200Plan p;
  p.cfg = *cfg;
  p.d = cfg->dim; p.h = cfg->hidden_dim; p.L = cfg->n_layers; p.H = cfg->n_heads; p.hs = cfg->dim / cfg->n_heads;
  p.V = cfg->vocab_size;
  p.d_loc = p.d; p.h_loc = p.h; p.V_loc = p.V; p.H_loc = p.H;
  p.dtype = cfg->dtype;
  p.esize = cfg->dtype == B200_BF16 ? 2 : 4;
  PackedLayout wl, gl;
  build_layout(p, p.esize, with_transposed != 0, &wl);
  build_layout(p, 4, false, &gl);
  if (packed_bytes) *packed_bytes = wl.total;
  if (grad_bytes) *grad_bytes = gl.total;
  if (token_workspace_bytes) *token_workspace_bytes = token_vjp_workspace_bytes(p, pos) + 256;
  return B200_OK;
}

int32_t b200_token_forward(B200Plan* p, const float* x, const void* key_cache, const void* value_cache, int32_t pos,
                           const void* packed_w, float* hidden_out, void* ws, size_t ws_bytes, b200_stream_t stream) {
  if (!p) return fail(B200_ERR_INVALID_ARG, "plan is null");
  if (p->tp_size != 1) return fail(B200_ERR_UNSUPPORTED, "the token forward over flat caches runs on one GPU (tp_size must be 1)");
  if (pos < 0 || pos >= p->cfg.seq_len) return fail(B200_ERR_BAD_SHAPE, "pos=%d outside the plan's seq_len=%d", pos, p->cfg.seq_len);
  if (!x || !packed_w || !hidden_out || !ws || (pos > 0 && (!key_cache || !value_cache)))
    return fail(B200_ERR_INVALID_ARG, "null argument");
  if (!aligned16(x) || !aligned16(packed_w) || !aligned16(hidden_out) || !aligned16(ws) ||
      (pos > 0 && (!aligned16(key_cache) || !aligned16(value_cache))))
    return fail(B200_ERR_MISALIGNED, "buffers must be 16-byte aligned");
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev != p->device) return fail(B200_ERR_INVALID_ARG, "wrong current device");
  return token_forward_impl(p, x, key_cache, value_cache, pos, reinterpret_cast<const uint8_t*>(packed_w), hidden_out, ws,
                            ws_bytes, reinterpret_cast<cudaStream_t>(stream));
}

int32_t b200_token_vjp(B200Plan* p, const float* x, const void* key_cache, const void* value_cache, int32_t pos,
                       const void* packed_w, const float* d_hidden, float* hidden_out, float* dx, float* grads,
                       float* d_key_cache, float* d_value_cache, void* ws, size_t ws_bytes, b200_stream_t stream) {
  if (!p) return fail(B200_ERR_INVALID_ARG, "plan is null");
  if (p->tp_size != 1) return fail(B200_ERR_UNSUPPORTED, "the token VJP runs on one GPU (tp_size must be 1)");
  if (pos < 0 || pos >= p->cfg.seq_len) return fail(B200_ERR_BAD_SHAPE, "pos=%d outside the plan's seq_len=%d", pos, p->cfg.seq_len);
  if (!x || !packed_w || !d_hidden || !dx || !grads || !ws) return fail(B200_ERR_INVALID_ARG, "null argument");
  if (pos > 0 && (!key_cache || !value_cache || !d_key_cache || !d_value_cache))
    return fail(B200_ERR_INVALID_ARG, "a cache of %d rows needs its four buffers", pos);
  if (!aligned16(x) || !aligned16(packed_w) || !aligned16(d_hidden) || !aligned16(dx) || !aligned16(grads) ||
      !aligned16(ws) || (pos > 0 && (!aligned16(key_cache) || !aligned16(value_cache) || !aligned16(d_key_cache) ||
                                     !aligned16(d_value_cache))) || (hidden_out && !aligned16(hidden_out)))
    return fail(B200_ERR_MISALIGNED, "buffers must be 16-byte aligned");
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev != p->device) return fail(B200_ERR_INVALID_ARG, "wrong current device");
  return token_vjp_impl(p, x, key_cache, value_cache, pos, reinterpret_cast<const uint8_t*>(packed_w), d_hidden,
                        hidden_out, dx, grads, d_key_cache, d_value_cache, ws, ws_bytes,
                        reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
