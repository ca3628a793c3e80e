// Reverse mode of the llama forward with respect to every weight leaf.
//
// The rules applied per block are the ones the reference's AD engine composes
// from its per-op table (Implementations/HLODerivatives.td): dot_general
// (:1166-1178) gives dX = dY W and dW = dY^T X; mul/div/rsqrt (:1221, :1133,
// :1283) give the RMSNorm rule; exp/div/reduce give the softmax rule used by
// the attention backward; logistic/mul give SwiGLU; add (:964-970) fans the
// residual cotangent out to both branches.
#include "attention.cuh"
#include "elementwise.cuh"
#include "gemm_epilogue.cuh"
#include "plan.cuh"

namespace b200 {

struct BwdWs {
  float* dx; void* dxb; void* dlog; void* dhg; void* dgu; void* d_o; void* dqkv; float* delta; float* dg_part;
  void* splitk; size_t splitk_bytes;
  int n_parts;
};

static void carve_backward(const B200Plan& p, Arena& a, int B, int S, BwdWs* w) {
  const size_t T = (size_t)B * S, es = p.esize;
  w->dx = a.take<float>(T * p.d * 4);
  w->dxb = a.take(T * p.d * es);
  w->dlog = p.dtype == B200_F32 ? nullptr : a.take(T * p.V * es);
  w->dhg = a.take(T * p.h * es);
  w->dgu = a.take(T * 2 * p.h * es);
  w->d_o = a.take(T * p.d * es);
  w->dqkv = a.take(T * 3 * p.d * es);
  w->delta = a.take<float>((size_t)B * p.H * S * 4);
  w->n_parts = rmsnorm_bwd_parts((int)T);
  w->dg_part = a.take<float>((size_t)w->n_parts * p.d * 4);
  // K-split partials of the weight-gradient GEMMs: room for at least one full fp32 copy of the largest gradient
  // (the classifier's, V x d), so that every weight gradient can take the K-range kernel
  w->splitk_bytes = (size_t)64 << 20;
  const size_t largest = align_up((size_t)p.V * p.d * 4, 256);
  const size_t widest = align_up((size_t)2 * p.h * p.d * 4, 256);
  if (w->splitk_bytes < largest) w->splitk_bytes = largest;
  if (w->splitk_bytes < widest) w->splitk_bytes = widest;
  w->splitk = a.take(w->splitk_bytes);
}

size_t backward_workspace_bytes(const B200Plan& p, int B, int S) {
  Arena a(nullptr);
  BwdWs w;
  carve_backward(p, a, B, S, &w);
  return a.used;
}

// Y[M,N] (+)= op(A) op(B)^T into `out` of dtype out_dtype.
static int32_t gemm(const B200Plan& p, const BwdWs& ws, const void* A, int lda, int ta, const void* Bm, int ldb, int tb,
                    int M, int N, int K, void* out, int ldo, int out_dtype, int accumulate, cudaStream_t stream) {
  GemmArgs g;
  g.splitk_scratch = ws.splitk; g.splitk_bytes = ws.splitk_bytes;
  g.A = A; g.B = Bm; g.M = M; g.N = N; g.K = K; g.lda = lda; g.ldb = ldb; g.ta = ta; g.tb = tb;
  g.in_dtype = p.dtype; g.out_dtype = out_dtype; g.kind = EPI_STORE;
  g.epi.out = out; g.epi.ldo = ldo; g.epi.accumulate = accumulate;
  return launch_gemm(g, p.gemm_impl, stream);
}

int32_t backward_impl(B200Plan* p, const int32_t* tokens, int B, int S, const uint8_t* w, const float* dlogits,
                      void* saved, float* grads, int accumulate, void* ws, size_t ws_bytes, cudaStream_t stream) {
  const int T = B * S, d = p->d, h = p->h, V = p->V, dt = p->dtype;
  const PackedLayout& wl = p->wlt;
  const PackedLayout& gl = p->gl;
  Arena sa(saved);
  FwdActs acts;
  carve_forward(*p, sa, B, S, true, &acts);
  Arena wa(ws);
  BwdWs b;
  carve_backward(*p, wa, B, S, &b);
  if (wa.used > ws_bytes) return fail(B200_ERR_WORKSPACE, "backward needs %zu workspace bytes, got %zu", wa.used, ws_bytes);
  uint8_t* g = reinterpret_cast<uint8_t*>(grads);
  auto gf = [&](size_t off) { return reinterpret_cast<float*>(g + off); };
  const float* g_att = reinterpret_cast<const float*>(w + wl.g_att);
  const float* g_ffn = reinterpret_cast<const float*>(w + wl.g_ffn);
  const float* g_fin = reinterpret_cast<const float*>(w + wl.g_final);

  if (!accumulate) B200_TRY(launch_zero_f32(gf(gl.emb), (size_t)V * d, stream));

  // logits = xf wcls^T
  const void* dlog = dlogits;
  if (dt != B200_F32) {
    B200_TRY(launch_convert(dlogits, B200_F32, b.dlog, dt, (size_t)T * V, stream));
    dlog = b.dlog;
  }
  B200_TRY(gemm(*p, b, dlog, V, 1, acts.fin.xf, d, 1, V, d, T, gf(gl.wcls), d, B200_F32, accumulate, stream));
  B200_TRY(gemm(*p, b, dlog, V, 0, w + wl.wcls_t, V, 0, T, d, V, b.dxb, d, dt, 0, stream));
  B200_TRY(launch_rmsnorm_bwd(acts.fin.x_last, g_fin, acts.fin.rinv_f, b.dxb, dt, b.dx, 0, b.dxb, b.dg_part, b.n_parts, T, d,
                              stream));
  B200_TRY(launch_colsum_parts(b.dg_part, b.n_parts, d, gf(gl.g_final), accumulate, stream));

  for (int l = p->L - 1; l >= 0; --l) {
    const LayerActs& a = acts.layer[l];
    const LayerOffsets& o = wl.layer[l];
    const LayerOffsets& go = gl.layer[l];
    // ---- feed-forward block: x_out = x_mid + hg W2^T  (b.dxb holds dx in the config dtype: written by the
    //      RMSNorm backward that produced dx)
    B200_TRY(gemm(*p, b, b.dxb, d, 1, a.hg, h, 1, d, h, T, gf(go.w2), h, B200_F32, accumulate, stream));
    B200_TRY(gemm(*p, b, b.dxb, d, 0, w + o.w2_t, d, 0, T, h, d, b.dhg, h, dt, 0, stream));
    B200_TRY(launch_swiglu_bwd(a.gate, a.up, b.dhg, b.dgu, dt, T, h, stream));
    B200_TRY(gemm(*p, b, b.dgu, 2 * h, 1, a.xb2, d, 1, 2 * h, d, T, gf(go.w13), d, B200_F32, accumulate, stream));
    B200_TRY(gemm(*p, b, b.dgu, 2 * h, 0, w + o.w13_t, 2 * h, 0, T, d, 2 * h, b.dxb, d, dt, 0, stream));
    B200_TRY(launch_rmsnorm_bwd(a.x_mid, g_ffn + (size_t)l * d, a.rinv2, b.dxb, dt, b.dx, 1, b.dxb, b.dg_part, b.n_parts, T, d,
                                stream));
    B200_TRY(launch_colsum_parts(b.dg_part, b.n_parts, d, gf(gl.g_ffn) + (size_t)l * d, accumulate, stream));
    // ---- attention block: x_mid = x_in + o Wo^T
    B200_TRY(gemm(*p, b, b.dxb, d, 1, a.o, d, 1, d, d, T, gf(go.wo), d, B200_F32, accumulate, stream));
    B200_TRY(gemm(*p, b, b.dxb, d, 0, w + o.wo_t, d, 0, T, d, d, b.d_o, d, dt, 0, stream));
    {
      AttnBwdArgs ab;
      const uint8_t* base = reinterpret_cast<const uint8_t*>(a.qkv);
      uint8_t* dbase = reinterpret_cast<uint8_t*>(b.dqkv);
      ab.f.q = base; ab.f.k = base + (size_t)d * p->esize; ab.f.v = base + (size_t)2 * d * p->esize;
      ab.f.o = a.o; ab.f.lse = a.lse;
      ab.f.batch = B; ab.f.seq = S; ab.f.n_heads = p->H; ab.f.head_size = p->hs;
      ab.f.ldq = 3 * d; ab.f.ldkv = 3 * d; ab.f.ldo = d; ab.f.dtype = dt;
      ab.d_o = b.d_o; ab.lddo = d;
      ab.dq = dbase; ab.dk = dbase + (size_t)d * p->esize; ab.dv = dbase + (size_t)2 * d * p->esize;
      ab.lddq = 3 * d; ab.lddkv = 3 * d;
      ab.delta = b.delta;
      B200_TRY(launch_attn_bwd(ab, p->attn_impl, stream));
    }
    B200_TRY(launch_rope_bwd(b.dqkv, dt, 3 * d, T, 2 * d, p->hs, S, p->rope_cos, p->rope_sin, stream));
    B200_TRY(gemm(*p, b, b.dqkv, 3 * d, 1, a.xb, d, 1, 3 * d, d, T, gf(go.wqkv), d, B200_F32, accumulate, stream));
    B200_TRY(gemm(*p, b, b.dqkv, 3 * d, 0, w + o.wqkv_t, 3 * d, 0, T, d, 3 * d, b.dxb, d, dt, 0, stream));
    B200_TRY(launch_rmsnorm_bwd(a.x_in, g_att + (size_t)l * d, a.rinv1, b.dxb, dt, b.dx, 1, b.dxb, b.dg_part, b.n_parts, T, d,
                                stream));
    B200_TRY(launch_colsum_parts(b.dg_part, b.n_parts, d, gf(gl.g_att) + (size_t)l * d, accumulate, stream));
  }
  return launch_embed_bwd(tokens, b.dx, gf(gl.emb), T, d, V, stream);
}

}  // namespace b200

using namespace b200;

extern "C" {

int32_t b200_backward(B200Plan* p, const int32_t* tokens, int32_t B, int32_t S, const void* packed_w,
                      const float* dlogits, const void* saved, float* grads, int32_t accumulate, void* ws,
                      size_t ws_bytes, b200_stream_t stream) {
  if (!p) return fail(B200_ERR_INVALID_ARG, "plan is null");
  if (p->tp_size != 1) return fail(B200_ERR_UNSUPPORTED, "backward runs data-parallel only (tp_size must be 1)");
  if (B <= 0 || S <= 0 || S > p->cfg.seq_len) return fail(B200_ERR_BAD_SHAPE, "bad batch=%d seq=%d", B, S);
  if (!tokens || !packed_w || !dlogits || !saved || !grads || !ws) return fail(B200_ERR_INVALID_ARG, "null argument");
  if (!aligned16(packed_w) || !aligned16(dlogits) || !aligned16(saved) || !aligned16(grads) || !aligned16(ws))
    return fail(B200_ERR_MISALIGNED, "buffers must be 16-byte aligned");
  return backward_impl(p, tokens, B, S, reinterpret_cast<const uint8_t*>(packed_w), dlogits, const_cast<void*>(saved),
                       grads, accumulate, ws, ws_bytes, reinterpret_cast<cudaStream_t>(stream));
}

// Packed gradients -> per-leaf gradients (fp32, B200Leaf order, full shapes).
int32_t b200_unpack_grads(const B200Plan* p, const float* grads, float* const* leaves, b200_stream_t stream_) {
  if (!p || !grads || !leaves) return fail(B200_ERR_INVALID_ARG, "null argument");
  if (p->tp_size != 1) return fail(B200_ERR_UNSUPPORTED, "gradients exist only for tp_size == 1");
  for (int i = 0; i < B200_NUM_LEAVES; ++i)
    if (!leaves[i] || !aligned16(leaves[i])) return fail(B200_ERR_INVALID_ARG, "gradient leaf %d is null or misaligned", i);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const PackedLayout& gl = p->gl;
  const uint8_t* g = reinterpret_cast<const uint8_t*>(grads);
  const int d = p->d, h = p->h, L = p->L, V = p->V;
  auto cp = [&](const void* src, int sld, float* dst, int dld, int rows, int cols) {
    return launch_copy_rows(src, B200_F32, sld, dst, B200_F32, dld, rows, cols, rows, rows, 0, s);
  };
  B200_TRY(cp(g + gl.g_att, d, leaves[B200_LEAF_RMS_ATT], d, L, d));
  B200_TRY(cp(g + gl.g_ffn, d, leaves[B200_LEAF_RMS_FFN], d, L, d));
  B200_TRY(cp(g + gl.g_final, d, leaves[B200_LEAF_RMS_FINAL], d, 1, d));
  B200_TRY(cp(g + gl.emb, d, leaves[B200_LEAF_TOK_EMB], d, V, d));
  B200_TRY(cp(g + gl.wcls, d, leaves[B200_LEAF_WCLS], d, V, d));
  for (int l = 0; l < L; ++l) {
    const LayerOffsets& o = gl.layer[l];
    const size_t dd = (size_t)l * d * d, hd = (size_t)l * h * d;
    const float* qkv = reinterpret_cast<const float*>(g + o.wqkv);
    B200_TRY(cp(qkv, d, leaves[B200_LEAF_WQ] + dd, d, d, d));
    B200_TRY(cp(qkv + (size_t)d * d, d, leaves[B200_LEAF_WK] + dd, d, d, d));
    B200_TRY(cp(qkv + (size_t)2 * d * d, d, leaves[B200_LEAF_WV] + dd, d, d, d));
    B200_TRY(cp(g + o.wo, d, leaves[B200_LEAF_WO] + dd, d, d, d));
    B200_TRY(cp(g + o.w2, h, leaves[B200_LEAF_W2] + hd, h, d, h));
    // de-interleave the [8 x w1 | 8 x w3] row groups: packed row (i/8)*16 + i%8 -> w1 row i
    const float* w13 = reinterpret_cast<const float*>(g + o.w13);
    for (int half = 0; half < 2; ++half) {
      float* dst = leaves[half ? B200_LEAF_W3 : B200_LEAF_W1] + hd;
      // copy 8-row groups: source rows start at half*8 with a stride of 16 rows
      B200_CUDA_OK(cudaMemcpy2DAsync(dst, (size_t)8 * d * 4, w13 + (size_t)half * 8 * d, (size_t)16 * d * 4,
                                     (size_t)8 * d * 4, h / 8, cudaMemcpyDeviceToDevice, s));
    }
  }
  return B200_OK;
}

}  // extern "C"
