// Forward mode (JVP) of the llama forward: the tangent of the result for given tangents of the inputs.
//
// The reference's harness times and checks a `Forward` row, jax.jvp of the decorated function
// (test/test_utils.py:689-735); the per-op forward rules are the `fwd` expressions of
// Implementations/HLODerivatives.td:964-1339 (dot_general: d(A B) = dA B + A dB; mul / div / rsqrt / exp / logistic
// by the product and chain rules; add: the sum of the tangents; shape ops applied to the tangent).  Composed per
// fused block of the forward they give:
//   linear     Y = X W^T            dY = dX W^T + X dW^T          (two GEMMs, the second accumulating)
//   RMSNorm    y = g x r            dy = dg x r + g (dx r - x r^3/d sum_j x_j dx_j)
//   rotation   linear               the same rotation applied to the tangent
//   attention  O = softmax(S) V     dS = (dQ K^T + Q dK^T)/sqrt(hs);  dO = P (dS - rowsum(P dS)) V + P dV
//   SwiGLU     h = a s(a) b         dh = da b s (1 + a (1 - s)) + a s db
//   residual   x + f(x)             dx + df
// The primal activations come from a forward that kept them (the same buffers the reverse mode reads).  Two call
// shapes, as in the reverse mode: the token sequence (tangents of the weight leaves -> tangent of the logits) and the
// reference's own call (tangents of x, the weights and both caches -> tangent of the hidden state), which is run as
// pos + 1 attention rows of which the last is live (see llama_token_vjp.cu).
#include "attention.cuh"
#include "elementwise.cuh"
#include "gemm_epilogue.cuh"
#include "plan.cuh"
#include "token_path.cuh"

namespace b200 {

namespace {

// dy = dg x r + g (dx r - x r^3/d <x, dx>) per row; dg may be null (no gain tangent).
template <typename TOut>
__global__ void __launch_bounds__(256) rmsnorm_jvp_kernel(const float* __restrict__ x, const float* __restrict__ dx,
                                                          const float* __restrict__ gain, const float* __restrict__ dgain,
                                                          const float* __restrict__ rinv, TOut* __restrict__ dy,
                                                          int dim) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const float* xr = x + (size_t)row * dim;
  const float* dxr = dx + (size_t)row * dim;
  float dot = 0.f;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) dot = fmaf(xr[c], dxr[c], dot);
  dot = block_sum(dot, red);
  const float r = rinv[row];
  const float coef = r * r * r / (float)dim * dot;
  TOut* out = dy + (size_t)row * dim;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    float v = gain[c] * (dxr[c] * r - xr[c] * coef);
    if (dgain) v = fmaf(dgain[c] * xr[c], r, v);
    out[c] = from_f32<TOut>(v);
  }
}

// Rotates adjacent pairs of the first rope_cols columns by the POSITIVE angle of the row's position, in place.
template <typename T>
__global__ void rope_tangent_kernel(T* __restrict__ d, int ld, int rows, int rope_cols, int head_size, int seq_len,
                                    const float* __restrict__ cos_t, const float* __restrict__ sin_t) {
  const int c2n = rope_cols / 2;
  const size_t total = (size_t)rows * c2n;
  const int half = head_size >> 1;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / c2n), c = (int)(i % c2n) * 2;
    const int pos = r % seq_len;
    const int j = (c % head_size) >> 1;
    const float cj = cos_t[(size_t)pos * half + j], sj = sin_t[(size_t)pos * half + j];
    T* p = d + (size_t)r * ld + c;
    const float e = to_f32(p[0]), o = to_f32(p[1]);
    p[0] = from_f32<T>(cj * e - sj * o);
    p[1] = from_f32<T>(sj * e + cj * o);
  }
}

// dh = da b s (1 + a (1 - s)) + a s db, with (da, db) in the interleaved [8 gate | 8 up] column layout of the fused
// W1|W3 product.
template <typename T>
__global__ void swiglu_jvp_kernel(const T* __restrict__ gate, const T* __restrict__ up, const T* __restrict__ dgu,
                                  T* __restrict__ dh, int rows, int hidden) {
  const size_t total = (size_t)rows * hidden;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / hidden), c = (int)(i % hidden);
    const float a = to_f32(gate[i]), b = to_f32(up[i]);
    const T* t = dgu + (size_t)r * (2 * hidden) + (size_t)(c / 8) * 16 + (c % 8);
    const float da = to_f32(t[0]), db = to_f32(t[8]);
    const float s = 1.f / (1.f + exp_by_build(-a));
    dh[i] = from_f32<T>(da * b * s * (1.f + a * (1.f - s)) + a * s * db);
  }
}

// Tangent of causal attention.  One warp per (sequence, head, query row); a lane owns the dimensions lane, lane + 32,
// ... of the head; the two dot products of a key are warp sums.
template <typename T>
__global__ void __launch_bounds__(256) attn_jvp_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                       const T* __restrict__ v, const T* __restrict__ dq,
                                                       const T* __restrict__ dk, const T* __restrict__ dv,
                                                       const T* __restrict__ o, const float* __restrict__ lse,
                                                       T* __restrict__ d_o, int batch, int seq, int n_heads, int hs,
                                                       int ldq, int ldkv, int ldo, int lddq, int lddkv, float scale) {
  const int lane = threadIdx.x & 31;
  const long w = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long)batch * n_heads * seq) return;
  const int t = (int)(w % seq), h = (int)((w / seq) % n_heads), b = (int)(w / ((long)seq * n_heads));
  const size_t row = (size_t)b * seq + t;
  constexpr int MAXE = 4;  // head sizes up to 128
  float qe[MAXE], dqe[MAXE], acc[MAXE];
#pragma unroll
  for (int i = 0; i < MAXE; ++i) {
    const int e = lane + 32 * i;
    qe[i] = e < hs ? to_f32(q[row * ldq + h * hs + e]) : 0.f;
    dqe[i] = e < hs ? to_f32(dq[row * lddq + h * hs + e]) : 0.f;
    acc[i] = 0.f;
  }
  const float l = lse[((size_t)b * n_heads + h) * seq + t];
  float a_sum = 0.f;
  for (int u = 0; u <= t; ++u) {
    const size_t kr = (size_t)b * seq + u;
    float ke[MAXE], dke[MAXE];
    float s = 0.f, ds = 0.f;
#pragma unroll
    for (int i = 0; i < MAXE; ++i) {
      const int e = lane + 32 * i;
      ke[i] = e < hs ? to_f32(k[kr * ldkv + h * hs + e]) : 0.f;
      dke[i] = e < hs ? to_f32(dk[kr * lddkv + h * hs + e]) : 0.f;
      s = fmaf(qe[i], ke[i], s);
      ds = fmaf(dqe[i], ke[i], fmaf(qe[i], dke[i], ds));
    }
    s = warp_sum(s) * scale;
    ds = warp_sum(ds) * scale;
    const float p = exp_by_build(s - l);
    a_sum = fmaf(p, ds, a_sum);
#pragma unroll
    for (int i = 0; i < MAXE; ++i) {
      const int e = lane + 32 * i;
      if (e < hs) {
        const float ve = to_f32(v[kr * ldkv + h * hs + e]), dve = to_f32(dv[kr * lddkv + h * hs + e]);
        acc[i] = fmaf(p, fmaf(ds, ve, dve), acc[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAXE; ++i) {
    const int e = lane + 32 * i;
    if (e < hs) d_o[row * ldo + h * hs + e] = from_f32<T>(acc[i] - a_sum * to_f32(o[row * ldo + h * hs + e]));
  }
}

int grid1d(size_t n, int block) {
  size_t g = (n + block - 1) / block;
  const size_t cap = (size_t)sm_count() * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

int32_t launch_rmsnorm_jvp(const float* x, const float* dx, const float* gain, const float* dgain, const float* rinv,
                           void* dy, int rows, int dim, int out_dtype, cudaStream_t stream) {
  if (out_dtype == B200_F32)
    rmsnorm_jvp_kernel<float><<<rows, 256, 0, stream>>>(x, dx, gain, dgain, rinv, (float*)dy, dim);
  else
    rmsnorm_jvp_kernel<bf16><<<rows, 256, 0, stream>>>(x, dx, gain, dgain, rinv, (bf16*)dy, dim);
  B200_LAUNCH_OK("rmsnorm_jvp_kernel");
  return B200_OK;
}

int32_t launch_rope_tangent(void* d, int dtype, int ld, int rows, int rope_cols, int head_size, int seq_len,
                            const float* cos_t, const float* sin_t, cudaStream_t stream) {
  const int g = grid1d((size_t)rows * (rope_cols / 2), 256);
  if (dtype == B200_F32)
    rope_tangent_kernel<float><<<g, 256, 0, stream>>>((float*)d, ld, rows, rope_cols, head_size, seq_len, cos_t, sin_t);
  else
    rope_tangent_kernel<bf16><<<g, 256, 0, stream>>>((bf16*)d, ld, rows, rope_cols, head_size, seq_len, cos_t, sin_t);
  B200_LAUNCH_OK("rope_tangent_kernel");
  return B200_OK;
}

int32_t launch_swiglu_jvp(const void* gate, const void* up, const void* dgu, void* dh, int dtype, int rows, int hidden,
                          cudaStream_t stream) {
  const int g = grid1d((size_t)rows * hidden, 256);
  if (dtype == B200_F32)
    swiglu_jvp_kernel<float><<<g, 256, 0, stream>>>((const float*)gate, (const float*)up, (const float*)dgu, (float*)dh,
                                                     rows, hidden);
  else
    swiglu_jvp_kernel<bf16><<<g, 256, 0, stream>>>((const bf16*)gate, (const bf16*)up, (const bf16*)dgu, (bf16*)dh, rows,
                                                    hidden);
  B200_LAUNCH_OK("swiglu_jvp_kernel");
  return B200_OK;
}

// q, k, v and their tangents: [batch*seq, ld] with heads side by side, as the forward attention takes them.
int32_t launch_attn_jvp(const void* qkv, const void* dqkv, const void* o, const float* lse, void* d_o, int batch, int seq,
                        int n_heads, int hs, int d, int dtype, cudaStream_t stream) {
  if (hs > 128) return fail(B200_ERR_BAD_SHAPE, "attention tangent: head size %d exceeds 128", hs);
  const long warps = (long)batch * n_heads * seq;
  const int blocks = (int)((warps + 7) / 8);
  const float scale = 1.f / sqrtf((float)hs);
  const size_t es = dtype == B200_BF16 ? 2 : 4;
  const uint8_t* b0 = reinterpret_cast<const uint8_t*>(qkv);
  const uint8_t* d0 = reinterpret_cast<const uint8_t*>(dqkv);
  if (dtype == B200_F32)
    attn_jvp_kernel<float><<<blocks, 256, 0, stream>>>(
        (const float*)b0, (const float*)(b0 + d * es), (const float*)(b0 + 2 * d * es), (const float*)d0,
        (const float*)(d0 + d * es), (const float*)(d0 + 2 * d * es), (const float*)o, lse, (float*)d_o, batch, seq,
        n_heads, hs, 3 * d, 3 * d, d, 3 * d, 3 * d, scale);
  else
    attn_jvp_kernel<bf16><<<blocks, 256, 0, stream>>>(
        (const bf16*)b0, (const bf16*)(b0 + d * es), (const bf16*)(b0 + 2 * d * es), (const bf16*)d0,
        (const bf16*)(d0 + d * es), (const bf16*)(d0 + 2 * d * es), (const bf16*)o, lse, (bf16*)d_o, batch, seq, n_heads,
        hs, 3 * d, 3 * d, d, 3 * d, 3 * d, scale);
  B200_LAUNCH_OK("attn_jvp_kernel");
  return B200_OK;
}

struct JvpWs {
  float* dx; void* dxb; void* dqkv; void* d_o; void* dgu; void* dhg;
  void* splitk; size_t splitk_bytes;
};

void carve_jvp(const B200Plan& p, Arena& a, size_t T, size_t S_att, JvpWs* w) {
  const size_t es = p.esize;
  w->dx = a.take<float>(T * p.d * 4);
  w->dxb = a.take(T * p.d * es);
  w->dqkv = a.take(S_att * 3 * p.d * es);
  w->d_o = a.take(S_att * p.d * es);
  w->dgu = a.take(T * 2 * p.h * es);
  w->dhg = a.take(T * p.h * es);
  w->splitk_bytes = (size_t)16 << 20;
  w->splitk = a.take(w->splitk_bytes);
}

// out (+)= A[M,K] W[N,K]^T, plain store of dtype out_dtype
int32_t lin(const B200Plan& p, const JvpWs& ws, const void* A, int lda, const void* W, int ldw, int M, int N, int K,
            void* out, int ldo, int out_dtype, int accumulate, cudaStream_t stream) {
  GemmArgs g;
  g.splitk_scratch = ws.splitk; g.splitk_bytes = ws.splitk_bytes;
  g.A = A; g.B = W; g.M = M; g.N = N; g.K = K; g.lda = lda; g.ldb = ldw;
  g.in_dtype = p.dtype; g.out_dtype = out_dtype; g.kind = EPI_STORE;
  g.epi.out = out; g.epi.ldo = ldo; g.epi.accumulate = accumulate;
  return launch_gemm(g, p.gemm_impl, stream);
}

// x_out = x_in + A W^T (fp32 residual stream; in place when x_out == x_in)
int32_t lin_resid(const B200Plan& p, const JvpWs& ws, const void* A, int lda, const void* W, int ldw, int M, int K,
                  const float* x_in, float* x_out, cudaStream_t stream) {
  GemmArgs g;
  g.splitk_scratch = ws.splitk; g.splitk_bytes = ws.splitk_bytes;
  g.A = A; g.B = W; g.M = M; g.N = p.d; g.K = K; g.lda = lda; g.ldb = ldw;
  g.in_dtype = p.dtype; g.out_dtype = B200_F32; g.kind = EPI_RESID;
  g.epi.out = x_out; g.epi.ldo = p.d; g.epi.resid_in = x_in;
  return launch_gemm(g, p.gemm_impl, stream);
}

// The tangent of one layer given the layer's primal activations.  T live rows (the rows whose residual stream
// exists), attention over `S_att` rows per sequence of which the live rows are the LAST T / batch of each sequence
// when S_att > T / batch never happens for the sequence form (S_att == seq) and is pos + 1 with one live row for the
// reference call shape; `live0` is the first live attention row (0 or pos).
struct LayerPrimal {
  const float* x_in; const void* xb; const float* rinv1; const void* qkv; const void* o; const float* lse;
  const float* x_mid; const void* xb2; const float* rinv2; const void* gate; const void* up; const void* hg;
};

int32_t layer_tangent(const B200Plan& p, const JvpWs& ws, const LayerPrimal& a, const LayerOffsets& o, const uint8_t* w,
                      const uint8_t* dw, const float* g_att, const float* dg_att, const float* g_ffn, const float* dg_ffn,
                      int T, int batch, int S_att, int live0, int pos_base, cudaStream_t stream) {
  const int d = p.d, h = p.h, dt = p.dtype;
  const size_t es = p.esize;
  uint8_t* dqkv_live = reinterpret_cast<uint8_t*>(ws.dqkv) + (size_t)live0 * 3 * d * es;
  const uint8_t* o_live = reinterpret_cast<const uint8_t*>(a.o) + (size_t)live0 * d * es;
  uint8_t* d_o_live = reinterpret_cast<uint8_t*>(ws.d_o) + (size_t)live0 * d * es;
  // attention block
  B200_TRY(launch_rmsnorm_jvp(a.x_in, ws.dx, g_att, dg_att, a.rinv1, ws.dxb, T, d, dt, stream));
  B200_TRY(lin(p, ws, ws.dxb, d, w + o.wqkv, d, T, 3 * d, d, dqkv_live, 3 * d, dt, 0, stream));
  B200_TRY(lin(p, ws, a.xb, d, dw + o.wqkv, d, T, 3 * d, d, dqkv_live, 3 * d, dt, 1, stream));
  B200_TRY(launch_rope_tangent(dqkv_live, dt, 3 * d, T, 2 * d, p.hs, S_att == T / batch ? S_att : 1,
                               p.rope_cos + (size_t)pos_base * (p.hs / 2), p.rope_sin + (size_t)pos_base * (p.hs / 2),
                               stream));
  B200_TRY(launch_attn_jvp(a.qkv, ws.dqkv, a.o, a.lse, ws.d_o, batch, S_att, p.H, p.hs, d, dt, stream));
  B200_TRY(lin_resid(p, ws, d_o_live, d, w + o.wo, d, T, d, ws.dx, ws.dx, stream));
  B200_TRY(lin_resid(p, ws, o_live, d, dw + o.wo, d, T, d, ws.dx, ws.dx, stream));
  // feed-forward block
  B200_TRY(launch_rmsnorm_jvp(a.x_mid, ws.dx, g_ffn, dg_ffn, a.rinv2, ws.dxb, T, d, dt, stream));
  B200_TRY(lin(p, ws, ws.dxb, d, w + o.w13, d, T, 2 * h, d, ws.dgu, 2 * h, dt, 0, stream));
  B200_TRY(lin(p, ws, a.xb2, d, dw + o.w13, d, T, 2 * h, d, ws.dgu, 2 * h, dt, 1, stream));
  B200_TRY(launch_swiglu_jvp(a.gate, a.up, ws.dgu, ws.dhg, dt, T, h, stream));
  B200_TRY(lin_resid(p, ws, ws.dhg, h, w + o.w2, h, T, h, ws.dx, ws.dx, stream));
  B200_TRY(lin_resid(p, ws, a.hg, h, dw + o.w2, h, T, h, ws.dx, ws.dx, stream));
  return B200_OK;
}

}  // namespace

size_t jvp_workspace_bytes(const B200Plan& p, int B, int S) {
  Arena a(nullptr);
  JvpWs w;
  carve_jvp(p, a, (size_t)B * S, (size_t)B * S, &w);
  return a.used + (size_t)B * S * p.d * p.esize + 256;  // + the tangent of the final normed rows
}

// Sequence form: tangents of the weight leaves (packed like the weights) -> tangent of the logits.
int32_t forward_jvp_impl(B200Plan* p, const int32_t* tokens, int B, int S, const uint8_t* w, const uint8_t* dw,
                         void* saved, float* dlogits, void* ws_, size_t ws_bytes, cudaStream_t stream) {
  const int T = B * S, d = p->d, dt = p->dtype;
  const PackedLayout& wl = p->wl;
  Arena sa(saved);
  FwdActs acts;
  carve_forward(*p, sa, B, S, true, &acts);
  Arena wa(ws_);
  JvpWs ws;
  carve_jvp(*p, wa, T, T, &ws);
  void* dxf = wa.take((size_t)T * d * p->esize);
  if (wa.used > ws_bytes) return fail(B200_ERR_WORKSPACE, "forward mode needs %zu workspace bytes, got %zu", wa.used, ws_bytes);
  auto gains = [&](const uint8_t* base, size_t off) { return reinterpret_cast<const float*>(base + off); };
  B200_TRY(launch_embed(tokens, dw + wl.emb, dt, ws.dx, T, d, p->V, stream));  // d x0 = dE[tokens]
  for (int l = 0; l < p->L; ++l) {
    const LayerActs& a = acts.layer[l];
    LayerPrimal pr{a.x_in, a.xb, a.rinv1, a.qkv, a.o, a.lse, a.x_mid, a.xb2, a.rinv2, a.gate, a.up, a.hg};
    B200_TRY(layer_tangent(*p, ws, pr, wl.layer[l], w, dw, gains(w, wl.g_att) + (size_t)l * d,
                           gains(dw, wl.g_att) + (size_t)l * d, gains(w, wl.g_ffn) + (size_t)l * d,
                           gains(dw, wl.g_ffn) + (size_t)l * d, T, B, S, 0, 0, stream));
  }
  B200_TRY(launch_rmsnorm_jvp(acts.fin.x_last, ws.dx, gains(w, wl.g_final), gains(dw, wl.g_final), acts.fin.rinv_f, dxf, T,
                              d, dt, stream));
  B200_TRY(lin(*p, ws, dxf, d, w + wl.wcls, d, T, p->V, d, dlogits, p->V, B200_F32, 0, stream));
  B200_TRY(lin(*p, ws, acts.fin.xf, d, dw + wl.wcls, d, T, p->V, d, dlogits, p->V, B200_F32, 1, stream));
  return B200_OK;
}

size_t token_jvp_workspace_bytes(const B200Plan& p, int pos) {
  Arena a(nullptr);
  TokWs t;
  carve_token(p, a, pos + 1, &t);
  JvpWs w;
  carve_jvp(p, a, 1, (size_t)pos + 1, &w);
  return a.used + 256;
}

// The reference's own call: tangents of x, the weight leaves and both caches -> tangent of the hidden state.
int32_t token_jvp_impl(B200Plan* p, const float* x, const void* key_cache, const void* value_cache, int pos,
                       const uint8_t* w, const float* dx_in, const uint8_t* dw, const void* d_key_cache,
                       const void* d_value_cache, float* hidden_out, float* d_hidden, void* ws_, size_t ws_bytes,
                       cudaStream_t stream) {
  const int d = p->d, S = pos + 1;
  const size_t es = p->esize;
  const PackedLayout& wl = p->wl;
  Arena wa(ws_);
  TokWs t;
  carve_token(*p, wa, S, &t);
  JvpWs ws;
  carve_jvp(*p, wa, 1, (size_t)S, &ws);
  if (wa.used > ws_bytes) return fail(B200_ERR_WORKSPACE, "token forward mode needs %zu workspace bytes, got %zu", wa.used, ws_bytes);
  B200_TRY(token_forward_run(p, t, x, key_cache, value_cache, pos, w, wl, hidden_out ? hidden_out : t.dx, stream));
  auto gains = [&](const uint8_t* base, size_t off) { return reinterpret_cast<const float*>(base + off); };
  B200_CUDA_OK(cudaMemcpyAsync(ws.dx, dx_in, (size_t)d * 4, cudaMemcpyDeviceToDevice, stream));
  for (int l = 0; l < p->L; ++l) {
    const TokLayer& a = t.layer[l];
    uint8_t* dqkv = reinterpret_cast<uint8_t*>(ws.dqkv);
    if (pos > 0) {
      // rows 0..pos-1: zero query tangents, the tangents of the cache rows as dK and dV
      B200_CUDA_OK(cudaMemset2DAsync(dqkv, (size_t)3 * d * es, 0, (size_t)d * es, pos, stream));
      const uint8_t* dk = reinterpret_cast<const uint8_t*>(d_key_cache) + (size_t)l * pos * d * es;
      const uint8_t* dv = reinterpret_cast<const uint8_t*>(d_value_cache) + (size_t)l * pos * d * es;
      B200_CUDA_OK(cudaMemcpy2DAsync(dqkv + (size_t)d * es, (size_t)3 * d * es, dk, (size_t)d * es, (size_t)d * es, pos,
                                     cudaMemcpyDeviceToDevice, stream));
      B200_CUDA_OK(cudaMemcpy2DAsync(dqkv + (size_t)2 * d * es, (size_t)3 * d * es, dv, (size_t)d * es, (size_t)d * es, pos,
                                     cudaMemcpyDeviceToDevice, stream));
    }
    LayerPrimal pr{a.x_in, a.xb, a.rinv1, a.qkv, a.o, a.lse, a.x_mid, a.xb2, a.rinv2, a.gate, a.up, a.hg};
    B200_TRY(layer_tangent(*p, ws, pr, wl.layer[l], w, dw, gains(w, wl.g_att) + (size_t)l * d,
                           gains(dw, wl.g_att) + (size_t)l * d, gains(w, wl.g_ffn) + (size_t)l * d,
                           gains(dw, wl.g_ffn) + (size_t)l * d, 1, 1, S, pos, pos, stream));
  }
  return launch_rmsnorm_jvp(t.x_last, ws.dx, gains(w, wl.g_final), gains(dw, wl.g_final), t.rinv_f, d_hidden, 1, d,
                            B200_F32, stream);
}

}  // namespace b200

using namespace b200;

extern "C" {

int32_t b200_token_jvp_workspace_bytes(const B200Plan* p, int32_t pos, size_t* bytes) {
  if (!p || !bytes) return fail(B200_ERR_INVALID_ARG, "null argument");
  if (pos < 0 || pos >= p->cfg.seq_len) return fail(B200_ERR_BAD_SHAPE, "pos=%d outside the plan's seq_len=%d", pos, p->cfg.seq_len);
  *bytes = token_jvp_workspace_bytes(*p, pos);
  return B200_OK;
}

int32_t b200_token_jvp(B200Plan* p, const float* x, const void* key_cache, const void* value_cache, int32_t pos,
                       const void* packed_w, const float* dx, const void* packed_dw, const void* d_key_cache,
                       const void* d_value_cache, float* hidden_out, float* d_hidden, void* ws, size_t ws_bytes,
                       b200_stream_t stream) {
  if (!p) return fail(B200_ERR_INVALID_ARG, "plan is null");
  if (p->tp_size != 1) return fail(B200_ERR_UNSUPPORTED, "forward mode runs on one GPU (tp_size must be 1)");
  if (pos < 0 || pos >= p->cfg.seq_len) return fail(B200_ERR_BAD_SHAPE, "pos=%d outside the plan's seq_len=%d", pos, p->cfg.seq_len);
  if (!x || !packed_w || !dx || !packed_dw || !d_hidden || !ws ||
      (pos > 0 && (!key_cache || !value_cache || !d_key_cache || !d_value_cache)))
    return fail(B200_ERR_INVALID_ARG, "null argument");
  if (!aligned16(x) || !aligned16(packed_w) || !aligned16(dx) || !aligned16(packed_dw) || !aligned16(d_hidden) ||
      !aligned16(ws) || (hidden_out && !aligned16(hidden_out)) ||
      (pos > 0 && (!aligned16(key_cache) || !aligned16(value_cache) || !aligned16(d_key_cache) || !aligned16(d_value_cache))))
    return fail(B200_ERR_MISALIGNED, "buffers must be 16-byte aligned");
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev != p->device) return fail(B200_ERR_INVALID_ARG, "wrong current device");
  return token_jvp_impl(p, x, key_cache, value_cache, pos, reinterpret_cast<const uint8_t*>(packed_w), dx,
                        reinterpret_cast<const uint8_t*>(packed_dw), d_key_cache, d_value_cache, hidden_out, d_hidden, ws,
                        ws_bytes, reinterpret_cast<cudaStream_t>(stream));
}

int32_t b200_jvp_workspace_bytes(const B200Plan* p, int32_t B, int32_t S, size_t* bytes) {
  if (!p || !bytes) return fail(B200_ERR_INVALID_ARG, "null argument");
  if (B <= 0 || S <= 0) return fail(B200_ERR_BAD_SHAPE, "batch and seq must be positive");
  *bytes = jvp_workspace_bytes(*p, B, S);
  return B200_OK;
}

int32_t b200_forward_jvp(B200Plan* p, const int32_t* tokens, int32_t B, int32_t S, const void* packed_w,
                         const void* packed_dw, const void* saved, float* dlogits, void* ws, size_t ws_bytes,
                         b200_stream_t stream) {
  if (!p) return fail(B200_ERR_INVALID_ARG, "plan is null");
  if (p->tp_size != 1) return fail(B200_ERR_UNSUPPORTED, "forward mode runs on one GPU (tp_size must be 1)");
  if (B <= 0 || S <= 0 || S > p->cfg.seq_len) return fail(B200_ERR_BAD_SHAPE, "bad batch=%d seq=%d", B, S);
  if (!tokens || !packed_w || !packed_dw || !saved || !dlogits || !ws) return fail(B200_ERR_INVALID_ARG, "null argument");
  if (!aligned16(packed_w) || !aligned16(packed_dw) || !aligned16(saved) || !aligned16(dlogits) || !aligned16(ws))
    return fail(B200_ERR_MISALIGNED, "buffers must be 16-byte aligned");
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev != p->device) return fail(B200_ERR_INVALID_ARG, "wrong current device");
  return forward_jvp_impl(p, tokens, B, S, reinterpret_cast<const uint8_t*>(packed_w),
                          reinterpret_cast<const uint8_t*>(packed_dw), const_cast<void*>(saved), dlogits, ws, ws_bytes,
                          reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
