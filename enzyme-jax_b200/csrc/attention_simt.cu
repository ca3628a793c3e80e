// Causal attention on the CUDA cores, any head size that is a multiple of 4 up
// to 128, fp32 or bf16 storage, fp32 softmax state (test/llama.py:177-209 of the
// reference, applied to every query position).  This is the exact-fp32 path and
// the fallback for head sizes the tensor-core kernel does not cover.
//
// A CTA of 128 threads owns 32 query rows of one (batch, head); 4 threads share
// a row and split the head dimension in four contiguous quarters.  Keys and values
// stream through shared memory in blocks of 32 rows with an online softmax.
#include "attention.cuh"

namespace b200 {

namespace {

constexpr int QB = 32;   // query rows per CTA
constexpr int KB = 32;   // keys per shared-memory block

template <typename T, int HS>
__global__ void __launch_bounds__(128) attn_fwd_simt_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                            const T* __restrict__ v, T* __restrict__ o,
                                                            float* __restrict__ lse, int seq, int n_heads, int ldq,
                                                            int ldkv, int ldo, float scale, bool vec) {
  constexpr int DPT = HS / 4;  // dims per thread: [part * DPT, (part + 1) * DPT), read from shared memory 16 bytes at a time
  static_assert(DPT % 4 == 0, "head size must be a multiple of 16");
  __shared__ __align__(16) float Ks[KB][HS];
  __shared__ __align__(16) float Vs[KB][HS];
  const int tid = threadIdx.x, r = tid >> 2, part = tid & 3;
  const int qblk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int t0 = qblk * QB;
  const int t = t0 + r;  // position inside the sequence
  const size_t row0 = (size_t)b * seq;
  const bool row_ok = t < seq;

  float qr[DPT], acc[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    qr[i] = row_ok ? to_f32(q[(row0 + t) * ldq + h * HS + part * DPT + i]) * scale : 0.f;
    acc[i] = 0.f;
  }
  float mx = -INFINITY, l = 0.f;

  const int last = min(t0 + QB, seq);  // keys needed by this CTA: [0, last)
  // A K / V block travels global -> registers -> shared memory in 8-element pieces; the pieces of block i+1 are
  // requested before the arithmetic of block i, so their round trip hides behind it.
  constexpr int PIECES = KB * HS / 8, PER = (PIECES + 127) / 128;
  float pk[PER][8], pv[PER][8];
  auto fetch = [&](int u0) {
#pragma unroll
    for (int it = 0; it < PER; ++it) {
      const int idx = tid + it * 128;
      if (idx < PIECES) {
        const int uu = idx / (HS / 8), d8 = (idx % (HS / 8)) * 8;
        const int u = u0 + uu;
        if (u < seq) {
          const size_t off = (row0 + u) * ldkv + h * HS + d8;
          if (vec) {
            load8(k + off, pk[it]);
            load8(v + off, pv[it]);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) { pk[it][j] = to_f32(k[off + j]); pv[it][j] = to_f32(v[off + j]); }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) { pk[it][j] = 0.f; pv[it][j] = 0.f; }
        }
      }
    }
  };
  fetch(0);
  for (int u0 = 0; u0 < last; u0 += KB) {
    __syncthreads();
#pragma unroll
    for (int it = 0; it < PER; ++it) {
      const int idx = tid + it * 128;
      if (idx < PIECES) {
        const int uu = idx / (HS / 8), d8 = (idx % (HS / 8)) * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) { Ks[uu][d8 + j] = pk[it][j]; Vs[uu][d8 + j] = pv[it][j]; }
      }
    }
    __syncthreads();
    if (u0 + KB < last) fetch(u0 + KB);
    float s[KB];
    float bm = -INFINITY;
#pragma unroll
    for (int uu = 0; uu < KB; ++uu) {
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < DPT; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(&Ks[uu][part * DPT + i]);
        d = fmaf(qr[i], k4.x, fmaf(qr[i + 1], k4.y, fmaf(qr[i + 2], k4.z, fmaf(qr[i + 3], k4.w, d))));
      }
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      s[uu] = (u0 + uu <= t && row_ok) ? d : -INFINITY;
      bm = fmaxf(bm, s[uu]);
    }
    if (bm > -INFINITY) {
      const float nm = fmaxf(mx, bm);
      const float corr = exp_by_build(mx - nm);
      l *= corr;
#pragma unroll
      for (int i = 0; i < DPT; ++i) acc[i] *= corr;
#pragma unroll
      for (int uu = 0; uu < KB; ++uu) {
        const float p = exp_by_build(s[uu] - nm);
        l += p;
#pragma unroll
        for (int i = 0; i < DPT; i += 4) {
          const float4 v4 = *reinterpret_cast<const float4*>(&Vs[uu][part * DPT + i]);
          acc[i] = fmaf(p, v4.x, acc[i]); acc[i + 1] = fmaf(p, v4.y, acc[i + 1]);
          acc[i + 2] = fmaf(p, v4.z, acc[i + 2]); acc[i + 3] = fmaf(p, v4.w, acc[i + 3]);
        }
      }
      mx = nm;
    }
  }
  if (row_ok) {
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < DPT; ++i) o[(row0 + t) * ldo + h * HS + part * DPT + i] = from_f32<T>(acc[i] * inv);
    if (lse && part == 0) lse[((size_t)b * n_heads + h) * seq + t] = mx + __logf(l);
  }
}

template <typename T, int HS>
int32_t launch_hs(const AttnArgs& a, cudaStream_t stream) {
  dim3 grid(cdiv(a.seq, QB), a.n_heads, a.batch);
  attn_fwd_simt_kernel<T, HS><<<grid, 128, 0, stream>>>((const T*)a.q, (const T*)a.k, (const T*)a.v, (T*)a.o, a.lse,
                                                        a.seq, a.n_heads, a.ldq, a.ldkv, a.ldo,
                                                        1.f / sqrtf((float)a.head_size),
                                                        aligned16(a.k) && aligned16(a.v) && a.ldkv % 8 == 0);
  B200_LAUNCH_OK("attn_fwd_simt_kernel");
  return B200_OK;
}

template <typename T>
int32_t launch_t(const AttnArgs& a, cudaStream_t stream) {
  switch (a.head_size) {
    case 16: return launch_hs<T, 16>(a, stream);
    case 32: return launch_hs<T, 32>(a, stream);
    case 48: return launch_hs<T, 48>(a, stream);
    case 64: return launch_hs<T, 64>(a, stream);
    case 128: return launch_hs<T, 128>(a, stream);
  }
  return fail(B200_ERR_BAD_SHAPE, "attention: head size %d is not one of 16/32/48/64/128", a.head_size);
}


// ---- backward -----------------------------------------------------------------
// delta[b,h,t] = sum_e dO[t,e] * O[t,e]
template <typename T, int HS>
__global__ void __launch_bounds__(128) attn_delta_kernel(const T* __restrict__ o, const T* __restrict__ d_o,
                                                         float* __restrict__ delta, int seq, int n_heads, int ldo,
                                                         int lddo) {
  constexpr int DPT = HS / 4;
  const int tid = threadIdx.x, r = tid >> 2, part = tid & 3;
  const int h = blockIdx.y, b = blockIdx.z;
  const int t = blockIdx.x * QB + r;
  const bool ok = t < seq;
  const size_t row = (size_t)b * seq + (ok ? t : 0);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < DPT; ++i)
    s = fmaf(to_f32(o[row * ldo + h * HS + part + 4 * i]), to_f32(d_o[row * lddo + h * HS + part + 4 * i]), s);
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  if (ok && part == 0) delta[((size_t)b * n_heads + h) * seq + t] = s;
}

// dQ: a CTA owns 32 query rows and streams the keys/values it may attend to.
template <typename T, int HS>
__global__ void __launch_bounds__(128)
    attn_bwd_dq_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                       const T* __restrict__ d_o, const float* __restrict__ lse, const float* __restrict__ delta,
                       T* __restrict__ dq, int seq, int n_heads, int ldq, int ldkv, int lddo, int lddq, float scale) {
  constexpr int DPT = HS / 4;
  __shared__ float Ks[KB][HS];
  __shared__ float Vs[KB][HS];
  const int tid = threadIdx.x, r = tid >> 2, part = tid & 3;
  const int h = blockIdx.y, b = blockIdx.z;
  const int t0 = blockIdx.x * QB, t = t0 + r;
  const size_t row0 = (size_t)b * seq;
  const bool row_ok = t < seq;
  float qr[DPT], dor[DPT], acc[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    qr[i] = row_ok ? to_f32(q[(row0 + t) * ldq + h * HS + part + 4 * i]) : 0.f;
    dor[i] = row_ok ? to_f32(d_o[(row0 + t) * lddo + h * HS + part + 4 * i]) : 0.f;
    acc[i] = 0.f;
  }
  const float my_lse = row_ok ? lse[((size_t)b * n_heads + h) * seq + t] : 0.f;
  const float my_delta = row_ok ? delta[((size_t)b * n_heads + h) * seq + t] : 0.f;
  const int last = min(t0 + QB, seq);
  for (int u0 = 0; u0 < last; u0 += KB) {
    __syncthreads();
    for (int idx = tid; idx < KB * HS; idx += 128) {
      const int uu = idx / HS, dd = idx % HS, u = u0 + uu;
      Ks[uu][dd] = u < seq ? to_f32(k[(row0 + u) * ldkv + h * HS + dd]) : 0.f;
      Vs[uu][dd] = u < seq ? to_f32(v[(row0 + u) * ldkv + h * HS + dd]) : 0.f;
    }
    __syncthreads();
#pragma unroll 4
    for (int uu = 0; uu < KB; ++uu) {
      float s = 0.f, dp = 0.f;
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        s = fmaf(qr[i], Ks[uu][part + 4 * i], s);
        dp = fmaf(dor[i], Vs[uu][part + 4 * i], dp);
      }
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      dp += __shfl_xor_sync(0xffffffffu, dp, 1);
      dp += __shfl_xor_sync(0xffffffffu, dp, 2);
      const bool live = row_ok && (u0 + uu <= t);
      const float p = live ? exp_by_build(s * scale - my_lse) : 0.f;
      const float ds = p * (dp - my_delta) * scale;
#pragma unroll
      for (int i = 0; i < DPT; ++i) acc[i] = fmaf(ds, Ks[uu][part + 4 * i], acc[i]);
    }
  }
  if (row_ok) {
#pragma unroll
    for (int i = 0; i < DPT; ++i) dq[(row0 + t) * lddq + h * HS + part + 4 * i] = from_f32<T>(acc[i]);
  }
}

// dK, dV: a CTA owns 32 key rows and streams the queries that attend to them.
template <typename T, int HS>
__global__ void __launch_bounds__(128)
    attn_bwd_dkv_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                        const T* __restrict__ d_o, const float* __restrict__ lse, const float* __restrict__ delta,
                        T* __restrict__ dk, T* __restrict__ dv, int seq, int n_heads, int ldq, int ldkv, int lddo,
                        int lddkv, float scale) {
  constexpr int DPT = HS / 4;
  __shared__ float Qs[KB][HS];
  __shared__ float Ds[KB][HS];
  __shared__ float Ls[KB], Dl[KB];
  const int tid = threadIdx.x, r = tid >> 2, part = tid & 3;
  const int h = blockIdx.y, b = blockIdx.z;
  const int u0 = blockIdx.x * QB, u = u0 + r;
  const size_t row0 = (size_t)b * seq;
  const bool row_ok = u < seq;
  float kr[DPT], vr[DPT], acck[DPT], accv[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    kr[i] = row_ok ? to_f32(k[(row0 + u) * ldkv + h * HS + part + 4 * i]) : 0.f;
    vr[i] = row_ok ? to_f32(v[(row0 + u) * ldkv + h * HS + part + 4 * i]) : 0.f;
    acck[i] = 0.f;
    accv[i] = 0.f;
  }
  for (int t0 = u0; t0 < seq; t0 += KB) {  // query blocks at or after this key block
    __syncthreads();
    for (int idx = tid; idx < KB * HS; idx += 128) {
      const int tt = idx / HS, dd = idx % HS, t = t0 + tt;
      Qs[tt][dd] = t < seq ? to_f32(q[(row0 + t) * ldq + h * HS + dd]) : 0.f;
      Ds[tt][dd] = t < seq ? to_f32(d_o[(row0 + t) * lddo + h * HS + dd]) : 0.f;
    }
    if (tid < KB) {
      const int t = t0 + tid;
      Ls[tid] = t < seq ? lse[((size_t)b * n_heads + h) * seq + t] : 0.f;
      Dl[tid] = t < seq ? delta[((size_t)b * n_heads + h) * seq + t] : 0.f;
    }
    __syncthreads();
#pragma unroll 4
    for (int tt = 0; tt < KB; ++tt) {
      float s = 0.f, dp = 0.f;
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        s = fmaf(kr[i], Qs[tt][part + 4 * i], s);
        dp = fmaf(vr[i], Ds[tt][part + 4 * i], dp);
      }
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      dp += __shfl_xor_sync(0xffffffffu, dp, 1);
      dp += __shfl_xor_sync(0xffffffffu, dp, 2);
      const int t = t0 + tt;
      const bool live = row_ok && t < seq && t >= u;
      const float p = live ? exp_by_build(s * scale - Ls[tt]) : 0.f;
      const float ds = p * (dp - Dl[tt]) * scale;
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        accv[i] = fmaf(p, Ds[tt][part + 4 * i], accv[i]);
        acck[i] = fmaf(ds, Qs[tt][part + 4 * i], acck[i]);
      }
    }
  }
  if (row_ok) {
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      dk[(row0 + u) * lddkv + h * HS + part + 4 * i] = from_f32<T>(acck[i]);
      dv[(row0 + u) * lddkv + h * HS + part + 4 * i] = from_f32<T>(accv[i]);
    }
  }
}

template <typename T, int HS>
int32_t launch_bwd_hs(const AttnBwdArgs& a, cudaStream_t stream) {
  const AttnArgs& f = a.f;
  dim3 grid(cdiv(f.seq, QB), f.n_heads, f.batch);
  const float scale = 1.f / sqrtf((float)f.head_size);
  attn_delta_kernel<T, HS><<<grid, 128, 0, stream>>>((const T*)f.o, (const T*)a.d_o, a.delta, f.seq, f.n_heads, f.ldo,
                                                     a.lddo);
  B200_LAUNCH_OK("attn_delta_kernel");
  attn_bwd_dq_kernel<T, HS><<<grid, 128, 0, stream>>>((const T*)f.q, (const T*)f.k, (const T*)f.v, (const T*)a.d_o,
                                                      f.lse, a.delta, (T*)a.dq, f.seq, f.n_heads, f.ldq, f.ldkv,
                                                      a.lddo, a.lddq, scale);
  B200_LAUNCH_OK("attn_bwd_dq_kernel");
  attn_bwd_dkv_kernel<T, HS><<<grid, 128, 0, stream>>>((const T*)f.q, (const T*)f.k, (const T*)f.v, (const T*)a.d_o,
                                                       f.lse, a.delta, (T*)a.dk, (T*)a.dv, f.seq, f.n_heads, f.ldq,
                                                       f.ldkv, a.lddo, a.lddkv, scale);
  B200_LAUNCH_OK("attn_bwd_dkv_kernel");
  return B200_OK;
}

template <typename T>
int32_t launch_bwd_t(const AttnBwdArgs& a, cudaStream_t stream) {
  switch (a.f.head_size) {
    case 16: return launch_bwd_hs<T, 16>(a, stream);
    case 32: return launch_bwd_hs<T, 32>(a, stream);
    case 48: return launch_bwd_hs<T, 48>(a, stream);
    case 64: return launch_bwd_hs<T, 64>(a, stream);
    case 128: return launch_bwd_hs<T, 128>(a, stream);
  }
  return fail(B200_ERR_BAD_SHAPE, "attention: head size %d is not one of 16/32/48/64/128", a.f.head_size);
}

}  // namespace

int32_t launch_attn_fwd_simt(const AttnArgs& a, cudaStream_t stream) {
  if (a.batch <= 0 || a.seq <= 0 || a.n_heads <= 0) return fail(B200_ERR_BAD_SHAPE, "attention: empty problem");
  if (a.dtype == B200_F32) return launch_t<float>(a, stream);
  if (a.dtype == B200_BF16) return launch_t<bf16>(a, stream);
  return fail(B200_ERR_BAD_DTYPE, "attention: unsupported dtype %d", a.dtype);
}

}  // namespace b200

namespace b200 {
namespace {
template <typename T, int HS>
int32_t launch_delta_hs(const AttnBwdArgs& a, cudaStream_t stream) {
  const AttnArgs& f = a.f;
  dim3 grid(cdiv(f.seq, QB), f.n_heads, f.batch);
  attn_delta_kernel<T, HS><<<grid, 128, 0, stream>>>((const T*)f.o, (const T*)a.d_o, a.delta, f.seq, f.n_heads, f.ldo,
                                                     a.lddo);
  B200_LAUNCH_OK("attn_delta_kernel");
  return B200_OK;
}
}  // namespace

int32_t launch_attn_delta(const AttnBwdArgs& a, cudaStream_t stream) {
  if (a.f.dtype == B200_BF16 && a.f.head_size == 64) return launch_delta_hs<bf16, 64>(a, stream);
  if (a.f.dtype == B200_BF16 && a.f.head_size == 128) return launch_delta_hs<bf16, 128>(a, stream);
  return fail(B200_ERR_UNSUPPORTED, "delta kernel: unsupported dtype/head size");
}

int32_t launch_attn_bwd(const AttnBwdArgs& a, int impl, cudaStream_t stream) {
  const AttnArgs& f = a.f;
  // forward + 2.5x: S and dP twice (two passes), dV, dK, dQ: 7 products of S^2*hs per (batch, head), causal half
  ProfScope prof(PROF_ATTN_BWD, 7.0 * f.batch * f.n_heads * (double)f.seq * f.seq * f.head_size, stream);
  if (impl == 2) return launch_attn_bwd_simt(a, stream);
  if (impl == 1) return launch_attn_bwd_tc(a, stream);
  if (attn_bwd_tc_supports(a)) return launch_attn_bwd_tc(a, stream);
  return launch_attn_bwd_simt(a, stream);
}

int32_t launch_attn_bwd_simt(const AttnBwdArgs& a, cudaStream_t stream) {
  if (!a.delta || !a.f.lse) return fail(B200_ERR_INVALID_ARG, "attention backward needs lse and a delta scratch");
  if (a.f.dtype == B200_F32) return launch_bwd_t<float>(a, stream);
  if (a.f.dtype == B200_BF16) return launch_bwd_t<bf16>(a, stream);
  return fail(B200_ERR_BAD_DTYPE, "attention: unsupported dtype %d", a.f.dtype);
}
}  // namespace b200
