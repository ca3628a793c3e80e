// Memory-bound kernels of the llama path.  All traffic is 128-bit where the
// shapes allow; reductions use warp shuffles and one shared-memory hop; math is
// fp32 whatever the storage type.
#include "elementwise.cuh"

namespace b200 {

namespace {

// ---- embedding --------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const int32_t* __restrict__ tokens, const T* __restrict__ table, float* __restrict__ x,
                             int dim, int vocab) {
  const int t = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  int tok = tokens[t];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  const T* src = table + (size_t)tok * dim;
  float* dst = x + (size_t)t * dim;
  for (int c = threadIdx.x * 8; c < dim; c += blockDim.x * 8) {
    float v[8];
    load8(src + c, v);
    store8(dst + c, v);
  }
}

// ---- RMSNorm forward --------------------------------------------------------
template <typename TOut>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                                                      TOut* __restrict__ y, float* __restrict__ rinv, int dim,
                                                      float eps) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const float* xr = x + (size_t)row * dim;
  float ss = 0.f;
  for (int c = threadIdx.x * 8; c < dim; c += blockDim.x * 8) {
    float v[8];
    load8(xr + c, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / (float)dim + eps);
  if (rinv && threadIdx.x == 0) rinv[row] = r;
  TOut* yr = y + (size_t)row * dim;
  for (int c = threadIdx.x * 8; c < dim; c += blockDim.x * 8) {
    float v[8], g[8];
    load8(xr + c, v);
    load8(gain + c, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = g[i] * v[i] * r;
    store8(yr + c, v);
  }
}

// Warp-per-row variant (dim <= 2048): the row is read once and stays in
// registers between the reduction and the scaling; no block barrier.
template <typename TOut, int NCH>
__global__ void __launch_bounds__(256) rmsnorm_warp_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                                                           TOut* __restrict__ y, float* __restrict__ rinv, int rows,
                                                           int dim, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp;
  pdl_launch_dependents();
  pdl_wait();
  if (row >= rows) return;
  const float* xr = x + (size_t)row * dim;
  float v[NCH][8];
  float ss = 0.f;
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    const int c = (ch * 32 + lane) * 8;
    if (c < dim) {
      load8_wide(xr + c, v[ch]);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(v[ch][i], v[ch][i], ss);
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)dim + eps);
  if (rinv && lane == 0) rinv[row] = r;
  TOut* yr = y + (size_t)row * dim;
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    const int c = (ch * 32 + lane) * 8;
    if (c < dim) {
      float g[8];
      load8(gain + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[ch][i] = g[i] * v[ch][i] * r;
      store8(yr + c, v[ch]);
    }
  }
}

template <typename T>
__global__ void add_to_f32_kernel(float* __restrict__ x, const T* __restrict__ d, size_t n8) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float a[8], b[8];
    load8(x + i * 8, a);
    load8(d + i * 8, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] += b[j];
    store8(x + i * 8, a);
  }
}

template <typename TS, typename TD>
__global__ void copy_rows_kernel(const TS* __restrict__ src, int src_ld, TD* __restrict__ dst, int dst_ld, int rows,
                                 int cols, int group, int gstride, int goff) {
  const int c8 = cols / 8;
  const size_t total = (size_t)rows * c8;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / c8), c = (int)(i % c8) * 8;
    const int dr = (r / group) * gstride + goff + r % group;
    float v[8];
    load8(src + (size_t)r * src_ld + c, v);
    store8(dst + (size_t)dr * dst_ld + c, v);
  }
}

template <typename TS, typename TD>
__global__ void transpose_kernel(const TS* __restrict__ src, int src_ld, TD* __restrict__ dst, int dst_ld, int rows,
                                 int cols) {
  __shared__ float tile[32][33];
  const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    tile[i][threadIdx.x] = (r < rows && c < cols) ? to_f32(src[(size_t)r * src_ld + c]) : 0.f;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i, r = r0 + threadIdx.x;
    if (r < rows && c < cols) dst[(size_t)c * dst_ld + r] = from_f32<TD>(tile[threadIdx.x][i]);
  }
}

__global__ void rope_table_kernel(float* cos_t, float* sin_t, int n_pos, int half, int head_size, float theta) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pos * half) return;
  const int pos = i / half, j = i % half;
  // freq = theta^(-(2j)/hs), evaluated in double so that the table is the
  // correctly rounded fp32 value of the exact angle's cos/sin.
  const double freq = 1.0 / pow((double)theta, (double)(2 * j) / (double)head_size);
  const double ang = (double)pos * freq;
  cos_t[i] = (float)cos(ang);
  sin_t[i] = (float)sin(ang);
}

// ---- RMSNorm backward -------------------------------------------------------
constexpr int RB_THREADS = 256;
constexpr int RB_MAXCH = 4;  // 8-wide chunks per thread: dim <= 256*8*4 = 8192

template <typename TDy>
__global__ void __launch_bounds__(RB_THREADS)
    rmsnorm_bwd_kernel(const float* __restrict__ x, const float* __restrict__ gain, const float* __restrict__ rinv,
                       const TDy* dy, float* __restrict__ dx, int accumulate_dx, TDy* dx_copy,
                       float* __restrict__ dg_part, int rows, int dim, int rows_per_part) {
  __shared__ float red[32];
  float dg[RB_MAXCH][8];
#pragma unroll
  for (int ch = 0; ch < RB_MAXCH; ++ch)
#pragma unroll
    for (int i = 0; i < 8; ++i) dg[ch][i] = 0.f;
  const int r_begin = blockIdx.x * rows_per_part;
  const int r_end = min(rows, r_begin + rows_per_part);
  for (int row = r_begin; row < r_end; ++row) {
    const float r = rinv[row];
    const float* xr = x + (size_t)row * dim;
    const TDy* dyr = dy + (size_t)row * dim;
    float dot = 0.f;
#pragma unroll
    for (int ch = 0; ch < RB_MAXCH; ++ch) {
      const int c = (ch * RB_THREADS + threadIdx.x) * 8;
      if (c < dim) {
        float xv[8], dv[8], g[8];
        load8(xr + c, xv);
        load8(dyr + c, dv);
        load8(gain + c, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          dot = fmaf(g[i] * dv[i], xv[i], dot);
          dg[ch][i] = fmaf(dv[i] * xv[i], r, dg[ch][i]);
        }
      }
    }
    dot = block_sum(dot, red);
    const float coef = r * r * r / (float)dim * dot;
    float* dxr = dx + (size_t)row * dim;
#pragma unroll
    for (int ch = 0; ch < RB_MAXCH; ++ch) {
      const int c = (ch * RB_THREADS + threadIdx.x) * 8;
      if (c < dim) {
        float xv[8], dv[8], g[8], out[8];
        load8(xr + c, xv);
        load8(dyr + c, dv);
        load8(gain + c, g);
        if (accumulate_dx) load8(dxr + c, out);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float val = r * g[i] * dv[i] - xv[i] * coef;
          out[i] = accumulate_dx ? out[i] + val : val;
        }
        store8(dxr + c, out);
        if (dx_copy) store8(dx_copy + (size_t)row * dim + c, out);  // may be dy itself: this thread has read its piece
      }
    }
  }
  float* part = dg_part + (size_t)blockIdx.x * dim;
#pragma unroll
  for (int ch = 0; ch < RB_MAXCH; ++ch) {
    const int c = (ch * RB_THREADS + threadIdx.x) * 8;
    if (c < dim) store8(part + c, dg[ch]);
  }
}

// Warp-per-row variant for dim <= 1536: no block-wide barrier per row.  Lane l
// owns columns {l*8 + 256*i}; the 8 warps of a CTA walk the CTA's rows round
// robin and their gain partials are summed through shared memory at the end in
// warp order (fixed order, no atomics).
constexpr int RW_WARPS = 8;
constexpr int RW_MAXCH = 6;  // 8-wide chunks per lane: dim <= 32*8*6 = 1536

template <typename TDy, int NCH>
__global__ void __launch_bounds__(RW_WARPS * 32)
    rmsnorm_bwd_warp_kernel(const float* __restrict__ x, const float* __restrict__ gain, const float* __restrict__ rinv,
                            const TDy* dy, float* __restrict__ dx, int accumulate_dx, TDy* dx_copy,
                            float* __restrict__ dg_part, int rows, int dim, int rows_per_part) {
  extern __shared__ float s_dg[];  // [RW_WARPS][dim]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  pdl_wait();
  float dg[NCH][8];
  float g[NCH][8];
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    const int c = (ch * 32 + lane) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) { dg[ch][i] = 0.f; g[ch][i] = 0.f; }
    if (c < dim) load8(gain + c, g[ch]);
  }
  const int r_begin = blockIdx.x * rows_per_part;
  const int r_end = min(rows, r_begin + rows_per_part);
  for (int row = r_begin + warp; row < r_end; row += RW_WARPS) {
    const float r = rinv[row];
    const float* xr = x + (size_t)row * dim;
    const TDy* dyr = dy + (size_t)row * dim;
    float xv[NCH][8], dv[NCH][8];
    float dot = 0.f;
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int c = (ch * 32 + lane) * 8;
      if (c < dim) {
        load8(xr + c, xv[ch]);
        load8(dyr + c, dv[ch]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          dot = fmaf(g[ch][i] * dv[ch][i], xv[ch][i], dot);
          dg[ch][i] = fmaf(dv[ch][i] * xv[ch][i], r, dg[ch][i]);
        }
      }
    }
    dot = warp_sum(dot);
    const float coef = r * r * r / (float)dim * dot;
    float* dxr = dx + (size_t)row * dim;
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int c = (ch * 32 + lane) * 8;
      if (c < dim) {
        float out[8];
        if (accumulate_dx) load8(dxr + c, out);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float val = r * g[ch][i] * dv[ch][i] - xv[ch][i] * coef;
          out[i] = accumulate_dx ? out[i] + val : val;
        }
        store8(dxr + c, out);
        if (dx_copy) store8(dx_copy + (size_t)row * dim + c, out);  // may be dy itself: the row is in registers
      }
    }
  }
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    const int c = (ch * 32 + lane) * 8;
    if (c < dim) store8(s_dg + (size_t)warp * dim + c, dg[ch]);
  }
  __syncthreads();
  float* part = dg_part + (size_t)blockIdx.x * dim;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < RW_WARPS; ++w) sum += s_dg[(size_t)w * dim + c];
    part[c] = sum;
  }
}

// out[c] (+)= sum_p part[p, c].  A CTA of 32 x 8 threads owns 32 columns; thread
// (c, g) adds parts g, g+8, ... and the 8 group sums are added in group order.
__global__ void __launch_bounds__(256) colsum_parts_kernel(const float* __restrict__ part, int n_parts, int dim,
                                                           float* __restrict__ out, int accumulate) {
  __shared__ float red[8][33];
  const int cx = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s = 0.f;
  if (c < dim)
    for (int p = g; p < n_parts; p += 8) s += part[(size_t)p * dim + c];
  red[g][cx] = s;
  __syncthreads();
  if (g == 0 && c < dim) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][cx];
    out[c] = accumulate ? out[c] + t : t;
  }
}

template <typename T>
__global__ void rope_bwd_kernel(T* __restrict__ d, int ld, int rows, int rope_cols, int head_size, int seq_len,
                                const float* __restrict__ cos_t, const float* __restrict__ sin_t) {
  const int c8n = rope_cols / 8;
  const size_t total = (size_t)rows * c8n;
  const int half = head_size >> 1;
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / c8n), c = (int)(i % c8n) * 8;
    const int pos = r % seq_len;
    float v[8];
    T* p = d + (size_t)r * ld + c;
    load8(p, v);
#pragma unroll
    for (int k = 0; k < 8; k += 2) {
      const int j = ((c + k) % head_size) >> 1;
      const float cj = cos_t[(size_t)pos * half + j], sj = sin_t[(size_t)pos * half + j];
      const float e = v[k], o = v[k + 1];
      v[k] = cj * e + sj * o;
      v[k + 1] = -sj * e + cj * o;
    }
    store8(p, v);
  }
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ gate, const T* __restrict__ up, const T* __restrict__ dh,
                                  T* __restrict__ dgu, int rows, int hidden) {
  const int c8n = hidden / 8;
  const size_t total = (size_t)rows * c8n;
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / c8n), c = (int)(i % c8n) * 8;
    float a[8], b[8], d[8], da[8], db[8];
    load8(gate + (size_t)r * hidden + c, a);
    load8(up + (size_t)r * hidden + c, b);
    load8(dh + (size_t)r * hidden + c, d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sg = 1.f / (1.f + exp_by_build(-a[k]));
      db[k] = d[k] * a[k] * sg;
      da[k] = d[k] * b[k] * sg * (1.f + a[k] * (1.f - sg));
    }
    T* o = dgu + (size_t)r * (2 * hidden) + (size_t)(c / 8) * 16;
    store8(o, da);
    store8(o + 8, db);
  }
}

// Each CTA owns the table rows [v0, v1).  It scans the token list 256 tokens at
// a time (one token per thread, matches recorded as warp ballots) and then
// applies the matching rows in token order, so that every table row receives its
// contributions in sequence order: deterministic, no atomics.
__global__ void __launch_bounds__(256) embed_bwd_kernel(const int32_t* __restrict__ tokens,
                                                        const float* __restrict__ dx, float* __restrict__ dtable,
                                                        int n_tokens, int dim, int vocab, int rows_per_cta) {
  __shared__ uint32_t hit[8];
  __shared__ int32_t toks[256];
  const int v0 = blockIdx.x * rows_per_cta;
  const int v1 = min(vocab, v0 + rows_per_cta);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int base = 0; base < n_tokens; base += 256) {
    const int i = base + threadIdx.x;
    const int tok = i < n_tokens ? tokens[i] : -1;
    const uint32_t b = __ballot_sync(0xffffffffu, tok >= v0 && tok < v1);
    __syncthreads();  // the previous chunk's lists are no longer read
    toks[threadIdx.x] = tok;
    if (lane == 0) hit[warp] = b;
    __syncthreads();
    for (int w = 0; w < 8; ++w) {
      uint32_t bits = hit[w];
      while (bits) {
        const int k = __ffs(bits) - 1;
        bits &= bits - 1;
        const int t = w * 32 + k;
        const float* src = dx + (size_t)(base + t) * dim;
        float* dst = dtable + (size_t)toks[t] * dim;
        for (int c = threadIdx.x * 4; c < dim; c += blockDim.x * 4) {
          float4 a = *reinterpret_cast<const float4*>(src + c);
          float4 d = *reinterpret_cast<float4*>(dst + c);
          d.x += a.x; d.y += a.y; d.z += a.z; d.w += a.w;
          *reinterpret_cast<float4*>(dst + c) = d;
        }
        __syncthreads();  // two hits of one chunk may target the same table row
      }
    }
  }
}

template <typename TS, typename TD>
__global__ void convert_kernel(const TS* __restrict__ s, TD* __restrict__ d, size_t n8) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float v[8];
    load8(s + i * 8, v);
    store8(d + i * 8, v);
  }
}

__global__ void zero_kernel(float4* p, size_t n4) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x)
    p[i] = make_float4(0.f, 0.f, 0.f, 0.f);
}

inline int grid_for(size_t work_items, int threads) {
  size_t g = (work_items + threads - 1) / threads;
  const size_t cap = (size_t)sm_count() * 16;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

#define DISPATCH2(sd, dd, CALL)                                                        \
  if (sd == B200_F32 && dd == B200_F32) { using TS = float; using TD = float; CALL; }  \
  else if (sd == B200_F32 && dd == B200_BF16) { using TS = float; using TD = bf16; CALL; } \
  else if (sd == B200_BF16 && dd == B200_F32) { using TS = bf16; using TD = float; CALL; } \
  else if (sd == B200_BF16 && dd == B200_BF16) { using TS = bf16; using TD = bf16; CALL; } \
  else return fail(B200_ERR_BAD_DTYPE, "unsupported dtype pair %d -> %d", sd, dd);

// ---- greedy sampling ---------------------------------------------------------
// out[r] = index of the largest of row r's `cols` values, the lowest index among equals (numpy / torch argmax).
__global__ void __launch_bounds__(256) argmax_rows_kernel(const float* __restrict__ x, int cols, int ld,
                                                          int32_t* __restrict__ out) {
  __shared__ float s_v[8];
  __shared__ int s_i[8];
  const int row = blockIdx.x;
  const float* xr = x + (size_t)row * ld;
  pdl_launch_dependents();
  pdl_wait();
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = xr[c];
    if (v > bv || (v == bv && c < bi)) { bv = v; bi = c; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { s_v[warp] = bv; s_i[warp] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (s_v[w] > bv || (s_v[w] == bv && s_i[w] < bi)) { bv = s_v[w]; bi = s_i[w]; }
    out[row] = bi == 0x7fffffff ? 0 : bi;  // a row of NaNs compares false everywhere: report index 0
  }
}

}  // namespace

int32_t launch_embed(const int32_t* tokens, const void* table, int table_dtype, float* x, int n_tokens, int dim,
                     int vocab, cudaStream_t stream) {
  if (dim % 8) return fail(B200_ERR_BAD_SHAPE, "embedding: dim=%d must be a multiple of 8", dim);
  const int threads = dim / 8 < 128 ? ((dim / 8 + 31) / 32) * 32 : 128;
  if (table_dtype == B200_F32)
    B200_CUDA_OK(launch_pdl(embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const float*)table,
                            x, dim, vocab));
  else if (table_dtype == B200_BF16)
    B200_CUDA_OK(launch_pdl(embed_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const bf16*)table,
                            x, dim, vocab));
  else
    return fail(B200_ERR_BAD_DTYPE, "embedding: unsupported dtype %d", table_dtype);
  B200_LAUNCH_OK("embed_kernel");
  return B200_OK;
}

int32_t launch_rmsnorm(const float* x, const float* gain, void* y, float* rinv, int rows, int dim, float eps,
                       int out_dtype, cudaStream_t stream) {
  if (dim % 8) return fail(B200_ERR_BAD_SHAPE, "rmsnorm: dim=%d must be a multiple of 8", dim);
  if (rows <= 0) return fail(B200_ERR_BAD_SHAPE, "rmsnorm: no rows");
  if (dim <= 2048 && (out_dtype == B200_F32 || out_dtype == B200_BF16)) {
    const int nch = cdiv(dim, 256);
    const int grid = cdiv(rows, 8);
#define B200_RN_CASE(N)                                                                                          \
  case N:                                                                                                        \
    if (out_dtype == B200_F32)                                                                                   \
      B200_CUDA_OK(launch_pdl(rmsnorm_warp_kernel<float, N>, dim3(grid), dim3(256), 0, stream, x, gain, (float*)y, \
                              rinv, rows, dim, eps));                                                            \
    else                                                                                                         \
      B200_CUDA_OK(launch_pdl(rmsnorm_warp_kernel<bf16, N>, dim3(grid), dim3(256), 0, stream, x, gain, (bf16*)y,  \
                              rinv, rows, dim, eps));                                                            \
    break;
    switch (nch) {
      B200_RN_CASE(1) B200_RN_CASE(2) B200_RN_CASE(3) B200_RN_CASE(4)
      B200_RN_CASE(5) B200_RN_CASE(6) B200_RN_CASE(7) B200_RN_CASE(8)
    }
#undef B200_RN_CASE
    B200_LAUNCH_OK("rmsnorm_warp_kernel");
    return B200_OK;
  }
  int threads = ((dim / 8 + 31) / 32) * 32;
  if (threads > 256) threads = 256;
  if (out_dtype == B200_F32)
    rmsnorm_kernel<float><<<rows, threads, 0, stream>>>(x, gain, (float*)y, rinv, dim, eps);
  else if (out_dtype == B200_BF16)
    rmsnorm_kernel<bf16><<<rows, threads, 0, stream>>>(x, gain, (bf16*)y, rinv, dim, eps);
  else
    return fail(B200_ERR_BAD_DTYPE, "rmsnorm: unsupported dtype %d", out_dtype);
  B200_LAUNCH_OK("rmsnorm_kernel");
  return B200_OK;
}

int32_t launch_add_to_f32(float* x, const void* delta, int dtype, size_t n, cudaStream_t stream) {
  if (n % 8) return fail(B200_ERR_BAD_SHAPE, "add: count must be a multiple of 8");
  if (dtype == B200_F32)
    add_to_f32_kernel<float><<<grid_for(n / 8, 256), 256, 0, stream>>>(x, (const float*)delta, n / 8);
  else
    add_to_f32_kernel<bf16><<<grid_for(n / 8, 256), 256, 0, stream>>>(x, (const bf16*)delta, n / 8);
  B200_LAUNCH_OK("add_to_f32_kernel");
  return B200_OK;
}

int32_t launch_copy_rows(const void* src, int sd, int src_ld, void* dst, int dd, int dst_ld, int rows, int cols,
                         int group, int gstride, int goff, cudaStream_t stream) {
  if (cols % 8 || src_ld % 8 || dst_ld % 8) return fail(B200_ERR_BAD_SHAPE, "copy_rows: widths must be multiples of 8");
  const int g = grid_for((size_t)rows * (cols / 8), 256);
  DISPATCH2(sd, dd, (copy_rows_kernel<TS, TD><<<g, 256, 0, stream>>>((const TS*)src, src_ld, (TD*)dst, dst_ld, rows,
                                                                      cols, group, gstride, goff)));
  B200_LAUNCH_OK("copy_rows_kernel");
  return B200_OK;
}

int32_t launch_transpose(const void* src, int sd, int src_ld, void* dst, int dd, int dst_ld, int rows, int cols,
                         cudaStream_t stream) {
  dim3 grid(cdiv(cols, 32), cdiv(rows, 32)), block(32, 8);
  DISPATCH2(sd, dd, (transpose_kernel<TS, TD><<<grid, block, 0, stream>>>((const TS*)src, src_ld, (TD*)dst, dst_ld,
                                                                           rows, cols)));
  B200_LAUNCH_OK("transpose_kernel");
  return B200_OK;
}

int32_t launch_rope_table(float* cos_t, float* sin_t, int n_pos, int head_size, float theta, cudaStream_t stream) {
  const int half = head_size / 2, n = n_pos * half;
  rope_table_kernel<<<cdiv(n, 256), 256, 0, stream>>>(cos_t, sin_t, n_pos, half, head_size, theta);
  B200_LAUNCH_OK("rope_table_kernel");
  return B200_OK;
}

int rmsnorm_bwd_parts(int rows) {
  const int cap = sm_count() * 4;
  return rows < cap ? rows : cap;
}

int32_t launch_rmsnorm_bwd(const float* x, const float* gain, const float* rinv, const void* dy, int dy_dtype,
                           float* dx, int accumulate_dx, void* dx_copy, float* dg_part, int n_parts, int rows, int dim,
                           cudaStream_t stream) {
  if (dim % 8 || dim > RB_THREADS * 8 * RB_MAXCH)
    return fail(B200_ERR_BAD_SHAPE, "rmsnorm backward: dim=%d must be a multiple of 8 and at most %d", dim,
                RB_THREADS * 8 * RB_MAXCH);
  const int rpp = cdiv(rows, n_parts);
  if (cdiv(rows, rpp) > n_parts) return fail(B200_ERR_INVALID_ARG, "rmsnorm backward: bad partition");
  if (dim <= 1536) {  // 8 warps x dim floats of shared memory stay within the default 48 KB
    const int nch = cdiv(dim, 256);
    const size_t smem = (size_t)RW_WARPS * dim * sizeof(float);
#define B200_RW_CASE(N)                                                                                              \
  case N:                                                                                                            \
    if (dy_dtype == B200_F32)                                                                                        \
      B200_CUDA_OK(launch_pdl(rmsnorm_bwd_warp_kernel<float, N>, dim3(n_parts), dim3(RW_WARPS * 32), smem, stream,   \
          x, gain, rinv, (const float*)dy, dx, accumulate_dx, (float*)dx_copy, dg_part, rows, dim, rpp));                              \
    else                                                                                                             \
      B200_CUDA_OK(launch_pdl(rmsnorm_bwd_warp_kernel<bf16, N>, dim3(n_parts), dim3(RW_WARPS * 32), smem, stream,    \
          x, gain, rinv, (const bf16*)dy, dx, accumulate_dx, (bf16*)dx_copy, dg_part, rows, dim, rpp));                               \
    break;
    switch (nch) {
      B200_RW_CASE(1) B200_RW_CASE(2) B200_RW_CASE(3) B200_RW_CASE(4) B200_RW_CASE(5) B200_RW_CASE(6)
    }
#undef B200_RW_CASE
    B200_LAUNCH_OK("rmsnorm_bwd_warp_kernel");
    return B200_OK;
  }
  // Parts beyond the last row still write zeros so that the column sum may read all of them.
  if (dy_dtype == B200_F32)
    rmsnorm_bwd_kernel<float><<<n_parts, RB_THREADS, 0, stream>>>(x, gain, rinv, (const float*)dy, dx, accumulate_dx,
                                                                  (float*)dx_copy, dg_part, rows, dim, rpp);
  else
    rmsnorm_bwd_kernel<bf16><<<n_parts, RB_THREADS, 0, stream>>>(x, gain, rinv, (const bf16*)dy, dx, accumulate_dx,
                                                                 (bf16*)dx_copy, dg_part, rows, dim, rpp);
  B200_LAUNCH_OK("rmsnorm_bwd_kernel");
  return B200_OK;
}

int32_t launch_colsum_parts(const float* part, int n_parts, int dim, float* out, int accumulate,
                            cudaStream_t stream) {
  colsum_parts_kernel<<<cdiv(dim, 32), 256, 0, stream>>>(part, n_parts, dim, out, accumulate);
  B200_LAUNCH_OK("colsum_parts_kernel");
  return B200_OK;
}

int32_t launch_rope_bwd(void* dqkv, int dtype, int ld, int rows, int rope_cols, int head_size, int seq_len,
                        const float* cos_t, const float* sin_t, cudaStream_t stream) {
  if (rope_cols % 8) return fail(B200_ERR_BAD_SHAPE, "rope backward: width must be a multiple of 8");
  const int g = grid_for((size_t)rows * (rope_cols / 8), 256);
  if (dtype == B200_F32)
    B200_CUDA_OK(launch_pdl(rope_bwd_kernel<float>, dim3(g), dim3(256), 0, stream, (float*)dqkv, ld, rows, rope_cols,
                            head_size, seq_len, cos_t, sin_t));
  else
    B200_CUDA_OK(launch_pdl(rope_bwd_kernel<bf16>, dim3(g), dim3(256), 0, stream, (bf16*)dqkv, ld, rows, rope_cols,
                            head_size, seq_len, cos_t, sin_t));
  B200_LAUNCH_OK("rope_bwd_kernel");
  return B200_OK;
}

int32_t launch_swiglu_bwd(const void* gate, const void* up, const void* dh, void* dgu, int dtype, int rows, int hidden,
                          cudaStream_t stream) {
  if (hidden % 8) return fail(B200_ERR_BAD_SHAPE, "swiglu backward: hidden must be a multiple of 8");
  const int g = grid_for((size_t)rows * (hidden / 8), 256);
  if (dtype == B200_F32)
    B200_CUDA_OK(launch_pdl(swiglu_bwd_kernel<float>, dim3(g), dim3(256), 0, stream, (const float*)gate, (const float*)up,
                            (const float*)dh, (float*)dgu, rows, hidden));
  else
    B200_CUDA_OK(launch_pdl(swiglu_bwd_kernel<bf16>, dim3(g), dim3(256), 0, stream, (const bf16*)gate, (const bf16*)up,
                            (const bf16*)dh, (bf16*)dgu, rows, hidden));
  B200_LAUNCH_OK("swiglu_bwd_kernel");
  return B200_OK;
}

int32_t launch_embed_bwd(const int32_t* tokens, const float* dx, float* dtable, int n_tokens, int dim, int vocab,
                         cudaStream_t stream) {
  if (dim % 4) return fail(B200_ERR_BAD_SHAPE, "embedding backward: dim must be a multiple of 4");
  int ctas = sm_count() * 4;
  if (ctas > vocab) ctas = vocab;
  const int rpc = cdiv(vocab, ctas);
  embed_bwd_kernel<<<cdiv(vocab, rpc), 256, 0, stream>>>(tokens, dx, dtable, n_tokens, dim, vocab, rpc);
  B200_LAUNCH_OK("embed_bwd_kernel");
  return B200_OK;
}

int32_t launch_convert(const void* src, int sd, void* dst, int dd, size_t n, cudaStream_t stream) {
  if (n % 8) return fail(B200_ERR_BAD_SHAPE, "convert: count must be a multiple of 8");
  const int g = grid_for(n / 8, 256);
  DISPATCH2(sd, dd, (convert_kernel<TS, TD><<<g, 256, 0, stream>>>((const TS*)src, (TD*)dst, n / 8)));
  B200_LAUNCH_OK("convert_kernel");
  return B200_OK;
}

int32_t launch_zero_f32(float* x, size_t n, cudaStream_t stream) {
  if (n % 4) return fail(B200_ERR_BAD_SHAPE, "zero: count must be a multiple of 4");
  zero_kernel<<<grid_for(n / 4, 256), 256, 0, stream>>>(reinterpret_cast<float4*>(x), n / 4);
  B200_LAUNCH_OK("zero_kernel");
  return B200_OK;
}

int32_t launch_argmax_rows(const float* x, int rows, int cols, int ld, int32_t* out, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || ld < cols) return fail(B200_ERR_BAD_SHAPE, "argmax: rows=%d cols=%d ld=%d", rows, cols, ld);
  B200_CUDA_OK(launch_pdl(argmax_rows_kernel, dim3(rows), dim3(256), 0, stream, x, cols, ld, out));
  B200_LAUNCH_OK("argmax_rows_kernel");
  return B200_OK;
}

}  // namespace b200
