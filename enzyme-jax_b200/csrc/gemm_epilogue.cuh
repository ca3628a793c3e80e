// Fused GEMM epilogues shared by the tcgen05 and the FFMA GEMM kernels.
//
// Every epilogue consumes one output row `m` and 16 consecutive fp32
// accumulator columns starting at `n` (n % 16 == 0, N % 16 == 0).
#pragma once

#include "common.cuh"

namespace b200 {

enum EpiKind : int {
  EPI_STORE = 0,   // out[m,n] (+)= acc
  EPI_ROPE = 1,    // rotate adjacent pairs of the first rope_cols columns, then store
  EPI_RESID = 2,   // fp32 residual stream: out[m,n] = resid_in[m,n] + acc (in place when equal)
  EPI_SWIGLU = 3,  // columns come as [8 x gate | 8 x up]; out[m, n/2 + i] = silu(gate_i) * up_i
};

struct EpiParams {
  void* out = nullptr;
  int ldo = 0;
  int accumulate = 0;
  // EPI_ROPE: rotation angle of row m is position pos_base + (m % seq_len);
  // tables are [positions, head_size/2] fp32 (test/llama.py:127-140).
  const float* rope_cos = nullptr;
  const float* rope_sin = nullptr;
  int seq_len = 1;
  int pos_base = 0;
  int head_size = 2;
  int rope_cols = 0;
  // EPI_RESID: fp32 [M, ldo] read side of the residual add (may alias out)
  const float* resid_in = nullptr;
  // EPI_SWIGLU: optional copies of the gate and up pre-activations, [M, ldo]
  void* out_gate = nullptr;
  void* out_up = nullptr;
};

template <typename TOut>
__device__ __forceinline__ void store16(TOut* p, const float (&v)[16]) {
  float lo[8], hi[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { lo[i] = v[i]; hi[i] = v[8 + i]; }
  store8(p, lo);
  store8(p + 8, hi);
}

template <int KIND, typename TOut>
__device__ __forceinline__ void epi_apply16(const EpiParams& p, int m, int n, float (&v)[16]) {
  if constexpr (KIND == EPI_STORE) {
    TOut* o = reinterpret_cast<TOut*>(p.out) + (size_t)m * p.ldo + n;
    if (p.accumulate) {
      float old[8];
      load8(o, old);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += old[i];
      load8(o + 8, old);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[8 + i] += old[i];
    }
    store16(o, v);
  } else if constexpr (KIND == EPI_ROPE) {
    if (n < p.rope_cols) {
      const int half = p.head_size >> 1;
      const int pos = p.pos_base + (m % p.seq_len);
      const float* c = p.rope_cos + (size_t)pos * half;
      const float* s = p.rope_sin + (size_t)pos * half;
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        const int j = ((n + i) % p.head_size) >> 1;
        const float cj = c[j], sj = s[j];
        const float e = v[i], o = v[i + 1];
        v[i] = cj * e - sj * o;
        v[i + 1] = sj * e + cj * o;
      }
    }
    store16(reinterpret_cast<TOut*>(p.out) + (size_t)m * p.ldo + n, v);
  } else if constexpr (KIND == EPI_RESID) {
    float* x = reinterpret_cast<float*>(p.out) + (size_t)m * p.ldo + n;
    const float* xi = p.resid_in + (size_t)m * p.ldo + n;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float old[8];
      load8(xi + 8 * h, old);
#pragma unroll
      for (int i = 0; i < 8; ++i) old[i] += v[8 * h + i];
      store8(x + 8 * h, old);
    }
  } else {  // EPI_SWIGLU
    const size_t off = (size_t)m * p.ldo + (n >> 1);
    float g[8], u[8], h[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      g[i] = v[i];
      u[i] = v[8 + i];
      h[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
    }
    store8(reinterpret_cast<TOut*>(p.out) + off, h);
    if (p.out_gate) {
      store8(reinterpret_cast<TOut*>(p.out_gate) + off, g);
      store8(reinterpret_cast<TOut*>(p.out_up) + off, u);
    }
  }
}

// Host-side launchers (definitions in gemm_simt.cu / gemm_tc.cu).
struct GemmArgs {
  const void* A = nullptr;  // [M,K] (or [K,M] when ta)
  const void* B = nullptr;  // [N,K] (or [K,N] when tb)
  int M = 0, N = 0, K = 0;
  int lda = 0, ldb = 0;
  int ta = 0, tb = 0;
  int in_dtype = B200_BF16;
  int out_dtype = B200_BF16;
  int kind = EPI_STORE;
  EpiParams epi;
};

int32_t launch_gemm_simt(const GemmArgs& g, cudaStream_t stream);
int32_t launch_gemm_tc(const GemmArgs& g, cudaStream_t stream);
// Picks the tensor-core kernel when it covers the problem, else FFMA.
int32_t launch_gemm(const GemmArgs& g, int impl, cudaStream_t stream);
bool gemm_tc_supports(const GemmArgs& g);

}  // namespace b200
