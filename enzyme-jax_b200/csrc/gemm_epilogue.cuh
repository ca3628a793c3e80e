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

// 16 consecutive outputs of one row: full 32-byte sectors per access where the
// address allows it (one for bf16, two for fp32).
__device__ __forceinline__ void store16(float* p, const float (&v)[16]) {
  float lo[8], hi[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { lo[i] = v[i]; hi[i] = v[8 + i]; }
  store8_wide(p, lo);
  store8_wide(p + 8, hi);
}
__device__ __forceinline__ void store16(bf16* p, const float (&v)[16]) {
  if (aligned32(p)) {
    uint32_t r[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      r[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    store32B(p, r);
  } else {
    float lo[8], hi[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { lo[i] = v[i]; hi[i] = v[8 + i]; }
    store8(p, lo);
    store8(p + 8, hi);
  }
}

// Per-row state computed once per output tile row (not once per 16 columns).
struct EpiRow {
  const float* rope_c = nullptr;  // cos/sin rows of this row's position
  const float* rope_s = nullptr;
};

template <int KIND>
__device__ __forceinline__ EpiRow epi_row_begin(const EpiParams& p, int m) {
  EpiRow r;
  if constexpr (KIND == EPI_ROPE) {
    const int pos = p.pos_base + (m % p.seq_len);
    const size_t off = (size_t)pos * (p.head_size >> 1);
    r.rope_c = p.rope_cos + off;
    r.rope_s = p.rope_sin + off;
  }
  return r;
}

template <int KIND, typename TOut>
__device__ __forceinline__ void epi_apply16(const EpiParams& p, const EpiRow& row, int m, int n, float (&v)[16]) {
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
      // the 16 columns lie inside one head (head sizes are multiples of 16):
      // pairs j0 .. j0+7 of that head, read as two 16-byte pieces per table
      const int j0 = (n % p.head_size) >> 1;
      float c[8], s[8];
      load8(row.rope_c + j0, c);
      load8(row.rope_s + j0, s);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float e = v[2 * i], o = v[2 * i + 1];
        v[2 * i] = c[i] * e - s[i] * o;
        v[2 * i + 1] = s[i] * e + c[i] * o;
      }
    }
    store16(reinterpret_cast<TOut*>(p.out) + (size_t)m * p.ldo + n, v);
  } else if constexpr (KIND == EPI_RESID) {
    float* x = reinterpret_cast<float*>(p.out) + (size_t)m * p.ldo + n;
    const float* xi = p.resid_in + (size_t)m * p.ldo + n;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float old[8];
      load8_wide(xi + 8 * h, old);
#pragma unroll
      for (int i = 0; i < 8; ++i) old[i] += v[8 * h + i];
      store8_wide(x + 8 * h, old);
    }
  } else {  // EPI_SWIGLU
    const size_t off = (size_t)m * p.ldo + (n >> 1);
    float g[8], u[8], h[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      g[i] = v[i];
      u[i] = v[8 + i];
      h[i] = g[i] / (1.f + exp_by_build(-g[i])) * u[i];
    }
    store8(reinterpret_cast<TOut*>(p.out) + off, h);
    if (p.out_gate) {
      store8(reinterpret_cast<TOut*>(p.out_gate) + off, g);
      store8(reinterpret_cast<TOut*>(p.out_up) + off, u);
    }
  }
}

// Tile order of the persistent tensor-core kernels: bands of GM row-tiles are
// walked column-tile by column-tile, so that the tiles in flight at any time
// share a few row-tiles of A and a few column-tiles of B (both stay in L2 even
// when a whole operand does not fit).
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int gm, int& mt, int& nt) {
  const int per_band = gm * n_tiles;
  const int band = tile / per_band;
  const int r = tile - band * per_band;
  const int rows = min(gm, m_tiles - band * gm);  // the last band may be short
  nt = r / rows;
  mt = band * gm + r % rows;
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
  // optional scratch for K-split partial sums (fp32); null disables splitting
  void* splitk_scratch = nullptr;
  size_t splitk_bytes = 0;
  // upper bound on the persistent grid (0 = every SM); lets a collective on another stream keep some SMs
  int max_ctas = 0;
  // Row-parallel projection of a tensor-parallel plan: rows [o * push_rows, (o + 1) * push_rows) of the output are
  // stored to push_base[o], a [push_rows, N] matrix of row pitch epi.ldo (memory of rank o, mapped into this
  // process), instead of epi.out: the partial product crosses NVLink tile by tile while the GEMM still computes.
  // Only the CTA-pair tensor kernel with the plain store does this; ask gemm_push_supported first.
  int push_rows = 0;
  void* push_base[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  // Column-parallel projection of a tensor-parallel plan whose A operand arrives in bands of band_rows rows, band o
  // written by rank o: before it first loads rows of band o the kernel waits (bounded by band_budget SM clocks)
  // until band_flags[o] has reached band_epoch, and it starts with the tiles of band band_first, whose rows are
  // already there.  Only the CTA-pair tensor kernel does this; ask gemm_bands_supported first.
  const uint32_t* band_flags = nullptr;
  uint32_t band_epoch = 0;
  int band_rows = 0, band_first = 0;
  long long band_budget = 0;
};
// whether launch_gemm(g, impl) would take the kernel that honours band_flags (see GemmArgs)
bool gemm_bands_supported(const GemmArgs& g, int impl);
// whether launch_gemm(g, impl) would take the kernel that honours push_rows / push_base
bool gemm_push_supported(const GemmArgs& g, int impl);
// Scratch that lets the tensor-core kernel split K whenever it wants to for an M x N output.
inline size_t gemm_splitk_scratch_bytes(int M, int N) { return (size_t)32 * M * N * sizeof(float); }

int32_t launch_gemm_simt(const GemmArgs& g, cudaStream_t stream);
int32_t launch_gemm_tc(const GemmArgs& g, cudaStream_t stream);
// Picks the tensor-core kernel when it covers the problem, else FFMA.
int32_t launch_gemm(const GemmArgs& g, int impl, cudaStream_t stream);
bool gemm_tc_supports(const GemmArgs& g);
int32_t launch_bounded_wait_selftest(long long budget_cycles, uint32_t* reached_end, cudaStream_t stream);
// CTA-pair (cta_group::2) variant for large K-major problems
int32_t launch_gemm_tc2(const GemmArgs& g, cudaStream_t stream);
bool gemm_tc2_supports(const GemmArgs& g);
// CTA-pair variant for weight gradients (both operands MN-major, fp32 out, K cut into ranges through the scratch)
int32_t launch_gemm_tc2_mn(const GemmArgs& g, cudaStream_t stream);
bool gemm_tc2_mn_supports(const GemmArgs& g);
// sums `splits` partial [M, N] fp32 results in g.splitk_scratch in split order and applies g's store epilogue
int32_t launch_splitk_reduce(const GemmArgs& g, int splits, cudaStream_t stream);

}  // namespace b200
