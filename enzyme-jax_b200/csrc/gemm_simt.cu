// FFMA GEMM: Y[M,N] = op(A) * op(B)^T with fp32 accumulation on the CUDA cores.
//
// This is the exact-fp32 path (the fp32 configuration needs products that are
// not rounded to tf32/bf16) and the kernel that covers operand layouts or
// shapes the tensor-core kernel does not.  128x64 output tile per CTA of 128
// threads; each thread owns 4 rows x 16 consecutive columns so that the fused
// epilogues see 16-column groups.
#include "gemm_epilogue.cuh"

namespace b200 {

namespace {

constexpr int BN = 64, BK = 16, NT = 128;  // rows per CTA: 32 * RPT (RPT rows per thread)

template <typename TIn, bool VEC>
__device__ __forceinline__ void fetch8(const TIn* base, int ld, int r, int c, int R, int C, float (&v)[8]) {
  // 8 consecutive elements of row r starting at column c of an [R, C] matrix; zero outside.
  if (VEC && r < R && c + 8 <= C) {
    load8(base + (size_t)r * ld + c, v);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (r < R && c + i < C) ? to_f32(base[(size_t)r * ld + c + i]) : 0.f;
  }
}

template <typename TIn, typename TOut, int KIND, bool TA, bool TB, bool VEC, int RPT>
__global__ void __launch_bounds__(NT) gemm_simt_kernel(const TIn* __restrict__ A, const TIn* __restrict__ B, int M,
                                                       int N, int K, int lda, int ldb, EpiParams ep) {
  constexpr int BM = 32 * RPT;
  // k-elements per shared-memory tile.  The small-problem form (32-row tiles, a handful of CTAs per SM, 16 FMAs per
  // k-step and thread) is bound by the round trip of each tile's global loads, so it takes 64 at a time: a 288-deep
  // product is 5 trips instead of 18.
  constexpr int BKT = RPT == 1 ? 64 : BK;
  __shared__ __align__(16) float As[BKT][BM + 4];
  __shared__ __align__(16) float Bs[BKT][BN + 4];
  const int tid = threadIdx.x;
  const int ty = tid >> 2, tx = tid & 3;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  float acc[RPT][16];
#pragma unroll
  for (int r = 0; r < RPT; ++r)
#pragma unroll
    for (int c = 0; c < 16; ++c) acc[r][c] = 0.f;

  // Global loads of k-tile i+1 are issued before the FMAs of k-tile i and land in registers meanwhile.
  constexpr int A_ITEMS = BM * BKT / 8 / NT;  // 8-element pieces of the A tile per thread
  constexpr int B_ITEMS = BN * BKT / 8 / NT;
  static_assert(BM * BKT % (8 * NT) == 0 && BN * BKT % (8 * NT) == 0, "tile pieces must divide over the threads");
  float va[A_ITEMS][8], vb[B_ITEMS][8];
  auto fetch_tile = [&](int k0) {
#pragma unroll
    for (int it = 0; it < A_ITEMS; ++it) {
      const int idx = tid + it * NT;
      if constexpr (!TA) {
        const int row = idx / (BKT / 8), k8 = (idx % (BKT / 8)) * 8;
        fetch8<TIn, VEC>(A, lda, m0 + row, k0 + k8, M, K, va[it]);
      } else {
        const int k = idx / (BM / 8), m8 = (idx % (BM / 8)) * 8;
        fetch8<TIn, VEC>(A, lda, k0 + k, m0 + m8, K, M, va[it]);
      }
    }
#pragma unroll
    for (int it = 0; it < B_ITEMS; ++it) {
      const int idx = tid + it * NT;
      if constexpr (!TB) {
        const int row = idx / (BKT / 8), k8 = (idx % (BKT / 8)) * 8;
        fetch8<TIn, VEC>(B, ldb, n0 + row, k0 + k8, N, K, vb[it]);
      } else {
        const int k = idx / (BN / 8), n8 = (idx % (BN / 8)) * 8;
        fetch8<TIn, VEC>(B, ldb, k0 + k, n0 + n8, K, N, vb[it]);
      }
    }
  };
  auto store_tile = [&]() {
#pragma unroll
    for (int it = 0; it < A_ITEMS; ++it) {
      const int idx = tid + it * NT;
      if constexpr (!TA) {
        const int row = idx / (BKT / 8), k8 = (idx % (BKT / 8)) * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) As[k8 + j][row] = va[it][j];
      } else {
        const int k = idx / (BM / 8), m8 = (idx % (BM / 8)) * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) As[k][m8 + j] = va[it][j];
      }
    }
#pragma unroll
    for (int it = 0; it < B_ITEMS; ++it) {
      const int idx = tid + it * NT;
      if constexpr (!TB) {
        const int row = idx / (BKT / 8), k8 = (idx % (BKT / 8)) * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) Bs[k8 + j][row] = vb[it][j];
      } else {
        const int k = idx / (BN / 8), n8 = (idx % (BN / 8)) * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) Bs[k][n8 + j] = vb[it][j];
      }
    }
  };

  fetch_tile(0);
  for (int k0 = 0; k0 < K; k0 += BKT) {
    store_tile();
    __syncthreads();
    if (k0 + BKT < K) fetch_tile(k0 + BKT);
#pragma unroll 16
    for (int k = 0; k < BKT; ++k) {
      float a[RPT];
#pragma unroll
      for (int r = 0; r < RPT; ++r) a[r] = As[k][ty * RPT + r];
      float b[16];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float4 b4 = *reinterpret_cast<const float4*>(&Bs[k][tx * 16 + q * 4]);
        b[q * 4 + 0] = b4.x; b[q * 4 + 1] = b4.y; b[q * 4 + 2] = b4.z; b[q * 4 + 3] = b4.w;
      }
#pragma unroll
      for (int r = 0; r < RPT; ++r)
#pragma unroll
        for (int c = 0; c < 16; ++c) acc[r][c] = fmaf(a[r], b[c], acc[r][c]);
    }
    __syncthreads();
  }

  const int n = n0 + tx * 16;
  if (n < N) {
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      const int m = m0 + ty * RPT + r;
      if (m < M) {
        const EpiRow row = epi_row_begin<KIND>(ep, m);
        epi_apply16<KIND, TOut>(ep, row, m, n, acc[r]);
      }
    }
  }
}

template <typename TIn, typename TOut, int KIND, bool TA, bool TB>
int32_t launch_t(const GemmArgs& g, cudaStream_t stream) {
  const bool vec = aligned16(g.A) && aligned16(g.B) && (g.lda % 8 == 0) && (g.ldb % 8 == 0);
  // 128-row tiles when they fill the machine, 32-row tiles (4x the CTAs) for small problems
  const bool small = (long)cdiv(g.M, 128) * cdiv(g.N, BN) < 2L * sm_count();
  const int bm = small ? 32 : 128;
  dim3 grid(cdiv(g.N, BN), cdiv(g.M, bm));
#define B200_SIMT_LAUNCH(V, R)                                                           \
  gemm_simt_kernel<TIn, TOut, KIND, TA, TB, V, R><<<grid, NT, 0, stream>>>(              \
      (const TIn*)g.A, (const TIn*)g.B, g.M, g.N, g.K, g.lda, g.ldb, g.epi)
  if (vec && small) B200_SIMT_LAUNCH(true, 1);
  else if (vec) B200_SIMT_LAUNCH(true, 4);
  else if (small) B200_SIMT_LAUNCH(false, 1);
  else B200_SIMT_LAUNCH(false, 4);
#undef B200_SIMT_LAUNCH
  B200_LAUNCH_OK("gemm_simt_kernel");
  return B200_OK;
}

template <typename TIn, typename TOut>
int32_t launch_io(const GemmArgs& g, cudaStream_t stream) {
  if (g.kind == EPI_STORE) {
    if (!g.ta && !g.tb) return launch_t<TIn, TOut, EPI_STORE, false, false>(g, stream);
    if (!g.ta && g.tb) return launch_t<TIn, TOut, EPI_STORE, false, true>(g, stream);
    if (g.ta && !g.tb) return launch_t<TIn, TOut, EPI_STORE, true, false>(g, stream);
    return launch_t<TIn, TOut, EPI_STORE, true, true>(g, stream);
  }
  if (g.ta || g.tb) return fail(B200_ERR_UNSUPPORTED, "fused epilogues need both operands K-major");
  switch (g.kind) {
    case EPI_ROPE: return launch_t<TIn, TOut, EPI_ROPE, false, false>(g, stream);
    case EPI_RESID: return launch_t<TIn, TOut, EPI_RESID, false, false>(g, stream);
    case EPI_SWIGLU: return launch_t<TIn, TOut, EPI_SWIGLU, false, false>(g, stream);
  }
  return fail(B200_ERR_INVALID_ARG, "unknown epilogue kind %d", g.kind);
}

}  // namespace

int32_t launch_gemm_simt(const GemmArgs& g, cudaStream_t stream) {
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return fail(B200_ERR_BAD_SHAPE, "gemm: empty problem %dx%dx%d", g.M, g.N, g.K);
  if (g.N % 16) return fail(B200_ERR_BAD_SHAPE, "gemm: N=%d must be a multiple of 16", g.N);
  if (g.epi.ldo % 8 || !aligned16(g.epi.out)) return fail(B200_ERR_MISALIGNED, "gemm: output not 16-byte aligned");
  if (g.in_dtype == B200_F32 && g.out_dtype == B200_F32) return launch_io<float, float>(g, stream);
  if (g.in_dtype == B200_BF16 && g.out_dtype == B200_BF16) return launch_io<bf16, bf16>(g, stream);
  if (g.in_dtype == B200_BF16 && g.out_dtype == B200_F32) return launch_io<bf16, float>(g, stream);
  return fail(B200_ERR_BAD_DTYPE, "gemm: unsupported dtype pair in=%d out=%d", g.in_dtype, g.out_dtype);
}

}  // namespace b200
