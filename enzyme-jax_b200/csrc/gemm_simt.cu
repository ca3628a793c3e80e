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

// Column c of the 64-wide B tile lives at shared-memory column bcol(c): the four 4-column groups that the four
// threads of a row group read in one instruction (columns 16 tx + 4 q, tx = 0..3) sit side by side (16 q + 4 tx), so
// that the instruction touches 64 contiguous bytes instead of four segments two of which share their banks.
__device__ __forceinline__ int bcol(int c) { return ((c >> 2) & 3) * 16 + (c >> 4) * 4 + (c & 3); }

// RPT is 4 (128-row tiles) or 1 (32-row tiles)
template <typename TIn, typename TOut, int KIND, bool TA, bool TB, bool VEC, int RPT>
__global__ void __launch_bounds__(NT) gemm_simt_kernel(const TIn* __restrict__ A, const TIn* __restrict__ B, int M,
                                                       int N, int K, int lda, int ldb, EpiParams ep) {
  constexpr int BM = 32 * RPT;
  // k-elements per shared-memory tile: 64 for the small-problem form (32-row tiles, 4 x 4 results per thread in the k
  // loop), 16 for the 128-row form.  Both forms are bound by shared-memory delivery, not by the FMA pipe: a 16-byte
  // load hands a warp 512 bytes in four passes whatever the lanes share, so 16 FMAs per two loads (small form) keep the
  // FMA pipe about a third busy and 64 per five loads (large form) about half; only wider register blocks would
  // change that, and the small form exists to have many CTAs.
  constexpr int BKT = RPT == 1 ? 64 : BK;
  constexpr int NTH = NT;
  __shared__ __align__(16) float As[BKT][BM + 4];
  __shared__ __align__(16) float Bs[BKT][BN + 4];
  const int tid = threadIdx.x;
  const int ty = tid >> 2, tx = tid & 3;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  pdl_launch_dependents();
  pdl_wait();

  float acc[RPT][16];
#pragma unroll
  for (int r = 0; r < RPT; ++r)
#pragma unroll
    for (int c = 0; c < 16; ++c) acc[r][c] = 0.f;

  // Global loads of k-tile i+1 are issued before the FMAs of k-tile i and land in registers meanwhile.  K-major
  // operands: consecutive threads take consecutive ROWS of the tile (one 8-element piece of a row each), so that the
  // transposing stores of a warp go to consecutive shared-memory words.
  constexpr int A_ITEMS = BM * BKT / 8 / NTH;  // 8-element pieces of the A tile per thread
  constexpr int B_ITEMS = BN * BKT / 8 / NTH;
  static_assert(BM * BKT % (8 * NTH) == 0 && BN * BKT % (8 * NTH) == 0, "tile pieces must divide over the threads");
  float va[A_ITEMS][8], vb[B_ITEMS][8];
  auto fetch_tile = [&](int k0) {
#pragma unroll
    for (int it = 0; it < A_ITEMS; ++it) {
      const int idx = tid + it * NTH;
      if constexpr (!TA) {
        const int row = idx % BM, k8 = (idx / BM) * 8;
        fetch8<TIn, VEC>(A, lda, m0 + row, k0 + k8, M, K, va[it]);
      } else {
        const int k = idx / (BM / 8), m8 = (idx % (BM / 8)) * 8;
        fetch8<TIn, VEC>(A, lda, k0 + k, m0 + m8, K, M, va[it]);
      }
    }
#pragma unroll
    for (int it = 0; it < B_ITEMS; ++it) {
      const int idx = tid + it * NTH;
      if constexpr (!TB) {
        const int row = idx % BN, k8 = (idx / BN) * 8;
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
      const int idx = tid + it * NTH;
      if constexpr (!TA) {
        const int row = idx % BM, k8 = (idx / BM) * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) As[k8 + j][row] = va[it][j];
      } else {
        const int k = idx / (BM / 8), m8 = (idx % (BM / 8)) * 8;
        *reinterpret_cast<float4*>(&As[k][m8]) = make_float4(va[it][0], va[it][1], va[it][2], va[it][3]);
        *reinterpret_cast<float4*>(&As[k][m8 + 4]) = make_float4(va[it][4], va[it][5], va[it][6], va[it][7]);
      }
    }
#pragma unroll
    for (int it = 0; it < B_ITEMS; ++it) {
      const int idx = tid + it * NTH;
      if constexpr (!TB) {
        const int row = idx % BN, k8 = (idx / BN) * 8;
        const int col = RPT == 1 ? row : bcol(row);
#pragma unroll
        for (int j = 0; j < 8; ++j) Bs[k8 + j][col] = vb[it][j];
      } else {
        const int k = idx / (BN / 8), n8 = (idx % (BN / 8)) * 8;
        const int c0 = RPT == 1 ? n8 : bcol(n8), c1 = RPT == 1 ? n8 + 4 : bcol(n8 + 4);
        *reinterpret_cast<float4*>(&Bs[k][c0]) = make_float4(vb[it][0], vb[it][1], vb[it][2], vb[it][3]);
        *reinterpret_cast<float4*>(&Bs[k][c1]) = make_float4(vb[it][4], vb[it][5], vb[it][6], vb[it][7]);
      }
    }
  };

  fetch_tile(0);
  if constexpr (RPT == 1) {
    // Small form: during the k loop a thread owns a 4 x 4 block (rows 4 cy.., columns 4 cx..), i.e. two 16-byte
    // shared-memory loads per 16 FMAs; the blocks then go through shared memory so that the epilogue sees one row
    // and 16 consecutive columns per thread like the large form.  Every element is still one fmaf chain in k order.
    const int cx = tid & 15, cy = tid >> 4;
    float c4[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) c4[r][c] = 0.f;
    for (int k0 = 0; k0 < K; k0 += BKT) {
      store_tile();
      __syncthreads();
      if (k0 + BKT < K) fetch_tile(k0 + BKT);
#pragma unroll 32
      for (int k = 0; k < BKT; ++k) {
        const float4 a4 = *reinterpret_cast<const float4*>(&As[k][cy * 4]);
        const float4 b4 = *reinterpret_cast<const float4*>(&Bs[k][cx * 4]);
        const float a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int c = 0; c < 4; ++c) c4[r][c] = fmaf(a[r], b[c], c4[r][c]);
      }
      __syncthreads();
    }
    float(*Cs)[BN + 4] = Bs;  // 32 x 64 results in the B tile's memory (free after the loop's last barrier)
#pragma unroll
    for (int r = 0; r < 4; ++r)
      *reinterpret_cast<float4*>(&Cs[cy * 4 + r][cx * 4]) = make_float4(c4[r][0], c4[r][1], c4[r][2], c4[r][3]);
    __syncthreads();
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 v = *reinterpret_cast<const float4*>(&Cs[ty][tx * 16 + q * 4]);
      acc[0][q * 4 + 0] = v.x; acc[0][q * 4 + 1] = v.y; acc[0][q * 4 + 2] = v.z; acc[0][q * 4 + 3] = v.w;
    }
  } else {
    for (int k0 = 0; k0 < K; k0 += BKT) {
      store_tile();
      __syncthreads();
      if (k0 + BKT < K) fetch_tile(k0 + BKT);
#pragma unroll 16
      for (int k = 0; k < BKT; ++k) {
        const float4 a4 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
        const float a[4] = {a4.x, a4.y, a4.z, a4.w};
        float b[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 b4 = *reinterpret_cast<const float4*>(&Bs[k][q * 16 + tx * 4]);
          b[q * 4 + 0] = b4.x; b[q * 4 + 1] = b4.y; b[q * 4 + 2] = b4.z; b[q * 4 + 3] = b4.w;
        }
#pragma unroll
        for (int r = 0; r < RPT; ++r)
#pragma unroll
          for (int c = 0; c < 16; ++c) acc[r][c] = fmaf(a[r], b[c], acc[r][c]);
      }
      __syncthreads();
    }
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
#define B200_SIMT_LAUNCH(V, R)                                                                               \
  B200_CUDA_OK(launch_pdl(gemm_simt_kernel<TIn, TOut, KIND, TA, TB, V, R>, grid, dim3(NT), 0, stream, (const TIn*)g.A, \
                          (const TIn*)g.B, g.M, g.N, g.K, g.lda, g.ldb, g.epi))
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
