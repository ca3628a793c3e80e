// tcgen05 / TMEM GEMM for sm_100a:  Y[M,N] = A[M,K] * B[N,K]^T, bf16 operands,
// fp32 accumulation in tensor memory, fused epilogues.
//
// One persistent CTA per SM walks output tiles of 128 x BN.  Warp roles:
//   warp 0      TMA producer: cp.async.bulk.tensor 2-D boxes (64 K-elements =
//               128 B wide, 128-byte swizzle) of A and B into a ring of stages
//   warp 1      allocates TMEM; one lane issues tcgen05.mma (128 x BN x 16 per
//               instruction) from shared-memory descriptors into one of two
//               TMEM accumulators and commits to mbarriers
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (lane = row),
//               apply the fused epilogue, store; runs while the next tile's
//               main loop fills the other accumulator
// All waits are bounded; a wait that runs out sets the device status word and
// the CTA unwinds (frees TMEM, returns).
#include <cuda.h>

#include <mutex>

#include "gemm_epilogue.cuh"
#include "ptx_sm100.cuh"
#include "plan.cuh"
#include "tensor_map.cuh"

namespace b200 {

namespace {

constexpr int TBM = 128;      // tile rows (TMEM lanes)
constexpr int TBK = 64;       // K elements per stage (128 bytes of bf16)
constexpr int UMMA_K = 16;    // K per tcgen05.mma for 16-bit operands
constexpr int TC_THREADS = 192;
constexpr int kMnBoxBytes = 64 * TBK * 2;  // one TMA box of an MN-major operand: TBK rows of 64 elements

template <int BN> struct TcCfg {
  static constexpr int kStages = (BN >= 256) ? 4 : (BN >= 128 ? 6 : 8);
  static constexpr int kABytes = TBM * TBK * 2;
  static constexpr int kBBytes = BN * TBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

enum : uint32_t {
  ST_PRODUCER_TIMEOUT = 1u << 0,
  ST_MMA_TIMEOUT = 1u << 1,
  ST_EPILOGUE_TIMEOUT = 1u << 2,
};

template <int BN, int KIND, typename TOut, bool AMN, bool BMN>
__global__ void __launch_bounds__(TC_THREADS, 1)
    gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int M, int N,
                   int K, EpiParams ep, int splits, float* __restrict__ partial, uint32_t* status) {
  using Cfg = TcCfg<BN>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  // Stage buffers must sit on 1024-byte boundaries for the 128-byte swizzle.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * Cfg::kStageBytes);
  uint64_t* full_bar = bars;                 // [S]   TMA bytes landed
  uint64_t* empty_bar = bars + S;            // [S]   MMAs reading the stage are done
  uint64_t* acc_full = bars + 2 * S;         // [2]   accumulator complete
  uint64_t* acc_empty = bars + 2 * S + 2;    // [2]   accumulator drained by the epilogue
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (M + TBM - 1) / TBM;
  const int n_tiles = (N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (K + TBK - 1) / TBK;
  // Work item w = (tile, K-split): tile = w % num_tiles, split = w / num_tiles; the
  // split covers k-blocks [split*num_kb/splits, (split+1)*num_kb/splits).
  const int num_items = num_tiles * splits;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      ptx::mbar_init(&full_bar[i], 1);
      ptx::mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&acc_full[i], 1);
      ptx::mbar_init(&acc_empty[i], 4);
    }
    *abort_flag = 0u;
    ptx::fence_barrier_init();
    ptx::tma_prefetch_desc(&tmA);
    ptx::tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();  // set-up above may overlap the previous kernel's tail; operands are touched from here on

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const int tile = item % num_tiles, split = item / num_tiles;
        int mt, nt;
        tile_coords(tile, m_tiles, n_tiles, 16, mt, nt);
        const int m0 = mt * TBM, n0 = nt * BN;
        const int kb0 = (int)((long)split * num_kb / splits), kb1 = (int)((long)(split + 1) * num_kb / splits);
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = ptx::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, status, ST_PRODUCER_TIMEOUT);
          if (!ok) break;
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          ptx::mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          if constexpr (!AMN) {
            ptx::tma_load_2d(sa, &tmA, kb * TBK, m0, &full_bar[stage]);
          } else {  // operand stored [K, M]: one 64-wide box per 64 rows of the tile
#pragma unroll
            for (int i = 0; i < TBM / 64; ++i)
              ptx::tma_load_2d(sa + i * kMnBoxBytes, &tmA, m0 + 64 * i, kb * TBK, &full_bar[stage]);
          }
          if constexpr (!BMN) {
            ptx::tma_load_2d(sa + Cfg::kABytes, &tmB, kb * TBK, n0, &full_bar[stage]);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              ptx::tma_load_2d(sa + Cfg::kABytes + i * kMnBoxBytes, &tmB, n0 + 64 * i, kb * TBK, &full_bar[stage]);
          }
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::idesc_bf16_f32(TBM, BN) | (AMN ? (1u << 15) : 0u) | (BMN ? (1u << 16) : 0u);
      // encoded (16-byte units) start-address step per 16 K-elements
      constexpr uint64_t a_step = AMN ? (16 * 128) / 16 : 2;
      constexpr uint64_t b_step = BMN ? (16 * 128) / 16 : 2;
      // descriptors of stage 0, built once: a stage adds its byte offset >> 4 to the 14-bit address field (shared-memory
      // addresses stay below 2^18, so it never carries); this thread's instruction stream is what bounds narrow tiles
      const uint32_t s0 = ptx::smem_u32(smem);
      const uint64_t a_base = AMN ? ptx::smem_desc_sw128_mn(s0, kMnBoxBytes) : ptx::smem_desc_sw128(s0);
      const uint64_t b_base = BMN ? ptx::smem_desc_sw128_mn(s0 + Cfg::kABytes, kMnBoxBytes)
                                  : ptx::smem_desc_sw128(s0 + Cfg::kABytes);
      constexpr uint64_t stage_step = Cfg::kStageBytes >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const int split = item / num_tiles;
        const int kb0 = (int)((long)split * num_kb / splits), kb1 = (int)((long)(split + 1) * num_kb / splits);
        ok = ptx::mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_flag, status, ST_MMA_TIMEOUT);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = ptx::mbar_wait(&full_bar[stage], phase, abort_flag, status, ST_MMA_TIMEOUT);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          const uint64_t adesc = a_base + (uint64_t)stage * stage_step;
          const uint64_t bdesc = b_base + (uint64_t)stage * stage_step;
#pragma unroll
          for (int k = 0; k < TBK / UMMA_K; ++k) {
            // K-major: 16 elements further along a 128-byte row = 32 bytes;
            // MN-major: 16 rows of 128 bytes further down.
            ptx::mma_bf16_ss(d_tmem, adesc + a_step * k, bdesc + b_step * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          ptx::mma_commit(&empty_bar[stage]);
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        ptx::mma_commit(&acc_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else {
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
      const int tile = item % num_tiles, split = item / num_tiles;
      int mt, nt;
      tile_coords(tile, m_tiles, n_tiles, 16, mt, nt);
      const int m0 = mt * TBM, n0 = nt * BN;
      const int m = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
      const bool row_ok = m < M;
      const EpiRow erow = epi_row_begin<KIND>(ep, row_ok ? m : 0);
      // Operands the epilogue reads from global memory are fetched BEFORE the
      // wait for the accumulator, so that their latency overlaps the main loop:
      // the residual row (first 128 columns of the tile) and, for head size 64,
      // the 32 cos/sin pairs of the row's position.
      constexpr int PRE = (KIND == EPI_RESID) ? (BN < 128 ? BN : 128) : 8;
      float rpre[PRE];
      float rc[32], rs[32];
      const bool rope64 = KIND == EPI_ROPE && ep.head_size == 64 && (BN % 64 == 0);
      if (KIND == EPI_RESID && splits == 1) {
        const float* xi = ep.resid_in + (size_t)(row_ok ? m : 0) * ep.ldo + n0;
#pragma unroll
        for (int c = 0; c < PRE; c += 8) {
          float t8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          if (row_ok && n0 + c < N) load8_wide(xi + c, t8);
#pragma unroll
          for (int i = 0; i < 8; ++i) rpre[c + i] = t8[i];
        }
      }
      if (KIND == EPI_ROPE && splits == 1) {
        if (rope64) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            float t8[8], u8[8];
            load8_wide(erow.rope_c + c, t8);
            load8_wide(erow.rope_s + c, u8);
#pragma unroll
            for (int i = 0; i < 8; ++i) { rc[c + i] = t8[i]; rs[c + i] = u8[i]; }
          }
        }
      }
      ok = ptx::mbar_wait_warp(&acc_full[acc], acc_phase, abort_flag, status, ST_EPILOGUE_TIMEOUT);
      if (!ok) break;
      ptx::tc_fence_after_sync();
      // 32 columns per TMEM round trip; the next pair of loads is in flight
      // while the current 32 columns go through the epilogue.
      float cur[2][16], nxt[2][16];
      ptx::tmem_ld16(taddr, cur[0]);
      ptx::tmem_ld16(taddr + 16u, cur[1]);
#pragma unroll
      for (int c = 0; c < BN; c += 32) {
        ptx::tmem_ld_wait();
        if (c + 32 < BN) {
          ptx::tmem_ld16(taddr + (uint32_t)(c + 32), nxt[0]);
          ptx::tmem_ld16(taddr + (uint32_t)(c + 48), nxt[1]);
        }
        if (row_ok) {
#pragma unroll
          for (int hlf = 0; hlf < 2; ++hlf) {
            const int cc = c + 16 * hlf;
            if (n0 + cc < N) {
              if (splits > 1) {  // K-split: raw fp32 partial sums, the fused epilogue runs in the reduction kernel
                store16(partial + ((size_t)split * M + m) * N + n0 + cc, cur[hlf]);
              } else if (KIND == EPI_RESID && cc < PRE) {
                float* xo = reinterpret_cast<float*>(ep.out) + (size_t)m * ep.ldo + n0 + cc;
                float lo[8], hi[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  lo[i] = rpre[(cc % PRE) + i] + cur[hlf][i];
                  hi[i] = rpre[(cc % PRE) + 8 + i] + cur[hlf][8 + i];
                }
                store8_wide(xo, lo);
                store8_wide(xo + 8, hi);
              } else if (KIND == EPI_ROPE && rope64) {
                if (n0 + cc < ep.rope_cols) {
                  const int j0 = (cc % 64) >> 1;  // compile-time after unrolling: tiles start on head boundaries
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    const float e = cur[hlf][2 * i], o = cur[hlf][2 * i + 1];
                    cur[hlf][2 * i] = rc[j0 + i] * e - rs[j0 + i] * o;
                    cur[hlf][2 * i + 1] = rs[j0 + i] * e + rc[j0 + i] * o;
                  }
                }
                store16(reinterpret_cast<TOut*>(ep.out) + (size_t)m * ep.ldo + n0 + cc, cur[hlf]);
              } else {
                epi_apply16<KIND, TOut>(ep, erow, m, n0 + cc, cur[hlf]);
              }
            }
          }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) { cur[0][i] = nxt[0][i]; cur[1][i] = nxt[1][i]; }
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&acc_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // Give copies that may still be in flight time to land before the CTA's
    // shared memory is released.
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ---- host side ---------------------------------------------------------------

// Sums the K-split partials in split order and applies the fused epilogue.
template <int KIND, typename TOut>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, int splits, int M, int N,
                                                            EpiParams ep) {
  const int per_row = N / 16;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();  // the partial sums come from the GEMM kernel before
  if (idx >= M * per_row) return;
  const int m = idx / per_row, n = (idx % per_row) * 16;
  float v[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = 0.f;
#pragma unroll 4  // the loads of four K ranges in flight together; the sum stays in range order
  for (int s = 0; s < splits; ++s) {
    const float* p = partial + ((size_t)s * M + m) * N + n;
    float a[8], b[8];
    load8_wide(p, a);
    load8_wide(p + 8, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) { v[i] += a[i]; v[8 + i] += b[i]; }
  }
  const EpiRow row = epi_row_begin<KIND>(ep, m);
  epi_apply16<KIND, TOut>(ep, row, m, n, v);
}

// K-splits for problems with too few output tiles to fill the machine (weight
// gradients: small M x N, K = tokens; decode projections: one row of tiles).
// Needs caller scratch for splits * M * N floats.
int pick_splits(const GemmArgs& g, int tiles) {
  if (!g.splitk_scratch) return 1;
  const int sms = sm_count();
  const int num_kb = cdiv(g.K, TBK);
  if (tiles >= 2 * sms || num_kb < 16) return 1;
  // cost of s splits in units of one full-K tile: rounds of the persistent grid, each 1/s long
  int best = 1;
  double best_cost = (double)cdiv(tiles, sms);
  for (int s = 2; s <= 32 && num_kb / s >= 8; ++s) {
    if ((size_t)s * g.M * g.N * sizeof(float) > g.splitk_bytes) break;
    const double cost = (double)cdiv(tiles * s, sms) / s + 0.02 * s;  // small charge for the extra partial traffic
    if (cost < best_cost * 0.95) { best = s; best_cost = cost; }
  }
  return best;
}

template <int BN, int KIND, typename TOut, bool AMN, bool BMN>
int32_t launch_cfg(const GemmArgs& g, cudaStream_t stream) {
  using Cfg = TcCfg<BN>;
  CUtensorMap tmA, tmB;
  // K-major operand: [rows = M or N, cols = K], box 64 (K) x tile rows.
  // MN-major operand: stored [K, M or N], box 64 (M or N) x TBK rows of K.
  if (AMN) B200_TRY(make_map_2d(&tmA, g.A, g.K, g.M, g.lda, TBK));
  else B200_TRY(make_map_2d(&tmA, g.A, g.M, g.K, g.lda, TBM));
  if (BMN) B200_TRY(make_map_2d(&tmB, g.B, g.K, g.N, g.ldb, TBK));
  else B200_TRY(make_map_2d(&tmB, g.B, g.N, g.K, g.ldb, BN));
  auto kern = gemm_tc_kernel<BN, KIND, TOut, AMN, BMN>;
  static PerDeviceOnce attr_once;  // per instantiation
  B200_TRY(attr_once.run([&](int&) -> int32_t {
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    return B200_OK;
  }));
  const int tiles = cdiv(g.M, TBM) * cdiv(g.N, BN);
  const int splits = pick_splits(g, tiles);
  const int items = tiles * splits;
  int limit = sm_count();
  if (g.max_ctas > 0 && g.max_ctas < limit) limit = g.max_ctas;
  const int grid = items < limit ? items : limit;
  B200_CUDA_OK(launch_pdl(kern, dim3(grid), dim3(TC_THREADS), Cfg::kSmemBytes, stream, tmA, tmB, g.M, g.N, g.K, g.epi,
                          splits, reinterpret_cast<float*>(g.splitk_scratch), device_status_word()));
  B200_LAUNCH_OK("gemm_tc_kernel");
  if (splits > 1) {
    const int chunks = g.M * (g.N / 16);
    B200_CUDA_OK(launch_pdl(splitk_reduce_kernel<KIND, TOut>, dim3(cdiv(chunks, 256)), dim3(256), 0, stream,
                            reinterpret_cast<const float*>(g.splitk_scratch), splits, g.M, g.N, g.epi));
    B200_LAUNCH_OK("splitk_reduce_kernel");
  }
  return B200_OK;
}

template <int KIND, typename TOut, bool AMN, bool BMN>
int32_t launch_bn(const GemmArgs& g, cudaStream_t stream) {
  const int sms = sm_count();
  const long mt = cdiv(g.M, TBM);
  if (g.splitk_scratch && mt * cdiv(g.N, 128) < 2 * sms) {
    // few output tiles and scratch for K-splitting: keep the tile wide (more bytes in flight per CTA) and split K
    if (g.N % 256 == 0 && mt * (g.N / 256) >= sms / 2) return launch_cfg<256, KIND, TOut, AMN, BMN>(g, stream);
    return launch_cfg<128, KIND, TOut, AMN, BMN>(g, stream);
  }
  if (mt == 1) {
    // One row of tiles (decode: the batch is the M dimension).  The kernel then
    // only streams the weights, so what matters is how many SMs pull on HBM:
    // take the widest tile that still gives every SM a tile.
    if (g.N % 256 == 0 && g.N / 256 >= sms) return launch_cfg<256, KIND, TOut, AMN, BMN>(g, stream);
    if (cdiv(g.N, 128) >= sms) return launch_cfg<128, KIND, TOut, AMN, BMN>(g, stream);
    if (BMN || cdiv(g.N, 64) >= sms) return launch_cfg<64, KIND, TOut, AMN, BMN>(g, stream);  // MN-major boxes are 64 wide
    return launch_cfg<32, KIND, TOut, AMN, false>(g, stream);
  }
  // Wide tiles when they still fill the machine, narrower ones otherwise.
  const long t256 = mt * cdiv(g.N, 256);
  if (g.N % 256 == 0 && t256 >= 2L * sms) return launch_cfg<256, KIND, TOut, AMN, BMN>(g, stream);
  const long t128 = mt * cdiv(g.N, 128);
  if (t128 >= sms || g.N >= 128) return launch_cfg<128, KIND, TOut, AMN, BMN>(g, stream);
  return launch_cfg<64, KIND, TOut, AMN, BMN>(g, stream);
}

template <typename TOut>
int32_t launch_kind(const GemmArgs& g, cudaStream_t stream) {
  if (g.ta || g.tb) {
    if (g.kind != EPI_STORE) return fail(B200_ERR_UNSUPPORTED, "fused epilogues need both operands K-major");
    if (g.ta && g.tb) return launch_bn<EPI_STORE, TOut, true, true>(g, stream);
    if (g.ta) return launch_bn<EPI_STORE, TOut, true, false>(g, stream);
    return launch_bn<EPI_STORE, TOut, false, true>(g, stream);
  }
  switch (g.kind) {
    case EPI_STORE: return launch_bn<EPI_STORE, TOut, false, false>(g, stream);
    case EPI_ROPE: return launch_bn<EPI_ROPE, TOut, false, false>(g, stream);
    case EPI_RESID: return launch_bn<EPI_RESID, TOut, false, false>(g, stream);
    case EPI_SWIGLU: return launch_bn<EPI_SWIGLU, TOut, false, false>(g, stream);
  }
  return fail(B200_ERR_INVALID_ARG, "unknown epilogue kind %d", g.kind);
}

}  // namespace

// Self-test of the bounded-wait path: one CTA waits on an mbarrier that nothing
// ever arrives on, with a budget of `budget_cycles`; the wait must give up,
// record ST_SELFTEST_TIMEOUT in the status word and let the kernel return.
namespace {
enum : uint32_t { ST_SELFTEST_TIMEOUT = 1u << 15 };
__global__ void bounded_wait_selftest_kernel(long long budget_cycles, uint32_t* status, uint32_t* reached_end) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    abort_flag = 0u;
    ptx::fence_barrier_init();
  }
  __syncthreads();
  // every thread waits; the first to run out raises the CTA-wide abort flag, which releases the others
  const bool ok = ptx::mbar_wait(&bar, 0, &abort_flag, status, ST_SELFTEST_TIMEOUT, budget_cycles);
  __syncthreads();
  if (threadIdx.x == 0) *reached_end = ok ? 2u : 1u;
}
}  // namespace

int32_t launch_bounded_wait_selftest(long long budget_cycles, uint32_t* reached_end, cudaStream_t stream) {
  bounded_wait_selftest_kernel<<<1, 64, 0, stream>>>(budget_cycles, device_status_word(), reached_end);
  B200_LAUNCH_OK("bounded_wait_selftest_kernel");
  return B200_OK;
}

bool gemm_tc_supports(const GemmArgs& g) {
  if ((g.ta || g.tb) && g.kind != EPI_STORE) return false;
  // TMA needs 16-byte aligned bases and row pitches; the extent of the
  // contiguous dimension needs no alignment (out-of-range elements read zero).
  return g.in_dtype == B200_BF16 && g.M > 0 && g.N > 0 && g.K > 0 && g.N % 16 == 0 && g.lda % 8 == 0 &&
         g.ldb % 8 == 0 && aligned16(g.A) && aligned16(g.B) && aligned16(g.epi.out) && g.epi.ldo % 8 == 0;
}

int32_t launch_gemm_tc(const GemmArgs& g, cudaStream_t stream) {
  if (!gemm_tc_supports(g))
    return fail(B200_ERR_UNSUPPORTED,
                "tcgen05 gemm needs bf16 operands, 16-byte aligned rows and N %% 16 == 0 (M=%d N=%d K=%d)",
                g.M, g.N, g.K);
  if (g.out_dtype == B200_BF16) return launch_kind<bf16>(g, stream);
  if (g.out_dtype == B200_F32) return launch_kind<float>(g, stream);
  return fail(B200_ERR_BAD_DTYPE, "gemm: unsupported output dtype %d", g.out_dtype);
}

int32_t launch_splitk_reduce(const GemmArgs& g, int splits, cudaStream_t stream) {
  if (g.kind != EPI_STORE) return fail(B200_ERR_UNSUPPORTED, "split-K reduction outside a GEMM launch covers the plain store only");
  const int chunks = g.M * (g.N / 16);
  if (g.out_dtype == B200_F32)
    B200_CUDA_OK(launch_pdl(splitk_reduce_kernel<EPI_STORE, float>, dim3(cdiv(chunks, 256)), dim3(256), 0, stream,
                            reinterpret_cast<const float*>(g.splitk_scratch), splits, g.M, g.N, g.epi));
  else
    B200_CUDA_OK(launch_pdl(splitk_reduce_kernel<EPI_STORE, bf16>, dim3(cdiv(chunks, 256)), dim3(256), 0, stream,
                            reinterpret_cast<const float*>(g.splitk_scratch), splits, g.M, g.N, g.epi));
  B200_LAUNCH_OK("splitk_reduce_kernel");
  return B200_OK;
}

bool gemm_bands_supported(const GemmArgs& g, int impl) {
  static const int use_pair = env_int("B200_GEMM_PAIR", 1);
  const bool tc = impl == 1 || (impl != 2 && gemm_tc_supports(g));
  return tc && use_pair && gemm_tc2_supports(g) && !g.ta && !g.tb && g.band_rows > 0 && g.band_rows % 256 == 0 &&
         g.M % g.band_rows == 0 && g.M / g.band_rows <= 8;
}

bool gemm_push_supported(const GemmArgs& g, int impl) {
  static const int use_pair = env_int("B200_GEMM_PAIR", 1);
  const bool tc = impl == 1 || (impl != 2 && gemm_tc_supports(g));
  return tc && use_pair && gemm_tc2_supports(g) && g.kind == EPI_STORE && !g.ta && !g.tb && g.push_rows > 0 &&
         g.push_rows % 32 == 0 && g.M % g.push_rows == 0 && g.M / g.push_rows <= 8;
}

int32_t launch_gemm(const GemmArgs& g, int impl, cudaStream_t stream) {
  const bool tc = impl == 1 || (impl != 2 && gemm_tc_supports(g));
  // B200_GEMM_PAIR=0 keeps every problem on the single-CTA kernel
  static const int use_pair = env_int("B200_GEMM_PAIR", 1);
  static const int pair_mn = env_int("B200_GEMM_PAIR_MN", 1);  // 0 keeps weight gradients on the single-CTA kernel
  const bool pair = tc && use_pair && gemm_tc2_supports(g);
  const bool pair_t = tc && !pair && use_pair && pair_mn && gemm_tc2_mn_supports(g);
  ProfScope prof(!tc ? PROF_GEMM_SIMT : (pair || pair_t) ? PROF_GEMM_PAIR : PROF_GEMM_TC,
                 2.0 * g.M * (double)g.N * g.K, stream);
  if (g.band_flags && !pair)
    return fail(B200_ERR_UNSUPPORTED, "banded A operand needs the CTA-pair tensor kernel (M=%d N=%d K=%d)", g.M, g.N, g.K);
  if (g.push_rows > 0 && !pair)
    return fail(B200_ERR_UNSUPPORTED, "pushed store needs the CTA-pair tensor kernel (M=%d N=%d K=%d)", g.M, g.N, g.K);
  if (!tc) return launch_gemm_simt(g, stream);
  if (pair) return launch_gemm_tc2(g, stream);
  if (pair_t) return launch_gemm_tc2_mn(g, stream);
  return launch_gemm_tc(g, stream);
}

}  // namespace b200
