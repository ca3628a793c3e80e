// tcgen05 GEMM with CTA pairs (cta_group::2):  Y[M,N] = A[M,K] * B[N,K]^T, bf16,
// both operands K-major, fused epilogues.
//
// Two CTAs of a cluster (two neighbouring SMs) share one 256 x BN output tile.
// Each CTA stages its own 128 rows of A and HALF of the B tile (BN/2 rows); one
// thread of the leader CTA issues tcgen05.mma.cta_group::2, which reads A and B
// from both CTAs' shared memory and writes each CTA's 128 x BN accumulator into
// that CTA's TMEM.  Per CTA and k-block this stages 16 KB + BN/2 * 128 B for
// 128 x BN x 64 MACs: twice the arithmetic intensity of the single-CTA kernel
// on the B side, which is what its shared-memory fill rate was short of.
//
// Plain per-CTA TMA loads only (each CTA loads what it alone needs); the loads
// of the second CTA complete their bytes on the leader's mbarrier.  tcgen05.commit
// reaches both CTAs' barriers.  All waits are bounded; the CTAs of a pair meet at
// a cluster barrier before the first remote signal and before exit.
#include <cuda.h>

#include "gemm_epilogue.cuh"
#include "ptx_sm100.cuh"
#include "tensor_map.cuh"

namespace b200 {

namespace {

constexpr int PM = 128;   // rows per CTA (256 per pair)
constexpr int PK = 64;    // K elements per stage
constexpr int P_THREADS = 192;

template <int BN> struct PairCfg {
  static constexpr int kABytes = PM * PK * 2;
  static constexpr int kBBytes = (BN / 2) * PK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (200 * 1024) / kStageBytes > 8 ? 8 : (200 * 1024) / kStageBytes;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
};

enum : uint32_t { ST_PAIR_PRODUCER = 1u << 8, ST_PAIR_MMA = 1u << 9, ST_PAIR_EPILOGUE = 1u << 10 };

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], "
      "[%4];" ::"r"(ptx::smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(leader_bar)
      : "memory");
}
__device__ __forceinline__ void mma_pair_bf16_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the barrier at this offset in both CTAs once the MMAs issued so far are done
__device__ __forceinline__ void mma_pair_commit(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::
                   "r"(ptx::smem_u32(bar)),
               "h"(mask)
               : "memory");
}

template <int BN, int KIND, typename TOut>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
    gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int M, int N,
                    int K, EpiParams ep, uint32_t* status) {
  using Cfg = PairCfg<BN>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * Cfg::kStageBytes);
  uint64_t* full_bar = bars;               // [S]  leader's: bytes of both CTAs landed
  uint64_t* empty_bar = bars + S;          // [S]  own: the pair's MMAs are done with the stage
  uint64_t* acc_full = bars + 2 * S;       // [2]  own: accumulator complete
  uint64_t* acc_empty = bars + 2 * S + 2;  // [2]  leader's: both CTAs' epilogues drained the accumulator
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int m_tiles = (M + 2 * PM - 1) / (2 * PM);
  const int n_tiles = (N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (K + PK - 1) / PK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      ptx::mbar_init(&full_bar[i], 1);
      ptx::mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&acc_full[i], 1);
      ptx::mbar_init(&acc_empty[i], 8);  // 4 epilogue warps of each CTA
    }
    *abort_flag = 0u;
    ptx::fence_barrier_init();
    ptx::tma_prefetch_desc(&tmA);
    ptx::tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_u32(tmem_slot)),
                 "r"((uint32_t)Cfg::kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything is signalled across the pair
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        int mt, nt;
        tile_coords(tile, m_tiles, n_tiles, 8, mt, nt);
        const int m0 = mt * (2 * PM) + (int)rank * PM;
        const int n0 = nt * BN + (int)rank * (BN / 2);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = ptx::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, status, ST_PAIR_PRODUCER);
          if (!ok) break;
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          const uint32_t leader_full = map_to_cta(ptx::smem_u32(&full_bar[stage]), 0);
          if (rank == 0) ptx::mbar_arrive_expect_tx(&full_bar[stage], 2 * Cfg::kStageBytes);
          tma_load_2d_pair(sa, &tmA, kb * PK, m0, leader_full);
          tma_load_2d_pair(sa + Cfg::kABytes, &tmB, kb * PK, n0, leader_full);
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = ptx::idesc_bf16_f32(2 * PM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        ok = ptx::mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_flag, status, ST_PAIR_MMA);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = ptx::mbar_wait(&full_bar[stage], phase, abort_flag, status, ST_PAIR_MMA);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          const uint32_t sa = ptx::smem_u32(smem + stage * Cfg::kStageBytes);
          const uint64_t adesc = ptx::smem_desc_sw128(sa);
          const uint64_t bdesc = ptx::smem_desc_sw128(sa + Cfg::kABytes);
#pragma unroll
          for (int k = 0; k < PK / 16; ++k)
            mma_pair_bf16_ss(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                             (kb > 0 || k > 0) ? 1u : 0u);
          mma_pair_commit(&empty_bar[stage]);
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        mma_pair_commit(&acc_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else {
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
      int mt, nt;
      tile_coords(tile, m_tiles, n_tiles, 8, mt, nt);
      const int m0 = mt * (2 * PM) + (int)rank * PM;
      const int n0 = nt * BN;
      const int m = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
      const bool row_ok = m < M;
      const EpiRow erow = epi_row_begin<KIND>(ep, row_ok ? m : 0);
      // operands of the epilogue are fetched before the accumulator wait (see the single-CTA kernel)
      constexpr int PRE = (KIND == EPI_RESID) ? (BN < 128 ? BN : 128) : 8;
      float rpre[PRE];
      float rc[32], rs[32];
      const bool rope64 = KIND == EPI_ROPE && ep.head_size == 64 && (BN % 64 == 0);
      if (KIND == EPI_RESID) {
        const float* xi = ep.resid_in + (size_t)(row_ok ? m : 0) * ep.ldo + n0;
#pragma unroll
        for (int c = 0; c < PRE; c += 8) {
          float t8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          if (row_ok && n0 + c < N) load8_wide(xi + c, t8);
#pragma unroll
          for (int i = 0; i < 8; ++i) rpre[c + i] = t8[i];
        }
      }
      if (KIND == EPI_ROPE && rope64) {
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
          float t8[8], u8[8];
          load8_wide(erow.rope_c + c, t8);
          load8_wide(erow.rope_s + c, u8);
#pragma unroll
          for (int i = 0; i < 8; ++i) { rc[c + i] = t8[i]; rs[c + i] = u8[i]; }
        }
      }
      ok = ptx::mbar_wait_warp(&acc_full[acc], acc_phase, abort_flag, status, ST_PAIR_EPILOGUE);
      if (!ok) break;
      ptx::tc_fence_after_sync();
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
              if (KIND == EPI_RESID && cc < PRE) {
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
                  const int j0 = (cc % 64) >> 1;
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
      if (lane == 0) mbar_arrive_remote(map_to_cta(ptx::smem_u32(&acc_empty[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  cluster_sync_all();  // neither CTA leaves while the other may still read its shared memory or signal its barriers
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::kTmemCols)
                 : "memory");
  }
}

template <int BN, int KIND, typename TOut>
int32_t launch_pair_cfg(const GemmArgs& g, cudaStream_t stream) {
  using Cfg = PairCfg<BN>;
  CUtensorMap tmA, tmB;
  B200_TRY(make_map_2d(&tmA, g.A, g.M, g.K, g.lda, PM));
  B200_TRY(make_map_2d(&tmB, g.B, g.N, g.K, g.ldb, BN / 2));
  auto kern = gemm_tc2_kernel<BN, KIND, TOut>;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set = true;
  }
  // Clusters are placed inside one GPC, so fewer than sm_count()/2 pairs may be resident at once; the
  // grid is persistent with a static tile assignment, so launch exactly the resident number.
  static int max_pairs = 0;
  if (max_pairs == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count() & ~1, 1, 1);
    cfg.blockDim = dim3(P_THREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / 2;
    }
    max_pairs = n < sm_count() / 2 ? n : sm_count() / 2;
  }
  const int tiles = cdiv(g.M, 2 * PM) * cdiv(g.N, BN);
  int pairs = max_pairs;
  if (g.max_ctas > 0 && g.max_ctas / 2 < pairs) pairs = g.max_ctas / 2;
  if (pairs > tiles) pairs = tiles;
  kern<<<2 * pairs, P_THREADS, Cfg::kSmemBytes, stream>>>(tmA, tmB, g.M, g.N, g.K, g.epi, device_status_word());
  B200_LAUNCH_OK("gemm_tc2_kernel");
  return B200_OK;
}

template <int KIND, typename TOut>
int32_t launch_pair_bn(const GemmArgs& g, cudaStream_t stream) {
  // rounds of the persistent grid times the tile width: prefer the wide tile unless it wastes a round
  const int pairs = sm_count() / 2;
  const long mt = cdiv(g.M, 2 * PM);
  const long cost256 = g.N % 256 == 0 ? (long)cdiv((int)(mt * (g.N / 256)), pairs) * 256 : -1;
  const long cost128 = (long)cdiv((int)(mt * cdiv(g.N, 128)), pairs) * 128;
  if (cost256 >= 0 && cost256 * 10 <= cost128 * 12) return  // the wide tile moves fewer bytes per flop: keep it unless it wastes > 20 % (a 40 % margin measured slower in the 110M step)
    launch_pair_cfg<256, KIND, TOut>(g, stream);
  return launch_pair_cfg<128, KIND, TOut>(g, stream);
}

template <typename TOut>
int32_t launch_pair_kind(const GemmArgs& g, cudaStream_t stream) {
  switch (g.kind) {
    case EPI_STORE: return launch_pair_bn<EPI_STORE, TOut>(g, stream);
    case EPI_ROPE: return launch_pair_bn<EPI_ROPE, TOut>(g, stream);
    case EPI_RESID: return launch_pair_bn<EPI_RESID, TOut>(g, stream);
    case EPI_SWIGLU: return launch_pair_bn<EPI_SWIGLU, TOut>(g, stream);
  }
  return fail(B200_ERR_INVALID_ARG, "unknown epilogue kind %d", g.kind);
}

}  // namespace

// The pair kernel takes K-major operands and problems with enough 256-row tiles to occupy every SM pair.
bool gemm_tc2_supports(const GemmArgs& g) {
  if (!gemm_tc_supports(g) || g.ta || g.tb) return false;
  if (g.N % 128) return false;
  const long tiles = (long)cdiv(g.M, 2 * PM) * cdiv(g.N, g.N % 256 == 0 ? 256 : 128);
  return g.M >= 2 * PM && tiles >= sm_count() / 2;
}

int32_t launch_gemm_tc2(const GemmArgs& g, cudaStream_t stream) {
  if (!gemm_tc2_supports(g)) return fail(B200_ERR_UNSUPPORTED, "the CTA-pair gemm does not cover this problem");
  if (g.out_dtype == B200_BF16) return launch_pair_kind<bf16>(g, stream);
  if (g.out_dtype == B200_F32) return launch_pair_kind<float>(g, stream);
  return fail(B200_ERR_BAD_DTYPE, "gemm: unsupported output dtype %d", g.out_dtype);
}

}  // namespace b200
