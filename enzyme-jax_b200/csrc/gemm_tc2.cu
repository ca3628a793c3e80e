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
//
// Epilogue: four warps per CTA take the accumulator TMEM -> registers -> 32-row
// boxes in shared memory (swizzled as the output tensor map expects) -> bulk
// tensor stores, a few boxes in flight per warp; the residual add receives its
// fp32 residual tile through TMA loads into the same boxes.
#include <cuda.h>

#include "gemm_epilogue.cuh"
#include "ptx_sm100.cuh"
#include "plan.cuh"
#include "tensor_map.cuh"

namespace b200 {

namespace {

constexpr int PM = 128;   // rows per CTA (256 per pair)
constexpr int PK = 64;    // K elements per stage
constexpr int P_THREADS = 192;

template <int BN, int KIND> struct PairCfg {
  static constexpr int kABytes = PM * PK * 2;
  static constexpr int kBBytes = (BN / 2) * PK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // staging buffers of the four epilogue warps: 32 rows x 128 bytes (x 64 bytes for SwiGLU, which has up to
  // three output matrices); two in flight per output, four for the residual add (they also receive its read side)
  static constexpr int kBufBytes = KIND == EPI_SWIGLU ? 2048 : 4096;
  // The residual add keeps as many residual chunks in flight as it has boxes; fewer boxes leave room for one more
  // pipeline stage, which the short mainloops (K = 768, 192-column tiles) need more than a deep epilogue.
  static constexpr int kBufs = KIND == EPI_SWIGLU ? 6 : (KIND == EPI_RESID ? (BN == 192 ? 3 : 2) : 2);
  static constexpr int kStagingBytes = 4 * kBufs * kBufBytes;
  // 1 KB alignment slack + 512 B of barriers; what is left of the SM's 228 KB (1.5 KB beside this CTA's own reserved
  // kilobyte) lets a small CTA of another kernel - the exchange of the other half of a tensor-parallel batch - run
  // on the same SM
  static constexpr int kBudget = 227 * 1024 - 1536 - kStagingBytes;
  static constexpr int kStages = kBudget / kStageBytes > 8 ? 8 : kBudget / kStageBytes;
  static constexpr int kAccStride = BN == 192 ? 256 : BN;  // TMEM columns between the two accumulators
  static constexpr int kTmemCols = 2 * kAccStride;         // a power of two, as the allocator wants
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1536;
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

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Output maps of a pushed store (GemmArgs::push_rows): one [push_rows, N] matrix per destination rank.
struct alignas(64) PushMaps {
  CUtensorMap m[8];
};

// Bands of A rows that other ranks deliver (GemmArgs::band_flags).
struct BandWait {
  const uint32_t* flags = nullptr;  // [bands]: band o is whole once flags[o] has reached `epoch`
  uint32_t epoch = 0;
  int rows = 0;     // rows per band, a multiple of the 256-row tile
  int mt_rot = 0;   // row tiles are visited starting at this one (the first tile of the band that is already there)
  long long budget = 0;
};

// MN: both operands are MN-major (A stored [K, M], B stored [K, N]: the weight-gradient products dY^T X).  Their
// tiles arrive as boxes of 64 columns x 64 k-rows and are described to the MMA as MN-major.  `splits` > 1 cuts K
// into that many ranges handled as separate work items whose fp32 partial tiles go to rows split * split_rows + m
// of the output map (a scratch of [splits * M, N]); a reduction kernel sums them in split order.
template <int BN, int KIND, typename TOut, bool MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
    gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmO, const __grid_constant__ CUtensorMap tmR,
                    const __grid_constant__ CUtensorMap tmG, const __grid_constant__ CUtensorMap tmU, int M, int N,
                    int K, EpiParams ep, int splits, int split_rows, uint32_t* status,
                    const __grid_constant__ PushMaps pm, int push_rows, BandWait bw) {
  using Cfg = PairCfg<BN, KIND>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * Cfg::kStageBytes + Cfg::kStagingBytes);
  uint64_t* full_bar = bars;               // [S]  leader's: bytes of both CTAs landed
  uint64_t* empty_bar = bars + S;          // [S]  own: the pair's MMAs are done with the stage
  uint64_t* acc_full = bars + 2 * S;       // [2]  own: accumulator complete
  uint64_t* acc_empty = bars + 2 * S + 2;  // [2]  leader's: both CTAs' epilogues drained the accumulator
  uint64_t* resid_bar = bars + 2 * S + 4;  // [4 warps][4]  own: a residual chunk has landed in its staging buffer
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4 + 16);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int m_tiles = (M + 2 * PM - 1) / (2 * PM);
  const int n_tiles = (N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (K + PK - 1) / PK;
  const int num_items = num_tiles * splits;  // item = (tile, K range): tile = item % num_tiles, split = item / num_tiles
  // row tiles per raster group (tiles of a group are visited before the next group: the A panel of the group stays
  // in L2); with a banded A operand a group does not reach into the next band, which arrives later
  const int raster_rows = bw.flags && bw.rows / (2 * PM) < 8 ? bw.rows / (2 * PM) : 8;
  constexpr int kMnBox = 64 * PK * 2;        // bytes of one MN-major box: 64 columns x 64 k-rows

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      ptx::mbar_init(&full_bar[i], 1);
      ptx::mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&acc_full[i], 1);
      ptx::mbar_init(&acc_empty[i], 8);  // 4 epilogue warps of each CTA
    }
    for (int i = 0; i < 16; ++i) ptx::mbar_init(&resid_bar[i], 1);
    *abort_flag = 0u;
    ptx::fence_barrier_init();
    ptx::tma_prefetch_desc(&tmA);
    ptx::tma_prefetch_desc(&tmB);
    ptx::tma_prefetch_desc(&tmO);
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
  pdl_wait();  // everything above overlapped the previous kernel's tail; operands are touched from here on

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t bands_seen = 0;  // bit o: band o of the A operand is known to be whole
      for (int item = pair; item < num_items && ok; item += n_pairs) {
        const int tile = item % num_tiles, split = item / num_tiles;
        const int kb0 = (int)((long)split * num_kb / splits), kb1 = (int)((long)(split + 1) * num_kb / splits);
        int mt, nt;
        tile_coords(tile, m_tiles, n_tiles, raster_rows, mt, nt);
        if (bw.flags) mt = (mt + bw.mt_rot) % m_tiles;
        const int m0 = mt * (2 * PM) + (int)rank * PM;
        const int n0 = nt * BN + (int)rank * (BN / 2);
        if (bw.flags) {
          // rows of a band another rank writes: wait for that rank's word, once per band (bounded; acquire at
          // system scope, then order the bulk loads of this thread behind it)
          const int band = m0 / bw.rows;
          if (!((bands_seen >> band) & 1u)) {
            const long long t0 = clock64();
            while ((int32_t)(ld_acquire_sys_u32(bw.flags + band) - bw.epoch) < 0) {
              __nanosleep(64);
              if (*abort_flag || clock64() - t0 > bw.budget) {
                atomicOr(status, (uint32_t)ST_PAIR_PRODUCER);
                *abort_flag = 1u;
                ok = false;
                break;
              }
            }
            if (!ok) break;
            asm volatile("fence.proxy.async;" ::: "memory");
            bands_seen |= 1u << band;
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = ptx::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, status, ST_PAIR_PRODUCER);
          if (!ok) break;
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          const uint32_t leader_full = map_to_cta(ptx::smem_u32(&full_bar[stage]), 0);
          if (rank == 0) ptx::mbar_arrive_expect_tx(&full_bar[stage], 2 * Cfg::kStageBytes);
          if constexpr (MN) {
#pragma unroll
            for (int i = 0; i < PM / 64; ++i) tma_load_2d_pair(sa + i * kMnBox, &tmA, m0 + 64 * i, kb * PK, leader_full);
#pragma unroll
            for (int i = 0; i < BN / 128; ++i)
              tma_load_2d_pair(sa + Cfg::kABytes + i * kMnBox, &tmB, n0 + 64 * i, kb * PK, leader_full);
          } else {
            tma_load_2d_pair(sa, &tmA, kb * PK, m0, leader_full);
            tma_load_2d_pair(sa + Cfg::kABytes, &tmB, kb * PK, n0, leader_full);
          }
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = ptx::idesc_bf16_f32(2 * PM, BN) | (MN ? ((1u << 15) | (1u << 16)) : 0u);
      constexpr uint64_t k_step = MN ? (16 * 128) / 16 : 2;  // start-address step per 16 K-elements, in 16-byte units
      // descriptors of stage 0, built once: a stage adds its byte offset >> 4 to the 14-bit address field (shared-memory
      // addresses stay below 2^18, so it never carries); this thread's instruction stream is what bounds narrow tiles
      const uint32_t s0 = ptx::smem_u32(smem);
      const uint64_t a_base = MN ? ptx::smem_desc_sw128_mn(s0, kMnBox) : ptx::smem_desc_sw128(s0);
      const uint64_t b_base = MN ? ptx::smem_desc_sw128_mn(s0 + Cfg::kABytes, kMnBox)
                                 : ptx::smem_desc_sw128(s0 + Cfg::kABytes);
      constexpr uint64_t stage_step = Cfg::kStageBytes >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int item = pair; item < num_items && ok; item += n_pairs) {
        const int split = item / num_tiles;
        const int kb0 = (int)((long)split * num_kb / splits), kb1 = (int)((long)(split + 1) * num_kb / splits);
        ok = ptx::mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_flag, status, ST_PAIR_MMA);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * Cfg::kAccStride);
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = ptx::mbar_wait(&full_bar[stage], phase, abort_flag, status, ST_PAIR_MMA);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          const uint64_t adesc = a_base + (uint64_t)stage * stage_step;
          const uint64_t bdesc = b_base + (uint64_t)stage * stage_step;
#pragma unroll
          for (int k = 0; k < PK / 16; ++k)
            mma_pair_bf16_ss(d_tmem, adesc + k_step * k, bdesc + k_step * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
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
    // ---- epilogue warps: TMEM -> registers -> swizzled shared-memory tile -> TMA store ----
    // A warp owns 32 rows (its TMEM lane quarter) of the CTA's accumulator; lane = row.  Writing whole
    // rows from registers would put every lane of a store on a different cache line, which the
    // load/store unit serialises; the bulk store writes full lines and runs beside the next chunk.
    const int q = warp & 3;
    constexpr int NBUF = Cfg::kBufs, BUFB = Cfg::kBufBytes;
    uint8_t* stg_ptr = smem + S * Cfg::kStageBytes + (warp - 2) * NBUF * BUFB;  // this warp's staging buffers
    const uint32_t stg = ptx::smem_u32(stg_ptr);
    uint64_t* rbar = resid_bar + (warp - 2) * 4;  // EPI_RESID: one barrier per staging buffer
    uint32_t rphase = 0;                          // bit b: parity the next wait on rbar[b] uses
    int ring = 0;                                 // staging buffers are used round-robin
    const uint32_t sw128 = (uint32_t)(lane & 7) << 4;
    const uint32_t row128 = stg + (uint32_t)lane * 128u;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int item = pair; item < num_items && ok; item += n_pairs) {
      const int tile = item % num_tiles, split = item / num_tiles;
      int mt, nt;
      tile_coords(tile, m_tiles, n_tiles, raster_rows, mt, nt);
      if (bw.flags) mt = (mt + bw.mt_rot) % m_tiles;
      const int m0 = mt * (2 * PM) + (int)rank * PM;
      const int n0 = nt * BN;
      const int mrow0 = m0 + q * 32;  // first row of this warp's boxes; rows past M are clipped by the store
      const int yrow0 = mrow0 + split * split_rows;  // row of the output map (partial sums: one M-row band per split)
      // where this warp's boxes go: the output map, or - pushed store - the map of the rank that owns these rows
      const CUtensorMap* out_map = &tmO;
      int out_y = yrow0, out_rows = 0x7fffffff;
      if constexpr (KIND == EPI_STORE && !MN) {
        if (push_rows > 0) {
          const int dst = yrow0 / push_rows;  // push_rows is a multiple of 32: a box never straddles two destinations
          out_rows = M;                       // no destination owns rows past M: such a box is not stored at all
          out_map = &pm.m[dst < 8 ? dst : 7];
          out_y = yrow0 - dst * push_rows;
        }
      }
      const int m = mrow0 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * Cfg::kAccStride);
      const EpiRow erow = epi_row_begin<KIND>(ep, m < M ? m : 0);
      float rc[32], rs[32];
      const bool rope64 = KIND == EPI_ROPE && ep.head_size == 64;
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
      if (KIND == EPI_RESID) {
        // the residual tile comes in by TMA too, into the buffers its sum leaves from; the first
        // 32-column chunks are requested before the accumulator is waited for
        if (lane == 0) {
          ptx::tma_store_wait_read<0>();
#pragma unroll
          for (int i = 0; i < (BN / 32 < NBUF ? BN / 32 : NBUF); ++i)
            if (n0 + 32 * i < N) {
              ptx::mbar_arrive_expect_tx(&rbar[i], 4096u);
              ptx::tma_load_2d(stg_ptr + i * BUFB, &tmR, n0 + 32 * i, mrow0, &rbar[i]);
            }
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
        } else {
          // the accumulator is in registers: hand it back to the MMA warp before the last chunk is stored
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_remote(map_to_cta(ptx::smem_u32(&acc_empty[acc]), 0));
        }
        if (n0 + c < N) {
          if constexpr (KIND == EPI_STORE || KIND == EPI_ROPE) {
            if constexpr (KIND == EPI_ROPE) {
#pragma unroll
              for (int hlf = 0; hlf < 2; ++hlf) {
                const int cc = c + 16 * hlf;
                if (n0 + cc < ep.rope_cols) {
                  const int j0 = ((n0 + cc) % ep.head_size) >> 1;
                  if (rope64) {
                    const int jj = (cc % 64) >> 1;  // n0 is a multiple of 64
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                      const float e = cur[hlf][2 * i], o = cur[hlf][2 * i + 1];
                      cur[hlf][2 * i] = rc[jj + i] * e - rs[jj + i] * o;
                      cur[hlf][2 * i + 1] = rs[jj + i] * e + rc[jj + i] * o;
                    }
                  } else {
                    float cs[8], sn[8];
                    load8(erow.rope_c + j0, cs);
                    load8(erow.rope_s + j0, sn);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                      const float e = cur[hlf][2 * i], o = cur[hlf][2 * i + 1];
                      cur[hlf][2 * i] = cs[i] * e - sn[i] * o;
                      cur[hlf][2 * i + 1] = sn[i] * e + cs[i] * o;
                    }
                  }
                }
              }
            }
            if constexpr (sizeof(TOut) == 4) {
              // one 32-column fp32 box per chunk
              const uint32_t buf = row128 + (uint32_t)((ring % NBUF) * BUFB);
              if (lane == 0) ptx::tma_store_wait_read<NBUF - 1>();
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 8; ++j)
                ptx::st_shared_v4(buf + (((uint32_t)j << 4) ^ sw128), __float_as_uint(cur[j >> 2][(j & 3) * 4 + 0]),
                                  __float_as_uint(cur[j >> 2][(j & 3) * 4 + 1]),
                                  __float_as_uint(cur[j >> 2][(j & 3) * 4 + 2]),
                                  __float_as_uint(cur[j >> 2][(j & 3) * 4 + 3]));
              ptx::fence_proxy_async();
              __syncwarp();
              if (lane == 0) {
                if (yrow0 < out_rows) ptx::tma_store_2d(out_map, stg + (uint32_t)((ring % NBUF) * BUFB), n0 + c, out_y);
                ptx::tma_store_commit();
              }
              ++ring;
            } else {
              // one 64-column bf16 box per two chunks
              const int half = (c >> 5) & 1;
              const uint32_t buf = row128 + (uint32_t)((ring % NBUF) * BUFB);
              if (half == 0) {
                if (lane == 0) ptx::tma_store_wait_read<NBUF - 1>();
                __syncwarp();
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t r[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  __nv_bfloat162 h2 = __floats2bfloat162_rn(cur[j >> 1][(j & 1) * 8 + 2 * i], cur[j >> 1][(j & 1) * 8 + 2 * i + 1]);
                  r[i] = *reinterpret_cast<uint32_t*>(&h2);
                }
                ptx::st_shared_v4(buf + (((uint32_t)(half * 4 + j) << 4) ^ sw128), r[0], r[1], r[2], r[3]);
              }
              if (half == 1) {
                ptx::fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                  if (yrow0 < out_rows)
                    ptx::tma_store_2d(out_map, stg + (uint32_t)((ring % NBUF) * BUFB), n0 + c - 32, out_y);
                  ptx::tma_store_commit();
                }
                ++ring;
              }
            }
          } else if constexpr (KIND == EPI_RESID) {
            const int i = c >> 5, b = i % NBUF;
            ok = ptx::mbar_wait_warp(&rbar[b], (rphase >> b) & 1u, abort_flag, status, ST_PAIR_EPILOGUE);
            if (!ok) break;
            rphase ^= 1u << b;
            const uint32_t buf = row128 + (uint32_t)(b * BUFB);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t a = buf + (((uint32_t)j << 4) ^ sw128);
              uint32_t x0, x1, x2, x3;
              ptx::ld_shared_v4(a, x0, x1, x2, x3);
              ptx::st_shared_v4(a, __float_as_uint(__uint_as_float(x0) + cur[j >> 2][(j & 3) * 4 + 0]),
                                __float_as_uint(__uint_as_float(x1) + cur[j >> 2][(j & 3) * 4 + 1]),
                                __float_as_uint(__uint_as_float(x2) + cur[j >> 2][(j & 3) * 4 + 2]),
                                __float_as_uint(__uint_as_float(x3) + cur[j >> 2][(j & 3) * 4 + 3]));
            }
            ptx::fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              ptx::tma_store_2d(&tmO, stg + (uint32_t)(b * BUFB), n0 + c, mrow0);
              ptx::tma_store_commit();
              // the next chunk without a box goes where chunk i-1 left from, once that store has read its tile
              if (i >= 1 && i - 1 + NBUF < BN / 32 && n0 + 32 * (i - 1 + NBUF) < N) {
                ptx::tma_store_wait_read<1>();
                const int nb = (i - 1) % NBUF;
                ptx::mbar_arrive_expect_tx(&rbar[nb], 4096u);
                ptx::tma_load_2d(stg_ptr + nb * BUFB, &tmR, n0 + 32 * (i - 1 + NBUF), mrow0, &rbar[nb]);
              }
            }
          } else {  // EPI_SWIGLU: 64 accumulator columns = 32 outputs = one 64-byte-wide box per output matrix
            const int half = (c >> 5) & 1;
            const bool has_gu = ep.out_gate != nullptr;
            const int set = ring & 1;
            const uint32_t base = stg + (uint32_t)(set * 3 * BUFB);
            const uint32_t row64 = base + (uint32_t)lane * 64u;
            const uint32_t sw64 = (uint32_t)((lane >> 1) & 3) << 4;
            if (half == 0) {
              if (lane == 0) ptx::tma_store_wait_read<1>();
              __syncwarp();
            }
#pragma unroll
            for (int grp = 0; grp < 2; ++grp) {
              uint32_t hr[4], gr[4], ur[4];
#pragma unroll
              for (int i2 = 0; i2 < 4; ++i2) {
                const float g0 = cur[grp][2 * i2], g1 = cur[grp][2 * i2 + 1];
                const float u0 = cur[grp][8 + 2 * i2], u1 = cur[grp][8 + 2 * i2 + 1];
                __nv_bfloat162 hh = __floats2bfloat162_rn(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
                __nv_bfloat162 gg = __floats2bfloat162_rn(g0, g1);
                __nv_bfloat162 uu = __floats2bfloat162_rn(u0, u1);
                hr[i2] = *reinterpret_cast<uint32_t*>(&hh);
                gr[i2] = *reinterpret_cast<uint32_t*>(&gg);
                ur[i2] = *reinterpret_cast<uint32_t*>(&uu);
              }
              const uint32_t off = ((uint32_t)(half * 2 + grp) << 4) ^ sw64;
              ptx::st_shared_v4(row64 + off, hr[0], hr[1], hr[2], hr[3]);
              if (has_gu) {
                ptx::st_shared_v4(row64 + (uint32_t)BUFB + off, gr[0], gr[1], gr[2], gr[3]);
                ptx::st_shared_v4(row64 + (uint32_t)(2 * BUFB) + off, ur[0], ur[1], ur[2], ur[3]);
              }
            }
            if (half == 1) {
              ptx::fence_proxy_async();
              __syncwarp();
              if (lane == 0) {
                const int x = (n0 + c - 32) >> 1;
                ptx::tma_store_2d(&tmO, base, x, mrow0);
                if (has_gu) {
                  ptx::tma_store_2d(&tmG, base + (uint32_t)BUFB, x, mrow0);
                  ptx::tma_store_2d(&tmU, base + (uint32_t)(2 * BUFB), x, mrow0);
                }
                ptx::tma_store_commit();
              }
              ++ring;
            }
          }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) { cur[0][i] = nxt[0][i]; cur[1][i] = nxt[1][i]; }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (lane == 0) ptx::tma_store_wait<0>();
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

// Tile width by modelled time: rounds of the persistent grid x columns per tile.  The 128-wide tile
// reads A and B from shared memory at the full 128 B/clk of an SM and measures about 1.5x slower per
// column than the wider ones, so it is charged that.
int pair_tile_width(int M, int N) {
  const int pairs = sm_count() / 2;
  const long mt = cdiv(M, 2 * PM);
  long best = -1;
  int bn = 128;
  const int widths[3] = {256, 192, 128};
  for (int w : widths) {
    // a width that does not divide N leaves a partly empty last column of tiles; its columns are computed and
    // dropped, which the round count below already charges
    long cost = (long)cdiv((int)(mt * cdiv(N, w)), pairs) * w * 2;
    if (w == 128) cost = cost * 3 / 2;
    if (best < 0 || cost < best) { best = cost; bn = w; }
  }
  return bn;
}

template <int BN, int KIND, typename TOut, bool MN = false>
int32_t launch_pair_cfg(const GemmArgs& g, cudaStream_t stream, int splits = 1) {
  using Cfg = PairCfg<BN, KIND>;
  CUtensorMap tmA, tmB, tmO, tmR, tmG, tmU;
  if (MN) {
    // operands stored [K, M] and [K, N]: boxes of 64 columns x 64 k-rows; fp32 partial tiles of every K range go to
    // the scratch, [splits * M, N]
    B200_TRY(make_map_2d(&tmA, g.A, g.K, g.M, g.lda, PK));
    B200_TRY(make_map_2d(&tmB, g.B, g.K, g.N, g.ldb, PK));
    B200_TRY(make_map_out(&tmO, g.splitk_scratch, splits * g.M, g.N, g.N, 4, 128));
    tmR = tmG = tmU = tmO;
  } else {
    B200_TRY(make_map_2d(&tmA, g.A, g.M, g.K, g.lda, PM));
    B200_TRY(make_map_2d(&tmB, g.B, g.N, g.K, g.ldb, BN / 2));
  }
  if (MN) {
  } else if (KIND == EPI_SWIGLU) {
    B200_TRY(make_map_out(&tmO, g.epi.out, g.M, g.N / 2, g.epi.ldo, 2, 64));
    tmG = tmU = tmO;
    if (g.epi.out_gate) {
      B200_TRY(make_map_out(&tmG, g.epi.out_gate, g.M, g.N / 2, g.epi.ldo, 2, 64));
      B200_TRY(make_map_out(&tmU, g.epi.out_up, g.M, g.N / 2, g.epi.ldo, 2, 64));
    }
    tmR = tmO;
  } else {
    B200_TRY(make_map_out(&tmO, g.epi.out, g.M, g.N, g.epi.ldo, (int)sizeof(TOut), 128));
    tmR = tmG = tmU = tmO;
    if (KIND == EPI_RESID) B200_TRY(make_map_out(&tmR, g.epi.resid_in, g.M, g.N, g.epi.ldo, 4, 128));
  }
  auto kern = gemm_tc2_kernel<BN, KIND, TOut, MN>;
  // The shared-memory attribute and the number of resident clusters are per device.  Clusters are placed inside one
  // GPC, so fewer than sm_count()/2 pairs may be resident at once; the grid is persistent with a static tile
  // assignment, so launch exactly the resident number.
  static PerDeviceOnce setup_once;  // per instantiation
  int max_pairs = 0;
  B200_TRY(setup_once.run([&](int& pairs_out) -> int32_t {
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
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
    pairs_out = n < sm_count() / 2 ? n : sm_count() / 2;
    return B200_OK;
  }, &max_pairs));
  const int items = cdiv(g.M, 2 * PM) * cdiv(g.N, BN) * splits;
  int pairs = max_pairs;
  if (g.max_ctas > 0 && g.max_ctas / 2 < pairs) pairs = g.max_ctas / 2;
  if (pairs > items) pairs = items;
  PushMaps pm;
  for (int i = 0; i < 8; ++i) pm.m[i] = tmO;
  int push_rows = 0;
  if (g.push_rows > 0) {
    if constexpr (MN || KIND != EPI_STORE) {
      return fail(B200_ERR_UNSUPPORTED, "pushed store: only the plain store epilogue of K-major operands");
    } else {
      if (g.push_rows % 32 || g.M % g.push_rows || g.M / g.push_rows > 8)
        return fail(B200_ERR_UNSUPPORTED, "pushed store: %d rows in bands of %d", g.M, g.push_rows);
      for (int o = 0; o < g.M / g.push_rows; ++o) {
        if (!g.push_base[o] || !aligned16(g.push_base[o]))
          return fail(B200_ERR_MISALIGNED, "pushed store: destination %d", o);
        B200_TRY(make_map_out(&pm.m[o], g.push_base[o], g.push_rows, g.N, g.epi.ldo, (int)sizeof(TOut), 128));
      }
      push_rows = g.push_rows;
    }
  }
  BandWait bw;
  if (g.band_flags) {
    if (MN || splits != 1 || g.band_rows <= 0 || g.band_rows % (2 * PM) || g.M % g.band_rows || g.M / g.band_rows > 8 ||
        g.band_first < 0 || g.band_first >= g.M / g.band_rows)
      return fail(B200_ERR_UNSUPPORTED, "banded A operand: %d rows in bands of %d", g.M, g.band_rows);
    bw.flags = g.band_flags;
    bw.epoch = g.band_epoch;
    bw.rows = g.band_rows;
    bw.mt_rot = g.band_first * (g.band_rows / (2 * PM));
    bw.budget = g.band_budget > 0 ? g.band_budget : 4000000000LL;
  }
  B200_CUDA_OK(launch_pdl(kern, dim3(2 * pairs), dim3(P_THREADS), Cfg::kSmemBytes, stream, tmA, tmB, tmO, tmR, tmG,
                          tmU, g.M, g.N, g.K, g.epi, splits, MN ? g.M : 0, device_status_word(), pm, push_rows, bw));
  B200_LAUNCH_OK("gemm_tc2_kernel");
  return B200_OK;
}

// Weight-gradient shape: both operands MN-major, fp32 output (+= when accumulate).  K is always cut into ranges
// whose partial tiles go through the scratch; launch_splitk_reduce sums them in split order and applies the store.
int32_t launch_pair_mn(const GemmArgs& g, cudaStream_t stream) {
  const int pairs = sm_count() / 2;
  const int bn = g.N % 256 == 0 ? 256 : 128;
  const int tiles = (g.M / (2 * PM)) * (g.N / bn);
  const int num_kb = cdiv(g.K, PK);
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= 16 && (s == 1 || num_kb / s >= 8); ++s) {
    if ((size_t)s * g.M * g.N * sizeof(float) > g.splitk_bytes) break;
    const double cost = (double)cdiv(tiles * s, pairs) / s + 0.02 * s;  // rounds of the grid, each 1/s long, + partial traffic
    if (cost < best_cost) { best = s; best_cost = cost; }
  }
  if (bn == 256) B200_TRY((launch_pair_cfg<256, EPI_STORE, float, true>(g, stream, best)));
  else B200_TRY((launch_pair_cfg<128, EPI_STORE, float, true>(g, stream, best)));
  return launch_splitk_reduce(g, best, stream);
}

template <int KIND, typename TOut>
int32_t launch_pair_bn(const GemmArgs& g, cudaStream_t stream) {
  static const int forced = env_int("B200_PAIR_BN", 0);  // tuning knob: 128, 192 or 256 overrides the choice below
  int bn = pair_tile_width(g.M, g.N);
  if (forced == 128 || forced == 192 || forced == 256) bn = forced;
  if (bn == 256) return launch_pair_cfg<256, KIND, TOut>(g, stream);
  if (bn == 192) return launch_pair_cfg<192, KIND, TOut>(g, stream);
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
  // the epilogue stores whole boxes: 32 fp32 columns, 64 bf16 columns (SwiGLU: 64 accumulator columns -> 32 outputs)
  if (g.N < 128 || g.N % (g.out_dtype == B200_F32 && g.kind != EPI_SWIGLU ? 32 : 64)) return false;
  // the staged epilogue writes whole tiles through TMA: no read-modify-write, 16-byte aligned rows
  if (g.kind == EPI_STORE && g.epi.accumulate) return false;
  if (g.kind == EPI_RESID && (g.out_dtype != B200_F32 || !g.epi.resid_in || !aligned16(g.epi.resid_in))) return false;
  if (g.kind == EPI_SWIGLU && g.out_dtype != B200_BF16) return false;
  const int oes = g.out_dtype == B200_F32 ? 4 : 2;
  if (!aligned16(g.epi.out) || ((size_t)g.epi.ldo * oes) % 16) return false;
  if (g.kind == EPI_SWIGLU && g.epi.out_gate && (!aligned16(g.epi.out_gate) || !aligned16(g.epi.out_up))) return false;
  const long tiles = (long)cdiv(g.M, 2 * PM) * cdiv(g.N, pair_tile_width(g.M, g.N));
  return g.M >= 2 * PM && tiles >= sm_count() / 2;
}

// MN-major pair path: dW = dY^T X with both operands stored [K, .], fp32 output, whole 256-row tiles, scratch for the
// partial sums of at least one K range.
bool gemm_tc2_mn_supports(const GemmArgs& g) {
  if (!g.ta || !g.tb || g.kind != EPI_STORE || g.in_dtype != B200_BF16 || g.out_dtype != B200_F32) return false;
  if (g.M % (2 * PM) || g.N % 128 || g.K % 8 || g.K < 8 * PK) return false;
  if (!g.splitk_scratch || g.splitk_bytes < (size_t)g.M * g.N * sizeof(float)) return false;
  if (!aligned16(g.A) || !aligned16(g.B) || !aligned16(g.splitk_scratch) || g.lda % 8 || g.ldb % 8) return false;
  if (!aligned16(g.epi.out) || g.epi.ldo % 4) return false;
  return true;
}

int32_t launch_gemm_tc2_mn(const GemmArgs& g, cudaStream_t stream) {
  if (!gemm_tc2_mn_supports(g)) return fail(B200_ERR_UNSUPPORTED, "the MN-major CTA-pair gemm does not cover this problem");
  return launch_pair_mn(g, stream);
}

int32_t launch_gemm_tc2(const GemmArgs& g, cudaStream_t stream) {
  if (!gemm_tc2_supports(g)) return fail(B200_ERR_UNSUPPORTED, "the CTA-pair gemm does not cover this problem");
  if (g.out_dtype == B200_BF16) return launch_pair_kind<bf16>(g, stream);
  if (g.out_dtype == B200_F32) return launch_pair_kind<float>(g, stream);
  return fail(B200_ERR_BAD_DTYPE, "gemm: unsupported output dtype %d", g.out_dtype);
}

}  // namespace b200
