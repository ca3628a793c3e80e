// Causal attention forward on the 5th-generation tensor cores (bf16, head size
// 64 or 128): test/llama.py:177-209 of the reference for every query position,
// flash-style (the score matrix never leaves the SM).
//
// A CTA owns 128 query rows of one (batch, head) and walks the key/value blocks
// of 128 rows it may attend to.  Warp roles:
//   warp 0      TMA producer: Q once, then K_j and V_j into two 2-stage rings of their own: a K stage is
//               free as soon as S_j is complete (its only reader), a V stage when O += P_j V_j is, so K runs a
//               whole block ahead and S_{j+1} never waits for its operand
//   warp 1      one lane issues tcgen05.mma:  S = Q K_j^T  (fp32, TMEM columns
//               0..127) and, once the probabilities are in shared memory,
//               O += P_j V_j (TMEM columns 128..128+hs, accumulated over all
//               key blocks).  S of block j+1 is issued as soon as the softmax
//               threads hold S of block j in registers, so it is computed
//               beside block j's exponentials.
//   warps 2..9  softmax.  A warp owns 16 query rows and all 128 keys of a block:
//               it reads S with the 16-lane x 256-bit TMEM load, which hands every
//               thread two rows (lane/4 and lane/4 + 8) and two of every eight
//               columns, the accumulator-fragment layout.  A row is therefore
//               spread over the four lanes of a quad: its maximum and its sum
//               take two shuffles, and no warp ever waits for another one
//               inside a block (no exchange through shared memory).  One pass:
//               S is read once, masked on the diagonal block, compared with the
//               row's reference maximum, turned into probabilities (packed fp32x2
//               arithmetic, exp2) and written as bf16 into shared memory in the
//               swizzled K-major layout the MMA reads.  The reference maximum of
//               a row is only raised -- and O in TMEM and the row sum rescaled --
//               when a block's maximum exceeds it by more than 2^8; until then
//               probabilities are taken against the older reference (they stay
//               below 2^8; O / l at the end is exact either way).
// V is consumed as an MN-major operand straight from its row-major layout.
// Head size 64: TMEM use is 256 columns and 115 KB of shared memory, so that two
// CTAs share an SM and one CTA's softmax overlaps the other's MMAs.  Head size
// 128 (one CTA per SM): P has two buffers, so the exponentials of block j+1 run
// beside O += P_j V_j.  All waits are bounded.
#include <cuda.h>

#include <mutex>

#include "attention.cuh"
#include "ptx_sm100.cuh"
#include "tensor_map.cuh"

namespace b200 {

namespace {

constexpr int AQ = 128;   // query rows per CTA
constexpr int AK = 128;   // keys per block
constexpr int A_THREADS = 320;  // producer warp, MMA warp, 8 softmax warps
constexpr int SUB = 128 * 128;  // bytes of one [128 rows x 64 columns] bf16 sub-tile

enum : uint32_t { ST_ATTN_TIMEOUT = 1u << 4, ST_ATTN_ALIGN = 1u << 5 };

template <int HS> struct ACfg {
  static constexpr int kSubs = HS / 64;               // 64-column sub-tiles per row block
  static constexpr int kTileBytes = kSubs * SUB;      // Q, K_j or V_j
  static constexpr int kStages = 2;
  static constexpr int kPBytes = 2 * SUB;             // P: 128 rows x 128 keys
  static constexpr int kPBufs = HS == 128 ? 2 : 1;    // one CTA per SM at head size 128: room for a second P
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kTileBytes;
  static constexpr int kVOff = kKOff + kStages * kTileBytes;
  static constexpr int kPOff = kVOff + kStages * kTileBytes;
  static constexpr int kBarOff = kPOff + kPBufs * kPBytes;
  static constexpr int kSmemBytes = kBarOff + 160;      // hs = 64: 114,816 B, two CTAs fit the 228 KB of an SM; hs = 128: 229,504 B
  static constexpr int kTmemCols = 256;
  static constexpr int kOCol = 128;
};

// 16 TMEM lanes x 256 bits per column group: thread t of the warp receives, for every group of 8 columns, the
// columns 2*(t%4) and 2*(t%4)+1 of lane (t/4) in r[4g], r[4g+1] and of lane (t/4 + 8) in r[4g+2], r[4g+3]
// (the layout of a 16x8 fp32 accumulator fragment).  taddr names the first of the 16 lanes and the first column.
__device__ __forceinline__ void tmem_ld_16x256b_x16(uint32_t taddr, float (&v)[64]) {
  uint32_t r[64];
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
      "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
      "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]),
        "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]),
        "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]),
        "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]),
        "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
// The same shape over 64 columns (8 groups): 32 registers.
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// 16 columns (2 groups): 8 registers.  The rare rescale of O goes through these so that it adds little to the
// register need of the main path.
__device__ __forceinline__ void tmem_ld_16x256b_x2(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st_16x256b_x2(uint32_t taddr, const float (&v)[8]) {
  asm volatile("tcgen05.st.sync.aligned.16x256b.x2.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
               "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
               "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
               "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7]))
               : "memory");
}
__device__ __forceinline__ void st_shared_b32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

template <int HS>
__global__ void __launch_bounds__(A_THREADS, HS == 64 ? 2 : 1)
    attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, bf16* __restrict__ o, float* __restrict__ lse, int seq,
                       int n_heads, int ldo, float scale, uint32_t* status) {
  using C = ACfg<HS>;
  constexpr int NP = C::kPBufs;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kBarOff);
  uint64_t* q_full = bars;          // Q landed
  uint64_t* k_full = bars + 1;      // [2] K_j landed
  uint64_t* v_full = bars + 3;      // [2] V_j landed
  uint64_t* k_empty = bars + 5;     // [2] S_j is complete: its K stage is free
  uint64_t* v_empty = bars + 7;     // [2] O += P_j V_j is complete: its V stage is free
  uint64_t* s_full = bars + 9;      // S_j complete in TMEM
  uint64_t* s_empty = bars + 10;    // softmax has read S_j
  uint64_t* p_full = bars + 11;     // [2] P_j is in its shared-memory buffer
  uint64_t* o_full = bars + 13;     // [2] O += P_j V_j complete in TMEM (P's buffer is free)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);  // 15 barriers + 2 words = 128 bytes
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  // Blocks are dispatched x-fastest: with (head, batch) in x/y and the query tile in z, every long tile (many
  // key blocks) of the whole launch starts before any short one, so the launch does not end on a long tile
  // that started late.
  const int qt = (int)gridDim.z - 1 - (int)blockIdx.z;
  const int h = blockIdx.x, b = blockIdx.y;
  const int t0 = qt * AQ;
  const int n_blocks = qt + 1;  // key blocks 0..qt

  if (threadIdx.x == 0) {
    if (ptx::smem_u32(smem) & 1023u) {
      atomicOr(status, ST_ATTN_ALIGN);
      *abort_flag = 1u;
    } else {
      *abort_flag = 0u;
    }
    ptx::mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&k_full[i], 1);
      ptx::mbar_init(&v_full[i], 1);
      ptx::mbar_init(&k_empty[i], 1);
      ptx::mbar_init(&v_empty[i], 1);
      ptx::mbar_init(&p_full[i], 256);
      ptx::mbar_init(&o_full[i], 1);
    }
    ptx::mbar_init(s_full, 1);
    ptx::mbar_init(s_empty, 256);
    ptx::fence_barrier_init();
    ptx::tma_prefetch_desc(&tmQ);
    ptx::tma_prefetch_desc(&tmK);
    ptx::tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, C::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool aborted = *abort_flag != 0u;
  pdl_wait();  // q, k and v come from the previous kernel

  if (aborted) {
    // fall through to the common exit
  } else if (warp == 0) {
    if (lane == 0) {
      ptx::mbar_arrive_expect_tx(q_full, C::kTileBytes);
#pragma unroll
      for (int s = 0; s < C::kSubs; ++s) ptx::tma_load_3d(smem + C::kQOff + s * SUB, &tmQ, h * HS + 64 * s, t0, b, q_full);
      bool ok = true;
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        ok = ptx::mbar_wait(&k_empty[st], ph ^ 1u, abort_flag, status, ST_ATTN_TIMEOUT);
        if (!ok) break;
        ptx::mbar_arrive_expect_tx(&k_full[st], C::kTileBytes);
#pragma unroll
        for (int s = 0; s < C::kSubs; ++s)
          ptx::tma_load_3d(smem + C::kKOff + st * C::kTileBytes + s * SUB, &tmK, h * HS + 64 * s, j * AK, b, &k_full[st]);
        ok = ptx::mbar_wait(&v_empty[st], ph ^ 1u, abort_flag, status, ST_ATTN_TIMEOUT);
        if (!ok) break;
        ptx::mbar_arrive_expect_tx(&v_full[st], C::kTileBytes);
#pragma unroll
        for (int s = 0; s < C::kSubs; ++s)
          ptx::tma_load_3d(smem + C::kVOff + st * C::kTileBytes + s * SUB, &tmV, h * HS + 64 * s, j * AK, b, &v_full[st]);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = ptx::idesc_bf16_f32(AQ, AK);
      constexpr uint32_t idesc_o = ptx::idesc_bf16_f32(AQ, HS) | (1u << 16);  // V is MN-major
      const uint32_t q_addr = ptx::smem_u32(smem + C::kQOff);
      const uint32_t p_addr = ptx::smem_u32(smem + C::kPOff);
      // Descriptors are built once; a stage or k-step adds its byte offset >> 4 to the address field (shared
      // memory addresses stay below 2^18, so the 14-bit field never carries): the issuing thread is a single
      // instruction stream and two descriptor builds per MMA are most of its work otherwise.
      const uint64_t q_desc = ptx::smem_desc_sw128(q_addr);
      const uint64_t k_desc = ptx::smem_desc_sw128(ptx::smem_u32(smem + C::kKOff));
      const uint64_t p_desc = ptx::smem_desc_sw128(p_addr);
      const uint64_t v_desc = ptx::smem_desc_sw128_mn(ptx::smem_u32(smem + C::kVOff), SUB);
      auto issue_s = [&](int st) {
        const uint64_t ka = k_desc + (uint64_t)st * (C::kTileBytes >> 4);
#pragma unroll
        for (int k = 0; k < HS / 16; ++k) {  // S = Q K^T, contraction over the head dimension
          const uint64_t off = (uint64_t)(((k >> 2) * SUB + (k & 3) * 32) >> 4);
          ptx::mma_bf16_ss(tmem_base, q_desc + off, ka + off, idesc_s, k > 0 ? 1u : 0u);
        }
        ptx::mma_commit(s_full);
        ptx::mma_commit(&k_empty[st]);
      };
      bool ok = ptx::mbar_wait(q_full, 0, abort_flag, status, ST_ATTN_TIMEOUT) &&
                ptx::mbar_wait(&k_full[0], 0, abort_flag, status, ST_ATTN_TIMEOUT);
      if (ok) {
        ptx::tc_fence_after_sync();
        issue_s(0);
      }
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int st = j & 1;
        const int pb = j % NP;
        if (j + 1 < n_blocks) {
          // scores of the next block, once this block's are in the softmax threads' registers
          ok = ptx::mbar_wait(&k_full[st ^ 1], (uint32_t)((j + 1) >> 1) & 1u, abort_flag, status, ST_ATTN_TIMEOUT) &&
               ptx::mbar_wait(s_empty, (uint32_t)j & 1u, abort_flag, status, ST_ATTN_TIMEOUT);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          issue_s(st ^ 1);
        }
        ok = ptx::mbar_wait(&v_full[st], (uint32_t)(j >> 1) & 1u, abort_flag, status, ST_ATTN_TIMEOUT) &&
             ptx::mbar_wait(&p_full[pb], (uint32_t)(j / NP) & 1u, abort_flag, status, ST_ATTN_TIMEOUT);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint64_t va = v_desc + (uint64_t)st * (C::kTileBytes >> 4);
        const uint64_t pa = p_desc + (uint64_t)pb * (C::kPBytes >> 4);
#pragma unroll
        for (int k = 0; k < AK / 16; ++k)  // O += P V, contraction over the 128 keys of the block, 16 rows of V per step
          ptx::mma_bf16_ss(tmem_base + C::kOCol, pa + (uint64_t)(((k >> 2) * SUB + (k & 3) * 32) >> 4),
                           va + (uint64_t)(k * (2048 >> 4)), idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        ptx::mma_commit(&o_full[pb]);
        ptx::mma_commit(&v_empty[st]);
      }
    }
    __syncwarp();
  } else {
    // 8 softmax warps.  Warp w may touch TMEM lanes 32*(w%4) .. +31; of those, warps 2..5 take the first 16
    // and warps 6..9 the other 16.  Thread: rows r0 = lane/4 and r0 + 8 of the warp's 16, columns 2*(lane%4)
    // and +1 of every group of 8.
    const int qd = warp & 3;
    const int hf = (warp - 2) >> 2;
    const int q4 = lane & 3;
    const int row0 = qd * 32 + hf * 16 + (lane >> 2);  // row of the tile == TMEM lane; the second row is row0 + 8
    const int ta = t0 + row0, tb = ta + 8;
    const uint32_t t_lane = tmem_base + ((uint32_t)(qd * 32 + hf * 16) << 16);
    const uint32_t t_o = t_lane + (uint32_t)C::kOCol;
    const float sl2 = scale * 1.4426950408889634f;  // scores are scaled inside the exp2
    // byte offsets of this thread's two P rows inside a 64-key sub-tile (rows are 128 B; the 16-byte chunk index is
    // XOR-ed with row % 8 by the swizzle; the thread's two keys of a chunk are 4 bytes at 4 * q4)
    const uint32_t p_base = ptx::smem_u32(smem + C::kPOff);
    const uint32_t pa_off = (uint32_t)row0 * 128u + 4u * (uint32_t)q4, pb_off = pa_off + 8u * 128u;
    const uint32_t swz = (uint32_t)(row0 & 7);  // (row0 + 8) % 8 is the same
    float ms_a = -INFINITY, ms_b = -INFINITY;  // reference maxima of the two rows, in exp2 units (score * sl2)
    float l_a = 0.f, l_b = 0.f;                // this thread's share of the row sums
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      const int pbuf = j % NP;
      ok = ptx::mbar_wait_warp(s_full, (uint32_t)j & 1u, abort_flag, status, ST_ATTN_TIMEOUT);
      if (!ok) break;
      ptx::tc_fence_after_sync();
      float sv[64];  // sv[4g + {0,1}]: row a, keys 8g + 2*q4 + {0,1};  sv[4g + {2,3}]: row b
      tmem_ld_16x256b_x16(t_lane, sv);
      ptx::tmem_ld_wait();
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(s_empty);  // the MMA warp may overwrite S with the next block's scores
      if (j == qt) {  // diagonal block: keys after the query are masked
        const int u0 = j * AK + 2 * q4;
#pragma unroll
        for (int g = 0; g < 16; ++g) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            if (u0 + 8 * g + e > ta) sv[4 * g + e] = -INFINITY;
            if (u0 + 8 * g + e > tb) sv[4 * g + 2 + e] = -INFINITY;
          }
        }
      }
      float bm_a = -INFINITY, bm_b = -INFINITY;
#pragma unroll
      for (int g = 0; g < 16; ++g) {
        bm_a = ptx::max3(bm_a, sv[4 * g], sv[4 * g + 1]);
        bm_b = ptx::max3(bm_b, sv[4 * g + 2], sv[4 * g + 3]);
      }
      bm_a = quad_max(bm_a) * sl2;  // every row of the diagonal block keeps at least its own key: finite
      bm_b = quad_max(bm_b) * sl2;
      bool o_waited = false;
      if (j == 0) {
        ms_a = bm_a;
        ms_b = bm_b;
      } else if (__any_sync(0xffffffffu, bm_a > ms_a + 8.f || bm_b > ms_b + 8.f)) {
        // raise the references of the warp's rows (tcgen05.ld/st are warp-wide; rows that need no raise get the
        // factor 1).  O must be at rest: every O += P V issued so far has completed.
        const float nm_a = bm_a > ms_a + 8.f ? bm_a : ms_a, nm_b = bm_b > ms_b + 8.f ? bm_b : ms_b;
        const float corr_a = exp2f(ms_a - nm_a), corr_b = exp2f(ms_b - nm_b);
        ms_a = nm_a; ms_b = nm_b;
        l_a *= corr_a; l_b *= corr_b;
        ok = ptx::mbar_wait_warp(&o_full[(j - 1) % NP], (uint32_t)((j - 1) / NP) & 1u, abort_flag, status, ST_ATTN_TIMEOUT);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        o_waited = true;
#pragma unroll 1
        for (int c = 0; c < HS; c += 16) {
          float v[8];
          tmem_ld_16x256b_x2(t_o + (uint32_t)c, v);
          ptx::tmem_ld_wait();
          v[0] *= corr_a; v[1] *= corr_a; v[2] *= corr_b; v[3] *= corr_b;
          v[4] *= corr_a; v[5] *= corr_a; v[6] *= corr_b; v[7] *= corr_b;
          tmem_st_16x256b_x2(t_o + (uint32_t)c, v);
        }
        ptx::tmem_st_wait();
        ptx::tc_fence_before_sync();
      }
      // probabilities against the reference -> bf16 pairs in registers.  The exponentials do not touch P's buffer,
      // so they run before the wait for the MMA that still reads it.
      float2 rs_a = make_float2(0.f, 0.f), rs_b = make_float2(0.f, 0.f);
      const float2 sl2v = make_float2(sl2, sl2);
      const float2 nm_av = make_float2(-ms_a, -ms_a), nm_bv = make_float2(-ms_b, -ms_b);
      uint32_t pk[32];  // pk[2g]: row a, pk[2g + 1]: row b (sv is dead once they are built)
#pragma unroll
      for (int g = 0; g < 16; ++g) {
        const float2 xa = __ffma2_rn(make_float2(sv[4 * g], sv[4 * g + 1]), sl2v, nm_av);
        const float2 xb = __ffma2_rn(make_float2(sv[4 * g + 2], sv[4 * g + 3]), sl2v, nm_bv);
        const float2 pa = make_float2(exp2f(xa.x), exp2f(xa.y));
        const float2 pb = make_float2(exp2f(xb.x), exp2f(xb.y));
        rs_a = __fadd2_rn(rs_a, pa);
        rs_b = __fadd2_rn(rs_b, pb);
        const __nv_bfloat162 ha = __floats2bfloat162_rn(pa.x, pa.y), hb = __floats2bfloat162_rn(pb.x, pb.y);
        pk[2 * g] = *reinterpret_cast<const uint32_t*>(&ha);
        pk[2 * g + 1] = *reinterpret_cast<const uint32_t*>(&hb);
      }
      if (j >= NP && !(o_waited && NP == 1)) {
        // this block's P buffer is being read until O += P_{j-NP} V_{j-NP} completes
        ok = ptx::mbar_wait_warp(&o_full[pbuf], (uint32_t)(j / NP - 1) & 1u, abort_flag, status, ST_ATTN_TIMEOUT);
        if (!ok) break;
      }
      const uint32_t pw = p_base + (uint32_t)(pbuf * C::kPBytes);
#pragma unroll
      for (int g = 0; g < 16; ++g) {
        const uint32_t chunk = (uint32_t)(g >> 3) * (uint32_t)SUB + ((((uint32_t)g & 7u) ^ swz) << 4);
        st_shared_b32(pw + chunk + pa_off, pk[2 * g]);
        st_shared_b32(pw + chunk + pb_off, pk[2 * g + 1]);
      }
      l_a += rs_a.x + rs_a.y;
      l_b += rs_b.x + rs_b.y;
      ptx::fence_proxy_async();  // make the generic-proxy writes of P visible to the MMA's async proxy
      ptx::mbar_arrive(&p_full[pbuf]);
    }
    if (ok) ok = ptx::mbar_wait_warp(&o_full[(n_blocks - 1) % NP], (uint32_t)((n_blocks - 1) / NP) & 1u, abort_flag,
                                     status, ST_ATTN_TIMEOUT);
    if (ok) {
      ptx::tc_fence_after_sync();
      l_a = quad_sum(l_a);
      l_b = quad_sum(l_b);
      const float inv_a = 1.f / l_a, inv_b = 1.f / l_b;
      bf16* dst_a = o + ((size_t)b * seq + ta) * ldo + h * HS + 2 * q4;
      bf16* dst_b = dst_a + (size_t)8 * ldo;
#pragma unroll
      for (int c = 0; c < HS; c += 64) {
        float v[32];
        tmem_ld_16x256b_x8(t_o + (uint32_t)c, v);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          if (ta < seq)
            *reinterpret_cast<__nv_bfloat162*>(dst_a + c + 8 * g) = __floats2bfloat162_rn(v[4 * g] * inv_a, v[4 * g + 1] * inv_a);
          if (tb < seq)
            *reinterpret_cast<__nv_bfloat162*>(dst_b + c + 8 * g) = __floats2bfloat162_rn(v[4 * g + 2] * inv_b, v[4 * g + 3] * inv_b);
        }
      }
      if (lse && q4 == 0) {
        float* lrow = lse + ((size_t)b * n_heads + h) * seq;
        if (ta < seq) lrow[ta] = ms_a * 0.6931471805599453f + __logf(l_a);
        if (tb < seq) lrow[tb] = ms_b * 0.6931471805599453f + __logf(l_b);
      }
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int HS>
int32_t launch_hs(const AttnArgs& a, cudaStream_t stream) {
  using C = ACfg<HS>;
  CUtensorMap tq, tk, tv;
  const int cols = a.n_heads * HS;
  B200_TRY(make_map_3d(&tq, a.q, a.batch, a.seq, cols, a.ldq));
  B200_TRY(make_map_3d(&tk, a.k, a.batch, a.seq, cols, a.ldkv));
  B200_TRY(make_map_3d(&tv, a.v, a.batch, a.seq, cols, a.ldkv));
  auto kern = attn_fwd_tc_kernel<HS>;
  static PerDeviceOnce attr_once;
  B200_TRY(attr_once.run([&](int&) -> int32_t {
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    return B200_OK;
  }));
  dim3 grid(a.n_heads, a.batch, cdiv(a.seq, AQ));
  B200_CUDA_OK(launch_pdl(kern, grid, dim3(A_THREADS), C::kSmemBytes, stream, tq, tk, tv, (bf16*)a.o, a.lse, a.seq,
                          a.n_heads, a.ldo, 1.f / sqrtf((float)HS), device_status_word()));
  B200_LAUNCH_OK("attn_fwd_tc_kernel");
  return B200_OK;
}

}  // namespace

bool attn_fwd_mma_supports(const AttnArgs& a) {
  return a.dtype == B200_BF16 && (a.head_size == 64 || a.head_size == 128) && a.ldq % 8 == 0 && a.ldkv % 8 == 0 &&
         a.ldo % 8 == 0 && aligned16(a.q) && aligned16(a.k) && aligned16(a.v) && aligned16(a.o) && a.batch > 0 &&
         a.seq > 0 && a.n_heads > 0;
}

int32_t launch_attn_fwd_mma(const AttnArgs& a, cudaStream_t stream) {
  if (!attn_fwd_mma_supports(a))
    return fail(B200_ERR_UNSUPPORTED, "tensor-core attention needs bf16, head size 64 or 128 and 16-byte aligned rows");
  if (a.head_size == 64) return launch_hs<64>(a, stream);
  return launch_hs<128>(a, stream);
}

}  // namespace b200
