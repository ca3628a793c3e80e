// Causal attention backward on the 5th-generation tensor cores (bf16, head
// size 64).  Given q, k, v, the forward's lse, dO and delta = rowsum(dO * O):
//   P  = exp(q k^T / sqrt(hs) - lse)          recomputed block by block
//   dV = P^T dO         dP = dO V^T
//   dS = P * (dP - delta) / sqrt(hs)
//   dK = dS^T Q         dQ = dS K
// which is what the reference's AD rules (exp, divide, reduce-add, dot_general:
// Implementations/HLODerivatives.td:1133-1182) compose for test/llama.py:177-209.
//
// Two passes of one kernel template, both free of atomics (fixed summation order):
//   MODE_DKV  a CTA owns 128 keys, streams the query blocks at or after them,
//             accumulates dV and dK in TMEM
//   MODE_DQ   a CTA owns 128 queries, streams the key blocks at or before
//             them, accumulates dQ in TMEM
// Per (query block, key block) pair: S and dP on the tensor cores into TMEM,
// 8 warps turn them into bf16 P and dS tiles in shared memory (swizzled, so the
// same bytes serve as a K-major or an MN-major operand), then the accumulating
// MMAs.  Warp 0 is the TMA producer, warp 1 issues the MMAs.  Waits are bounded.
#include <cuda.h>

#include "attention.cuh"
#include "ptx_sm100.cuh"
#include "tensor_map.cuh"

namespace b200 {

namespace {

constexpr int BQ = 128, BK_ = 128, HSB = 64;
constexpr int BW_THREADS = 320;
constexpr int SUBT = 128 * 128;  // bytes of one [128 rows x 64 columns] bf16 tile
enum { MODE_DKV = 0, MODE_DQ = 1 };
enum : uint32_t { ST_ATTNB_TIMEOUT = 1u << 6, ST_ATTNB_ALIGN = 1u << 7 };

// shared memory map (bytes)
constexpr int kFix0 = 0;                 // fixed tile 0 (DKV: K_j, DQ: Q_i)
constexpr int kFix1 = SUBT;              // fixed tile 1 (DKV: V_j, DQ: dO_i)
constexpr int kStr = 2 * SUBT;           // 2 stages x {tile 0 (DKV: Q_i, DQ: K_j), tile 1 (DKV: dO_i, DQ: V_j)}
constexpr int kP = kStr + 4 * SUBT;      // 2 x P  [128 q][128 k] as two sub-tiles (keys 0..63, 64..127); pairs alternate
constexpr int kDS = kP + 4 * SUBT;       // 2 x dS, same layout
constexpr int kBars = kDS + 4 * SUBT;    // 14 sub-tiles = 224 KB
constexpr int kBwdSmem = kBars + 256;
// TMEM columns
constexpr int cS = 0, cDP = 128, cAcc0 = 256, cAcc1 = 320, kBwdTmem = 512;

struct BwdParams {
  const float* lse;
  const float* delta;
  bf16* out0;  // DKV: dV, DQ: dQ
  bf16* out1;  // DKV: dK
  int ld_out;
  int seq, n_heads;
  float scale;
};

template <int MODE>
__global__ void __launch_bounds__(BW_THREADS, 1)
    attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, BwdParams prm,
                       uint32_t* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBars);
  uint64_t* fix_full = bars;        // fixed tiles landed
  uint64_t* str_full = bars + 1;    // [2] streamed tiles landed
  uint64_t* str_empty = bars + 3;   // [2] every MMA reading the stage is done
  uint64_t* s_full = bars + 5;      // S and dP complete in TMEM
  uint64_t* s_empty = bars + 6;     // S and dP have been read
  uint64_t* p_full = bars + 7;      // P / dS tiles written
  uint64_t* g_done = bars + 8;      // [2] accumulating MMAs of a pair are done (its P / dS buffer is free); pairs alternate
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  // (head, batch) in x/y, the block index in z: blocks are dispatched x-fastest, so the longest loops of the
  // whole launch start first
  const int own = blockIdx.z, h = blockIdx.x, b = blockIdx.y;
  const int nblk = (prm.seq + 127) / 128;
  // DKV: own key block `own`, query blocks own..nblk-1.  DQ: own query block nblk-1-own (long ones first), key blocks 0..it.
  const int own_blk = MODE == MODE_DKV ? own : nblk - 1 - own;
  const int first = MODE == MODE_DKV ? own_blk : 0;
  const int n_it = MODE == MODE_DKV ? nblk - own_blk : own_blk + 1;
  const int col = h * HSB;

  if (threadIdx.x == 0) {
    if (ptx::smem_u32(smem) & 1023u) {
      atomicOr(status, ST_ATTNB_ALIGN);
      *abort_flag = 1u;
    } else {
      *abort_flag = 0u;
    }
    ptx::mbar_init(fix_full, 1);
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&str_full[i], 1);
      ptx::mbar_init(&str_empty[i], 1);
    }
    ptx::mbar_init(s_full, 1);
    ptx::mbar_init(s_empty, 256);
    ptx::mbar_init(p_full, 256);
    ptx::mbar_init(&g_done[0], 1);
    ptx::mbar_init(&g_done[1], 1);
    ptx::fence_barrier_init();
    ptx::tma_prefetch_desc(&tmQ);
    ptx::tma_prefetch_desc(&tmK);
    ptx::tma_prefetch_desc(&tmV);
    ptx::tma_prefetch_desc(&tmDO);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kBwdTmem);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool aborted = *abort_flag != 0u;
  pdl_wait();  // the operands come from the kernels before; everything above overlapped their tail

  if (aborted) {
    // common exit below
  } else if (warp == 0) {
    if (lane == 0) {
      const int own_row = own_blk * 128;
      ptx::mbar_arrive_expect_tx(fix_full, 2 * SUBT);
      if (MODE == MODE_DKV) {
        ptx::tma_load_3d(smem + kFix0, &tmK, col, own_row, b, fix_full);
        ptx::tma_load_3d(smem + kFix1, &tmV, col, own_row, b, fix_full);
      } else {
        ptx::tma_load_3d(smem + kFix0, &tmQ, col, own_row, b, fix_full);
        ptx::tma_load_3d(smem + kFix1, &tmDO, col, own_row, b, fix_full);
      }
      bool ok = true;
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it & 1;
        const uint32_t ph = (uint32_t)(it >> 1) & 1u;
        ok = ptx::mbar_wait(&str_empty[st], ph ^ 1u, abort_flag, status, ST_ATTNB_TIMEOUT);
        if (!ok) break;
        const int row = (first + it) * 128;
        uint8_t* dst = smem + kStr + st * 2 * SUBT;
        ptx::mbar_arrive_expect_tx(&str_full[st], 2 * SUBT);
        if (MODE == MODE_DKV) {
          ptx::tma_load_3d(dst, &tmQ, col, row, b, &str_full[st]);
          ptx::tma_load_3d(dst + SUBT, &tmDO, col, row, b, &str_full[st]);
        } else {
          ptx::tma_load_3d(dst, &tmK, col, row, b, &str_full[st]);
          ptx::tma_load_3d(dst + SUBT, &tmV, col, row, b, &str_full[st]);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t id_kk = ptx::idesc_bf16_f32(128, 128);                          // A, B K-major
      constexpr uint32_t id_mm = ptx::idesc_bf16_f32(128, HSB) | (1u << 15) | (1u << 16);  // A, B MN-major
      constexpr uint32_t id_km = ptx::idesc_bf16_f32(128, HSB) | (1u << 16);               // A K-major, B MN-major
      // Descriptors are built once; a stage or a k-step adds its byte offset >> 4 to the address field (shared-memory
      // addresses stay below 2^18, so the 14-bit field never carries).  One thread issues the 16 to 24 MMAs of an
      // iteration: two descriptor builds per MMA were most of its instruction stream.
      const uint32_t str_addr = ptx::smem_u32(smem + kStr), fix_addr = ptx::smem_u32(smem + kFix0);
      const uint64_t str_k = ptx::smem_desc_sw128(str_addr), str_m = ptx::smem_desc_sw128_mn(str_addr, SUBT);
      const uint64_t fix_k = ptx::smem_desc_sw128(fix_addr), fix_m = ptx::smem_desc_sw128_mn(fix_addr, SUBT);
      const uint64_t p_m = ptx::smem_desc_sw128_mn(ptx::smem_u32(smem + kP), SUBT);
      const uint64_t ds_m = ptx::smem_desc_sw128_mn(ptx::smem_u32(smem + kDS), SUBT);
      const uint64_t ds_k = ptx::smem_desc_sw128(ptx::smem_u32(smem + kDS));
      constexpr uint64_t kSub = SUBT >> 4;
      // S = Q K^T and dP = dO V^T of one streamed pair (stage st)
      auto issue_scores = [&](int st) {
        const uint64_t s0k = str_k + (uint64_t)(2 * st) * kSub, s1k = s0k + kSub;
        const uint64_t f0k = fix_k, f1k = fix_k + kSub;
        const uint64_t q_k = MODE == MODE_DKV ? s0k : f0k, do_k = MODE == MODE_DKV ? s1k : f1k;
        const uint64_t k_k = MODE == MODE_DKV ? f0k : s0k, v_k = MODE == MODE_DKV ? f1k : s1k;
#pragma unroll
        for (int k = 0; k < HSB / 16; ++k)
          ptx::mma_bf16_ss(tmem_base + cS, q_k + (uint64_t)(2 * k), k_k + (uint64_t)(2 * k), id_kk, k > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < HSB / 16; ++k)
          ptx::mma_bf16_ss(tmem_base + cDP, do_k + (uint64_t)(2 * k), v_k + (uint64_t)(2 * k), id_kk, k > 0 ? 1u : 0u);
        ptx::mma_commit(s_full);
      };
      bool ok = ptx::mbar_wait(fix_full, 0, abort_flag, status, ST_ATTNB_TIMEOUT) &&
                ptx::mbar_wait(&str_full[0], 0, abort_flag, status, ST_ATTNB_TIMEOUT);
      if (ok) {
        ptx::tc_fence_after_sync();
        issue_scores(0);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it & 1;
        const uint32_t ip = (uint32_t)it & 1u;
        if (it + 1 < n_it) {
          // the next pair's scores as soon as the softmax threads hold this pair's S and dP in registers: they are
          // computed beside this pair's exponentials
          ok = ptx::mbar_wait(&str_full[st ^ 1], (uint32_t)((it + 1) >> 1) & 1u, abort_flag, status, ST_ATTNB_TIMEOUT) &&
               ptx::mbar_wait(s_empty, ip, abort_flag, status, ST_ATTNB_TIMEOUT);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          issue_scores(st ^ 1);
        }
        const uint64_t s0m = str_m + (uint64_t)(2 * st) * kSub, s1m = s0m + kSub;
        const uint64_t q_m = MODE == MODE_DKV ? s0m : fix_m, do_m = s1m;  // MN-major views (do_m: dKV pass only)
        const uint64_t k_m = s0m;                                        // dQ pass only
        const uint64_t pb = (uint64_t)(2 * st) * kSub;                   // this pair's P / dS buffer
        ok = ptx::mbar_wait(p_full, ip, abort_flag, status, ST_ATTNB_TIMEOUT);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        if (MODE == MODE_DKV) {
#pragma unroll
          for (int k = 0; k < BQ / 16; ++k) {  // contraction over the 128 queries, 16 rows (2048 B) per step
            const uint64_t off = (uint64_t)(k * (2048 >> 4));
            // dV[key, e] += sum_q P[q, key] dO[q, e]
            ptx::mma_bf16_ss(tmem_base + cAcc0, p_m + pb + off, do_m + off, id_mm, (it > 0 || k > 0) ? 1u : 0u);
          }
#pragma unroll
          for (int k = 0; k < BQ / 16; ++k) {
            const uint64_t off = (uint64_t)(k * (2048 >> 4));
            // dK[key, e] += sum_q dS[q, key] Q[q, e]
            ptx::mma_bf16_ss(tmem_base + cAcc1, ds_m + pb + off, q_m + off, id_mm, (it > 0 || k > 0) ? 1u : 0u);
          }
        } else {
#pragma unroll
          for (int k = 0; k < BK_ / 16; ++k) {  // dQ[q, e] += sum_key dS[q, key] K[key, e]
            const uint64_t aoff = (uint64_t)(((k >> 2) * SUBT + (k & 3) * 32) >> 4);
            ptx::mma_bf16_ss(tmem_base + cAcc0, ds_k + pb + aoff, k_m + (uint64_t)(k * (2048 >> 4)), id_km,
                             (it > 0 || k > 0) ? 1u : 0u);
          }
        }
        ptx::mma_commit(&g_done[st]);
        ptx::mma_commit(&str_empty[st]);
      }
    }
    __syncwarp();
  } else {
    const int qd = warp & 3;
    const int hf = (warp - 2) >> 2;
    const int row = qd * 32 + lane;  // TMEM lane: the query row of the pair
    const uint32_t lane_base = tmem_base + ((uint32_t)(qd * 32) << 16);
    const float sl2 = prm.scale * 1.4426950408889634f;
    uint8_t* p_row0 = smem + kP + hf * SUBT + row * 128;
    uint8_t* ds_row0 = smem + kDS + hf * SUBT + row * 128;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const uint32_t ip = (uint32_t)it & 1u;
      const int qb = MODE == MODE_DKV ? first + it : own_blk;
      const int kb = MODE == MODE_DKV ? own_blk : it;
      const int t = qb * 128 + row;
      const bool valid = t < prm.seq;
      const size_t stat = ((size_t)b * prm.n_heads + h) * prm.seq + (valid ? t : 0);
      const float lse2 = prm.lse[stat] * 1.4426950408889634f;
      const float dlt = prm.delta[stat];
      const bool diag = qb == kb;
      const int u0 = kb * 128 + hf * 64;
      uint8_t* p_row = p_row0 + (it & 1) * 2 * SUBT;  // pairs alternate between two P / dS buffers
      uint8_t* ds_row = ds_row0 + (it & 1) * 2 * SUBT;
      ok = ptx::mbar_wait(s_full, ip, abort_flag, status, ST_ATTNB_TIMEOUT);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < 64; c += 32) {
        float sv[32], dp[32];
        ptx::tmem_ld32(lane_base + (uint32_t)(cS + hf * 64 + c), sv);
        ptx::tmem_ld32(lane_base + (uint32_t)(cDP + hf * 64 + c), dp);
        ptx::tmem_ld_wait();
        if (c == 32) {
          // S and dP of this pair are in registers: the MMA warp may compute the next pair's
          ptx::tc_fence_before_sync();
          ptx::mbar_arrive(s_empty);
        }
        if (c == 0 && it > 1) {
          // this buffer's P / dS of two pairs ago must have been consumed before they are overwritten
          ok = ptx::mbar_wait(&g_done[it & 1], (uint32_t)((it - 2) >> 1) & 1u, abort_flag, status, ST_ATTNB_TIMEOUT);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 praw, draw;
          __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(&praw);
          __nv_bfloat162* dd = reinterpret_cast<__nv_bfloat162*>(&draw);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int e0 = g * 8 + 2 * i;
            float p0 = exp2f(fmaf(sv[e0], sl2, -lse2));
            float p1 = exp2f(fmaf(sv[e0 + 1], sl2, -lse2));
            if (!valid || (diag && u0 + c + e0 > t)) p0 = 0.f;
            if (!valid || (diag && u0 + c + e0 + 1 > t)) p1 = 0.f;
            const float d0 = p0 * (dp[e0] - dlt) * prm.scale;
            const float d1 = p1 * (dp[e0 + 1] - dlt) * prm.scale;
            pp[i] = __floats2bfloat162_rn(p0, p1);
            dd[i] = __floats2bfloat162_rn(d0, d1);
          }
          const int ch = (c >> 3) + g;
          const int off = (ch ^ (row & 7)) << 4;
          if (MODE == MODE_DKV) *reinterpret_cast<uint4*>(p_row + off) = praw;
          *reinterpret_cast<uint4*>(ds_row + off) = draw;
        }
      }
      if (!ok) break;
      ptx::fence_proxy_async();
      ptx::mbar_arrive(p_full);
    }
    // epilogue: the last pair's accumulating MMAs complete the sums
    if (ok) ok = ptx::mbar_wait(&g_done[(n_it - 1) & 1], (uint32_t)((n_it - 1) >> 1) & 1u, abort_flag, status,
                                ST_ATTNB_TIMEOUT);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      ptx::tc_fence_after_sync();
      const int r_glob = own_blk * 128 + row;  // DKV: key row, DQ: query row
      if (MODE == MODE_DKV) {
        // hf 0 writes dV (columns cAcc0..), hf 1 writes dK (columns cAcc1..)
        bf16* dst = (hf == 0 ? prm.out0 : prm.out1) + ((size_t)b * prm.seq + r_glob) * prm.ld_out + col;
        const uint32_t src = lane_base + (uint32_t)(hf == 0 ? cAcc0 : cAcc1);
#pragma unroll
        for (int c = 0; c < 64; c += 32) {
          float v[32];
          ptx::tmem_ld32(src + (uint32_t)c, v);
          ptx::tmem_ld_wait();
          if (r_glob < prm.seq) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float w[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) w[i] = v[g * 8 + i];
              store8(dst + c + g * 8, w);
            }
          }
        }
      } else {
        bf16* dst = prm.out0 + ((size_t)b * prm.seq + r_glob) * prm.ld_out + col + hf * 32;
        float v[32];
        ptx::tmem_ld32(lane_base + (uint32_t)(cAcc0 + hf * 32), v);
        ptx::tmem_ld_wait();
        if (r_glob < prm.seq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = v[g * 8 + i];
            store8(dst + g * 8, w);
          }
        }
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
    ptx::tmem_dealloc(tmem_base, kBwdTmem);
  }
}

}  // namespace

bool attn_bwd_tc_supports(const AttnBwdArgs& a) {
  const AttnArgs& f = a.f;
  return f.dtype == B200_BF16 && f.head_size == 64 && f.ldq % 8 == 0 && f.ldkv % 8 == 0 && a.lddo % 8 == 0 &&
         a.lddq % 8 == 0 && a.lddkv % 8 == 0 && a.lddq == a.lddkv && aligned16(f.q) && aligned16(f.k) &&
         aligned16(f.v) && aligned16(a.d_o) && aligned16(a.dq) && aligned16(a.dk) && aligned16(a.dv) && f.lse &&
         a.delta && f.batch > 0 && f.seq > 0 && f.n_heads > 0;
}

int32_t launch_attn_bwd_tc(const AttnBwdArgs& a, cudaStream_t stream) {
  if (!attn_bwd_tc_supports(a))
    return fail(B200_ERR_UNSUPPORTED, "tensor-core attention backward needs bf16, head size 64 and 16-byte aligned rows");
  const AttnArgs& f = a.f;
  B200_TRY(launch_attn_delta(a, stream));
  CUtensorMap tq, tk, tv, tdo;
  const int cols = f.n_heads * 64;
  B200_TRY(make_map_3d(&tq, f.q, f.batch, f.seq, cols, f.ldq));
  B200_TRY(make_map_3d(&tk, f.k, f.batch, f.seq, cols, f.ldkv));
  B200_TRY(make_map_3d(&tv, f.v, f.batch, f.seq, cols, f.ldkv));
  B200_TRY(make_map_3d(&tdo, a.d_o, f.batch, f.seq, cols, a.lddo));
  static PerDeviceOnce attr_once;
  B200_TRY(attr_once.run([&](int&) -> int32_t {
    B200_CUDA_OK(cudaFuncSetAttribute(attn_bwd_tc_kernel<MODE_DKV>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem));
    B200_CUDA_OK(cudaFuncSetAttribute(attn_bwd_tc_kernel<MODE_DQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem));
    return B200_OK;
  }));
  BwdParams prm;
  prm.lse = f.lse; prm.delta = a.delta; prm.seq = f.seq; prm.n_heads = f.n_heads;
  prm.scale = 1.f / sqrtf(64.f);
  dim3 grid(f.n_heads, f.batch, cdiv(f.seq, 128));
  prm.out0 = (bf16*)a.dv; prm.out1 = (bf16*)a.dk; prm.ld_out = a.lddkv;
  B200_CUDA_OK(launch_pdl(attn_bwd_tc_kernel<MODE_DKV>, grid, dim3(BW_THREADS), kBwdSmem, stream, tq, tk, tv, tdo, prm,
                          device_status_word()));
  B200_LAUNCH_OK("attn_bwd_tc_kernel<dkv>");
  prm.out0 = (bf16*)a.dq; prm.out1 = nullptr; prm.ld_out = a.lddq;
  B200_CUDA_OK(launch_pdl(attn_bwd_tc_kernel<MODE_DQ>, grid, dim3(BW_THREADS), kBwdSmem, stream, tq, tk, tv, tdo, prm,
                          device_status_word()));
  B200_LAUNCH_OK("attn_bwd_tc_kernel<dq>");
  return B200_OK;
}

}  // namespace b200
