// Causal attention forward on the 5th-generation tensor cores (bf16, head size
// 64 or 128): test/llama.py:177-209 of the reference for every query position,
// flash-style (the score matrix never leaves the SM).
//
// A CTA owns 128 query rows of one (batch, head) and walks the key/value blocks
// of 128 rows it may attend to.  Warp roles:
//   warp 0      TMA producer: Q once, then K_j / V_j into a 2-stage ring
//   warp 1      one lane issues tcgen05.mma:  S = Q K_j^T  (fp32, TMEM columns
//               0..127) and, once the probabilities are in shared memory,
//               O += P_j V_j (TMEM columns 128..128+hs, accumulated over all
//               key blocks).  S of block j+1 is issued as soon as the softmax
//               threads hold S of block j in registers, so it is computed
//               beside block j's exponentials.
//   warps 2..9  softmax, two threads per query row (64 keys each): read S from
//               TMEM once, mask the diagonal block, running reference maximum
//               and row sum in fp32, write P as bf16 into shared memory in the
//               swizzled K-major layout the MMA reads.  The reference maximum of
//               a row is only raised -- and O in TMEM and the row sum rescaled --
//               when a block's maximum exceeds it by more than 2^8; until then
//               probabilities are taken against the older reference (they stay
//               below 2^8; O / l at the end is exact either way).
// V is consumed as an MN-major operand straight from its row-major layout.
// TMEM use is 256 columns so that two CTAs share an SM and one CTA's softmax
// overlaps the other's MMAs.  All waits are bounded.
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
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kTileBytes;
  static constexpr int kVOff = kKOff + kStages * kTileBytes;
  static constexpr int kPOff = kVOff + kStages * kTileBytes;
  static constexpr int kXchgOff = kPOff + kPBytes;      // [2][128] bf16 block maxima exchanged between the halves of a row
  static constexpr int kBarOff = kXchgOff + 2 * 128 * 2;
  static constexpr int kSmemBytes = kBarOff + 128;      // hs = 64: 115,328 B, two CTAs fit the 228 KB of an SM
  static constexpr int kTmemCols = 256;
  static constexpr int kOCol = 128;
};

template <int HS>
__global__ void __launch_bounds__(A_THREADS, HS == 64 ? 2 : 1)
    attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, bf16* __restrict__ o, float* __restrict__ lse, int seq,
                       int n_heads, int ldo, float scale, uint32_t* status) {
  using C = ACfg<HS>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kBarOff);
  uint64_t* q_full = bars;          // Q landed
  uint64_t* kv_full = bars + 1;     // [2] K_j and V_j landed
  uint64_t* kv_empty = bars + 3;    // [2] both MMAs of block j are done with the stage
  uint64_t* s_full = bars + 5;      // S_j complete in TMEM
  uint64_t* s_empty = bars + 6;     // softmax has read S_j
  uint64_t* p_full = bars + 7;      // P_j is in shared memory
  uint64_t* o_full = bars + 8;      // O += P_j V_j complete in TMEM (P_j and the stage are free, O at rest)
  uint64_t* x_bar = bars + 10;      // the two threads of every row have published their block maximum
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);  // 11 barriers + 2 words = 96 bytes
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
      ptx::mbar_init(&kv_full[i], 1);
      ptx::mbar_init(&kv_empty[i], 1);
    }
    ptx::mbar_init(s_full, 1);
    ptx::mbar_init(s_empty, 256);
    ptx::mbar_init(p_full, 256);
    ptx::mbar_init(o_full, 1);
    ptx::mbar_init(x_bar, 256);
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
        ok = ptx::mbar_wait(&kv_empty[st], ph ^ 1u, abort_flag, status, ST_ATTN_TIMEOUT);
        if (!ok) break;
        ptx::mbar_arrive_expect_tx(&kv_full[st], 2 * C::kTileBytes);
#pragma unroll
        for (int s = 0; s < C::kSubs; ++s) {
          ptx::tma_load_3d(smem + C::kKOff + st * C::kTileBytes + s * SUB, &tmK, h * HS + 64 * s, j * AK, b, &kv_full[st]);
          ptx::tma_load_3d(smem + C::kVOff + st * C::kTileBytes + s * SUB, &tmV, h * HS + 64 * s, j * AK, b, &kv_full[st]);
        }
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
      };
      bool ok = ptx::mbar_wait(q_full, 0, abort_flag, status, ST_ATTN_TIMEOUT) &&
                ptx::mbar_wait(&kv_full[0], 0, abort_flag, status, ST_ATTN_TIMEOUT);
      if (ok) {
        ptx::tc_fence_after_sync();
        issue_s(0);
      }
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int st = j & 1;
        const uint32_t jp = (uint32_t)j & 1u;
        if (j + 1 < n_blocks) {
          // scores of the next block, once this block's are in the softmax threads' registers
          ok = ptx::mbar_wait(&kv_full[st ^ 1], (uint32_t)((j + 1) >> 1) & 1u, abort_flag, status, ST_ATTN_TIMEOUT) &&
               ptx::mbar_wait(s_empty, jp, abort_flag, status, ST_ATTN_TIMEOUT);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          issue_s(st ^ 1);
        }
        ok = ptx::mbar_wait(p_full, jp, abort_flag, status, ST_ATTN_TIMEOUT);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint64_t va = v_desc + (uint64_t)st * (C::kTileBytes >> 4);
#pragma unroll
        for (int k = 0; k < AK / 16; ++k)  // O += P V, contraction over the 128 keys of the block, 16 rows of V per step
          ptx::mma_bf16_ss(tmem_base + C::kOCol, p_desc + (uint64_t)(((k >> 2) * SUB + (k & 3) * 32) >> 4),
                           va + (uint64_t)(k * (2048 >> 4)), idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        ptx::mma_commit(o_full);
        ptx::mma_commit(&kv_empty[st]);
      }
    }
    __syncwarp();
  } else {
    // 8 softmax warps: warps 2..5 take keys 0..63 of every block and the first
    // half of the output columns, warps 6..9 the other halves; the two threads
    // of a row exchange their block maxima through shared memory.
    const int qd = warp & 3;
    const int hf = (warp - 2) >> 2;
    const int row = qd * 32 + lane;  // row of the tile == TMEM lane
    const int t = t0 + row;
    constexpr int OH = HS / 2;       // output columns per thread
    const uint32_t t_s = tmem_base + ((uint32_t)(qd * 32) << 16) + (uint32_t)(hf * 64);
    const uint32_t t_o = tmem_base + ((uint32_t)(qd * 32) << 16) + (uint32_t)(C::kOCol + hf * OH);
    const float sl2 = scale * 1.4426950408889634f;  // scores are scaled inside the exp2
    uint8_t* p_row = smem + C::kPOff + hf * SUB + row * 128;
    bf16* xchg = reinterpret_cast<bf16*>(smem + C::kXchgOff);  // [2][128]
    float ms = -INFINITY;  // reference maximum of the row, in exp2 units (score * sl2)
    float l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      const uint32_t jp = (uint32_t)j & 1u;
      ok = ptx::mbar_wait(s_full, jp, abort_flag, status, ST_ATTN_TIMEOUT);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after_sync();
      const bool diag = (j == qt);  // diagonal block: keys after the query are masked
      const int u0 = j * AK + hf * 64;
      // pass 1: maximum of this thread's 64 scores, 32 at a time (the 64 live values of pass 2 and the
      // 32 of a rescale would not fit the register budget of two CTAs per SM together)
      float bm = -INFINITY;
#pragma unroll
      for (int c = 0; c < 64; c += 32) {
        float s32[32];
        ptx::tmem_ld32(t_s + (uint32_t)c, s32);
        ptx::tmem_ld_wait();
        if (diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (u0 + c + i > t) s32[i] = -INFINITY;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) bm = ptx::max3(bm, s32[i], s32[i + 1]);
      }
      // Both threads of a row must adopt the same maximum, but it need not be
      // exact: each rounds its own to bf16 and both take the larger of the two
      // rounded values.
      const bf16 bmh = __float2bfloat16_rn(bm);
      xchg[hf * 128 + row] = bmh;
      ptx::mbar_arrive(x_bar);  // release: the store above is visible to whoever sees the phase complete
      ok = ptx::mbar_wait(x_bar, jp, abort_flag, status, ST_ATTN_TIMEOUT);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      bm = fmaxf(__bfloat162float(bmh), __bfloat162float(xchg[(hf ^ 1) * 128 + row]));
      const float bms = bm * sl2;  // finite or -inf only for a fully masked half, which the partner's value covers
      bool o_waited = false;
      if (j == 0) {
        ms = bms;
      } else if (__any_sync(0xffffffffu, bms > ms + 8.f)) {
        // raise the reference of every row of the warp (tcgen05.ld/st are warp-wide); the partner warp sees the same
        // maxima and decides the same.  O must be at rest: O += P_{j-1} V_{j-1} has completed.
        const float nm = fmaxf(ms, bms);
        const float corr = exp2f(ms - nm);
        ms = nm;
        l *= corr;
        ok = ptx::mbar_wait(o_full, jp ^ 1u, abort_flag, status, ST_ATTN_TIMEOUT);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        o_waited = true;
#pragma unroll
        for (int c = 0; c < OH; c += 32) {
          float v[32];
          ptx::tmem_ld32(t_o + (uint32_t)c, v);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] *= corr;
          ptx::tmem_st32(t_o + (uint32_t)c, v);
        }
        ptx::tmem_st_wait();
        ptx::tc_fence_before_sync();
      }
      if (j > 0 && !o_waited) {
        // P_{j-1} is being read until O += P_{j-1} V_{j-1} completes
        ok = ptx::mbar_wait(o_full, jp ^ 1u, abort_flag, status, ST_ATTN_TIMEOUT);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      // pass 2: the 64 scores into registers; the MMA warp may then overwrite S with the next block's scores
      // (the partner's maximum was read above, so the partner, which waits for those scores, cannot have
      // reused the exchange slot before)
      float sv[64];
      ptx::tmem_ld32_at<0>(t_s, sv);
      ptx::tmem_ld32_at<32>(t_s + 32u, sv);
      ptx::tmem_ld_wait();
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(s_empty);
      if (diag) {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (u0 + i > t) sv[i] = -INFINITY;
      }
      // probabilities against the reference -> bf16 -> shared memory
      float2 rs2 = make_float2(0.f, 0.f);
      const float2 sl2v = make_float2(sl2, sl2), nmsv = make_float2(-ms, -ms);
#pragma unroll
      for (int c = 0; c < 64; c += 8) {  // 16-byte pieces of 8 keys
        uint4 raw;
        __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // packed fp32x2 arithmetic: two keys per instruction
          const float2 x = __ffma2_rn(make_float2(sv[c + 2 * i], sv[c + 2 * i + 1]), sl2v, nmsv);
          const float2 pr = make_float2(exp2f(x.x), exp2f(x.y));
          rs2 = __fadd2_rn(rs2, pr);
          hp[i] = __floats2bfloat162_rn(pr.x, pr.y);
        }
        *reinterpret_cast<uint4*>(p_row + (((c >> 3) ^ (row & 7)) << 4)) = raw;
      }
      l += rs2.x + rs2.y;
      ptx::fence_proxy_async();  // make the generic-proxy writes of P visible to the MMA's async proxy
      ptx::mbar_arrive(p_full);
    }
    if (ok) {
      ok = ptx::mbar_wait(o_full, (uint32_t)(n_blocks - 1) & 1u, abort_flag, status, ST_ATTN_TIMEOUT);
      ok = __all_sync(0xffffffffu, ok);
    }
    // the two halves of a row hold partial sums under the same running maximum
    if (ok) {
      // every MMA that reads Q has completed (the last s_full was consumed): its tile holds the partial sums
      float* lx = reinterpret_cast<float*>(smem + C::kQOff);
      lx[hf * 128 + row] = l;
      ptx::mbar_arrive(x_bar);
      ok = ptx::mbar_wait(x_bar, (uint32_t)n_blocks & 1u, abort_flag, status, ST_ATTN_TIMEOUT);
      if (ok) l += lx[(hf ^ 1) * 128 + row];
    }
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      ptx::tc_fence_after_sync();
      const float inv = 1.f / l;
      bf16* dst = o + ((size_t)b * seq + t) * ldo + h * HS + hf * OH;
#pragma unroll
      for (int c = 0; c < OH; c += 32) {
        float v[32];
        ptx::tmem_ld32(t_o + (uint32_t)c, v);
        ptx::tmem_ld_wait();
        if (t < seq) {
#pragma unroll
          for (int g = 0; g < 32; g += 8) {
            float w8[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) w8[i] = v[g + i] * inv;
            store8(dst + c + g, w8);
          }
        }
      }
      if (lse && hf == 0 && t < seq) lse[((size_t)b * n_heads + h) * seq + t] = ms * 0.6931471805599453f + __logf(l);
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
