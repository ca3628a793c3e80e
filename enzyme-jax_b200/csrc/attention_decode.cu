// Decode attention over the paged KV cache: one query row per (sequence, head)
// against `ctx` cached rows (test/llama.py:177-209 of the reference, where the
// cache holds pos rows plus the new one).
//
// Pass 1: CTA (split, head, sequence) of 4 warps walks its slice of the context
// 32 keys at a time per warp.  For q.k each lane owns one key and streams that
// key's row in 16-byte pieces; for p.v the lanes own head dimensions and the
// probabilities are broadcast by shuffle.  Each CTA leaves (acc[hs], max, sum)
// in scratch.  Pass 2 merges the splits.  HBM-bound: every cached byte is read
// exactly once per step.
#include <mutex>

#include "attention.cuh"

namespace b200 {

namespace {

constexpr int DW = 4;  // warps per CTA

template <typename T>
// Pages are head-major: [page][head][row][head_size], so the rows of one (sequence, head) are contiguous
// within a page (page_size * head_size elements) instead of head_size elements out of every d-wide row.
__device__ __forceinline__ const T* page_row(const T* base, const int32_t* table, int u, int page_size, int n_heads,
                                             int h, int hs) {
  const int page = table[u / page_size];
  return base + (((size_t)page * n_heads + h) * page_size + (u % page_size)) * hs;
}

template <typename T, int HS>
__global__ void __launch_bounds__(DW * 32)
    attn_decode_kernel(const T* __restrict__ q, const T* __restrict__ kpages, const T* __restrict__ vpages,
                       const int32_t* __restrict__ page_table, float* __restrict__ scratch, int ctx, int n_heads,
                       int ldq, int page_size, int max_pages, int d_local, int n_splits, float scale) {
  constexpr int DPL = (HS + 31) / 32;  // head dims per lane in the p.v phase
  __shared__ float qs[HS];
  __shared__ float part_acc[DW][HS];
  __shared__ float part_m[DW], part_l[DW];
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int32_t* table = page_table + (size_t)b * max_pages;
  for (int i = threadIdx.x; i < HS; i += blockDim.x) qs[i] = to_f32(q[(size_t)b * ldq + h * HS + i]) * scale;
  __syncthreads();

  const int per = (ctx + n_splits - 1) / n_splits;
  const int c0 = split * per, c1 = min(ctx, c0 + per);
  float m = -INFINITY, l = 0.f, acc[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) acc[i] = 0.f;

  for (int u0 = c0 + warp * 32; u0 < c1; u0 += DW * 32) {
    const int u = u0 + lane;
    float s = -INFINITY;
    if (u < c1) {
      const T* kr = page_row(kpages, table, u, page_size, n_heads, h, HS);
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < HS; e += 8) {
        float kv[8];
        load8(kr + e, kv);
#pragma unroll
        for (int i = 0; i < 8; ++i) d = fmaf(qs[e + i], kv[i], d);
      }
      s = d;
    }
    const float bm = warp_max(s);
    const float nm = fmaxf(m, bm);
    const float corr = __expf(m - nm);
    const float p = (u < c1) ? __expf(s - nm) : 0.f;
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] *= corr;
    const int n = min(32, c1 - u0);
    for (int j = 0; j < n; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const T* vr = page_row(vpages, table, u0 + j, page_size, n_heads, h, HS);
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const int e = lane + 32 * i;
        if (e < HS) acc[i] = fmaf(pj, to_f32(vr[e]), acc[i]);
      }
    }
    m = nm;
  }
  // merge the warps of this CTA
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int e = lane + 32 * i;
    if (e < HS) part_acc[warp][e] = acc[i];
  }
  if (lane == 0) { part_m[warp] = m; part_l[warp] = l; }
  __syncthreads();
  float gm = -INFINITY;
#pragma unroll
  for (int w = 0; w < DW; ++w) gm = fmaxf(gm, part_m[w]);
  float* out = scratch + (((size_t)b * n_heads + h) * n_splits + split) * (HS + 2);
  for (int e = threadIdx.x; e < HS; e += blockDim.x) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < DW; ++w)
      if (part_m[w] > -INFINITY) a += part_acc[w][e] * __expf(part_m[w] - gm);
    out[e] = a;
  }
  if (threadIdx.x == 0) {
    float gl = 0.f;
#pragma unroll
    for (int w = 0; w < DW; ++w)
      if (part_m[w] > -INFINITY) gl += part_l[w] * __expf(part_m[w] - gm);
    out[HS] = gm;
    out[HS + 1] = gl;
  }
}

// bf16 fast path.  A key or value row of one head is HS*2 bytes; LPK = HS/8
// lanes each fetch 16 bytes of it, so one warp-wide load brings in 32/LPK whole
// rows, fully coalesced.  Every lane keeps G such loads of K and of V in flight.
// The dot product is finished with log2(LPK) shuffles; each group of LPK lanes
// runs its own online softmax over the keys it sees and the groups, warps and
// (when the context is split) CTAs are merged at the end.
constexpr int VW = 8;  // warps per CTA
constexpr int VG = 4;  // loads in flight per lane and operand

__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

template <int HS>
__global__ void __launch_bounds__(VW * 32)
    attn_decode_vec_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kpages, const bf16* __restrict__ vpages,
                           const int32_t* __restrict__ page_table, float* __restrict__ scratch, bf16* __restrict__ o,
                           int ctx, int n_heads, int ldq, int ldo, int page_size, int max_pages, int d_local,
                           int n_splits, float scale) {
  constexpr int LPK = HS / 8;
  constexpr int KPW = 32 / LPK;
  __shared__ float s_acc[VW][HS];
  __shared__ float s_m[VW], s_l[VW];
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPK, li = lane % LPK;
  const int32_t* table = page_table + (size_t)b * max_pages;
  pdl_launch_dependents();
  pdl_wait();  // q and this step's K/V row come from the kernels before
  float qf[8];
  load8(q + (size_t)b * ldq + h * HS + li * 8, qf);
#pragma unroll
  for (int i = 0; i < 8; ++i) qf[i] *= scale;

  const int per = (ctx + n_splits - 1) / n_splits;
  const int c0 = split * per, c1 = min(ctx, c0 + per);
  float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;

  for (int u0 = c0 + warp * (VG * KPW); u0 < c1; u0 += VW * VG * KPW) {
    uint4 kr[VG], vr[VG];
    bool live[VG];
#pragma unroll
    for (int g = 0; g < VG; ++g) {
      const int u = u0 + g * KPW + sub;
      live[g] = u < c1;
      kr[g] = make_uint4(0u, 0u, 0u, 0u);
      vr[g] = make_uint4(0u, 0u, 0u, 0u);
      if (live[g]) {
        const int page = table[u / page_size];
        const size_t off = (((size_t)page * n_heads + h) * page_size + (u % page_size)) * HS + li * 8;
        kr[g] = *reinterpret_cast<const uint4*>(kpages + off);
        vr[g] = *reinterpret_cast<const uint4*>(vpages + off);
      }
    }
    float s[VG];
    float bm = -INFINITY;
#pragma unroll
    for (int g = 0; g < VG; ++g) {
      float kf[8];
      unpack8(kr[g], kf);
      float2 d2 = make_float2(0.f, 0.f);  // packed fp32x2 FMAs: two head dimensions per instruction
#pragma unroll
      for (int i = 0; i < 8; i += 2)
        d2 = __ffma2_rn(make_float2(qf[i], qf[i + 1]), make_float2(kf[i], kf[i + 1]), d2);
      float d = d2.x + d2.y;
#pragma unroll
      for (int off = LPK / 2; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
      s[g] = live[g] ? d : -INFINITY;
      bm = fmaxf(bm, s[g]);
    }
    if (bm > -INFINITY) {  // uniform within a group of LPK lanes
      const float nm = fmaxf(m, bm);
      const float corr = __expf(m - nm);
      l *= corr;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] *= corr;
#pragma unroll
      for (int g = 0; g < VG; ++g) {
        const float p = __expf(s[g] - nm);  // exp(-inf) = 0 for keys past the end
        l += p;
        float vf[8];
        unpack8(vr[g], vf);
        const float2 p2 = make_float2(p, p);
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          const float2 r = __ffma2_rn(p2, make_float2(vf[i], vf[i + 1]), make_float2(acc[i], acc[i + 1]));
          acc[i] = r.x;
          acc[i + 1] = r.y;
        }
      }
      m = nm;
    }
  }
  // merge the key groups of the warp (they hold the same head dimensions)
#pragma unroll
  for (int off = LPK; off < 32; off <<= 1) {
    const float mo = __shfl_xor_sync(0xffffffffu, m, off);
    const float lo = __shfl_xor_sync(0xffffffffu, l, off);
    const float nm = fmaxf(m, mo);
    const float a = m > -INFINITY ? __expf(m - nm) : 0.f;
    const float c = mo > -INFINITY ? __expf(mo - nm) : 0.f;
    l = l * a + lo * c;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float ao = __shfl_xor_sync(0xffffffffu, acc[i], off);
      acc[i] = acc[i] * a + ao * c;
    }
    m = nm;
  }
  if (sub == 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) s_acc[warp][li * 8 + i] = acc[i];
  }
  if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
  __syncthreads();
  float gm = -INFINITY;
#pragma unroll
  for (int w = 0; w < VW; ++w) gm = fmaxf(gm, s_m[w]);
  float gl = 0.f;
#pragma unroll
  for (int w = 0; w < VW; ++w)
    if (s_m[w] > -INFINITY) gl += s_l[w] * __expf(s_m[w] - gm);
  float* part = scratch + (((size_t)b * n_heads + h) * n_splits + split) * (HS + 2);
  for (int e = threadIdx.x; e < HS; e += blockDim.x) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < VW; ++w)
      if (s_m[w] > -INFINITY) a += s_acc[w][e] * __expf(s_m[w] - gm);
    if (n_splits == 1) o[(size_t)b * ldo + h * HS + e] = __float2bfloat16_rn(a / gl);
    else part[e] = a;
  }
  if (n_splits > 1 && threadIdx.x == 0) { part[HS] = gm; part[HS + 1] = gl; }
}

template <typename T, int HS>
__global__ void attn_decode_combine_kernel(const float* __restrict__ scratch, T* __restrict__ o, int n_heads, int ldo,
                                           int n_splits) {
  const int h = blockIdx.x, b = blockIdx.y;
  const float* base = scratch + ((size_t)b * n_heads + h) * n_splits * (HS + 2);
  pdl_launch_dependents();
  pdl_wait();
  float gm = -INFINITY;
  for (int s = 0; s < n_splits; ++s) gm = fmaxf(gm, base[(size_t)s * (HS + 2) + HS]);
  float gl = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = base[(size_t)s * (HS + 2) + HS];
    if (ms > -INFINITY) gl += base[(size_t)s * (HS + 2) + HS + 1] * __expf(ms - gm);
  }
  for (int e = threadIdx.x; e < HS; e += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = base[(size_t)s * (HS + 2) + HS];
      if (ms > -INFINITY) a += base[(size_t)s * (HS + 2) + e] * __expf(ms - gm);
    }
    o[(size_t)b * ldo + h * HS + e] = from_f32<T>(a / gl);
  }
}

template <typename T, int HS>
int32_t launch_hs(const AttnDecodeArgs& a, cudaStream_t stream) {
  const size_t page_elems = (size_t)a.n_pages * a.page_size * a.d_local;
  const T* kp = reinterpret_cast<const T*>(a.kv_pages);
  const T* vp = kp + page_elems;
  dim3 grid(a.n_splits, a.n_heads, a.batch);
  if constexpr (sizeof(T) == 2 && (HS == 64 || HS == 128)) {
    B200_CUDA_OK(launch_pdl(attn_decode_vec_kernel<HS>, grid, dim3(VW * 32), 0, stream, (const bf16*)a.q, (const bf16*)kp,
                            (const bf16*)vp, a.page_table, a.scratch, (bf16*)a.o, a.ctx, a.n_heads, a.ldq, a.ldo,
                            a.page_size, a.max_pages, a.d_local, a.n_splits, 1.f / sqrtf((float)HS)));
    B200_LAUNCH_OK("attn_decode_vec_kernel");
    if (a.n_splits == 1) return B200_OK;  // the kernel wrote the output itself
    dim3 grid2v(a.n_heads, a.batch);
    B200_CUDA_OK(launch_pdl(attn_decode_combine_kernel<T, HS>, grid2v, dim3(HS), 0, stream, (const float*)a.scratch, (T*)a.o,
                            a.n_heads, a.ldo, a.n_splits));
    B200_LAUNCH_OK("attn_decode_combine_kernel");
    return B200_OK;
  }
  attn_decode_kernel<T, HS><<<grid, DW * 32, 0, stream>>>((const T*)a.q, kp, vp, a.page_table, a.scratch, a.ctx,
                                                          a.n_heads, a.ldq, a.page_size, a.max_pages, a.d_local,
                                                          a.n_splits, 1.f / sqrtf((float)HS));
  B200_LAUNCH_OK("attn_decode_kernel");
  dim3 grid2(a.n_heads, a.batch);
  attn_decode_combine_kernel<T, HS><<<grid2, HS < 32 ? 32 : HS, 0, stream>>>(a.scratch, (T*)a.o, a.n_heads, a.ldo,
                                                                             a.n_splits);
  B200_LAUNCH_OK("attn_decode_combine_kernel");
  return B200_OK;
}

template <typename T>
int32_t launch_t(const AttnDecodeArgs& a, cudaStream_t stream) {
  switch (a.head_size) {
    case 16: return launch_hs<T, 16>(a, stream);
    case 32: return launch_hs<T, 32>(a, stream);
    case 48: return launch_hs<T, 48>(a, stream);
    case 64: return launch_hs<T, 64>(a, stream);
    case 128: return launch_hs<T, 128>(a, stream);
  }
  return fail(B200_ERR_BAD_SHAPE, "decode attention: head size %d is not one of 16/32/48/64/128", a.head_size);
}

}  // namespace

size_t decode_scratch_floats(int batch, int n_heads, int head_size, int n_splits) {
  return (size_t)batch * n_heads * n_splits * (head_size + 2);
}

int decode_pick_splits(int batch, int n_heads, int ctx) {
  const int want = 8 * sm_count();  // the bf16 kernel wants several 8-warp CTAs per SM to cover HBM latency
  int s = cdiv(want, batch * n_heads);
  const int max_s = ctx / 128 > 0 ? ctx / 128 : 1;
  if (s > max_s) s = max_s;
  if (s < 1) s = 1;
  if (s > 64) s = 64;
  return s;
}

int32_t launch_attn_decode(const AttnDecodeArgs& a, cudaStream_t stream) {
  if (a.batch <= 0 || a.ctx <= 0 || a.n_heads <= 0 || a.n_splits <= 0)
    return fail(B200_ERR_BAD_SHAPE, "decode attention: empty problem");
  if (a.d_local % 8 || a.head_size % 8) return fail(B200_ERR_BAD_SHAPE, "decode attention: row width must be a multiple of 8");
  if (cdiv(a.ctx, a.page_size) > a.max_pages)
    return fail(B200_ERR_BAD_SHAPE, "decode attention: context %d needs more than %d pages of %d rows", a.ctx,
                a.max_pages, a.page_size);
  if (!a.scratch) return fail(B200_ERR_INVALID_ARG, "decode attention: scratch is null");
  const double es = a.dtype == B200_BF16 ? 2.0 : 4.0;
  ProfScope prof(PROF_ATTN_DECODE, 2.0 * a.batch * (double)a.ctx * a.n_heads * a.head_size * es, stream);
  if (a.dtype == B200_F32) return launch_t<float>(a, stream);
  if (a.dtype == B200_BF16) return launch_t<bf16>(a, stream);
  return fail(B200_ERR_BAD_DTYPE, "decode attention: unsupported dtype %d", a.dtype);
}

}  // namespace b200

using namespace b200;

extern "C" {

int32_t b200_attention_decode_scratch_bytes(int32_t batch, int32_t n_heads, int32_t head_size, int32_t ctx,
                                            size_t* bytes) {
  if (!bytes) return fail(B200_ERR_INVALID_ARG, "bytes is null");
  if (batch <= 0 || n_heads <= 0 || head_size <= 0 || ctx <= 0) return fail(B200_ERR_BAD_SHAPE, "sizes must be positive");
  *bytes = decode_scratch_floats(batch, n_heads, head_size, decode_pick_splits(batch, n_heads, ctx)) * sizeof(float);
  return B200_OK;
}

int32_t b200_attention_decode(const void* q, const void* kv_pages, const int32_t* page_table, void* o, void* scratch,
                              size_t scratch_bytes, int32_t batch, int32_t ctx, int32_t n_heads, int32_t head_size,
                              int32_t ldq, int32_t ldo, int32_t n_pages, int32_t page_size, int32_t max_pages,
                              int32_t dtype, b200_stream_t stream) {
  if (!q || !kv_pages || !page_table || !o || !scratch) return fail(B200_ERR_INVALID_ARG, "null operand");
  if (!aligned16(q) || !aligned16(kv_pages) || !aligned16(o) || !aligned16(scratch))
    return fail(B200_ERR_MISALIGNED, "operands must be 16-byte aligned");
  if (batch <= 0 || ctx <= 0 || n_heads <= 0 || n_pages <= 0 || page_size <= 0 || max_pages <= 0)
    return fail(B200_ERR_BAD_SHAPE, "sizes must be positive");
  AttnDecodeArgs a;
  a.q = q; a.kv_pages = kv_pages; a.page_table = page_table; a.o = o; a.scratch = reinterpret_cast<float*>(scratch);
  a.batch = batch; a.ctx = ctx; a.n_heads = n_heads; a.head_size = head_size; a.ldq = ldq; a.ldo = ldo;
  a.n_pages = n_pages; a.page_size = page_size; a.max_pages = max_pages; a.d_local = n_heads * head_size;
  a.dtype = dtype; a.n_splits = decode_pick_splits(batch, n_heads, ctx);
  if (decode_scratch_floats(batch, n_heads, head_size, a.n_splits) * sizeof(float) > scratch_bytes)
    return fail(B200_ERR_WORKSPACE, "decode attention scratch too small: %zu bytes given", scratch_bytes);
  return launch_attn_decode(a, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"

// ---- decode attention without any allocation --------------------------------------
//
// Some callers may not allocate device memory at the point where they need
// decode attention: code that runs between the capture of other work, a
// serving loop whose memory pool is fixed at start-up, or a host runtime that
// hands this library only the input and output buffers of a custom call and
// has no way to pass (or size) an extra scratch operand.  For them the split
// partials live in a fixed array inside the library image instead of a
// caller buffer.  Every GPU that loads the library holds these 4 MiB until the
// process exits.
namespace {

constexpr size_t kStaticScratchFloats = size_t(1) << 20;  // 4 MiB
static __device__ __align__(256) float g_static_decode_scratch[kStaticScratchFloats];

std::mutex g_static_mu;
float* g_static_ptr[64] = {nullptr};

// Device address of the array on the current device.  In host code the array's
// name is only a handle, so the address is asked for once per device.
int32_t static_scratch(float** out) {
  int dev = -1;
  B200_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(B200_ERR_INVALID_ARG, "device ordinal %d is out of range", dev);
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (!g_static_ptr[dev]) {
    float* p = nullptr;
    B200_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_decode_scratch));
    if (!p) return fail(B200_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return B200_OK;
}

}  // namespace

extern "C" int32_t b200_attention_decode_static(const void* q, const void* kv_pages, const int32_t* page_table,
                                                void* o, int32_t batch, int32_t ctx, int32_t n_heads,
                                                int32_t head_size, int32_t ldq, int32_t ldo, int32_t n_pages,
                                                int32_t page_size, int32_t max_pages, int32_t dtype,
                                                b200_stream_t stream) {
  if (!q || !kv_pages || !page_table || !o) return fail(B200_ERR_INVALID_ARG, "null operand");
  if (!aligned16(q) || !aligned16(kv_pages) || !aligned16(o))
    return fail(B200_ERR_MISALIGNED, "operands must be 16-byte aligned");
  if (batch <= 0 || ctx <= 0 || n_heads <= 0 || head_size <= 0 || n_pages <= 0 || page_size <= 0 || max_pages <= 0)
    return fail(B200_ERR_BAD_SHAPE, "sizes must be positive");
  AttnDecodeArgs a;
  a.n_splits = decode_pick_splits(batch, n_heads, ctx);
  const size_t need = decode_scratch_floats(batch, n_heads, head_size, a.n_splits);
  if (need > kStaticScratchFloats)
    return fail(B200_ERR_WORKSPACE,
                "decode attention needs %zu scratch bytes for batch=%d heads=%d head_size=%d (%d splits); the built-in "
                "scratch holds %zu bytes: use b200_attention_decode with a caller buffer",
                need * sizeof(float), batch, n_heads, head_size, a.n_splits, kStaticScratchFloats * sizeof(float));
  float* scratch = nullptr;
  B200_TRY(static_scratch(&scratch));
  a.q = q; a.kv_pages = kv_pages; a.page_table = page_table; a.o = o; a.scratch = scratch;
  a.batch = batch; a.ctx = ctx; a.n_heads = n_heads; a.head_size = head_size; a.ldq = ldq; a.ldo = ldo;
  a.n_pages = n_pages; a.page_size = page_size; a.max_pages = max_pages; a.d_local = n_heads * head_size;
  a.dtype = dtype;
  if (a.d_local % 8 || a.head_size % 8) return fail(B200_ERR_BAD_SHAPE, "row width must be a multiple of 8");
  if (cdiv(a.ctx, a.page_size) > a.max_pages)
    return fail(B200_ERR_BAD_SHAPE, "context %d needs more than %d pages of %d rows", a.ctx, a.max_pages, a.page_size);
  // Nothing in the array has to start at zero: the first kernel writes every
  // (sequence, head, split) slot, empty splits included, before the second reads it.
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == B200_F32) return launch_t<float>(a, s);
  if (dtype == B200_BF16) return launch_t<bf16>(a, s);
  return fail(B200_ERR_BAD_DTYPE, "unsupported dtype %d", dtype);
}
