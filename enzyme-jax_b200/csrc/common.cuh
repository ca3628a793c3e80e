// Shared helpers for the llama path kernels: status/error plumbing, numeric
// type traits, vector loads, warp reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "../../include/b200_llama.h"

namespace b200 {

// ---- host-side error plumbing --------------------------------------------
void set_error(const char* fmt, ...);
int32_t fail(int32_t code, const char* fmt, ...);

#define B200_CUDA_OK(expr)                                                              \
  do {                                                                                  \
    cudaError_t _e = (expr);                                                            \
    if (_e != cudaSuccess)                                                              \
      return ::b200::fail(B200_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                \
                          cudaGetErrorString(_e), __FILE__, __LINE__);                  \
  } while (0)

#define B200_LAUNCH_OK(name)                                                            \
  do {                                                                                  \
    ::b200::count_launch();                                                             \
    cudaError_t _e = cudaGetLastError();                                                \
    if (_e != cudaSuccess)                                                              \
      return ::b200::fail(B200_ERR_CUDA, "launch of %s failed: %s", name,               \
                          cudaGetErrorString(_e));                                      \
  } while (0)

#define B200_TRY(expr)                  \
  do {                                  \
    int32_t _s = (expr);                \
    if (_s != B200_OK) return _s;       \
  } while (0)

void count_launch();

// Event-pair profiling of kernel classes (off unless enabled through the ABI).
enum ProfClass : int { PROF_GEMM_TC = 0, PROF_GEMM_SIMT = 1, PROF_ATTN_FWD = 2, PROF_ATTN_BWD = 3, PROF_ATTN_DECODE = 4, PROF_COMM = 5, PROF_GEMM_PAIR = 6, PROF_NUM = 7 };
struct ProfScope {
  int slot = -1;
  cudaStream_t stream;
  ProfScope(int cls, double work, cudaStream_t s);
  ~ProfScope();
};

// Device word that kernels with bounded waits OR their failure code into.
uint32_t* device_status_word();  // lazily allocated per device, never on a hot path

// ---- programmatic dependent launch -------------------------------------------
// Kernels of the forward chain are launched so that the next kernel's CTAs may start (set up barriers,
// allocate tensor memory, prefetch descriptors) while the last CTAs of the previous kernel drain.  Such a
// kernel calls pdl_launch_dependents() at its start and pdl_wait() before it first touches global memory
// that an earlier kernel wrote or still reads; pdl_wait returns once every earlier kernel has completed.
// Both are no-ops in a kernel launched the ordinary way.  B200_PDL=0 turns the launch attribute off.
bool pdl_enabled();
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// One-time set-up per device (kernel attributes, occupancy queries are per device, and a process may
// drive several).  run(f) calls f(value) once for the current device, under a lock, and later returns
// the value it left; concurrent callers on the same device wait for the first to finish.
struct PerDeviceOnce {
  std::mutex mu;
  bool done[64] = {};
  int value[64] = {};
  template <typename F> int32_t run(F&& f, int* out = nullptr) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
      return ::b200::fail(B200_ERR_CUDA, "no current CUDA device");
    std::lock_guard<std::mutex> lk(mu);
    if (!done[dev]) {
      const int32_t st = f(value[dev]);
      if (st != B200_OK) return st;
      done[dev] = true;
    }
    if (out) *out = value[dev];
    return B200_OK;
  }
};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline int cdiv(int a, int b) { return (a + b - 1) / b; }
int sm_count();

// ---- numeric helpers -------------------------------------------------------
using bf16 = __nv_bfloat16;

template <typename T> struct DTypeOf;
template <> struct DTypeOf<float> { static constexpr int value = B200_F32; };
template <> struct DTypeOf<bf16> { static constexpr int value = B200_BF16; };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Loads 8 consecutive elements as fp32 (16 B for bf16, 32 B for fp32).
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p);
  float4 b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(bf16* p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// 32-byte (256-bit) global accesses of sm_100: one full sector per thread.
__device__ __forceinline__ void store32B(void* p, const uint32_t (&r)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(r[0]), "r"(r[1]), "r"(r[2]),
               "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void load32B(const void* p, uint32_t (&r)[8]) {
  asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "l"(p)
               : "memory");
}
__device__ __forceinline__ bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }

// 8 consecutive floats, as one 32-byte access when the address allows it
__device__ __forceinline__ void store8_wide(float* p, const float (&v)[8]) {
  if (aligned32(p)) {
    uint32_t r[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] = __float_as_uint(v[i]);
    store32B(p, r);
  } else {
    store8(p, v);
  }
}
__device__ __forceinline__ void load8_wide(const float* p, float (&v)[8]) {
  if (aligned32(p)) {
    uint32_t r[8];
    load32B(p, r);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
  } else {
    load8(p, v);
  }
}

// exp(x): the fast approximation in files built with fast math (B200_FAST_MATH, the bf16 tensor-core kernels), the accurate
// library function elsewhere (the fp32 configuration).
__device__ __forceinline__ float exp_by_build(float x) {
#ifdef B200_FAST_MATH
  return __expf(x);
#else
  return expf(x);
#endif
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum for blocks of up to 1024 threads; `red` is 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

}  // namespace b200
