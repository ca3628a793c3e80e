// Communication between the ranks of one node.
//
// (1) NCCL glue.  The library does not link NCCL: the symbols are resolved at
//     first use from the libnccl already loaded into the process (the one
//     PyTorch ships) or from the system library, so single-GPU users need no
//     NCCL at all.
// (2) A peer-memory all-reduce fused with the residual add for the tensor
//     parallel projections: every rank keeps its partial product in a buffer the
//     other ranks map through CUDA IPC; one kernel reduces this rank's slice by
//     plain loads over NVLink and stores the sum into every rank's buffer, a
//     second kernel adds the complete sum to the residual stream.  No NVLink
//     multicast object, no TMA: plain ld/st with system-scope flags.  Every wait
//     on a peer is bounded.
#include <dlfcn.h>
#include <string.h>

#include <mutex>

#include "plan.cuh"

namespace b200 {

namespace {

typedef struct { char internal[128]; } NcclUniqueId;
typedef void* NcclComm;
typedef int (*GetUniqueIdFn)(NcclUniqueId*);
typedef int (*CommInitRankFn)(NcclComm*, int, NcclUniqueId, int);
typedef int (*CommDestroyFn)(NcclComm);
typedef int (*AllReduceFn)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t);
typedef int (*AllGatherFn)(const void*, void*, size_t, int, NcclComm, cudaStream_t);
typedef const char* (*GetErrorStringFn)(int);

struct NcclApi {
  GetUniqueIdFn get_unique_id = nullptr;
  CommInitRankFn comm_init_rank = nullptr;
  CommDestroyFn comm_destroy = nullptr;
  AllReduceFn all_reduce = nullptr;
  AllGatherFn all_gather = nullptr;
  GetErrorStringFn error_string = nullptr;
  bool ok = false;
};

// ncclDataType_t / ncclRedOp_t values of the public nccl.h
constexpr int kNcclChar = 0, kNcclFloat32 = 7, kNcclBfloat16 = 9, kNcclSum = 0;

NcclApi& api() {
  static NcclApi a;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen(nullptr, RTLD_NOW);  // already loaded by the host process?
    if (!h || !dlsym(h, "ncclAllReduce")) {
      const char* names[] = {"libnccl.so.2", "libnccl.so"};
      for (const char* n : names) {
        h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
      }
    }
    if (!h) return;
    a.get_unique_id = (GetUniqueIdFn)dlsym(h, "ncclGetUniqueId");
    a.comm_init_rank = (CommInitRankFn)dlsym(h, "ncclCommInitRank");
    a.comm_destroy = (CommDestroyFn)dlsym(h, "ncclCommDestroy");
    a.all_reduce = (AllReduceFn)dlsym(h, "ncclAllReduce");
    a.all_gather = (AllGatherFn)dlsym(h, "ncclAllGather");
    a.error_string = (GetErrorStringFn)dlsym(h, "ncclGetErrorString");
    a.ok = a.get_unique_id && a.comm_init_rank && a.comm_destroy && a.all_reduce && a.all_gather && a.error_string;
  });
  return a;
}

int32_t nccl_fail(const char* what, int rc) {
  return fail(B200_ERR_NCCL, "%s failed: %s", what, api().error_string ? api().error_string(rc) : "?");
}

constexpr int kMaxPeers = 8;
constexpr int kFlagWords = 64;  // [0..7] "partial ready" per source rank, [8..15] "slice written" per source rank, [32] CTA counter, [40..47] epoch ring

struct PeerMem {
  bool on = false;
  size_t bytes = 0;
  void* buf[kMaxPeers] = {};       // buf[r]: rank r's exchange buffer as seen from this process
  uint32_t* flags[kMaxPeers] = {}; // flags[r]: rank r's flag words
  uint32_t epoch = 0;
  bool external = false;           // the memory belongs to the caller (b200_comm_attach_memory): never freed here
  uint8_t* mc = nullptr;           // multicast address of the same buffers (NVLink SHARP), or null
};

}  // namespace

// What the opaque communicator handle of the C ABI points to.
struct Comm {
  NcclComm nccl = nullptr;
  int rank = 0, world = 1;
  PeerMem pm;
  long long wait_budget = 4000000000LL;  // SM clocks a kernel waits for its peers before it gives up (B200_PEER_WAIT_MCYCLES)
  // Copy-engine delivery of this rank's normed rows (comm_peer_reduce_norm_at with bands): a stream of its own, an
  // event that follows the exchange kernel and one that follows the last copy of the latest exchange.
  cudaStream_t ce_stream = nullptr;
  cudaEvent_t ev_rows = nullptr, ev_sent = nullptr;
  bool sent_pending = false;
};

namespace {

struct IpcBlob {
  cudaIpcMemHandle_t buf, flags;
  int valid;
};

// Allocates this rank's exchange buffer and flag words and maps every peer's
// through CUDA IPC.  The handles travel by an NCCL all-gather and the ranks
// agree on the outcome with an NCCL all-reduce, so that either all of them use
// the peer path or none does.  Every rank takes part in both collectives
// whatever happened locally.  Failure only disables the peer path.
void setup_peer_memory(Comm* c) {
  if (c->world < 2 || c->world > kMaxPeers || env_int("B200_P2P", 1) == 0) return;
  NcclApi& a = api();
  PeerMem& pm = c->pm;
  pm.bytes = (size_t)env_int("B200_P2P_MB", 136) << 20;
  void* lbuf = nullptr;
  uint32_t* lflags = nullptr;
  uint8_t* dscratch = nullptr;  // [world + 1] blobs, then one float for the agreement
  IpcBlob mine, all[kMaxPeers];
  memset(&mine, 0, sizeof(mine));
  const size_t blob_bytes = sizeof(IpcBlob) * (kMaxPeers + 1);
  if (cudaMalloc(&dscratch, blob_bytes + 256) != cudaSuccess) {  // without it this rank cannot even take part
    cudaGetLastError();
    return;
  }
  bool ok = cudaMalloc(&lbuf, pm.bytes) == cudaSuccess && cudaMalloc(&lflags, kFlagWords * 4) == cudaSuccess &&
            cudaMemset(lflags, 0, kFlagWords * 4) == cudaSuccess &&
            cudaIpcGetMemHandle(&mine.buf, lbuf) == cudaSuccess &&
            cudaIpcGetMemHandle(&mine.flags, lflags) == cudaSuccess;
  mine.valid = ok ? 1 : 0;
  IpcBlob* dblobs = reinterpret_cast<IpcBlob*>(dscratch);
  bool gathered = cudaMemcpy(dblobs + kMaxPeers, &mine, sizeof(mine), cudaMemcpyHostToDevice) == cudaSuccess &&
                  a.all_gather(dblobs + kMaxPeers, dblobs, sizeof(IpcBlob), kNcclChar, c->nccl, 0) == 0 &&
                  cudaStreamSynchronize(0) == cudaSuccess &&
                  cudaMemcpy(all, dblobs, sizeof(IpcBlob) * c->world, cudaMemcpyDeviceToHost) == cudaSuccess;
  ok = ok && gathered;
  for (int r = 0; ok && r < c->world; ++r) ok = all[r].valid == 1;
  for (int r = 0; ok && r < c->world; ++r) {
    if (r == c->rank) {
      pm.buf[r] = lbuf;
      pm.flags[r] = lflags;
    } else {
      void* pb = nullptr;
      void* pf = nullptr;
      ok = cudaIpcOpenMemHandle(&pb, all[r].buf, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess &&
           cudaIpcOpenMemHandle(&pf, all[r].flags, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
      pm.buf[r] = pb;
      pm.flags[r] = reinterpret_cast<uint32_t*>(pf);
    }
  }
  // agreement: the sum of the ranks' verdicts must equal the world size
  float verdict = ok ? 1.f : 0.f, total = 0.f;
  float* dv = reinterpret_cast<float*>(dscratch + blob_bytes);
  const bool agreed = cudaMemcpy(dv, &verdict, 4, cudaMemcpyHostToDevice) == cudaSuccess &&
                      a.all_reduce(dv, dv, 1, kNcclFloat32, kNcclSum, c->nccl, 0) == 0 &&
                      cudaStreamSynchronize(0) == cudaSuccess &&
                      cudaMemcpy(&total, dv, 4, cudaMemcpyDeviceToHost) == cudaSuccess;
  ok = ok && agreed && total == (float)c->world;
  cudaFree(dscratch);
  if (!ok) {
    cudaGetLastError();
    for (int r = 0; r < c->world; ++r) {
      if (r == c->rank) continue;
      if (pm.buf[r]) cudaIpcCloseMemHandle(pm.buf[r]);
      if (pm.flags[r]) cudaIpcCloseMemHandle(pm.flags[r]);
    }
    if (lbuf) cudaFree(lbuf);
    if (lflags) cudaFree(lflags);
    pm = PeerMem();
    return;
  }
  pm.on = true;
}

void free_peer_memory(Comm* c) {
  PeerMem& pm = c->pm;
  if (!pm.on) return;
  if (pm.external) {
    pm = PeerMem();
    return;
  }
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    cudaIpcCloseMemHandle(pm.buf[r]);
    cudaIpcCloseMemHandle(pm.flags[r]);
  }
  cudaFree(pm.buf[c->rank]);
  cudaFree(pm.flags[c->rank]);
  pm = PeerMem();
}

}  // namespace

int32_t comm_allreduce(void* comm, void* data, size_t count, int dtype, cudaStream_t stream) {
  if (!comm) return fail(B200_ERR_INVALID_ARG, "communicator is null");
  Comm* c = reinterpret_cast<Comm*>(comm);
  NcclApi& a = api();
  if (!a.ok) return fail(B200_ERR_NCCL, "NCCL is not available in this process");
  const int nt = dtype == B200_BF16 ? kNcclBfloat16 : kNcclFloat32;
  ProfScope prof(PROF_COMM, (double)count * (dtype == B200_BF16 ? 2 : 4), stream);
  const int rc = a.all_reduce(data, data, count, nt, kNcclSum, c->nccl, stream);
  if (rc != 0) return nccl_fail("ncclAllReduce", rc);
  return B200_OK;
}

}  // namespace b200

// ---- peer-memory all-reduce + residual add --------------------------------------
namespace b200 {

namespace {

enum : uint32_t { ST_PEER_TIMEOUT = 1u << 12 };
constexpr int kReadyBase = 0, kDoneBase = 8, kCounter = 32;
constexpr int kEpochRing = 40;  // [40..47]: the epochs of the latest exchanges, sources of the copy-engine flag copies
constexpr long long kPeerWaitCycles = 4000000000LL;

__device__ __forceinline__ void flag_store_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t flag_load_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// 16 bytes from memory that another GPU owns or may have written: skip the L1, which is not coherent with peers
// (ordering comes from the acquire on the flag that precedes these loads)
__device__ __forceinline__ uint4 load16_sys(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

struct PeerPtrs {
  void* buf[kMaxPeers];
  uint32_t* flags[kMaxPeers];
};

// Thread 0 of the CTA waits until every rank's flag word `base + r` in this
// rank's flag array has reached `epoch`, for at most `budget` SM clocks in all
// (the default, kPeerWaitCycles, is about two seconds).  Returns false (for the
// whole CTA) when the wait ran out; the status word then carries ST_PEER_TIMEOUT.
__device__ int g_poll_ns = 100;  // pause between two looks at a peer flag (B200_PEER_POLL_NS; 0 = none)

__device__ __forceinline__ bool wait_all_peers(const uint32_t* my_flags, int base, int world, uint32_t epoch,
                                               uint32_t* status, long long budget) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    int ok = 1;
    const long long t0 = clock64();
    const int pause = g_poll_ns;
    for (int r = 0; r < world && ok; ++r) {
      while ((int32_t)(flag_load_sys(my_flags + base + r) - epoch) < 0) {
        if (pause > 0) __nanosleep(pause);  // the waiting CTA may share its SM with a compute kernel: leave it the issue slots
        if (clock64() - t0 > budget) {
          ok = 0;
          atomicOr(status, ST_PEER_TIMEOUT);
          break;
        }
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

__device__ __forceinline__ void accum8(const uint4& raw, float (&acc)[8], bf16) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}
__device__ __forceinline__ void accum8(const uint4& raw, float (&acc)[8], float) {
  acc[0] += __uint_as_float(raw.x); acc[1] += __uint_as_float(raw.y);
  acc[2] += __uint_as_float(raw.z); acc[3] += __uint_as_float(raw.w);
}

// Pass 1: tell the peers this rank's partial is complete, wait for theirs, then
// sum this rank's slice over all ranks (rank order, fp32) and store the result
// into every rank's buffer.  The last CTA to finish tells the peers.
template <typename T>
__global__ void __launch_bounds__(512) peer_reduce_kernel(PeerPtrs pp, int rank, int world, size_t n_vec16,
                                                          uint32_t epoch, uint32_t* status, long long budget) {
  uint32_t* my_flags = pp.flags[rank];
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    flag_store_sys(pp.flags[threadIdx.x] + kReadyBase + rank, epoch);
  }
  const bool ok = wait_all_peers(my_flags, kReadyBase, world, epoch, status, budget);
  if (ok) {
    const size_t per = (n_vec16 + world - 1) / world;
    const size_t v0 = (size_t)rank * per, v1 = min(n_vec16, v0 + per);
    for (size_t i = v0 + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < v1; i += (size_t)gridDim.x * blockDim.x) {
      uint4 raw[kMaxPeers];
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r)
        if (r < world) raw[r] = load16_sys(reinterpret_cast<const uint4*>(pp.buf[r]) + i);
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r)
        if (r < world) accum8(raw[r], acc, T());
      uint4 out;
      if (sizeof(T) == 2) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
        for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
      } else {
        out = make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]));
      }
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r)
        if (r < world) reinterpret_cast<uint4*>(pp.buf[r])[i] = out;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t done = atomicAdd(my_flags + kCounter, 1u);
    if (done == gridDim.x - 1) {
      my_flags[kCounter] = 0u;
      __threadfence_system();
      for (int r = 0; r < world; ++r) flag_store_sys(pp.flags[r] + kDoneBase + rank, epoch);
    }
  }
}

// Pass 2: once every rank has written its slice, out = resid + sum.
template <typename T>
__global__ void __launch_bounds__(512) peer_add_kernel(PeerPtrs pp, int rank, int world, size_t n_vec16,
                                                       uint32_t epoch, const float* __restrict__ resid,
                                                       float* __restrict__ out, uint32_t* status, long long budget) {
  if (!wait_all_peers(pp.flags[rank], kDoneBase, world, epoch, status, budget)) return;
  constexpr int E = 16 / sizeof(T);  // elements per 16 bytes
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_vec16; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 raw = load16_sys(reinterpret_cast<const uint4*>(pp.buf[rank]) + i);
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    accum8(raw, s, T());
    const float4 a = *reinterpret_cast<const float4*>(resid + i * E);
    *reinterpret_cast<float4*>(out + i * E) = make_float4(a.x + s[0], a.y + s[1], a.z + s[2], a.w + s[3]);
    if (E == 8) {
      const float4 b = *reinterpret_cast<const float4*>(resid + i * E + 4);
      *reinterpret_cast<float4*>(out + i * E + 4) = make_float4(b.x + s[4], b.y + s[5], b.z + s[6], b.w + s[7]);
    }
  }
}

// Small messages (decode): one pass.  Every rank reads all ranks' partials and
// adds the sum to its residual rows itself; one flag round instead of two.  The
// exchange buffer is used in halves that alternate from call to call, so a
// peer may still be reading the previous half while this rank fills the next.
template <typename T>
__global__ void __launch_bounds__(512) peer_oneshot_kernel(PeerPtrs pp, int rank, int world, size_t n_vec16,
                                                           size_t half_off, uint32_t epoch,
                                                           const float* __restrict__ resid, float* __restrict__ out,
                                                           uint32_t* status, long long budget) {
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    flag_store_sys(pp.flags[threadIdx.x] + kReadyBase + rank, epoch);
  }
  if (!wait_all_peers(pp.flags[rank], kReadyBase, world, epoch, status, budget)) return;
  constexpr int E = 16 / sizeof(T);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_vec16; i += (size_t)gridDim.x * blockDim.x) {
    uint4 raw[kMaxPeers];
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < world) raw[r] = load16_sys(reinterpret_cast<const uint8_t*>(pp.buf[r]) + half_off + i * 16);
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < world) accum8(raw[r], s, T());
    const float4 a = *reinterpret_cast<const float4*>(resid + i * E);
    *reinterpret_cast<float4*>(out + i * E) = make_float4(a.x + s[0], a.y + s[1], a.z + s[2], a.w + s[3]);
    if (E == 8) {
      const float4 b = *reinterpret_cast<const float4*>(resid + i * E + 4);
      *reinterpret_cast<float4*>(out + i * E + 4) = make_float4(b.x + s[4], b.y + s[5], b.z + s[6], b.w + s[7]);
    }
  }
}

// Row-sharded residual stream (tensor-parallel prefill).  Every rank owns T / world consecutive rows of the fp32
// residual stream.  One kernel replaces the all-reduce, the residual add and the RMSNorm that follows them:
//   - tell the peers this rank's partial product (all T rows, in its exchange buffer) is complete, wait for theirs;
//   - for every own row: sum the row's partials over the ranks with plain peer loads (rank order, fp32), add the
//     sum to the residual row (kept in fp32, never rounded), take the row's RMS, and store gain * x * rinv in the
//     activation type into the gathered-activation region of EVERY rank (plain peer stores);
//   - the last CTA tells the peers this rank's rows are written and then waits until every peer has said the same,
//     so that the kernel's completion means this rank's gathered activations are whole.
// The reduce-scatter and the all-gather thus cross NVLink once each, and the residual stream, the add and the norm
// touch T / world rows per rank instead of T.  REDUCE = false skips the partial sums (the norm after the embedding).
// A CTA takes one row at a time; a thread keeps its NCH 16-byte chunks of the row in registers between the two
// passes.  While a row is reduced, normed and stored, the loads of the CTA's next row (from every rank, over NVLink)
// are already in flight: the peer-load latency of one row hides behind the arithmetic and the stores of the one
// before (PREFETCH; chosen on the host where the second set of loads fits the register budget of two CTAs per SM).
// NW is the number of ranks rounded up to 2, 4 or 8 (0: no partial sums, the norm after the embedding) and NCH the
// chunks per thread, both compile-time so that the loads stay in registers.
template <typename T, int NW, int NCH>
struct RowRegs {
  static constexpr int E = 16 / sizeof(T);
  uint4 part[NW > 0 ? NW : 1][NCH];
  float4 x[NCH][E / 4];
};

// Where rank r's partial product of a row lives.  Pulled form: in rank r's own partial region, at the row's index in
// [T].  Pushed form (push_rows > 0: the producing GEMM stored every row band straight into its owner's memory): in
// THIS rank's region, slot r, at the row's index inside the band.
struct PartSrc {
  const uint8_t* base;
  size_t row;
};
__device__ __forceinline__ PartSrc part_src(const PeerPtrs& pp, int r, int self, int only, size_t grow, int row0,
                                            int push_rows) {
  if (push_rows > 0) return PartSrc{reinterpret_cast<const uint8_t*>(pp.buf[self]), (size_t)r * push_rows + (grow - row0)};
  return PartSrc{reinterpret_cast<const uint8_t*>(pp.buf[only >= 0 ? only : r]), grow};
}

template <typename T, int NW, int NCH>
__device__ __forceinline__ void rownorm_load(RowRegs<T, NW, NCH>& g, const PeerPtrs& pp, int world, size_t part_off,
                                             size_t grow, int d, const float* xr, int n_chunks, int only, int self,
                                             int row0, int push_rows) {
  constexpr int E = 16 / sizeof(T);
#pragma unroll
  for (int k = 0; k < NCH; ++k) {
    const int c = threadIdx.x + k * 256;
    if (c < n_chunks) {
#pragma unroll
      for (int r = 0; r < NW; ++r)
        if (r < world) {
          const PartSrc ps = part_src(pp, r, self, only, grow, row0, push_rows);
          g.part[r][k] = load16_sys(ps.base + part_off + (ps.row * d + (size_t)c * E) * sizeof(T));
        }
#pragma unroll
      for (int i = 0; i < E / 4; ++i) g.x[k][i] = *reinterpret_cast<const float4*>(xr + c * E + 4 * i);
    }
  }
}

template <typename T, int NW, int NCH, bool PREFETCH, bool LEAN = false>
__device__ __forceinline__ void rownorm_body(const PeerPtrs& pp, int rank, int world, size_t part_off, size_t xb_off,
                                             int rows, int row0, int d, float* __restrict__ x_own,
                                             const float* __restrict__ gain, float eps, uint32_t epoch,
                                             uint32_t* status, long long budget, int dbg) {
  constexpr int E = 16 / sizeof(T);  // elements per 16-byte chunk
  constexpr bool REDUCE = NW > 0;
  const int only = (dbg & 1) ? rank : -1;  // measurement aid: every load from this rank's own buffer
  const int push_rows = (dbg & 4) ? rows : 0;  // the partial products were pushed into this rank's slots
  __shared__ float red[32];
  __shared__ int s_last;
  uint32_t* my_flags = pp.flags[rank];
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    flag_store_sys(pp.flags[threadIdx.x] + kReadyBase + rank, epoch);
  }
  const bool ok = wait_all_peers(my_flags, kReadyBase, world, epoch, status, budget);
  const int n_chunks = d / E;
  if (ok) {
    // LEAN: no row held ahead; each 16-byte chunk's loads (one per rank) are summed as they arrive, so that eight
    // ranks' partials never sit in registers at once
    RowRegs<T, LEAN ? 0 : NW, LEAN ? 1 : NCH> cur, nxt;
    int row = blockIdx.x;
    if (!LEAN && row < rows)
      rownorm_load(cur, pp, world, part_off, (size_t)(row0 + row), d, x_own + (size_t)row * d, n_chunks, only, rank, row0, push_rows);
    for (; row < rows; row += gridDim.x) {
      const size_t grow = (size_t)(row0 + row);
      float* xr = x_own + (size_t)row * d;
      const int next = row + gridDim.x;
      if (PREFETCH && !LEAN && next < rows)
        rownorm_load(nxt, pp, world, part_off, (size_t)(row0 + next), d, x_own + (size_t)next * d, n_chunks, only, rank, row0,
                     push_rows);
      float v[NCH][E];
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < NCH; ++k) {
        const int c = threadIdx.x + k * 256;
        if (c < n_chunks) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          uint4 part[NW > 0 ? NW : 1];
          float4 xk[E / 4];
          if constexpr (LEAN) {
#pragma unroll
            for (int r = 0; r < NW; ++r)
              if (r < world) {
                const PartSrc ps = part_src(pp, r, rank, only, grow, row0, push_rows);
                part[r] = load16_sys(ps.base + part_off + (ps.row * d + (size_t)c * E) * sizeof(T));
              }
#pragma unroll
            for (int i = 0; i < E / 4; ++i) xk[i] = *reinterpret_cast<const float4*>(xr + c * E + 4 * i);
          } else {
#pragma unroll
            for (int r = 0; r < NW; ++r) part[r] = cur.part[r][k];
#pragma unroll
            for (int i = 0; i < E / 4; ++i) xk[i] = cur.x[k][i];
          }
#pragma unroll
          for (int r = 0; r < NW; ++r)
            if (r < world) accum8(part[r], acc, T());  // rank order: the sum is the same on every run
#pragma unroll
          for (int i = 0; i < E; i += 4) {
            float4 a = xk[i / 4];
            a.x += acc[i]; a.y += acc[i + 1]; a.z += acc[i + 2]; a.w += acc[i + 3];
            if (REDUCE) *reinterpret_cast<float4*>(xr + c * E + i) = a;
            v[k][i] = a.x; v[k][i + 1] = a.y; v[k][i + 2] = a.z; v[k][i + 3] = a.w;
            ss = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(a.z, a.z, fmaf(a.w, a.w, ss))));
          }
        }
      }
      ss = block_sum(ss, red);
      const float rinv = rsqrtf(ss / (float)d + eps);
#pragma unroll
      for (int k = 0; k < NCH; ++k) {
        const int c = threadIdx.x + k * 256;
        if (c < n_chunks) {
          float y[8];
#pragma unroll
          for (int i = 0; i < E; i += 4) {
            const float4 gn = *reinterpret_cast<const float4*>(gain + c * E + i);
            y[i] = gn.x * v[k][i] * rinv; y[i + 1] = gn.y * v[k][i + 1] * rinv;
            y[i + 2] = gn.z * v[k][i + 2] * rinv; y[i + 3] = gn.w * v[k][i + 3] * rinv;
          }
          uint4 out;
          if (sizeof(T) == 2) {
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
            for (int k2 = 0; k2 < 4; ++k2) h[k2] = __floats2bfloat162_rn(y[2 * k2], y[2 * k2 + 1]);
          } else {
            out = make_uint4(__float_as_uint(y[0]), __float_as_uint(y[1]), __float_as_uint(y[2]), __float_as_uint(y[3]));
          }
          const size_t off = xb_off + (grow * d + (size_t)c * E) * sizeof(T);
#pragma unroll
          for (int r = 0; r < kMaxPeers; ++r)
            if (r < world && (!(dbg & 18) || r == rank)) *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(pp.buf[r]) + off) = out;
        }
      }
      if constexpr (LEAN) {
      } else if (PREFETCH) {
        cur = nxt;
      } else if (next < rows) {
        rownorm_load(cur, pp, world, part_off, (size_t)(row0 + next), d, x_own + (size_t)next * d, n_chunks, only, rank, row0,
                     push_rows);
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t done = atomicAdd(my_flags + kCounter, 1u);
    s_last = done == gridDim.x - 1;
    if (s_last) {
      my_flags[kCounter] = 0u;
      __threadfence_system();
      if (dbg & 16) {
        // copy-engine delivery: the rows are whole in THIS rank's region only; copies that the host queued behind
        // this kernel carry them and then this epoch (from the ring) to the peers
        my_flags[kEpochRing + (epoch & 7u)] = epoch;
        flag_store_sys(my_flags + kDoneBase + rank, epoch);
      } else {
        for (int r = 0; r < world; ++r) flag_store_sys(pp.flags[r] + kDoneBase + rank, epoch);
      }
    }
  }
  __syncthreads();
  if (s_last && ok && !(dbg & 8)) wait_all_peers(my_flags, kDoneBase, world, epoch, status, budget);
}

template <typename T, int NW, int NCH, bool PREFETCH>
__global__ void __launch_bounds__(256, 2) peer_rownorm_kernel(PeerPtrs pp, int rank, int world, size_t part_off,
                                                              size_t xb_off, int rows, int row0, int d,
                                                              float* __restrict__ x_own, const float* __restrict__ gain,
                                                              float eps, uint32_t epoch, uint32_t* status,
                                                              long long budget, int dbg) {
  rownorm_body<T, NW, NCH, PREFETCH>(pp, rank, world, part_off, xb_off, rows, row0, d, x_own, gain, eps, epoch, status,
                                     budget, dbg);
}

// The same kernel held to 96 registers and launched with one CTA per SM: the form that runs BESIDE the compute
// kernels of the other half of the batch (a GEMM CTA of 192 threads x 192 registers or an attention CTA of 320 x 128
// leaves 24 K registers and about 1.5 KB of shared memory on its SM; 256 x 96 is exactly that), so that the exchange of one half crosses NVLink while the
// other half computes.
template <typename T, int NW, int NCH>
__global__ void __maxnreg__(96) peer_rownorm_lean_kernel(PeerPtrs pp, int rank, int world, size_t part_off,
                                                         size_t xb_off, int rows, int row0, int d,
                                                         float* __restrict__ x_own, const float* __restrict__ gain,
                                                         float eps, uint32_t epoch, uint32_t* status, long long budget,
                                                         int dbg) {
  // up to four ranks a row's loads all go out together (8 in flight per thread keep the links busy with one CTA per
  // SM); with eight ranks that many would not fit the register cap, so each chunk's eight loads are summed as they arrive
  rownorm_body<T, NW, NCH, false, (NW > 4)>(pp, rank, world, part_off, xb_off, rows, row0, d, x_own, gain, eps, epoch,
                                            status, budget, dbg);
}

// ---- the same exchange through the NVLink switch (multimem) -----------------------------------------------------
// When the ranks' exchange buffers are bound to one multicast object, a load from the multicast address returns the
// SUM of the addressed word over all ranks, added inside the switch (multimem.ld_reduce), and a store to it lands in
// every rank's buffer (multimem.st).  A rank then pulls only its own rows - already reduced - and sends its normed
// rows once: 1/world of the bytes of the peer-load version cross each link.  Flags stay plain peer stores.
__device__ __forceinline__ uint4 mc_ld_reduce(const uint8_t* p, bf16) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 mc_ld_reduce(const uint8_t* p, float) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void mc_st(uint8_t* p, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

template <typename T, int NCH, bool REDUCE>
__global__ void __launch_bounds__(256, 4) peer_rownorm_mc_kernel(PeerPtrs pp, uint8_t* mc, int rank, int world,
                                                                 size_t part_off, size_t xb_off, int rows, int row0,
                                                                 int d, float* __restrict__ x_own,
                                                                 const float* __restrict__ gain, float eps,
                                                                 uint32_t epoch, uint32_t* status, long long budget) {
  constexpr int E = 16 / sizeof(T);
  __shared__ float red[32];
  __shared__ int s_last;
  uint32_t* my_flags = pp.flags[rank];
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    flag_store_sys(pp.flags[threadIdx.x] + kReadyBase + rank, epoch);
  }
  const bool ok = wait_all_peers(my_flags, kReadyBase, world, epoch, status, budget);
  const int n_chunks = d / E;
  if (ok) {
    uint4 cur[NCH], nxt[NCH];
    auto load = [&](uint4 (&g)[NCH], int row) {
      if (!REDUCE) return;
#pragma unroll
      for (int k = 0; k < NCH; ++k) {
        const int c = threadIdx.x + k * 256;
        if (c < n_chunks) g[k] = mc_ld_reduce(mc + part_off + ((size_t)(row0 + row) * d + (size_t)c * E) * sizeof(T), T());
      }
    };
    int row = blockIdx.x;
    if (row < rows) load(cur, row);
    for (; row < rows; row += gridDim.x) {
      const size_t grow = (size_t)(row0 + row);
      float* xr = x_own + (size_t)row * d;
      const int next = row + gridDim.x;
      if (next < rows) load(nxt, next);
      float v[NCH][E];
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < NCH; ++k) {
        const int c = threadIdx.x + k * 256;
        if (c < n_chunks) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          if (REDUCE) accum8(cur[k], acc, T());
#pragma unroll
          for (int i = 0; i < E; i += 4) {
            float4 a = *reinterpret_cast<const float4*>(xr + c * E + i);
            a.x += acc[i]; a.y += acc[i + 1]; a.z += acc[i + 2]; a.w += acc[i + 3];
            if (REDUCE) *reinterpret_cast<float4*>(xr + c * E + i) = a;
            v[k][i] = a.x; v[k][i + 1] = a.y; v[k][i + 2] = a.z; v[k][i + 3] = a.w;
            ss = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(a.z, a.z, fmaf(a.w, a.w, ss))));
          }
        }
      }
      ss = block_sum(ss, red);
      const float rinv = rsqrtf(ss / (float)d + eps);
#pragma unroll
      for (int k = 0; k < NCH; ++k) {
        const int c = threadIdx.x + k * 256;
        if (c < n_chunks) {
          float y[8];
#pragma unroll
          for (int i = 0; i < E; i += 4) {
            const float4 gn = *reinterpret_cast<const float4*>(gain + c * E + i);
            y[i] = gn.x * v[k][i] * rinv; y[i + 1] = gn.y * v[k][i + 1] * rinv;
            y[i + 2] = gn.z * v[k][i + 2] * rinv; y[i + 3] = gn.w * v[k][i + 3] * rinv;
          }
          uint4 out;
          if (sizeof(T) == 2) {
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
            for (int k2 = 0; k2 < 4; ++k2) h[k2] = __floats2bfloat162_rn(y[2 * k2], y[2 * k2 + 1]);
          } else {
            out = make_uint4(__float_as_uint(y[0]), __float_as_uint(y[1]), __float_as_uint(y[2]), __float_as_uint(y[3]));
          }
          mc_st(mc + xb_off + (grow * d + (size_t)c * E) * sizeof(T), out);
        }
      }
#pragma unroll
      for (int k = 0; k < NCH; ++k) cur[k] = nxt[k];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t done = atomicAdd(my_flags + kCounter, 1u);
    s_last = done == gridDim.x - 1;
    if (s_last) {
      my_flags[kCounter] = 0u;
      __threadfence_system();
      for (int r = 0; r < world; ++r) flag_store_sys(pp.flags[r] + kDoneBase + rank, epoch);
    }
  }
  __syncthreads();
  if (s_last && ok) wait_all_peers(my_flags, kDoneBase, world, epoch, status, budget);
}

// One CTA waits, with the given budget, on peer flags that nothing ever sets (a flag array private to this
// self-test): the wait gives up, the status word receives ST_PEER_TIMEOUT, the kernel writes 1 to *reached_end.
__device__ uint32_t g_selftest_peer_flags[kFlagWords];
__global__ void peer_wait_selftest_kernel(long long budget, uint32_t* reached_end, uint32_t* status) {
  const bool ok = wait_all_peers(g_selftest_peer_flags, kReadyBase, 2, 1u, status, budget);
  if (threadIdx.x == 0) *reached_end = ok ? 2u : 1u;
}

constexpr size_t kOneShotMaxBytes = (size_t)2 << 20;

}  // namespace

// The caller writes its partial into the returned buffer and then calls
// comm_peer_allreduce_add with the same size; the two calls must alternate.
void* comm_peer_buffer(void* comm, size_t bytes) {
  if (!comm) return nullptr;
  Comm* c = reinterpret_cast<Comm*>(comm);
  if (!c->pm.on || c->pm.bytes < 2 * kOneShotMaxBytes) return nullptr;
  uint8_t* base = reinterpret_cast<uint8_t*>(c->pm.buf[c->rank]);
  // layout: two alternating halves for the one-pass path, then the region of the two-pass path
  // (separate regions: a peer may still read a half when this rank already fills the large region)
  if (bytes <= kOneShotMaxBytes) return base + ((c->pm.epoch + 1) & 1u) * kOneShotMaxBytes;
  if (bytes > c->pm.bytes - 2 * kOneShotMaxBytes) return nullptr;
  return base + 2 * kOneShotMaxBytes;
}

static int32_t reject_capture(cudaStream_t stream, const char* what) {
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess) {
    cudaGetLastError();
    return B200_OK;
  }
  if (cs != cudaStreamCaptureStatusNone)
    return fail(B200_ERR_UNSUPPORTED,
                "%s cannot be captured into a CUDA graph: its epoch number is a launch argument, so a replay would "
                "find the peers' flags already set; launch tensor-parallel steps eagerly", what);
  return B200_OK;
}

// Regions of this rank's exchange buffer for the row-sharded prefill: `part` receives this rank's partial product
// [T, d], `xb` is where every rank deposits its rows of the normed activations.  False when the peer path is off or
// the two regions do not fit.
bool comm_peer_rowshard_buffers(void* comm, size_t bytes_each, void** part, void** xb) {
  if (!comm) return false;
  Comm* c = reinterpret_cast<Comm*>(comm);
  const size_t each = align_up(bytes_each, 256);
  if (!c->pm.on || c->pm.bytes < 2 * kOneShotMaxBytes + 2 * each) return false;
  uint8_t* base = reinterpret_cast<uint8_t*>(c->pm.buf[c->rank]) + 2 * kOneShotMaxBytes;
  *part = base;
  *xb = base + each;
  return true;
}

// In-switch reduction halves the bytes on every link from four ranks on ((world + 1) / world of the buffer each way
// instead of 2 (world - 1) / world); it was never faster on the boxes this was measured on (200 us against 118 us per
// exchange of 64 MiB between two ranks, 216 against 197 us among four), so it is off unless B200_TP_MULTIMEM = 1.
// Work queued on the copy stream by an earlier exchange reads this rank's gathered rows: whatever overwrites them or
// frees the memory goes behind it.
static int32_t join_copies(Comm* c, cudaStream_t stream) {
  if (c->sent_pending) {
    B200_CUDA_OK(cudaStreamWaitEvent(stream, c->ev_sent, 0));
    c->sent_pending = false;
  }
  return B200_OK;
}

static bool use_multimem(const Comm* c) {
  static const int mc_env = env_int("B200_TP_MULTIMEM", -1);
  return c->pm.mc && mc_env > 0;
}

int32_t comm_peer_reduce_norm(void* comm, int T, int d, int dtype, bool reduce, float* x_own, const float* gain,
                              float eps, cudaStream_t stream, bool pushed, PeerBands* bands) {
  const size_t each = align_up((size_t)T * d * (dtype == B200_BF16 ? 2 : 4), 256);
  return comm_peer_reduce_norm_at(comm, T, d, dtype, reduce, x_own, gain, eps, 0, each, false, stream, pushed, bands);
}

// Where a pushed store of a [T, d] partial product goes: bases[o] is slot `rank` of rank o's partial region, a
// [T / world, d] matrix, for every rank o (this one included).  False when the exchange cannot take pushed partials
// (no peer memory, in-switch reduction selected, rows not a multiple of 32).
bool comm_peer_push_bases(void* comm, int T, int d, int dtype, void** bases) {
  if (!comm) return false;
  Comm* c = reinterpret_cast<Comm*>(comm);
  const size_t es = dtype == B200_BF16 ? 2 : 4;
  if (!c->pm.on || use_multimem(c) || T % c->world || (T / c->world) % 32 || c->world > 8) return false;
  if (c->pm.bytes < 2 * kOneShotMaxBytes + 2 * align_up((size_t)T * d * es, 256)) return false;
  const size_t rows = (size_t)(T / c->world);
  for (int o = 0; o < c->world; ++o)
    bases[o] = reinterpret_cast<uint8_t*>(c->pm.buf[o]) + 2 * kOneShotMaxBytes + (size_t)c->rank * rows * d * es;
  return true;
}

// The exchange over `T` rows whose partial products start `part_rel` bytes and whose gathered rows start `xb_rel`
// bytes into the row-shard area of every rank's exchange memory.  lean: the form that runs beside compute kernels
// (one CTA per SM, 96 registers).
int32_t comm_peer_reduce_norm_at(void* comm, int T, int d, int dtype, bool reduce, float* x_own, const float* gain,
                                 float eps, size_t part_rel, size_t xb_rel, bool lean, cudaStream_t stream,
                                 bool pushed, PeerBands* bands) {
  Comm* c = reinterpret_cast<Comm*>(comm);
  if (!c || !c->pm.on) return fail(B200_ERR_INVALID_ARG, "peer memory is not set up for this communicator");
  const size_t es = dtype == B200_BF16 ? 2 : 4;
  if (T % c->world || ((size_t)d * es) % 16 || d % 4)
    return fail(B200_ERR_BAD_SHAPE, "row-sharded exchange: %d rows over %d ranks, row of %d elements", T, c->world, d);
  B200_TRY(reject_capture(stream, "the tensor-parallel exchange over peer memory"));
  B200_TRY(join_copies(c, stream));
  ProfScope prof(PROF_COMM, (double)T * d * es, stream);
  PeerPtrs pp;
  for (int r = 0; r < kMaxPeers; ++r) {
    pp.buf[r] = c->pm.buf[r];
    pp.flags[r] = c->pm.flags[r];
  }
  const uint32_t epoch = ++c->pm.epoch;
  const int rows = T / c->world, row0 = c->rank * rows;
  const size_t part_off = 2 * kOneShotMaxBytes + part_rel, xb_off = 2 * kOneShotMaxBytes + xb_rel;
  int grid = sm_count() * (lean ? 1 : 2);  // two CTAs of 256 threads are resident per SM (register tile of the row)
  if (grid > rows) grid = rows;
  uint32_t* status = device_status_word();
  const int n_chunks = (int)((size_t)d * es / 16);
  const int nch = n_chunks <= 256 ? 1 : n_chunks <= 512 ? 2 : 4;
  if (n_chunks > 1024)
    return fail(B200_ERR_BAD_SHAPE, "row-sharded exchange: rows of %d elements exceed 16 KB", d);
  const int nw = !reduce ? 0 : c->world <= 2 ? 2 : c->world <= 4 ? 4 : 8;
  const bool use_mc = use_multimem(c);
  if (use_mc && pushed) return fail(B200_ERR_UNSUPPORTED, "pushed partial products and in-switch reduction exclude each other");
  if (use_mc) {
    int grid_mc = sm_count() * (lean ? 1 : 4);
    if (grid_mc > rows) grid_mc = rows;
#define B200_ROWNORM_MC(TT, NCH)                                                                                    \
  do {                                                                                                              \
    if (reduce)                                                                                                     \
      peer_rownorm_mc_kernel<TT, NCH, true><<<grid_mc, 256, 0, stream>>>(pp, c->pm.mc, c->rank, c->world, part_off, \
                                                                         xb_off, rows, row0, d, x_own, gain, eps,   \
                                                                         epoch, status, c->wait_budget);            \
    else                                                                                                            \
      peer_rownorm_mc_kernel<TT, NCH, false><<<grid_mc, 256, 0, stream>>>(pp, c->pm.mc, c->rank, c->world, part_off, \
                                                                          xb_off, rows, row0, d, x_own, gain, eps,  \
                                                                          epoch, status, c->wait_budget);           \
  } while (0)
    if (dtype == B200_BF16) {
      if (nch == 1) B200_ROWNORM_MC(bf16, 1); else if (nch == 2) B200_ROWNORM_MC(bf16, 2); else B200_ROWNORM_MC(bf16, 4);
    } else {
      if (nch == 1) B200_ROWNORM_MC(float, 1); else if (nch == 2) B200_ROWNORM_MC(float, 2); else B200_ROWNORM_MC(float, 4);
    }
#undef B200_ROWNORM_MC
    B200_LAUNCH_OK("peer_rownorm_mc_kernel");
    return B200_OK;
  }
  // registers of one row's loads: NW * NCH * 4 (partials) + NCH * (4 or 8) (residual); two sets fit below about 72
  const int regs_row = (nw > 0 ? nw : 1) * nch * 4 + nch * (int)(16 / es);
  static const int pf_env = env_int("B200_ROWNORM_PREFETCH", -1);  // -1: decide by the register estimate
  static const int dbg_env = env_int("B200_EXCH_LOCAL_ONLY", 0);   // measurement aid: 1 loads, 2 stores stay on this GPU
  // bit 2: partial products sit in this rank's slots; bit 3: the consumer waits for the peers' rows, not this kernel
  // bit 4: the kernel leaves its normed rows in this rank's region only and the copy engines deliver them (below)
  static const int ce_env = env_int("B200_TP_COPY_ENGINE", 1);
  bool ce = bands && ce_env && c->world > 1;
  if (ce && !c->ce_stream) {
    if (cudaStreamCreateWithFlags(&c->ce_stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_rows, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_sent, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      return fail(B200_ERR_CUDA, "creating the copy stream of the tensor-parallel exchange failed");
    }
  }
  const int dbg = (dbg_env & 3) | (pushed ? 4 : 0) | (bands ? 8 : 0) | (ce ? 16 : 0);
  if (bands) {
    bands->flags = c->pm.flags[c->rank] + kDoneBase;
    bands->epoch = epoch;
    bands->rows = rows;
    bands->first = c->rank;
    bands->budget = c->wait_budget;
  }
  const bool prefetch = pf_env >= 0 ? pf_env != 0 : regs_row <= 72;
#define B200_ROWNORM(TT, NW, NCH)                                                                                    \
  do {                                                                                                               \
    if (lean)                                                                                                        \
      peer_rownorm_lean_kernel<TT, NW, NCH><<<grid, 256, 0, stream>>>(pp, c->rank, c->world, part_off, xb_off, rows, \
                                                                      row0, d, x_own, gain, eps, epoch, status,      \
                                                                      c->wait_budget, dbg);                          \
    else if (prefetch)                                                                                               \
      peer_rownorm_kernel<TT, NW, NCH, true><<<grid, 256, 0, stream>>>(pp, c->rank, c->world, part_off, xb_off, rows, \
                                                                       row0, d, x_own, gain, eps, epoch, status,     \
                                                                       c->wait_budget, dbg);                         \
    else                                                                                                             \
      peer_rownorm_kernel<TT, NW, NCH, false><<<grid, 256, 0, stream>>>(pp, c->rank, c->world, part_off, xb_off,     \
                                                                        rows, row0, d, x_own, gain, eps, epoch,      \
                                                                        status, c->wait_budget, dbg);                \
  } while (0)
#define B200_ROWNORM_NCH(TT, NW)                       \
  do {                                                 \
    if (nch == 1) B200_ROWNORM(TT, NW, 1);             \
    else if (nch == 2) B200_ROWNORM(TT, NW, 2);        \
    else B200_ROWNORM(TT, NW, 4);                      \
  } while (0)
#define B200_ROWNORM_NW(TT)                            \
  do {                                                 \
    if (nw == 0) B200_ROWNORM_NCH(TT, 0);              \
    else if (nw == 2) B200_ROWNORM_NCH(TT, 2);         \
    else if (nw == 4) B200_ROWNORM_NCH(TT, 4);         \
    else B200_ROWNORM_NCH(TT, 8);                      \
  } while (0)
  if (dtype == B200_BF16) B200_ROWNORM_NW(bf16);
  else B200_ROWNORM_NW(float);
#undef B200_ROWNORM_NW
#undef B200_ROWNORM_NCH
#undef B200_ROWNORM
  B200_LAUNCH_OK("peer_rownorm_kernel");
  if (ce) {
    // This rank's normed rows, then the epoch, to every peer by copies on a stream of their own: they cross NVLink
    // on the copy engines while the GEMM that consumes the gathered rows already works on this rank's band.  One
    // copy per destination and word, one after the other (side by side on a stream per destination every band
    // arrived at the END of the transfer and the consumers waited longer: 26.8 against 25.5 ms per step on eight
    // ranks); copies of one stream complete in order, so a peer that sees the epoch has the rows.
    B200_CUDA_OK(cudaEventRecord(c->ev_rows, stream));
    B200_CUDA_OK(cudaStreamWaitEvent(c->ce_stream, c->ev_rows, 0));
    const size_t row_bytes = (size_t)d * es;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(c->pm.buf[c->rank]) + xb_off + (size_t)row0 * row_bytes;
    const uint32_t* epoch_src = c->pm.flags[c->rank] + kEpochRing + (epoch & 7u);
    // Destinations in the order rank - 1, rank - 2, ...: the consumer visits the bands rank, rank + 1, rank + 2, ...,
    // so the band it needs first after its own is the first one its neighbour sends.
    for (int i = 1; i < c->world; ++i) {
      const int r = (c->rank - i + c->world) % c->world;
      uint8_t* dst = reinterpret_cast<uint8_t*>(c->pm.buf[r]) + xb_off + (size_t)row0 * row_bytes;
      B200_CUDA_OK(cudaMemcpyAsync(dst, src, (size_t)rows * row_bytes, cudaMemcpyDeviceToDevice, c->ce_stream));
      B200_CUDA_OK(cudaMemcpyAsync(c->pm.flags[r] + kDoneBase + c->rank, epoch_src, sizeof(uint32_t),
                                   cudaMemcpyDeviceToDevice, c->ce_stream));
    }
    B200_CUDA_OK(cudaEventRecord(c->ev_sent, c->ce_stream));
    c->sent_pending = true;
  }
  return B200_OK;
}

int32_t launch_peer_wait_selftest(long long budget, uint32_t* reached_end, cudaStream_t stream) {
  peer_wait_selftest_kernel<<<1, 32, 0, stream>>>(budget, reached_end, device_status_word());
  B200_LAUNCH_OK("peer_wait_selftest_kernel");
  return B200_OK;
}

int32_t comm_peer_allreduce_add(void* comm, size_t count, int dtype, const float* resid, float* out,
                                cudaStream_t stream) {
  Comm* c = reinterpret_cast<Comm*>(comm);
  if (!c || !c->pm.on) return fail(B200_ERR_INVALID_ARG, "peer memory is not set up for this communicator");
  const size_t es = dtype == B200_BF16 ? 2 : 4;
  if ((count * es) % 16 || count * es > c->pm.bytes - 2 * kOneShotMaxBytes)
    return fail(B200_ERR_BAD_SHAPE, "peer all-reduce: bad size");
  B200_TRY(reject_capture(stream, "the tensor-parallel all-reduce over peer memory"));
  B200_TRY(join_copies(c, stream));  // a flag copy of an earlier exchange must not land behind this kernel's flags
  ProfScope prof(PROF_COMM, (double)count * es, stream);
  const bool small = count * es <= kOneShotMaxBytes;
  PeerPtrs pp;
  for (int r = 0; r < kMaxPeers; ++r) {
    // the two-pass kernels index from the start of the large region
    pp.buf[r] = c->pm.buf[r] ? reinterpret_cast<uint8_t*>(c->pm.buf[r]) + (small ? 0 : 2 * kOneShotMaxBytes) : nullptr;
    pp.flags[r] = c->pm.flags[r];
  }
  const uint32_t epoch = ++c->pm.epoch;
  const size_t n_vec = count * es / 16;
  uint32_t* status = device_status_word();
  if (small) {
    const size_t half_off = (size_t)(epoch & 1u) * kOneShotMaxBytes;
    int g1 = (int)((n_vec + 511) / 512);
    if (g1 > sm_count()) g1 = sm_count();
    if (dtype == B200_BF16)
      peer_oneshot_kernel<bf16><<<g1, 512, 0, stream>>>(pp, c->rank, c->world, n_vec, half_off, epoch, resid, out, status, c->wait_budget);
    else
      peer_oneshot_kernel<float><<<g1, 512, 0, stream>>>(pp, c->rank, c->world, n_vec, half_off, epoch, resid, out, status, c->wait_budget);
    B200_LAUNCH_OK("peer_oneshot_kernel");
    return B200_OK;
  }
  int grid = sm_count();
  const size_t want = (n_vec / c->world + 511) / 512;
  if ((size_t)grid > want) grid = want < 1 ? 1 : (int)want;
  if (dtype == B200_BF16)
    peer_reduce_kernel<bf16><<<grid, 512, 0, stream>>>(pp, c->rank, c->world, n_vec, epoch, status, c->wait_budget);
  else
    peer_reduce_kernel<float><<<grid, 512, 0, stream>>>(pp, c->rank, c->world, n_vec, epoch, status, c->wait_budget);
  B200_LAUNCH_OK("peer_reduce_kernel");
  int grid2 = sm_count() * 2;
  const size_t want2 = (n_vec + 511) / 512;
  if ((size_t)grid2 > want2) grid2 = want2 < 1 ? 1 : (int)want2;
  if (dtype == B200_BF16)
    peer_add_kernel<bf16><<<grid2, 512, 0, stream>>>(pp, c->rank, c->world, n_vec, epoch, resid, out, status, c->wait_budget);
  else
    peer_add_kernel<float><<<grid2, 512, 0, stream>>>(pp, c->rank, c->world, n_vec, epoch, resid, out, status, c->wait_budget);
  B200_LAUNCH_OK("peer_add_kernel");
  return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" {

int32_t b200_comm_unique_id(void* id128) {
  if (!id128) return fail(B200_ERR_INVALID_ARG, "id buffer is null");
  NcclApi& a = api();
  if (!a.ok) return fail(B200_ERR_NCCL, "NCCL is not available in this process");
  const int rc = a.get_unique_id(reinterpret_cast<NcclUniqueId*>(id128));
  if (rc != 0) return nccl_fail("ncclGetUniqueId", rc);
  return B200_OK;
}

int32_t b200_comm_init_rank(const void* id128, int32_t rank, int32_t world, void** comm) {
  if (!id128 || !comm) return fail(B200_ERR_INVALID_ARG, "null argument");
  if (world < 1 || rank < 0 || rank >= world) return fail(B200_ERR_INVALID_ARG, "bad rank %d of %d", rank, world);
  NcclApi& a = api();
  if (!a.ok) return fail(B200_ERR_NCCL, "NCCL is not available in this process");
  NcclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  NcclComm nc = nullptr;
  const int rc = a.comm_init_rank(&nc, world, id, rank);
  if (rc != 0) return nccl_fail("ncclCommInitRank", rc);
  Comm* c = new Comm();
  c->nccl = nc;
  c->rank = rank;
  c->world = world;
  const int budget_m = env_int("B200_PEER_WAIT_MCYCLES", 4000);  // millions of SM clocks
  c->wait_budget = (long long)(budget_m > 0 ? budget_m : 4000) * 1000000LL;
  const int poll_ns = env_int("B200_PEER_POLL_NS", -1);
  if (poll_ns >= 0 && cudaMemcpyToSymbol(g_poll_ns, &poll_ns, sizeof(int)) != cudaSuccess)
    return fail(B200_ERR_CUDA, "setting the flag poll pause failed");
  setup_peer_memory(c);
  *comm = c;
  return B200_OK;
}

// A communicator whose peer-mapped exchange memory the caller brings (b200_comm_attach_memory) does not set up its
// own at creation.
int32_t b200_comm_init_rank_ex(const void* id128, int32_t rank, int32_t world, int32_t own_peer_memory, void** comm) {
  if (!id128 || !comm) return fail(B200_ERR_INVALID_ARG, "null argument");
  if (world < 1 || rank < 0 || rank >= world) return fail(B200_ERR_INVALID_ARG, "bad rank %d of %d", rank, world);
  NcclApi& a = api();
  if (!a.ok) return fail(B200_ERR_NCCL, "NCCL is not available in this process");
  NcclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  NcclComm nc = nullptr;
  const int rc = a.comm_init_rank(&nc, world, id, rank);
  if (rc != 0) return nccl_fail("ncclCommInitRank", rc);
  Comm* c = new Comm();
  c->nccl = nc;
  c->rank = rank;
  c->world = world;
  const int budget_m = env_int("B200_PEER_WAIT_MCYCLES", 4000);  // millions of SM clocks
  c->wait_budget = (long long)(budget_m > 0 ? budget_m : 4000) * 1000000LL;
  const int poll_ns = env_int("B200_PEER_POLL_NS", -1);
  if (poll_ns >= 0 && cudaMemcpyToSymbol(g_poll_ns, &poll_ns, sizeof(int)) != cudaSuccess)
    return fail(B200_ERR_CUDA, "setting the flag poll pause failed");
  if (own_peer_memory) setup_peer_memory(c);
  *comm = c;
  return B200_OK;
}

int32_t b200_comm_setup_peer_memory(void* comm) {
  if (!comm) return fail(B200_ERR_INVALID_ARG, "communicator is null");
  Comm* c = reinterpret_cast<Comm*>(comm);
  if (c->pm.on) return B200_OK;
  setup_peer_memory(c);
  return B200_OK;
}

int32_t b200_comm_attach_memory(void* comm, size_t bytes, const void* const* peer_ptrs, void* multicast_ptr) {
  if (!comm || !peer_ptrs) return fail(B200_ERR_INVALID_ARG, "null argument");
  Comm* c = reinterpret_cast<Comm*>(comm);
  NcclApi& a = api();
  if (!a.ok) return fail(B200_ERR_NCCL, "NCCL is not available in this process");
  if (c->world < 2 || c->world > kMaxPeers) return fail(B200_ERR_UNSUPPORTED, "peer memory serves 2..%d ranks", kMaxPeers);
  if (c->pm.on) return fail(B200_ERR_INVALID_ARG, "the communicator already has exchange memory");
  constexpr size_t kFlagBytes = 4096;
  bool ok = bytes >= 4 * kOneShotMaxBytes + kFlagBytes && bytes % 256 == 0;
  for (int r = 0; ok && r < c->world; ++r) ok = peer_ptrs[r] != nullptr && aligned16(peer_ptrs[r]);
  PeerMem pm;
  if (ok) {
    pm.bytes = bytes - kFlagBytes;
    for (int r = 0; r < c->world; ++r) {
      pm.buf[r] = const_cast<void*>(peer_ptrs[r]);
      pm.flags[r] = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(pm.buf[r]) + pm.bytes);
    }
    pm.mc = reinterpret_cast<uint8_t*>(multicast_ptr);
    pm.external = true;
    // this rank's flag words start at zero; nobody may signal before every rank has cleared its own
    ok = cudaMemset(pm.flags[c->rank], 0, kFlagBytes) == cudaSuccess && cudaDeviceSynchronize() == cudaSuccess;
  }
  // agreement (doubles as the barrier after the clearing): every rank must have accepted its pointers, and either all
  // or none bring a multicast address
  float verdict[2] = {ok ? 1.f : 0.f, (ok && multicast_ptr) ? 1.f : 0.f}, total[2] = {0.f, 0.f};
  float* dv = nullptr;
  const bool agreed = cudaMalloc(&dv, 256) == cudaSuccess &&
                      cudaMemcpy(dv, verdict, 8, cudaMemcpyHostToDevice) == cudaSuccess &&
                      a.all_reduce(dv, dv, 2, kNcclFloat32, kNcclSum, c->nccl, 0) == 0 &&
                      cudaStreamSynchronize(0) == cudaSuccess &&
                      cudaMemcpy(total, dv, 8, cudaMemcpyDeviceToHost) == cudaSuccess;
  if (dv) cudaFree(dv);
  if (!agreed || total[0] != (float)c->world) {
    cudaGetLastError();
    return fail(B200_ERR_UNSUPPORTED, "not every rank could attach its exchange memory");
  }
  if (total[1] != (float)c->world) pm.mc = nullptr;
  pm.on = true;
  c->pm = pm;
  return B200_OK;
}

int32_t b200_comm_destroy(void* comm) {
  if (!comm) return B200_OK;
  Comm* c = reinterpret_cast<Comm*>(comm);
  NcclApi& a = api();
  if (!a.ok) return fail(B200_ERR_NCCL, "NCCL is not available in this process");
  cudaDeviceSynchronize();
  // The exchange buffer and flag words are mapped by the peers: nobody frees them until every rank has finished
  // its own work (a slower peer may still be reading this rank's buffer or storing into its flags).  A one-float
  // all-reduce is the agreement; a rank whose peers are gone gets an error from it and frees anyway.
  if (c->world > 1) {
    float* token = nullptr;
    if (cudaMalloc(&token, 256) == cudaSuccess) {
      cudaMemset(token, 0, 256);
      if (a.all_reduce(token, token, 1, kNcclFloat32, kNcclSum, c->nccl, 0) == 0) cudaStreamSynchronize(0);
      cudaFree(token);
    }
    cudaGetLastError();
  }
  if (c->ce_stream) {
    cudaStreamSynchronize(c->ce_stream);
    cudaStreamDestroy(c->ce_stream);
    cudaEventDestroy(c->ev_rows);
    cudaEventDestroy(c->ev_sent);
  }
  free_peer_memory(c);
  const int rc = a.comm_destroy(c->nccl);
  delete c;
  if (rc != 0) return nccl_fail("ncclCommDestroy", rc);
  return B200_OK;
}

int32_t b200_allreduce_f32(void* comm, float* data, size_t count, b200_stream_t stream) {
  return comm_allreduce(comm, data, count, B200_F32, reinterpret_cast<cudaStream_t>(stream));
}

int32_t b200_tp_exchange_buffers(void* comm, size_t bytes_each, void** part, void** gathered) {
  if (!comm || !part || !gathered) return fail(B200_ERR_INVALID_ARG, "null argument");
  if (!comm_peer_rowshard_buffers(comm, bytes_each, part, gathered))
    return fail(B200_ERR_UNSUPPORTED, "the communicator has no exchange memory for two regions of %zu bytes", bytes_each);
  return B200_OK;
}

int32_t b200_tp_reduce_norm(void* comm, int32_t rows_total, int32_t dim, int32_t dtype, int32_t reduce, float* x_own,
                            const float* gain, float eps, b200_stream_t stream) {
  if (!comm || !x_own || !gain) return fail(B200_ERR_INVALID_ARG, "null argument");
  if (dtype != B200_F32 && dtype != B200_BF16) return fail(B200_ERR_BAD_DTYPE, "dtype must be fp32 or bf16");
  if (rows_total <= 0 || dim <= 0) return fail(B200_ERR_BAD_SHAPE, "rows=%d dim=%d", rows_total, dim);
  if (!aligned16(x_own) || !aligned16(gain)) return fail(B200_ERR_MISALIGNED, "buffers must be 16-byte aligned");
  return comm_peer_reduce_norm(comm, rows_total, dim, dtype, reduce != 0, x_own, gain, eps,
                               reinterpret_cast<cudaStream_t>(stream));
}

int32_t b200_selftest_peer_wait(int64_t budget_cycles, uint32_t* reached_end_device, b200_stream_t stream) {
  if (!reached_end_device) return fail(B200_ERR_INVALID_ARG, "null argument");
  if (budget_cycles <= 0 || budget_cycles > 4000000000LL) return fail(B200_ERR_INVALID_ARG, "budget out of range");
  return launch_peer_wait_selftest(budget_cycles, reached_end_device, reinterpret_cast<cudaStream_t>(stream));
}

int32_t b200_comm_peer_memory(void* comm, int32_t* enabled) {
  if (!comm || !enabled) return fail(B200_ERR_INVALID_ARG, "null argument");
  const Comm* c = reinterpret_cast<Comm*>(comm);
  *enabled = !c->pm.on ? 0 : (c->pm.mc ? 2 : 1);
  return B200_OK;
}

}  // extern "C"
