// NCCL glue.  The library does not link NCCL: the symbols are resolved at first
// use from the libnccl already loaded into the process (the one PyTorch ships)
// or from the system library, so single-GPU users need no NCCL at all.
#include <dlfcn.h>

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
typedef const char* (*GetErrorStringFn)(int);

struct NcclApi {
  GetUniqueIdFn get_unique_id = nullptr;
  CommInitRankFn comm_init_rank = nullptr;
  CommDestroyFn comm_destroy = nullptr;
  AllReduceFn all_reduce = nullptr;
  GetErrorStringFn error_string = nullptr;
  bool ok = false;
};

// ncclDataType_t / ncclRedOp_t values of the public nccl.h
constexpr int kNcclFloat32 = 7, kNcclBfloat16 = 9, kNcclSum = 0;

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
    a.error_string = (GetErrorStringFn)dlsym(h, "ncclGetErrorString");
    a.ok = a.get_unique_id && a.comm_init_rank && a.comm_destroy && a.all_reduce && a.error_string;
  });
  return a;
}

int32_t nccl_fail(const char* what, int rc) {
  return fail(B200_ERR_NCCL, "%s failed: %s", what, api().error_string ? api().error_string(rc) : "?");
}

}  // namespace

int32_t comm_allreduce(void* comm, void* data, size_t count, int dtype, cudaStream_t stream) {
  if (!comm) return fail(B200_ERR_INVALID_ARG, "communicator is null");
  NcclApi& a = api();
  if (!a.ok) return fail(B200_ERR_NCCL, "NCCL is not available in this process");
  const int nt = dtype == B200_BF16 ? kNcclBfloat16 : kNcclFloat32;
  const int rc = a.all_reduce(data, data, count, nt, kNcclSum, comm, stream);
  if (rc != 0) return nccl_fail("ncclAllReduce", rc);
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
  NcclComm c = nullptr;
  const int rc = a.comm_init_rank(&c, world, id, rank);
  if (rc != 0) return nccl_fail("ncclCommInitRank", rc);
  *comm = c;
  return B200_OK;
}

int32_t b200_comm_destroy(void* comm) {
  if (!comm) return B200_OK;
  NcclApi& a = api();
  if (!a.ok) return fail(B200_ERR_NCCL, "NCCL is not available in this process");
  const int rc = a.comm_destroy(comm);
  if (rc != 0) return nccl_fail("ncclCommDestroy", rc);
  return B200_OK;
}

int32_t b200_allreduce_f32(void* comm, float* data, size_t count, b200_stream_t stream) {
  return comm_allreduce(comm, data, count, B200_F32, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
