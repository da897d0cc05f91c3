// Tensor-parallel exchange steps of a session: sum of the ranks' partial o_proj / down products
// and the gather of the ranks' lm_head slices. NCCL is looked up at run time (the library the
// process already has loaded, normally the one bundled with torch), so the shared library has no
// link-time dependency on it and single-GPU users never touch it.
#include <dlfcn.h>
#include <nccl.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <string>

#include "common.cuh"

namespace dyn {
namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  std::string error;
};

NcclApi* nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[3] = {getenv("DYNINFER_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      if (!n || !*n) continue;
      api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (api.handle) break;
      api.error = dlerror();
    }
    if (!api.handle) return;
    bool ok = true;
    auto sym = [&](const char* name) {
      void* p = dlsym(api.handle, name);
      if (!p) {
        ok = false;
        api.error = std::string("symbol ") + name + " not found";
      }
      return p;
    };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    if (!ok) {
      dlclose(api.handle);
      api.handle = nullptr;
    }
  });
  return &api;
}

int need_api(NcclApi** out) {
  NcclApi* a = nccl_api();
  DYN_CHECK(a->handle != nullptr, "tensor parallelism needs NCCL and it cannot be loaded: %s",
            a->error.c_str());
  *out = a;
  return 0;
}

#define DYN_NCCL(api, call)                                                              \
  do {                                                                                   \
    ncclResult_t r_ = (call);                                                            \
    if (r_ != ncclSuccess) {                                                             \
      set_error("%s failed: %s", #call, (api)->GetErrorString(r_));                      \
      return 1;                                                                          \
    }                                                                                    \
  } while (0)

}  // namespace

size_t tp_unique_id_bytes() { return sizeof(ncclUniqueId); }

int tp_unique_id(uint8_t* out) {
  NcclApi* a;
  if (need_api(&a)) return 1;
  ncclUniqueId id;
  DYN_NCCL(a, a->GetUniqueId(&id));
  memcpy(out, &id, sizeof id);
  return 0;
}

int tp_comm_init(void** comm, const uint8_t* id_bytes, int rank, int world) {
  NcclApi* a;
  if (need_api(&a)) return 1;
  ncclUniqueId id;
  memcpy(&id, id_bytes, sizeof id);
  ncclComm_t c = nullptr;
  DYN_NCCL(a, a->CommInitRank(&c, world, id, rank));
  *comm = c;
  return 0;
}

void tp_comm_destroy(void* comm) {
  NcclApi* a = nccl_api();
  if (comm && a->handle) a->CommDestroy(reinterpret_cast<ncclComm_t>(comm));
}

int tp_all_reduce_sum(void* comm, const float* send, float* recv, size_t count, cudaStream_t st) {
  NcclApi* a;
  if (need_api(&a)) return 1;
  DYN_NCCL(a, a->AllReduce(send, recv, count, ncclFloat32, ncclSum, reinterpret_cast<ncclComm_t>(comm), st));
  return 0;
}

int tp_all_gather(void* comm, const float* send, float* recv, size_t count_per_rank, cudaStream_t st) {
  NcclApi* a;
  if (need_api(&a)) return 1;
  DYN_NCCL(a, a->AllGather(send, recv, count_per_rank, ncclFloat32, reinterpret_cast<ncclComm_t>(comm), st));
  return 0;
}

}  // namespace dyn
