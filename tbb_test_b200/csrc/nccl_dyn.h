// Run-time binding of the few NCCL entry points the gradient allreduce needs.
// The library is looked up when the first multi-GPU handle is created, so a
// single-GPU job has no NCCL dependency, and a process that already loaded NCCL
// (for instance through PyTorch) shares that copy instead of loading a second one.
#pragma once

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stddef.h>

#include <mutex>
#include <string>

namespace b2 {

// ABI-stable subset of nccl.h (NCCL 2.x).
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0, ncclInProgress = 7 };
enum { ncclFloat32 = 7, ncclBfloat16 = 9 };
enum { ncclSum = 0 };

// ncclConfig_t as laid out since NCCL 2.27 (the library reads `size` and `version` and
// treats fields beyond an older caller's size as unset). Unset: INT_MIN / nullptr.
struct ncclConfigCompat {
  size_t size;
  unsigned int magic;
  unsigned int version;
  int blocking, cgaClusterSize, minCTAs, maxCTAs;
  const char* netName;
  int splitShare, trafficClass;
  const char* commName;
  int collnetEnable, CTAPolicy, shrinkShare, nvlsCTAs;
};
inline ncclConfigCompat nccl_config_unset() {
  const int U = -2147483647 - 1;
  ncclConfigCompat c = {sizeof(ncclConfigCompat), 0xcafebeefu, 22703u, U, U, U, U, nullptr, U, U, nullptr, U, U, U, U};
  return c;
}

struct NcclApi {
  int (*GetUniqueId)(ncclUniqueId*) = nullptr;
  int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  int (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfigCompat*) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*CommAbort)(ncclComm_t) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*ReduceScatter)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;  // optional
  int (*GroupEnd)() = nullptr;
  int (*CommGetAsyncError)(ncclComm_t, int*) = nullptr;
  // optional: buffers allocated by the library and registered with the communicator let its
  // collectives work on them in place (NVLink SHARP: fewer CTAs, no staging copies)
  int (*MemAlloc)(void**, size_t) = nullptr;
  int (*MemFree)(void*) = nullptr;
  int (*CommRegister)(ncclComm_t, void*, size_t, void**) = nullptr;
  int (*CommDeregister)(ncclComm_t, void*) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  int (*GetVersion)(int*) = nullptr;
  std::string path, error;
  bool ok = false;
};

inline NcclApi& nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = nullptr;
    const char* env = getenv("B2_NCCL_PATH");
    if (env) h = dlopen(env, RTLD_NOW | RTLD_GLOBAL);
    if (h) api.path = env;
    if (!h) {
      // already mapped by the hosting process?
      h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
      if (h) api.path = "libnccl.so.2 (already loaded)";
    }
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
      api.error = "libnccl.so.2 not found (set B2_NCCL_PATH)";
      return;
    }
    auto sym = [&](const char* n) { return dlsym(h, n); };
    api.GetUniqueId = (decltype(api.GetUniqueId))sym("ncclGetUniqueId");
    api.CommInitRank = (decltype(api.CommInitRank))sym("ncclCommInitRank");
    api.CommInitRankConfig = (decltype(api.CommInitRankConfig))sym("ncclCommInitRankConfig");
    api.CommDestroy = (decltype(api.CommDestroy))sym("ncclCommDestroy");
    api.CommAbort = (decltype(api.CommAbort))sym("ncclCommAbort");
    api.AllReduce = (decltype(api.AllReduce))sym("ncclAllReduce");
    api.ReduceScatter = (decltype(api.ReduceScatter))sym("ncclReduceScatter");
    api.AllGather = (decltype(api.AllGather))sym("ncclAllGather");
    api.GroupStart = (decltype(api.GroupStart))sym("ncclGroupStart");
    api.GroupEnd = (decltype(api.GroupEnd))sym("ncclGroupEnd");
    api.CommGetAsyncError = (decltype(api.CommGetAsyncError))sym("ncclCommGetAsyncError");
    api.MemAlloc = (decltype(api.MemAlloc))sym("ncclMemAlloc");
    api.MemFree = (decltype(api.MemFree))sym("ncclMemFree");
    api.CommRegister = (decltype(api.CommRegister))sym("ncclCommRegister");
    api.CommDeregister = (decltype(api.CommDeregister))sym("ncclCommDeregister");
    api.GetErrorString = (decltype(api.GetErrorString))sym("ncclGetErrorString");
    api.GetVersion = (decltype(api.GetVersion))sym("ncclGetVersion");
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.ReduceScatter &&
             api.AllGather && api.GetErrorString;
    if (!api.ok) api.error = "libnccl.so.2 lacks a required symbol";
  });
  return api;
}

}  // namespace b2
