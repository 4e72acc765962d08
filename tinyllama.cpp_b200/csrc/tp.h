// Tensor parallelism inside one node: Megatron-style sharding of the packed weights and the two
// all-reduces per layer over NCCL (loaded at run time from the process's libnccl.so.2, so the
// library itself links only the CUDA runtime). The reference has no tensor parallelism; its MPI
// coordinator (distributed_coordinator.cpp) only routes whole requests.
#pragma once
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstdint>
#include <stdexcept>
#include <string>

namespace b200 {

// Contiguous share [begin, end) of `units` for rank r of n: the first (units % n) ranks get one extra.
inline void tp_share(int64_t units, int n, int r, int64_t& begin, int64_t& end) {
  const int64_t base = units / n, extra = units % n;
  begin = r * base + (r < extra ? r : extra);
  end = begin + base + (r < extra ? 1 : 0);
}

struct Nccl {
  typedef struct { char internal[128]; } UniqueId;
  int (*GetUniqueId)(UniqueId*) = nullptr;
  int (*CommInitRank)(void**, int, UniqueId, int) = nullptr;
  int (*CommDestroy)(void*) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  void* handle = nullptr;
  static constexpr int kFloat32 = 7, kInt32 = 2, kInt8 = 0, kSum = 0, kMin = 3;  // ncclFloat32, ncclInt32, ncclInt8; ncclSum, ncclMin

  static Nccl& get() {
    static Nccl n;
    if (!n.handle) {
      void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
      if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
      if (!h) throw std::runtime_error(std::string("cannot load libnccl: ") + dlerror());
      auto sym = [&](const char* name) {
        void* p = dlsym(h, name);
        if (!p) throw std::runtime_error(std::string("libnccl lacks ") + name);
        return p;
      };
      // resolve into a scratch copy: the singleton is published only when every symbol is there
      Nccl t;
      t.GetUniqueId = reinterpret_cast<decltype(t.GetUniqueId)>(sym("ncclGetUniqueId"));
      t.CommInitRank = reinterpret_cast<decltype(t.CommInitRank)>(sym("ncclCommInitRank"));
      t.CommDestroy = reinterpret_cast<decltype(t.CommDestroy)>(sym("ncclCommDestroy"));
      t.AllReduce = reinterpret_cast<decltype(t.AllReduce)>(sym("ncclAllReduce"));
      t.AllGather = reinterpret_cast<decltype(t.AllGather)>(sym("ncclAllGather"));
      t.GetErrorString = reinterpret_cast<decltype(t.GetErrorString)>(sym("ncclGetErrorString"));
      t.handle = h;
      n = t;
    }
    return n;
  }
  void check(int rc, const char* what) {
    if (rc != 0) throw std::runtime_error(std::string(what) + ": " + (GetErrorString ? GetErrorString(rc) : "NCCL error"));
  }
};

}  // namespace b200
