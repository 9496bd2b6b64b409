// Multi-GPU exchange step of a sharded fused operator: an NCCL all-reduce of the outputs that hold per-rank partials.
//
// A kernel compiled with shard_world > 1 works on its rank's slice of the leading axis.  Outputs of reductions over
// that axis are partials (akgb_tensor_desc.shard_kind = AKGB_PARTIAL_*); everything else needs no exchange.  The
// reference has no multi-GPU path for fused operators (one kernel, one device: akg-mlir/python/akg_mlir/utils/
// code_template.py:181); this file is the exchange the sharded launch adds.  NCCL is resolved at run time from the
// library already in the process (PyTorch's) or the system one, so the kernel library itself has no link-time
// dependency on it.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstring>
#include <mutex>
#include <string>

#include "../../include/akgb.h"
#include "kernels.hpp"

namespace akgb {
namespace {

// The handful of NCCL declarations this file needs (public API of nccl.h, stable across 2.x).
typedef struct ncclComm* ncclComm_t;
struct NcclUniqueId { char internal[128]; };
enum { kNcclSuccess = 0 };
enum NcclType { kNcclInt8 = 0, kNcclInt32 = 2, kNcclInt64 = 4, kNcclFloat16 = 6, kNcclFloat32 = 7, kNcclFloat64 = 8, kNcclBfloat16 = 9 };
enum NcclOp { kNcclSum = 0, kNcclProd = 1, kNcclMax = 2, kNcclMin = 3 };

struct Nccl {
  bool ok = false;
  int (*GetUniqueId)(NcclUniqueId*) = nullptr;
  int (*CommInitRank)(ncclComm_t*, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
};

Nccl& nccl() {
  static Nccl n;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = nullptr;
    for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
      h = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (h) break;
    }
    if (!h) return;
    bool all = true;
    auto sym = [&](const char* s) {
      void* p = dlsym(h, s);
      all = all && p != nullptr;
      return p;
    };
    n.GetUniqueId = reinterpret_cast<decltype(n.GetUniqueId)>(sym("ncclGetUniqueId"));
    n.CommInitRank = reinterpret_cast<decltype(n.CommInitRank)>(sym("ncclCommInitRank"));
    n.CommDestroy = reinterpret_cast<decltype(n.CommDestroy)>(sym("ncclCommDestroy"));
    n.AllReduce = reinterpret_cast<decltype(n.AllReduce)>(sym("ncclAllReduce"));
    n.GroupStart = reinterpret_cast<decltype(n.GroupStart)>(sym("ncclGroupStart"));
    n.GroupEnd = reinterpret_cast<decltype(n.GroupEnd)>(sym("ncclGroupEnd"));
    n.GetErrorString = reinterpret_cast<decltype(n.GetErrorString)>(sym("ncclGetErrorString"));
    n.ok = all;
  });
  return n;
}

akgb_status nccl_fail(int rc, const char* what) {
  Nccl& n = nccl();
  set_last_error((std::string(what) + ": " + (n.GetErrorString ? n.GetErrorString(rc) : "NCCL error")).c_str());
  return AKGB_CUDA_ERROR;
}

int nccl_type(int dtype) {
  switch (dtype) {
    case AKGB_FLOAT32: return kNcclFloat32;
    case AKGB_FLOAT16: return kNcclFloat16;
    case AKGB_BFLOAT16: return kNcclBfloat16;
    case AKGB_FLOAT64: return kNcclFloat64;
    case AKGB_INT32: return kNcclInt32;
    case AKGB_INT64: return kNcclInt64;
    case AKGB_INT8: case AKGB_BOOL: return kNcclInt8;
    default: return -1;
  }
}

}  // namespace
}  // namespace akgb

using namespace akgb;

struct akgb_comm {
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1, device = 0;
  bool owned = false;
};

extern "C" {

akgb_status akgb_comm_unique_id(void* id, size_t cap) {
  if (!id || cap < AKGB_COMM_ID_BYTES) {
    set_last_error("akgb_comm_unique_id: buffer of AKGB_COMM_ID_BYTES bytes required");
    return AKGB_INVALID_ARG;
  }
  Nccl& n = nccl();
  if (!n.ok) {
    set_last_error("NCCL (libnccl.so.2) could not be loaded");
    return AKGB_UNSUPPORTED;
  }
  NcclUniqueId u;
  const int rc = n.GetUniqueId(&u);
  if (rc != kNcclSuccess) return nccl_fail(rc, "ncclGetUniqueId");
  std::memcpy(id, &u, sizeof(u));
  return AKGB_OK;
}

akgb_status akgb_comm_create(const void* id, int32_t rank, int32_t world, int32_t device, akgb_comm** out) {
  if (!id || !out || world < 1 || rank < 0 || rank >= world) {
    set_last_error("akgb_comm_create: bad arguments");
    return AKGB_INVALID_ARG;
  }
  Nccl& n = nccl();
  if (!n.ok) {
    set_last_error("NCCL (libnccl.so.2) could not be loaded");
    return AKGB_UNSUPPORTED;
  }
  if (device >= 0) {
    const cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) {
      set_last_error((std::string("cudaSetDevice: ") + cudaGetErrorString(e)).c_str());
      return AKGB_CUDA_ERROR;
    }
  } else {
    cudaGetDevice(&device);
  }
  NcclUniqueId u;
  std::memcpy(&u, id, sizeof(u));
  ncclComm_t c = nullptr;
  const int rc = n.CommInitRank(&c, world, u, rank);
  if (rc != kNcclSuccess) return nccl_fail(rc, "ncclCommInitRank");
  akgb_comm* k = new akgb_comm;
  k->comm = c;
  k->rank = rank;
  k->world = world;
  k->device = device;
  k->owned = true;
  *out = k;
  return AKGB_OK;
}

akgb_status akgb_comm_wrap(void* nccl_comm, int32_t rank, int32_t world, akgb_comm** out) {
  if (!nccl_comm || !out || world < 1 || rank < 0 || rank >= world) {
    set_last_error("akgb_comm_wrap: bad arguments");
    return AKGB_INVALID_ARG;
  }
  if (!nccl().ok) {
    set_last_error("NCCL (libnccl.so.2) could not be loaded");
    return AKGB_UNSUPPORTED;
  }
  akgb_comm* k = new akgb_comm;
  k->comm = static_cast<ncclComm_t>(nccl_comm);
  k->rank = rank;
  k->world = world;
  cudaGetDevice(&k->device);
  k->owned = false;
  *out = k;
  return AKGB_OK;
}

void akgb_comm_destroy(akgb_comm* c) {
  if (!c) return;
  if (c->owned && c->comm) nccl().CommDestroy(c->comm);
  delete c;
}

akgb_status akgb_allreduce_partials(const akgb_kernel* k, akgb_comm* c, void* const* tensors, void* stream) {
  if (!k || !c || !tensors) {
    set_last_error("akgb_allreduce_partials: null argument");
    return AKGB_INVALID_ARG;
  }
  const int n = akgb_num_tensors(k);
  Nccl& lib = nccl();
  int pending = 0;
  for (int i = 0; i < n; ++i) {
    akgb_tensor_desc d;
    if (akgb_tensor_info(k, i, &d) != AKGB_OK) return AKGB_INVALID_ARG;
    if (d.shard_kind < AKGB_PARTIAL_SUM) continue;
    int op;
    switch (d.shard_kind) {
      case AKGB_PARTIAL_SUM: op = kNcclSum; break;
      case AKGB_PARTIAL_MAX: op = kNcclMax; break;
      case AKGB_PARTIAL_MIN: op = kNcclMin; break;
      case AKGB_PARTIAL_PROD: op = kNcclProd; break;
      default: set_last_error("unknown shard kind"); return AKGB_INVALID_ARG;
    }
    const int ty = nccl_type(d.dtype);
    if (ty < 0) {
      set_last_error("akgb_allreduce_partials: element type has no NCCL counterpart");
      return AKGB_UNSUPPORTED;
    }
    size_t count = 1;
    for (int r = 0; r < d.rank; ++r) count *= (size_t)d.shape[r];
    if (pending++ == 0) lib.GroupStart();
    const int rc = lib.AllReduce(tensors[i], tensors[i], count, ty, op, c->comm, static_cast<cudaStream_t>(stream));
    if (rc != kNcclSuccess) {
      lib.GroupEnd();
      return nccl_fail(rc, "ncclAllReduce");
    }
  }
  if (pending) {
    const int rc = lib.GroupEnd();
    if (rc != kNcclSuccess) return nccl_fail(rc, "ncclGroupEnd");
  }
  return AKGB_OK;
}

akgb_status akgb_launch_sharded(akgb_kernel* k, akgb_comm* c, void* const* tensors, void* workspace,
                                size_t workspace_bytes, void* stream) {
  const akgb_status st = akgb_launch(k, tensors, workspace, workspace_bytes, stream);
  if (st != AKGB_OK) return st;
  return akgb_allreduce_partials(k, c, tensors, stream);
}

}  // extern "C"
