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
  // exchange over peer memory (k_exchange.cu)
  void* local_buf = nullptr;               // this rank's exchange buffer (cudaMalloc)
  void* peer_buf[kExchangeMaxRanks] = {};  // every rank's buffer as mapped into this process
  bool peers_ready = false;
  bool in_reduction = true;                // reductions complete the exchange in their own launch where they can
  double timeout_ms = 1000.0;
  int clock_khz = 0;
};

namespace {
akgb_status cuda_fail_comm(cudaError_t e, const char* what) {
  set_last_error((std::string(what) + ": " + cudaGetErrorString(e)).c_str());
  return AKGB_CUDA_ERROR;
}
akgb_status ensure_local_buffer(akgb_comm* c) {
  if (c->local_buf) return AKGB_OK;
  cudaError_t e = cudaSetDevice(c->device);
  if (e != cudaSuccess) return cuda_fail_comm(e, "cudaSetDevice");
  e = cudaMalloc(&c->local_buf, kExchangeBytes);
  if (e != cudaSuccess) return cuda_fail_comm(e, "cudaMalloc (exchange buffer)");
  e = cudaMemset(c->local_buf, 0, kExchangeBytes);
  if (e != cudaSuccess) return cuda_fail_comm(e, "cudaMemset (exchange buffer)");
  return AKGB_OK;
}
}  // namespace

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
  if (c->local_buf) {
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    for (int q = 0; q < c->world && q < kExchangeMaxRanks; ++q)
      if (c->peer_buf[q] && c->peer_buf[q] != c->local_buf) cudaIpcCloseMemHandle(c->peer_buf[q]);
    cudaFree(c->local_buf);
  }
  if (c->owned && c->comm) nccl().CommDestroy(c->comm);
  delete c;
}

akgb_status akgb_comm_exchange_handle(akgb_comm* c, void* handle, size_t cap) {
  if (!c || !handle || cap < AKGB_COMM_HANDLE_BYTES) {
    set_last_error("akgb_comm_exchange_handle: buffer of AKGB_COMM_HANDLE_BYTES bytes required");
    return AKGB_INVALID_ARG;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) <= AKGB_COMM_HANDLE_BYTES, "handle size");
  const akgb_status st = ensure_local_buffer(c);
  if (st != AKGB_OK) return st;
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, c->local_buf);
  if (e != cudaSuccess) return cuda_fail_comm(e, "cudaIpcGetMemHandle");
  std::memset(handle, 0, AKGB_COMM_HANDLE_BYTES);
  std::memcpy(handle, &h, sizeof(h));
  return AKGB_OK;
}

akgb_status akgb_comm_attach_peers(akgb_comm* c, const void* handles, size_t bytes) {
  if (!c) {
    set_last_error("akgb_comm_attach_peers: null communicator");
    return AKGB_INVALID_ARG;
  }
  if (c->world > kExchangeMaxRanks) {
    set_last_error("akgb_comm_attach_peers: more than 8 ranks");
    return AKGB_UNSUPPORTED;
  }
  const akgb_status st = ensure_local_buffer(c);
  if (st != AKGB_OK) return st;
  if (!handles) {
    // loop-back: every slot owner is this process (single-rank use, and the bounded-wait test: with world > 1 the other
    // ranks' flags are never raised)
    for (int q = 0; q < c->world; ++q) c->peer_buf[q] = c->local_buf;
    c->peers_ready = true;
    return AKGB_OK;
  }
  if (bytes < (size_t)c->world * AKGB_COMM_HANDLE_BYTES) {
    set_last_error("akgb_comm_attach_peers: one handle of AKGB_COMM_HANDLE_BYTES bytes per rank required");
    return AKGB_INVALID_ARG;
  }
  for (int q = 0; q < c->world; ++q) {
    if (q == c->rank) {
      c->peer_buf[q] = c->local_buf;
      continue;
    }
    cudaIpcMemHandle_t h;
    std::memcpy(&h, static_cast<const char*>(handles) + (size_t)q * AKGB_COMM_HANDLE_BYTES, sizeof(h));
    const cudaError_t e = cudaIpcOpenMemHandle(&c->peer_buf[q], h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      c->peer_buf[q] = nullptr;
      return cuda_fail_comm(e, "cudaIpcOpenMemHandle");  // peers_ready stays false: NCCL carries the exchange
    }
  }
  c->peers_ready = true;
  return AKGB_OK;
}

akgb_status akgb_comm_create_local(int32_t rank, int32_t world, int32_t device, akgb_comm** out) {
  if (!out || world < 1 || world > kExchangeMaxRanks || rank < 0 || rank >= world) {
    set_last_error("akgb_comm_create_local: bad arguments (1..8 ranks)");
    return AKGB_INVALID_ARG;
  }
  if (device < 0) cudaGetDevice(&device);
  akgb_comm* k = new akgb_comm;
  k->rank = rank;
  k->world = world;
  k->device = device;
  *out = k;
  return AKGB_OK;
}

akgb_status akgb_comm_set_peer_exchange(akgb_comm* c, int32_t enabled) {
  if (!c) {
    set_last_error("akgb_comm_set_peer_exchange: null communicator");
    return AKGB_INVALID_ARG;
  }
  if (enabled) {
    for (int q = 0; q < c->world; ++q)
      if (c->world > kExchangeMaxRanks || !c->peer_buf[q]) {
        set_last_error("akgb_comm_set_peer_exchange: the peers' buffers are not attached");
        return AKGB_INVALID_ARG;
      }
  }
  if (c->local_buf && device_exchange_failed(c->device)) {
    // after a wait that ran out the ranks' call counters may differ: start again from call 0 (every rank does this,
    // then the ranks synchronise before their next sharded launch)
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    const cudaError_t e = cudaMemset(c->local_buf, 0, kExchangeBytes);
    if (e != cudaSuccess) return cuda_fail_comm(e, "cudaMemset (exchange buffer)");
  }
  device_exchange_set_failed(c->device, false);
  c->peers_ready = enabled != 0;
  return AKGB_OK;
}

akgb_status akgb_comm_set_exchange_in_reduction(akgb_comm* c, int32_t enabled) {
  if (!c) {
    set_last_error("akgb_comm_set_exchange_in_reduction: null communicator");
    return AKGB_INVALID_ARG;
  }
  c->in_reduction = enabled != 0;
  return AKGB_OK;
}

akgb_status akgb_comm_set_timeout_ms(akgb_comm* c, double ms) {
  if (!c || !(ms > 0.0)) {
    set_last_error("akgb_comm_set_timeout_ms: bad arguments");
    return AKGB_INVALID_ARG;
  }
  c->timeout_ms = ms;
  return AKGB_OK;
}

namespace {
akgb_status refuse_after_timeout(const akgb_comm* c) {
  if (!c->peers_ready || c->world <= 1 || !device_exchange_failed(c->device)) return AKGB_OK;
  set_last_error("a peer-memory exchange on this device gave up earlier, the ranks' call counters may disagree: call "
                 "akgb_comm_set_peer_exchange on ALL ranks (1 to restart the path, 0 to continue over NCCL) and "
                 "synchronise the ranks before the next sharded launch");
  return AKGB_DEVICE_TIMEOUT;
}
void fill_exchange_base(akgb_comm* c, FinishExchange* fx) {
  for (int q = 0; q < c->world; ++q) fx->peer[q] = c->peer_buf[q];
  fx->rank = c->rank;
  fx->world = c->world;
  if (c->clock_khz == 0) {  // queried once: this attribute is slow to read
    int khz = 0;
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, c->device);
    c->clock_khz = khz > 0 ? khz : 1500000;
  }
  fx->limit_cycles = (long long)(c->timeout_ms * c->clock_khz);
}
}  // namespace

int32_t akgb_sharded_exchange_kind(const akgb_kernel* k, const akgb_comm* c) {
  if (!k || !c || c->world <= 1) return AKGB_EXCHANGE_NONE;
  if (kernel_is_staged(k)) {  // the least direct way any of the stages' exchanges goes
    int32_t kind = AKGB_EXCHANGE_NONE;
    for (int i = 0; const akgb_kernel* sk = kernel_stage(k, i); ++i) {
      const int32_t sk_kind = akgb_sharded_exchange_kind(sk, c);
      if (sk_kind != AKGB_EXCHANGE_NONE && (kind == AKGB_EXCHANGE_NONE || sk_kind < kind)) kind = sk_kind;
    }
    return kind;
  }
  const int n = akgb_num_tensors(k);
  bool any = false, all_small_f32 = true;
  size_t total = 0;
  int segs = 0;
  for (int i = 0; i < n; ++i) {
    akgb_tensor_desc d;
    if (akgb_tensor_info(k, i, &d) != AKGB_OK || d.shard_kind < AKGB_PARTIAL_SUM) continue;
    any = true;
    size_t count = 1;
    for (int r = 0; r < d.rank; ++r) count *= (size_t)d.shape[r];
    total += count;
    ++segs;
    if (d.dtype != AKGB_FLOAT32) all_small_f32 = false;
  }
  if (!any) return AKGB_EXCHANGE_NONE;
  if (!c->peers_ready) return AKGB_EXCHANGE_NCCL;
  if (c->in_reduction && kernel_exchange_fusable(k)) return AKGB_EXCHANGE_IN_REDUCTION;
  return all_small_f32 && total <= (size_t)kExchangeSlotElems && segs <= kExchangeMaxSegs ? AKGB_EXCHANGE_PEER_KERNEL
                                                                                         : AKGB_EXCHANGE_NCCL;
}

akgb_status akgb_allreduce_partials(const akgb_kernel* k, akgb_comm* c, void* const* tensors, void* stream) {
  if (!k || !c || !tensors) {
    set_last_error("akgb_allreduce_partials: null argument");
    return AKGB_INVALID_ARG;
  }
  {
    const akgb_status rs = refuse_after_timeout(c);
    if (rs != AKGB_OK) return rs;
  }
  const int n = akgb_num_tensors(k);
  Nccl& lib = nccl();
  int pending = 0;
  ExchangeArgs xa;
  size_t xtotal = 0;
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
    size_t count = 1;
    for (int r = 0; r < d.rank; ++r) count *= (size_t)d.shape[r];
    if (c->peers_ready && d.dtype == AKGB_FLOAT32 && xa.n_seg < kExchangeMaxSegs &&
        xtotal + count <= (size_t)kExchangeSlotElems) {
      // small float32 partials: they all travel in one kernel over the ranks' mapped buffers (after this loop)
      xa.seg_count[xa.n_seg] = (int)count;
      xa.seg_op[xa.n_seg] = (int)(op == kNcclSum ? RedOp::Sum : op == kNcclMax ? RedOp::Max : op == kNcclMin ? RedOp::Min : RedOp::Prod);
      xa.seg_ptr[xa.n_seg] = static_cast<float*>(tensors[i]);
      ++xa.n_seg;
      xtotal += count;
      continue;
    }
    if (!c->comm) {
      set_last_error("akgb_allreduce_partials: this communicator has no NCCL handle and the tensor does not fit the "
                     "peer-memory exchange (float32, at most 16384 elements, peers attached)");
      return AKGB_UNSUPPORTED;
    }
    const int ty = nccl_type(d.dtype);
    if (ty < 0) {
      set_last_error("akgb_allreduce_partials: element type has no NCCL counterpart");
      return AKGB_UNSUPPORTED;
    }
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
  if (xa.n_seg) {
    FinishExchange base;
    fill_exchange_base(c, &base);
    for (int q = 0; q < c->world; ++q) xa.peer[q] = base.peer[q];
    xa.rank = c->rank;
    xa.world = c->world;
    xa.limit_cycles = base.limit_cycles;
    xa.err = kernel_error_word(const_cast<akgb_kernel*>(k));
    if (!xa.err) return AKGB_CUDA_ERROR;
    const cudaError_t e = exchange_allreduce(xa, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail_comm(e, "exchange_allreduce");
  }
  return AKGB_OK;
}

akgb_status akgb_launch_sharded(akgb_kernel* k, akgb_comm* c, void* const* tensors, void* workspace,
                                size_t workspace_bytes, void* stream) {
  if (!k || !c || !tensors) {
    set_last_error("akgb_launch_sharded: null argument");
    return AKGB_INVALID_ARG;
  }
  if (kernel_is_staged(k)) return launch_staged(k, c, tensors, workspace, workspace_bytes, stream);
  if (c->world > 1 && c->peers_ready && c->in_reduction) {
    const akgb_status rs = refuse_after_timeout(c);
    if (rs != AKGB_OK) return rs;
    // a reduction that produces all the partial outputs completes their exchange in its own launch
    FinishExchange base;
    fill_exchange_base(c, &base);
    bool fused = false;
    const akgb_status fs = launch_with_exchange(k, base, tensors, workspace, workspace_bytes, stream, &fused);
    if (fs != AKGB_OK || fused) return fs;
  }
  const akgb_status st = akgb_launch(k, tensors, workspace, workspace_bytes, stream);
  if (st != AKGB_OK) return st;
  return akgb_allreduce_partials(k, c, tensors, stream);
}

}  // extern "C"
