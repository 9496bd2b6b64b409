// One-shot all-reduce of small partial results over peer memory (NVLink / NVSwitch), for the exchange step of a
// sharded reduction: every rank stores its values into a slot of every rank's exchange buffer, raises a flag there, waits
// for the flags of all ranks in its own buffer and folds the slots in rank order -- one kernel, one NVLink crossing per
// value, the same bits on every rank.  Used instead of NCCL when the ranks' buffers are mapped into one another
// (akgb_comm_attach_peers) and the tensor fits a slot; NCCL remains the general path.
//
// Every wait is bounded: a rank whose peers do not arrive within the limit sets bit 8 of the device error word and
// returns without touching its output, and the context stays usable.  Only plain peer stores and loads are used (no
// multimem, no tensor-map copies from peer memory).
#include <cuda_runtime.h>

#include <cstdint>

#include "common.cuh"
#include "kernels.hpp"

namespace akgb {
namespace {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ float fold(int op, float a, float b) {
  return op == (int)RedOp::Sum ? SumOp::apply(a, b) : op == (int)RedOp::Max ? MaxOp::apply(a, b)
       : op == (int)RedOp::Min ? MinOp::apply(a, b) : ProdOp::apply(a, b);
}

__global__ void __launch_bounds__(256) exchange_allreduce_kernel(ExchangeArgs a) {
  const int tid = threadIdx.x, cta = blockIdx.x;
  // The number of this call lives in the rank's own buffer (every rank makes the same calls in the same order, so the
  // counters agree); keeping it on the device lets a captured graph replay the launch.
  uint32_t* counter = exchange_counter(a.peer[a.rank]);
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(counter) + 1u;
  const int par = (int)(epoch & 1u);
  int total = 0;
  for (int g = 0; g < a.n_seg; ++g) total += a.seg_count[g];
  const int chunk = (total + gridDim.x - 1) / gridDim.x;
  const int lo = cta * chunk, hi = min(total, lo + chunk);
  // position i of the slot -> (segment, element)
  auto locate = [&](int i, int* seg) {
    int g = 0;
    while (g + 1 < a.n_seg && i >= a.seg_count[g]) i -= a.seg_count[g++];
    *seg = g;
    return i;
  };
  // 1. my values into slot [par][my rank] of every rank (peer stores)
  for (int i = lo + tid; i < hi; i += blockDim.x) {
    int g;
    const int e = locate(i, &g);
    const float v = a.seg_ptr[g][e];
    for (int q = 0; q < a.world; ++q) exchange_slot(a.peer[q], par, a.rank)[i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (tid < a.world) st_release_sys(exchange_flag(a.peer[tid], par, a.rank, cta), epoch);
  // 2. every rank's flag in MY buffer, with a limit
  int timed_out = 0;
  if (tid < a.world) {
    const uint32_t* f = exchange_flag(a.peer[a.rank], par, tid, cta);
    const long long t0 = clock64();
    while (ld_acquire_sys(f) != epoch) {
      if (clock64() - t0 > a.limit_cycles) {
        timed_out = 1;
        break;
      }
      __nanosleep(64);
    }
  }
  const bool failed = __syncthreads_or(timed_out) != 0;
  if (failed) {
    if (tid == 0) atomicOr(a.err, 256u);
  } else {
    // 3. fold in rank order: the same bits everywhere
    for (int i = lo + tid; i < hi; i += blockDim.x) {
      int g;
      const int e = locate(i, &g);
      float v = exchange_slot(a.peer[a.rank], par, 0)[i];
      for (int q = 1; q < a.world; ++q) v = fold(a.seg_op[g], v, exchange_slot(a.peer[a.rank], par, q)[i]);
      a.seg_ptr[g][e] = v;
    }
  }
  // the last CTA to get here closes the call (every CTA has read the counter by then)
  __syncthreads();
  if (tid == 0) {
    uint32_t* ticket = counter + 1;
    if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
      *ticket = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(counter) = epoch;
    }
  }
}

}  // namespace

cudaError_t exchange_allreduce(const ExchangeArgs& a, cudaStream_t s) {
  int total = 0;
  for (int g = 0; g < a.n_seg; ++g) total += a.seg_count[g];
  if (total <= 0) return cudaSuccess;
  if (total > kExchangeSlotElems || a.n_seg > kExchangeMaxSegs || a.world < 1 || a.world > kExchangeMaxRanks)
    return cudaErrorInvalidValue;
  const int ctas = std::min(kExchangeMaxCtas, (total + 1023) / 1024);
  exchange_allreduce_kernel<<<ctas, 256, 0, s>>>(a);
  return cudaGetLastError();
}

}  // namespace akgb
