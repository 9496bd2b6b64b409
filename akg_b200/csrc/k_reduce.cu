// Reduction class: column (reduce-Y), global (reduce-ALL) and plain row
// (reduce-X) reductions of float32 tensors.
//
// Init values and combiners follow the reference lowering
// (akg-mlir/lib/Conversion/MindSporeToLinalg/MindSporeToLinalg.cpp:791-843 and
// :845-901): sum 0, prod 1, max -FLT_MAX, min +FLT_MAX; max/min skip NaN
// operands.  The reference's GPU schedule walks the reduced axis sequentially
// per thread and combines with atomics
// (akg-mlir/lib/Dialect/Affine/Analysis/GpuTemplateTilingSolver.cpp:458-542);
// here every stage is a fixed tree, so results do not depend on scheduling:
// per-thread strided partials -> shared-memory tree -> per-CTA partial in
// scratch -> a small second kernel folds the partials in a fixed order.
#include <algorithm>
#include <cstdio>
#include <mutex>

#include "../../include/akgb.h"
#include "common.cuh"
#include "kernels.hpp"

namespace akgb {
namespace {

constexpr int kColTx = 32;   // threads across columns (each owns a float4)
constexpr int kColTy = 8;    // threads across rows
constexpr int kColTile = kColTx * 4;

inline int64_t col_row_splits(int64_t red, int64_t inner, int sm_count) {
  const int64_t col_tiles = (inner + kColTile - 1) / kColTile;
  int64_t want = ((int64_t)sm_count * 8 + col_tiles - 1) / col_tiles;
  // each split should own at least a few sweeps of kColTy rows
  const int64_t max_splits = std::max<int64_t>(1, red / (kColTy * 4));
  return std::max<int64_t>(1, std::min(want, max_splits));
}

template <class Op>
__device__ __forceinline__ float4 apply4(float4 a, float4 b) {
  return make_float4(Op::apply(a.x, b.x), Op::apply(a.y, b.y), Op::apply(a.z, b.z), Op::apply(a.w, b.w));
}

// x[red, inner] -> partial[split, inner]; VEC: inner % 4 == 0 and 16-byte aligned rows
template <class Op, bool VEC>
__global__ void __launch_bounds__(kColTx* kColTy) reduce_col_f32_kernel(const float* __restrict__ x,
                                                                        float* __restrict__ partial, int64_t red,
                                                                        int64_t inner, int64_t rows_per_split) {
  __shared__ float4 sm[kColTy][kColTx];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int64_t col = ((int64_t)blockIdx.x * kColTx + tx) * 4;
  const int64_t r0 = (int64_t)blockIdx.y * rows_per_split;
  const int64_t r1 = min(red, r0 + rows_per_split);
  const float id = Op::identity();
  float4 acc0 = make_float4(id, id, id, id), acc1 = acc0, acc2 = acc0, acc3 = acc0;
  if (VEC) {
    if (col < inner) {
      const float* base = x + col;
      int64_t r = r0 + ty;
      for (; r + 3 * kColTy < r1; r += 4 * kColTy) {
        const float4 a = ld_stream_f4(base + r * inner);
        const float4 b = ld_stream_f4(base + (r + kColTy) * inner);
        const float4 c = ld_stream_f4(base + (r + 2 * kColTy) * inner);
        const float4 d = ld_stream_f4(base + (r + 3 * kColTy) * inner);
        acc0 = apply4<Op>(acc0, a);
        acc1 = apply4<Op>(acc1, b);
        acc2 = apply4<Op>(acc2, c);
        acc3 = apply4<Op>(acc3, d);
      }
      for (; r < r1; r += kColTy) acc0 = apply4<Op>(acc0, ld_stream_f4(base + r * inner));
    }
  } else {
    for (int64_t r = r0 + ty; r < r1; r += kColTy) {
      const float* row = x + r * inner;
      float4 a = make_float4(id, id, id, id);
      if (col + 0 < inner) a.x = row[col + 0];
      if (col + 1 < inner) a.y = row[col + 1];
      if (col + 2 < inner) a.z = row[col + 2];
      if (col + 3 < inner) a.w = row[col + 3];
      acc0 = apply4<Op>(acc0, a);
    }
  }
  acc0 = apply4<Op>(apply4<Op>(acc0, acc1), apply4<Op>(acc2, acc3));
  sm[ty][tx] = acc0;
  __syncthreads();
#pragma unroll
  for (int h = kColTy / 2; h > 0; h >>= 1) {
    if (ty < h) sm[ty][tx] = apply4<Op>(sm[ty][tx], sm[ty + h][tx]);
    __syncthreads();
  }
  if (ty == 0) {
    const float4 r = sm[0][tx];
    float* o = partial + (int64_t)blockIdx.y * inner + col;
    if (col + 0 < inner) o[0] = r.x;
    if (col + 1 < inner) o[1] = r.y;
    if (col + 2 < inner) o[2] = r.z;
    if (col + 3 < inner) o[3] = r.w;
  }
}

// Column reduction with Op1 and, in the same pass over x, a reduction of every element with Op2
// (e.g. column sums and the global maximum of one tensor): x is read from HBM once.
template <class Op1, class Op2>
__global__ void __launch_bounds__(kColTx* kColTy) reduce_col_dual_f32_kernel(const float* __restrict__ x,
                                                                             float* __restrict__ partial,
                                                                             float* __restrict__ partial2, int64_t red,
                                                                             int64_t inner, int64_t rows_per_split) {
  __shared__ float4 sm[kColTy][kColTx];
  __shared__ float red2[32];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int64_t col = ((int64_t)blockIdx.x * kColTx + tx) * 4;
  const int64_t r0 = (int64_t)blockIdx.y * rows_per_split;
  const int64_t r1 = min(red, r0 + rows_per_split);
  const float id = Op1::identity(), id2 = Op2::identity();
  float4 acc0 = make_float4(id, id, id, id), acc1 = acc0, acc2 = acc0, acc3 = acc0;
  float4 b0 = make_float4(id2, id2, id2, id2), b1 = b0;
  if (col < inner) {
    const float* base = x + col;
    int64_t r = r0 + ty;
    for (; r + 3 * kColTy < r1; r += 4 * kColTy) {
      const float4 a = ld_stream_f4(base + r * inner);
      const float4 b = ld_stream_f4(base + (r + kColTy) * inner);
      const float4 c = ld_stream_f4(base + (r + 2 * kColTy) * inner);
      const float4 d = ld_stream_f4(base + (r + 3 * kColTy) * inner);
      acc0 = apply4<Op1>(acc0, a);
      acc1 = apply4<Op1>(acc1, b);
      acc2 = apply4<Op1>(acc2, c);
      acc3 = apply4<Op1>(acc3, d);
      b0 = apply4<Op2>(b0, apply4<Op2>(a, b));
      b1 = apply4<Op2>(b1, apply4<Op2>(c, d));
    }
    for (; r < r1; r += kColTy) {
      const float4 a = ld_stream_f4(base + r * inner);
      acc0 = apply4<Op1>(acc0, a);
      b0 = apply4<Op2>(b0, a);
    }
  }
  acc0 = apply4<Op1>(apply4<Op1>(acc0, acc1), apply4<Op1>(acc2, acc3));
  sm[ty][tx] = acc0;
  __syncthreads();
#pragma unroll
  for (int h = kColTy / 2; h > 0; h >>= 1) {
    if (ty < h) sm[ty][tx] = apply4<Op1>(sm[ty][tx], sm[ty + h][tx]);
    __syncthreads();
  }
  if (ty == 0) {
    const float4 r = sm[0][tx];
    float* o = partial + (int64_t)blockIdx.y * inner + col;
    if (col + 0 < inner) o[0] = r.x;
    if (col + 1 < inner) o[1] = r.y;
    if (col + 2 < inner) o[2] = r.z;
    if (col + 3 < inner) o[3] = r.w;
  }
  // second reduction: fold the CTA's values, one partial per CTA
  b0 = apply4<Op2>(b0, b1);
  float s2 = Op2::apply(Op2::apply(b0.x, b0.y), Op2::apply(b0.z, b0.w));
  s2 = warp_reduce<Op2>(s2);
  const int tid = ty * kColTx + tx, lane = tid & 31, warp = tid >> 5;
  if (lane == 0) red2[warp] = s2;
  __syncthreads();
  if (warp == 0) {
    float v = lane < (kColTx * kColTy) / 32 ? red2[lane] : id2;
    v = warp_reduce<Op2>(v);
    if (lane == 0) partial2[(int64_t)blockIdx.y * gridDim.x + blockIdx.x] = v;
  }
}

// Fold of column c over the row splits, in split order.  The loads of eight splits are issued together (they do not
// depend on one another), the combines stay one after the other, so the result has the bits of the plain loop.
template <class Op>
__device__ __forceinline__ float fold_splits(const float* __restrict__ partial, int64_t splits, int64_t inner, int64_t c) {
  float a = Op::identity();
  const float* p = partial + c;
  int64_t s = 0;
  for (; s + 8 <= splits; s += 8) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = __ldcg(p + (s + u) * inner);
#pragma unroll
    for (int u = 0; u < 8; ++u) a = Op::apply(a, v[u]);
  }
  for (; s < splits; ++s) a = Op::apply(a, __ldcg(p + s * inner));
  return a;
}

// partial[splits, inner] -> out[inner], fixed order
template <class Op>
__global__ void __launch_bounds__(256) reduce_col_finish_kernel(const float* __restrict__ partial,
                                                                float* __restrict__ out, int64_t splits,
                                                                int64_t inner) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= inner) return;
  out[c] = fold_splits<Op>(partial, splits, inner, c);
}

// x[n] -> partial[grid]
template <class Op, bool VEC>
__global__ void __launch_bounds__(256) reduce_all_f32_kernel(const float* __restrict__ x, float* __restrict__ partial,
                                                             int64_t n) {
  __shared__ float red[32];
  const float id = Op::identity();
  float a0 = id, a1 = id, a2 = id, a3 = id;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (VEC) {
    const int64_t n4 = n >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    int64_t i = tid;
    for (; i + 3 * stride < n4; i += 4 * stride) {
      const float4 p = ld_stream_f4(x4 + i), q = ld_stream_f4(x4 + i + stride);
      const float4 r = ld_stream_f4(x4 + i + 2 * stride), t = ld_stream_f4(x4 + i + 3 * stride);
      a0 = Op::apply(a0, Op::apply(Op::apply(p.x, p.y), Op::apply(p.z, p.w)));
      a1 = Op::apply(a1, Op::apply(Op::apply(q.x, q.y), Op::apply(q.z, q.w)));
      a2 = Op::apply(a2, Op::apply(Op::apply(r.x, r.y), Op::apply(r.z, r.w)));
      a3 = Op::apply(a3, Op::apply(Op::apply(t.x, t.y), Op::apply(t.z, t.w)));
    }
    for (; i < n4; i += stride) {
      const float4 p = ld_stream_f4(x4 + i);
      a0 = Op::apply(a0, Op::apply(Op::apply(p.x, p.y), Op::apply(p.z, p.w)));
    }
    for (int64_t j = (n4 << 2) + tid; j < n; j += stride) a1 = Op::apply(a1, x[j]);
  } else {
    for (int64_t j = tid; j < n; j += stride) a0 = Op::apply(a0, x[j]);
  }
  float a = Op::apply(Op::apply(a0, a1), Op::apply(a2, a3));
  a = block_reduce<Op>(a, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = a;
}

template <class Op>
__global__ void __launch_bounds__(1024) reduce_all_finish_kernel(const float* __restrict__ partial,
                                                                 float* __restrict__ out, int n) {
  __shared__ float red[32];
  float a = Op::identity();
  for (int i = threadIdx.x; i < n; i += blockDim.x) a = Op::apply(a, partial[i]);
  a = block_reduce<Op>(a, red);
  if (threadIdx.x == 0) out[0] = a;
}

// x[rows, cols] -> out[rows]; one warp per row
template <class Op>
__global__ void __launch_bounds__(256) reduce_row_f32_kernel(const float* __restrict__ x, float* __restrict__ out,
                                                             int64_t rows, int64_t cols, int vec) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * 8;
  for (int64_t row = warp; row < rows; row += nwarps) {
    const float* xr = x + row * cols;
    float a = Op::identity(), b = Op::identity();
    if (vec) {
      const float4* x4 = reinterpret_cast<const float4*>(xr);
      const int64_t c4 = cols >> 2;
      int64_t i = lane;
      for (; i + 32 < c4; i += 64) {
        const float4 p = ld_stream_f4(x4 + i), q = ld_stream_f4(x4 + i + 32);
        a = Op::apply(a, Op::apply(Op::apply(p.x, p.y), Op::apply(p.z, p.w)));
        b = Op::apply(b, Op::apply(Op::apply(q.x, q.y), Op::apply(q.z, q.w)));
      }
      for (; i < c4; i += 32) {
        const float4 p = ld_stream_f4(x4 + i);
        a = Op::apply(a, Op::apply(Op::apply(p.x, p.y), Op::apply(p.z, p.w)));
      }
    } else {
      for (int64_t i = lane; i < cols; i += 32) a = Op::apply(a, xr[i]);
    }
    a = warp_reduce<Op>(Op::apply(a, b));
    if (lane == 0) out[row] = a;
  }
}

// ---- fold by the finishing CTA, optionally with the exchange over peer memory ------------------------------------
__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// the number of the exchange call in progress on this rank (read early: the load overlaps the fold of the partials)
__device__ __forceinline__ uint32_t exchange_epoch(const FinishExchange& fx) {
  return *reinterpret_cast<volatile uint32_t*>(exchange_counter(fx.peer[fx.rank])) + 1u;
}

// Called by ALL threads of a finishing CTA (any block shape).  Thread `tid` holds value `v` for position `pos` of the
// call's values when `active`.  Stores (value, call number) as one 64-bit word into this rank's slot of every rank's
// buffer, then polls (bounded) the same position of every rank's slot in its own buffer until the word carries this
// call's number, and folds the values in rank order, so that every rank gets the same bits.  No flag and no fence: the
// 8-byte store is single-copy atomic, a word with the right number holds the right value.  Returns false when a wait
// ran out (bit 8 of the error word is set, `v` is unchanged).  The finisher that closes the call (the last of
// fx.finishers) advances the call counter.
template <class Op>
__device__ __forceinline__ bool finish_exchange(const FinishExchange& fx, uint32_t epoch, float& v, bool active, int pos,
                                                int tid) {
  void* own = fx.peer[fx.rank];
  const int par = (int)(epoch & 1u);
  int timed_out = 0;
  if (active) {
    const unsigned long long word = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v);
    for (int q = 0; q < fx.world; ++q) st_relaxed_sys_u64(exchange_tagged(fx.peer[q], par, fx.rank) + pos, word);
    float r = 0.f;
    const long long t0 = clock64();
    for (int q = 0; q < fx.world && !timed_out; ++q) {
      const unsigned long long* src = exchange_tagged(own, par, q) + pos;
      unsigned long long w = ld_relaxed_sys_u64(src);
      while ((uint32_t)(w >> 32) != epoch) {
        if (clock64() - t0 > fx.limit_cycles) {
          timed_out = 1;
          break;
        }
        __nanosleep(20);
        w = ld_relaxed_sys_u64(src);
      }
      const float x = __uint_as_float((uint32_t)w);
      r = q == 0 ? x : Op::apply(r, x);
    }
    if (!timed_out) v = r;
  }
  const bool failed = __syncthreads_or(timed_out) != 0;
  if (tid == 0) {
    if (failed) atomicOr(fx.err, 256u);
    uint32_t* counter = exchange_counter(own);
    uint32_t* ticket = counter + 1;
    if (atomicInc(ticket, (uint32_t)fx.finishers - 1u) == (uint32_t)fx.finishers - 1u) {  // wraps to 0 by itself
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(counter) = epoch;
    }
  }
  return !failed;
}

// true in every thread of exactly one CTA among the `expected` that call this with the same ticket word: the one that
// arrives last.  The caller has written its partials before the call; the last CTA may read everybody's afterwards.
__device__ __forceinline__ bool arrive_last(uint32_t* ticket, unsigned expected, int tid) {
  __shared__ int last;
  __syncthreads();  // every thread's partials are ordered before thread 0's fence (the fence is cumulative)
  if (tid == 0) {
    __threadfence();
    const unsigned t = atomicAdd(ticket, 1u);
    last = t == expected - 1u;
    if (last) *ticket = 0;  // ready for the next launch
    __threadfence();        // the others' partials are read after their arrivals were seen
  }
  __syncthreads();
  return last != 0;
}

// fold of partial[splits, inner] over the splits for the 128 columns of tile `tile`, in split order (the order of
// reduce_col_finish_kernel: same bits), then the exchange, then the store
template <class Op>
__device__ __forceinline__ void finish_col_tile(const float* partial, float* out, int64_t splits, int64_t inner,
                                                int tile, int tid, const FinishExchange& fx) {
  const int64_t c = (int64_t)tile * kColTile + tid;
  const bool active = tid < kColTile && c < inner;
  const uint32_t epoch = fx.world > 1 ? exchange_epoch(fx) : 0u;
  float a = Op::identity();
  if (active) a = fold_splits<Op>(partial, splits, inner, c);
  // when the wait runs out the value stays this rank's own partial (and the error word says so)
  if (fx.world > 1) finish_exchange<Op>(fx, epoch, a, active, fx.slot_off + (int)c, tid);
  if (active) out[c] = a;
}

// fold of partial[n] by a 256-thread CTA in a fixed order, then the exchange of the one value, then the store
template <class Op>
__device__ __forceinline__ void finish_all(const float* partial, float* out, int n, int tid, float* red,
                                           const FinishExchange& fx, int slot_pos) {
  const uint32_t epoch = fx.world > 1 ? exchange_epoch(fx) : 0u;
  float a = Op::identity();
  for (int i = tid; i < n; i += 256) a = Op::apply(a, __ldcg(partial + i));
  // block_reduce by linear thread id (the CTA may be 32x8)
  a = warp_reduce<Op>(a);
  __syncthreads();
  if ((tid & 31) == 0) red[tid >> 5] = a;
  __syncthreads();
  float r = (tid & 31) < 8 ? red[tid & 31] : Op::identity();
  r = warp_reduce<Op>(r);
  if (fx.world > 1) finish_exchange<Op>(fx, epoch, r, tid == 0, slot_pos, tid);
  if (tid == 0) out[0] = r;
}

// reduce_col_f32_kernel + fold by the last CTA of every column tile (+ exchange)
template <class Op, bool VEC>
__global__ void __launch_bounds__(kColTx* kColTy) reduce_col_fused_f32_kernel(const float* __restrict__ x,
                                                                              float* __restrict__ partial,
                                                                              float* __restrict__ out, int64_t red,
                                                                              int64_t inner, int64_t rows_per_split,
                                                                              uint32_t* tickets, FinishExchange fx) {
  __shared__ float4 sm[kColTy][kColTx];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int64_t col = ((int64_t)blockIdx.x * kColTx + tx) * 4;
  const int64_t r0 = (int64_t)blockIdx.y * rows_per_split;
  const int64_t r1 = min(red, r0 + rows_per_split);
  const float id = Op::identity();
  float4 acc0 = make_float4(id, id, id, id), acc1 = acc0, acc2 = acc0, acc3 = acc0;
  if (VEC) {
    if (col < inner) {
      const float* base = x + col;
      int64_t r = r0 + ty;
      for (; r + 3 * kColTy < r1; r += 4 * kColTy) {
        const float4 a = ld_stream_f4(base + r * inner);
        const float4 b = ld_stream_f4(base + (r + kColTy) * inner);
        const float4 c = ld_stream_f4(base + (r + 2 * kColTy) * inner);
        const float4 d = ld_stream_f4(base + (r + 3 * kColTy) * inner);
        acc0 = apply4<Op>(acc0, a);
        acc1 = apply4<Op>(acc1, b);
        acc2 = apply4<Op>(acc2, c);
        acc3 = apply4<Op>(acc3, d);
      }
      for (; r < r1; r += kColTy) acc0 = apply4<Op>(acc0, ld_stream_f4(base + r * inner));
    }
  } else {
    for (int64_t r = r0 + ty; r < r1; r += kColTy) {
      const float* row = x + r * inner;
      float4 a = make_float4(id, id, id, id);
      if (col + 0 < inner) a.x = row[col + 0];
      if (col + 1 < inner) a.y = row[col + 1];
      if (col + 2 < inner) a.z = row[col + 2];
      if (col + 3 < inner) a.w = row[col + 3];
      acc0 = apply4<Op>(acc0, a);
    }
  }
  acc0 = apply4<Op>(apply4<Op>(acc0, acc1), apply4<Op>(acc2, acc3));
  sm[ty][tx] = acc0;
  __syncthreads();
#pragma unroll
  for (int h = kColTy / 2; h > 0; h >>= 1) {
    if (ty < h) sm[ty][tx] = apply4<Op>(sm[ty][tx], sm[ty + h][tx]);
    __syncthreads();
  }
  if (ty == 0) {
    const float4 r = sm[0][tx];
    float* o = partial + (int64_t)blockIdx.y * inner + col;
    if (col + 0 < inner) o[0] = r.x;
    if (col + 1 < inner) o[1] = r.y;
    if (col + 2 < inner) o[2] = r.z;
    if (col + 3 < inner) o[3] = r.w;
  }
  const int tid = ty * kColTx + tx;
  if (!arrive_last(tickets + blockIdx.x, gridDim.y, tid)) return;
  finish_col_tile<Op>(partial, out, gridDim.y, inner, blockIdx.x, tid, fx);
}

// reduce_col_dual_f32_kernel + both folds in the same launch (+ exchange of both results)
template <class Op1, class Op2>
__global__ void __launch_bounds__(kColTx* kColTy) reduce_col_dual_fused_f32_kernel(
    const float* __restrict__ x, float* __restrict__ partial, float* __restrict__ partial2, float* __restrict__ out1,
    float* __restrict__ out2, int64_t red, int64_t inner, int64_t rows_per_split, uint32_t* tickets, FinishExchange fx) {
  __shared__ float4 sm[kColTy][kColTx];
  __shared__ float red2[32];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int64_t col = ((int64_t)blockIdx.x * kColTx + tx) * 4;
  const int64_t r0 = (int64_t)blockIdx.y * rows_per_split;
  const int64_t r1 = min(red, r0 + rows_per_split);
  const float id = Op1::identity(), id2 = Op2::identity();
  float4 acc0 = make_float4(id, id, id, id), acc1 = acc0, acc2 = acc0, acc3 = acc0;
  float4 b0 = make_float4(id2, id2, id2, id2), b1 = b0;
  if (col < inner) {
    const float* base = x + col;
    int64_t r = r0 + ty;
    for (; r + 3 * kColTy < r1; r += 4 * kColTy) {
      const float4 a = ld_stream_f4(base + r * inner);
      const float4 b = ld_stream_f4(base + (r + kColTy) * inner);
      const float4 c = ld_stream_f4(base + (r + 2 * kColTy) * inner);
      const float4 d = ld_stream_f4(base + (r + 3 * kColTy) * inner);
      acc0 = apply4<Op1>(acc0, a);
      acc1 = apply4<Op1>(acc1, b);
      acc2 = apply4<Op1>(acc2, c);
      acc3 = apply4<Op1>(acc3, d);
      b0 = apply4<Op2>(b0, apply4<Op2>(a, b));
      b1 = apply4<Op2>(b1, apply4<Op2>(c, d));
    }
    for (; r < r1; r += kColTy) {
      const float4 a = ld_stream_f4(base + r * inner);
      acc0 = apply4<Op1>(acc0, a);
      b0 = apply4<Op2>(b0, a);
    }
  }
  acc0 = apply4<Op1>(apply4<Op1>(acc0, acc1), apply4<Op1>(acc2, acc3));
  sm[ty][tx] = acc0;
  __syncthreads();
#pragma unroll
  for (int h = kColTy / 2; h > 0; h >>= 1) {
    if (ty < h) sm[ty][tx] = apply4<Op1>(sm[ty][tx], sm[ty + h][tx]);
    __syncthreads();
  }
  if (ty == 0) {
    const float4 r = sm[0][tx];
    float* o = partial + (int64_t)blockIdx.y * inner + col;
    if (col + 0 < inner) o[0] = r.x;
    if (col + 1 < inner) o[1] = r.y;
    if (col + 2 < inner) o[2] = r.z;
    if (col + 3 < inner) o[3] = r.w;
  }
  b0 = apply4<Op2>(b0, b1);
  float s2 = Op2::apply(Op2::apply(b0.x, b0.y), Op2::apply(b0.z, b0.w));
  s2 = warp_reduce<Op2>(s2);
  const int tid = ty * kColTx + tx, lane = tid & 31, warp = tid >> 5;
  if (lane == 0) red2[warp] = s2;
  __syncthreads();
  if (warp == 0) {
    float v = lane < (kColTx * kColTy) / 32 ? red2[lane] : id2;
    v = warp_reduce<Op2>(v);
    if (lane == 0) partial2[(int64_t)blockIdx.y * gridDim.x + blockIdx.x] = v;
  }
  // one arrival covers both partials of this CTA: first the column tile's counter, then the counter of the whole grid
  const bool last_of_tile = arrive_last(tickets + blockIdx.x, gridDim.y, tid);
  if (last_of_tile) finish_col_tile<Op1>(partial, out1, gridDim.y, inner, blockIdx.x, tid, fx);
  const bool last_of_grid = arrive_last(tickets + gridDim.x, gridDim.x * gridDim.y, tid);
  if (last_of_grid)
    finish_all<Op2>(partial2, out2, (int)(gridDim.x * gridDim.y), tid, red2, fx, fx.slot_off2);
}

// reduce_all_f32_kernel + fold by the last CTA (+ exchange)
template <class Op, bool VEC>
__global__ void __launch_bounds__(256) reduce_all_fused_f32_kernel(const float* __restrict__ x,
                                                                   float* __restrict__ partial,
                                                                   float* __restrict__ out, int64_t n,
                                                                   uint32_t* tickets, FinishExchange fx) {
  __shared__ float red[32];
  const float id = Op::identity();
  float a0 = id, a1 = id, a2 = id, a3 = id;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (VEC) {
    const int64_t n4 = n >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    int64_t i = tid;
    for (; i + 3 * stride < n4; i += 4 * stride) {
      const float4 p = ld_stream_f4(x4 + i), q = ld_stream_f4(x4 + i + stride);
      const float4 r = ld_stream_f4(x4 + i + 2 * stride), t = ld_stream_f4(x4 + i + 3 * stride);
      a0 = Op::apply(a0, Op::apply(Op::apply(p.x, p.y), Op::apply(p.z, p.w)));
      a1 = Op::apply(a1, Op::apply(Op::apply(q.x, q.y), Op::apply(q.z, q.w)));
      a2 = Op::apply(a2, Op::apply(Op::apply(r.x, r.y), Op::apply(r.z, r.w)));
      a3 = Op::apply(a3, Op::apply(Op::apply(t.x, t.y), Op::apply(t.z, t.w)));
    }
    for (; i < n4; i += stride) {
      const float4 p = ld_stream_f4(x4 + i);
      a0 = Op::apply(a0, Op::apply(Op::apply(p.x, p.y), Op::apply(p.z, p.w)));
    }
    for (int64_t j = (n4 << 2) + tid; j < n; j += stride) a1 = Op::apply(a1, x[j]);
  } else {
    for (int64_t j = tid; j < n; j += stride) a0 = Op::apply(a0, x[j]);
  }
  float a = Op::apply(Op::apply(a0, a1), Op::apply(a2, a3));
  a = block_reduce<Op>(a, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = a;
  if (!arrive_last(tickets, gridDim.x, threadIdx.x)) return;
  finish_all<Op>(partial, out, (int)gridDim.x, threadIdx.x, red, fx, fx.slot_off);
}

// The fold of the partials as a launch of its own that also completes the exchange: one CTA per finisher.
// grid = column tiles (+ 1 CTA for the all-elements result when `partial2` is given), 256 threads.
template <class Op1, class Op2>
__global__ void __launch_bounds__(256) reduce_finish_exchange_kernel(const float* __restrict__ partial,
                                                                     float* __restrict__ out, int64_t splits,
                                                                     int64_t inner, int col_tiles,
                                                                     const float* __restrict__ partial2,
                                                                     float* __restrict__ out2, int n2,
                                                                     FinishExchange fx) {
  __shared__ float red[32];
  const int tid = threadIdx.x;
  if ((int)blockIdx.x < col_tiles) finish_col_tile<Op1>(partial, out, splits, inner, blockIdx.x, tid, fx);
  else finish_all<Op2>(partial2, out2, n2, tid, red, fx, fx.slot_off2);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <class Op>
cudaError_t col_impl(const float* x, float* out, int64_t red, int64_t inner, void* ws, int sm_count, cudaStream_t s,
                     LaunchDims* dims, uint32_t* tickets, const FinishExchange* fx) {
  const int64_t splits = col_row_splits(red, inner, sm_count);
  const int64_t rows_per_split = (red + splits - 1) / splits;
  dim3 grid((unsigned)((inner + kColTile - 1) / kColTile), (unsigned)splits), block(kColTx, kColTy);
  if (dims) {
    dims->grid[0] = grid.x;
    dims->grid[1] = grid.y;
    dims->block[0] = block.x;
    dims->block[1] = block.y;
    dims->smem = sizeof(float4) * kColTx * kColTy;
  }
  float* partial = splits == 1 ? out : reinterpret_cast<float*>(ws);
  const bool vec = inner % 4 == 0 && aligned16(x);
  const bool fused = tickets && splits > 1 && grid.x <= (unsigned)kReduceMaxTicketTiles;
  const bool exchange = fx && fx->world > 1;
  if (fused) {
    FinishExchange none;
    const FinishExchange& f = fx ? *fx : none;
    if (vec)
      reduce_col_fused_f32_kernel<Op, true><<<grid, block, 0, s>>>(x, partial, out, red, inner, rows_per_split, tickets, f);
    else
      reduce_col_fused_f32_kernel<Op, false><<<grid, block, 0, s>>>(x, partial, out, red, inner, rows_per_split, tickets, f);
    return cudaGetLastError();
  }
  if (vec)
    reduce_col_f32_kernel<Op, true><<<grid, block, 0, s>>>(x, partial, red, inner, rows_per_split);
  else
    reduce_col_f32_kernel<Op, false><<<grid, block, 0, s>>>(x, partial, red, inner, rows_per_split);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (exchange) {  // the fold of the splits (a single split: the result itself) and the exchange in one launch
    reduce_finish_exchange_kernel<Op, Op><<<grid.x, 256, 0, s>>>(partial, out, splits, inner, (int)grid.x, nullptr,
                                                                 nullptr, 0, *fx);
    return cudaGetLastError();
  }
  if (splits == 1) return e;
  reduce_col_finish_kernel<Op><<<(unsigned)((inner + 255) / 256), 256, 0, s>>>(partial, out, splits, inner);
  return cudaGetLastError();
}

template <class Op>
cudaError_t all_impl(const float* x, float* out, int64_t n, void* ws, int sm_count, cudaStream_t s, LaunchDims* dims,
                     uint32_t* tickets, const FinishExchange* fx) {
  const int64_t want = (n / 4 + 255) / 256;
  static const int per_sm = std::min(8, resident_ctas_per_sm(reduce_all_f32_kernel<Op, true>, 256));
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(want, (int64_t)sm_count * per_sm));
  if (dims) {
    dims->grid[0] = grid;
    dims->block[0] = 256;
  }
  float* partial = reinterpret_cast<float*>(ws);
  if (tickets) {
    FinishExchange none;
    const FinishExchange& f = fx ? *fx : none;
    if (aligned16(x)) reduce_all_fused_f32_kernel<Op, true><<<grid, 256, 0, s>>>(x, partial, out, n, tickets, f);
    else reduce_all_fused_f32_kernel<Op, false><<<grid, 256, 0, s>>>(x, partial, out, n, tickets, f);
    return cudaGetLastError();
  }
  if (aligned16(x)) reduce_all_f32_kernel<Op, true><<<grid, 256, 0, s>>>(x, partial, n);
  else reduce_all_f32_kernel<Op, false><<<grid, 256, 0, s>>>(x, partial, n);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (fx && fx->world > 1) {
    FinishExchange f = *fx;
    f.slot_off2 = f.slot_off;  // the one result sits at the first output's slot position, flag 0
    reduce_finish_exchange_kernel<Op, Op><<<1, 256, 0, s>>>(nullptr, nullptr, 0, 0, 0, partial, out, grid, f);
    return cudaGetLastError();
  }
  reduce_all_finish_kernel<Op><<<1, 1024, 0, s>>>(partial, out, grid);
  return cudaGetLastError();
}

template <class Op>
cudaError_t row_impl(const float* x, float* out, int64_t rows, int64_t cols, cudaStream_t s, LaunchDims* dims) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((rows + 7) / 8, (int64_t)sms * 8));
  if (dims) {
    dims->grid[0] = grid;
    dims->block[0] = 256;
  }
  const int vec = cols % 4 == 0 && aligned16(x);
  reduce_row_f32_kernel<Op><<<grid, 256, 0, s>>>(x, out, rows, cols, vec);
  return cudaGetLastError();
}

}  // namespace

size_t reduce_col_workspace(int64_t red, int64_t inner, int sm_count) {
  const int64_t splits = col_row_splits(red, inner, sm_count);
  return splits == 1 ? 0 : (size_t)(splits * inner) * sizeof(float);
}
size_t reduce_all_workspace(int sm_count) { return (size_t)sm_count * 8 * sizeof(float); }
bool reduce_col_fusable(int64_t red, int64_t inner, int sm_count) {
  return col_row_splits(red, inner, sm_count) > 1 && (inner + kColTile - 1) / kColTile <= kReduceMaxTicketTiles;
}

int reduce_col_launches(int64_t red, int64_t inner, int sm_count, bool tickets) {
  if (col_row_splits(red, inner, sm_count) == 1) return 1;
  return tickets && reduce_col_fusable(red, inner, sm_count) ? 1 : 2;
}

namespace {
template <class Op1, class Op2>
cudaError_t dual_impl(const float* x, float* out1, float* out2, int64_t red, int64_t inner, void* ws, int sm_count,
                      cudaStream_t s, LaunchDims* dims, uint32_t* tickets, const FinishExchange* fx) {
  const int64_t splits = col_row_splits(red, inner, sm_count);
  const int64_t rows_per_split = (red + splits - 1) / splits;
  dim3 grid((unsigned)((inner + kColTile - 1) / kColTile), (unsigned)splits), block(kColTx, kColTy);
  if (dims) {
    dims->grid[0] = grid.x;
    dims->grid[1] = grid.y;
    dims->block[0] = block.x;
    dims->block[1] = block.y;
    dims->smem = sizeof(float4) * kColTx * kColTy + 128;
  }
  float* partial = reinterpret_cast<float*>(ws);
  float* partial2 = partial + splits * inner;
  const bool fused = tickets && grid.x <= (unsigned)kReduceMaxTicketTiles;
  if (fused) {
    FinishExchange none;
    reduce_col_dual_fused_f32_kernel<Op1, Op2><<<grid, block, 0, s>>>(x, partial, partial2, out1, out2, red, inner,
                                                                      rows_per_split, tickets, fx ? *fx : none);
    return cudaGetLastError();
  }
  reduce_col_dual_f32_kernel<Op1, Op2><<<grid, block, 0, s>>>(x, partial, partial2, red, inner, rows_per_split);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  // both folds (and, between ranks, both exchanges) in one launch: a CTA per column tile and one for the all-elements result
  FinishExchange none;
  reduce_finish_exchange_kernel<Op1, Op2><<<grid.x + 1, 256, 0, s>>>(partial, out1, splits, inner, (int)grid.x, partial2,
                                                                     out2, (int)(grid.x * grid.y), fx ? *fx : none);
  return cudaGetLastError();
}
template <class Op1>
cudaError_t dual_pick(RedOp op2, const float* x, float* o1, float* o2, int64_t red, int64_t inner, void* ws, int sms,
                      cudaStream_t s, LaunchDims* dims, uint32_t* tk, const FinishExchange* fx) {
  switch (op2) {
    case RedOp::Sum: return dual_impl<Op1, SumOp>(x, o1, o2, red, inner, ws, sms, s, dims, tk, fx);
    case RedOp::Max: return dual_impl<Op1, MaxOp>(x, o1, o2, red, inner, ws, sms, s, dims, tk, fx);
    case RedOp::Min: return dual_impl<Op1, MinOp>(x, o1, o2, red, inner, ws, sms, s, dims, tk, fx);
    case RedOp::Prod: return dual_impl<Op1, ProdOp>(x, o1, o2, red, inner, ws, sms, s, dims, tk, fx);
  }
  return cudaErrorInvalidValue;
}
}  // namespace

bool reduce_col_dual_supported(int64_t inner, const void* x) {
  return inner % 4 == 0 && (x == nullptr || aligned16(x));
}
size_t reduce_col_dual_workspace(int64_t red, int64_t inner, int sm_count) {
  const int64_t splits = col_row_splits(red, inner, sm_count);
  const int64_t ctas = splits * ((inner + kColTile - 1) / kColTile);
  return (size_t)(splits * inner + ctas) * sizeof(float);
}
cudaError_t reduce_col_dual_f32(RedOp op1, RedOp op2, const float* x, float* out1, float* out2, int64_t red,
                                int64_t inner, void* ws, int sm_count, cudaStream_t s, LaunchDims* dims,
                                uint32_t* tickets, const FinishExchange* fx) {
  switch (op1) {
    case RedOp::Sum: return dual_pick<SumOp>(op2, x, out1, out2, red, inner, ws, sm_count, s, dims, tickets, fx);
    case RedOp::Max: return dual_pick<MaxOp>(op2, x, out1, out2, red, inner, ws, sm_count, s, dims, tickets, fx);
    case RedOp::Min: return dual_pick<MinOp>(op2, x, out1, out2, red, inner, ws, sm_count, s, dims, tickets, fx);
    case RedOp::Prod: return dual_pick<ProdOp>(op2, x, out1, out2, red, inner, ws, sm_count, s, dims, tickets, fx);
  }
  return cudaErrorInvalidValue;
}

#define AKGB_DISPATCH(fn, ...)                         \
  switch (op) {                                        \
    case RedOp::Sum: return fn<SumOp>(__VA_ARGS__);    \
    case RedOp::Max: return fn<MaxOp>(__VA_ARGS__);    \
    case RedOp::Min: return fn<MinOp>(__VA_ARGS__);    \
    case RedOp::Prod: return fn<ProdOp>(__VA_ARGS__);  \
  }                                                    \
  return cudaErrorInvalidValue;

cudaError_t reduce_col_f32(RedOp op, const float* x, float* out, int64_t red, int64_t inner, void* ws, int sm_count,
                           cudaStream_t s, LaunchDims* dims, uint32_t* tickets, const FinishExchange* fx) {
  AKGB_DISPATCH(col_impl, x, out, red, inner, ws, sm_count, s, dims, tickets, fx)
}
cudaError_t reduce_all_f32(RedOp op, const float* x, float* out, int64_t n, void* ws, int sm_count, cudaStream_t s,
                           LaunchDims* dims, uint32_t* tickets, const FinishExchange* fx) {
  AKGB_DISPATCH(all_impl, x, out, n, ws, sm_count, s, dims, tickets, fx)
}
cudaError_t reduce_row_f32(RedOp op, const float* x, float* out, int64_t rows, int64_t cols, cudaStream_t s,
                           LaunchDims* dims) {
  AKGB_DISPATCH(row_impl, x, out, rows, cols, s, dims)
}

}  // namespace akgb

// ---------------------------------------------------------------------------------------------------
// Column sum without any allocation.
//
// Some callers may not allocate device memory at the point where they need a reduction: code running
// inside a framework's memory-planned region (every buffer was sized and placed ahead of time), an
// allocator that is itself being torn down or is out of memory, or a real-time loop where cudaMalloc's
// implicit device synchronisation is not acceptable.  For them the split partials of the column
// reduction live in the fixed array below instead of a caller- or library-allocated workspace.
//
// The array is part of the library image: every GPU that loads the library holds these 1 MiB until the
// process exits.  All calls on a device share it.  Nothing in it has to start at zero — each launch
// overwrites every partial it later reads — so stale contents of the previous call are harmless; two
// calls whose kernels overlap on the GPU (different streams, no ordering) would overwrite each other's
// partials and must not be issued.
namespace akgb {
namespace {
constexpr size_t kNoAllocScratchFloats = 262144;  // 1 MiB
constexpr int64_t kNoAllocMaxCols = 65536;        // widest row the entry point accepts
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];

struct NoAllocDevice {
  bool ready = false;
  float* scratch = nullptr;  // DEVICE address of g_noalloc_scratch on this device
  int sm_count = 0;
};
NoAllocDevice g_noalloc_dev[64];
std::mutex g_noalloc_mu;
}  // namespace
}  // namespace akgb

extern "C" akgb_status akgb_reduce_sum_axis0_f32_noalloc(const float* x, float* out, int64_t rows, int64_t cols,
                                                         void* stream) {
  using namespace akgb;
  if (!x || !out || rows <= 0 || cols <= 0) {
    set_last_error("akgb_reduce_sum_axis0_f32_noalloc: null pointer or empty extent");
    return AKGB_INVALID_ARG;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    set_last_error("akgb_reduce_sum_axis0_f32_noalloc: no current CUDA device");
    return AKGB_CUDA_ERROR;
  }
  NoAllocDevice& d = g_noalloc_dev[dev];
  {
    // First call on this device: translate the array's name into its device address.  In host code the
    // name g_noalloc_scratch is only a handle for the runtime, not something a kernel can dereference.
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!d.ready) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess || !p) {
        set_last_error("akgb_reduce_sum_axis0_f32_noalloc: cudaGetSymbolAddress failed");
        return AKGB_CUDA_ERROR;
      }
      int sms = 0;
      e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess || sms <= 0) {
        set_last_error("akgb_reduce_sum_axis0_f32_noalloc: cannot query the SM count");
        return AKGB_CUDA_ERROR;
      }
      d.scratch = static_cast<float*>(p);
      d.sm_count = sms;
      d.ready = true;
    }
  }
  const size_t need = reduce_col_workspace(rows, cols, d.sm_count);  // bytes of partials, 0 = single split
  if (cols > kNoAllocMaxCols || need > kNoAllocScratchFloats * sizeof(float)) {
    char msg[224];
    std::snprintf(msg, sizeof(msg),
                  "akgb_reduce_sum_axis0_f32_noalloc: %lld x %lld is beyond the built-in scratch (at most %lld "
                  "columns, %zu bytes of partials; this shape needs %zu); use akgb_launch with a caller workspace",
                  (long long)rows, (long long)cols, (long long)kNoAllocMaxCols,
                  kNoAllocScratchFloats * sizeof(float), need);
    set_last_error(msg);
    return AKGB_TOO_LARGE;
  }
  e = reduce_col_f32(RedOp::Sum, x, out, rows, cols, d.scratch, d.sm_count, reinterpret_cast<cudaStream_t>(stream),
                     nullptr);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return AKGB_CUDA_ERROR;
  }
  return AKGB_OK;
}
