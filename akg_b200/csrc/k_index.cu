// Index ops of the JSON factory: Gather (np.take along one axis) and UnsortedSegmentSum (scatter-add by segment id).
//
// Gather follows the reference lowering (akg-mlir/lib/Conversion/MindSporeToLinalg/MindSporeToLinalg.cpp:526-594):
// out[o, i, r] = data[o, indices[i], r], batch_dims = 0.  UnsortedSegmentSum follows :596-744 and the
// expected-value generator's np.add.at (akg-mlir/python/akg_mlir/utils/op_dsl.py:1109-1116).  An index outside the
// axis is undefined in the reference (tensor.extract out of bounds); here such a row reads as zeros / is skipped, so
// that bad indices can never fault the device.  Segment sums use float atomics: the order of additions, and with
// it the last bits, is not fixed.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <type_traits>

#include "graph.hpp"

#include "common.cuh"
#include "kernels.hpp"

namespace akgb {
namespace {

__device__ __forceinline__ int64_t load_index(const void* idx, int64_t i, int idx64) {
  return idx64 ? reinterpret_cast<const int64_t*>(idx)[i] : (int64_t)reinterpret_cast<const int32_t*>(idx)[i];
}

// units of T: T = uint4 when the copied rows are 16-byte multiples and aligned, else the element's own width
template <typename T>
__global__ void __launch_bounds__(256) gather_kernel(const T* __restrict__ data, const void* __restrict__ idx,
                                                     T* __restrict__ out, int64_t outer, int64_t dim, int64_t nidx,
                                                     int64_t inner, int idx64) {
  const int64_t total = outer * nidx * inner;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const int64_t r = e % inner;
    const int64_t t = e / inner;
    const int64_t i = t % nidx;
    const int64_t o = t / nidx;
    const int64_t j = load_index(idx, i, idx64);
    T v;
    if (j >= 0 && j < dim) v = data[(o * dim + j) * inner + r];
    else v = T{};
    out[e] = v;
  }
}

// T: float, int32, __half, __nv_bfloat16 -- the sum accumulates in the element type, as the reference's loop nest does
// (akg-mlir/lib/Conversion/MindSporeToLinalg/MindSporeToLinalg.cpp:596-744); atomics make the order of the additions
// (and with it the last bits of floating-point results) vary from run to run
template <typename T>
__global__ void __launch_bounds__(256) segment_sum_kernel(const T* __restrict__ data, const void* __restrict__ ids,
                                                          T* __restrict__ out, int64_t nids, int64_t inner,
                                                          int64_t num_segments, int idx64) {
  const int64_t total = nids * inner;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const int64_t i = e / inner, r = e - i * inner;
    const int64_t sgm = load_index(ids, i, idx64);
    if (sgm >= 0 && sgm < num_segments) atomicAdd(out + sgm * inner + r, data[e]);
  }
}

template <typename T>
__device__ __forceinline__ float as_key(T v);
template <>
__device__ __forceinline__ float as_key<float>(float v) { return v; }
template <>
__device__ __forceinline__ float as_key<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float as_key<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// (value, index) pairs ordered as np.argmax orders them: a NaN beats everything, then the larger value, then the
// smaller index
template <typename K>
__device__ __forceinline__ bool better(K v, int64_t i, K bv, int64_t bi) {
  const bool vn = v != v, bn = bv != bv;
  if (vn || bn) return vn && (!bn || i < bi);
  return v > bv || (v == bv && i < bi);
}

// inner == 1: one warp per row, lanes stride over the row (coalesced), then a shuffle tree over (value, index)
template <typename T, typename K>
__global__ void __launch_bounds__(256) argmax_rows_kernel(const T* __restrict__ data, void* __restrict__ out,
                                                          int64_t rows, int64_t dim, int out64) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t r = warp; r < rows; r += nwarps) {
    const T* row = data + r * dim;
    K bv{};
    int64_t bi = -1;
    for (int64_t j = lane; j < dim; j += 32) {
      K v;
      if constexpr (sizeof(K) == sizeof(T) && !std::is_same<T, __half>::value && !std::is_same<T, __nv_bfloat16>::value)
        v = row[j];
      else
        v = as_key(row[j]);
      if (bi < 0 || better(v, j, bv, bi)) {
        bv = v;
        bi = j;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      K ov = __shfl_xor_sync(0xffffffffu, bv, o);
      int64_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi >= 0 && (bi < 0 || better(ov, oi, bv, bi))) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      if (out64) reinterpret_cast<int64_t*>(out)[r] = bi;
      else reinterpret_cast<int32_t*>(out)[r] = (int32_t)bi;
    }
  }
}

// inner > 1: one thread per (outer, inner) column walking the axis; neighbouring threads read neighbouring addresses
template <typename T, typename K>
__global__ void __launch_bounds__(256) argmax_cols_kernel(const T* __restrict__ data, void* __restrict__ out,
                                                          int64_t outer, int64_t dim, int64_t inner, int out64) {
  const int64_t total = outer * inner;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const int64_t o = e / inner, r = e - o * inner;
    const T* col = data + o * dim * inner + r;
    K bv{};
    int64_t bi = -1;
    for (int64_t j = 0; j < dim; ++j) {
      K v;
      if constexpr (std::is_same<T, __half>::value || std::is_same<T, __nv_bfloat16>::value) v = as_key(col[j * inner]);
      else v = col[j * inner];
      if (bi < 0 || better(v, j, bv, bi)) {
        bv = v;
        bi = j;
      }
    }
    if (out64) reinterpret_cast<int64_t*>(out)[e] = bi;
    else reinterpret_cast<int32_t*>(out)[e] = (int32_t)bi;
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
int grid_for(int64_t n) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return (int)std::max<int64_t>(1, std::min<int64_t>((n + 255) / 256, (int64_t)sms * 8));
}

}  // namespace

cudaError_t gather_rows(const void* data, const void* idx, void* out, int64_t outer, int64_t dim, int64_t nidx,
                        int64_t inner, int esize, int idx64, cudaStream_t s, LaunchDims* dims) {
  const int64_t total = outer * nidx * inner;
  if (total == 0) return cudaSuccess;
  const int64_t row_bytes = inner * esize;
  if (row_bytes % 16 == 0 && aligned16(data) && aligned16(out)) {
    const int64_t iv = row_bytes / 16;
    const int grid = grid_for(outer * nidx * iv);
    if (dims) {
      dims->grid[0] = grid;
      dims->block[0] = 256;
    }
    gather_kernel<uint4><<<grid, 256, 0, s>>>((const uint4*)data, idx, (uint4*)out, outer, dim, nidx, iv, idx64);
    return cudaGetLastError();
  }
  const int grid = grid_for(total);
  if (dims) {
    dims->grid[0] = grid;
    dims->block[0] = 256;
  }
  switch (esize) {
    case 1: gather_kernel<uint8_t><<<grid, 256, 0, s>>>((const uint8_t*)data, idx, (uint8_t*)out, outer, dim, nidx, inner, idx64); break;
    case 2: gather_kernel<uint16_t><<<grid, 256, 0, s>>>((const uint16_t*)data, idx, (uint16_t*)out, outer, dim, nidx, inner, idx64); break;
    case 4: gather_kernel<uint32_t><<<grid, 256, 0, s>>>((const uint32_t*)data, idx, (uint32_t*)out, outer, dim, nidx, inner, idx64); break;
    case 8: gather_kernel<uint64_t><<<grid, 256, 0, s>>>((const uint64_t*)data, idx, (uint64_t*)out, outer, dim, nidx, inner, idx64); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

template <typename T, typename K>
cudaError_t argmax_launch(const void* data, void* out, int64_t outer, int64_t dim, int64_t inner, int out64,
                          cudaStream_t s, LaunchDims* dims) {
  int grid;
  if (inner == 1) {
    grid = grid_for(outer * 32);
    argmax_rows_kernel<T, K><<<grid, 256, 0, s>>>((const T*)data, out, outer, dim, out64);
  } else {
    grid = grid_for(outer * inner);
    argmax_cols_kernel<T, K><<<grid, 256, 0, s>>>((const T*)data, out, outer, dim, inner, out64);
  }
  if (dims) {
    dims->grid[0] = grid;
    dims->block[0] = 256;
  }
  return cudaGetLastError();
}

cudaError_t argmax_axis(const void* data, void* out, int64_t outer, int64_t dim, int64_t inner, int in_dt, int out64,
                        cudaStream_t s, LaunchDims* dims) {
  if (outer * inner == 0 || dim == 0) return cudaSuccess;
  switch ((DT)in_dt) {
    case DT::F32: return argmax_launch<float, float>(data, out, outer, dim, inner, out64, s, dims);
    case DT::F16: return argmax_launch<__half, float>(data, out, outer, dim, inner, out64, s, dims);
    case DT::BF16: return argmax_launch<__nv_bfloat16, float>(data, out, outer, dim, inner, out64, s, dims);
    case DT::I32: return argmax_launch<int32_t, int32_t>(data, out, outer, dim, inner, out64, s, dims);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t segment_sum(const void* data, const void* ids, void* out, int64_t nids, int64_t inner,
                        int64_t num_segments, int idx64, int dt, cudaStream_t s, LaunchDims* dims) {
  const size_t esize = dt == kF32 || dt == 3 /* int32 */ ? 4 : 2;
  cudaError_t e = cudaMemsetAsync(out, 0, (size_t)(num_segments * inner) * esize, s);  // zero bits are 0 in every type
  if (e != cudaSuccess || nids * inner == 0) return e;
  const int grid = grid_for(nids * inner);
  if (dims) {
    dims->grid[0] = grid;
    dims->block[0] = 256;
  }
  if (dt == kF32)
    segment_sum_kernel<float><<<grid, 256, 0, s>>>((const float*)data, ids, (float*)out, nids, inner, num_segments, idx64);
  else if (dt == 3)
    segment_sum_kernel<int><<<grid, 256, 0, s>>>((const int*)data, ids, (int*)out, nids, inner, num_segments, idx64);
  else if (dt == kF16)
    segment_sum_kernel<__half><<<grid, 256, 0, s>>>((const __half*)data, ids, (__half*)out, nids, inner, num_segments, idx64);
  else if (dt == kBF16)
    segment_sum_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)data, ids, (__nv_bfloat16*)out, nids, inner,
                                                           num_segments, idx64);
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

}  // namespace akgb
