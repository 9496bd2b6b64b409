// Index ops of the JSON factory: Gather (np.take along one axis) and UnsortedSegmentSum (scatter-add by segment id).
//
// Gather follows the reference lowering (akg-mlir/lib/Conversion/MindSporeToLinalg/MindSporeToLinalg.cpp:526-594):
// out[o, i, r] = data[o, indices[i], r], batch_dims = 0.  UnsortedSegmentSum follows :596-744 and the
// expected-value generator's np.add.at (akg-mlir/python/akg_mlir/utils/op_dsl.py:1109-1116).  An index outside the
// axis is undefined in the reference (tensor.extract out of bounds); here such a row reads as zeros / is skipped, so
// that bad indices can never fault the device.  Segment sums use float atomics: the order of additions, and with
// it the last bits, is not fixed.
#include <algorithm>

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

__global__ void __launch_bounds__(256) segment_sum_f32_kernel(const float* __restrict__ data,
                                                              const void* __restrict__ ids, float* __restrict__ out,
                                                              int64_t nids, int64_t inner, int64_t num_segments,
                                                              int idx64) {
  const int64_t total = nids * inner;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const int64_t i = e / inner, r = e - i * inner;
    const int64_t sgm = load_index(ids, i, idx64);
    if (sgm >= 0 && sgm < num_segments) atomicAdd(out + sgm * inner + r, data[e]);
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

cudaError_t segment_sum_f32(const float* data, const void* ids, float* out, int64_t nids, int64_t inner,
                            int64_t num_segments, int idx64, cudaStream_t s, LaunchDims* dims) {
  cudaError_t e = cudaMemsetAsync(out, 0, (size_t)(num_segments * inner) * sizeof(float), s);
  if (e != cudaSuccess || nids * inner == 0) return e;
  const int grid = grid_for(nids * inner);
  if (dims) {
    dims->grid[0] = grid;
    dims->block[0] = 256;
  }
  segment_sum_f32_kernel<<<grid, 256, 0, s>>>(data, ids, out, nids, inner, num_segments, idx64);
  return cudaGetLastError();
}

}  // namespace akgb
