// Device helpers shared by the kernel templates: 128-bit global access with
// cache hints, exact narrowing conversions, warp/block reduction trees.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cfloat>
#include <cstdint>

namespace akgb {

// element-type codes shared with the host (same order as DT in graph.hpp)
enum : int { kF16 = 5, kF32 = 6, kBF16 = 8 };

// ---- 128-bit streaming loads/stores ------------------------------------------
// Inputs are read once: bypass L1 allocation.  Outputs are written once:
// streaming stores (evict-first).
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ float4 ld_stream_f4(const void* p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}
// small operands re-read by many CTAs (bias, gamma, mask): keep them cached
__device__ __forceinline__ uint4 ld_cached(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ float4 ld_cached_f4(const void* p) { return __ldg(reinterpret_cast<const float4*>(p)); }

__device__ __forceinline__ void st_stream(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_stream_f4(void* p, float4 v) {
  asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

// ---- conversions ---------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t lo16) { return __uint_as_float(lo16 << 16); }
// round-to-nearest-even f32 -> bf16 (arith.truncf), NaN kept quiet
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// 8 consecutive 16-bit elements (one uint4) -> 8 floats
__device__ __forceinline__ void unpack8(uint4 v, int dt, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  if (dt == kF16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
}
__device__ __forceinline__ uint4 pack8(const float* f, int dt) {
  uint4 v;
  if (dt == kF16) {
    v.x = pack_f16x2(f[0], f[1]);
    v.y = pack_f16x2(f[2], f[3]);
    v.z = pack_f16x2(f[4], f[5]);
    v.w = pack_f16x2(f[6], f[7]);
  } else {
    v.x = pack_bf16x2(f[0], f[1]);
    v.y = pack_bf16x2(f[2], f[3]);
    v.z = pack_bf16x2(f[4], f[5]);
    v.w = pack_bf16x2(f[6], f[7]);
  }
  return v;
}

// ---- launch sizing ---------------------------------------------------------------
// CTAs of `kernel` that fit on one SM at once.  Persistent (grid-stride) kernels launch exactly
// sm_count * this many CTAs, so that no partial second wave trails the first.
template <class Kernel>
inline int resident_ctas_per_sm(Kernel kernel, int block_threads, size_t dyn_smem = 0) {
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, block_threads, dyn_smem) != cudaSuccess || n < 1) {
    cudaGetLastError();
    n = 1;
  }
  return n;
}

// ---- reduction trees -------------------------------------------------------------
struct SumOp {
  __device__ __forceinline__ static float identity() { return 0.f; }
  __device__ __forceinline__ static float apply(float a, float b) { return a + b; }
};
// max/min ignore NaN operands like arith.maxnumf/minnumf, and start from
// -FLT_MAX/+FLT_MAX like the reference's init values
// (akg-mlir/lib/Conversion/MindSporeToLinalg/MindSporeToLinalg.cpp:791-843, :845-901)
struct MaxOp {
  __device__ __forceinline__ static float identity() { return -FLT_MAX; }
  __device__ __forceinline__ static float apply(float a, float b) { return fmaxf(a, b); }
};
struct MinOp {
  __device__ __forceinline__ static float identity() { return FLT_MAX; }
  __device__ __forceinline__ static float apply(float a, float b) { return fminf(a, b); }
};
struct ProdOp {
  __device__ __forceinline__ static float identity() { return 1.f; }
  __device__ __forceinline__ static float apply(float a, float b) { return a * b; }
};

template <class Op>
__device__ __forceinline__ float warp_reduce(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// All threads of the CTA get the result.  `smem` needs 32 floats.
template <class Op>
__device__ __forceinline__ float block_reduce(float v, float* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_reduce<Op>(v);
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = lane < nwarp ? smem[lane] : Op::identity();
  return warp_reduce<Op>(r);
}

}  // namespace akgb
