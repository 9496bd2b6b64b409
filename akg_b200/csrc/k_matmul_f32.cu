// float32 MatMul on the CUDA cores.
//
// The reference multiplies float32 operands with float32 mul/add per k, in k order, accumulating in the result type
// (akg-mlir/lib/Conversion/MindSporeToLinalg/MindSporeToLinalg.cpp:1453-1546).  The tensor cores have no float32
// operand format (tf32 drops 13 mantissa bits), so this kernel keeps the arithmetic in float32: every output element
// is one chain of fused multiply-adds over k = 0..K-1 in order, owned by one thread, so the result does not depend on
// the grid or on timing.  128x128 tiles, 8 k per step, 256 threads with an 8x8 register block each, shared-memory
// double buffering fed by 128-bit global loads.
#include <algorithm>

#include "common.cuh"
#include "kernels.hpp"

namespace akgb {
namespace {

constexpr int FBM = 128, FBN = 128, FBK = 8, FTHREADS = 256;

struct SgemmDev {
  const float* A;
  const float* B;
  float* C;
  const float* bias;
  int M, N, K;
  int has_bias, relu;
  int64_t stride_a, stride_b, stride_c;  // elements between batch entries
  int a_vec, b_vec, c_vec;               // rows are 16-byte aligned: 128-bit accesses allowed
};

// 4 consecutive k of row `r` (A, or B given as [N, K]); zero beyond the edges
__device__ __forceinline__ float4 load_k4(const float* base, int rows, int K, int r, int k, int vec) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (r >= rows) return v;
  const float* p = base + (size_t)r * K + k;
  if (vec && k + 4 <= K) return __ldg(reinterpret_cast<const float4*>(p));
  if (k + 0 < K) v.x = __ldg(p + 0);
  if (k + 1 < K) v.y = __ldg(p + 1);
  if (k + 2 < K) v.z = __ldg(p + 2);
  if (k + 3 < K) v.w = __ldg(p + 3);
  return v;
}
// 4 consecutive n of row k of B given as [K, N]
__device__ __forceinline__ float4 load_n4(const float* base, int K, int N, int k, int n, int vec) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (k >= K) return v;
  const float* p = base + (size_t)k * N + n;
  if (vec && n + 4 <= N) return __ldg(reinterpret_cast<const float4*>(p));
  if (n + 0 < N) v.x = __ldg(p + 0);
  if (n + 1 < N) v.y = __ldg(p + 1);
  if (n + 2 < N) v.z = __ldg(p + 2);
  if (n + 3 < N) v.w = __ldg(p + 3);
  return v;
}

template <bool TB>
__global__ void __launch_bounds__(FTHREADS) sgemm_f32_kernel(const SgemmDev p) {
  __shared__ __align__(16) float As[2][FBK][FBM];
  __shared__ __align__(16) float Bs[2][FBK][FBN];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * FBM, n0 = blockIdx.x * FBN;
  const float* A = p.A + (size_t)blockIdx.z * p.stride_a;
  const float* B = p.B + (size_t)blockIdx.z * p.stride_b;
  float* C = p.C + (size_t)blockIdx.z * p.stride_c;

  // global -> register staging coordinates
  const int a_row = tid >> 1, a_k = (tid & 1) * 4;        // A tile: 128 rows x 8 k
  const int b_krow = tid >> 5, b_col = (tid & 31) * 4;    // B tile [K, N]: 8 k x 128 n
  float4 ra, rb;
  auto fetch = [&](int k0) {
    ra = load_k4(A, p.M, p.K, m0 + a_row, k0 + a_k, p.a_vec);
    if (TB) rb = load_k4(B, p.N, p.K, n0 + a_row, k0 + a_k, p.b_vec);
    else rb = load_n4(B, p.K, p.N, k0 + b_krow, n0 + b_col, p.b_vec);
  };
  auto stage = [&](int buf) {
    As[buf][a_k + 0][a_row] = ra.x;
    As[buf][a_k + 1][a_row] = ra.y;
    As[buf][a_k + 2][a_row] = ra.z;
    As[buf][a_k + 3][a_row] = ra.w;
    if (TB) {
      Bs[buf][a_k + 0][a_row] = rb.x;
      Bs[buf][a_k + 1][a_row] = rb.y;
      Bs[buf][a_k + 2][a_row] = rb.z;
      Bs[buf][a_k + 3][a_row] = rb.w;
    } else {
      *reinterpret_cast<float4*>(&Bs[buf][b_krow][b_col]) = rb;
    }
  };

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  fetch(0);
  stage(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < p.K; k0 += FBK) {
    const bool more = k0 + FBK < p.K;
    if (more) fetch(k0 + FBK);
#pragma unroll
    for (int k = 0; k < FBK; ++k) {
      float a[8], b[8];
      *reinterpret_cast<float4*>(a) = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
      *reinterpret_cast<float4*>(a + 4) = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
      *reinterpret_cast<float4*>(b) = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
      *reinterpret_cast<float4*>(b + 4) = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
    }
    if (more) {
      stage(buf ^ 1);
      __syncthreads();
      buf ^= 1;
    }
  }

  // epilogue: bias, ReLU (NaN stays NaN), store
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (row >= p.M) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int col = n0 + h * 64 + tx * 4;
      if (col >= p.N) continue;
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[j] = acc[i][h * 4 + j];
        if (p.has_bias && col + j < p.N) v[j] = __fadd_rn(v[j], __ldg(p.bias + col + j));
        if (p.relu) v[j] = v[j] != v[j] ? v[j] : fmaxf(v[j], 0.f);
      }
      float* o = C + (size_t)row * p.N + col;
      if (p.c_vec && col + 4 <= p.N) {
        *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (col + j < p.N) o[j] = v[j];
      }
    }
  }
}

inline bool al16(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; }

}  // namespace

cudaError_t matmul_f32(const MatmulParams& p, const void* A, const void* B, const void* bias, void* out,
                       int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_o, cudaStream_t s,
                       LaunchDims* dims) {
  if (p.M <= 0 || p.N <= 0 || p.K <= 0 || batch <= 0) return cudaErrorInvalidValue;
  if (batch > 65535) return cudaErrorInvalidValue;
  SgemmDev d;
  d.A = (const float*)A;
  d.B = (const float*)B;
  d.C = (float*)out;
  d.bias = (const float*)bias;
  d.M = (int)p.M;
  d.N = (int)p.N;
  d.K = (int)p.K;
  d.has_bias = p.has_bias;
  d.relu = p.relu;
  d.stride_a = stride_a;
  d.stride_b = stride_b;
  d.stride_c = stride_o;
  d.a_vec = al16(A) && p.K % 4 == 0 && stride_a % 4 == 0;
  d.b_vec = al16(B) && (p.transpose_b ? p.K % 4 == 0 : p.N % 4 == 0) && stride_b % 4 == 0;
  d.c_vec = al16(out) && p.N % 4 == 0 && stride_o % 4 == 0;
  dim3 grid((unsigned)((p.N + FBN - 1) / FBN), (unsigned)((p.M + FBM - 1) / FBM), (unsigned)batch);
  if (grid.y > 65535) return cudaErrorInvalidValue;
  if (dims) {
    dims->grid[0] = (int)grid.x;
    dims->grid[1] = (int)grid.y;
    dims->grid[2] = (int)grid.z;
    dims->block[0] = FTHREADS;
  }
  if (p.transpose_b) sgemm_f32_kernel<true><<<grid, FTHREADS, 0, s>>>(d);
  else sgemm_f32_kernel<false><<<grid, FTHREADS, 0, s>>>(d);
  return cudaGetLastError();
}

}  // namespace akgb
