// Elementwise / broadcast class: the float16 bias + tanh-GELU (+ multiply)
// (+ cast to float32) chain.
//
// The reference lowers every op of the chain to arithmetic in the op's own
// element type (akg-mlir/lib/Conversion/MindSporeToLinalg/MindSporeToLinalg.cpp:377-483,
// akg-mlir/lib/Conversion/MindSporeToTosa/MindSporeToTosa.cpp:475-504), so a
// float16 chain rounds to float16 after each op.  The kernel replays exactly
// that: native f16x2 add/mul with round-to-nearest (an f16 add or mul rounded
// once equals the f32 operation rounded to f16, because 24 >= 2*11+2 bits), and
// tanh through a table of correctly rounded f16 results, so the output is
// bit-identical to a per-op evaluation.
#include <cmath>
#include <cstdlib>
#include <vector>

#include "async.cuh"
#include "common.cuh"
#include "hostconv.hpp"
#include "kernels.hpp"

namespace akgb {

namespace {
// The table holds RN_f16(tanh(x)) for every f16 magnitude 0 .. kLutHi (5.0); larger magnitudes
// (infinity included) clamp to the last entry, which is 1.0.
constexpr unsigned kLutHi = 0x4500;
constexpr int kLutN = ((int)kLutHi + 1 + 7) / 8 * 8;  // padded to whole 16-byte vectors
}  // namespace

int gelu_lut_entries() { return kLutN; }
void gelu_lut_build(uint16_t* out) {
  for (int i = 0; i < kLutN; ++i) {
    const unsigned m = (unsigned)i < kLutHi ? (unsigned)i : kLutHi;
    out[i] = f64_to_f16_bits(std::tanh(f16_bits_to_f64((uint16_t)m)));
  }
}

namespace {

// tanh of two f16 values through the table, two lanes per instruction where the ISA allows:
// magnitude = bits & 0x7fff; index = min(magnitude, 5.0) (an f16 min on the magnitudes orders them like
// integers and maps NaN to the clamp); |tanh| <= |x| always, so a NaN-propagating min against the
// magnitude changes nothing for numbers and restores NaN inputs; the sign bits are OR-ed back.
__device__ __forceinline__ __half2 tanh2(__half2 d, const uint16_t* lut) {
  const uint32_t w = *reinterpret_cast<uint32_t*>(&d);
  const uint32_t mag2 = w & 0x7fff7fffu;
  const __half2 magh = *reinterpret_cast<const __half2*>(&mag2);
  const uint32_t clamp = 0x45004500u;
  const __half2 idxh = __hmin2(magh, *reinterpret_cast<const __half2*>(&clamp));
  const uint32_t idx2 = *reinterpret_cast<const uint32_t*>(&idxh);
  const uint32_t lo = lut[idx2 & 0xffffu], hi = lut[idx2 >> 16];
  const uint32_t t2 = __byte_perm(lo, hi, 0x5410);
  const __half2 r = __hmin2_nan(*reinterpret_cast<const __half2*>(&t2), magh);
  const uint32_t out = *reinterpret_cast<const uint32_t*>(&r) | (w & 0x80008000u);
  return *reinterpret_cast<const __half2*>(&out);
}

struct Consts {
  __half2 c0, c1, c2, one;
};

template <bool BIAS, bool MUL>
__device__ __forceinline__ __half2 chain2(__half2 x, __half2 bias, __half2 y, const Consts& k, const uint16_t* lut) {
  const __half2 t = BIAS ? __hadd2_rn(x, bias) : x;
  const __half2 a = __hmul2_rn(t, t);
  const __half2 t3 = __hmul2_rn(a, t);
  const __half2 b = __hmul2_rn(t3, k.c0);
  const __half2 c = __hadd2_rn(t, b);
  const __half2 d = __hmul2_rn(c, k.c1);
  const __half2 e = tanh2(d, lut);
  const __half2 f = __hadd2_rn(e, k.one);
  const __half2 g = __hmul2_rn(t, k.c2);
  __half2 h = __hmul2_rn(g, f);
  if (MUL) h = __hmul2_rn(h, y);
  return h;
}

template <bool BIAS, bool MUL, bool OUTF32>
__device__ __forceinline__ void do_vec(uint4 xv, uint4 bv, uint4 yv, void* out, int64_t i, const Consts& k,
                                       const uint16_t* lut) {
  const __half2* xs = reinterpret_cast<const __half2*>(&xv);
  const __half2* bs = reinterpret_cast<const __half2*>(&bv);
  const __half2* ys = reinterpret_cast<const __half2*>(&yv);
  __half2 r[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) r[j] = chain2<BIAS, MUL>(xs[j], bs[j], ys[j], k, lut);
  if (OUTF32) {
    const float2 f0 = __half22float2(r[0]), f1 = __half22float2(r[1]);
    const float2 f2 = __half22float2(r[2]), f3 = __half22float2(r[3]);
    float4* o = reinterpret_cast<float4*>(out) + 2 * i;
    st_stream_f4(o, make_float4(f0.x, f0.y, f1.x, f1.y));
    st_stream_f4(o + 1, make_float4(f2.x, f2.y, f3.x, f3.y));
  } else {
    st_stream(reinterpret_cast<uint4*>(out) + i, *reinterpret_cast<uint4*>(r));
  }
}

// A CTA of kOsThreads threads handles kOsIter contiguous groups of kOsU 8-element vectors per thread and
// exits.  Short-lived CTAs sustain more HBM bandwidth on B200 than a grid-stride loop with the same
// traffic (measured: a persistent variant of this kernel reached 5.5 TB/s, this one 6.7 TB/s); the price
// is one table load from L2 per CTA, issued as a single bulk asynchronous copy.
template <bool BIAS, bool MUL, bool OUTF32, int kOsThreads, int kOsU, int kOsIter>
__global__ void __launch_bounds__(kOsThreads) gelu_chain_f16_oneshot_kernel(
    const uint4* __restrict__ x, const uint4* __restrict__ bias, const uint4* __restrict__ y, void* __restrict__ out,
    int64_t nvec, int64_t inner_vec, float c0, float c1, float c2, float c_one, const uint16_t* __restrict__ lut_g,
    uint32_t* __restrict__ err) {
  __shared__ __align__(128) uint16_t lut[kLutN];
  __shared__ __align__(8) uint64_t lut_bar;
  // the table arrives by one bulk asynchronous copy (L2 -> shared) while the threads fetch their data
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&lut_bar), 1);
    mbar_fence_init();
    mbar_expect_tx(smem_u32(&lut_bar), kLutN * 2);
    bulk_load(smem_u32(lut), lut_g, kLutN * 2, smem_u32(&lut_bar));
  }
  const uint4 z = make_uint4(0, 0, 0, 0);
  const uint32_t iv = BIAS ? (uint32_t)inner_vec : 1u;
  Consts k;
  k.c0 = __float2half2_rn(c0);
  k.c1 = __float2half2_rn(c1);
  k.c2 = __float2half2_rn(c2);
  k.one = __float2half2_rn(c_one);
  bool have_lut = false;
#pragma unroll 1
  for (int it = 0; it < kOsIter; ++it) {
    const int64_t base = ((int64_t)blockIdx.x * kOsIter + it) * (kOsThreads * kOsU) + threadIdx.x;
    uint4 xv[kOsU], yv[kOsU], bv[kOsU];
#pragma unroll
    for (int u = 0; u < kOsU; ++u) {
      const int64_t i = base + u * kOsThreads;
      xv[u] = i < nvec ? ld_stream(x + i) : z;
      yv[u] = (MUL && i < nvec) ? ld_stream(y + i) : z;
    }
    // bias vector index: one 64-bit remainder per thread, then 32-bit steps
    const uint32_t b0 = BIAS ? (uint32_t)(base % inner_vec) : 0u;
#pragma unroll
    for (int u = 0; u < kOsU; ++u) {
      const int64_t i = base + u * kOsThreads;
      bv[u] = (BIAS && i < nvec) ? ld_cached(bias + (b0 + (uint32_t)(u * kOsThreads)) % iv) : z;
    }
    if (!have_lut) {
      __syncthreads();  // the barrier is initialised
      if (!mbar_wait(smem_u32(&lut_bar), 0, nullptr)) {
        if (threadIdx.x == 0) atomicOr(err, 16u);
        return;  // the table never arrived: report instead of computing with garbage
      }
      have_lut = true;
    }
#pragma unroll
    for (int u = 0; u < kOsU; ++u) {
      const int64_t i = base + u * kOsThreads;
      if (i < nvec) do_vec<BIAS, MUL, OUTF32>(xv[u], bv[u], yv[u], out, i, k, lut);
    }
  }
}

// Any length / alignment: one element per thread-iteration, same arithmetic.
__global__ void __launch_bounds__(256) gelu_chain_f16_scalar_kernel(const __half* __restrict__ x,
                                                                    const __half* __restrict__ bias,
                                                                    const __half* __restrict__ y, void* __restrict__ out,
                                                                    int64_t begin, int64_t n, int64_t inner, int has_mul,
                                                                    int out_f32, float c0, float c1, float c2,
                                                                    float c_one, const uint16_t* __restrict__ lut_g) {
  Consts k;
  k.c0 = __float2half2_rn(c0);
  k.c1 = __float2half2_rn(c1);
  k.c2 = __float2half2_rn(c2);
  k.one = __float2half2_rn(c_one);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const __half2 xv = __half2half2(x[i]);
    const __half2 bv = inner ? __half2half2(bias[i % inner]) : xv;
    const __half2 yv = has_mul ? __half2half2(y[i]) : xv;
    __half2 h;
    if (inner) h = has_mul ? chain2<true, true>(xv, bv, yv, k, lut_g) : chain2<true, false>(xv, bv, yv, k, lut_g);
    else h = has_mul ? chain2<false, true>(xv, bv, yv, k, lut_g) : chain2<false, false>(xv, bv, yv, k, lut_g);
    if (out_f32) reinterpret_cast<float*>(out)[i] = __low2float(h);
    else reinterpret_cast<__half*>(out)[i] = __low2half(h);
  }
}

template <bool BIAS, bool MUL, bool OUTF32, int U>
cudaError_t launch_vec_shape(const GeluChainParams& p, const void* x, const void* bias, const void* y, void* out,
                             const void* lut, uint32_t* err, int64_t nvec, cudaStream_t s, LaunchDims* dims) {
  constexpr int T = 512, I = 2;
  const int64_t per_cta = (int64_t)T * U * I;
  const int64_t grid = (nvec + per_cta - 1) / per_cta;
  if (dims) {
    dims->grid[0] = (unsigned)grid;
    dims->block[0] = T;
    dims->smem = kLutN * 2;
  }
  gelu_chain_f16_oneshot_kernel<BIAS, MUL, OUTF32, T, U, I><<<(unsigned)grid, T, 0, s>>>(
      (const uint4*)x, (const uint4*)bias, (const uint4*)y, out, nvec, p.inner / 8, p.c0, p.c1, p.c2, p.c_one,
      (const uint16_t*)lut, err);
  return cudaGetLastError();
}

// CTA shapes measured at 4 / 8 / 16 / 32 / 64 x [512,4096] (0.07 - 1.07 GB, 20 launches in a graph): 512 threads x 2
// vectors x 2 iterations 13.9 / 23.3 / 42.7 / 81.2 / 158.1 us; one vector per thread and iteration 12.9 / 22.8 / 42.4 /
// 81.0 / 158.8 us; one iteration per CTA, or 256 threads, 7 - 25 % slower at every size (every CTA stages the table).  Small
// launches, as a shard of a split tensor is, take the finer shape.
template <bool BIAS, bool MUL, bool OUTF32>
cudaError_t launch_vec(const GeluChainParams& p, const void* x, const void* bias, const void* y, void* out,
                       const void* lut, uint32_t* err, int64_t nvec, int /*sms*/, cudaStream_t s, LaunchDims* dims) {
  if (nvec <= (int64_t)3 << 20) return launch_vec_shape<BIAS, MUL, OUTF32, 1>(p, x, bias, y, out, lut, err, nvec, s, dims);
  return launch_vec_shape<BIAS, MUL, OUTF32, 2>(p, x, bias, y, out, lut, err, nvec, s, dims);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

cudaError_t gelu_chain_f16(const GeluChainParams& p, const void* x, const void* bias, const void* y, void* out,
                           const void* lut, uint32_t* err_word, cudaStream_t s, LaunchDims* dims) {
  if (p.n == 0) return cudaSuccess;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const bool vec_ok = aligned16(x) && aligned16(out) && (!p.has_mul || aligned16(y)) &&
                      (!p.inner || (aligned16(bias) && p.inner % 8 == 0));
  int64_t nvec = vec_ok ? p.n / 8 : 0;
  cudaError_t e = cudaSuccess;
  if (nvec > 0) {
    // persistent CTAs: the table is staged into shared memory once per CTA
    const bool B = p.inner != 0, Mu = p.has_mul != 0, F = p.out_f32 != 0;
#define AKGB_GELU_CASE(b, m, f) \
  if (B == b && Mu == m && F == f) e = launch_vec<b, m, f>(p, x, bias, y, out, lut, err_word, nvec, sms, s, dims);
    AKGB_GELU_CASE(true, true, true)
    AKGB_GELU_CASE(true, true, false)
    AKGB_GELU_CASE(true, false, true)
    AKGB_GELU_CASE(true, false, false)
    AKGB_GELU_CASE(false, true, true)
    AKGB_GELU_CASE(false, true, false)
    AKGB_GELU_CASE(false, false, true)
    AKGB_GELU_CASE(false, false, false)
#undef AKGB_GELU_CASE
    if (e != cudaSuccess) return e;
  }
  const int64_t done = nvec * 8;
  if (done < p.n) {
    int64_t rest = p.n - done;
    int grid = (int)std::min<int64_t>((rest + 255) / 256, (int64_t)sms * 8);
    if (dims && nvec == 0) {
      dims->grid[0] = grid;
      dims->block[0] = 256;
    }
    gelu_chain_f16_scalar_kernel<<<grid, 256, 0, s>>>((const __half*)x, (const __half*)bias, (const __half*)y, out, done,
                                                      p.n, p.inner, p.has_mul, p.out_f32, p.c0, p.c1, p.c2, p.c_one,
                                                      (const uint16_t*)lut);
    e = cudaGetLastError();
  }
  return e;
}

}  // namespace akgb
