// Row-fused patterns of the reduce-X class: LayerNorm and (masked) softmax.
// One warp owns one row and keeps it in registers, so the row is read from
// HBM once; the reductions are warp-shuffle trees.  Rows too wide for the
// register file (or with an odd width/alignment) go to a CTA-per-row variant
// that re-reads the row through L1/L2.
//
// Arithmetic follows the op chain the description spells
// (mean = sum*1/N; d = x-mean; var = sum(d*d)*1/N; rstd = 1/sqrt(var+eps);
//  y = ((d*rstd)*gamma)+beta) with one f32 rounding per op, no contraction;
// Rsqrt is 1/sqrt like the reference's expected-value generator
// (akg-mlir/python/akg_mlir/utils/op_dsl.py:792-794).  Only the summation
// order differs from a sequential loop
// (akg-mlir/lib/Conversion/MindSporeToLinalg/MindSporeToLinalg.cpp:1401-1426).
#include <algorithm>
#include <mutex>

#include "async.cuh"
#include "common.cuh"
#include "kernels.hpp"

namespace akgb {
namespace {

constexpr int kWarpsPerCta = 8;

// ------------------------------------------------------------------ LayerNorm
template <int VPL, int kWarpsPerCta, int kMinCtas>  // float4 vectors per lane; covers cols <= 128*VPL, cols % 4 == 0
__global__ void __launch_bounds__(kWarpsPerCta * 32, kMinCtas) layernorm_rows_f32_kernel(
    LayerNormParams p, const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
    float* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ var_out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerCta;
  const int cols4 = (int)(p.cols >> 2);
  for (int64_t row = warp; row < p.rows; row += nwarps) {
    const float4* xr = reinterpret_cast<const float4*>(x + row * p.cols);
    float4 v[VPL];
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int c = lane + 32 * k;
      v[k] = c < cols4 ? ld_stream_f4(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
    s = warp_reduce<SumOp>(s);
    const float mean = p.div_n != 0.f ? __fdiv_rn(s, p.div_n) : __fmul_rn(s, p.inv_n);
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int c = lane + 32 * k;
      v[k].x = __fsub_rn(v[k].x, mean);
      v[k].y = __fsub_rn(v[k].y, mean);
      v[k].z = __fsub_rn(v[k].z, mean);
      v[k].w = __fsub_rn(v[k].w, mean);
      if (c < cols4)
        q += (__fmul_rn(v[k].x, v[k].x) + __fmul_rn(v[k].y, v[k].y)) +
             (__fmul_rn(v[k].z, v[k].z) + __fmul_rn(v[k].w, v[k].w));
    }
    q = warp_reduce<SumOp>(q);
    const float var = p.div_n != 0.f ? __fdiv_rn(q, p.div_n) : __fmul_rn(q, p.inv_n);
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, p.eps)));
    float4* yr = reinterpret_cast<float4*>(y + row * p.cols);
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int c = lane + 32 * k;
      if (c < cols4) {
        float4 o;
        o.x = __fmul_rn(v[k].x, rstd);
        o.y = __fmul_rn(v[k].y, rstd);
        o.z = __fmul_rn(v[k].z, rstd);
        o.w = __fmul_rn(v[k].w, rstd);
        if (p.has_gamma) {
          const float4 g = ld_cached_f4(reinterpret_cast<const float4*>(gamma) + c);
          o.x = __fmul_rn(o.x, g.x);
          o.y = __fmul_rn(o.y, g.y);
          o.z = __fmul_rn(o.z, g.z);
          o.w = __fmul_rn(o.w, g.w);
        }
        if (p.has_beta) {
          const float4 b = ld_cached_f4(reinterpret_cast<const float4*>(beta) + c);
          o.x = __fadd_rn(o.x, b.x);
          o.y = __fadd_rn(o.y, b.y);
          o.z = __fadd_rn(o.z, b.z);
          o.w = __fadd_rn(o.w, b.w);
        }
        st_stream_f4(yr + c, o);
      }
    }
    if (lane == 0) {
      if (p.write_mean) mean_out[row] = mean;
      if (p.write_var) var_out[row] = var;
    }
  }
}

// any width/alignment: one CTA per row, three passes over the row
__global__ void __launch_bounds__(256) layernorm_rows_f32_generic_kernel(
    LayerNormParams p, const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
    float* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ var_out) {
  __shared__ float red[32];
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const float* xr = x + row * p.cols;
    float s = 0.f;
    for (int64_t c = threadIdx.x; c < p.cols; c += blockDim.x) s += xr[c];
    s = block_reduce<SumOp>(s, red);
    const float mean = p.div_n != 0.f ? __fdiv_rn(s, p.div_n) : __fmul_rn(s, p.inv_n);
    float q = 0.f;
    for (int64_t c = threadIdx.x; c < p.cols; c += blockDim.x) {
      const float d = __fsub_rn(xr[c], mean);
      q += __fmul_rn(d, d);
    }
    q = block_reduce<SumOp>(q, red);
    const float var = p.div_n != 0.f ? __fdiv_rn(q, p.div_n) : __fmul_rn(q, p.inv_n);
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, p.eps)));
    for (int64_t c = threadIdx.x; c < p.cols; c += blockDim.x) {
      float o = __fmul_rn(__fsub_rn(xr[c], mean), rstd);
      if (p.has_gamma) o = __fmul_rn(o, gamma[c]);
      if (p.has_beta) o = __fadd_rn(o, beta[c]);
      y[row * p.cols + c] = o;
    }
    if (threadIdx.x == 0) {
      if (p.write_mean) mean_out[row] = mean;
      if (p.write_var) var_out[row] = var;
    }
    __syncthreads();
  }
}

// -------------------------------------------------------------------- softmax
// Loads 8 consecutive elements of a row as floats.
__device__ __forceinline__ void load8(const void* base, int64_t elem, int dt, bool stream, float* f) {
  if (dt == kF32) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + elem);
    const float4 a = stream ? ld_stream_f4(p) : ld_cached_f4(p);
    const float4 b = stream ? ld_stream_f4(p + 1) : ld_cached_f4(p + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
    const void* p = reinterpret_cast<const uint16_t*>(base) + elem;
    unpack8(stream ? ld_stream(p) : ld_cached(p), dt, f);
  }
}
__device__ __forceinline__ void store8(void* base, int64_t elem, int dt, const float* f) {
  if (dt == kF32) {
    float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + elem);
    st_stream_f4(p, make_float4(f[0], f[1], f[2], f[3]));
    st_stream_f4(p + 1, make_float4(f[4], f[5], f[6], f[7]));
  } else {
    st_stream(reinterpret_cast<uint16_t*>(base) + elem, pack8(f, dt));
  }
}

constexpr float kLog2e = 1.4426950408889634f;

template <int VPL>  // groups of 8 elements per lane; covers cols <= 256*VPL, cols % 8 == 0
__global__ void __launch_bounds__(kWarpsPerCta * 32) softmax_rows_kernel(SoftmaxParams p, const void* __restrict__ x,
                                                                         const void* __restrict__ mask,
                                                                         void* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerCta;
  const int groups = (int)(p.cols >> 3);
  for (int64_t row = warp; row < p.rows; row += nwarps) {
    float v[VPL][8];
    const int64_t rbase = row * p.cols;
    const int64_t mbase = p.has_mask ? (row % p.mask_rows) * p.cols : 0;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int gidx = lane + 32 * k;
      if (gidx < groups) load8(x, rbase + 8 * (int64_t)gidx, p.in_dt, true, v[k]);
    }
    float mx = -FLT_MAX;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int gidx = lane + 32 * k;
      if (gidx < groups) {
        float mk[8];
        if (p.has_mask) load8(mask, mbase + 8 * (int64_t)gidx, p.mask_dt, false, mk);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float s = v[k][j];
          if (p.has_scale) s = __fmul_rn(s, p.scale);
          if (p.has_mask) s = __fadd_rn(s, mk[j]);
          v[k][j] = s;
          mx = fmaxf(mx, s);
        }
      }
    }
    mx = warp_reduce<MaxOp>(mx);
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int gidx = lane + 32 * k;
      if (gidx < groups) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float e = exp2f(__fmul_rn(__fsub_rn(v[k][j], mx), kLog2e));
          v[k][j] = e;
          sum += e;
        }
      }
    }
    sum = warp_reduce<SumOp>(sum);
    const float inv = __fdiv_rn(1.0f, sum);
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int gidx = lane + 32 * k;
      if (gidx < groups) {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[k][j] = __fmul_rn(v[k][j], inv);
        store8(out, rbase + 8 * (int64_t)gidx, p.out_dt, v[k]);
      }
    }
  }
}

// ---- softmax, staged variant for 16-bit scores/mask/output and rows of at most 4 KiB -------------
// Every warp runs its own two-slot pipeline of bulk asynchronous copies (global -> shared, completing
// on an mbarrier): while it works on row i out of registers, rows i+1 and i+2 are in flight, so a
// 16-warp CTA keeps up to 128 KiB of HBM reads outstanding per SM without spending registers on them.
// Rows are visited mask-row-major (all batches of mask row m, then m+1): a warp stages the mask row
// into shared memory once and reuses it for every batch, so the mask is read from L2 once per warp.
constexpr int kStWarps = 16;
constexpr int kStRowBytes = 4096;
constexpr int kStSlotBytes = 3 * kStRowBytes;  // two score slots + the mask row, per warp
constexpr int kStSmem = kStWarps * kStSlotBytes + kStWarps * 4 * 8 + 128;

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <int DT>
__global__ void __launch_bounds__(kStWarps * 32, 1) softmax_rows_staged_kernel(SoftmaxParams p,
                                                                               const uint16_t* __restrict__ x,
                                                                               const uint16_t* __restrict__ mask,
                                                                               uint16_t* __restrict__ out,
                                                                               uint32_t* __restrict__ err,
                                                                               int rows_per_warp) {
  constexpr int VPL = 8;  // groups of 8 elements per lane: rows up to 2048 elements
  extern __shared__ __align__(128) uint8_t st_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t sbase = smem_u32(st_smem) + warp * kStSlotBytes;
  const uint32_t mbuf = sbase + 2 * kStRowBytes;
  const uint32_t bar0 = smem_u32(st_smem) + kStWarps * kStSlotBytes + warp * 32;
  const uint32_t barm = bar0 + 16;  // completion of the mask row copy
  if (lane == 0) {
    mbar_init(bar0, 1);
    mbar_init(bar0 + 8, 1);
    mbar_init(barm, 1);
    mbar_fence_init();
  }
  __syncwarp();

  const int groups = (int)(p.cols >> 3);
  const uint32_t row_bytes = (uint32_t)p.cols * 2u;
  const int64_t nb = p.rows / p.mask_rows;  // batches per mask row
  const int64_t per = rows_per_warp;
  const int64_t v0 = ((int64_t)blockIdx.x * kStWarps + warp) * per;
  const int64_t v1 = min(p.rows, v0 + per);
  if (v0 >= v1) return;

  // virtual index v = m * nb + b  <->  row = b * mask_rows + m
  int64_t m = v0 / nb, b = v0 - m * nb;
  auto row_of = [&](int64_t mm, int64_t bb) { return bb * p.mask_rows + mm; };
  // (m, b) of v0+1 and v0+2 for the prefetches
  int64_t pm = m, pb = b;  // position of the next row to request
  auto advance = [&](int64_t& mm, int64_t& bb) {
    if (++bb == nb) {
      bb = 0;
      ++mm;
    }
  };
  auto request = [&](int slot) {
    if (lane == 0) {
      const uint32_t bar = bar0 + slot * 8;
      mbar_expect_tx(bar, row_bytes);
      bulk_load(sbase + slot * kStRowBytes, x + row_of(pm, pb) * p.cols, row_bytes, bar);
    }
    advance(pm, pb);
  };
  int64_t requested = 0;
  request(0);
  ++requested;
  if (v0 + 1 < v1) {
    request(1);
    ++requested;
  }
  uint32_t phase[2] = {0u, 0u};
  uint32_t mphase = 0u;
  int64_t cur_m = -1;
  bool ok = true;
  const float log2e = 1.4426950408889634f;
  int64_t done = 0;
  for (int64_t v = v0; v < v1; ++v, ++done) {
    const int slot = (int)(done & 1);
    if (p.has_mask && m != cur_m) {
      // stage mask row m (an L2-resident operand) for all batches that follow: one bulk copy
      __syncwarp();  // every lane is done with the previous mask row
      if (lane == 0) {
        fence_proxy_async_smem();
        mbar_expect_tx(barm, row_bytes);
        bulk_load(mbuf, mask + m * p.cols, row_bytes, barm);
      }
      if (!mbar_wait(barm, mphase, nullptr)) {
        ok = false;
        break;
      }
      mphase ^= 1u;
      cur_m = m;
    }
    if (!mbar_wait(bar0 + slot * 8, phase[slot], nullptr)) {
      ok = false;
      break;
    }
    phase[slot] ^= 1u;
    float s[VPL][8];
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int gidx = lane + 32 * k;
      if (gidx < groups) unpack8(lds128(sbase + slot * kStRowBytes + gidx * 16), DT, s[k]);
    }
    __syncwarp();  // every lane has taken its part of the slot
    if (requested < v1 - v0) {
      fence_proxy_async_smem();
      request(slot);
      ++requested;
    }
    float mx = -FLT_MAX;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int gidx = lane + 32 * k;
      if (gidx < groups) {
        float mk[8];
        if (p.has_mask) unpack8(lds128(mbuf + gidx * 16), DT, mk);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // Mul then Add of the description, contracted: the 16-bit result absorbs the difference
          const float t = p.has_mask ? fmaf(s[k][j], p.scale, mk[j]) : s[k][j] * p.scale;
          s[k][j] = t;
          mx = fmaxf(mx, t);
        }
      }
    }
    mx = warp_reduce<MaxOp>(mx);
    const float neg_mxl = -mx * log2e;
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int gidx = lane + 32 * k;
      if (gidx < groups) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float e = ex2_approx(fmaf(s[k][j], log2e, neg_mxl));
          s[k][j] = e;
          sum += e;
        }
      }
    }
    sum = warp_reduce<SumOp>(sum);
    const float inv = __fdiv_rn(1.0f, sum);
    uint16_t* orow = out + row_of(m, b) * p.cols;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int gidx = lane + 32 * k;
      if (gidx < groups) {
#pragma unroll
        for (int j = 0; j < 8; ++j) s[k][j] *= inv;
        st_stream(orow + 8 * gidx, pack8(s[k], DT));
      }
    }
    advance(m, b);
  }
  if (!ok) {
    // a copy never completed: report, then give the copies still in flight a bounded chance to land
    if (lane == 0) {
      atomicOr(err, 8u);
      const int64_t pending = requested - done;
      for (int64_t i = 0; i < pending && i < 2; ++i) {
        const int slot = (int)((done + i) & 1);
        mbar_wait(bar0 + slot * 8, phase[slot], nullptr);
      }
    }
    __syncwarp();
  }
}

__device__ __forceinline__ float load1(const void* base, int64_t i, int dt) {
  if (dt == kF32) return reinterpret_cast<const float*>(base)[i];
  if (dt == kF16) return __half2float(reinterpret_cast<const __half*>(base)[i]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
}
__device__ __forceinline__ void store1(void* base, int64_t i, int dt, float f) {
  if (dt == kF32) reinterpret_cast<float*>(base)[i] = f;
  else if (dt == kF16) reinterpret_cast<__half*>(base)[i] = __float2half_rn(f);
  else reinterpret_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(f);
}

// any width/alignment: one CTA per row, three passes
__global__ void __launch_bounds__(256) softmax_rows_generic_kernel(SoftmaxParams p, const void* __restrict__ x,
                                                                   const void* __restrict__ mask,
                                                                   void* __restrict__ out) {
  __shared__ float red[32];
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const int64_t rbase = row * p.cols;
    const int64_t mbase = p.has_mask ? (row % p.mask_rows) * p.cols : 0;
    auto score = [&](int64_t c) {
      float s = load1(x, rbase + c, p.in_dt);
      if (p.has_scale) s = __fmul_rn(s, p.scale);
      if (p.has_mask) s = __fadd_rn(s, load1(mask, mbase + c, p.mask_dt));
      return s;
    };
    float mx = -FLT_MAX;
    for (int64_t c = threadIdx.x; c < p.cols; c += blockDim.x) mx = fmaxf(mx, score(c));
    mx = block_reduce<MaxOp>(mx, red);
    float sum = 0.f;
    for (int64_t c = threadIdx.x; c < p.cols; c += blockDim.x)
      sum += exp2f(__fmul_rn(__fsub_rn(score(c), mx), kLog2e));
    sum = block_reduce<SumOp>(sum, red);
    const float inv = __fdiv_rn(1.0f, sum);
    for (int64_t c = threadIdx.x; c < p.cols; c += blockDim.x)
      store1(out, rbase + c, p.out_dt, __fmul_rn(exp2f(__fmul_rn(__fsub_rn(score(c), mx), kLog2e)), inv));
    __syncthreads();
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int sm_count_now() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

}  // namespace

cudaError_t layernorm_f32(const LayerNormParams& p, const float* x, const float* gamma, const float* beta, float* y,
                          float* mean, float* var, uint32_t* /*err_word*/, cudaStream_t s, LaunchDims* dims) {
  if (p.rows == 0 || p.cols == 0) return cudaSuccess;
  const int sms = sm_count_now();
  const bool vec = p.cols % 4 == 0 && p.cols <= 128 * 16 && aligned16(x) && aligned16(y) &&
                   (!p.has_gamma || aligned16(gamma)) && (!p.has_beta || aligned16(beta));
  if (vec) {
    // one row per warp, 4 warps per CTA: measured equal or better than 1, 2 or 8 warps per CTA and than
    // register caps that raise occupancy (13.4 us for [8192,1024], 42.2 us for [32768,1024])
    constexpr int WPC = 4;
    int64_t grid = (p.rows + WPC - 1) / WPC;
    const int64_t v = (p.cols + 127) / 128;
    // 1024-column rows: the kernel needs 82 registers (6 CTAs per SM).  When the grid is just above six CTAs per SM
    // but within seven, the variant capped at 72 registers keeps every CTA resident at once instead of leaving a
    // small second wave: [4096,1024] 9.1 -> 8.0 us.  With several waves the uncapped kernel is the faster one
    // ([8192,1024]: 13.4 against 14.2 us), and fewer, longer-lived CTAs (one wave, rows in a grid-stride loop) are
    // slower still (14.2 us).
    if (v == 8 && grid > (int64_t)sms * 6 && grid <= (int64_t)sms * 7) {
      if (dims) {
        dims->grid[0] = (unsigned)grid;
        dims->block[0] = WPC * 32;
      }
      layernorm_rows_f32_kernel<8, WPC, 7><<<(unsigned)grid, WPC * 32, 0, s>>>(p, x, gamma, beta, y, mean, var);
      return cudaGetLastError();
    }
    if (dims) {
      dims->grid[0] = (unsigned)grid;
      dims->block[0] = WPC * 32;
    }
#define AKGB_LN(V) layernorm_rows_f32_kernel<V, WPC, 1><<<(unsigned)grid, WPC * 32, 0, s>>>(p, x, gamma, beta, y, mean, var)
    if (v <= 1) AKGB_LN(1);
    else if (v <= 2) AKGB_LN(2);
    else if (v <= 4) AKGB_LN(4);
    else if (v <= 8) AKGB_LN(8);
    else AKGB_LN(16);
#undef AKGB_LN
  } else {
    const int grid = (int)std::min<int64_t>(p.rows, (int64_t)sms * 8);
    if (dims) {
      dims->grid[0] = grid;
      dims->block[0] = 256;
    }
    layernorm_rows_f32_generic_kernel<<<grid, 256, 0, s>>>(p, x, gamma, beta, y, mean, var);
  }
  return cudaGetLastError();
}

cudaError_t softmax_rows(const SoftmaxParams& p, const void* x, const void* mask, void* out, uint32_t* err_word,
                         cudaStream_t s, LaunchDims* dims) {
  if (p.rows == 0 || p.cols == 0) return cudaSuccess;
  const int sms = sm_count_now();
  const bool vec = p.cols % 8 == 0 && p.cols <= 256 * 16 && aligned16(x) && aligned16(out) &&
                   (!p.has_mask || aligned16(mask));
  const bool staged = vec && err_word && p.cols <= 2048 && (p.in_dt == kF16 || p.in_dt == kBF16) &&
                      p.out_dt == p.in_dt && (!p.has_mask || p.mask_dt == p.in_dt) && p.rows >= 4 * kStWarps &&
                      p.rows % p.mask_rows == 0;
  if (staged) {
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
      attr_err = cudaFuncSetAttribute(softmax_rows_staged_kernel<kF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kStSmem);
      if (attr_err == cudaSuccess)
        attr_err = cudaFuncSetAttribute(softmax_rows_staged_kernel<kBF16>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, kStSmem);
    });
    if (attr_err != cudaSuccess) return attr_err;
    // short-lived CTAs: a warp takes a few consecutive rows (of one mask row where possible) and exits
    // about 32 rows per warp (measured optimum on B200: fewer leaves the two-slot pipeline mostly in its
    // prologue, many more lets the single resident CTA per SM run as one long wave), rounded so that the
    // CTAs fill whole waves
    const int64_t waves = std::max<int64_t>(1, (p.rows + (int64_t)sms * kStWarps * 16) / ((int64_t)sms * kStWarps * 32));
    const int rpw = (int)((p.rows + (int64_t)sms * kStWarps * waves - 1) / ((int64_t)sms * kStWarps * waves));
    const int64_t warps = (p.rows + rpw - 1) / rpw;
    const int64_t grid = (warps + kStWarps - 1) / kStWarps;
    if (dims) {
      dims->grid[0] = (unsigned)grid;
      dims->block[0] = kStWarps * 32;
      dims->smem = kStSmem;
    }
    SoftmaxParams q = p;
    if (!q.has_scale) q.scale = 1.0f;
    if (!q.has_mask) q.mask_rows = 1;
    if (p.in_dt == kF16)
      softmax_rows_staged_kernel<kF16><<<(unsigned)grid, kStWarps * 32, kStSmem, s>>>(
          q, (const uint16_t*)x, (const uint16_t*)mask, (uint16_t*)out, err_word, rpw);
    else
      softmax_rows_staged_kernel<kBF16><<<(unsigned)grid, kStWarps * 32, kStSmem, s>>>(
          q, (const uint16_t*)x, (const uint16_t*)mask, (uint16_t*)out, err_word, rpw);
    return cudaGetLastError();
  }
  if (vec) {
    const int64_t want = (p.rows + kWarpsPerCta - 1) / kWarpsPerCta;
    const int grid = (int)std::min<int64_t>(want, (int64_t)sms * 8);
    if (dims) {
      dims->grid[0] = grid;
      dims->block[0] = kWarpsPerCta * 32;
    }
    const int64_t v = (p.cols + 255) / 256;
#define AKGB_SM(V) softmax_rows_kernel<V><<<grid, kWarpsPerCta * 32, 0, s>>>(p, x, mask, out)
    if (v <= 1) AKGB_SM(1);
    else if (v <= 2) AKGB_SM(2);
    else if (v <= 4) AKGB_SM(4);
    else if (v <= 8) AKGB_SM(8);
    else AKGB_SM(16);
#undef AKGB_SM
  } else {
    const int grid = (int)std::min<int64_t>(p.rows, (int64_t)sms * 8);
    if (dims) {
      dims->grid[0] = grid;
      dims->block[0] = 256;
    }
    softmax_rows_generic_kernel<<<grid, 256, 0, s>>>(p, x, mask, out);
  }
  return cudaGetLastError();
}

}  // namespace akgb
