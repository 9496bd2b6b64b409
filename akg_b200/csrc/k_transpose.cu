// Transpose class: bit-exact permutation copies.
//
// The host folds the permutation (extent-1 axes dropped, axes that stay
// adjacent merged) into at most 6 output dims with an input stride each.  Two
// kernels cover every case:
//   * row mode — the innermost output dim is also contiguous in the input, so
//     the copy moves 16-byte vectors and both sides are coalesced;
//   * tile mode — the innermost output dim is strided in the input: tiles go
//     through shared memory so that reads run along the input's contiguous
//     axis and writes along the output's (the reference maps a 32x32 thread
//     tile onto the same two axes,
//     akg-mlir/lib/Analysis/TilingStrategy.cpp:330-408).  2- and 4-byte
//     elements move as 16-byte loads and 128-byte stores through a
//     conflict-free transposed block (transpose_tile_vec_kernel: 6.0-6.7 TB/s
//     measured on B200, at the copy bandwidth); other sizes and unaligned
//     shapes use 32x33 element tiles.
#include <algorithm>

#include "common.cuh"
#include "kernels.hpp"

namespace akgb {
namespace {

struct Shape6 {
  int rank;
  int64_t ext[6];
  int64_t istr[6];
};

// Division by a run-time constant as multiply-high + shift; exact for
// numerators below 2^31.
struct FastDiv6 {
  uint32_t mul[6];
  uint32_t shr[6];
};
inline void fastdiv_init(uint32_t d, uint32_t* mul, uint32_t* shr) {
  if (d <= 1) {
    *mul = 0;
    *shr = 0;
    return;
  }
  uint32_t sh = 0;
  while ((1ull << sh) < d) ++sh;
  *shr = sh;
  *mul = (uint32_t)((((1ull << 32) * ((1ull << sh) - d)) / d) + 1);
}

// row mode: 16-byte vectors, 4 per thread.  FAST: the vector count fits 31 bits, so the index split
// uses 32-bit multiply-shift.
template <bool FAST>
__global__ void __launch_bounds__(256) transpose_rows_kernel(Shape6 sh, FastDiv6 fd, const uint4* __restrict__ x,
                                                             uint4* __restrict__ out, int64_t nvec) {
  // one-shot CTAs (no grid-stride loop): each owns 1024 consecutive output vectors, 4 per thread,
  // all four loads issued before the first store
  const int64_t base = (int64_t)blockIdx.x * 1024 + threadIdx.x;
  uint4 v[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int64_t o = base + u * 256;
    if (o < nvec) {
      int64_t off = 0;
      if (FAST) {
        uint32_t rem = (uint32_t)o, acc = 0;
#pragma unroll
        for (int d = 5; d >= 0; --d) {
          if (d < sh.rank) {
            const uint32_t q = (__umulhi(rem, fd.mul[d]) + rem) >> fd.shr[d];
            acc += (rem - q * (uint32_t)sh.ext[d]) * (uint32_t)sh.istr[d];
            rem = q;
          }
        }
        off = acc;
      } else {
        int64_t rem = o;
#pragma unroll
        for (int d = 5; d >= 0; --d) {
          if (d < sh.rank) {
            const int64_t q = rem / sh.ext[d];
            off += (rem - q * sh.ext[d]) * sh.istr[d];
            rem = q;
          }
        }
      }
      v[u] = ld_stream(x + off);
    }
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int64_t o = base + u * 256;
    if (o < nvec) st_stream(out + o, v[u]);
  }
}

// tile mode over elements of T; dim `pin` of the output is the input's contiguous axis
template <typename T>
__global__ void __launch_bounds__(256) transpose_tile_kernel(Shape6 sh, int pin, const T* __restrict__ x,
                                                             T* __restrict__ out, int64_t ostr_pin) {
  __shared__ T tile[32][33];
  const int last = sh.rank - 1;
  const int64_t W = sh.ext[last], H = sh.ext[pin];
  const int64_t w0 = (int64_t)blockIdx.x * 32, h0 = (int64_t)blockIdx.y * 32;
  // batch offset from blockIdx.z over the remaining dims
  int64_t rem = blockIdx.z, ioff = 0, ooff = 0, ostride = 1;
  // output strides: contiguous row-major over sh.ext
  int64_t ostr[6];
  for (int d = sh.rank - 1; d >= 0; --d) {
    ostr[d] = ostride;
    ostride *= sh.ext[d];
  }
  for (int d = sh.rank - 2; d >= 0; --d) {
    if (d == pin) continue;
    const int64_t q = rem / sh.ext[d];
    const int64_t i = rem - q * sh.ext[d];
    ioff += i * sh.istr[d];
    ooff += i * ostr[d];
    rem = q;
  }
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  // read: threads run along the input-contiguous axis (h)
  for (int r = ty; r < 32; r += 8) {
    const int64_t w = w0 + r, h = h0 + tx;
    if (w < W && h < H) tile[r][tx] = x[ioff + w * sh.istr[last] + h];
  }
  __syncthreads();
  // write: threads run along the output-contiguous axis (w)
  for (int r = ty; r < 32; r += 8) {
    const int64_t h = h0 + r, w = w0 + tx;
    if (w < W && h < H) out[ooff + h * ostr_pin + w] = tile[tx][r];
  }
}

// tile mode for 2- and 4-byte elements with vector traffic on both sides.  A CTA moves a block of NW x NH base
// tiles; a base tile is 32 words of an output row (w, strided in the input: 64 two-byte or 32 four-byte elements) by
// 128 bytes of an input row (h, contiguous in the input).  With NH = NW = 2 every visit of an input row reads 256
// contiguous bytes and every output row gets 256, and a CTA moves 16 or 32 KB instead of 4 or 8.
//   in : every thread loads 16 bytes along h (consecutive lanes cover 128 or 64 contiguous bytes of an input row;
//        two-byte elements: the same piece of rows w and w+1, whose halves a byte permute interleaves into words that
//        hold (w, w+1) for one h) and scatters them as 32-bit words into a transposed block in shared memory whose
//        pitch is 1 word more than a multiple of 32: conflict-free;
//   out: every warp reads rows of the transposed block (32 consecutive words per instruction) and stores them as
//        128-byte lines of the output.
// Requirements (checked by the host, else transpose_tile_kernel): h extent, input strides and base allow 16-byte
// loads; two-byte elements: even w extent.  Ragged blocks are predicated per vector / per word.
// the batch dims of a tile-mode transpose (every output dim but the two that are transposed), innermost first
struct TileBatch {
  int n;
  int64_t ext[4], istr[4], ostr[4];
};

template <int ES, int NH, int NW>
__global__ void __launch_bounds__(256, 4) transpose_tile_vec_kernel(TileBatch tb, int64_t W, int64_t H, int64_t sw,
                                                                 const uint8_t* __restrict__ x,
                                                                 uint8_t* __restrict__ out, int64_t ostr_pin) {
  constexpr int TH = ES == 2 ? 64 : 32;  // base tile extent along h (128 bytes of an input row)
  constexpr int TW = ES == 2 ? 64 : 32;  // base tile extent along w: 32 words of an output row
  constexpr int VH = 16 / ES;            // elements per 16-byte load
  constexpr int PITCH = 32 * NW + 1;
  extern __shared__ uint32_t tile[];     // [TH * NH][PITCH]
  const int64_t w0 = (int64_t)blockIdx.x * TW * NW, h0 = (int64_t)blockIdx.y * TH * NH;
  int64_t rem = blockIdx.z, ioff = 0, ooff = 0;
#pragma unroll
  for (int d = 0; d < 4; ++d) {
    if (d < tb.n) {
      const int64_t q = rem / tb.ext[d];
      const int64_t i = rem - q * tb.ext[d];
      ioff += i * tb.istr[d];
      ooff += i * tb.ostr[d];
      rem = q;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // ---- in: lanes = 8 h-chunks x 4 word columns, so a warp instruction reads 128 contiguous bytes of 4 input rows
  // and scatters 32 words whose banks (row * PITCH + column, PITCH = 1 mod 32) are all different:
  //   4-byte elements: rows 4c + e, columns 4 * warp + q: banks 4c + q + const;
  //   2-byte elements: rows 8c + 2e + k: chunks c and c + 4 would meet in a bank, so the upper four chunks store to
  //   column ^ 4 (the rows of those chunks are read back with the same flip).
  const int c = lane & 7;                  // 16-byte chunk along h
  const int wc = warp * 4 + (lane >> 3);   // word column of a base tile (one w for 4-byte elements, a pair for 2-byte)
  const int flip = ES == 2 ? (c & 4) : 0;
  uint4 va[NH][NW], vb[NH][NW];
#pragma unroll
  for (int ih = 0; ih < NH; ++ih) {
#pragma unroll
    for (int iw = 0; iw < NW; ++iw) {
      const int64_t h = h0 + ih * TH + c * VH;
      const int64_t w = w0 + iw * TW + (ES == 4 ? wc : 2 * wc);
      va[ih][iw] = make_uint4(0, 0, 0, 0);
      vb[ih][iw] = make_uint4(0, 0, 0, 0);
      if (w < W && h < H) {  // two-byte elements: W is even, so w + 1 < W as well
        va[ih][iw] = ld_stream(x + (ioff + w * sw + h) * ES);
        if (ES == 2) vb[ih][iw] = ld_stream(x + (ioff + (w + 1) * sw + h) * ES);
      }
    }
  }
#pragma unroll
  for (int ih = 0; ih < NH; ++ih) {
#pragma unroll
    for (int iw = 0; iw < NW; ++iw) {
      const uint4 a = va[ih][iw], b = vb[ih][iw];
      const int col = iw * 32 + (wc ^ flip);
      if (ES == 4) {
        uint32_t* t = tile + (ih * TH + c * 4) * PITCH + col;
        t[0] = a.x;
        t[PITCH] = a.y;
        t[2 * PITCH] = a.z;
        t[3 * PITCH] = a.w;
      } else {
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
        uint32_t* t = tile + (ih * TH + c * 8) * PITCH + col;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          // aw[e] = (row w: h+2e, h+2e+1), bw[e] = (row w+1: h+2e, h+2e+1)  ->  words (w, w+1) at h+2e and at h+2e+1
          t[(2 * e) * PITCH] = __byte_perm(aw[e], bw[e], 0x5410);
          t[(2 * e + 1) * PITCH] = __byte_perm(aw[e], bw[e], 0x7632);
        }
      }
    }
  }
  __syncthreads();
  // ---- out: warp -> rows h of the transposed block, lane -> word of the row
  const int64_t wwords = ES == 2 ? W / 2 : W;
  const int64_t word0 = ES == 2 ? w0 / 2 : w0;
  for (int r = warp; r < TH * NH; r += 8) {
    const int64_t h = h0 + r;
    if (h >= H) break;
    uint32_t* orow = reinterpret_cast<uint32_t*>(out + (ooff + h * ostr_pin) * ES);
#pragma unroll
    for (int iw = 0; iw < NW; ++iw) {
      const int64_t word = word0 + iw * 32 + lane;
      // two-byte elements: rows of the upper four chunks of a base tile were stored with column ^ 4
      const int pl = ES == 2 ? (lane ^ ((r >> 3) & 4)) : lane;
      if (word < wwords) __stcs(orow + word, tile[r * PITCH + iw * 32 + pl]);
    }
  }
}

// scalar fallback for anything else (odd element sizes are handled bytewise by the caller's esize)
template <typename T>
__global__ void __launch_bounds__(256) transpose_scalar_kernel(Shape6 sh, const T* __restrict__ x, T* __restrict__ out,
                                                               int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < n; o += stride) {
    int64_t rem = o, off = 0;
    for (int d = sh.rank - 1; d >= 0; --d) {
      const int64_t q = rem / sh.ext[d];
      off += (rem - q * sh.ext[d]) * sh.istr[d];
      rem = q;
    }
    out[o] = x[off];
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
cudaError_t tile_or_scalar(const Shape6& sh, const void* x, void* out, int sms, cudaStream_t s, LaunchDims* dims) {
  int64_t n = 1;
  for (int d = 0; d < sh.rank; ++d) n *= sh.ext[d];
  int pin = -1;
  for (int d = 0; d < sh.rank - 1; ++d)
    if (sh.istr[d] == 1) pin = d;
  if (pin >= 0 && sh.rank >= 2) {
    int64_t batch = 1, ostr_pin = 1;
    for (int d = 0; d < sh.rank - 1; ++d)
      if (d != pin) batch *= sh.ext[d];
    for (int d = sh.rank - 1; d > pin; --d) ostr_pin *= sh.ext[d];
    if (sizeof(T) == 2 || sizeof(T) == 4) {
      // vector traffic on both sides when the extents and strides allow 16-byte loads along h and word stores along w
      constexpr int ES = (int)sizeof(T), VH = 16 / ES, TT = ES == 2 ? 64 : 32, NB = 2;
      const int64_t W = sh.ext[sh.rank - 1], H = sh.ext[pin];
      bool ok = H % VH == 0 && aligned16(x) && (reinterpret_cast<uintptr_t>(out) & 3) == 0 && (ES == 4 || W % 2 == 0);
      for (int d = 0; d < sh.rank && ok; ++d)
        if (d != pin && sh.istr[d] % VH != 0) ok = false;
      const int64_t gx = (W + TT * NB - 1) / (TT * NB), gy = (H + TT * NB - 1) / (TT * NB);
      if (ok && gy <= 65535 && batch <= 65535) {
        dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)batch);
        const unsigned smem = 4u * TT * NB * (32 * NB + 1);
        if (dims) {
          dims->grid[0] = grid.x;
          dims->grid[1] = grid.y;
          dims->grid[2] = grid.z;
          dims->block[0] = 256;
          dims->smem = smem;
        }
        TileBatch tb;
        tb.n = 0;
        int64_t ostride = sh.ext[sh.rank - 1];
        for (int d = sh.rank - 2; d >= 0; --d) {
          if (d != pin) {
            if (tb.n < 4) {
              tb.ext[tb.n] = sh.ext[d];
              tb.istr[tb.n] = sh.istr[d];
              tb.ostr[tb.n] = ostride;
            }
            ++tb.n;
          }
          ostride *= sh.ext[d];
        }
        for (int d = tb.n; d < 4; ++d) tb.ext[d] = 1, tb.istr[d] = 0, tb.ostr[d] = 0;
        transpose_tile_vec_kernel<ES, NB, NB><<<grid, 256, smem, s>>>(tb, W, H, sh.istr[sh.rank - 1], (const uint8_t*)x,
                                                                      (uint8_t*)out, ostr_pin);
        return cudaGetLastError();
      }
    }
    const int64_t gx = (sh.ext[sh.rank - 1] + 31) / 32, gy = (sh.ext[pin] + 31) / 32;
    if (gy <= 65535 && batch <= 65535) {
      dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)batch);
      if (dims) {
        dims->grid[0] = grid.x;
        dims->grid[1] = grid.y;
        dims->grid[2] = grid.z;
        dims->block[0] = 256;
        dims->smem = sizeof(T) * 32 * 33;
      }
      transpose_tile_kernel<T><<<grid, 256, 0, s>>>(sh, pin, (const T*)x, (T*)out, ostr_pin);
      return cudaGetLastError();
    }
  }
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((n + 255) / 256, (int64_t)sms * 16));
  if (dims) {
    dims->grid[0] = grid;
    dims->block[0] = 256;
  }
  transpose_scalar_kernel<T><<<grid, 256, 0, s>>>(sh, (const T*)x, (T*)out, n);
  return cudaGetLastError();
}

}  // namespace

cudaError_t transpose_nd(const TransposeParams& p, const void* x, void* out, cudaStream_t s, LaunchDims* dims) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  Shape6 sh;
  sh.rank = p.rank;
  int64_t n = 1;
  for (int d = 0; d < 6; ++d) {
    sh.ext[d] = d < p.rank ? p.out_shape[d] : 1;
    sh.istr[d] = d < p.rank ? p.in_stride[d] : 0;
    n *= sh.ext[d];
  }
  if (n == 0) return cudaSuccess;
  const int last = p.rank - 1;
  const int per_vec = 16 / p.esize;
  bool row_mode = p.in_stride[last] == 1 && (p.out_shape[last] % per_vec) == 0 && aligned16(x) && aligned16(out);
  for (int d = 0; d < last && row_mode; ++d)
    if (p.in_stride[d] % per_vec != 0) row_mode = false;
  if (row_mode) {
    Shape6 v = sh;
    v.ext[last] = sh.ext[last] / per_vec;
    for (int d = 0; d < last; ++d) v.istr[d] = sh.istr[d] / per_vec;
    const int64_t nvec = n / per_vec;
    const unsigned grid = (unsigned)((nvec + 1023) / 1024);
    if (dims) {
      dims->grid[0] = grid;
      dims->block[0] = 256;
    }
    FastDiv6 fd;
    for (int d = 0; d < 6; ++d) fastdiv_init((uint32_t)std::min<int64_t>(v.ext[d], 0x7fffffff), &fd.mul[d], &fd.shr[d]);
    if (nvec < (1ll << 31))
      transpose_rows_kernel<true><<<grid, 256, 0, s>>>(v, fd, (const uint4*)x, (uint4*)out, nvec);
    else
      transpose_rows_kernel<false><<<grid, 256, 0, s>>>(v, fd, (const uint4*)x, (uint4*)out, nvec);
    return cudaGetLastError();
  }
  switch (p.esize) {
    case 1: return tile_or_scalar<uint8_t>(sh, x, out, sms, s, dims);
    case 2: return tile_or_scalar<uint16_t>(sh, x, out, sms, s, dims);
    case 4: return tile_or_scalar<uint32_t>(sh, x, out, sms, s, dims);
    case 8: return tile_or_scalar<uint64_t>(sh, x, out, sms, s, dims);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace akgb
