// Matmul class: C = A x B with the bias / ReLU / cast epilogue fused, on the
// 5th-generation tensor cores (tcgen05) with the accumulator in tensor memory.
//
// The reference lowers MatMul to a plain linalg loop nest that the GPU mapping
// spreads over CUDA cores (akg-mlir/lib/Conversion/MindSporeToLinalg/MindSporeToLinalg.cpp:1453-1546),
// with the epilogue ops fused elementwise behind it.  Here:
//   * one persistent CTA per SM walks 128x256 output tiles;
//   * warp 0 streams 128x64 (A) and 64x256 (B) bf16 tiles through a 4-stage
//     shared-memory ring with TMA (tiled tensor-map copies, 128-byte swizzle;
//     every CTA fetches its own tiles);
//   * warp 1 issues tcgen05.mma (M=128, N=256, K=16) into one of two 256-column
//     TMEM accumulators, so the epilogue of tile i overlaps the MMAs of tile i+1;
//   * warps 2-5 read the accumulator with tcgen05.ld, add the bias in f32,
//     apply max(.,0), round to the output type and store.
// Accumulation is f32 (the description gives MatMul an f32 result); bias Add,
// Maximum and Cast follow in that order, one rounding each.
//
// Two variants share the epilogue: a single-CTA kernel (128x256 tiles, used when M <= 128) and a CTA-pair
// kernel (tcgen05 cta_group::2, 256x256 tiles over two SMs, 5-stage ring, 16-bit results stored through shared memory by tensor-map stores), which is the default.
//
// Every wait on an mbarrier is bounded: when a limit is hit the kernel writes
// an error word, drains its copies and MMAs, frees its TMEM and returns.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>

#include "async.cuh"
#include "common.cuh"
#include "kernels.hpp"

namespace akgb {
namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;          // 16 KiB
constexpr int B_BYTES = BN * BK * 2;          // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int B_BOX_N = 64;                   // N-major B arrives as 4 boxes of 64(n) x 64(k)
constexpr int B_BOX_BYTES = B_BOX_N * BK * 2; // 8 KiB
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int THREADS = 192;

struct Bars {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t drain;
  uint32_t tmem_base;
  uint32_t abort;
};

struct MatmulDev {
  int M, N, K;
  int transpose_b, has_bias, bias_dt, relu, out_dt;
  int in_f16;  // operands are float16 instead of bfloat16
  int batch;             // independent products; tensor maps are 3-D with the batch outermost
  int b_batched;         // 0: every batch entry multiplies by the same B
  long long out_stride;  // elements between the outputs of consecutive batch entries
  const void* bias;
  void* out;
  uint32_t* err;
  uint32_t b_lbo, b_sbo;  // descriptor offsets of the N-major B tile, in bytes
};

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor (sm_100): start address, leading/stride byte
// offsets in 16-byte units, version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int* m_tile, int* n_tile) {
  // groups of 16 M-tiles sweep N together, so that the CTAs running at the
  // same time share A and B tiles in L2
  constexpr int G = 16;
  const int per_group = G * num_n;
  const int group = tile / per_group;
  const int first_m = group * G;
  const int rows = min(G, num_m - first_m);
  const int in_group = tile - group * per_group;
  *m_tile = first_m + in_group % rows;
  *n_tile = in_group / rows;
}

// Bias, then ReLU, on the 32 accumulator columns starting at col0 (this lane's row); columns at or beyond N keep
// whatever the accumulator held and are never stored.
__device__ __forceinline__ void epilogue_values(const MatmulDev& p, const uint32_t* r, int col0, float* v) {
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
  if (p.has_bias) {
    if (col0 + 32 <= p.N) {
      if (p.bias_dt != kF32) {
        const uint4* bp = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.bias) + col0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float b8[8];
          unpack8(__ldg(bp + q), p.bias_dt, b8);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[q * 8 + j] = __fadd_rn(v[q * 8 + j], b8[j]);
        }
      } else {
        const float4* bp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.bias) + col0);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float4 b = __ldg(bp + q);
          v[q * 4 + 0] = __fadd_rn(v[q * 4 + 0], b.x);
          v[q * 4 + 1] = __fadd_rn(v[q * 4 + 1], b.y);
          v[q * 4 + 2] = __fadd_rn(v[q * 4 + 2], b.z);
          v[q * 4 + 3] = __fadd_rn(v[q * 4 + 3], b.w);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (col0 + j < p.N) {
          const float b = p.bias_dt == kBF16
                              ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(p.bias)[col0 + j])
                              : p.bias_dt == kF16 ? __half2float(reinterpret_cast<const __half*>(p.bias)[col0 + j])
                                                  : reinterpret_cast<const float*>(p.bias)[col0 + j];
          v[j] = __fadd_rn(v[j], b);
        }
      }
    }
  }
  if (p.relu) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = v[j] != v[j] ? v[j] : fmaxf(v[j], 0.f);  // NaN stays NaN
  }
}

// Reads one 128x256 accumulator (this warp's 32 lanes) in chunks of 32 columns, applies bias / ReLU / cast in
// that order and stores the row segment.
__device__ __forceinline__ void epilogue_tile(const MatmulDev& p, uint32_t taddr, int row, int n0, size_t out_off) {
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(taddr + c * 32, r);
    tmem_ld_wait();
    const int col0 = n0 + c * 32;
    if (col0 >= p.N) continue;
    float v[32];
    epilogue_values(p, r, col0, v);
    if (row < p.M) {
      if (p.out_dt != kF32) {
        uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + out_off + (size_t)row * p.N + col0;
        if (col0 + 32 <= p.N) {
#pragma unroll
          for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(o + q * 8) = pack8(v + q * 8, p.out_dt);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N)
              o[j] = p.out_dt == kBF16 ? (uint16_t)f32_to_bf16_bits(v[j]) : __half_as_ushort(__float2half_rn(v[j]));
        }
      } else {
        float* o = reinterpret_cast<float*>(p.out) + out_off + (size_t)row * p.N + col0;
        if (col0 + 32 <= p.N) {
#pragma unroll
          for (int q = 0; q < 8; ++q)
            *reinterpret_cast<float4*>(o + q * 4) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) o[j] = v[j];
        }
      }
    }
  }
}

// The same for a 16-bit result, through shared memory: the warp's 32 rows x 256 columns are laid out as four boxes of
// 32 rows x 64 columns (128-byte rows in the 128-byte swizzle: 16-byte chunk c of row r sits at chunk c ^ (r & 7), so
// the 32 lanes' 16-byte stores of one instruction touch every bank once), which four tensor-map stores then write as
// whole 128-byte lines; rows at or beyond M and columns at or beyond N are clipped by the tensor map.
__device__ __forceinline__ void epilogue_tile_staged(const MatmulDev& p, uint32_t taddr, uint32_t stage_smem, int lane,
                                                     int n0) {
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(taddr + c * 32, r);
    tmem_ld_wait();
    const int col0 = n0 + c * 32;
    if (col0 >= p.N) continue;
    float v[32];
    epilogue_values(p, r, col0, v);
    const uint32_t row_smem = stage_smem + (uint32_t)(c >> 1) * 4096u + (uint32_t)lane * 128u;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint4 w = pack8(v + q * 8, p.out_dt);
      const uint32_t chunk = (uint32_t)(((c & 1) * 4 + q) ^ (lane & 7));
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_smem + chunk * 16u), "r"(w.x), "r"(w.y), "r"(w.z),
                   "r"(w.w)
                   : "memory");
    }
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the stores above become visible to the bulk copies
}
// `policy`: the result is written once and not read again by this kernel, so its lines are the first to leave L2 and
// the operands, which every CTA pair of a wave re-reads, stay
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z, uint64_t policy) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3, %4}], [%1], %5;" ::"l"(map),
               "r"(src), "r"(x), "r"(y), "r"(z), "l"(policy)
               : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the bulk stores issued by this thread have finished reading shared memory
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__global__ void __launch_bounds__(THREADS, 1)
matmul_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                           const MatmulDev p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  Bars* bars = reinterpret_cast<Bars*>(smem + STAGES * STAGE_BYTES);
  volatile uint32_t* abort_flag = &bars->abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bars->tmem_full[a]), 1);
      mbar_init(smem_u32(&bars->tmem_empty[a]), 4);  // one arrival per epilogue warp
    }
    mbar_init(smem_u32(&bars->drain), 1);
    bars->abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  const int per_batch = num_m * num_n;
  const int num_tiles = per_batch * p.batch;
  const int num_k = (p.K + BK - 1) / BK;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------ TMA producer
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int issued = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mt, nt;
        const int bt = tile / per_batch;
        tile_coords(tile - bt * per_batch, num_m, num_n, &mt, &nt);
        const int m0 = mt * BM, n0 = nt * BN, bz = p.b_batched ? bt : 0;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bars->full[stage]);
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
          mbar_expect_tx(full, STAGE_BYTES);
          tma_load_3d(sa, &tmA, full, kb * BK, m0, bt);
          if (p.transpose_b) {
            tma_load_3d(sb, &tmB, full, kb * BK, n0, bz);
          } else {
#pragma unroll
            for (int j = 0; j < BN / B_BOX_N; ++j)
              tma_load_3d(sb + j * B_BOX_BYTES, &tmB, full, n0 + j * B_BOX_N, kb * BK, bz);
          }
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicOr(p.err, 1u);
        // let the copies already issued land before the CTA gives up its shared memory
        const int pending = min(issued, STAGES);
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < pending; ++i) {
          if (--s < 0) {
            s = STAGES - 1;
            ph ^= 1u;
          }
          mbar_wait(smem_u32(&bars->full[s]), ph, nullptr);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------ MMA issuer
      const uint32_t fmt = p.in_f16 ? 0u : 1u;  // operand format field: 0 = f16, 1 = bf16
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((p.transpose_b ? 0u : 1u) << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(smem_u32(&bars->tmem_empty[acc]), acc_phase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)acc * BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // A, K-major: 8-row groups are 1024 B apart; 16 elements of K = 32 B inside the swizzled row
            const uint64_t adesc = make_desc(sa + k * 32, 16, 1024);
            const uint64_t bdesc = p.transpose_b ? make_desc(sb + k * 32, 16, 1024)
                                                 : make_desc(sb + k * 2048, p.b_lbo, p.b_sbo);
            umma_f16(tmem_d, adesc, bdesc, idesc, (kb | k) != 0);
          }
          umma_commit(smem_u32(&bars->empty[stage]));  // frees the stage once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(smem_u32(&bars->tmem_full[acc]));
        if ((acc ^= 1) == 0) acc_phase ^= 1u;
      }
      if (!ok) {
        *abort_flag = 1;
        atomicOr(p.err, 2u);
      }
      // every MMA issued has completed before TMEM is released
      umma_commit(smem_u32(&bars->drain));
      mbar_wait(smem_u32(&bars->drain), 0, nullptr);
    }
  } else {
    // -------------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 are visible to this warp
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int mt, nt;
      const int bt = tile / per_batch;
      tile_coords(tile - bt * per_batch, num_m, num_n, &mt, &nt);
      const int row = mt * BM + quarter * 32 + lane;
      const int n0 = nt * BN;
      if (!mbar_wait(smem_u32(&bars->tmem_full[acc]), acc_phase, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)acc * BN;
      epilogue_tile(p, taddr, row, n0, (size_t)bt * (size_t)p.out_stride);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->tmem_empty[acc]));
      if ((acc ^= 1) == 0) acc_phase ^= 1u;
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      atomicOr(p.err, 4u);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------ CTA-pair variant
// Two CTAs of a cluster (two SMs) work on one 256x256 tile: each loads its own 128 rows of A and its own 128
// columns of B, the pair's leader issues tcgen05.mma.cta_group::2 (M=256, N=256, K=16) that reads both CTAs'
// shared memory, and each CTA's TMEM receives its 128 rows of the accumulator.  Per CTA a stage is 32 KiB
// instead of 48, so the ring is 6 deep, and B is fetched from L2 once per pair.  Every CTA issues its own plain
// tensor-map copies; only the MMA-completion signal (tcgen05.commit) is delivered to both CTAs' barriers.
constexpr int STAGES2 = 5;
constexpr int B2_BYTES = (BN / 2) * BK * 2;             // this CTA's half of B: 16 KiB
constexpr int STAGE2_BYTES = A_BYTES + B2_BYTES;        // 32 KiB
constexpr int OUT_STAGE_BYTES = 32 * BN * 2;                  // one epilogue warp's 32 rows x 256 columns of a 16-bit result
constexpr int SMEM2_BYTES = STAGES2 * STAGE2_BYTES + 4 * OUT_STAGE_BYTES + 1024 + 512;
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;             // shared::cluster address of the same offset in the pair's leader

struct Bars2 {
  uint64_t full[STAGES2];    // leader's copy is the one in use: both CTAs' loads complete on it
  uint64_t empty[STAGES2];   // per CTA: the leader's commit signals both CTAs
  uint64_t tmem_full[2];     // per CTA: same
  uint64_t tmem_empty[2];    // leader's copy in use: 8 arrivals (4 epilogue warps x 2 CTAs)
  uint64_t drain;
  uint32_t tmem_base;
  uint32_t abort;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar, int x, int y,
                                                 int z, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(dst), "l"(map), "r"(leader_bar), "r"(x), "r"(y), "r"(z), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the barrier at this offset in BOTH CTAs of the pair once the MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(mask)
               : "memory");
}
// same completion signal, delivered to the issuing CTA's barrier only
__device__ __forceinline__ void umma_commit_pair_local(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// arrive on the barrier at the same shared-memory offset in CTA `target_rank` of the cluster
__device__ __forceinline__ void mbar_arrive_remote(uint32_t local_addr, uint32_t target_rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(target_rank));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
matmul_bf16_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                const __grid_constant__ CUtensorMap tmC, const MatmulDev p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  Bars2* bars = reinterpret_cast<Bars2*>(smem + STAGES2 * STAGE2_BYTES + 4 * OUT_STAGE_BYTES);
  volatile uint32_t* abort_flag = &bars->abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bars->tmem_full[a]), 1);
      mbar_init(smem_u32(&bars->tmem_empty[a]), 8);
    }
    mbar_init(smem_u32(&bars->drain), 1);
    bars->abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {  // both CTAs of the pair execute the paired allocation
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  const int num_m = (p.M + 2 * BM - 1) / (2 * BM), num_n = (p.N + BN - 1) / BN;  // 256 x 256 tiles
  const int per_batch = num_m * num_n;
  const int num_tiles = per_batch * p.batch;
  const int num_k = (p.K + BK - 1) / BK;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------ TMA producer (both CTAs)
      const uint64_t load_policy = l2_policy_evict_last();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int mt, nt;
        const int bt = tile / per_batch;
        tile_coords(tile - bt * per_batch, num_m, num_n, &mt, &nt);
        const int m0 = mt * 2 * BM + (int)rank * BM, n0 = nt * BN + (int)rank * (BN / 2), bz = p.b_batched ? bt : 0;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t full_leader = smem_u32(&bars->full[stage]) & kPeerMask;
          const uint32_t sa = base + stage * STAGE2_BYTES, sb = sa + A_BYTES;
          if (leader) mbar_expect_tx(smem_u32(&bars->full[stage]), 2 * STAGE2_BYTES);
          tma_load_3d_pair(sa, &tmA, full_leader, kb * BK, m0, bt, load_policy);
          if (p.transpose_b) {
            tma_load_3d_pair(sb, &tmB, full_leader, kb * BK, n0, bz, load_policy);
          } else {
#pragma unroll
            for (int j = 0; j < (BN / 2) / B_BOX_N; ++j)
              tma_load_3d_pair(sb + j * B_BOX_BYTES, &tmB, full_leader, n0 + j * B_BOX_N, kb * BK, bz, load_policy);
          }
          if (++stage == STAGES2) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicOr(p.err, 1u);
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // bounded grace period for copies already issued
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ------------------------------------------------------------ MMA issuer (leader CTA only)
      const uint32_t fmt = p.in_f16 ? 0u : 1u;  // operand format field: 0 = f16, 1 = bf16
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((p.transpose_b ? 0u : 1u) << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        if (!mbar_wait(smem_u32(&bars->tmem_empty[acc]), acc_phase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)acc * BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = base + stage * STAGE2_BYTES, sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = make_desc(sa + k * 32, 16, 1024);
            const uint64_t bdesc = p.transpose_b ? make_desc(sb + k * 32, 16, 1024)
                                                 : make_desc(sb + k * 2048, p.b_lbo, p.b_sbo);
            umma_f16_pair(tmem_d, adesc, bdesc, idesc, (kb | k) != 0);
          }
          umma_commit_pair(smem_u32(&bars->empty[stage]));  // frees the stage in both CTAs
          if (++stage == STAGES2) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_pair(smem_u32(&bars->tmem_full[acc]));  // both CTAs' epilogues may read their halves
        if ((acc ^= 1) == 0) acc_phase ^= 1u;
      }
      if (!ok) {
        *abort_flag = 1;
        atomicOr(p.err, 2u);
      }
      umma_commit_pair_local(smem_u32(&bars->drain));
      mbar_wait(smem_u32(&bars->drain), 0, nullptr);
    }
  } else {
    // -------------------------------------------------------------- epilogue (both CTAs, own 128 rows)
    const int quarter = warp & 3;
    const bool staged = p.out_dt != kF32;  // 16-bit results leave through shared memory and tensor-map stores
    const uint64_t store_policy = l2_policy_evict_first();
    const uint32_t out_smem = base + STAGES2 * STAGE2_BYTES + (uint32_t)quarter * OUT_STAGE_BYTES;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      int mt, nt;
      const int bt = tile / per_batch;
      tile_coords(tile - bt * per_batch, num_m, num_n, &mt, &nt);
      const int row = mt * 2 * BM + (int)rank * BM + quarter * 32 + lane;
      const int n0 = nt * BN;
      if (!mbar_wait(smem_u32(&bars->tmem_full[acc]), acc_phase, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)acc * BN;
      if (staged) {
        if (lane == 0) bulk_wait_read();  // the previous tile's stores have read this warp's staging area
        __syncwarp();
        epilogue_tile_staged(p, taddr, out_smem, lane, n0);
      } else {
        epilogue_tile(p, taddr, row, n0, (size_t)bt * (size_t)p.out_stride);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_remote(smem_u32(&bars->tmem_empty[acc]), 0);  // the accumulator is read: the next tile may use it
        if (staged) {
          const int row0 = row - lane;
          if (row0 < p.M) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              if (n0 + j * 64 < p.N) tma_store_3d(&tmC, out_smem + (uint32_t)j * 4096u, n0 + j * 64, row0, bt, store_policy);
          }
          bulk_commit();
        }
      }
      if ((acc ^= 1) == 0) acc_phase ^= 1u;
    }
    if (staged && lane == 0) bulk_wait_all();
    if (!ok && lane == 0) {
      *abort_flag = 1;
      atomicOr(p.err, 4u);
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA releases TMEM or exits while its peer may still use it
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 3-D tensor map over 16-bit elements: `batch` matrices of `outer` rows of `inner` contiguous elements, one matrix
// after the other; a box never spans two matrices, so rows beyond `outer` read as zeros in every batch entry.
bool encode_3d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t batch, uint32_t box_inner,
               uint32_t box_outer, bool f16) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {inner, outer, batch};
  cuuint64_t strides[2] = {inner * 2, inner * outer * 2};
  cuuint32_t box[3] = {box_inner, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace

bool matmul_bf16_supported(const MatmulParams& p, const char** why) {
  const char* w = nullptr;
  if (p.M <= 0 || p.N <= 0 || p.K <= 0) w = "empty extent";
  else if (p.K % 8 != 0) w = "K must be a multiple of 8 (16-byte TMA row pitch)";
  else if (p.N % 8 != 0) w = "N must be a multiple of 8 (16-byte rows of B and of the output)";
  else if (p.M > (1 << 30) || p.N > (1 << 30) || p.K > (1 << 30)) w = "extent above 2^30";
  if (why) *why = w;
  return w == nullptr;
}

cudaError_t matmul_bf16(const MatmulParams& p, const void* A, const void* B, const void* bias, void* out,
                        int64_t batch, bool b_batched, uint32_t* err_word, int sm_count, cudaStream_t s,
                        LaunchDims* dims) {
  if (batch < 1 || batch > (1 << 20)) return cudaErrorInvalidValue;
  const uint64_t bb = b_batched ? (uint64_t)batch : 1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(bias)) & 15)
    return cudaErrorMisalignedAddress;
  CUtensorMap tmA, tmB;
  const bool f16 = p.in_dt == kF16;
  if (!encode_3d(&tmA, A, (uint64_t)p.K, (uint64_t)p.M, (uint64_t)batch, BK, BM, f16)) return cudaErrorInvalidValue;
  const bool okb = p.transpose_b ? encode_3d(&tmB, B, (uint64_t)p.K, (uint64_t)p.N, bb, BK, BN, f16)
                                 : encode_3d(&tmB, B, (uint64_t)p.N, (uint64_t)p.K, bb, B_BOX_N, BK, f16);
  if (!okb) return cudaErrorInvalidValue;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(matmul_bf16_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    SMEM_BYTES);
  });
  if (attr_err != cudaSuccess) return attr_err;
  MatmulDev d;
  d.M = (int)p.M;
  d.N = (int)p.N;
  d.K = (int)p.K;
  d.transpose_b = p.transpose_b;
  d.has_bias = p.has_bias;
  d.bias_dt = p.bias_dt;
  d.relu = p.relu;
  d.out_dt = p.out_dt;
  d.in_f16 = f16;
  d.batch = (int)batch;
  d.b_batched = b_batched ? 1 : 0;
  d.out_stride = (long long)p.M * p.N;
  d.bias = bias;
  d.out = out;
  d.err = err_word;
  // N-major B tile: 64-element N atoms are one TMA box (8 KiB) apart, 8-row K groups 1 KiB apart
  d.b_lbo = B_BOX_BYTES;
  d.b_sbo = 1024;
  // two-CTA tiles whenever there is more than one 128-row block and the device has SM pairs to run them
  if (p.M > BM && sm_count >= 2) {
    static std::once_flag once2;
    static cudaError_t attr_err2 = cudaSuccess;
    std::call_once(once2, [] {
      attr_err2 = cudaFuncSetAttribute(matmul_bf16_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       SMEM2_BYTES);
    });
    if (attr_err2 != cudaSuccess) return attr_err2;
    // the pair kernel's B tile per CTA is 128 columns: re-encode B with the narrower box for the K-major case
    CUtensorMap tmB2 = tmB;
    if (p.transpose_b && !encode_3d(&tmB2, B, (uint64_t)p.K, (uint64_t)p.N, bb, BK, BN / 2, f16)) return cudaErrorInvalidValue;
    const int64_t tiles2 = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + BN - 1) / BN) * batch;
    const int grid2 = 2 * (int)std::min<int64_t>(tiles2, sm_count / 2);
    if (dims) {
      dims->grid[0] = grid2;
      dims->block[0] = THREADS;
      dims->smem = SMEM2_BYTES;
    }
    // 16-bit results: the output as boxes of 64 columns x 32 rows (one epilogue warp's share of a 128-byte-swizzled box)
    CUtensorMap tmC;
    std::memset(&tmC, 0, sizeof(tmC));
    if (p.out_dt != kF32 &&
        !encode_3d(&tmC, out, (uint64_t)p.N, (uint64_t)p.M, (uint64_t)batch, 64, 32, p.out_dt == kF16))
      return cudaErrorInvalidValue;
    matmul_bf16_tcgen05_pair_kernel<<<grid2, THREADS, SMEM2_BYTES, s>>>(tmA, tmB2, tmC, d);
    return cudaGetLastError();
  }
  const int64_t tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * batch;
  const int grid = (int)std::min<int64_t>(tiles, sm_count);
  if (dims) {
    dims->grid[0] = grid;
    dims->block[0] = THREADS;
    dims->smem = SMEM_BYTES;
  }
  matmul_bf16_tcgen05_kernel<<<grid, THREADS, SMEM_BYTES, s>>>(tmA, tmB, d);
  return cudaGetLastError();
}

}  // namespace akgb
