// Generic elementwise/broadcast kernel: interprets an EwProgram (ew_program.hpp)
// for fused regions that no specialised template covers.
//
// Semantics follow the reference lowering of elementwise ops
// (akg-mlir/lib/Conversion/MindSporeToLinalg/MindSporeToLinalg.cpp:377-483 and the TOSA table in
// akg-mlir/lib/Conversion/MindSporeToTosa/MindSporeToTosa.cpp:475-504): every op computes in its own element type.
// Floating types are held as f32 and rounded to the op's type after EVERY op (for + - * / sqrt an f32 operation
// rounded to f16/bf16 equals the operation done in that type; transcendentals use the accurate CUDA math library,
// as the reference's CPU route extends to f32, calls libm and truncates).  Operands broadcast by dropped or
// extent-1 dims (:432-459).  The register file lives in shared memory, one 32-bit slot per register, lane and
// element, so that register numbers can be data; each thread works on 4 elements per instruction decode.
#include <algorithm>

#include "common.cuh"
#include "ew_program.hpp"
#include "kernels.hpp"

namespace akgb {
namespace {

constexpr int kEwThreads = 256, kEwVec = 4;
enum : int { kBool = 0, kI8 = 1, kI16 = 2, kI32 = 3 };

struct EwPtrs {
  const void* in[kEwMaxIn];
  void* out[kEwMaxOut];
};

__device__ __forceinline__ float round_to(float x, int dt) {
  if (dt == kF16) return __half2float(__float2half_rn(x));
  if (dt == kBF16) return __bfloat162float(__float2bfloat16_rn(x));
  return x;
}
__device__ __forceinline__ int wrap_int(int x, int dt) {
  if (dt == kI8) return (int)(signed char)x;
  if (dt == kI16) return (int)(short)x;
  return x;
}

__device__ __forceinline__ uint32_t load_elem(const void* p, int64_t i, int dt) {
  switch (dt) {
    case kF32: return __float_as_uint(reinterpret_cast<const float*>(p)[i]);
    case kF16: return __float_as_uint(__half2float(reinterpret_cast<const __half*>(p)[i]));
    case kBF16: return ((uint32_t)reinterpret_cast<const uint16_t*>(p)[i]) << 16;
    case kI32: return (uint32_t)reinterpret_cast<const int*>(p)[i];
    case kI16: return (uint32_t)(int)reinterpret_cast<const short*>(p)[i];
    case kI8: return (uint32_t)(int)reinterpret_cast<const signed char*>(p)[i];
    default: return reinterpret_cast<const uint8_t*>(p)[i] != 0 ? 1u : 0u;  // bool
  }
}
__device__ __forceinline__ void store_elem(void* p, int64_t i, int dt, uint32_t bits) {
  switch (dt) {
    case kF32: reinterpret_cast<float*>(p)[i] = __uint_as_float(bits); break;
    case kF16: reinterpret_cast<__half*>(p)[i] = __float2half_rn(__uint_as_float(bits)); break;
    case kBF16: reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(__uint_as_float(bits)); break;
    case kI32: reinterpret_cast<int*>(p)[i] = (int)bits; break;
    case kI16: reinterpret_cast<short*>(p)[i] = (short)(int)bits; break;
    case kI8: reinterpret_cast<signed char*>(p)[i] = (signed char)(int)bits; break;
    default: reinterpret_cast<uint8_t*>(p)[i] = bits ? 1 : 0; break;
  }
}

__device__ __forceinline__ int64_t operand_index(const EwProgram& P, const EwOperand& o, int64_t e) {
  if (o.kind == EWI_FULL) return e;
  if (o.kind == EWI_SCALAR) return 0;
  if (o.kind == EWI_MOD) return e % o.mod;
  int64_t rem = e, idx = o.offset;
  for (int d = P.rank - 1; d >= 0; --d) {
    const int64_t q = rem / P.shape[d];
    int64_t i = rem - q * P.shape[d];
    if (o.wrap[d]) i %= o.wrap[d];
    idx += i * o.stride[d];
    rem = q;
  }
  return idx;
}

__device__ __forceinline__ float unary_f(int op, float x) {
  switch (op) {
    case EW_ABS: return fabsf(x);
    case EW_NEG: return -x;
    case EW_EXP: return expf(x);
    case EW_LOG: return logf(x);
    case EW_TANH: return tanhf(x);
    case EW_RSQRT: return __fdiv_rn(1.0f, __fsqrt_rn(x));
    case EW_SQRT: return __fsqrt_rn(x);
    case EW_RECIP: return __fdiv_rn(1.0f, x);
    case EW_FLOOR: return floorf(x);
    case EW_SQUARE: return __fmul_rn(x, x);
    case EW_SIN: return sinf(x);
    case EW_COS: return cosf(x);
    case EW_ASINH: return asinhf(x);
    case EW_ACOSH: return acoshf(x);
    case EW_ATAN: return atanf(x);
    case EW_ASIN: return asinf(x);
    case EW_ACOS: return acosf(x);
    default: return x;  // EW_COPY
  }
}
__device__ __forceinline__ float binary_f(int op, float a, float b) {
  switch (op) {
    case EW_ADD: return __fadd_rn(a, b);
    case EW_SUB: return __fsub_rn(a, b);
    case EW_MUL: return __fmul_rn(a, b);
    case EW_DIV: return __fdiv_rn(a, b);
    case EW_MAX: return (a != a || b != b) ? __int_as_float(0x7fc00000) : fmaxf(a, b);  // np.maximum keeps NaN
    case EW_MIN: return (a != a || b != b) ? __int_as_float(0x7fc00000) : fminf(a, b);
    case EW_POW: return powf(a, b);
    default: return atan2f(a, b);
  }
}
__device__ __forceinline__ int binary_i(int op, int a, int b) {
  switch (op) {
    case EW_ADD: return a + b;
    case EW_SUB: return a - b;
    case EW_MUL: return a * b;
    case EW_DIV: return b == 0 ? 0 : a / b;  // arith.divsi; division by zero is undefined there
    case EW_MAX: return max(a, b);
    default: return min(a, b);
  }
}
__device__ __forceinline__ bool compare_f(int op, float a, float b) {
  switch (op) {  // ordered comparisons: false on NaN, except NE
    case EW_EQ: return a == b;
    case EW_NE: return !(a == b);
    case EW_GT: return a > b;
    case EW_GE: return a >= b;
    case EW_LT: return a < b;
    default: return a <= b;
  }
}
__device__ __forceinline__ bool compare_i(int op, int a, int b) {
  switch (op) {
    case EW_EQ: return a == b;
    case EW_NE: return a != b;
    case EW_GT: return a > b;
    case EW_GE: return a >= b;
    case EW_LT: return a < b;
    default: return a <= b;
  }
}

__global__ void __launch_bounds__(kEwThreads) ew_generic_kernel(const __grid_constant__ EwProgram P, const EwPtrs ptrs) {
  extern __shared__ uint32_t rf[];
#define EW_R(reg, v) rf[((int)(reg) * kEwVec + (v)) * kEwThreads + threadIdx.x]
  const int64_t base = (int64_t)blockIdx.x * (kEwThreads * kEwVec) + threadIdx.x;
  for (int c = 0; c < P.n_const; ++c)
#pragma unroll
    for (int v = 0; v < kEwVec; ++v) EW_R(P.const_reg[c], v) = P.const_bits[c];
  for (int i = 0; i < P.n_in; ++i) {
    const EwOperand& o = P.in[i];
#pragma unroll
    for (int v = 0; v < kEwVec; ++v) {
      const int64_t e = base + (int64_t)v * kEwThreads;
      EW_R(o.reg, v) = e < P.n ? load_elem(ptrs.in[i], operand_index(P, o, e), o.dt) : 0u;
    }
  }
  for (int k = 0; k < P.n_instr; ++k) {
    const EwInstr ins = P.instr[k];
    const int op = ins.op;
#pragma unroll
    for (int v = 0; v < kEwVec; ++v) {
      const uint32_t a = EW_R(ins.a, v);
      uint32_t r;
      if (op == EW_CAST) {
        if (ins.cls == EWC_FLOAT) {
          const float f = ins.src_cls == EWC_FLOAT ? __uint_as_float(a) : (float)(int)a;  // bool holds 0/1
          r = __float_as_uint(round_to(f, ins.dt));
        } else if (ins.cls == EWC_BOOL) {
          r = ins.src_cls == EWC_FLOAT ? (__uint_as_float(a) != 0.f ? 1u : 0u) : (a != 0u ? 1u : 0u);
        } else if (ins.src_cls == EWC_FLOAT) {
          // as tosa.cast: round to nearest even, clamp to the type's range (cvt.rni saturates; NaN gives 0)
          const int q = __float2int_rn(__uint_as_float(a));
          r = (uint32_t)(ins.dt == kI8 ? max(-128, min(127, q)) : ins.dt == kI16 ? max(-32768, min(32767, q)) : q);
        } else {
          r = (uint32_t)wrap_int((int)a, ins.dt);  // int/bool -> int
        }
      } else if (op <= EW_ACOS) {  // EW_COPY and the value-producing unary ops
        if (ins.cls == EWC_FLOAT) r = __float_as_uint(round_to(unary_f(op, __uint_as_float(a)), ins.dt));
        else if (op == EW_ABS) r = (uint32_t)wrap_int(abs((int)a), ins.dt);
        else if (op == EW_NEG) r = (uint32_t)wrap_int(-(int)a, ins.dt);
        else if (op == EW_SQUARE) r = (uint32_t)wrap_int((int)a * (int)a, ins.dt);
        else r = a;
      } else if (op <= EW_ISNAN) {
        const float f = __uint_as_float(a);
        r = op == EW_ISINF ? (isinf(f) ? 1u : 0u) : op == EW_ISFINITE ? (isfinite(f) ? 1u : 0u) : (f != f ? 1u : 0u);
      } else if (op == EW_NOT) {
        r = a ? 0u : 1u;
      } else {
        const uint32_t b = EW_R(ins.b, v);
        if (op <= EW_ATAN2) {
          if (ins.cls == EWC_FLOAT)
            r = __float_as_uint(round_to(binary_f(op, __uint_as_float(a), __uint_as_float(b)), ins.dt));
          else
            r = (uint32_t)wrap_int(binary_i(op, (int)a, (int)b), ins.dt);
        } else if (op <= EW_LE) {
          r = (ins.src_cls == EWC_FLOAT ? compare_f(op, __uint_as_float(a), __uint_as_float(b))
                                        : compare_i(op, (int)a, (int)b))
                  ? 1u
                  : 0u;
        } else if (op == EW_AND) {
          r = (a && b) ? 1u : 0u;
        } else if (op == EW_OR) {
          r = (a || b) ? 1u : 0u;
        } else {  // EW_SELECT: a = condition
          r = a ? b : EW_R(ins.c, v);
        }
      }
      EW_R(ins.dst, v) = r;
    }
  }
  for (int i = 0; i < P.n_out; ++i) {
    const EwOperand& o = P.out[i];
#pragma unroll
    for (int v = 0; v < kEwVec; ++v) {
      const int64_t e = base + (int64_t)v * kEwThreads;
      if (e < P.n) store_elem(ptrs.out[i], operand_index(P, o, e), o.dt, EW_R(o.reg, v));
    }
  }
#undef EW_R
}

}  // namespace

size_t ew_generic_smem(const EwProgram& p) { return (size_t)p.n_reg * kEwVec * kEwThreads * sizeof(uint32_t); }

cudaError_t ew_generic(const EwProgram& p, const void* const* in, void* const* out, bool allow_jit, cudaStream_t s,
                       LaunchDims* dims) {
  if (p.n == 0) return cudaSuccess;
  if (allow_jit) {
    const cudaError_t je = ew_jit_launch(p, in, out, s, dims);
    if (je != cudaErrorNotSupported) return je;
  }
  if (ew_program_needs_jit(p)) return cudaErrorNotSupported;  // 64-bit integers: no interpreter behind the generated kernel
  EwPtrs ptrs;
  for (int i = 0; i < kEwMaxIn; ++i) ptrs.in[i] = i < p.n_in ? in[i] : nullptr;
  for (int i = 0; i < kEwMaxOut; ++i) ptrs.out[i] = i < p.n_out ? out[i] : nullptr;
  const size_t smem = ew_generic_smem(p);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(ew_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured = smem;
  }
  const int64_t per_cta = (int64_t)kEwThreads * kEwVec;
  const int64_t grid = (p.n + per_cta - 1) / per_cta;
  if (grid > 0x7fffffff) return cudaErrorInvalidValue;
  if (dims) {
    dims->grid[0] = (unsigned)grid;
    dims->block[0] = kEwThreads;
    dims->smem = (unsigned)smem;
  }
  ew_generic_kernel<<<(unsigned)grid, kEwThreads, smem, s>>>(p, ptrs);
  return cudaGetLastError();
}

}  // namespace akgb
