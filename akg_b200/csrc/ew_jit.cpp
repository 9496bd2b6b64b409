// Run-time instantiation of the elementwise template for one fused chain.
//
// The interpreter in k_ewgeneric.cu runs any chain but pays a decode per op.  Here the same EwProgram is
// printed as straight-line CUDA C++ inside a fixed, hand-written kernel skeleton (one-shot CTAs, 128-bit
// streaming loads/stores, 8 consecutive elements per thread-vector, two vectors per thread), compiled once
// with NVRTC for sm_100a and cached.  Arithmetic is emitted with the same primitives as the interpreter
// (typed rounding after every op, __f*_rn, no contraction), so both paths give identical results; the
// interpreter remains the fallback when NVRTC is not present or a chain uses strided operands.
//
// This takes the place of the reference's NVVM/PTX emission for the elementwise class
// (akg-mlir/lib/Target/PTX/GPUKernelToPTX.cpp:108-172) with a far smaller surface: only the op chain is
// generated, never the loop structure or the memory access pattern.
#include <cuda.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include "ew_program.hpp"
#include "graph.hpp"
#include "kernels.hpp"

namespace akgb {
namespace {

// ---- NVRTC and driver entry points, resolved at run time -----------------------------------------
typedef struct _nvrtcProgram* nvrtcProgram;
typedef int nvrtcResult;
struct Nvrtc {
  void* lib = nullptr;
  nvrtcResult (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*);
  nvrtcResult (*CompileProgram)(nvrtcProgram, int, const char* const*);
  nvrtcResult (*GetCUBINSize)(nvrtcProgram, size_t*);
  nvrtcResult (*GetCUBIN)(nvrtcProgram, char*);
  nvrtcResult (*GetProgramLogSize)(nvrtcProgram, size_t*);
  nvrtcResult (*GetProgramLog)(nvrtcProgram, char*);
  nvrtcResult (*DestroyProgram)(nvrtcProgram*);
  nvrtcResult (*Version)(int*, int*) = nullptr;
  bool ok = false;
};
struct Driver {
  CUresult (*ModuleLoadData)(CUmodule*, const void*);
  CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*);
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                           void**, void**);
  CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
  bool ok = false;
};

Nvrtc& nvrtc() {
  static Nvrtc n;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so.12", "libnvrtc.so"};
    for (const char* nm : names) {
      n.lib = dlopen(nm, RTLD_NOW | RTLD_LOCAL);
      if (n.lib) break;
    }
    if (!n.lib) return;
#define AKGB_SYM(field, name)                                     \
  *reinterpret_cast<void**>(&n.field) = dlsym(n.lib, name);       \
  if (!n.field) return;
    AKGB_SYM(CreateProgram, "nvrtcCreateProgram")
    AKGB_SYM(CompileProgram, "nvrtcCompileProgram")
    AKGB_SYM(GetCUBINSize, "nvrtcGetCUBINSize")
    AKGB_SYM(GetCUBIN, "nvrtcGetCUBIN")
    AKGB_SYM(GetProgramLogSize, "nvrtcGetProgramLogSize")
    AKGB_SYM(GetProgramLog, "nvrtcGetProgramLog")
    AKGB_SYM(DestroyProgram, "nvrtcDestroyProgram")
    AKGB_SYM(Version, "nvrtcVersion")
#undef AKGB_SYM
    n.ok = true;
  });
  return n;
}

Driver& driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    auto get = [](const char* name, void** out) {
      cudaDriverEntryPointQueryResult q;
      return cudaGetDriverEntryPoint(name, out, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess &&
             *out;
    };
    if (!get("cuModuleLoadData", reinterpret_cast<void**>(&d.ModuleLoadData))) return;
    if (!get("cuModuleGetFunction", reinterpret_cast<void**>(&d.ModuleGetFunction))) return;
    if (!get("cuLaunchKernel", reinterpret_cast<void**>(&d.LaunchKernel))) return;
    if (!get("cuFuncSetAttribute", reinterpret_cast<void**>(&d.FuncSetAttribute))) return;
    d.ok = true;
  });
  return d;
}

// ---- source generation ---------------------------------------------------------------------------
const char* kPreamble = R"SRC(
typedef unsigned int u32; typedef unsigned short u16; typedef unsigned char u8; typedef long long i64;
struct __align__(16) U4 { u32 x, y, z, w; };
struct __align__(8) U2 { u32 x, y; };
// Checked build (the source then starts with "#define AKGB_CHECKED 1"): every access to global memory is tested
// against the address ranges of the launch's tensors and workspace; one that falls outside any of them sets bit 9 of
// the device error word and is skipped (a load gives zeros) -- no assert, no trap.
#ifdef AKGB_CHECKED
struct AkgbRanges { unsigned long long lo[32], hi[32]; int n; u32* err; };
__device__ AkgbRanges akgb_rng;  // the same table from every block of a launch (its last kernel argument)
__device__ __noinline__ bool akgb_ok(const void* p, int bytes) {
  const unsigned long long a = (unsigned long long)p;
  for (int i = 0; i < akgb_rng.n; ++i)
    if (a >= akgb_rng.lo[i] && a + (unsigned long long)bytes <= akgb_rng.hi[i]) return true;
  atomicOr(akgb_rng.err, 512u);
  return false;
}
#define AKGB_CHK(p, bytes, zero) if (!akgb_ok(p, bytes)) return zero;
#define AKGB_CHKV(p, bytes) if (!akgb_ok(p, bytes)) return;
#else
#define AKGB_CHK(p, bytes, zero)
#define AKGB_CHKV(p, bytes)
#endif
__device__ __forceinline__ U4 ld16s(const void* p) { U4 v; v.x = v.y = v.z = v.w = 0; AKGB_CHK(p, 16, v)
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p)); return v; }
__device__ __forceinline__ U4 ld16c(const void* p) { U4 v; v.x = v.y = v.z = v.w = 0; AKGB_CHK(p, 16, v)
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p)); return v; }
__device__ __forceinline__ U2 ld8s(const void* p) { U2 v; v.x = v.y = 0; AKGB_CHK(p, 8, v)
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p)); return v; }
__device__ __forceinline__ void st16(void* p, U4 v) { AKGB_CHKV(p, 16)
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory"); }
__device__ __forceinline__ void st8(void* p, U2 v) { AKGB_CHKV(p, 8)
  asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" :: "l"(p), "r"(v.x), "r"(v.y) : "memory"); }
__device__ __forceinline__ float h2f(u16 h) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h)); return f; }
__device__ __forceinline__ u16 f2h(float f) { u16 h; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f)); return h; }
__device__ __forceinline__ float b2f(u16 b) { return __uint_as_float(((u32)b) << 16); }
__device__ __forceinline__ u16 f2b(float f) { u16 h; asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(f)); return h; }
__device__ __forceinline__ float rn_f16(float x) { return h2f(f2h(x)); }
__device__ __forceinline__ float rn_bf16(float x) { return b2f(f2b(x)); }
__device__ __forceinline__ float rn_f32(float x) { return x; }
__device__ __forceinline__ int wr_i8(int x) { return (int)(signed char)x; }
__device__ __forceinline__ int wr_i16(int x) { return (int)(short)x; }
__device__ __forceinline__ int wr_i32(int x) { return x; }
// float -> integer as tosa.cast: round to nearest even, clamp to the type's range (cvt.rni saturates; NaN gives 0)
__device__ __forceinline__ int f2i_i32(float x) { return __float2int_rn(x); }
__device__ __forceinline__ int f2i_i16(float x) { return max(-32768, min(32767, __float2int_rn(x))); }
__device__ __forceinline__ int f2i_i8(float x) { return max(-128, min(127, __float2int_rn(x))); }
__device__ __forceinline__ float mx_f(float a, float b) { return (a != a || b != b) ? __int_as_float(0x7fc00000) : fmaxf(a, b); }
__device__ __forceinline__ float mn_f(float a, float b) { return (a != a || b != b) ? __int_as_float(0x7fc00000) : fminf(a, b); }
// 8 consecutive elements starting at element e0 (e0 % 8 == 0, base 16-byte aligned)
#define LD8_16(NAME, CVT) __device__ __forceinline__ void NAME(const void* p, i64 e0, float* r, bool stream) { \
  const U4 v = stream ? ld16s((const u16*)p + e0) : ld16c((const u16*)p + e0); const u32 w[4] = {v.x, v.y, v.z, v.w}; \
  _Pragma("unroll") for (int i = 0; i < 4; ++i) { r[2*i] = CVT((u16)(w[i] & 0xffffu)); r[2*i+1] = CVT((u16)(w[i] >> 16)); } }
LD8_16(ld8_f16, h2f)
LD8_16(ld8_bf16, b2f)
// the same widening applied to a granule that was loaded earlier and kept packed
#define CVT8_16(NAME, CVT) __device__ __forceinline__ void NAME(U4 v, float* r) { const u32 w[4] = {v.x, v.y, v.z, v.w}; \
  _Pragma("unroll") for (int i = 0; i < 4; ++i) { r[2*i] = CVT((u16)(w[i] & 0xffffu)); r[2*i+1] = CVT((u16)(w[i] >> 16)); } }
CVT8_16(cvt8_f16, h2f)
CVT8_16(cvt8_bf16, b2f)
__device__ __forceinline__ void ld8_f32(const void* p, i64 e0, float* r, bool stream) {
  const U4 a = stream ? ld16s((const float*)p + e0) : ld16c((const float*)p + e0);
  const U4 b = stream ? ld16s((const float*)p + e0 + 4) : ld16c((const float*)p + e0 + 4);
  r[0] = __uint_as_float(a.x); r[1] = __uint_as_float(a.y); r[2] = __uint_as_float(a.z); r[3] = __uint_as_float(a.w);
  r[4] = __uint_as_float(b.x); r[5] = __uint_as_float(b.y); r[6] = __uint_as_float(b.z); r[7] = __uint_as_float(b.w); }
template <class I> __device__ __forceinline__ void ld8_i32(const void* p, i64 e0, I* r, bool stream) {
  const U4 a = stream ? ld16s((const int*)p + e0) : ld16c((const int*)p + e0);
  const U4 b = stream ? ld16s((const int*)p + e0 + 4) : ld16c((const int*)p + e0 + 4);
  r[0] = (int)a.x; r[1] = (int)a.y; r[2] = (int)a.z; r[3] = (int)a.w; r[4] = (int)b.x; r[5] = (int)b.y; r[6] = (int)b.z; r[7] = (int)b.w; }
template <class I> __device__ __forceinline__ void ld8_i16(const void* p, i64 e0, I* r, bool stream) {
  const U4 v = stream ? ld16s((const u16*)p + e0) : ld16c((const u16*)p + e0); const u32 w[4] = {v.x, v.y, v.z, v.w};
  _Pragma("unroll") for (int i = 0; i < 4; ++i) { r[2*i] = (int)(short)(w[i] & 0xffffu); r[2*i+1] = (int)(short)(w[i] >> 16); } }
template <class I> __device__ __forceinline__ void ld8_i8(const void* p, i64 e0, I* r, bool stream) {
  const U2 v = ld8s((const u8*)p + e0); const u32 w[2] = {v.x, v.y};
  _Pragma("unroll") for (int i = 0; i < 8; ++i) r[i] = (int)(signed char)((w[i >> 2] >> (8 * (i & 3))) & 0xffu); }
template <class I> __device__ __forceinline__ void ld8_bool(const void* p, i64 e0, I* r, bool stream) {
  const U2 v = ld8s((const u8*)p + e0); const u32 w[2] = {v.x, v.y};
  _Pragma("unroll") for (int i = 0; i < 8; ++i) r[i] = ((w[i >> 2] >> (8 * (i & 3))) & 0xffu) ? 1 : 0; }
// two floats rounded to nearest even and packed in one instruction (lo in the low half); the same bits as f2h / f2b give
__device__ __forceinline__ u32 f2h2(float lo, float hi) { u32 p; asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(p) : "f"(hi), "f"(lo)); return p; }
__device__ __forceinline__ u32 f2b2(float lo, float hi) { u32 p; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(p) : "f"(hi), "f"(lo)); return p; }
// a granule of float32 values rounded in place to values of the 16-bit type
#define RN8_16(NAME, PACK, CVT) __device__ __forceinline__ void NAME(float* r) { \
  _Pragma("unroll") for (int i = 0; i < 4; ++i) { const u32 p = PACK(r[2*i], r[2*i+1]); \
    r[2*i] = CVT((u16)(p & 0xffffu)); r[2*i+1] = CVT((u16)(p >> 16)); } }
RN8_16(rn8_f16, f2h2, h2f)
RN8_16(rn8_bf16, f2b2, b2f)
#define ST8_16(NAME, PACK) __device__ __forceinline__ void NAME(void* p, i64 e0, const float* r) { U4 v; \
  v.x = PACK(r[0], r[1]); v.y = PACK(r[2], r[3]); v.z = PACK(r[4], r[5]); v.w = PACK(r[6], r[7]); st16((u16*)p + e0, v); }
ST8_16(st8_f16, f2h2)
ST8_16(st8_bf16, f2b2)
__device__ __forceinline__ void st8_f32(void* p, i64 e0, const float* r) {
  U4 a, b; a.x = __float_as_uint(r[0]); a.y = __float_as_uint(r[1]); a.z = __float_as_uint(r[2]); a.w = __float_as_uint(r[3]);
  b.x = __float_as_uint(r[4]); b.y = __float_as_uint(r[5]); b.z = __float_as_uint(r[6]); b.w = __float_as_uint(r[7]);
  st16((float*)p + e0, a); st16((float*)p + e0 + 4, b); }
template <class I> __device__ __forceinline__ void st8_i32(void* p, i64 e0, const I* r) {
  U4 a, b; a.x = (u32)r[0]; a.y = (u32)r[1]; a.z = (u32)r[2]; a.w = (u32)r[3]; b.x = (u32)r[4]; b.y = (u32)r[5]; b.z = (u32)r[6]; b.w = (u32)r[7];
  st16((int*)p + e0, a); st16((int*)p + e0 + 4, b); }
template <class I> __device__ __forceinline__ void st8_i16(void* p, i64 e0, const I* r) { U4 v;
  v.x = (u32)(u16)r[0] | ((u32)(u16)r[1] << 16); v.y = (u32)(u16)r[2] | ((u32)(u16)r[3] << 16);
  v.z = (u32)(u16)r[4] | ((u32)(u16)r[5] << 16); v.w = (u32)(u16)r[6] | ((u32)(u16)r[7] << 16); st16((u16*)p + e0, v); }
template <class I> __device__ __forceinline__ void st8_i8(void* p, i64 e0, const I* r) { U2 v; v.x = 0; v.y = 0;
  _Pragma("unroll") for (int i = 0; i < 4; ++i) { v.x |= ((u32)(u8)r[i]) << (8 * i); v.y |= ((u32)(u8)r[4 + i]) << (8 * i); } st8((u8*)p + e0, v); }
template <class I> __device__ __forceinline__ void st8_bool(void* p, i64 e0, const I* r) { U2 v; v.x = 0; v.y = 0;
  _Pragma("unroll") for (int i = 0; i < 4; ++i) { v.x |= (r[i] ? 1u : 0u) << (8 * i); v.y |= (r[4 + i] ? 1u : 0u) << (8 * i); } st8((u8*)p + e0, v); }
// scalar element access (any alignment)
__device__ __forceinline__ float ld1_f16(const void* p, i64 i) { AKGB_CHK((const u16*)p + i, 2, 0.f) return h2f(((const u16*)p)[i]); }
__device__ __forceinline__ float ld1_bf16(const void* p, i64 i) { AKGB_CHK((const u16*)p + i, 2, 0.f) return b2f(((const u16*)p)[i]); }
__device__ __forceinline__ float ld1_f32(const void* p, i64 i) { AKGB_CHK((const float*)p + i, 4, 0.f) return ((const float*)p)[i]; }
__device__ __forceinline__ int ld1_i32(const void* p, i64 i) { AKGB_CHK((const int*)p + i, 4, 0) return ((const int*)p)[i]; }
__device__ __forceinline__ int ld1_i16(const void* p, i64 i) { AKGB_CHK((const short*)p + i, 2, 0) return (int)((const short*)p)[i]; }
__device__ __forceinline__ int ld1_i8(const void* p, i64 i) { AKGB_CHK((const u8*)p + i, 1, 0) return (int)((const signed char*)p)[i]; }
__device__ __forceinline__ int ld1_bool(const void* p, i64 i) { AKGB_CHK((const u8*)p + i, 1, 0) return ((const u8*)p)[i] ? 1 : 0; }
__device__ __forceinline__ void st1_f16(void* p, i64 i, float v) { AKGB_CHKV((u16*)p + i, 2) ((u16*)p)[i] = f2h(v); }
__device__ __forceinline__ void st1_bf16(void* p, i64 i, float v) { AKGB_CHKV((u16*)p + i, 2) ((u16*)p)[i] = f2b(v); }
__device__ __forceinline__ void st1_f32(void* p, i64 i, float v) { AKGB_CHKV((float*)p + i, 4) ((float*)p)[i] = v; }
__device__ __forceinline__ void st1_i32(void* p, i64 i, int v) { AKGB_CHKV((int*)p + i, 4) ((int*)p)[i] = v; }
__device__ __forceinline__ void st1_i16(void* p, i64 i, int v) { AKGB_CHKV((short*)p + i, 2) ((short*)p)[i] = (short)v; }
__device__ __forceinline__ void st1_i8(void* p, i64 i, int v) { AKGB_CHKV((u8*)p + i, 1) ((signed char*)p)[i] = (signed char)v; }
__device__ __forceinline__ void st1_bool(void* p, i64 i, int v) { AKGB_CHKV((u8*)p + i, 1) ((u8*)p)[i] = v ? 1 : 0; }
// 64-bit integers (programs that hold any keep ALL their integer registers in 64 bits)
__device__ __forceinline__ i64 wr_i64(i64 x) { return x; }
__device__ __forceinline__ i64 f2i_i64(float x) { return x != x ? 0 : __float2ll_rn(x); }  // saturating; NaN gives 0
__device__ __forceinline__ i64 ld1_i64(const void* p, i64 i) { AKGB_CHK((const i64*)p + i, 8, 0) return ((const i64*)p)[i]; }
__device__ __forceinline__ void st1_i64(void* p, i64 i, i64 v) { AKGB_CHKV((i64*)p + i, 8) ((i64*)p)[i] = v; }
__device__ __forceinline__ void ld8_i64(const void* p, i64 e0, i64* r, bool stream) {
  _Pragma("unroll") for (int q = 0; q < 4; ++q) {
    const U4 v = stream ? ld16s((const i64*)p + e0 + 2 * q) : ld16c((const i64*)p + e0 + 2 * q);
    r[2*q] = (i64)(((unsigned long long)v.y << 32) | v.x); r[2*q+1] = (i64)(((unsigned long long)v.w << 32) | v.z); } }
__device__ __forceinline__ void st8_i64(void* p, i64 e0, const i64* r) {
  _Pragma("unroll") for (int q = 0; q < 4; ++q) { U4 v;
    v.x = (u32)r[2*q]; v.y = (u32)((unsigned long long)r[2*q] >> 32); v.z = (u32)r[2*q+1]; v.w = (u32)((unsigned long long)r[2*q+1] >> 32);
    st16((i64*)p + e0 + 2 * q, v); } }
)SRC";

// Appended for programs that hold a float64 value: ALL their floating-point registers are doubles.  Values of a
// narrower type are the doubles that type can represent; an op computes in double and rounds once to its own type,
// which for + - * / sqrt is the correctly rounded result of that type (53 bits >= 2 * 24 + 2).  double -> 16-bit goes
// through a float32 rounded to odd, so that the second rounding sees what the first one dropped.
const char* kPreambleF64 = R"SRC(
__device__ __forceinline__ float odd_f32(double x) { float f = __double2float_rz(x);
  if (x == x && (double)f != x) f = __uint_as_float(__float_as_uint(f) | 1u); return f; }
__device__ __forceinline__ double rn_f64(double x) { return x; }
__device__ __forceinline__ double rn_f32_d(double x) { return (double)__double2float_rn(x); }
__device__ __forceinline__ double rn_f16_d(double x) { return (double)rn_f16(odd_f32(x)); }
__device__ __forceinline__ double rn_bf16_d(double x) { return (double)rn_bf16(odd_f32(x)); }
// (the conversion from a double NaN gives INT_MIN, not the 0 it gives from a float NaN)
__device__ __forceinline__ int f2i_i32_d(double x) { return x != x ? 0 : __double2int_rn(x); }
__device__ __forceinline__ i64 f2i_i64_d(double x) { return x != x ? 0 : __double2ll_rn(x); }
__device__ __forceinline__ int f2i_i16_d(double x) { return max(-32768, min(32767, f2i_i32_d(x))); }
__device__ __forceinline__ int f2i_i8_d(double x) { return max(-128, min(127, f2i_i32_d(x))); }
__device__ __forceinline__ double mx_d(double a, double b) { return (a != a || b != b) ? __longlong_as_double(0x7ff8000000000000LL) : fmax(a, b); }
__device__ __forceinline__ double mn_d(double a, double b) { return (a != a || b != b) ? __longlong_as_double(0x7ff8000000000000LL) : fmin(a, b); }
#define LD8_D(NAME, BASE) __device__ __forceinline__ void NAME(const void* p, i64 e0, double* r, bool stream) { \
  float t[8]; BASE(p, e0, t, stream); _Pragma("unroll") for (int i = 0; i < 8; ++i) r[i] = (double)t[i]; }
LD8_D(ld8_f32_d, ld8_f32)
LD8_D(ld8_f16_d, ld8_f16)
LD8_D(ld8_bf16_d, ld8_bf16)
#define ST8_D(NAME, BASE) __device__ __forceinline__ void NAME(void* p, i64 e0, const double* r) { \
  float t[8]; _Pragma("unroll") for (int i = 0; i < 8; ++i) t[i] = (float)r[i]; BASE(p, e0, t); }
ST8_D(st8_f32_d, st8_f32)
ST8_D(st8_f16_d, st8_f16)
ST8_D(st8_bf16_d, st8_bf16)
__device__ __forceinline__ void ld8_f64(const void* p, i64 e0, double* r, bool stream) {
  _Pragma("unroll") for (int q = 0; q < 4; ++q) {
    const U4 v = stream ? ld16s((const double*)p + e0 + 2 * q) : ld16c((const double*)p + e0 + 2 * q);
    r[2*q] = __hiloint2double((int)v.y, (int)v.x); r[2*q+1] = __hiloint2double((int)v.w, (int)v.z); } }
__device__ __forceinline__ void st8_f64(void* p, i64 e0, const double* r) {
  _Pragma("unroll") for (int q = 0; q < 4; ++q) { U4 v;
    v.x = (u32)__double2loint(r[2*q]); v.y = (u32)__double2hiint(r[2*q]); v.z = (u32)__double2loint(r[2*q+1]); v.w = (u32)__double2hiint(r[2*q+1]);
    st16((double*)p + e0 + 2 * q, v); } }
__device__ __forceinline__ double ld1_f64(const void* p, i64 i) { AKGB_CHK((const double*)p + i, 8, 0.0) return ((const double*)p)[i]; }
__device__ __forceinline__ void st1_f64(void* p, i64 i, double v) { AKGB_CHKV((double*)p + i, 8) ((double*)p)[i] = v; }
)SRC";

const char* dt_tag(int dt) {
  switch ((DT)dt) {
    case DT::F64: return "f64";
    case DT::F16: return "f16";
    case DT::BF16: return "bf16";
    case DT::F32: return "f32";
    case DT::I32: return "i32";
    case DT::I16: return "i16";
    case DT::I8: return "i8";
    case DT::I64: return "i64";
    default: return "bool";
  }
}
// a program with a 64-bit integer operand or result keeps all its integer registers in 64 bits
bool ew_has_i64(const EwProgram& P) {
  for (int i = 0; i < P.n_in; ++i)
    if ((DT)P.in[i].dt == DT::I64) return true;
  for (int i = 0; i < P.n_out; ++i)
    if ((DT)P.out[i].dt == DT::I64) return true;
  for (int k = 0; k < P.n_instr; ++k)
    if ((DT)P.instr[k].dt == DT::I64) return true;
  return false;
}
// a program with a float64 operand or result keeps all its floating-point registers as doubles
bool ew_has_f64(const EwProgram& P) {
  for (int i = 0; i < P.n_in; ++i)
    if ((DT)P.in[i].dt == DT::F64) return true;
  for (int i = 0; i < P.n_out; ++i)
    if ((DT)P.out[i].dt == DT::F64) return true;
  for (int k = 0; k < P.n_instr; ++k)
    if ((DT)P.instr[k].dt == DT::F64) return true;
  return false;
}
bool is_float_dt(int dt) { return (DT)dt == DT::F16 || (DT)dt == DT::BF16 || (DT)dt == DT::F32 || (DT)dt == DT::F64; }
const char* round_fn(int dt) { return (DT)dt == DT::F16 ? "rn_f16" : (DT)dt == DT::BF16 ? "rn_bf16" : "rn_f32"; }
// the same in a program whose registers are doubles
const char* round_fn_d(int dt) {
  return (DT)dt == DT::F16 ? "rn_f16_d" : (DT)dt == DT::BF16 ? "rn_bf16_d" : (DT)dt == DT::F64 ? "rn_f64" : "rn_f32_d";
}
const char* wrap_fn(int dt) { return (DT)dt == DT::I8 ? "wr_i8" : (DT)dt == DT::I16 ? "wr_i16" : (DT)dt == DT::I64 ? "wr_i64" : "wr_i32"; }

// results of a 16-bit floating-point type over a whole granule: computed unrounded, then rounded two per instruction
bool pair_rounded(bool vec, int op, int dt, int cls) {
  return vec && cls == EWC_FLOAT && ((DT)dt == DT::F16 || (DT)dt == DT::BF16) && op != EW_COPY && op != EW_SELECT;
}

struct Var {
  std::string name;
  bool is_float = true;
  bool is_const = false;
  std::string literal;
  std::string literal64;      // the expression of a float64 constant
  std::string int64_literal;  // the expression of a 64-bit integer constant outside the 32-bit range
};

std::string float_unary(int op, const std::string& a) {
  switch (op) {
    case EW_ABS: return "fabsf(" + a + ")";
    case EW_NEG: return "(-" + a + ")";
    case EW_EXP: return "expf(" + a + ")";
    case EW_LOG: return "logf(" + a + ")";
    case EW_TANH: return "tanhf(" + a + ")";
    case EW_RSQRT: return "__fdiv_rn(1.0f, __fsqrt_rn(" + a + "))";
    case EW_SQRT: return "__fsqrt_rn(" + a + ")";
    case EW_RECIP: return "__fdiv_rn(1.0f, " + a + ")";
    case EW_FLOOR: return "floorf(" + a + ")";
    case EW_SQUARE: return "__fmul_rn(" + a + ", " + a + ")";
    case EW_SIN: return "sinf(" + a + ")";
    case EW_COS: return "cosf(" + a + ")";
    case EW_ASINH: return "asinhf(" + a + ")";
    case EW_ACOSH: return "acoshf(" + a + ")";
    case EW_ATAN: return "atanf(" + a + ")";
    case EW_ASIN: return "asinf(" + a + ")";
    case EW_ACOS: return "acosf(" + a + ")";
    default: return a;
  }
}
std::string double_unary(int op, const std::string& a) {
  switch (op) {
    case EW_ABS: return "fabs(" + a + ")";
    case EW_NEG: return "(-" + a + ")";
    case EW_EXP: return "exp(" + a + ")";
    case EW_LOG: return "log(" + a + ")";
    case EW_TANH: return "tanh(" + a + ")";
    case EW_RSQRT: return "__ddiv_rn(1.0, __dsqrt_rn(" + a + "))";
    case EW_SQRT: return "__dsqrt_rn(" + a + ")";
    case EW_RECIP: return "__ddiv_rn(1.0, " + a + ")";
    case EW_FLOOR: return "floor(" + a + ")";
    case EW_SQUARE: return "__dmul_rn(" + a + ", " + a + ")";
    case EW_SIN: return "sin(" + a + ")";
    case EW_COS: return "cos(" + a + ")";
    case EW_ASINH: return "asinh(" + a + ")";
    case EW_ACOSH: return "acosh(" + a + ")";
    case EW_ATAN: return "atan(" + a + ")";
    case EW_ASIN: return "asin(" + a + ")";
    case EW_ACOS: return "acos(" + a + ")";
    default: return a;
  }
}
std::string double_binary(int op, const std::string& a, const std::string& b) {
  switch (op) {
    case EW_ADD: return "__dadd_rn(" + a + ", " + b + ")";
    case EW_SUB: return "__dsub_rn(" + a + ", " + b + ")";
    case EW_MUL: return "__dmul_rn(" + a + ", " + b + ")";
    case EW_DIV: return "__ddiv_rn(" + a + ", " + b + ")";
    case EW_MAX: return "mx_d(" + a + ", " + b + ")";
    case EW_MIN: return "mn_d(" + a + ", " + b + ")";
    case EW_POW: return "pow(" + a + ", " + b + ")";
    default: return "atan2(" + a + ", " + b + ")";
  }
}
std::string float_binary(int op, const std::string& a, const std::string& b) {
  switch (op) {
    case EW_ADD: return "__fadd_rn(" + a + ", " + b + ")";
    case EW_SUB: return "__fsub_rn(" + a + ", " + b + ")";
    case EW_MUL: return "__fmul_rn(" + a + ", " + b + ")";
    case EW_DIV: return "__fdiv_rn(" + a + ", " + b + ")";
    case EW_MAX: return "mx_f(" + a + ", " + b + ")";
    case EW_MIN: return "mn_f(" + a + ", " + b + ")";
    case EW_POW: return "powf(" + a + ", " + b + ")";
    default: return "atan2f(" + a + ", " + b + ")";
  }
}
std::string int_binary(int op, const std::string& a, const std::string& b) {
  switch (op) {
    case EW_ADD: return "(" + a + " + " + b + ")";
    case EW_SUB: return "(" + a + " - " + b + ")";
    case EW_MUL: return "(" + a + " * " + b + ")";
    case EW_DIV: return "(" + b + " == 0 ? 0 : " + a + " / " + b + ")";
    case EW_MAX: return "max(" + a + ", " + b + ")";
    default: return "min(" + a + ", " + b + ")";
  }
}
const char* cmp_op(int op) {
  switch (op) {
    case EW_EQ: return "==";
    case EW_GT: return ">";
    case EW_GE: return ">=";
    case EW_LT: return "<";
    default: return "<=";
  }
}

// The expression of one elementwise op in generated code; `ref(value, want_float)` yields an operand's expression.
template <class Ref>
std::string instr_expr(int op, int dt, int cls, int src_cls, int a, int b, int c, Ref&& ref, bool f64 = false) {
  const bool fl = cls == EWC_FLOAT;
  const bool sfl = src_cls == EWC_FLOAT;
  const std::string rnd = f64 ? round_fn_d(dt) : round_fn(dt);
  std::string expr;
  if (op == EW_COPY) {
    expr = ref(a, fl);
  } else if (op == EW_CAST) {
    if (fl) expr = rnd + "(" + (sfl ? ref(a, true) : (f64 ? "(double)" : "(float)") + ref(a, false)) + ")";
    else if (cls == EWC_BOOL) expr = sfl ? "(" + ref(a, true) + " != 0.f ? 1 : 0)" : "(" + ref(a, false) + " != 0 ? 1 : 0)";
    else if (sfl) expr = std::string((DT)dt == DT::I8 ? "f2i_i8" : (DT)dt == DT::I16 ? "f2i_i16" : (DT)dt == DT::I64 ? "f2i_i64" : "f2i_i32") + (f64 ? "_d(" : "(") + ref(a, true) + ")";
    else expr = std::string(wrap_fn(dt)) + "(" + ref(a, false) + ")";
  } else if (op <= EW_ACOS) {
    if (fl) expr = rnd + "(" + (f64 ? double_unary(op, ref(a, true)) : float_unary(op, ref(a, true))) + ")";
    else if (op == EW_ABS) expr = std::string(wrap_fn(dt)) + "(abs(" + ref(a, false) + "))";
    else if (op == EW_NEG) expr = std::string(wrap_fn(dt)) + "(-" + ref(a, false) + ")";
    else if (op == EW_SQUARE) expr = std::string(wrap_fn(dt)) + "(" + ref(a, false) + " * " + ref(a, false) + ")";
    else expr = ref(a, false);
  } else if (op <= EW_ISNAN) {
    const std::string x = ref(a, true);
    expr = op == EW_ISINF ? "(isinf(" + x + ") ? 1 : 0)" : op == EW_ISFINITE ? "(isfinite(" + x + ") ? 1 : 0)"
                                                                              : "(" + x + " != " + x + " ? 1 : 0)";
  } else if (op == EW_NOT) {
    expr = "(" + ref(a, false) + " ? 0 : 1)";
  } else if (op <= EW_ATAN2) {
    if (fl) expr = rnd + "(" + (f64 ? double_binary(op, ref(a, true), ref(b, true)) : float_binary(op, ref(a, true), ref(b, true))) + ")";
    else expr = std::string(wrap_fn(dt)) + "(" + int_binary(op, ref(a, false), ref(b, false)) + ")";
  } else if (op <= EW_LE) {
    const std::string x = ref(a, sfl), y = ref(b, sfl);
    if (op == EW_NE) expr = "(!(" + x + " == " + y + ") ? 1 : 0)";
    else expr = "((" + x + " " + cmp_op(op) + " " + y + ") ? 1 : 0)";
  } else if (op == EW_AND) {
    expr = "((" + ref(a, false) + " && " + ref(b, false) + ") ? 1 : 0)";
  } else if (op == EW_OR) {
    expr = "((" + ref(a, false) + " || " + ref(b, false) + ") ? 1 : 0)";
  } else {  // select: a = condition
    expr = "(" + ref(a, false) + " ? " + ref(b, fl) + " : " + ref(c, fl) + ")";
  }
  return expr;
}

// Emits the op chain for element lane `j` of vector slot `u`.  `ref(reg)` yields the expression of a register.
// Element index of a strided operand for the linear index `e` of the iteration space: the coordinates of `e` (constant
// divisors, which the compiler turns into multiply-shift) times the operand's strides, a wrapped coordinate for Tile.
std::string strided_index(const EwProgram& P, const EwOperand& o, const std::string& e) {
  std::ostringstream x;
  x << "(" << o.offset << "LL";
  int64_t suffix = 1;
  for (int d = P.rank - 1; d >= 0; --d) {
    if (o.stride[d] != 0 && P.shape[d] > 1) {
      std::ostringstream c;
      c << "(" << e;
      if (suffix > 1) c << " / " << suffix << "LL";
      c << ")";
      std::string coord = c.str();
      if (d > 0) coord = "(" + coord + " % " + std::to_string(P.shape[d]) + "LL)";
      if (o.wrap[d] != 0) coord = "(" + coord + " % " + std::to_string(o.wrap[d]) + "LL)";
      x << " + " << coord << " * " << o.stride[d] << "LL";
    }
    suffix *= P.shape[d];
  }
  x << ")";
  return x.str();
}
// 8 consecutive elements of the iteration space are 8 consecutive, 16-byte aligned elements of the operand
bool strided_vec8_ok(const EwProgram& P, const EwOperand& o) {
  const int last = P.rank - 1;
  if (last < 0 || P.shape[last] % 8 != 0 || o.stride[last] != 1 || o.offset % 8 != 0) return false;
  if (o.wrap[last] != 0 && o.wrap[last] % 8 != 0) return false;
  for (int d = 0; d < last; ++d)
    if (o.stride[d] % 8 != 0) return false;
  return true;
}

// 8 consecutive elements of the iteration space read ONE element of the operand: the operand does not move along the
// innermost dimension and rows of that dimension hold whole granules
bool strided_run8_const(const EwProgram& P, const EwOperand& o) {
  const int last = P.rank - 1;
  return last >= 0 && P.shape[last] % 8 == 0 && o.stride[last] == 0;
}

// How one thread of the generated elementwise kernel is laid out: U granules (of 8 elements with 16-byte accesses, of 1
// otherwise), all loaded before the first is computed.  Measured on 0.5-1 GB chains: 16-bit granules that stay packed
// until their turn (4 registers instead of 8) took a float16-in / float32-math GELU chain from 204 to 168 us and a
// bfloat16 multiply-add from 153 to 120 us; four granules per thread, or one, were never faster than two at that size; a register
// cap for six resident CTAs gained another 1-10 % on the programs small enough to fit it.
struct EwShape {
  int U = 2;
  int min_blocks = 0;  // second argument of __launch_bounds__; 0 = none
};
bool packed_load(const EwProgram& P, const EwOperand& o);
EwShape ew_shape(const EwProgram& P, bool vec) {
  EwShape sh;
  sh.U = vec ? 2 : 4;
  if (!vec) return sh;
  // small launches (a shard of a split tensor, a 67 MB copy) run faster with twice the CTAs of half the work: float32
  // copy of 2^23 elements 13.2 -> 11.8 us, the float32-math GELU chain on 2^23 elements 15.2 -> 14.6 us; from 2^24
  // elements on the two shapes time alike (25.1 / 24.9 us) and two granules win at 2^27 (168.6 / 172.5 us)
  if (P.n <= ((int64_t)3 << 22)) sh.U = 1;
  // registers the loaded granules hold, plus 8 per value alive at once in the op chain
  int regs = 0;
  for (int i = 0; i < P.n_in; ++i) regs += sh.U * (packed_load(P, P.in[i]) ? 4 : 8);
  std::vector<int> last(kEwMaxReg, -1);
  for (int k = 0; k < P.n_instr; ++k)
    for (int r : {P.instr[k].a, P.instr[k].b, P.instr[k].c})
      if (r >= 0 && r < kEwMaxReg) last[r] = k;
  for (int i = 0; i < P.n_out; ++i)
    if (P.out[i].reg >= 0 && P.out[i].reg < kEwMaxReg) last[P.out[i].reg] = P.n_instr;
  int live_max = 0;
  for (int k = 0; k < P.n_instr; ++k) {
    int live = 0;
    for (int d = 0; d <= k; ++d)
      if (last[P.instr[d].dst] > k) ++live;
    live_max = std::max(live_max, live + 1);
  }
  regs += 8 * live_max;
  if (ew_has_f64(P)) return sh;  // doubles: twice the registers of this estimate
  if (regs <= 40) sh.min_blocks = 6;
  else if (regs <= 48) sh.min_blocks = 5;
  return sh;
}
bool packed_load(const EwProgram& P, const EwOperand& o) {
  if (((DT)o.dt != DT::F16 && (DT)o.dt != DT::BF16) || ew_has_f64(P)) return false;
  return o.kind == EWI_FULL || (o.kind == EWI_MOD && o.mod % 8 == 0) ||
         (o.kind == EWI_STRIDED && !strided_run8_const(P, o) && strided_vec8_ok(P, o));
}

bool generate(const EwProgram& P, bool vec, std::string* out) {
  for (int i = 0; i < P.n_out; ++i)
    if (P.out[i].kind != EWI_FULL && P.out[i].kind != EWI_STRIDED) return false;
  std::ostringstream s;
  const bool i64 = ew_has_i64(P);
  const std::string ity = i64 ? "long long" : "int";
  const bool f64 = ew_has_f64(P);
  const std::string fty = f64 ? "double" : "float";
  // loads and stores of floating-point tensors narrower than the registers convert through float32
  auto ld8_name = [&](int dt) { return std::string("ld8_") + dt_tag(dt) + (f64 && is_float_dt(dt) && (DT)dt != DT::F64 ? "_d" : ""); };
  auto st8_name = [&](int dt) { return std::string("st8_") + dt_tag(dt) + (f64 && is_float_dt(dt) && (DT)dt != DT::F64 ? "_d" : ""); };
  const EwShape sh = ew_shape(P, vec);
  s << kPreamble;
  if (f64) s << kPreambleF64;
  s << "extern \"C\" __global__ void __launch_bounds__(256";
  if (sh.min_blocks > 0) s << ", " << sh.min_blocks;
  s << ") akgb_ew_jit(";
  for (int i = 0; i < P.n_in; ++i) s << "const void* __restrict__ in" << i << ", ";
  for (int i = 0; i < P.n_out; ++i) s << "void* __restrict__ out" << i << ", ";
  s << "i64 n) {\n";
  const int U = sh.U, E = vec ? 8 : 1;
  s << "  constexpr int U = " << U << ", E = " << E << ";\n";
  s << "  const i64 nv = n / E;\n";
  s << "  const i64 vbase = (i64)blockIdx.x * (256 * U) + threadIdx.x;\n";
  // register -> current variable
  std::vector<Var> regs(kEwMaxReg);
  for (int c = 0; c < P.n_const; ++c) {
    Var v;
    v.is_const = true;
    char buf[64];
    std::snprintf(buf, sizeof(buf), "0x%08xu", P.const_bits[c]);
    v.literal = buf;
    if (P.const_f64[c] == 1) {
      std::snprintf(buf, sizeof(buf), "__longlong_as_double(0x%08x%08xLL)", P.const_hi[c], P.const_bits[c]);
      v.literal64 = buf;
    } else if (P.const_f64[c] == 2) {
      std::snprintf(buf, sizeof(buf), "((long long)0x%08x%08xULL)", P.const_hi[c], P.const_bits[c]);
      v.int64_literal = buf;
    }
    regs[P.const_reg[c]] = v;  // class decided at use (float bits or int)
  }
  // loads
  for (int i = 0; i < P.n_in; ++i) {
    const EwOperand& o = P.in[i];
    const bool fl = is_float_dt(o.dt);
    Var v;
    v.is_float = fl;
    if (vec && packed_load(P, o)) {
      s << "  U4 r" << i << "[U];\n";
      v.name = "a" + std::to_string(i) + "#";  // widened per granule in the compute loop: indexed [j] only
    } else {
      s << "  " << (fl ? fty : ity) << " a" << i << "[U][E];\n";
      v.name = "a" + std::to_string(i);
    }
    regs[o.reg] = v;
  }
  s << "  #pragma unroll\n  for (int u = 0; u < U; ++u) {\n    const i64 v = vbase + (i64)u * 256;\n    if (v < nv) {\n";
  for (int i = 0; i < P.n_in; ++i) {
    const EwOperand& o = P.in[i];
    const char* tag = dt_tag(o.dt);
    if (vec && packed_load(P, o)) {
      const std::string at = "(const u16*)in" + std::to_string(i) + " + ";
      if (o.kind == EWI_FULL) s << "      r" << i << "[u] = ld16s(" << at << "v * 8);\n";
      else if (o.kind == EWI_MOD) s << "      r" << i << "[u] = ld16c(" << at << "(v * 8) % " << o.mod << "LL);\n";
      else s << "      r" << i << "[u] = ld16c(" << at << strided_index(P, o, "(v * 8)") << ");\n";
    } else if (vec) {
      if (o.kind == EWI_FULL) s << "      " << ld8_name(o.dt) << "(in" << i << ", v * 8, a" << i << "[u], true);\n";
      else if (o.kind == EWI_MOD && o.mod % 8 == 0)
        s << "      " << ld8_name(o.dt) << "(in" << i << ", (v * 8) % " << o.mod << "LL, a" << i << "[u], false);\n";
      else if (o.kind == EWI_MOD)
        s << "      #pragma unroll\n      for (int j = 0; j < 8; ++j) a" << i << "[u][j] = ld1_" << tag << "(in" << i
          << ", (v * 8 + j) % " << o.mod << "LL);\n";
      else if (o.kind == EWI_STRIDED && strided_run8_const(P, o))  // one value for the whole granule (a per-channel operand)
        s << "      { const " << (is_float_dt(o.dt) ? fty : ity) << " t = ld1_" << tag << "(in" << i << ", "
          << strided_index(P, o, "(v * 8)") << ");\n        #pragma unroll\n        for (int j = 0; j < 8; ++j) a" << i
          << "[u][j] = t; }\n";
      else if (o.kind == EWI_STRIDED && strided_vec8_ok(P, o))
        s << "      " << ld8_name(o.dt) << "(in" << i << ", " << strided_index(P, o, "(v * 8)") << ", a" << i << "[u], false);\n";
      else if (o.kind == EWI_STRIDED)
        s << "      #pragma unroll\n      for (int j = 0; j < 8; ++j) a" << i << "[u][j] = ld1_" << tag << "(in" << i
          << ", " << strided_index(P, o, "(v * 8 + j)") << ");\n";
      else  // scalar
        s << "      { const " << (is_float_dt(o.dt) ? fty : ity) << " t = ld1_" << tag << "(in" << i
          << ", 0);\n        #pragma unroll\n        for (int j = 0; j < 8; ++j) a" << i << "[u][j] = t; }\n";
    } else {
      if (o.kind == EWI_FULL) s << "      a" << i << "[u][0] = ld1_" << tag << "(in" << i << ", v);\n";
      else if (o.kind == EWI_MOD) s << "      a" << i << "[u][0] = ld1_" << tag << "(in" << i << ", v % " << o.mod << "LL);\n";
      else if (o.kind == EWI_STRIDED)
        s << "      a" << i << "[u][0] = ld1_" << tag << "(in" << i << ", " << strided_index(P, o, "v") << ");\n";
      else s << "      a" << i << "[u][0] = ld1_" << tag << "(in" << i << ", 0);\n";
    }
  }
  s << "    }\n  }\n";
  // compute + store
  s << "  #pragma unroll\n  for (int u = 0; u < U; ++u) {\n    const i64 v = vbase + (i64)u * 256;\n    if (v < nv) {\n";
  for (int i = 0; i < P.n_in; ++i)
    if (vec && packed_load(P, P.in[i]))
      s << "      float a" << i << "[E];\n      cvt8_" << dt_tag(P.in[i].dt) << "(r" << i << "[u], a" << i << ");\n";
  auto ref = [&](int reg, bool want_float) -> std::string {
    const Var& v = regs[reg];
    if (v.is_const && want_float && f64)
      return !v.literal64.empty() ? v.literal64 : "(double)__uint_as_float(" + v.literal + ")";
    if (v.is_const && !want_float && !v.int64_literal.empty()) return v.int64_literal;
    if (v.is_const) return want_float ? "__uint_as_float(" + v.literal + ")" : (i64 ? "(long long)(int)" : "(int)") + v.literal;
    return v.name + "[u][j]";
  };
  int tcount = 0;
  for (int k = 0; k < P.n_instr; ++k) {
    const EwInstr& ins = P.instr[k];
    const bool fl = ins.cls == EWC_FLOAT;
    std::string name = "t" + std::to_string(tcount++);
    // results of a 16-bit type: the granule is computed unrounded, then rounded two values per instruction
    const bool pair_round = !f64 && pair_rounded(vec, ins.op, ins.dt, ins.cls);
    const std::string expr =
        instr_expr(ins.op, pair_round ? (int)DT::F32 : ins.dt, ins.cls, ins.src_cls, ins.a, ins.b, ins.c, ref, f64);
    s << "      " << (fl ? fty : ity) << " " << name << "[E];\n";
    s << "      #pragma unroll\n      for (int j = 0; j < E; ++j) " << name << "[j] = " << expr << ";\n";
    if (pair_round) s << "      rn8_" << dt_tag(ins.dt) << "(" << name << ");\n";
    Var nv;
    nv.name = name;
    nv.is_float = fl;
    regs[ins.dst] = nv;
    // later references use name[j], not name[u][j]
    regs[ins.dst].name = name + "#";
  }
  // fix-up of references: temporaries are indexed [j] only
  std::string body = s.str();
  {
    std::string fixed;
    fixed.reserve(body.size());
    for (size_t i = 0; i < body.size(); ++i) {
      if (body[i] == '#' && body.compare(i, 7, "#[u][j]") == 0) {
        fixed += "[j]";
        i += 6;
      } else {
        fixed.push_back(body[i]);
      }
    }
    body.swap(fixed);
  }
  std::ostringstream t;
  t << body;
  for (int i = 0; i < P.n_out; ++i) {
    const EwOperand& o = P.out[i];
    const Var& v = regs[o.reg];
    const char* tag = dt_tag(o.dt);
    const bool fl = is_float_dt(o.dt);
    std::string src;
    if (v.is_const) {
      const std::string cexpr = !fl ? (!v.int64_literal.empty() ? v.int64_literal : "(int)" + v.literal)
                                : f64 && !v.literal64.empty() ? v.literal64
                                                               : (f64 ? "(double)" : "") + ("__uint_as_float(" + v.literal + ")");
      t << "      " << (fl ? fty : ity) << " oc" << i << "[E];\n      #pragma unroll\n      for (int j = 0; j < E; ++j) oc"
        << i << "[j] = " << cexpr << ";\n";
      src = "oc" + std::to_string(i);
    } else if (!v.name.empty() && v.name.back() == '#') {
      src = v.name.substr(0, v.name.size() - 1);
    } else {
      src = v.name + "[u]";
    }
    if (o.kind == EWI_STRIDED) {
      if (vec && strided_vec8_ok(P, o))
        t << "      " << st8_name(o.dt) << "(out" << i << ", " << strided_index(P, o, "(v * 8)") << ", " << src << ");\n";
      else if (vec)
        t << "      #pragma unroll\n      for (int j = 0; j < 8; ++j) st1_" << tag << "(out" << i << ", "
          << strided_index(P, o, "(v * 8 + j)") << ", " << src << "[j]);\n";
      else
        t << "      st1_" << tag << "(out" << i << ", " << strided_index(P, o, "v") << ", " << src << "[0]);\n";
    } else if (vec) {
      t << "      " << st8_name(o.dt) << "(out" << i << ", v * 8, " << src << ");\n";
    } else {
      t << "      st1_" << tag << "(out" << i << ", v, " << src << "[0]);\n";
    }
  }
  t << "    }\n  }\n}\n";
  *out = t.str();
  return true;
}


// ---- row programs --------------------------------------------------------------------------------------------------
struct RowShape {
  int vw = 8;    // elements per granule: 8 (16-byte accesses) or 1
  int nv = 1;    // granules per thread
  int t = 32;    // threads that own one row (a power of two)
  int tpb = 128; // threads per CTA
  int cluster = 1;        // CTAs that share one row (multi-pass schedule with the row staged in shared memory)
  unsigned dyn_smem = 0;  // dynamic shared memory of the kernel, bytes
};

int max_live_full(const RowProgram& P) {
  const int n = P.n_val, ni = (int)P.instr.size();
  std::vector<int> def(n, -1), last(n, -1);
  for (int i = 0; i < ni; ++i) {
    const RowInstr& x = P.instr[i];
    def[x.dst] = i;
    last[x.a] = i;
    if (!x.reduce) {
      last[x.b] = std::max(last[x.b], i);
      last[x.c] = std::max(last[x.c], i);
    }
  }
  for (auto& o : P.out) last[o.val] = ni;
  int best = 1;
  for (int i = 0; i <= ni; ++i) {
    int live = 0;
    for (int v = 0; v < n; ++v)
      if (P.val_full[v] && def[v] < i && last[v] >= i) ++live;
    best = std::max(best, live);
  }
  return best;
}

bool row_shape(const RowProgram& P, bool vec, RowShape* rs) {
  rs->vw = vec ? 8 : 1;
  const int64_t granules = (P.cols + rs->vw - 1) / rs->vw;
  int live = max_live_full(P);
  for (auto& o : P.out) live += o.kind == RK_COL && !P.col_reduce;  // column sums are kept in registers too
  // about 96 registers per thread for the per-element values that are live at once (measured: 160 costs occupancy
  // on 16-bit rows, 32 makes the thread groups too wide)
  int nv_max = std::max(1, 96 / (rs->vw * live));
  nv_max = std::min(nv_max, vec ? 8 : 32);
  int64_t t = 1;
  while (t * nv_max < granules) t <<= 1;
  int64_t coalesce = 1;
  while (coalesce < granules && coalesce < 32) coalesce <<= 1;
  t = std::max(t, coalesce);
  if (t > 512) return false;  // 1024-thread groups leave 64 registers per thread: the multi-pass schedule takes over
  rs->t = (int)t;
  rs->nv = (int)((granules + t - 1) / t);
  rs->tpb = std::max(128, rs->t);
  return true;
}


// Rows too long for registers: one CTA of 512 threads walks its row once per reduction and once more for the results,
// recomputing the per-element values each pass needs from the inputs (the later passes find the row in L2).  The same
// row program, the same per-op rounding; only the schedule differs from row_generate.
bool row_generate_multipass(const RowProgram& P, bool vec, std::string* out, RowShape* shape) {
  // sums over all rows: every thread keeps the sums of its own columns, NIT granules per result (registers)
  const int64_t nit = (P.cols + 512 * (vec ? 8 : 1) - 1) / (512 * (vec ? 8 : 1));
  if (P.col_sums && nit * (vec ? 8 : 1) > 32) return false;
  RowShape rs;
  rs.vw = vec ? 8 : 1;
  rs.t = 512;
  rs.tpb = 512;
  rs.nv = 0;  // marks the multi-pass schedule
  const int ni = (int)P.instr.size();
  // Which per-element inputs are read by more than one pass?  Those are staged: the first pass that reads them leaves
  // their bytes in shared memory and the later passes read them there, so the row crosses HBM/L2 once.  A row that
  // does not fit one CTA's shared memory is shared by a cluster of K CTAs (K = 2, 4 or 8): each keeps one K-th of the
  // columns, and the per-row reductions are completed through distributed shared memory (every CTA reads the K
  // partial results, in CTA order).
  std::vector<int> pass_uses(P.in.size(), 0);
  {
    std::vector<int> def_i(P.n_val, -1), def_in(P.n_val, -1);
    for (size_t i = 0; i < P.in.size(); ++i) def_in[P.in[i].val] = (int)i;
    for (int k = 0; k < ni; ++k) def_i[P.instr[k].dst] = k;
    auto count = [&](std::vector<int> stack) {
      std::vector<char> seen_i(ni, 0), seen_in(P.in.size(), 0);
      while (!stack.empty()) {
        const int v = stack.back();
        stack.pop_back();
        if (v < 0 || v >= P.n_val || !P.val_full[v]) continue;
        if (def_in[v] >= 0) {
          if (!seen_in[def_in[v]]) ++pass_uses[def_in[v]];
          seen_in[def_in[v]] = 1;
          continue;
        }
        const int k = def_i[v];
        if (k < 0 || seen_i[k]) continue;
        seen_i[k] = 1;
        stack.push_back(P.instr[k].a);
        if (!P.instr[k].reduce) {
          stack.push_back(P.instr[k].b);
          stack.push_back(P.instr[k].c);
        }
      }
    };
    std::vector<int> final_roots;
    for (int k = 0; k < ni; ++k)
      if (!P.instr[k].full && P.instr[k].reduce) count({P.instr[k].a});
    for (auto& o : P.out)
      if (o.kind == RK_FULL || o.kind == RK_COL) final_roots.push_back(o.val);
    if (!final_roots.empty()) count(final_roots);
  }
  std::vector<int64_t> stage_off(P.in.size(), -1);  // byte offset of a staged input in the CTA's dynamic shared memory
  int K = 1;
  int64_t CH = P.cols;  // columns per CTA
  if (vec && !P.col_sums && P.stage_long_rows) {
    int64_t row_bytes = 0;
    for (size_t i = 0; i < P.in.size(); ++i)
      if (P.in[i].kind == RK_FULL && is_float_dt(P.in[i].dt) && pass_uses[i] >= 2)
        row_bytes += P.cols * (int64_t)((DT)P.in[i].dt == DT::F32 ? 4 : 2);
    if (row_bytes > 0) {
      // at most 72 KB per CTA, so that three CTAs of 512 threads stay resident per SM
      while (K < 8 && (row_bytes + K - 1) / K > 72 * 1024) K *= 2;
      const int64_t granules = (P.cols + 7) / 8;
      CH = ((granules + K - 1) / K) * 8;
      int64_t off = 0;
      for (size_t i = 0; i < P.in.size(); ++i)
        if (P.in[i].kind == RK_FULL && is_float_dt(P.in[i].dt) && pass_uses[i] >= 2) {
          stage_off[i] = off;
          off += CH * (int64_t)((DT)P.in[i].dt == DT::F32 ? 4 : 2);
        }
      if (off > 200 * 1024) {  // does not fit even as a cluster of 8: the passes re-read the row through L2
        K = 1;
        CH = P.cols;
        std::fill(stage_off.begin(), stage_off.end(), -1);
      } else {
        rs.cluster = K;
        rs.dyn_smem = (unsigned)off;
      }
    }
  }
  const bool staged = rs.dyn_smem > 0;
  *shape = rs;
  std::ostringstream s;
  s << kPreamble;
  s << "constexpr int C = " << P.cols << ", T = 512, TPB = 512, VW = " << rs.vw << ", K = " << K << ";\n";
  s << "constexpr i64 CH = " << CH << ";\n";
  s << R"SRC(
__device__ __forceinline__ U4 ld16p(const void* p, unsigned long long pol) { U4 v; v.x = v.y = v.z = v.w = 0; AKGB_CHK(p, 16, v)
  asm volatile("ld.global.nc.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(pol)); return v; }
__device__ __forceinline__ void ld8p_f32(const void* p, i64 e0, float* r, unsigned long long pol) {
  const U4 a = ld16p((const float*)p + e0, pol), b = ld16p((const float*)p + e0 + 4, pol);
  r[0] = __uint_as_float(a.x); r[1] = __uint_as_float(a.y); r[2] = __uint_as_float(a.z); r[3] = __uint_as_float(a.w);
  r[4] = __uint_as_float(b.x); r[5] = __uint_as_float(b.y); r[6] = __uint_as_float(b.z); r[7] = __uint_as_float(b.w); }
__device__ __forceinline__ void ld8p_f16(const void* p, i64 e0, float* r, unsigned long long pol) {
  const U4 v = ld16p((const u16*)p + e0, pol); const u32 w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { r[2*i] = h2f((u16)(w[i] & 0xffffu)); r[2*i+1] = h2f((u16)(w[i] >> 16)); } }
__device__ __forceinline__ void ld8p_bf16(const void* p, i64 e0, float* r, unsigned long long pol) {
  const U4 v = ld16p((const u16*)p + e0, pol); const u32 w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { r[2*i] = b2f((u16)(w[i] & 0xffffu)); r[2*i+1] = b2f((u16)(w[i] >> 16)); } }
template <int OP> __device__ __forceinline__ float comb(float a, float b) {
  return OP == 0 ? __fadd_rn(a, b) : OP == 1 ? fmaxf(a, b) : OP == 2 ? fminf(a, b) : __fmul_rn(a, b);
}
template <int OP> __device__ __forceinline__ float row_reduce(float v, float* sm) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = comb<OP>(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
  __syncthreads();
  v = sm[0];
#pragma unroll
  for (int w = 1; w < T / 32; ++w) v = comb<OP>(v, sm[w]);
  return v;
}
// staged rows: the first pass keeps the bytes it loads in shared memory (sp, element s0), later passes read them there
__device__ __forceinline__ void ld8ps_f32(const void* p, i64 e0, float* r, unsigned long long pol, void* sp, i64 s0) {
  const U4 a = ld16p((const float*)p + e0, pol), b = ld16p((const float*)p + e0 + 4, pol);
  U4* d = (U4*)((float*)sp + s0); d[0] = a; d[1] = b;
  r[0] = __uint_as_float(a.x); r[1] = __uint_as_float(a.y); r[2] = __uint_as_float(a.z); r[3] = __uint_as_float(a.w);
  r[4] = __uint_as_float(b.x); r[5] = __uint_as_float(b.y); r[6] = __uint_as_float(b.z); r[7] = __uint_as_float(b.w); }
__device__ __forceinline__ void ld8s_f32(const void* sp, i64 s0, float* r) {
  const U4* d = (const U4*)((const float*)sp + s0); const U4 a = d[0], b = d[1];
  r[0] = __uint_as_float(a.x); r[1] = __uint_as_float(a.y); r[2] = __uint_as_float(a.z); r[3] = __uint_as_float(a.w);
  r[4] = __uint_as_float(b.x); r[5] = __uint_as_float(b.y); r[6] = __uint_as_float(b.z); r[7] = __uint_as_float(b.w); }
__device__ __forceinline__ void ld8ps_f16(const void* p, i64 e0, float* r, unsigned long long pol, void* sp, i64 s0) {
  const U4 v = ld16p((const u16*)p + e0, pol); *(U4*)((u16*)sp + s0) = v; const u32 w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { r[2*i] = h2f((u16)(w[i] & 0xffffu)); r[2*i+1] = h2f((u16)(w[i] >> 16)); } }
__device__ __forceinline__ void ld8s_f16(const void* sp, i64 s0, float* r) {
  const U4 v = *(const U4*)((const u16*)sp + s0); const u32 w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { r[2*i] = h2f((u16)(w[i] & 0xffffu)); r[2*i+1] = h2f((u16)(w[i] >> 16)); } }
__device__ __forceinline__ void ld8ps_bf16(const void* p, i64 e0, float* r, unsigned long long pol, void* sp, i64 s0) {
  const U4 v = ld16p((const u16*)p + e0, pol); *(U4*)((u16*)sp + s0) = v; const u32 w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { r[2*i] = b2f((u16)(w[i] & 0xffffu)); r[2*i+1] = b2f((u16)(w[i] >> 16)); } }
__device__ __forceinline__ void ld8s_bf16(const void* sp, i64 s0, float* r) {
  const U4 v = *(const U4*)((const u16*)sp + s0); const u32 w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { r[2*i] = b2f((u16)(w[i] & 0xffffu)); r[2*i+1] = b2f((u16)(w[i] >> 16)); } }
// every thread of every CTA of the cluster arrives; nobody passes before all have (a hardware barrier, like
// __syncthreads for the cluster), with release / acquire ordering of shared-memory accesses across the CTAs
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the row's reduction over all K CTAs: each CTA publishes its own result, then reads everybody's through distributed
// shared memory and folds them in CTA order, so all CTAs hold the same bits
template <int OP> __device__ __forceinline__ float row_reduce_cl(float v, float* sm, float* slot) {
  v = row_reduce<OP>(v, sm);
  if (K == 1) return v;
  if (threadIdx.x == 0) *slot = v;
  cluster_sync();
  const u32 a = (u32)__cvta_generic_to_shared(slot);
  float r = 0.f;
#pragma unroll
  for (int q = 0; q < K; ++q) {
    u32 ra; float x;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(q));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(x) : "r"(ra) : "memory");
    r = q == 0 ? x : comb<OP>(r, x);
  }
  return r;
}
)SRC";
  s << "extern \"C\" __global__ void ";
  if (K > 1) s << "__cluster_dims__(" << K << ", 1, 1) ";
  s << "__launch_bounds__(TPB) akgb_row_jit(";
  for (size_t i = 0; i < P.in.size(); ++i) s << "const void* __restrict__ in" << i << ", ";
  for (size_t i = 0; i < P.out.size(); ++i) s << "void* __restrict__ out" << i << ", ";
  s << "i64 rows) {\n";
  s << "  __shared__ float sm[TPB / 32];\n  const int tr = threadIdx.x;\n";
  if (staged) {
    s << "  extern __shared__ __align__(16) unsigned char stage_mem[];\n";
    s << "  __shared__ float cl_slot[" << std::max(1, ni) << "];\n";
    s << "  const i64 c_lo = (i64)(blockIdx.x % K) * CH, c_hi = c_lo + CH < C ? c_lo + CH : (i64)C;\n";
  } else {
    s << "  constexpr i64 c_lo = 0, c_hi = C;\n";
  }
  if (P.col_sums) {
    s << "  constexpr int NIT = " << nit << ";\n";
    for (size_t i = 0; i < P.out.size(); ++i)
      if (P.out[i].kind == RK_COL)
        s << "  float cs" << i << "[NIT][VW];\n#pragma unroll\n  for (int q = 0; q < NIT; ++q) {\n#pragma unroll\n"
             "    for (int j = 0; j < VW; ++j) cs" << i << "[q][j] = 0.f;\n  }\n";
    s << "  for (i64 r = blockIdx.x; r < rows; r += gridDim.x) {\n";  // a fixed number of CTAs walk the rows
  } else {
    s << "  const i64 r = blockIdx.x / K;\n";
  }
  // L2 policies: a row stays resident while later passes still need it and leaves first once the last pass has read it
  s << "  unsigned long long pol_last, pol_first;\n"
         "  asm volatile(\"createpolicy.fractional.L2::evict_last.b64 %0, 1.0;\" : \"=l\"(pol_last));\n"
         "  asm volatile(\"createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\" : \"=l\"(pol_first));\n";
  std::vector<std::string> name(P.n_val);
  std::vector<char> is_const(P.n_val, 0);
  std::vector<int> def_instr(P.n_val, -1), def_input(P.n_val, -1);
  for (size_t c = 0; c < P.const_val.size(); ++c) {
    char buf[32];
    std::snprintf(buf, sizeof(buf), "0x%08xu", P.const_bits[c]);
    name[P.const_val[c]] = buf;
    is_const[P.const_val[c]] = 1;
  }
  for (size_t i = 0; i < P.in.size(); ++i) {
    const RowOperand& o = P.in[i];
    name[o.val] = "x" + std::to_string(i);
    def_input[o.val] = (int)i;
    if (o.kind == RK_ROW || o.kind == RK_SCALAR) {
      std::string idx = o.kind == RK_ROW ? "r" : "0";
      if (o.kind == RK_ROW && o.row_mod != 0)
        idx = "(r / " + std::to_string(o.row_div) + "LL) % " + std::to_string(o.row_mod) + "LL";
      s << "  const " << (is_float_dt(o.dt) ? "float " : "int ") << name[o.val] << " = ld1_" << dt_tag(o.dt) << "(in" << i
        << ", " << idx << ");\n";
    }
  }
  for (int k = 0; k < ni; ++k) {
    def_instr[P.instr[k].dst] = k;
    name[P.instr[k].dst] = "t" + std::to_string(k);
  }
  auto ref = [&](int val, bool want_float) -> std::string {
    if (is_const[val]) return want_float ? "__uint_as_float(" + name[val] + ")" : "(int)" + name[val];
    return P.val_full[val] ? name[val] + "[j]" : name[val];
  };
  // one pass over the row: everything per-element that `roots` need, recomputed from the inputs, then `tail`
  int pass_no = 0;
  std::vector<char> stage_filled(P.in.size(), 0);
  auto emit_pass = [&](const std::vector<int>& roots, const std::string& tail, bool last = false) {
    std::vector<int> filled_now;
    std::vector<char> need_instr(ni, 0), need_input(P.in.size(), 0);
    std::vector<int> stack(roots.begin(), roots.end());
    while (!stack.empty()) {
      const int v = stack.back();
      stack.pop_back();
      if (!P.val_full[v] || is_const[v]) continue;
      if (def_input[v] >= 0) {
        need_input[def_input[v]] = 1;
        continue;
      }
      const int k = def_instr[v];
      if (k < 0 || need_instr[k]) continue;
      need_instr[k] = 1;
      const RowInstr& x = P.instr[k];
      stack.push_back(x.a);
      if (!x.reduce) {
        stack.push_back(x.b);
        stack.push_back(x.c);
      }
    }
    const bool rev = !staged && (pass_no & 1);  // every other pass walks backwards: it starts with what the pass before left in L2
    if (P.col_sums && last)  // fully unrolled, so that the column sums are indexed statically
      s << "#pragma unroll\n  for (int q = 0; q < NIT; ++q) {\n    const int it = " << (rev ? "NIT - 1 - q" : "q")
        << ";\n    const i64 c = (i64)tr * VW + (i64)it * (T * VW);\n    if (c >= C) continue;\n";
    else if (rev) s << "#pragma unroll 2\n  for (i64 c = (i64)tr * VW + (i64)((C - 1) / (T * VW)) * (T * VW); c >= 0; c -= (i64)T * VW) {\n    if (c >= C) continue;\n";
    else s << "#pragma unroll 2\n  for (i64 c = c_lo + (i64)tr * VW; c < c_hi; c += (i64)T * VW) {\n";
    ++pass_no;
    for (size_t i = 0; i < P.in.size(); ++i) {
      if (!need_input[i]) continue;
      const RowOperand& o = P.in[i];
      const std::string base = o.kind == RK_FULL ? "r * C" : o.kind == RK_COL ? "(i64)0" : "(r % " + std::to_string(o.mod_rows) + "LL) * C";
      s << "    " << (is_float_dt(o.dt) ? "float " : "int ") << name[o.val] << "[VW];\n";
      const bool pol = vec && o.kind == RK_FULL && is_float_dt(o.dt);
      if (stage_off[i] >= 0 && !stage_filled[i]) {  // first pass over this input: from memory, kept in shared memory
        s << "    ld8ps_" << dt_tag(o.dt) << "(in" << i << ", " << base << " + c, " << name[o.val] << ", pol_first, stage_mem + "
          << stage_off[i] << ", c - c_lo);\n";
        filled_now.push_back((int)i);
      } else if (stage_off[i] >= 0) {
        s << "    ld8s_" << dt_tag(o.dt) << "(stage_mem + " << stage_off[i] << ", c - c_lo, " << name[o.val] << ");\n";
      } else if (pol) s << "    ld8p_" << dt_tag(o.dt) << "(in" << i << ", " << base << " + c, " << name[o.val] << ", " << (last ? "pol_first" : "pol_last") << ");\n";
      else if (vec) s << "    ld8_" << dt_tag(o.dt) << "(in" << i << ", " << base << " + c, " << name[o.val] << ", false);\n";
      else s << "    " << name[o.val] << "[0] = ld1_" << dt_tag(o.dt) << "(in" << i << ", " << base << " + c);\n";
    }
    for (int k = 0; k < ni; ++k) {
      if (!need_instr[k]) continue;
      const RowInstr& x = P.instr[k];
      const bool pr = pair_rounded(vec, x.op, x.dt, x.cls);
      const std::string expr = instr_expr(x.op, pr ? (int)DT::F32 : x.dt, x.cls, x.src_cls, x.a, x.b, x.c, ref);
      s << "    " << (x.cls == EWC_FLOAT ? "float " : "int ") << name[x.dst] << "[VW];\n#pragma unroll\n    for (int j = 0; j < VW; ++j) "
        << name[x.dst] << "[j] = " << expr << ";\n";
      if (pr) s << "    rn8_" << dt_tag(x.dt) << "(" << name[x.dst] << ");\n";
    }
    s << tail << "  }\n";
    // (every pass gives a thread the same columns, so a thread reads back only what it staged itself: no barrier)
    for (int i : filled_now) stage_filled[i] = 1;
  };
  for (int k = 0; k < ni; ++k) {
    const RowInstr& x = P.instr[k];
    if (x.full) continue;  // per-element values are computed inside the passes that need them
    if (x.reduce) {
      const char* ident = x.red_op == 0 ? "0.f" : x.red_op == 1 ? "-3.402823466e+38f" : x.red_op == 2 ? "3.402823466e+38f" : "1.f";
      s << "  float acc" << k << " = " << ident << ";\n";
      std::ostringstream tail;
      tail << "#pragma unroll\n    for (int j = 0; j < VW; ++j) acc" << k << " = comb<" << x.red_op << ">(acc" << k << ", "
           << name[x.a] << "[j]);\n";
      emit_pass({x.a}, tail.str());
      if (staged)
        s << "  const float " << name[x.dst] << " = " << round_fn(x.dt) << "(row_reduce_cl<" << x.red_op << ">(acc" << k
          << ", sm, cl_slot + " << k << "));\n";
      else
        s << "  const float " << name[x.dst] << " = " << round_fn(x.dt) << "(row_reduce<" << x.red_op << ">(acc" << k << ", sm));\n";
    } else {
      const std::string expr = instr_expr(x.op, x.dt, x.cls, x.src_cls, x.a, x.b, x.c, ref);
      s << "  const " << (x.cls == EWC_FLOAT ? "float " : "int ") << name[x.dst] << " = " << expr << ";\n";
    }
  }
  std::vector<int> roots;
  std::ostringstream tail;
  for (size_t i = 0; i < P.out.size(); ++i) {
    const RowOperand& o = P.out[i];
    if (o.kind != RK_FULL) continue;
    roots.push_back(o.val);
    if (vec) tail << "    st8_" << dt_tag(o.dt) << "(out" << i << ", r * C + c, " << name[o.val] << ");\n";
    else tail << "    st1_" << dt_tag(o.dt) << "(out" << i << ", r * C + c, " << name[o.val] << "[0]);\n";
  }
  for (size_t i = 0; i < P.out.size(); ++i) {
    const RowOperand& o = P.out[i];
    if (o.kind != RK_COL) continue;
    roots.push_back(o.val);
    tail << "#pragma unroll\n    for (int j = 0; j < VW; ++j) cs" << i << "[it][j] = __fadd_rn(cs" << i << "[it][j], "
         << name[o.val] << "[j]);\n";
  }
  if (!roots.empty()) emit_pass(roots, tail.str(), true);
  for (size_t i = 0; i < P.out.size(); ++i) {
    const RowOperand& o = P.out[i];
    if (o.kind == RK_ROW)
      s << "  if (tr == 0) st1_" << dt_tag(o.dt) << "(out" << i << ", r, " << ref(o.val, is_float_dt(o.dt)) << ");\n";
  }
  if (staged && K > 1) s << "  cluster_sync();\n";  // no CTA leaves while another may still read its partial results
  if (P.col_sums) {
    s << "  }\n";  // the walk over the rows
    for (size_t i = 0; i < P.out.size(); ++i) {
      if (P.out[i].kind != RK_COL) continue;
      s << "#pragma unroll\n  for (int q = 0; q < NIT; ++q) {\n    const i64 c = (i64)tr * VW + (i64)q * (T * VW);\n#pragma unroll\n"
           "    for (int j = 0; j < VW; ++j)\n      if (c + j < C) st1_f32(out" << i << ", (i64)blockIdx.x * C + c + j, cs" << i
        << "[q][j]);\n  }\n";
    }
  }
  s << "}\n";
  *out = s.str();
  return true;
}

bool row_generate(const RowProgram& P, bool vec, std::string* out, RowShape* shape) {
  RowShape rs;
  if (!row_shape(P, vec, &rs)) return row_generate_multipass(P, vec, out, shape);
  *shape = rs;
  std::ostringstream s;
  s << kPreamble;
  s << "constexpr int C = " << P.cols << ", T = " << rs.t << ", TPB = " << rs.tpb << ", VW = " << rs.vw
    << ", NV = " << rs.nv << ", RPB = TPB / T;\n";
  s << R"SRC(
template <int OP> __device__ __forceinline__ float comb(float a, float b) {
  return OP == 0 ? __fadd_rn(a, b) : OP == 1 ? fmaxf(a, b) : OP == 2 ? fminf(a, b) : __fmul_rn(a, b);
}
// the same value in every thread of the row's group: butterfly inside a warp, then the group's warps through shared memory
template <int OP> __device__ __forceinline__ float row_reduce(float v, float* sm) {
#pragma unroll
  for (int o = (T < 32 ? T : 32) / 2; o > 0; o >>= 1) v = comb<OP>(v, __shfl_xor_sync(0xffffffffu, v, o));
  if (T > 32) {
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
    __syncthreads();
    const int first = (threadIdx.x / T) * (T / 32);
    v = sm[first];
#pragma unroll
    for (int w = 1; w < T / 32; ++w) v = comb<OP>(v, sm[first + w]);
  }
  return v;
}
)SRC";
  s << "extern \"C\" __global__ void __launch_bounds__(TPB) akgb_row_jit(";
  for (size_t i = 0; i < P.in.size(); ++i) s << "const void* __restrict__ in" << i << ", ";
  for (size_t i = 0; i < P.out.size(); ++i) s << "void* __restrict__ out" << i << ", ";
  s << "i64 rows) {\n";
  s << "  __shared__ float sm[TPB / 32];\n";
  s << "  const int tr = threadIdx.x % T;\n";
  if (P.col_sums) {
    // a fixed number of CTAs walk the row blocks; every thread keeps the sums of its own columns
    s << "  __shared__ float smc[TPB][VW];\n";
    for (size_t i = 0; i < P.out.size(); ++i)
      if (P.out[i].kind == RK_COL)
        s << "  float cs" << i << "[NV][VW];\n#pragma unroll\n  for (int k = 0; k < NV; ++k) {\n#pragma unroll\n"
             "    for (int j = 0; j < VW; ++j) cs" << i << "[k][j] = 0.f;\n  }\n";
    s << "  const i64 nblk = (rows + RPB - 1) / RPB;\n";
    s << "  for (i64 rb = blockIdx.x; rb < nblk; rb += gridDim.x) {\n";
    s << "  const i64 row0 = rb * RPB + threadIdx.x / T;\n";
  } else {
    s << "  const i64 row0 = (i64)blockIdx.x * RPB + threadIdx.x / T;\n";
  }
  s << "  const bool active = row0 < rows;\n";
  s << "  const i64 r = active ? row0 : rows - 1;\n";
  std::vector<std::string> name(P.n_val);
  std::vector<char> is_float(P.n_val, 1), is_const(P.n_val, 0);
  for (size_t c = 0; c < P.const_val.size(); ++c) {
    char buf[32];
    std::snprintf(buf, sizeof(buf), "0x%08xu", P.const_bits[c]);
    name[P.const_val[c]] = buf;
    is_const[P.const_val[c]] = 1;
  }
  // loads
  for (size_t i = 0; i < P.in.size(); ++i) {
    const RowOperand& o = P.in[i];
    const bool fl = is_float_dt(o.dt);
    const char* ty = fl ? "float" : "int";
    const char* tag = dt_tag(o.dt);
    const std::string v = "x" + std::to_string(i);
    name[o.val] = v;
    is_float[o.val] = fl;
    if (o.kind == RK_ROW || o.kind == RK_SCALAR) {
      std::string idx = o.kind == RK_ROW ? "r" : "0";
      if (o.kind == RK_ROW && o.row_mod != 0)
        idx = "(r / " + std::to_string(o.row_div) + "LL) % " + std::to_string(o.row_mod) + "LL";
      s << "  const " << ty << " " << v << " = ld1_" << tag << "(in" << i << ", " << idx << ");\n";
      continue;
    }
    std::string base = o.kind == RK_FULL ? "r * C" : o.kind == RK_COL ? "(i64)0" : "(r % " + std::to_string(o.mod_rows) + "LL) * C";
    s << "  " << ty << " " << v << "[NV][VW];\n";
    s << "#pragma unroll\n  for (int k = 0; k < NV; ++k) {\n    const int c = (tr + T * k) * VW;\n";
    if (vec) {
      s << "    if (c < C) ld8_" << tag << "(in" << i << ", " << base << " + c, " << v << "[k], "
        << (o.kind == RK_FULL ? "true" : "false") << ");\n";
      s << "    else {\n#pragma unroll\n      for (int j = 0; j < VW; ++j) " << v << "[k][j] = 0; }\n";
    } else {
      s << "    " << v << "[k][0] = c < C ? ld1_" << tag << "(in" << i << ", " << base << " + c) : 0;\n";
    }
    s << "  }\n";
  }
  auto ref_full = [&](int val, bool want_float) -> std::string {
    if (is_const[val]) return want_float ? "__uint_as_float(" + name[val] + ")" : "(int)" + name[val];
    return P.val_full[val] ? name[val] + "[k][j]" : name[val];
  };
  for (size_t k = 0; k < P.instr.size(); ++k) {
    const RowInstr& x = P.instr[k];
    const bool fl = x.cls == EWC_FLOAT;
    const std::string v = "t" + std::to_string(k);
    name[x.dst] = v;
    is_float[x.dst] = fl;
    if (x.reduce) {
      const char* ident = x.red_op == 0 ? "0.f" : x.red_op == 1 ? "-3.402823466e+38f" : x.red_op == 2 ? "3.402823466e+38f" : "1.f";
      s << "  float " << v << ";\n  {\n    float acc = " << ident << ";\n";
      s << "#pragma unroll\n    for (int k = 0; k < NV; ++k) {\n#pragma unroll\n      for (int j = 0; j < VW; ++j)\n";
      s << "        if ((tr + T * k) * VW + j < C) acc = comb<" << x.red_op << ">(acc, " << name[x.a] << "[k][j]);\n    }\n";
      s << "    " << v << " = " << round_fn(x.dt) << "(row_reduce<" << x.red_op << ">(acc, sm));\n  }\n";
      continue;
    }
    const bool pr = x.full && pair_rounded(vec, x.op, x.dt, x.cls);
    const std::string expr = instr_expr(x.op, pr ? (int)DT::F32 : x.dt, x.cls, x.src_cls, x.a, x.b, x.c, ref_full);
    if (x.full) {
      s << "  " << (fl ? "float " : "int ") << v << "[NV][VW];\n";
      s << "#pragma unroll\n  for (int k = 0; k < NV; ++k) {\n#pragma unroll\n    for (int j = 0; j < VW; ++j) " << v
        << "[k][j] = " << expr << ";\n";
      if (pr) s << "    rn8_" << dt_tag(x.dt) << "(" << v << "[k]);\n";
      s << "  }\n";
    } else {
      s << "  const " << (fl ? "float " : "int ") << v << " = " << expr << ";\n";
    }
  }
  // stores
  for (size_t i = 0; i < P.out.size(); ++i) {
    const RowOperand& o = P.out[i];
    const char* tag = dt_tag(o.dt);
    if (o.kind == RK_ROW) {
      const bool fl = is_float_dt(o.dt);
      s << "  if (active && tr == 0) st1_" << tag << "(out" << i << ", r, " << ref_full(o.val, fl) << ");\n";
      continue;
    }
    if (o.kind == RK_COL) {
      s << "  if (active) {\n#pragma unroll\n    for (int k = 0; k < NV; ++k) {\n#pragma unroll\n      for (int j = 0; j < VW; ++j) cs"
        << i << "[k][j] = __fadd_rn(cs" << i << "[k][j], " << name[o.val] << "[k][j]);\n    }\n  }\n";
      continue;
    }
    s << "  if (active) {\n#pragma unroll\n    for (int k = 0; k < NV; ++k) {\n      const int c = (tr + T * k) * VW;\n";
    if (vec) s << "      if (c < C) st8_" << tag << "(out" << i << ", r * C + c, " << name[o.val] << "[k]);\n";
    else s << "      if (c < C) st1_" << tag << "(out" << i << ", r * C + c, " << name[o.val] << "[k][0]);\n";
    s << "    }\n  }\n";
  }
  if (P.col_sums) {
    s << "  }\n";  // the walk over the row blocks
    // the row groups of the CTA hold sums of the same columns: folded in group order, one partial vector per CTA
    for (size_t i = 0; i < P.out.size(); ++i) {
      if (P.out[i].kind != RK_COL) continue;
      s << "#pragma unroll\n  for (int k = 0; k < NV; ++k) {\n    __syncthreads();\n#pragma unroll\n"
           "    for (int j = 0; j < VW; ++j) smc[threadIdx.x][j] = cs" << i << "[k][j];\n    __syncthreads();\n"
           "    if (threadIdx.x < T) {\n      const int c = (tr + T * k) * VW;\n#pragma unroll\n      for (int j = 0; j < VW; ++j) {\n"
           "        float a = smc[tr][j];\n        for (int g2 = 1; g2 < RPB; ++g2) a = __fadd_rn(a, smc[g2 * T + tr][j]);\n"
           "        if (c + j < C) st1_f32(out" << i << ", (i64)blockIdx.x * C + c + j, a);\n      }\n    }\n  }\n";
    }
  }
  s << "}\n";
  *out = s.str();
  return true;
}


// ---- column programs: an elementwise chain folded over the rows of [rows, cols] in the pass that reads it --------
struct ColShape {
  int vw = 8, tx = 32, ty = 8;
};

bool col_generate(const RowProgram& P, bool vec, std::string* out, ColShape* shape) {
  if (!P.col_reduce || P.out.empty() || P.out.size() > 4) return false;
  ColShape cs;
  cs.vw = vec ? 8 : 1;
  const int64_t granules = (P.cols + cs.vw - 1) / cs.vw;
  cs.tx = 1;
  while (cs.tx < 32 && cs.tx < granules) cs.tx <<= 1;
  cs.ty = 256 / cs.tx;
  *shape = cs;
  std::ostringstream s;
  s << kPreamble;
  s << "constexpr int C = " << P.cols << ", TX = " << cs.tx << ", TY = " << cs.ty << ", VW = " << cs.vw << ";\n";
  s << R"SRC(
template <int OP> __device__ __forceinline__ float comb(float a, float b) {
  return OP == 0 ? __fadd_rn(a, b) : OP == 1 ? fmaxf(a, b) : OP == 2 ? fminf(a, b) : __fmul_rn(a, b);
}
)SRC";
  auto ident_of = [](int op) { return op == 0 ? "0.f" : op == 1 ? "-3.402823466e+38f" : op == 2 ? "3.402823466e+38f" : "1.f"; };
  s << "extern \"C\" __global__ void __launch_bounds__(256) akgb_col_jit(";
  for (size_t i = 0; i < P.in.size(); ++i) s << "const void* __restrict__ in" << i << ", ";
  for (size_t i = 0; i < P.out.size(); ++i) s << "float* __restrict__ partial" << i << ", ";
  s << "i64 rows, i64 rows_per_split) {\n";
  s << "  __shared__ float sm[TY][TX * VW + 1];\n";
  s << "  const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;\n";
  s << "  const i64 c = ((i64)blockIdx.x * TX + tx) * VW;\n";
  s << "  const bool valid = c < C;\n";
  s << "  const i64 r0 = (i64)blockIdx.y * rows_per_split;\n";
  s << "  const i64 r1 = r0 + rows_per_split < rows ? r0 + rows_per_split : rows;\n";
  std::vector<std::string> name(P.n_val);
  std::vector<char> is_const(P.n_val, 0);
  for (size_t k = 0; k < P.const_val.size(); ++k) {
    char buf[32];
    std::snprintf(buf, sizeof(buf), "0x%08xu", P.const_bits[k]);
    name[P.const_val[k]] = buf;
    is_const[P.const_val[k]] = 1;
  }
  auto load_full = [&](std::ostream& o, size_t i, const std::string& base) {
    const RowOperand& op = P.in[i];
    const char* tag = dt_tag(op.dt);
    const std::string v = "x" + std::to_string(i);
    if (vec) o << "ld8_" << tag << "(in" << i << ", " << base << " + c, " << v << ", " << (op.kind == RK_FULL ? "true" : "false") << ");\n";
    else o << v << "[0] = ld1_" << tag << "(in" << i << ", " << base << " + c);\n";
  };
  // operands that do not change from row to row
  for (size_t i = 0; i < P.in.size(); ++i) {
    const RowOperand& op = P.in[i];
    const bool fl = is_float_dt(op.dt);
    const std::string v = "x" + std::to_string(i);
    name[op.val] = v;
    if (op.kind == RK_SCALAR) {
      s << "  const " << (fl ? "float " : "int ") << v << " = ld1_" << dt_tag(op.dt) << "(in" << i << ", 0);\n";
    } else if (op.kind == RK_COL) {
      s << "  " << (fl ? "float " : "int ") << v << "[VW];\n#pragma unroll\n  for (int j = 0; j < VW; ++j) " << v << "[j] = 0;\n";
      s << "  if (valid) { ";
      load_full(s, i, "(i64)0");
      s << "  }\n";
    }
  }
  for (size_t i = 0; i < P.out.size(); ++i)
    s << "  float acc" << i << "[VW];\n#pragma unroll\n  for (int j = 0; j < VW; ++j) acc" << i << "[j] = "
      << ident_of(P.out[i].red_op) << ";\n";
  s << "  if (valid) {\n#pragma unroll 4\n    for (i64 r = r0 + ty; r < r1; r += TY) {\n";
  for (size_t i = 0; i < P.in.size(); ++i) {
    const RowOperand& op = P.in[i];
    const bool fl = is_float_dt(op.dt);
    const std::string v = "x" + std::to_string(i);
    if (op.kind == RK_ROW) {
      s << "      const " << (fl ? "float " : "int ") << v << " = ld1_" << dt_tag(op.dt) << "(in" << i << ", r);\n";
    } else if (op.kind == RK_FULL || op.kind == RK_ROWMOD) {
      s << "      " << (fl ? "float " : "int ") << v << "[VW];\n      ";
      load_full(s, i, op.kind == RK_FULL ? "r * C" : "(r % " + std::to_string(op.mod_rows) + "LL) * C");
    }
  }
  auto ref = [&](int val, bool want_float) -> std::string {
    if (is_const[val]) return want_float ? "__uint_as_float(" + name[val] + ")" : "(int)" + name[val];
    return P.val_full[val] ? name[val] + "[j]" : name[val];
  };
  for (size_t k = 0; k < P.instr.size(); ++k) {
    const RowInstr& x = P.instr[k];
    if (x.reduce) return false;
    const bool fl = x.cls == EWC_FLOAT;
    const std::string v = "t" + std::to_string(k);
    name[x.dst] = v;
    const bool pr = x.full && pair_rounded(vec, x.op, x.dt, x.cls);
    const std::string expr = instr_expr(x.op, pr ? (int)DT::F32 : x.dt, x.cls, x.src_cls, x.a, x.b, x.c, ref);
    if (x.full) {
      s << "      " << (fl ? "float " : "int ") << v << "[VW];\n#pragma unroll\n      for (int j = 0; j < VW; ++j) " << v
        << "[j] = " << expr << ";\n";
      if (pr) s << "      rn8_" << dt_tag(x.dt) << "(" << v << ");\n";
    } else {
      s << "      const " << (fl ? "float " : "int ") << v << " = " << expr << ";\n";
    }
  }
  for (size_t i = 0; i < P.out.size(); ++i)
    s << "#pragma unroll\n      for (int j = 0; j < VW; ++j) acc" << i << "[j] = comb<" << P.out[i].red_op << ">(acc" << i
      << "[j], " << name[P.out[i].val] << "[j]);\n";
  s << "    }\n  }\n";
  for (size_t i = 0; i < P.out.size(); ++i) {
    const int op = P.out[i].red_op;
    if (i) s << "  __syncthreads();\n";
    s << "#pragma unroll\n  for (int j = 0; j < VW; ++j) sm[ty][tx * VW + j] = acc" << i << "[j];\n  __syncthreads();\n";
    s << "#pragma unroll\n  for (int h = TY / 2; h > 0; h >>= 1) {\n    if (ty < h) {\n#pragma unroll\n      for (int j = 0; j < VW; ++j) "
         "sm[ty][tx * VW + j] = comb<" << op << ">(sm[ty][tx * VW + j], sm[ty + h][tx * VW + j]);\n    }\n    __syncthreads();\n  }\n";
    s << "  if (ty == 0 && valid) {\n#pragma unroll\n    for (int j = 0; j < VW; ++j)\n      if (c + j < C) st1_f32(partial" << i
      << ", (i64)blockIdx.y * C + c + j, sm[0][tx * VW + j]);\n  }\n";
  }
  s << "}\n";
  *out = s.str();
  return true;
}

constexpr const char* kJitOptionsTag = "akgb-ew-jit-2 sm_100a c++17 fmad=false";

struct JitKernel {
  CUfunction fn = nullptr;
  bool failed = false;
  unsigned dyn_smem_allowed = 0;  // what cuFuncSetAttribute(MAX_DYNAMIC_SHARED_SIZE_BYTES) was last set to
};
std::mutex g_mu;
std::map<std::string, JitKernel> g_cache;  // device + source text -> kernel (per process; modules live until exit)
std::string g_cache_dir;                   // set by jit_set_cache_dir; empty = look at the environment
bool g_cache_dir_set = false;
uint64_t g_n_compiled = 0, g_n_from_disk = 0;

// Directory of the on-disk cubin cache: the explicit setting, else AKGB_JIT_CACHE_DIR, else KERNEL_META_DIR (where
// the reference keeps its compiled kernels, akg-mlir/python/akg_mlir/mlir_driver.py:47-53); empty = no disk cache.
std::string cache_dir() {
  if (g_cache_dir_set) return g_cache_dir;
  for (const char* name : {"AKGB_JIT_CACHE_DIR", "KERNEL_META_DIR"}) {
    const char* v = std::getenv(name);
    if (v && *v) return v;
  }
  return "";
}

bool read_file(const std::string& path, std::vector<char>* out) {
  FILE* f = std::fopen(path.c_str(), "rb");
  if (!f) return false;
  std::fseek(f, 0, SEEK_END);
  const long n = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  bool ok = n > 4;
  if (ok) {
    out->resize((size_t)n);
    ok = std::fread(out->data(), 1, (size_t)n, f) == (size_t)n;
  }
  std::fclose(f);
  // an ELF image, as NVRTC produced it; anything else (a torn or foreign file) is ignored
  return ok && (*out)[0] == 0x7f && (*out)[1] == 'E' && (*out)[2] == 'L' && (*out)[3] == 'F';
}

void write_file_atomically(const std::string& path, const std::vector<char>& data) {
  const std::string tmp = path + ".tmp." + std::to_string((long long)getpid());
  const int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0600);  // readable by its owner only
  if (fd < 0) return;
  FILE* f = ::fdopen(fd, "wb");
  if (!f) {
    ::close(fd);
    return;
  }
  const bool ok = std::fwrite(data.data(), 1, data.size(), f) == data.size();
  std::fclose(f);
  if (!ok || std::rename(tmp.c_str(), path.c_str()) != 0) std::remove(tmp.c_str());
}

// A cached image is launched on the device, so it is only accepted when (1) the file belongs to this user and
// (2) the digest recorded beside it (<file>.sha256, written together with the image) is the digest of its bytes: a
// truncated, stale or foreign file at the expected path is ignored and the kernel is compiled again.
bool owned_by_this_user(const std::string& path) {
  struct stat st;
  return ::stat(path.c_str(), &st) == 0 && st.st_uid == ::geteuid() && S_ISREG(st.st_mode);
}
bool read_verified_image(const std::string& path, std::vector<char>* image) {
  if (!owned_by_this_user(path) || !owned_by_this_user(path + ".sha256")) return false;
  std::vector<char> digest;
  {
    FILE* f = std::fopen((path + ".sha256").c_str(), "rb");
    if (!f) return false;
    digest.resize(64);
    const bool ok = std::fread(digest.data(), 1, 64, f) == 64;
    std::fclose(f);
    if (!ok) return false;
  }
  if (!read_file(path, image)) return false;
  return sha256_hex(image->data(), image->size()) == std::string(digest.data(), 64);
}
void write_image_with_digest(const std::string& path, const std::vector<char>& image) {
  const std::string hex = sha256_hex(image.data(), image.size());
  write_file_atomically(path + ".sha256", std::vector<char>(hex.begin(), hex.end()));
  write_file_atomically(path, image);
}

// the compile options and the version of the compiler that produced an image are part of its cache key
std::string jit_options_tag();

// source text -> cubin image for sm_100a (no device needed); empty on failure (the log goes to akgb_last_error)
std::vector<char> compile_to_cubin(const std::string& src) {
  std::vector<char> cubin;
  Nvrtc& n = nvrtc();
  if (!n.ok) return cubin;
  nvrtcProgram prog = nullptr;
  if (n.CreateProgram(&prog, src.c_str(), "akgb_ew_jit.cu", 0, nullptr, nullptr) != 0) return cubin;
  const char* opts[] = {"--gpu-architecture=sm_100a", "-std=c++17", "--fmad=false", "-default-device"};
  const nvrtcResult r = n.CompileProgram(prog, 4, opts);
  if (r != 0) {
    size_t ls = 0;
    if (n.GetProgramLogSize(prog, &ls) == 0 && ls > 1) {
      std::string log(ls, '\0');
      n.GetProgramLog(prog, &log[0]);
      set_last_error(("elementwise JIT: " + log.substr(0, 400)).c_str());
    }
    n.DestroyProgram(&prog);
    return cubin;
  }
  size_t sz = 0;
  if (n.GetCUBINSize(prog, &sz) == 0 && sz > 0) {
    cubin.resize(sz);
    if (n.GetCUBIN(prog, cubin.data()) != 0) cubin.clear();
  }
  n.DestroyProgram(&prog);
  return cubin;
}

JitKernel* compile(const std::string& src, const char* entry = "akgb_ew_jit") {
  std::lock_guard<std::mutex> lock(g_mu);
  int dev = 0;
  cudaGetDevice(&dev);
  const std::string key = std::to_string(dev) + ":" + src;  // a loaded function belongs to one device's context
  auto it = g_cache.find(key);
  if (it != g_cache.end()) return &it->second;
  JitKernel& k = g_cache[key];
  k.failed = true;
  Nvrtc& n = nvrtc();
  Driver& d = driver();
  if (!d.ok) return &k;
  // on-disk cache, keyed by the digest of the generated text and the compile options
  const std::string dir = cache_dir();
  std::string path;
  if (!dir.empty()) {
    const std::string tagged = jit_options_tag() + "\n" + src;
    path = dir + "/akgb_ew_" + sha256_hex(tagged.data(), tagged.size()) + ".sm_100a.cubin";
    std::vector<char> image;
    if (read_verified_image(path, &image)) {
      CUmodule mod = nullptr;
      if (d.ModuleLoadData(&mod, image.data()) == CUDA_SUCCESS &&
          d.ModuleGetFunction(&k.fn, mod, entry) == CUDA_SUCCESS) {
        k.failed = false;
        ++g_n_from_disk;
        return &k;
      }
    }
  }
  const std::vector<char> cubin = compile_to_cubin(src);
  if (cubin.empty()) return &k;
  CUmodule mod = nullptr;
  if (d.ModuleLoadData(&mod, cubin.data()) != CUDA_SUCCESS) return &k;
  if (d.ModuleGetFunction(&k.fn, mod, entry) != CUDA_SUCCESS) return &k;
  k.failed = false;
  ++g_n_compiled;
  if (!path.empty()) write_image_with_digest(path, cubin);
  return &k;
}

std::string jit_options_tag() {
  int major = 0, minor = 0;
  Nvrtc& n = nvrtc();
  if (n.ok && n.Version) n.Version(&major, &minor);
  return std::string(kJitOptionsTag) + " nvrtc " + std::to_string(major) + "." + std::to_string(minor);
}

// The generated text with its entry point renamed to `entry` and the trailing element / row count turned into a
// constant, so that the kernel takes the tensors' bare pointers and nothing else -- the signature a runtime that loads
// <kernel>.cubin + <kernel>.json from the kernel meta directory launches.
std::string standalone_source(std::string src, const char* generated_entry, const std::string& entry,
                              const char* count_name, long long count) {
  const std::string from = std::string(generated_entry) + "(";
  const size_t at = src.find(from);
  if (at == std::string::npos) return "";
  src.replace(at, from.size(), entry + "(");
  const std::string tail = std::string(", i64 ") + count_name + ") {\n";
  const size_t tp = src.find(tail, at);
  if (tp == std::string::npos) return "";
  // the last pointer parameter ends in ", " before the count: drop the count, keep the pointers
  src.replace(tp, tail.size(), std::string(") {\n  constexpr i64 ") + count_name + " = " + std::to_string(count) + "LL;\n");
  return src;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// The address ranges the launches of the calling thread are checked against (null: ordinary kernels).
thread_local const CheckedRanges* t_checked = nullptr;

// The checked form of a generated source: the checker compiled in, the table as last kernel argument, stored by every
// block before its first access.
std::string checked_source(const std::string& src, const char* entry) {
  const size_t at = src.find(std::string(entry) + "(");
  if (at == std::string::npos) return "";
  const size_t close = src.find(") {\n", at);
  if (close == std::string::npos) return "";
  std::string out = "#define AKGB_CHECKED 1\n" + src.substr(0, close) + ", AkgbRanges akgb_rng_arg" +
                    ") {\n  if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) akgb_rng = akgb_rng_arg;\n  __syncthreads();\n" +
                    src.substr(close + 4);
  return out;
}

}  // namespace

void jit_set_checked_ranges(const CheckedRanges* r) { t_checked = r; }

void jit_set_cache_dir(const char* dir) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_cache_dir = dir ? dir : "";
  g_cache_dir_set = dir != nullptr;
}

void jit_cache_stats(uint64_t* compiled, uint64_t* from_disk) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (compiled) *compiled = g_n_compiled;
  if (from_disk) *from_disk = g_n_from_disk;
}

// Column program: partial[splits, cols] (or the result itself when splits == 1); the caller folds the partials.
int64_t col_jit_splits(const RowProgram& P, int sm_count) {
  const int vw = P.cols % 8 == 0 ? 8 : 1;
  const int64_t granules = (P.cols + vw - 1) / vw;
  int tx = 1;
  while (tx < 32 && tx < granules) tx <<= 1;
  const int ty = 256 / tx;
  const int64_t col_ctas = (granules + tx - 1) / tx;
  const int64_t want = ((int64_t)sm_count * 8 + col_ctas - 1) / col_ctas;
  const int64_t max_splits = std::max<int64_t>(1, P.rows / ((int64_t)ty * 4));
  return std::max<int64_t>(1, std::min<int64_t>(std::min(want, max_splits), 1024));
}

cudaError_t col_jit_launch(const RowProgram& P, const void* const* in, float* const* partials, int64_t splits,
                           cudaStream_t s, LaunchDims* dims) {
  if (P.rows == 0 || P.cols == 0) return cudaSuccess;
  bool vec = P.cols % 8 == 0;
  for (size_t i = 0; i < P.in.size() && vec; ++i)
    if (P.in[i].kind != RK_ROW && P.in[i].kind != RK_SCALAR) vec = aligned16(in[i]);
  std::string src;
  ColShape cs;
  if (!col_generate(P, vec, &src, &cs)) return cudaErrorNotSupported;
  const CheckedRanges* ck = t_checked;
  if (ck && (src = checked_source(src, "akgb_col_jit")).empty()) return cudaErrorNotSupported;
  JitKernel* k = compile(src, "akgb_col_jit");
  if (!k || k->failed) return cudaErrorNotSupported;
  const int64_t granules = (P.cols + cs.vw - 1) / cs.vw;
  const int64_t gx = (granules + cs.tx - 1) / cs.tx;
  if (gx > 0x7fffffff || splits > 65535) return cudaErrorNotSupported;
  long long rows = P.rows, rps = (P.rows + splits - 1) / splits;
  void* args[32];
  const void* inp[16];
  int a = 0;
  for (size_t i = 0; i < P.in.size(); ++i) {
    inp[i] = in[i];
    args[a++] = &inp[i];
  }
  float* parts[4];
  for (size_t i = 0; i < P.out.size(); ++i) {
    parts[i] = partials[i];
    args[a++] = &parts[i];
  }
  args[a++] = &rows;
  args[a++] = &rps;
  CheckedRanges ckv;
  if (ck) {
    ckv = *ck;
    args[a++] = &ckv;
  }
  if (dims) {
    dims->grid[0] = (unsigned)gx;
    dims->grid[1] = (unsigned)splits;
    dims->block[0] = 256;
  }
  const CUresult r = driver().LaunchKernel(k->fn, (unsigned)gx, (unsigned)splits, 1, 256, 1, 1, 0, (CUstream)s, args, nullptr);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorLaunchFailure;
}

bool row_jit_fits_registers(const RowProgram& P) {
  RowShape rs;
  return row_shape(P, true, &rs) && row_shape(P, false, &rs);
}

// The same for both access widths, so that the planner can size the partial vectors: about 1024 threads per SM of a
// 148-SM part with the CTA size of the 16-byte variant (measured on LayerNorm backward: 2 CTAs of 512 threads per SM
// for 4096 columns, 8 of 128 for 1024 columns), never more than there are rows (a CTA without rows writes zeros).
int64_t row_jit_col_sum_ctas(const RowProgram& P) {
  RowShape rs;
  const int tpb = row_shape(P, true, &rs) ? rs.tpb : 512;
  return std::min<int64_t>(148 * std::max(1, 1024 / tpb), std::max<int64_t>(1, P.rows));
}

std::string row_jit_source(const RowProgram& P, bool vec) {
  std::string src;
  if (P.col_reduce) {
    ColShape cs;
    if (!col_generate(P, vec, &src, &cs)) src.clear();
    return src;
  }
  RowShape rs;
  if (!row_generate(P, vec, &src, &rs)) src.clear();
  return src;
}

// One generated kernel for a whole reduce-X region; cudaErrorNotSupported when it cannot be generated or compiled (the
// caller then runs the region as separate launches).
cudaError_t row_jit_launch(const RowProgram& P, const void* const* in, void* const* out, cudaStream_t s, LaunchDims* dims) {
  if (P.rows == 0) return cudaSuccess;
  bool vec = P.cols % 8 == 0;
  for (size_t i = 0; i < P.in.size() && vec; ++i)
    if (P.in[i].kind != RK_ROW && P.in[i].kind != RK_SCALAR) vec = aligned16(in[i]);
  for (size_t i = 0; i < P.out.size() && vec; ++i)
    if (P.out[i].kind == RK_FULL) vec = aligned16(out[i]);
  std::string src;
  RowShape rs;
  if (!row_generate(P, vec, &src, &rs)) return cudaErrorNotSupported;
  const CheckedRanges* ck = t_checked;
  if (ck && (src = checked_source(src, "akgb_row_jit")).empty()) return cudaErrorNotSupported;
  JitKernel* k = compile(src, "akgb_row_jit");
  if (!k || k->failed) return cudaErrorNotSupported;
  const int rpb = rs.tpb / rs.t;  // 1 for the multi-pass schedule
  const int64_t grid = P.col_sums ? row_jit_col_sum_ctas(P) : ((P.rows + rpb - 1) / rpb) * rs.cluster;
  if (grid > 0x7fffffff) return cudaErrorNotSupported;
  if (rs.dyn_smem > 32 * 1024 && k->dyn_smem_allowed < rs.dyn_smem) {  // static + dynamic above the 48 KB default
    if (driver().FuncSetAttribute(k->fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)rs.dyn_smem) != CUDA_SUCCESS)
      return cudaErrorNotSupported;
    k->dyn_smem_allowed = rs.dyn_smem;
  }
  long long rows = P.rows;
  void* args[32];
  const void* inp[16];
  void* outp[16];
  int a = 0;
  for (size_t i = 0; i < P.in.size(); ++i) {
    inp[i] = in[i];
    args[a++] = &inp[i];
  }
  for (size_t i = 0; i < P.out.size(); ++i) {
    outp[i] = out[i];
    args[a++] = &outp[i];
  }
  args[a++] = &rows;
  CheckedRanges ckv;
  if (ck) {
    ckv = *ck;
    args[a++] = &ckv;
  }
  if (dims) {
    dims->grid[0] = (unsigned)grid;
    dims->block[0] = (unsigned)rs.tpb;
    dims->smem = rs.dyn_smem;
  }
  const CUresult r = driver().LaunchKernel(k->fn, (unsigned)grid, 1, 1, (unsigned)rs.tpb, 1, 1, rs.dyn_smem, (CUstream)s, args, nullptr);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorLaunchFailure;
}

// Compiles (or loads from the disk cache) the variant a launch on 16-byte aligned tensors will use, so that the first
// launch does no compilation and no module load -- both are illegal while a stream is being captured into a graph.
void ew_jit_prepare(const EwProgram& P) {
  std::string src;
  if (P.n > 0 && generate(P, P.n % 8 == 0, &src)) compile(src);
}
void row_jit_prepare(const RowProgram& P) {
  std::string src;
  const bool vec = P.cols % 8 == 0;
  if (P.col_reduce) {
    ColShape cs;
    if (col_generate(P, vec, &src, &cs)) compile(src, "akgb_col_jit");
  } else {
    RowShape rs;
    if (row_generate(P, vec, &src, &rs)) compile(src, "akgb_row_jit");
  }
}

// Stand-alone binaries of generated kernels (the reference leaves <kernel>.ptx + <kernel>.json for the framework's
// runtime, akg-mlir/python/akg_mlir/mlir_driver.py:776-815): the image of the kernel with entry point `entry` taking
// only the tensors' pointers (inputs then outputs), and the launch dimensions.  The 16-byte-vector variant is exported
// when the extents allow it; it then requires 16-byte aligned tensors, which `*needs_align16` reports.
bool ew_jit_export(const EwProgram& P, const std::string& entry, std::vector<char>* cubin, LaunchDims* dims,
                   bool* needs_align16) {
  if (P.n <= 0) return false;
  const bool vec = P.n % 8 == 0;
  std::string src;
  if (!generate(P, vec, &src)) return false;
  src = standalone_source(src, "akgb_ew_jit", entry, "n", (long long)P.n);
  if (src.empty()) return false;
  *cubin = compile_to_cubin(src);
  if (cubin->empty()) return false;
  const int U = ew_shape(P, vec).U, E = vec ? 8 : 1;
  const int64_t nv = P.n / E;
  const int64_t grid = (nv + 256 * U - 1) / (256 * U);
  if (grid > 0x7fffffff) return false;
  *dims = LaunchDims();
  dims->grid[0] = (unsigned)grid;
  dims->block[0] = 256;
  *needs_align16 = vec;
  return true;
}
bool row_jit_export(const RowProgram& P, const std::string& entry, std::vector<char>* cubin, LaunchDims* dims,
                    bool* needs_align16) {
  if (P.rows <= 0 || P.col_reduce || P.col_sums) return false;  // those write partials another launch folds
  const bool vec = P.cols % 8 == 0;
  std::string src;
  RowShape rs;
  if (!row_generate(P, vec, &src, &rs)) return false;
  src = standalone_source(src, "akgb_row_jit", entry, "rows", (long long)P.rows);
  if (src.empty()) return false;
  *cubin = compile_to_cubin(src);
  if (cubin->empty()) return false;
  const int rpb = rs.tpb / rs.t;
  const int64_t grid = ((P.rows + rpb - 1) / rpb) * rs.cluster;
  if (grid > 0x7fffffff) return false;
  *dims = LaunchDims();
  dims->grid[0] = (unsigned)grid;
  dims->block[0] = (unsigned)rs.tpb;
  dims->smem = rs.dyn_smem;  // above 48 KB the loader must raise the function's dynamic shared memory limit first
  *needs_align16 = vec;
  return true;
}

bool ew_program_needs_jit(const EwProgram& P) { return ew_has_i64(P) || ew_has_f64(P); }

// The CUDA C++ text that would be compiled for this program (empty when the program needs the interpreter).
std::string ew_jit_source(const EwProgram& P, bool vec) {
  std::string src;
  if (!generate(P, vec, &src)) src.clear();
  return src;
}

// Tries the run-time instantiated kernel; returns cudaErrorNotSupported when the caller should interpret.
cudaError_t ew_jit_launch(const EwProgram& P, const void* const* in, void* const* out, cudaStream_t s, LaunchDims* dims) {
  if (P.n == 0) return cudaSuccess;
  bool vec = P.n % 8 == 0;
  for (int i = 0; i < P.n_in && vec; ++i) vec = aligned16(in[i]);
  for (int i = 0; i < P.n_out && vec; ++i) vec = aligned16(out[i]);
  std::string src;
  if (!generate(P, vec, &src)) return cudaErrorNotSupported;
  const CheckedRanges* ck = t_checked;
  if (ck && (src = checked_source(src, "akgb_ew_jit")).empty()) return cudaErrorNotSupported;
  JitKernel* k = compile(src);
  if (!k || k->failed) return cudaErrorNotSupported;
  const int U = ew_shape(P, vec).U, E = vec ? 8 : 1;
  const int64_t nv = P.n / E;
  const int64_t grid = (nv + 256 * U - 1) / (256 * U);
  if (grid > 0x7fffffff) return cudaErrorNotSupported;
  long long n = P.n;
  void* args[kEwMaxIn + kEwMaxOut + 2];
  const void* inp[kEwMaxIn];
  void* outp[kEwMaxOut];
  int a = 0;
  for (int i = 0; i < P.n_in; ++i) {
    inp[i] = in[i];
    args[a++] = &inp[i];
  }
  for (int i = 0; i < P.n_out; ++i) {
    outp[i] = out[i];
    args[a++] = &outp[i];
  }
  args[a++] = &n;
  CheckedRanges ckv;
  if (ck) {
    ckv = *ck;
    args[a++] = &ckv;
  }
  if (dims) {
    dims->grid[0] = (unsigned)grid;
    dims->block[0] = 256;
    dims->smem = 0;
  }
  const CUresult r = driver().LaunchKernel(k->fn, (unsigned)grid, 1, 1, 256, 1, 1, 0, (CUstream)s, args, nullptr);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorLaunchFailure;
}

}  // namespace akgb
