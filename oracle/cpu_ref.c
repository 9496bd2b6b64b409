/*
 * CPU restatement of AKG-MLIR's CPU pipeline for the benchmarked fused ops —
 * TEST INFRASTRUCTURE and timed CPU baseline, never a product path.  Only
 * tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs load it.
 *
 * What it follows (paths inside akg-mlir/):
 *   - loop structure: one fused scalar loop nest per linalg group, as
 *     `--cpu-opt` without cpu-fast produces (lib/Pipelines/CPUOpt.cpp:185-209);
 *     the *_rp variants add an OpenMP parallel-for on the outer loop, the
 *     analogue of cpu-fast / AKGLoopParallelize (CPUOpt.cpp:142, :193-198);
 *   - per-op arithmetic in the op's element type
 *     (lib/Conversion/MindSporeToLinalg/MindSporeToLinalg.cpp:377-483);
 *   - reductions: init + sequential combine in the result type
 *     (MindSporeToLinalg.cpp:791-901, :1401-1426); max starts at -FLT_MAX and
 *     skips NaN (fmaxf);
 *   - float16 transcendentals extend to float, call libm, truncate
 *     (MathToLibm in CPUOpt.cpp:162);
 *   - matmul: zero-filled f32 result, k innermost (MindSporeToLinalg.cpp:1501-1533).
 *
 * The reference's ABI is `void kernel(void** tensors)` with static shapes
 * compiled in (lib/Dialect/LLVMIR/Transforms/LLVMParameterPacking.cpp:57-89);
 * here the extents arrive in a second argument so one build serves all sizes.
 *
 * Build: -O3 -ffp-contract=off (no fused multiply-add: every op rounds).
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

typedef _Float16 f16;

static inline float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
/* arith.truncf f32 -> bf16: round to nearest even */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

int akg_ref_num_threads(void) {
#ifdef _OPENMP
  extern int omp_get_max_threads(void);
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Thread count of the parallel variants; a launcher may have exported OMP_NUM_THREADS=1 for its workers, which the
 * timed baseline must not inherit.  Returns the count now in effect. */
int akg_ref_set_num_threads(int n) {
#ifdef _OPENMP
  extern void omp_set_num_threads(int);
  if (n > 0) omp_set_num_threads(n);
#endif
  return akg_ref_num_threads();
}

/* ---- LayerNorm: tensors = {x, gamma, beta, y, mean, var}; dims = {rows, cols}; scal = {1/N, eps} */
static void layernorm_row(const float* x, const float* g, const float* b, float* y, float* mean, float* var, int64_t r,
                          int64_t cols, float inv_n, float eps) {
  const float* xr = x + r * cols;
  float s = 0.0f;
  for (int64_t c = 0; c < cols; ++c) s = s + xr[c];
  const float m = s * inv_n;
  float q = 0.0f;
  for (int64_t c = 0; c < cols; ++c) {
    const float d = xr[c] - m;
    q = q + d * d;
  }
  const float v = q * inv_n;
  const float rstd = 1.0f / sqrtf(v + eps);
  for (int64_t c = 0; c < cols; ++c) {
    const float d = xr[c] - m;
    float o = d * rstd;
    o = o * g[c];
    o = o + b[c];
    y[r * cols + c] = o;
  }
  if (mean) mean[r] = m;
  if (var) var[r] = v;
}
void akg_ref_layernorm_f32_r1(void** t, const int64_t* dims, const double* scal) {
  for (int64_t r = 0; r < dims[0]; ++r)
    layernorm_row(t[0], t[1], t[2], t[3], t[4], t[5], r, dims[1], (float)scal[0], (float)scal[1]);
}
void akg_ref_layernorm_f32_rp(void** t, const int64_t* dims, const double* scal) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < dims[0]; ++r)
    layernorm_row(t[0], t[1], t[2], t[3], t[4], t[5], r, dims[1], (float)scal[0], (float)scal[1]);
}

/* ---- f16 bias + tanh-GELU * y -> f32: tensors = {x, bias, y, out}; dims = {n, inner}; scal = {c0, c1, c2, one} */
static inline float gelu_elem(f16 x, f16 bias, f16 y, f16 c0, f16 c1, f16 c2, f16 one) {
  const f16 t = (f16)((float)x + (float)bias);
  const f16 a = (f16)((float)t * (float)t);
  const f16 t3 = (f16)((float)a * (float)t);
  const f16 b = (f16)((float)t3 * (float)c0);
  const f16 c = (f16)((float)t + (float)b);
  const f16 d = (f16)((float)c * (float)c1);
  const f16 e = (f16)tanhf((float)d);
  const f16 f = (f16)((float)e + (float)one);
  const f16 g = (f16)((float)t * (float)c2);
  const f16 h = (f16)((float)g * (float)f);
  const f16 k = (f16)((float)h * (float)y);
  return (float)k;
}
void akg_ref_gelu_chain_f16_r1(void** t, const int64_t* dims, const double* scal) {
  const f16 *x = t[0], *bias = t[1], *y = t[2];
  float* out = t[3];
  const f16 c0 = (f16)scal[0], c1 = (f16)scal[1], c2 = (f16)scal[2], one = (f16)scal[3];
  for (int64_t i = 0; i < dims[0]; ++i) out[i] = gelu_elem(x[i], bias[i % dims[1]], y[i], c0, c1, c2, one);
}
void akg_ref_gelu_chain_f16_rp(void** t, const int64_t* dims, const double* scal) {
  const f16 *x = t[0], *bias = t[1], *y = t[2];
  float* out = t[3];
  const f16 c0 = (f16)scal[0], c1 = (f16)scal[1], c2 = (f16)scal[2], one = (f16)scal[3];
  const int64_t inner = dims[1], rows = dims[0] / inner;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < inner; ++c) out[r * inner + c] = gelu_elem(x[r * inner + c], bias[c], y[r * inner + c], c0, c1, c2, one);
}

/* ---- masked softmax f16: tensors = {scores, mask, out}; dims = {rows, cols, mask_rows}; scal = {scale} */
static void softmax_row(const f16* x, const f16* mask, f16* out, float* tmp, int64_t r, int64_t cols, int64_t mask_rows,
                        float scale) {
  const f16* xr = x + r * cols;
  const f16* mr = mask + (r % mask_rows) * cols;
  float mx = -FLT_MAX;
  for (int64_t c = 0; c < cols; ++c) {
    float s = (float)xr[c] * scale;
    s = s + (float)mr[c];
    tmp[c] = s;
    mx = fmaxf(mx, s);
  }
  float sum = 0.0f;
  for (int64_t c = 0; c < cols; ++c) {
    const float e = expf(tmp[c] - mx);
    tmp[c] = e;
    sum = sum + e;
  }
  for (int64_t c = 0; c < cols; ++c) out[r * cols + c] = (f16)(tmp[c] / sum);
}
void akg_ref_softmax_f16_r1(void** t, const int64_t* dims, const double* scal) {
  float tmp[dims[1]];
  for (int64_t r = 0; r < dims[0]; ++r) softmax_row(t[0], t[1], t[2], tmp, r, dims[1], dims[2], (float)scal[0]);
}
void akg_ref_softmax_f16_rp(void** t, const int64_t* dims, const double* scal) {
#pragma omp parallel
  {
    float tmp[dims[1]];
#pragma omp for schedule(static)
    for (int64_t r = 0; r < dims[0]; ++r) softmax_row(t[0], t[1], t[2], tmp, r, dims[1], dims[2], (float)scal[0]);
  }
}

/* ---- column sum: tensors = {x, out}; dims = {rows, cols} */
void akg_ref_reduce_sum_axis0_f32_r1(void** t, const int64_t* dims, const double* scal) {
  (void)scal;
  const float* x = t[0];
  float* out = t[1];
  for (int64_t c = 0; c < dims[1]; ++c) out[c] = 0.0f;
  for (int64_t r = 0; r < dims[0]; ++r)
    for (int64_t c = 0; c < dims[1]; ++c) out[c] = out[c] + x[r * dims[1] + c];
}
void akg_ref_reduce_sum_axis0_f32_rp(void** t, const int64_t* dims, const double* scal) {
  (void)scal;
  const float* x = t[0];
  float* out = t[1];
  const int64_t rows = dims[0], cols = dims[1];
  /* parallel over the non-reduced axis in blocks of 64 columns; each column still sums sequentially */
#pragma omp parallel for schedule(static)
  for (int64_t c0 = 0; c0 < cols; c0 += 64) {
    const int64_t c1 = c0 + 64 < cols ? c0 + 64 : cols;
    for (int64_t c = c0; c < c1; ++c) out[c] = 0.0f;
    for (int64_t r = 0; r < rows; ++r)
      for (int64_t c = c0; c < c1; ++c) out[c] = out[c] + x[r * cols + c];
  }
}

/* ---- global max: tensors = {x, out}; dims = {n} */
void akg_ref_reduce_max_all_f32_r1(void** t, const int64_t* dims, const double* scal) {
  (void)scal;
  const float* x = t[0];
  float m = -FLT_MAX;
  for (int64_t i = 0; i < dims[0]; ++i) m = fmaxf(m, x[i]);
  ((float*)t[1])[0] = m;
}
void akg_ref_reduce_max_all_f32_rp(void** t, const int64_t* dims, const double* scal) {
  (void)scal;
  const float* x = t[0];
  float m = -FLT_MAX;
#pragma omp parallel for reduction(max : m) schedule(static)
  for (int64_t i = 0; i < dims[0]; ++i) m = fmaxf(m, x[i]);
  ((float*)t[1])[0] = m;
}

/* ---- matmul + bias + ReLU -> bf16: tensors = {A, B, bias, out}; dims = {M, K, N} */
static void matmul_row(const uint16_t* A, const uint16_t* B, const uint16_t* bias, uint16_t* out, float* acc, int64_t m,
                       int64_t K, int64_t N) {
  for (int64_t n = 0; n < N; ++n) acc[n] = 0.0f;
  for (int64_t k = 0; k < K; ++k) {
    const float a = bf16_to_f32(A[m * K + k]);
    const uint16_t* br = B + k * N;
    for (int64_t n = 0; n < N; ++n) acc[n] = acc[n] + a * bf16_to_f32(br[n]);
  }
  for (int64_t n = 0; n < N; ++n) {
    float v = acc[n] + bf16_to_f32(bias[n]);
    v = fmaxf(v, 0.0f);
    out[m * N + n] = f32_to_bf16(v);
  }
}
void akg_ref_matmul_bias_relu_bf16_r1(void** t, const int64_t* dims, const double* scal) {
  (void)scal;
  float acc[dims[2]];
  for (int64_t m = 0; m < dims[0]; ++m) matmul_row(t[0], t[1], t[2], t[3], acc, m, dims[1], dims[2]);
}
void akg_ref_matmul_bias_relu_bf16_rp(void** t, const int64_t* dims, const double* scal) {
  (void)scal;
#pragma omp parallel
  {
    float acc[dims[2]];
#pragma omp for schedule(static)
    for (int64_t m = 0; m < dims[0]; ++m) matmul_row(t[0], t[1], t[2], t[3], acc, m, dims[1], dims[2]);
  }
}

/* ---- transpose of 2-byte elements, rank 4: tensors = {x, out}; dims = {d0,d1,d2,d3, p0,p1,p2,p3} */
static void transpose4_outer(const uint16_t* x, uint16_t* out, const int64_t* d, const int64_t* p, int64_t i0) {
  int64_t xs[4] = {d[1] * d[2] * d[3], d[2] * d[3], d[3], 1};
  int64_t od[4] = {d[p[0]], d[p[1]], d[p[2]], d[p[3]]};
  for (int64_t i1 = 0; i1 < od[1]; ++i1)
    for (int64_t i2 = 0; i2 < od[2]; ++i2)
      for (int64_t i3 = 0; i3 < od[3]; ++i3)
        out[((i0 * od[1] + i1) * od[2] + i2) * od[3] + i3] = x[i0 * xs[p[0]] + i1 * xs[p[1]] + i2 * xs[p[2]] + i3 * xs[p[3]]];
}
void akg_ref_transpose4_b2_r1(void** t, const int64_t* dims, const double* scal) {
  (void)scal;
  for (int64_t i0 = 0; i0 < dims[dims[4]]; ++i0) transpose4_outer(t[0], t[1], dims, dims + 4, i0);
}
void akg_ref_transpose4_b2_rp(void** t, const int64_t* dims, const double* scal) {
  (void)scal;
#pragma omp parallel for schedule(static)
  for (int64_t i0 = 0; i0 < dims[dims[4]]; ++i0) transpose4_outer(t[0], t[1], dims, dims + 4, i0);
}
