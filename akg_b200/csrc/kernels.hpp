// Host-callable launchers of the sm_100a kernel templates.  Each returns the
// cudaError_t of its launch; none allocates or synchronises.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

namespace akgb {

// Records the text akgb_last_error() returns on the calling thread (defined beside the C ABI).
void set_last_error(const char* text);

struct LaunchDims {
  unsigned grid[3] = {1, 1, 1};
  unsigned block[3] = {1, 1, 1};
  unsigned smem = 0;
};

enum class RedOp : int { Sum = 0, Max = 1, Min = 2, Prod = 3 };

// ---- elementwise: (x [+ bias]) -> tanh-GELU [* y] -> cast ---------------------
// Per-op rounding in the chain's element type is replayed:
//   t=x+bias; a=t*t; t3=a*t; b=t3*c0; c=t+b; d=c*c1; e=tanh(d); f=e+1; g=t*c2; h=g*f; k=h*y
struct GeluChainParams {
  int64_t n = 0;         // elements
  int64_t inner = 0;     // bias length (bias index = element index % inner); 0 = no bias
  int has_mul = 0;       // multiply by y
  int out_f32 = 0;       // final Cast to float32 (else output stays float16)
  float c0 = 0.044715f, c1 = 0.7978845608f, c2 = 0.5f, c_one = 1.0f;  // already rounded to f16
};
cudaError_t gelu_chain_f16(const GeluChainParams& p, const void* x, const void* bias, const void* y, void* out,
                           const void* tanh_lut, uint32_t* err_word, cudaStream_t s, LaunchDims* dims);
// 16-bit table of correctly rounded tanh over the f16 magnitudes the kernel
// looks up; built on the host, `out` needs gelu_lut_entries() uint16 slots.
int gelu_lut_entries();
void gelu_lut_build(uint16_t* out);

// ---- row-wise fused patterns ---------------------------------------------------
struct LayerNormParams {
  int64_t rows = 0, cols = 0;
  float inv_n = 0.f, eps = 0.f;
  float div_n = 0.f;  // non-zero: the description divides the sums by this count instead of multiplying by inv_n
  int has_gamma = 0, has_beta = 0, write_mean = 0, write_var = 0;
};
cudaError_t layernorm_f32(const LayerNormParams& p, const float* x, const float* gamma, const float* beta, float* y,
                          float* mean, float* var, uint32_t* err_word, cudaStream_t s, LaunchDims* dims);

struct SoftmaxParams {
  int64_t rows = 0, cols = 0;
  int in_dt = 0, out_dt = 0, mask_dt = 0;  // DT codes: F16/F32/BF16
  int has_scale = 0, has_mask = 0;
  float scale = 1.f;
  int64_t mask_rows = 1;  // mask row = row % mask_rows
};
cudaError_t softmax_rows(const SoftmaxParams& p, const void* x, const void* mask, void* out, uint32_t* err_word,
                         cudaStream_t s, LaunchDims* dims);

// ---- reductions ----------------------------------------------------------------
// A reduction whose per-CTA partials are folded by the CTA that finishes last ("finisher": one per column tile, one for
// a reduction of all elements) needs no second launch.  The finishers are found with arrival counters (`tickets`,
// kReduceTicketWords zero-initialised words that every launch leaves at zero again; launches that share them must be
// ordered on the device).  Without `tickets` the fold is a second, small launch with one CTA per finisher.  With an
// exchange attached, each finisher (in either form) also completes the all-reduce of its values over the ranks' mapped
// exchange buffers (layout below): every value goes to every rank as one 64-bit word tagged with the call number, the
// finisher polls (bounded) the words of the other ranks and folds them in rank order, then writes the final result.
constexpr int kReduceMaxTicketTiles = 4096;
constexpr int kReduceTicketWords = kReduceMaxTicketTiles + 8;
struct FinishExchange {
  void* peer[8] = {};           // every rank's exchange buffer as mapped here; peer[rank] is this rank's own
  int rank = 0, world = 1;      // world == 1: no exchange
  long long limit_cycles = 0;   // bound of the wait for the peers' flags
  uint32_t* err = nullptr;      // device error word (bit 8: the wait ran out)
  int slot_off = 0;             // slot position of the first output's first element
  int slot_off2 = 0;            // slot position of the second output (column + all-elements kernel)
  int finishers = 0;            // finishers of the launch: the last one closes the call
};
// x[outer, red, inner] -> out[outer, inner]; f32 only.  With `tickets` the fold of the row splits happens in the same
// launch (see above) when reduce_col_fusable(); `fx` adds the exchange to the fold, wherever it happens.
size_t reduce_col_workspace(int64_t red, int64_t inner, int sm_count);
bool reduce_col_fusable(int64_t red, int64_t inner, int sm_count);
int reduce_col_launches(int64_t red, int64_t inner, int sm_count, bool tickets);
cudaError_t reduce_col_f32(RedOp op, const float* x, float* out, int64_t red, int64_t inner, void* ws, int sm_count,
                           cudaStream_t s, LaunchDims* dims, uint32_t* tickets = nullptr,
                           const FinishExchange* fx = nullptr);
// one pass over x: column reduction with op1 into out1[inner] and reduction of all elements with op2 into out2[1]
// (inner % 4 == 0, x 16-byte aligned)
bool reduce_col_dual_supported(int64_t inner, const void* x);
size_t reduce_col_dual_workspace(int64_t red, int64_t inner, int sm_count);
cudaError_t reduce_col_dual_f32(RedOp op1, RedOp op2, const float* x, float* out1, float* out2, int64_t red,
                                int64_t inner, void* ws, int sm_count, cudaStream_t s, LaunchDims* dims,
                                uint32_t* tickets = nullptr, const FinishExchange* fx = nullptr);
size_t reduce_all_workspace(int sm_count);
cudaError_t reduce_all_f32(RedOp op, const float* x, float* out, int64_t n, void* ws, int sm_count, cudaStream_t s,
                           LaunchDims* dims, uint32_t* tickets = nullptr, const FinishExchange* fx = nullptr);
cudaError_t reduce_row_f32(RedOp op, const float* x, float* out, int64_t rows, int64_t cols, cudaStream_t s,
                           LaunchDims* dims);

// ---- generic elementwise/broadcast interpreter (program in ew_program.hpp) ----------
struct EwProgram;
size_t ew_generic_smem(const EwProgram& p);
cudaError_t ew_generic(const EwProgram& p, const void* const* in, void* const* out, bool allow_jit, cudaStream_t s,
                       LaunchDims* dims);
// run-time instantiated variant (ew_jit.cpp); cudaErrorNotSupported = fall back to the interpreter
std::string ew_jit_source(const EwProgram& p, bool vec);
struct RowProgram;
cudaError_t row_jit_launch(const RowProgram& p, const void* const* in, void* const* out, cudaStream_t s,
                           LaunchDims* dims);
std::string row_jit_source(const RowProgram& p, bool vec);
int64_t col_jit_splits(const RowProgram& p, int sm_count);
bool row_jit_fits_registers(const RowProgram& p);  // the register schedule applies (in both access widths)
int64_t row_jit_col_sum_ctas(const RowProgram& p);  // CTAs (= partial vectors per result) of a program with column sums
cudaError_t col_jit_launch(const RowProgram& p, const void* const* in, float* const* partials, int64_t splits,
                           cudaStream_t s, LaunchDims* dims);
}  // namespace akgb
#include <vector>
namespace akgb {
// stand-alone image of a generated kernel whose entry point `entry` takes only the tensors' pointers (ew_jit.cpp)
bool ew_jit_export(const EwProgram& p, const std::string& entry, std::vector<char>* cubin, LaunchDims* dims,
                   bool* needs_align16);
bool row_jit_export(const RowProgram& p, const std::string& entry, std::vector<char>* cubin, LaunchDims* dims,
                    bool* needs_align16);
// Checked launches of generated kernels (AKGB_FLAG_CHECKED): the address ranges of the launch's tensors and workspace.
// While a table is set for the calling thread, generated kernels are built with every global access tested against it
// (outside all ranges: bit 9 of the error word, the access skipped).  Layout shared with the generated source.
struct CheckedRanges {
  unsigned long long lo[32], hi[32];
  int n = 0;
  uint32_t* err = nullptr;
};
void jit_set_checked_ranges(const CheckedRanges* r);
// programs the interpreting kernel cannot run (64-bit integer or float64 values): they need the run-time compiler
bool ew_program_needs_jit(const EwProgram& p);
void ew_jit_prepare(const EwProgram& p);
void row_jit_prepare(const RowProgram& p);
void jit_set_cache_dir(const char* dir);  // nullptr: environment's choice; "": no disk cache
void jit_cache_stats(uint64_t* compiled, uint64_t* from_disk);
cudaError_t ew_jit_launch(const EwProgram& p, const void* const* in, void* const* out, cudaStream_t s, LaunchDims* dims);

// ---- exchange over peer memory -----------------------------------------------------------------
// Layout of one rank's exchange buffer: [2 parities][kExchangeMaxRanks slots][kExchangeSlotElems floats], then the flags
// [2][kExchangeMaxRanks][kExchangeMaxFlags] uint32 (the exchange kernel raises one flag per CTA).
constexpr int kExchangeMaxRanks = 8, kExchangeSlotElems = 16384, kExchangeMaxCtas = 16, kExchangeMaxFlags = 16;
constexpr size_t kExchangeDataBytes = (size_t)2 * kExchangeMaxRanks * kExchangeSlotElems * sizeof(float);
constexpr size_t kExchangeFlagBytes = (size_t)2 * kExchangeMaxRanks * kExchangeMaxFlags * sizeof(uint32_t);
// after the flags: the call counter (epoch) and the ticket that lets the last CTA of a call advance it; then, 256-byte
// aligned, the region of the exchanges that reductions complete themselves: [2 parities][kExchangeMaxRanks]
// [kExchangeTaggedElems] 64-bit words, each a float32 value with the call number it belongs to in the upper half.  Value
// and tag travel in ONE 8-byte store, so a receiver that sees the tag has the value: no flag, no fence, one NVLink
// crossing on the critical path.
constexpr int kExchangeTaggedElems = 8192;
constexpr size_t kExchangeTaggedOffset = (kExchangeDataBytes + kExchangeFlagBytes + 2 * sizeof(uint32_t) + 255) / 256 * 256;
constexpr size_t kExchangeTaggedBytes = (size_t)2 * kExchangeMaxRanks * kExchangeTaggedElems * sizeof(unsigned long long);
constexpr size_t kExchangeBytes = kExchangeTaggedOffset + kExchangeTaggedBytes;
__host__ __device__ inline unsigned long long* exchange_tagged(void* base, int parity, int rank) {
  return reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(base) + kExchangeTaggedOffset) +
         ((size_t)parity * kExchangeMaxRanks + rank) * kExchangeTaggedElems;
}
__host__ __device__ inline float* exchange_slot(void* base, int parity, int rank) {
  return reinterpret_cast<float*>(base) + ((size_t)parity * kExchangeMaxRanks + rank) * kExchangeSlotElems;
}
__host__ __device__ inline uint32_t* exchange_flag(void* base, int parity, int rank, int cta) {
  return reinterpret_cast<uint32_t*>(reinterpret_cast<char*>(base) + kExchangeDataBytes) +
         ((size_t)parity * kExchangeMaxRanks + rank) * kExchangeMaxFlags + cta;
}
__host__ __device__ inline uint32_t* exchange_counter(void* base) {
  return reinterpret_cast<uint32_t*>(reinterpret_cast<char*>(base) + kExchangeDataBytes + kExchangeFlagBytes);
}
struct ExchangeArgs {
  void* peer[kExchangeMaxRanks];  // every rank's exchange buffer as mapped here; peer[rank] is this rank's own
  int rank = 0, world = 1;
  long long limit_cycles = 0;     // bound of the wait for the peers' flags
  // up to kExchangeMaxSegs tensors travel in one call, one after the other in the slot
  int n_seg = 0;
  int seg_count[4] = {0, 0, 0, 0};
  int seg_op[4] = {0, 0, 0, 0};   // RedOp
  float* seg_ptr[4] = {nullptr, nullptr, nullptr, nullptr};
  uint32_t* err = nullptr;
};
constexpr int kExchangeMaxSegs = 4;
cudaError_t exchange_allreduce(const ExchangeArgs& a, cudaStream_t s);
}  // namespace akgb
#include "../../include/akgb.h"
namespace akgb {
// A bounded wait of a peer-memory exchange ran out on this device (seen by akgb_check_device_error): the ranks' call
// counters may disagree from here on, so further peer-memory exchanges are refused until the caller turns the path on
// again on all ranks (akgb_comm_set_peer_exchange), which also restarts the counters.
bool device_exchange_failed(int device);
void device_exchange_set_failed(int device, bool failed);
// the device error word of the kernel's device (allocated on first use); nullptr on failure
uint32_t* kernel_error_word(akgb_kernel* k);
// Sharded launch whose reduction completes the exchange itself: if the kernel's partial outputs all come from one
// reduction step that can do so, launches the plan with `base` (peers, rank, world, wait limit) attached and sets
// *fused; otherwise launches nothing and leaves *fused false.
bool kernel_exchange_fusable(const akgb_kernel* k);
// a sharded region that runs as stages with the exchange step between them: launches every stage through
// akgb_launch_sharded (kernel, then the exchange of its partial results)
bool kernel_is_staged(const akgb_kernel* k);
const akgb_kernel* kernel_stage(const akgb_kernel* k, int i);  // nullptr past the last stage
akgb_status launch_staged(akgb_kernel* k, akgb_comm* c, void* const* tensors, void* workspace, size_t workspace_bytes,
                          void* stream);
akgb_status launch_with_exchange(akgb_kernel* k, const FinishExchange& base, void* const* tensors, void* workspace,
                                 size_t workspace_bytes, void* stream, bool* fused);

// ---- index ops ---------------------------------------------------------------------
// out[o, i, r] = data[o, idx[i], r]; data is [outer, dim, inner] elements of `esize` bytes; idx int32 or int64
cudaError_t gather_rows(const void* data, const void* idx, void* out, int64_t outer, int64_t dim, int64_t nidx,
                        int64_t inner, int esize, int idx64, cudaStream_t s, LaunchDims* dims);
// out[num_segments, inner] = 0; out[ids[i], :] += data[i, :]; dt = DT code of data and out (float32, int32, float16,
// bfloat16), the sum accumulates in that type
cudaError_t segment_sum(const void* data, const void* ids, void* out, int64_t nids, int64_t inner, int64_t num_segments,
                        int idx64, int dt, cudaStream_t s, LaunchDims* dims);

// index of the first maximum along `dim` of a [outer, dim, inner] tensor (NaN counts as the maximum, as np.argmax);
// in_dt is the DT code of the data (float32, float16, bfloat16, int32), out64 selects int64 indices
cudaError_t argmax_axis(const void* data, void* out, int64_t outer, int64_t dim, int64_t inner, int in_dt, int out64,
                        cudaStream_t s, LaunchDims* dims);

// ---- transpose -----------------------------------------------------------------
// General permutation of up to 6 folded dims over elements of `esize` bytes.
struct TransposeParams {
  int rank = 0;                 // folded rank, <= 6
  int64_t out_shape[6] = {0};   // output extents
  int64_t in_stride[6] = {0};   // input stride (elements) of each OUTPUT dim
  int esize = 0;                // element size in bytes
};
cudaError_t transpose_nd(const TransposeParams& p, const void* x, void* out, cudaStream_t s, LaunchDims* dims);

// ---- matmul + epilogue -----------------------------------------------------------
struct MatmulParams {
  int64_t M = 0, N = 0, K = 0;
  int transpose_b = 0;  // 0: B is [K,N]; 1: B is [N,K]
  int has_bias = 0;     // bias[N] added in f32
  int bias_dt = 0;      // DT code of bias (BF16, F16 or F32)
  int relu = 0;         // max(., 0)
  int out_dt = 0;       // DT code of the output: the operand type (BF16 / F16) or F32
  int in_dt = 8;        // DT code of A and B: BF16 (8) or F16 (5) on the tensor cores, F32 (6) on the CUDA cores
};
// Encodes the TMA descriptors for (A, B) and launches the tcgen05 kernel: `batch` independent products in one launch
// (A and the output hold one matrix after the other; B too when b_batched, else every entry uses the same B).
cudaError_t matmul_bf16(const MatmulParams& p, const void* A, const void* B, const void* bias, void* out,
                        int64_t batch, bool b_batched, uint32_t* err_word, int sm_count, cudaStream_t s,
                        LaunchDims* dims);
bool matmul_bf16_supported(const MatmulParams& p, const char** why);
// float32 operands and result on the CUDA cores (in_dt = F32); `batch` entries `stride_*` elements apart, one launch
cudaError_t matmul_f32(const MatmulParams& p, const void* A, const void* B, const void* bias, void* out,
                       int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_o, cudaStream_t s,
                       LaunchDims* dims);

}  // namespace akgb
