// Program of the generic elementwise/broadcast kernel: a straight-line list of
// typed ops over a small register file, one value per register per element.
// Built on the host from any group of elementwise ops of a fused region that no
// specialised template claims; executed by ew_generic_kernel.
#pragma once
#include <cstdint>

namespace akgb {

enum EwOp : uint8_t {
  EW_COPY = 0,  // BroadcastTo / identity
  // unary
  EW_ABS, EW_NEG, EW_EXP, EW_LOG, EW_TANH, EW_RSQRT, EW_SQRT, EW_RECIP, EW_FLOOR, EW_SQUARE, EW_SIN, EW_COS,
  EW_ASINH, EW_ACOSH, EW_ATAN, EW_ASIN, EW_ACOS, EW_ISINF, EW_ISFINITE, EW_ISNAN, EW_NOT, EW_CAST,
  // binary
  EW_ADD, EW_SUB, EW_MUL, EW_DIV, EW_MAX, EW_MIN, EW_POW, EW_ATAN2, EW_EQ, EW_NE, EW_GT, EW_GE, EW_LT, EW_LE,
  EW_AND, EW_OR,
  // ternary
  EW_SELECT
};

// how a register holds its value
enum EwClass : uint8_t { EWC_FLOAT = 0, EWC_INT = 1, EWC_BOOL = 2 };

struct EwInstr {
  uint8_t op;       // EwOp
  uint8_t dt;       // DT code of the result (rounding target)
  uint8_t cls;      // EwClass of the result
  uint8_t src_cls;  // EwClass of the operands (compares, casts)
  uint8_t dst, a, b, c;
};

enum EwIndexKind : int32_t { EWI_FULL = 0, EWI_MOD = 1, EWI_SCALAR = 2, EWI_STRIDED = 3 };

constexpr int kEwMaxIn = 10, kEwMaxOut = 6, kEwMaxInstr = 96, kEwMaxReg = 48, kEwMaxConst = 24, kEwMaxRank = 6;

struct EwOperand {
  int32_t dt;          // DT code of the tensor in memory
  int32_t kind;        // EwIndexKind
  int32_t reg;         // register loaded from / stored to
  int32_t pad;
  int64_t mod;         // EWI_MOD: index = e % mod
  int64_t offset;      // EWI_STRIDED: first element (Slice / StridedSlice begin, Concat position)
  int64_t stride[kEwMaxRank];  // EWI_STRIDED: element stride per iteration dim (0 = broadcast)
  int64_t wrap[kEwMaxRank];    // EWI_STRIDED: if non-zero the dim's index is taken modulo this (Tile)
};

struct EwProgram {
  int32_t n_in, n_out, n_instr, n_reg, n_const, rank;
  int64_t n;                     // elements of the iteration space
  int64_t shape[kEwMaxRank];     // iteration space (folded), row-major
  EwOperand in[kEwMaxIn];
  EwOperand out[kEwMaxOut];
  uint32_t const_bits[kEwMaxConst];  // already rounded to the constant's declared type
  uint8_t const_reg[kEwMaxConst];
  EwInstr instr[kEwMaxInstr];
  // 64-bit constants: const_bits holds the low word, const_hi the high word; const_f64 = 1 a double, 2 a 64-bit integer
  uint32_t const_hi[kEwMaxConst];
  uint8_t const_f64[kEwMaxConst];
};

}  // namespace akgb

// ---- row program --------------------------------------------------------------------------------------------------
// A fused region whose iteration space is [rows, cols] with reductions along cols only (the reduce-X class: softmax,
// LayerNorm, RMSNorm, log-softmax, L2-normalise ... in any spelling).  Values are either per element of the row
// ("full") or one per row; the program is a static single assignment list that the run-time generator prints as one
// kernel in which a group of threads owns a row and keeps it in registers.  Host-side only.
#include <vector>

namespace akgb {

enum RowKind : int32_t {
  RK_FULL = 0,    // [rows, cols]
  RK_ROW = 1,     // [rows] / [rows, 1]
  RK_COL = 2,     // [cols], the same for every row
  RK_SCALAR = 3,  // one element
  RK_ROWMOD = 4   // [mod_rows, cols] with rows % mod_rows == 0: row r reads row r % mod_rows (a mask shared by batches)
};

struct RowOperand {
  int32_t dt = 0;
  int32_t kind = RK_FULL;
  int32_t val = 0;  // value loaded into / stored from
  int64_t mod_rows = 0;
  int64_t row_div = 1, row_mod = 0;  // RK_ROW read through (row / row_div) % row_mod when row_mod != 0 (a per-channel value)
  int32_t red_op = 0;  // column mode results: 0 sum, 1 max, 2 min, 3 prod over the rows of `val`
};

struct RowInstr {
  uint8_t op = 0;  // EwOp, unless `reduce`
  uint8_t dt = 0, cls = 0, src_cls = 0;
  bool reduce = false;  // dst (per row) = reduction of a (full) along the row
  int32_t red_op = 0;   // 0 sum, 1 max, 2 min, 3 prod
  bool full = false;    // the result is per element
  int32_t dst = 0, a = 0, b = 0, c = 0;
};

struct RowProgram {
  int64_t rows = 0, cols = 0;
  int32_t n_val = 0;
  std::vector<RowOperand> in, out;
  std::vector<RowInstr> instr;
  std::vector<int32_t> const_val;
  std::vector<uint32_t> const_bits;
  std::vector<uint8_t> val_full;  // per value: per element (1) or per row (0)
  // column mode: the program ends in one or more reductions that fold the ROWS (axis 0 of [rows, cols]); every result
  // is [cols].  Generated as a kernel that walks rows and keeps 8 column accumulators per thread and result.
  bool col_reduce = false;
  // A row program may also sum some of its per-element values over ALL rows (LayerNorm backward: the weight and bias
  // gradients next to the row-wise input gradient).  Those results are outputs of kind RK_COL; the kernel is then
  // launched with a fixed number of CTAs that walk the rows and writes one partial [cols] vector per CTA and result.
  bool col_sums = false;
  // Rows too long for registers: keep the inputs that several passes read in shared memory (a cluster of CTAs per row
  // when one CTA's shared memory is too small, reductions completed through distributed shared memory) instead of
  // re-reading them through L2.  Off by default: measured slower than the L2 schedule on B200 (AKGB_FLAG_STAGE_LONG_ROWS).
  bool stage_long_rows = false;
};

}  // namespace akgb
