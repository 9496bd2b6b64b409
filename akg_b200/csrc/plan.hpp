// Execution plan of one fused region: an ordered list of kernel-template
// instantiations over argument slots and workspace offsets.
#pragma once
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "ew_program.hpp"
#include "graph.hpp"
#include "kernels.hpp"

namespace akgb {

// Where a kernel operand lives at launch: a caller tensor (index into the
// inputs-then-outputs list) or an offset into the caller's workspace.
struct Ref {
  int arg = -1;
  int64_t ws_off = -1;
  bool valid() const { return arg >= 0 || ws_off >= 0; }
};

enum class StepK : int { GeluChain, LayerNorm, Softmax, ReduceCol, ReduceAll, ReduceRow, ReduceColDual, Transpose, Matmul, Ew, Gather, SegmentSum, ArgMax, RowJit, ColJit };

struct Step {
  StepK kind;
  std::string kernel_name;  // device symbol family, for the metadata JSON
  Ref a, b, c, out, out2, out3;
  Ref scratch;              // partials
  GeluChainParams gelu;
  LayerNormParams ln;
  SoftmaxParams sm;
  RedOp red_op = RedOp::Sum, red_op2 = RedOp::Max;
  int64_t red_outer = 1, red_len = 1, red_inner = 1;
  TransposeParams tp;
  MatmulParams mm;
  EwProgram ew;              // StepK::Ew
  std::shared_ptr<RowProgram> row;  // StepK::RowJit (operands in ew_in / ew_out)
  std::vector<Ref> ew_in, ew_out;
  int64_t ix_outer = 1, ix_dim = 1, ix_n = 1, ix_inner = 1, ix_segments = 0;  // Gather / SegmentSum extents
  int ix_esize = 4, ix_idx64 = 0;
  int64_t mm_batch = 1, mm_stride_a = 0, mm_stride_b = 0, mm_stride_o = 0;  // BatchMatMul: byte strides per entry
  int64_t red_batch_in = 0, red_batch_out = 0;  // batched column reductions: element stride per outer index
  LaunchDims dims;          // filled at first launch
};

struct Plan {
  std::string klass;        // operator class reported to the caller
  std::vector<Step> steps;
  size_t workspace_bytes = 0;
  int64_t bytes = 0;        // algorithmic bytes: inputs read once + outputs written once
  int64_t flops = 0;
  bool needs_gelu_lut = false;
  // A plan made of one run-time generated row kernel carries the multi-launch plan of the same region; it takes over
  // for good if the kernel cannot be generated or compiled on this host.
  std::shared_ptr<Plan> fallback;
  bool use_fallback = false;
  // bytes of every argument (inputs then outputs) of the graph this plan was built for: the ranges of checked launches
  std::vector<size_t> arg_bytes;
};

// Pattern matcher: places the region on kernel templates or throws Unsupported.
Plan build_plan(const Graph& g, int sm_count, bool allow_jit = true);
// Reduce-X regions as one row program (rowfuse.cpp); `in_values` / `out_values` receive the graph values of the operands.
bool build_row_program(const Graph& g, RowProgram* out, std::vector<int>* in_values, std::vector<int>* out_values,
                       bool col_mode = false, const std::map<int, std::pair<int64_t, int64_t>>* row_index = nullptr,
                       bool allow_col_sums = false);
// Fallback of build_plan: splits the region into elementwise groups (generic kernel), reductions, transposes and
// matmuls that run one after the other with intermediates in the workspace.
Plan build_generic_plan(const Graph& g, int sm_count);

}  // namespace akgb
