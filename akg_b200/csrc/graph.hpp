// Typed op-DAG of one fused region, built from the ".info" JSON.
//
// Mirrors what MindConverter/MindBuilder extract from the same file
// (akg-mlir/lib/Target/MindsporeDialect/TranslateToMindsporeDialect.cpp:295-415
// for the top-level keys, :417-486 for the operator names, :488-502 for the
// element types, :650-658 for constant operands).
#pragma once
#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "json.hpp"

namespace akgb {

enum class DT : int { Bool = 0, I8, I16, I32, I64, F16, F32, F64, BF16, Invalid = -1 };

inline size_t dt_size(DT d) {
  switch (d) {
    case DT::Bool: case DT::I8: return 1;
    case DT::I16: case DT::F16: case DT::BF16: return 2;
    case DT::I32: case DT::F32: return 4;
    case DT::I64: case DT::F64: return 8;
    default: return 0;
  }
}
inline bool dt_is_float(DT d) { return d == DT::F16 || d == DT::F32 || d == DT::F64 || d == DT::BF16; }
const char* dt_name(DT d);
DT dt_from_name(const std::string& s);  // "uint8" maps to I8 like the reference (:331-333)

enum class OpK : int {
  // unary
  Abs, Neg, Exp, Log, Tanh, Rsqrt, Sqrt, Reciprocal, Floor, Square, Sin, Cos, Asinh, Acosh, Atan, ASin, ACos,
  IsInf, IsFinite, IsNan, LogicalNot, Cast,
  // binary
  Add, Sub, Mul, Div, Maximum, Minimum, Pow, Atan2, Equal, NotEqual, Greater, GreaterEqual, Less, LessEqual,
  LogicalAnd, LogicalOr,
  // ternary
  Select,
  // n-ary elementwise
  AddN,
  // shape
  BroadcastTo, Reshape, Transpose, Tile, Slice, StridedSlice, Concat,
  // reductions
  ReduceSum, ReduceMax, ReduceMin, ReduceProd, ReduceAll, ReduceAny,
  // contractions
  MatMul, BatchMatMul,
  // index ops
  Gather, UnsortedSegmentSum, ArgMax, Pad,
  // in-place
  Assign,
  Unknown
};
const char* opk_name(OpK k);
bool opk_is_unary(OpK k);
bool opk_is_binary(OpK k);
bool opk_is_reduce(OpK k);
bool opk_is_elementwise(OpK k);  // unary | binary | Select

// Operator classes in the reference's precedence order
// (akg-mlir/lib/Transforms/OperatorIdentify.cpp:51-93: the tag of a fused
// region is the highest class among its ops).
enum class OpClass : int { Elementwise = 0, Broadcast, Reshape, Transpose, Reduction, Matmul, Conv };
// Direction of a reduction (akg-mlir/lib/Dialect/Linalg/Transforms/MatchAndMarkReductionOps.cpp:51-89):
// X if the last axis is reduced, ALL if every axis is, otherwise Y.
enum class ReduceDir : int { None = 0, X, Y, All };

struct Value {
  std::string name;
  std::vector<int64_t> shape;
  DT dt = DT::Invalid;
  bool is_const = false;
  std::vector<double> cval;  // constant payload (one entry = splat)
  int producer = -1;         // op index, -1 for graph inputs/constants
  int input_index = -1;      // position in input_desc, -1 otherwise
  int output_index = -1;     // position in output_desc, -1 otherwise
  std::vector<int> users;    // op indices
  std::vector<std::string> sym;  // "symbolic_shape" of a region argument: one symbol or number per dim ("" = none)
  // sharding (filled by infer_sharding)
  bool split0 = false;       // axis 0 holds only this rank's slice
  int partial = 0;           // akgb_shard_kind of a partial result, 0 = none

  int64_t numel() const {
    int64_t n = 1;
    for (auto s : shape) n *= s;
    return n;
  }
  bool is_scalar_const() const { return is_const && cval.size() == 1; }
};

struct Node {
  OpK kind = OpK::Unknown;
  std::string name;          // JSON operator name
  std::vector<int> in;       // value ids
  int out = -1;              // value id
  std::vector<int64_t> axes; // reductions: normalised, sorted, unique
  bool keep_dims = false;
  std::vector<int64_t> perm; // transpose
  bool transpose_a = false, transpose_b = false;
  // Tile: multiples; Slice: begin/size; StridedSlice: begin/end/strides (masks already applied); Concat: axis
  std::vector<int64_t> multiples, begin, size, end, strides;
  int64_t axis = 0;
  int64_t num_segments = 0;  // UnsortedSegmentSum
  std::vector<int64_t> pad_low, pad_high;  // Pad, per dimension
  double pad_value = 0.0;
  bool enable_atomic_add = false;
};

struct Graph {
  std::string kernel_name;
  std::string process;
  std::string compute_capability;
  std::vector<Value> values;
  std::vector<Node> nodes;
  std::vector<int> inputs;   // value ids in input_desc order
  std::vector<int> outputs;  // value ids in output_desc order
  OpClass op_class = OpClass::Elementwise;
  ReduceDir reduce_dir = ReduceDir::None;
  std::string sha256_hex;    // of the JSON text
  bool dynamic = false;      // some extent is -1: shapes are bound at launch (bind_shapes)
  // "symbol_calc_expr": symbol -> expression over other symbols (integers, + - * /, parentheses); bind_shapes
  // evaluates them from the extents the caller binds and checks every argument dim that names a symbol against it
  std::vector<std::pair<std::string, std::string>> symbol_expr;

  const Value& v(int id) const { return values[id]; }
  Value& v(int id) { return values[id]; }
  const Node* producer(int vid) const {
    int p = values[vid].producer;
    return p < 0 ? nullptr : &nodes[p];
  }
};

struct Unsupported : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// Front end: JSON text -> Graph (throws JsonError / Unsupported).
Graph parse_info(const char* text, size_t len);
// Class tag + reduction direction, by the reference's rules.
void classify(Graph& g);
// Leading-axis sharding: rewrites shapes to the local slice of rank `rank` of
// `world` and marks values as split / partial.  Throws Unsupported when the
// region cannot be split on axis 0 without more than an all-reduce of outputs.
void infer_sharding(Graph& g, int rank, int world);

// Dynamic-shape regions (extents written as -1, the form MindSpore emits and the reference's --gpu-dyn-opt
// pipeline consumes, akg-mlir/lib/Pipelines/GPUPipelines/GPUDynOpt.cpp:47-143): substitutes the extents of every
// argument (inputs then outputs, `shapes[i]` = extents of argument i) and infers the shapes in between, op by op.
// Returns a static copy of the graph; throws JsonError when the extents contradict the description.
Graph bind_shapes(const Graph& g, const std::vector<std::vector<int64_t>>& shapes);

// Sharded regions in which a reduction over the split axis feeds later ops, cut into stages at those reductions
// (stages.cpp).  Every stage is a region of its own with GLOBAL shapes (infer_sharding is applied to it afterwards);
// its arguments are the parent's arguments or "carried" values: partial results an earlier stage produced and the
// exchange step completed.
struct StageGraph {
  Graph g;
  std::vector<int> in_parent;    // per stage input: index among the parent's inputs, or -1
  std::vector<int> in_carried;   // per stage input: index of the carried value it reads, or -1
  std::vector<int> out_parent;   // per stage output: index among the parent's outputs, or -1
  std::vector<int> out_carried;  // per stage output: index of the carried value it defines, or -1
};
struct StagePlan {
  std::vector<StageGraph> stages;
  std::vector<int> carried;      // value ids (in the parent graph) of the carried values
};
// false when the region has no reduction over the split axis that feeds another op (or holds ops the cut does not
// handle: matmuls, in-place stores)
bool split_at_sharded_reductions(const Graph& g, StagePlan* out);

std::string sha256_hex(const char* data, size_t len);

}  // namespace akgb
