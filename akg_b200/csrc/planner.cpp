// Generic planner: runs any region made of supported ops as a sequence of kernels.
//
// The reference compiles every fused region into one kernel through its polyhedral pipeline
// (akg-mlir/lib/Pipelines/GPUPipelines/GPUOpt.cpp:45-132).  Here the specialised templates cover the shapes that
// matter for bandwidth; everything else is split at the points where the iteration space changes:
//   * consecutive elementwise / BroadcastTo ops over one iteration shape -> one launch of the generic
//     elementwise kernel (per-op typed arithmetic, broadcast by dropped dims);
//   * each reduction, transpose and matmul -> its own template launch;
//   * Reshape is a view (EliminateReshape in the reference drops boundary reshapes the same way).
// Values that cross a launch boundary live in the caller's workspace.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <set>

#include "hostconv.hpp"
#include "plan.hpp"

namespace akgb {
namespace {

EwClass cls_of(DT d) { return dt_is_float(d) ? EWC_FLOAT : (d == DT::Bool ? EWC_BOOL : EWC_INT); }

bool ew_opcode(OpK k, EwOp* op) {
  switch (k) {
    case OpK::Abs: *op = EW_ABS; return true;
    case OpK::Neg: *op = EW_NEG; return true;
    case OpK::Exp: *op = EW_EXP; return true;
    case OpK::Log: *op = EW_LOG; return true;
    case OpK::Tanh: *op = EW_TANH; return true;
    case OpK::Rsqrt: *op = EW_RSQRT; return true;
    case OpK::Sqrt: *op = EW_SQRT; return true;
    case OpK::Reciprocal: *op = EW_RECIP; return true;
    case OpK::Floor: *op = EW_FLOOR; return true;
    case OpK::Square: *op = EW_SQUARE; return true;
    case OpK::Sin: *op = EW_SIN; return true;
    case OpK::Cos: *op = EW_COS; return true;
    case OpK::Asinh: *op = EW_ASINH; return true;
    case OpK::Acosh: *op = EW_ACOSH; return true;
    case OpK::Atan: *op = EW_ATAN; return true;
    case OpK::ASin: *op = EW_ASIN; return true;
    case OpK::ACos: *op = EW_ACOS; return true;
    case OpK::IsInf: *op = EW_ISINF; return true;
    case OpK::IsFinite: *op = EW_ISFINITE; return true;
    case OpK::IsNan: *op = EW_ISNAN; return true;
    case OpK::LogicalNot: *op = EW_NOT; return true;
    case OpK::Cast: *op = EW_CAST; return true;
    case OpK::Add: *op = EW_ADD; return true;
    case OpK::Sub: *op = EW_SUB; return true;
    case OpK::Mul: *op = EW_MUL; return true;
    case OpK::Div: *op = EW_DIV; return true;
    case OpK::Maximum: *op = EW_MAX; return true;
    case OpK::Minimum: *op = EW_MIN; return true;
    case OpK::Pow: *op = EW_POW; return true;
    case OpK::Atan2: *op = EW_ATAN2; return true;
    case OpK::Equal: *op = EW_EQ; return true;
    case OpK::NotEqual: *op = EW_NE; return true;
    case OpK::Greater: *op = EW_GT; return true;
    case OpK::GreaterEqual: *op = EW_GE; return true;
    case OpK::Less: *op = EW_LT; return true;
    case OpK::LessEqual: *op = EW_LE; return true;
    case OpK::LogicalAnd: *op = EW_AND; return true;
    case OpK::LogicalOr: *op = EW_OR; return true;
    case OpK::Select: *op = EW_SELECT; return true;
    case OpK::BroadcastTo: *op = EW_COPY; return true;
    default: return false;
  }
}

// int64 and float64 values run in generated kernels only (all integer registers widened to 64 bits, all
// floating-point registers to double)
bool ew_dtype_ok(DT d) { return d != DT::Invalid; }

uint32_t const_bits(double v, DT d) {
  float f;
  switch (d) {
    case DT::F16: f = round_f64_to_f16(v); break;
    case DT::BF16: f = round_f64_to_bf16(v); break;
    case DT::F32: f = (float)v; break;
    case DT::Bool: return v != 0.0 ? 1u : 0u;
    default:
      if (d == DT::I64 && (v > 2147483647.0 || v < -2147483648.0))
        throw Unsupported("64-bit integer constant outside the 32-bit range");
      return (uint32_t)(int32_t)std::llround(v);
  }
  uint32_t b;
  std::memcpy(&b, &f, 4);
  return b;
}

}  // namespace

// shared with the row-program builder (rowfuse.cpp)
bool ew_opcode_of(OpK k, EwOp* op) { return ew_opcode(k, op); }
uint32_t ew_const_bits(double v, DT d) { return const_bits(v, d); }
bool ew_type_ok(DT d) { return ew_dtype_ok(d) && d != DT::I64 && d != DT::F64; }  // row / column programs keep 32-bit registers

namespace {

struct Builder {
  const Graph& g;
  int sm_count;
  Plan plan;
  std::map<int, Ref> where;     // value id -> buffer (only materialised values)
  std::map<int, int> alias;     // value id -> value id it is a view of
  size_t ws = 0;
  std::vector<int> group;       // node indices of the open elementwise group
  std::vector<int64_t> group_shape;

  Builder(const Graph& gr, int sms) : g(gr), sm_count(sms) {}

  int root(int v) const {
    auto it = alias.find(v);
    while (it != alias.end()) {
      v = it->second;
      it = alias.find(v);
    }
    return v;
  }
  Ref arg_ref(int vid) const {
    const Value& v = g.v(vid);
    Ref r;
    if (v.input_index >= 0) r.arg = v.input_index;
    else if (v.output_index >= 0) r.arg = (int)g.inputs.size() + v.output_index;
    return r;
  }
  // buffer holding value vid (allocating workspace for intermediates on first use)
  Ref buffer(int vid) {
    vid = root(vid);
    auto it = where.find(vid);
    if (it != where.end()) return it->second;
    Ref r = arg_ref(vid);
    if (!r.valid()) {
      // a view of this value may be a graph output: then the producer writes there directly
      for (auto& kv : alias)
        if (root(kv.first) == vid && g.v(kv.first).output_index >= 0) r = arg_ref(kv.first);
    }
    if (!r.valid()) {
      r.ws_off = (int64_t)ws;
      ws += ((size_t)g.v(vid).numel() * dt_size(g.v(vid).dt) + 255) / 256 * 256;
    }
    where[vid] = r;
    return r;
  }
  bool produced_in_group(int vid) const {
    int p = g.v(vid).producer;
    return p >= 0 && std::find(group.begin(), group.end(), p) != group.end();
  }
  bool used_outside_group(int vid) const {
    const Value& v = g.v(vid);
    if (v.output_index >= 0) return true;
    for (int u : v.users)
      if (std::find(group.begin(), group.end(), u) == group.end()) return true;
    for (auto& kv : alias)  // a view of it is needed later (or is an output)
      if (kv.second == vid) return true;
    return false;
  }

  // Would the open group, with node `cand` added, still fit one launch of the elementwise kernel (tensor operands,
  // constants, results, instructions)?  Results are counted as "used by something not in the group so far", which
  // over-counts values whose consumers have not been visited yet; that only splits a very wide group early.
  bool group_fits_with(int cand) const {
    std::vector<int> list = group;
    list.push_back(cand);
    std::set<int> inside, ext, consts;
    for (int ni : list) inside.insert(g.nodes[ni].out);
    int instr = 0, outs = 0;
    for (int ni : list) {
      const Node& n = g.nodes[ni];
      instr += n.kind == OpK::AddN ? (int)n.in.size() : 1;
      for (int vid : n.in) {
        if (inside.count(vid)) continue;
        if (g.v(vid).is_const) consts.insert(vid);
        else ext.insert(vid);
      }
      const Value& o = g.v(n.out);
      bool outside = o.output_index >= 0 || n.kind == OpK::Assign;
      for (int u : o.users)
        if (std::find(list.begin(), list.end(), u) == list.end()) outside = true;
      for (auto& kv : alias)
        if (kv.second == n.out) outside = true;
      outs += outside;
    }
    return (int)ext.size() <= kEwMaxIn && (int)consts.size() <= kEwMaxConst && outs <= kEwMaxOut &&
           instr <= kEwMaxInstr - 8 && (int)(ext.size() + consts.size()) <= kEwMaxReg - 8;
  }

  void flush_group() {
    if (group.empty()) return;
    Step st;
    st.kind = StepK::Ew;
    st.kernel_name = "ew_generic";
    EwProgram& P = st.ew;
    std::memset(&P, 0, sizeof(P));
    const std::vector<int64_t>& S = group_shape;
    if (S.size() > (size_t)kEwMaxRank) throw Unsupported("elementwise group of rank above 6");
    P.rank = (int)S.size();
    P.n = 1;
    for (size_t i = 0; i < S.size(); ++i) {
      P.shape[i] = S[i];
      P.n *= S[i];
    }
    // last use of every value inside the group, for register reuse
    std::map<int, int> last_use;
    for (size_t gi = 0; gi < group.size(); ++gi)
      for (int vid : g.nodes[group[gi]].in) last_use[vid] = (int)gi;
    for (size_t gi = 0; gi < group.size(); ++gi)  // values stored by an Assign stay live to the end
      if (g.nodes[group[gi]].kind == OpK::Assign)
        for (int vid : g.nodes[group[gi]].in) last_use[vid] = (int)group.size();
    std::map<int, int> reg_of;  // value id -> register
    std::set<int> external;     // operands that come from outside the group
    std::vector<int> free_regs;
    int next_reg = 0;
    auto alloc_reg = [&]() {
      if (!free_regs.empty()) {
        int r = free_regs.back();
        free_regs.pop_back();
        return r;
      }
      if (next_reg >= kEwMaxReg) throw Unsupported("elementwise group needs more than 48 live values");
      return next_reg++;
    };
    auto operand_reg = [&](int vid) -> int {
      auto it = reg_of.find(vid);
      if (it != reg_of.end()) return it->second;
      const Value& v = g.v(vid);
      if (!ew_dtype_ok(v.dt)) throw Unsupported(std::string("generic elementwise kernel: type ") + dt_name(v.dt));
      // operands from outside the group are loaded before the first instruction runs, so their registers are
      // never shared with values computed in the group
      if (next_reg >= kEwMaxReg) throw Unsupported("elementwise group needs more than 48 live values");
      int r = next_reg++;
      reg_of[vid] = r;
      external.insert(vid);
      if (v.is_const) {
        if (v.cval.size() != 1) throw Unsupported("constant tensors with more than one element");
        if (P.n_const >= kEwMaxConst) throw Unsupported("too many constants in one elementwise group");
        if (v.dt == DT::F64) {
          uint64_t b;
          const double dv = v.cval[0];
          std::memcpy(&b, &dv, 8);
          P.const_bits[P.n_const] = (uint32_t)b;
          P.const_hi[P.n_const] = (uint32_t)(b >> 32);
          P.const_f64[P.n_const] = 1;
        } else if (v.dt == DT::I64 && (v.cval[0] > 2147483647.0 || v.cval[0] < -2147483648.0)) {
          // a 64-bit integer constant outside the 32-bit range (the description carries it as a number: exact to 2^53)
          if (!(std::fabs(v.cval[0]) < 9.2e18)) throw Unsupported("64-bit integer constant out of range");
          const uint64_t b = (uint64_t)(int64_t)std::llround(v.cval[0]);
          P.const_bits[P.n_const] = (uint32_t)b;
          P.const_hi[P.n_const] = (uint32_t)(b >> 32);
          P.const_f64[P.n_const] = 2;
        } else {
          P.const_bits[P.n_const] = const_bits(v.cval[0], v.dt);
        }
        P.const_reg[P.n_const] = (uint8_t)r;
        ++P.n_const;
        return r;
      }
      // external tensor operand
      if (P.n_in >= kEwMaxIn) throw Unsupported("elementwise group with more than 10 tensor operands");
      EwOperand& o = P.in[P.n_in];
      o.dt = (int)v.dt;
      o.reg = r;
      std::vector<int64_t> vs = v.shape;
      const int64_t vn = v.numel();
      if (vn == P.n) o.kind = EWI_FULL;
      else if (vn == 1) o.kind = EWI_SCALAR;
      else {
        while (vs.size() > 1 && vs.front() == 1) vs.erase(vs.begin());
        bool trailing = vs.size() <= S.size();
        for (size_t i = 0; trailing && i < vs.size(); ++i)
          if (vs[vs.size() - 1 - i] != S[S.size() - 1 - i]) trailing = false;
        if (trailing) {
          o.kind = EWI_MOD;
          o.mod = vn;
        } else {
          if (vs.size() > S.size()) throw Unsupported("operand rank above the iteration space");
          o.kind = EWI_STRIDED;
          int64_t stride = 1;
          for (int i = (int)S.size() - 1, j = (int)vs.size() - 1; i >= 0; --i, --j) {
            if (j >= 0) {
              if (vs[j] == S[i]) o.stride[i] = stride;
              else if (vs[j] == 1) o.stride[i] = 0;
              else throw Unsupported("operand does not broadcast to the iteration space");
              stride *= vs[j];
            } else {
              o.stride[i] = 0;
            }
          }
        }
      }
      st.ew_in.push_back(buffer(vid));
      ++P.n_in;
      return r;
    };
    for (size_t gi = 0; gi < group.size(); ++gi) {  // all outside operands first
      const Node& gn = g.nodes[group[gi]];
      if (gn.kind == OpK::Tile || gn.kind == OpK::Slice || gn.kind == OpK::StridedSlice) continue;
      for (int vid : gn.in)
        if (!produced_in_group(vid)) operand_reg(vid);
    }
    for (size_t gi = 0; gi < group.size(); ++gi) {
      const Node& n = g.nodes[group[gi]];
      const Value& out = g.v(n.out);
      if (!ew_dtype_ok(out.dt)) throw Unsupported(std::string("generic elementwise kernel: type ") + dt_name(out.dt));
      EwInstr ins;
      std::memset(&ins, 0, sizeof(ins));
      EwOp op;
      const bool view_copy = n.kind == OpK::Tile || n.kind == OpK::Slice || n.kind == OpK::StridedSlice;
      if (n.kind == OpK::Assign) {
        // Assign(dst, value): the value is stored into the caller's dst tensor and is also the op's result;
        // InplaceAssign(dst, value, passthrough): same store, the result is the third operand
        // (MindSporeToLinalg.cpp:495-524; op_dsl.py:956-961, 1032-1037)
        const int dstv = n.in[0];
        const Value& dv = g.v(dstv);
        if (dv.input_index < 0) throw Unsupported("Assign target must be an input of the region");
        if (dv.shape != S || n.in.size() < 2 || g.v(n.in[1]).dt != dv.dt)
          throw Unsupported("Assign needs a value of the target's shape and type");
        const int val_reg = operand_reg(n.in[1]);
        const int res_reg = n.in.size() >= 3 ? operand_reg(n.in[2]) : val_reg;
        if (P.n_out + 2 > kEwMaxOut) throw Unsupported("elementwise group with more than 6 results");
        EwOperand& od = P.out[P.n_out++];
        od.dt = (int)dv.dt;
        od.kind = EWI_FULL;
        od.reg = val_reg;
        st.ew_out.push_back(arg_ref(dstv));
        reg_of[n.out] = res_reg;
        external.insert(n.out);  // shares a register with its source: never recycled
        if (used_outside_group(n.out)) {
          EwOperand& oo = P.out[P.n_out++];
          oo.dt = (int)out.dt;
          oo.kind = EWI_FULL;
          oo.reg = res_reg;
          st.ew_out.push_back(buffer(n.out));
        }
        continue;
      }
      if (n.kind == OpK::Reshape || view_copy) op = EW_COPY;
      else if (n.kind == OpK::AddN) op = EW_ADD;
      else if (!ew_opcode(n.kind, &op)) throw Unsupported(std::string("op '") + n.name + "' in an elementwise group");
      if (view_copy) {
        // the source is read through its own index map: a dedicated operand and register
        const Value& src = g.v(n.in[0]);
        if (!ew_dtype_ok(src.dt)) throw Unsupported(std::string("generic elementwise kernel: type ") + dt_name(src.dt));
        if (P.n_in >= kEwMaxIn) throw Unsupported("elementwise group with more than 10 tensor operands");
        if (next_reg >= kEwMaxReg) throw Unsupported("elementwise group needs more than 48 live values");
        if (src.shape.size() != S.size()) throw Unsupported(std::string(n.name) + " that changes the rank");
        EwOperand& o = P.in[P.n_in++];
        o.dt = (int)src.dt;
        o.kind = EWI_STRIDED;
        o.reg = next_reg++;
        int64_t stride = 1;
        for (int d = (int)S.size() - 1; d >= 0; --d) {
          if (n.kind == OpK::Tile) {
            o.stride[d] = stride;
            o.wrap[d] = src.shape[d];
          } else if (n.kind == OpK::Slice) {
            o.stride[d] = stride;
            o.offset += n.begin[d] * stride;
          } else {
            o.stride[d] = stride * n.strides[d];
            o.offset += n.begin[d] * stride;
          }
          stride *= src.shape[d];
        }
        st.ew_in.push_back(buffer(n.in[0]));
        EwInstr ins;
        std::memset(&ins, 0, sizeof(ins));
        ins.op = EW_COPY;
        ins.dt = (uint8_t)out.dt;
        ins.cls = cls_of(out.dt);
        ins.src_cls = cls_of(src.dt);
        ins.a = (uint8_t)o.reg;
        const int dst = alloc_reg();
        reg_of[n.out] = dst;
        ins.dst = (uint8_t)dst;
        if (P.n_instr >= kEwMaxInstr) throw Unsupported("elementwise group with more than 96 ops");
        P.instr[P.n_instr++] = ins;
        if (used_outside_group(n.out)) {
          if (P.n_out >= kEwMaxOut) throw Unsupported("elementwise group with more than 6 results");
          EwOperand& oo = P.out[P.n_out++];
          oo.dt = (int)out.dt;
          oo.kind = EWI_FULL;
          oo.reg = dst;
          st.ew_out.push_back(buffer(n.out));
        }
        continue;
      }
      if (n.kind == OpK::AddN && n.in.size() > 2) {
        // a left-to-right chain of adds in the result type, like the expected-value generator's "a + b + c"
        int acc = operand_reg(n.in[0]);
        for (size_t j = 1; j < n.in.size(); ++j) {
          EwInstr a2;
          std::memset(&a2, 0, sizeof(a2));
          a2.op = EW_ADD;
          a2.dt = (uint8_t)out.dt;
          a2.cls = cls_of(out.dt);
          a2.src_cls = a2.cls;
          a2.a = (uint8_t)acc;
          a2.b = (uint8_t)operand_reg(n.in[j]);
          const int dst = alloc_reg();
          a2.dst = (uint8_t)dst;
          if (P.n_instr >= kEwMaxInstr) throw Unsupported("elementwise group with more than 96 ops");
          P.instr[P.n_instr++] = a2;
          acc = dst;
        }
        reg_of[n.out] = acc;
        if (used_outside_group(n.out)) {
          if (P.n_out >= kEwMaxOut) throw Unsupported("elementwise group with more than 6 results");
          EwOperand& oo = P.out[P.n_out++];
          oo.dt = (int)out.dt;
          oo.kind = EWI_FULL;
          oo.reg = acc;
          st.ew_out.push_back(buffer(n.out));
        }
        continue;
      }
      ins.op = op;
      ins.dt = (uint8_t)out.dt;
      ins.cls = cls_of(out.dt);
      ins.src_cls = cls_of(g.v(n.in[0]).dt);
      if (op == EW_SELECT) ins.src_cls = cls_of(g.v(n.in[1]).dt);
      // float -> integer Cast follows the reference's compiled route (tosa.cast: round to nearest even, clamp to the
      // result type; the expected-value generator would truncate like NumPy).  NaN gives 0.
      int regs[3] = {0, 0, 0};
      const size_t nin = std::min<size_t>(n.in.size(), 3);
      for (size_t j = 0; j < nin; ++j) regs[j] = operand_reg(n.in[j]);
      // operands whose last use is this instruction give their register back (unless they must be stored)
      for (size_t j = 0; j < nin; ++j) {
        int vid = n.in[j];
        if (last_use[vid] == (int)gi && !(produced_in_group(vid) && used_outside_group(vid)) && reg_of.count(vid)) {
          bool dup = false;
          for (size_t q = 0; q < j; ++q) dup |= n.in[q] == vid;
          if (!dup && !external.count(vid)) free_regs.push_back(reg_of[vid]);
        }
      }
      int dst = alloc_reg();
      reg_of[n.out] = dst;
      ins.dst = (uint8_t)dst;
      ins.a = (uint8_t)regs[0];
      ins.b = (uint8_t)regs[1];
      ins.c = (uint8_t)regs[2];
      if (P.n_instr >= kEwMaxInstr) throw Unsupported("elementwise group with more than 96 ops");
      P.instr[P.n_instr++] = ins;
      if (used_outside_group(n.out)) {
        if (P.n_out >= kEwMaxOut) throw Unsupported("elementwise group with more than 6 results");
        EwOperand& o = P.out[P.n_out++];
        o.dt = (int)out.dt;
        o.kind = EWI_FULL;
        o.reg = dst;
        st.ew_out.push_back(buffer(n.out));
      }
    }
    P.n_reg = next_reg;
    if (ew_generic_smem(P) > 200 * 1024) throw Unsupported("elementwise group needs too many live values");
    plan.steps.push_back(std::move(st));
    group.clear();
    group_shape.clear();
  }

  void add_reduce(const Node& n) {
    RedOp op;
    switch (n.kind) {
      case OpK::ReduceSum: op = RedOp::Sum; break;
      case OpK::ReduceMax: op = RedOp::Max; break;
      case OpK::ReduceMin: op = RedOp::Min; break;
      case OpK::ReduceProd: op = RedOp::Prod; break;
      case OpK::ReduceAll: op = RedOp::Min; break;  // over 0/1 values
      case OpK::ReduceAny: op = RedOp::Max; break;
      default: throw Unsupported(std::string("reduction '") + n.name + "' is not placed");
    }
    const Value& x = g.v(n.in[0]);
    const Value& ov = g.v(n.out);
    const bool narrow = x.dt == DT::F16 || x.dt == DT::BF16 || x.dt == DT::Bool;
    if (!(x.dt == DT::F32 || narrow) || ov.dt != x.dt)
      throw Unsupported(std::string("reduction over ") + dt_name(x.dt) + " is not placed");
    if ((n.kind == OpK::ReduceAll || n.kind == OpK::ReduceAny) != (x.dt == DT::Bool))
      throw Unsupported("ReduceAll/ReduceAny take bool, the arithmetic reductions do not");
    // float16 / bfloat16 / bool inputs are widened to float32, reduced there and narrowed once at the end: the
    // accumulator type of the reference's expected-value generator (op_dsl.py:126-154).  Its CPU pipeline
    // accumulates in the narrow type instead (MindSporeToLinalg.cpp:1344, 1401-1426); descriptions that need
    // that behaviour pinned should cast explicitly.
    Ref src = buffer(n.in[0]), dst = buffer(n.out);
    if (narrow) {
      Ref wide_in, wide_out;
      wide_in.ws_off = (int64_t)ws;
      ws += ((size_t)x.numel() * 4 + 255) / 256 * 256;
      wide_out.ws_off = (int64_t)ws;
      ws += ((size_t)ov.numel() * 4 + 255) / 256 * 256;
      add_convert(src, (int)x.dt, wide_in, (int)DT::F32, x.numel());
      pending_narrow = true;
      narrow_src = wide_out;
      narrow_dst = dst;
      narrow_dt = (int)ov.dt;
      narrow_n = ov.numel();
      src = wide_in;
      dst = wide_out;
    }
    std::vector<bool> red(x.shape.size(), false);
    for (auto a : n.axes) red[a] = true;
    // runs of adjacent reduced axes (extent-1 axes neither break nor make a run); several runs are folded one after
    // the other, the last run first, through float32 temporaries
    std::vector<int64_t> shape = x.shape;
    std::vector<std::vector<size_t>> runs;
    {
      bool open = false;
      for (size_t i = 0; i < shape.size(); ++i) {
        if (shape[i] == 1) continue;
        if (red[i]) {
          if (!open) runs.emplace_back();
          runs.back().push_back(i);
          open = true;
        } else {
          open = false;
        }
      }
    }
    if (runs.empty()) runs.emplace_back();  // nothing but extent-1 axes: a copy through the reduction kernel
    Step st;
    for (size_t ri = runs.size(); ri-- > 0;) {
      std::vector<bool> in_run(shape.size(), false);
      for (size_t d : runs[ri]) in_run[d] = true;
      int64_t outer = 1, len = 1, inner = 1;
      int phase = 0;
      for (size_t i = 0; i < shape.size(); ++i) {
        if (shape[i] == 1) continue;
        if (in_run[i]) {
          phase = 1;
          len *= shape[i];
        } else {
          if (phase == 1) phase = 2;
          (phase == 0 ? outer : inner) *= shape[i];
        }
      }
      Ref to = dst;
      if (ri > 0) {  // more runs to go: this pass writes a temporary
        to = Ref();
        to.ws_off = (int64_t)ws;
        ws += ((size_t)(outer * inner) * 4 + 255) / 256 * 256;
      }
      st = Step();
      st.red_op = op;
      st.red_outer = outer;
      st.red_len = len;
      st.red_inner = inner;
      st.a = src;
      st.out = to;
      if (inner == 1 && outer == 1) {
        st.kind = StepK::ReduceAll;
        st.kernel_name = "reduce_all_f32";
        st.scratch.ws_off = (int64_t)ws;
        ws += (reduce_all_workspace(sm_count) + 255) / 256 * 256;
      } else if (inner == 1) {
        st.kind = StepK::ReduceRow;
        st.kernel_name = "reduce_row_f32";
      } else {
        st.kind = StepK::ReduceCol;
        st.kernel_name = "reduce_col_f32";
        if (outer > 4096) throw Unsupported("batched column reduction with more than 4096 batches");
        st.red_batch_in = len * inner;
        st.red_batch_out = inner;
        st.scratch.ws_off = (int64_t)ws;
        ws += (reduce_col_workspace(len, inner, sm_count) + 255) / 256 * 256;
      }
      for (size_t d : runs[ri]) shape[d] = 1;
      src = to;
      if (ri > 0) plan.steps.push_back(std::move(st));
    }
    plan.steps.push_back(std::move(st));
    if (pending_narrow) {
      add_convert(narrow_src, (int)DT::F32, narrow_dst, narrow_dt, narrow_n);
      pending_narrow = false;
    }
  }

  bool pending_narrow = false;
  Ref narrow_src, narrow_dst;
  int narrow_dt = 0;
  int64_t narrow_n = 0;

  // one elementwise launch that converts n elements from one type to another (Cast semantics)
  void add_convert(const Ref& from, int from_dt, const Ref& to, int to_dt, int64_t n) {
    Step st;
    st.kind = StepK::Ew;
    st.kernel_name = "ew_generic";
    EwProgram& P = st.ew;
    std::memset(&P, 0, sizeof(P));
    P.rank = 1;
    P.n = n;
    P.shape[0] = n;
    P.n_in = 1;
    P.in[0].dt = from_dt;
    P.in[0].kind = EWI_FULL;
    P.in[0].reg = 0;
    EwInstr ins;
    std::memset(&ins, 0, sizeof(ins));
    ins.op = EW_CAST;
    ins.dt = (uint8_t)to_dt;
    ins.cls = cls_of((DT)to_dt);
    ins.src_cls = cls_of((DT)from_dt);
    ins.a = 0;
    ins.dst = 1;
    P.instr[0] = ins;
    P.n_instr = 1;
    P.n_out = 1;
    P.out[0].dt = to_dt;
    P.out[0].kind = EWI_FULL;
    P.out[0].reg = 1;
    P.n_reg = 2;
    st.ew_in.push_back(from);
    st.ew_out.push_back(to);
    plan.steps.push_back(std::move(st));
  }

  void add_transpose(const Node& n) {
    const std::vector<int64_t>& xs = g.v(n.in[0]).shape;
    const size_t R = xs.size();
    std::vector<int64_t> xstride(R, 1);
    for (int i = (int)R - 2; i >= 0; --i) xstride[i] = xstride[i + 1] * xs[i + 1];
    std::vector<int64_t> oshape, istride, src_axis;
    for (size_t i = 0; i < R; ++i) {
      int64_t ax = n.perm[i];
      if (xs[ax] == 1) continue;
      if (!src_axis.empty() && src_axis.back() + 1 == ax) {
        oshape.back() *= xs[ax];
        istride.back() = xstride[ax];
        src_axis.back() = ax;
      } else {
        oshape.push_back(xs[ax]);
        istride.push_back(xstride[ax]);
        src_axis.push_back(ax);
      }
    }
    if (oshape.empty()) {
      oshape.push_back(1);
      istride.push_back(1);
    }
    if (oshape.size() > 6) throw Unsupported("transpose of more than 6 independent axes");
    Step st;
    st.kind = StepK::Transpose;
    st.kernel_name = "transpose_nd";
    st.a = buffer(n.in[0]);
    st.out = buffer(n.out);
    st.tp.rank = (int)oshape.size();
    for (size_t i = 0; i < oshape.size(); ++i) {
      st.tp.out_shape[i] = oshape[i];
      st.tp.in_stride[i] = istride[i];
    }
    st.tp.esize = (int)dt_size(g.v(n.in[0]).dt);
    plan.steps.push_back(std::move(st));
  }

  // Concat: one copy launch per input, each writing its slab of the output
  void add_concat(const Node& n) {
    const Value& out = g.v(n.out);
    if (!ew_dtype_ok(out.dt)) throw Unsupported(std::string("generic elementwise kernel: type ") + dt_name(out.dt));
    const size_t R = out.shape.size();
    if (R > (size_t)kEwMaxRank || n.axis < 0 || n.axis >= (int64_t)R) throw Unsupported("Concat rank/axis");
    std::vector<int64_t> ostride(R, 1);
    for (int d = (int)R - 2; d >= 0; --d) ostride[d] = ostride[d + 1] * out.shape[d + 1];
    int64_t pos = 0;
    for (int vid : n.in) {
      const Value& x = g.v(vid);
      if (x.shape.size() != R || x.dt != out.dt) throw Unsupported("Concat operands must share rank and type");
      Step st;
      st.kind = StepK::Ew;
      st.kernel_name = "ew_generic";
      EwProgram& P = st.ew;
      std::memset(&P, 0, sizeof(P));
      P.rank = (int)R;
      P.n = x.numel();
      for (size_t d = 0; d < R; ++d) P.shape[d] = x.shape[d];
      P.n_in = 1;
      P.in[0].dt = (int)x.dt;
      P.in[0].kind = EWI_FULL;
      P.in[0].reg = 0;
      P.n_out = 1;
      P.out[0].dt = (int)out.dt;
      P.out[0].kind = EWI_STRIDED;
      P.out[0].reg = 0;
      P.out[0].offset = pos * ostride[n.axis];
      for (size_t d = 0; d < R; ++d) P.out[0].stride[d] = ostride[d];
      P.n_reg = 1;
      st.ew_in.push_back(buffer(vid));
      st.ew_out.push_back(buffer(n.out));
      plan.steps.push_back(std::move(st));
      pos += x.shape[n.axis];
    }
    if (pos != out.shape[n.axis]) throw JsonError("Concat extents do not add up to the output");
  }

  void add_gather(const Node& n) {
    const Value& data = g.v(n.in[0]);
    const Value& idx = g.v(n.in[1]);
    if (idx.dt != DT::I32 && idx.dt != DT::I64) throw Unsupported("Gather indices must be int32 or int64");
    if (n.axis < 0 || n.axis >= (int64_t)data.shape.size()) throw JsonError("Gather axis out of range");
    Step st;
    st.kind = StepK::Gather;
    st.kernel_name = "gather_rows";
    st.a = buffer(n.in[0]);
    st.b = buffer(n.in[1]);
    st.out = buffer(n.out);
    for (int64_t i = 0; i < n.axis; ++i) st.ix_outer *= data.shape[i];
    st.ix_dim = data.shape[n.axis];
    for (size_t i = n.axis + 1; i < data.shape.size(); ++i) st.ix_inner *= data.shape[i];
    st.ix_n = idx.numel();
    st.ix_esize = (int)dt_size(data.dt);
    st.ix_idx64 = idx.dt == DT::I64;
    if (g.v(n.out).numel() != st.ix_outer * st.ix_n * st.ix_inner) throw JsonError("Gather output shape");
    plan.steps.push_back(std::move(st));
  }

  void add_argmax(const Node& n) {
    const Value& x = g.v(n.in[0]);
    const Value& out = g.v(n.out);
    if (x.dt != DT::F32 && x.dt != DT::F16 && x.dt != DT::BF16 && x.dt != DT::I32)
      throw Unsupported(std::string("ArgMax over ") + dt_name(x.dt));
    if (out.dt != DT::I32 && out.dt != DT::I64) throw Unsupported("ArgMax result must be int32 or int64");
    Step st;
    st.kind = StepK::ArgMax;
    st.kernel_name = "argmax_axis";
    st.a = buffer(n.in[0]);
    st.out = buffer(n.out);
    for (int64_t i = 0; i < n.axis; ++i) st.ix_outer *= x.shape[i];
    st.ix_dim = x.shape[n.axis];
    for (size_t i = n.axis + 1; i < x.shape.size(); ++i) st.ix_inner *= x.shape[i];
    st.ix_esize = (int)x.dt;  // carries the element type of the data
    st.ix_idx64 = out.dt == DT::I64;
    if (out.numel() != st.ix_outer * st.ix_inner) throw JsonError("ArgMax output shape");
    plan.steps.push_back(std::move(st));
  }

  // Pad = fill the whole output with the constant, then copy the input into its window
  void add_pad(const Node& n) {
    const Value& x = g.v(n.in[0]);
    const Value& out = g.v(n.out);
    if (!ew_dtype_ok(out.dt) || x.dt != out.dt) throw Unsupported(std::string("Pad of ") + dt_name(out.dt));
    const size_t R = out.shape.size();
    if (R > (size_t)kEwMaxRank || x.shape.size() != R) throw Unsupported("Pad rank");
    std::vector<int64_t> ostride(R, 1);
    for (int d = (int)R - 2; d >= 0; --d) ostride[d] = ostride[d + 1] * out.shape[d + 1];
    int64_t off = 0;
    for (size_t d = 0; d < R; ++d) {
      if (out.shape[d] != x.shape[d] + n.pad_low[d] + n.pad_high[d]) throw JsonError("Pad output shape");
      off += n.pad_low[d] * ostride[d];
    }
    {
      Step st;
      st.kind = StepK::Ew;
      st.kernel_name = "ew_generic";
      EwProgram& P = st.ew;
      std::memset(&P, 0, sizeof(P));
      P.rank = 1;
      P.n = out.numel();
      P.shape[0] = P.n;
      P.n_const = 1;
      if (out.dt == DT::F64) {
        uint64_t b;
        const double dv = n.pad_value;
        std::memcpy(&b, &dv, 8);
        P.const_bits[0] = (uint32_t)b;
        P.const_hi[0] = (uint32_t)(b >> 32);
        P.const_f64[0] = 1;
      } else {
        P.const_bits[0] = const_bits(n.pad_value, out.dt);
      }
      P.const_reg[0] = 0;
      P.n_out = 1;
      P.out[0].dt = (int)out.dt;
      P.out[0].kind = EWI_FULL;
      P.out[0].reg = 0;
      P.n_reg = 1;
      st.ew_out.push_back(buffer(n.out));
      plan.steps.push_back(std::move(st));
    }
    Step st;
    st.kind = StepK::Ew;
    st.kernel_name = "ew_generic";
    EwProgram& P = st.ew;
    std::memset(&P, 0, sizeof(P));
    P.rank = (int)R;
    P.n = x.numel();
    for (size_t d = 0; d < R; ++d) P.shape[d] = x.shape[d];
    P.n_in = 1;
    P.in[0].dt = (int)x.dt;
    P.in[0].kind = EWI_FULL;
    P.in[0].reg = 0;
    P.n_out = 1;
    P.out[0].dt = (int)out.dt;
    P.out[0].kind = EWI_STRIDED;
    P.out[0].reg = 0;
    P.out[0].offset = off;
    for (size_t d = 0; d < R; ++d) P.out[0].stride[d] = ostride[d];
    P.n_reg = 1;
    st.ew_in.push_back(buffer(n.in[0]));
    st.ew_out.push_back(buffer(n.out));
    plan.steps.push_back(std::move(st));
  }

  void add_segment_sum(const Node& n) {
    const Value& data = g.v(n.in[0]);
    const Value& ids = g.v(n.in[1]);
    if (data.dt != g.v(n.out).dt || (data.dt != DT::F32 && data.dt != DT::I32 && data.dt != DT::F16 && data.dt != DT::BF16))
      throw Unsupported("UnsortedSegmentSum over float32, float16, bfloat16 or int32 (data and result of one type)");
    if (ids.dt != DT::I32 && ids.dt != DT::I64) throw Unsupported("segment ids must be int32 or int64");
    Step st;
    st.kind = StepK::SegmentSum;
    st.kernel_name = "segment_sum";
    st.ix_esize = (int)data.dt;  // the element type of data and result
    st.a = buffer(n.in[0]);
    st.b = buffer(n.in[1]);
    st.out = buffer(n.out);
    st.ix_n = ids.numel();
    if (st.ix_n == 0 || data.numel() % st.ix_n) throw JsonError("UnsortedSegmentSum: ids do not divide the data");
    st.ix_inner = data.numel() / st.ix_n;
    st.ix_segments = n.num_segments;
    st.ix_idx64 = ids.dt == DT::I64;
    if (g.v(n.out).numel() != st.ix_segments * st.ix_inner) throw JsonError("UnsortedSegmentSum output shape");
    plan.steps.push_back(std::move(st));
  }

  // Epilogues the matmul kernels apply to their accumulators: bias[N] added in float32, max(., 0), conversion to the
  // operand type.  Found before planning, so that the ops they replace (and a Cast that only widens the bias) are
  // skipped wherever they stand in the op list.
  struct Epilogue {
    int bias = -1;  // value id of the bias as it lies in memory
    int relu = 0;
    int out = -1;   // value the kernel writes instead of the MatMul's own result
  };
  std::map<int, Epilogue> epilogue;  // MatMul node index -> epilogue
  std::set<int> eaten;               // node indices folded into a matmul launch

  bool sole_user(int vid, int* user) const {
    const Value& v = g.v(vid);
    if (v.output_index >= 0 || v.users.size() != 1) return false;
    for (auto& kv : alias)
      if (kv.second == vid) return false;
    *user = v.users[0];
    return true;
  }

  void plan_matmul_epilogues() {
    for (size_t i = 0; i < g.nodes.size(); ++i) {
      const Node& n = g.nodes[i];
      if (n.kind != OpK::MatMul || n.transpose_a) continue;
      const Value& a = g.v(n.in[0]);
      if (g.v(n.out).dt != DT::F32 || a.shape.size() != 2) continue;
      const DT in_dt = a.dt;
      const int64_t N = g.v(n.out).shape.back();
      Epilogue e;
      std::vector<int> taken;
      int cur = n.out, u;
      if (sole_user(cur, &u) && g.nodes[u].kind == OpK::Add) {
        const Node& add = g.nodes[u];
        const int other = add.in[0] == cur ? add.in[1] : add.in[0];
        const Value& ov = g.v(other);
        int src = -1, cast_node = -1;
        if (ov.input_index >= 0 && ov.dt == DT::F32) {
          src = other;
        } else if (ov.producer >= 0 && g.nodes[ov.producer].kind == OpK::Cast && ov.dt == DT::F32 &&
                   ov.users.size() == 1 && ov.output_index < 0) {
          const int s0 = g.nodes[ov.producer].in[0];
          if (g.v(s0).input_index >= 0 && g.v(s0).dt == in_dt && in_dt != DT::F32) {
            src = s0;
            cast_node = ov.producer;
          }
        }
        if (src >= 0 && add.in[0] != add.in[1] && ov.numel() == N && ov.shape.back() == N &&
            g.v(add.out).shape == g.v(n.out).shape) {
          e.bias = src;
          taken.push_back(u);
          if (cast_node >= 0) taken.push_back(cast_node);
          cur = add.out;
        }
      }
      if (sole_user(cur, &u) && g.nodes[u].kind == OpK::Maximum) {
        const Node& mx = g.nodes[u];
        const int other = mx.in[0] == cur ? mx.in[1] : mx.in[0];
        const Value& ov = g.v(other);
        if (ov.is_const && ov.cval.size() == 1 && ov.cval[0] == 0.0 && mx.in[0] != mx.in[1]) {
          e.relu = 1;
          taken.push_back(u);
          cur = mx.out;
        }
      }
      if (in_dt != DT::F32 && sole_user(cur, &u) && g.nodes[u].kind == OpK::Cast && g.v(g.nodes[u].out).dt == in_dt) {
        taken.push_back(u);
        cur = g.nodes[u].out;
        // max(., 0) after the conversion equals the conversion after max(., 0): rounding is monotonic and keeps 0
        if (!e.relu && sole_user(cur, &u) && g.nodes[u].kind == OpK::Maximum) {
          const Node& mx = g.nodes[u];
          const int other = mx.in[0] == cur ? mx.in[1] : mx.in[0];
          const Value& ov = g.v(other);
          if (ov.is_const && ov.cval.size() == 1 && ov.cval[0] == 0.0 && mx.in[0] != mx.in[1]) {
            e.relu = 1;
            taken.push_back(u);
            cur = mx.out;
          }
        }
      }
      if (taken.empty()) continue;
      e.out = cur;
      epilogue[(int)i] = e;
      eaten.insert(taken.begin(), taken.end());
    }
  }

  void add_matmul(const Node& n, int node_index) {
    if (n.kind == OpK::BatchMatMul) {
      add_batch_matmul(n);
      return;
    }
    if (n.transpose_a) throw Unsupported("MatMul with transpose_a is rejected (as by the reference lowering)");
    const Value& a = g.v(n.in[0]);
    const Value& b = g.v(n.in[1]);
    auto ep = epilogue.find(node_index);
    const int out_vid = ep != epilogue.end() ? ep->second.out : n.out;
    const Value& o = g.v(out_vid);
    if ((a.dt != DT::BF16 && a.dt != DT::F16 && a.dt != DT::F32) || b.dt != a.dt || a.shape.size() != 2 ||
        b.shape.size() != 2)
      throw Unsupported("only 2-D bfloat16 / float16 / float32 MatMul is placed");
    if (o.dt != DT::F32 && o.dt != a.dt) throw Unsupported("MatMul result type");
    MatmulParams p;
    p.M = a.shape[0];
    p.K = a.shape[1];
    p.transpose_b = n.transpose_b;
    p.N = n.transpose_b ? b.shape[0] : b.shape[1];
    p.out_dt = (int)o.dt;
    p.in_dt = (int)a.dt;
    p.bias_dt = (int)DT::F32;
    if (ep != epilogue.end()) {
      p.relu = ep->second.relu;
      if (ep->second.bias >= 0) {
        p.has_bias = 1;
        p.bias_dt = (int)g.v(ep->second.bias).dt;
      }
    }
    const char* why = nullptr;
    if (a.dt != DT::F32 && !matmul_bf16_supported(p, &why))
      throw Unsupported(std::string("matmul shape not placed: ") + why);
    Step st;
    st.kind = StepK::Matmul;
    st.kernel_name = a.dt == DT::F32 ? "sgemm_f32" : "matmul_bf16_tcgen05";
    st.a = buffer(n.in[0]);
    st.b = buffer(n.in[1]);
    if (p.has_bias) st.c = buffer(ep->second.bias);
    st.out = buffer(out_vid);
    st.mm = p;
    plan.flops += 2 * p.M * p.N * p.K;
    plan.steps.push_back(std::move(st));
  }

  // Decides, before any buffer is assigned, which Reshape ops are views and which need a copy, and binds the
  // buffer of a viewed intermediate to the graph output that views it.
  std::set<int> reshape_copy;  // node indices
  void plan_reshapes() {
    std::map<int, int> bound_output;  // root value -> output value already bound to it
    for (size_t i = 0; i < g.nodes.size(); ++i) {
      const Node& n = g.nodes[i];
      if (n.kind != OpK::Reshape) continue;
      const int r = root(n.in[0]);
      const Value& rv = g.v(r);
      const bool out_is_output = g.v(n.out).output_index >= 0;
      const bool root_is_io = rv.input_index >= 0 || rv.output_index >= 0;
      if (out_is_output && (root_is_io || bound_output.count(r))) {
        reshape_copy.insert((int)i);  // two caller buffers must hold the same values
        continue;
      }
      alias[n.out] = n.in[0];
      if (out_is_output) {
        bound_output[r] = n.out;
        where[r] = arg_ref(n.out);  // the producer of the viewed value writes into the output directly
      }
    }
  }

  // BatchMatMul: one launch, the batch entry is a tile coordinate (leading dims of both operands must agree, or the
  // right operand may be 2-D and shared)
  void add_batch_matmul(const Node& n) {
    if (n.transpose_a) throw Unsupported("BatchMatMul with transpose_a is rejected (as by the reference lowering)");
    const Value& a = g.v(n.in[0]);
    const Value& b = g.v(n.in[1]);
    const Value& o = g.v(n.out);
    if ((a.dt != DT::BF16 && a.dt != DT::F16 && a.dt != DT::F32) || b.dt != a.dt || a.shape.size() < 2 ||
        b.shape.size() < 2)
      throw Unsupported("only bfloat16 / float16 / float32 BatchMatMul is placed");
    if (o.dt != DT::F32 && o.dt != a.dt) throw Unsupported("BatchMatMul result type");
    const size_t ra = a.shape.size(), rb = b.shape.size();
    int64_t batch = 1;
    for (size_t i = 0; i + 2 < ra; ++i) batch *= a.shape[i];
    int64_t bbatch = 1;
    for (size_t i = 0; i + 2 < rb; ++i) bbatch *= b.shape[i];
    if (bbatch != batch && bbatch != 1) throw Unsupported("BatchMatMul operands with different batch extents");
    if (batch > (1 << 20)) throw Unsupported("BatchMatMul with more than 2^20 batch entries");
    MatmulParams p;
    p.M = a.shape[ra - 2];
    p.K = a.shape[ra - 1];
    p.transpose_b = n.transpose_b;
    p.N = n.transpose_b ? b.shape[rb - 2] : b.shape[rb - 1];
    // the launch writes batch * M * N elements: the declared result must be exactly that (a result whose batch
    // differs from the left operand's, e.g. after an inconsistent split over ranks, would be overrun)
    if (o.numel() != batch * p.M * p.N) throw Unsupported("BatchMatMul result does not hold batch x M x N elements");
    p.out_dt = (int)o.dt;
    p.in_dt = (int)a.dt;
    p.bias_dt = (int)DT::F32;
    const char* why = nullptr;
    const bool f32 = a.dt == DT::F32;
    if (!f32 && !matmul_bf16_supported(p, &why)) throw Unsupported(std::string("matmul shape not placed: ") + why);
    if (!f32 && ((p.M * p.K) % 8 || (p.K * p.N) % 8 || (p.M * p.N) % 8))
      throw Unsupported("BatchMatMul slices must stay 16-byte aligned");
    Step st;
    st.kind = StepK::Matmul;
    st.kernel_name = f32 ? "sgemm_f32" : "matmul_bf16_tcgen05";
    st.a = buffer(n.in[0]);
    st.b = buffer(n.in[1]);
    st.out = buffer(n.out);
    st.mm = p;
    st.mm_batch = batch;
    st.mm_stride_a = p.M * p.K * (int64_t)dt_size(a.dt);
    st.mm_stride_b = bbatch == 1 ? 0 : p.K * p.N * (int64_t)dt_size(a.dt);
    st.mm_stride_o = p.M * p.N * (int64_t)dt_size(o.dt);
    plan.flops += 2 * p.M * p.N * p.K * batch;
    plan.steps.push_back(std::move(st));
  }

  Plan run() {
    plan_reshapes();
    plan_matmul_epilogues();
    // Small elementwise ops on the region's inputs (a Cast of a bias vector, say) go first: between two ops of the
    // large iteration shape they would close the open group and force its values through memory.
    std::vector<size_t> order;
    {
      int64_t largest = 1;
      for (auto& v : g.values) largest = std::max(largest, v.numel());
      std::vector<size_t> later;
      std::set<int> early_nodes;  // chains of such ops too: an operand may be the result of an earlier early op
      for (size_t i = 0; i < g.nodes.size(); ++i) {
        const Node& n = g.nodes[i];
        bool early = opk_is_elementwise(n.kind) && n.kind != OpK::AddN && g.v(n.out).numel() * 4 <= largest;
        for (int vid : n.in) {
          const Value& rv = g.v(root(vid));  // also through views
          early = early && (g.v(vid).is_const || rv.input_index >= 0 || (rv.producer >= 0 && early_nodes.count(rv.producer)));
        }
        if (early) early_nodes.insert((int)i);
        (early ? order : later).push_back(i);
      }
      order.insert(order.end(), later.begin(), later.end());
    }
    for (size_t i : order) {
      const Node& n = g.nodes[i];
      if (eaten.count((int)i)) continue;  // runs inside a matmul launch
      if (n.kind == OpK::Reshape && !reshape_copy.count((int)i)) continue;  // a view
      const bool view_copy = n.kind == OpK::Tile || n.kind == OpK::Slice || n.kind == OpK::StridedSlice;
      if (view_copy && produced_in_group(n.in[0])) flush_group();  // the source is read from memory
      if (n.kind == OpK::Concat) {
        flush_group();
        add_concat(n);
        continue;
      }
      if (opk_is_elementwise(n.kind) || n.kind == OpK::BroadcastTo || n.kind == OpK::Reshape || view_copy ||
          n.kind == OpK::Assign) {
        const std::vector<int64_t>& S = g.v(n.out).shape;
        if (!group.empty() && group_shape != S) flush_group();
        // an operand that views a value still being computed in the open group must be materialised first
        for (int vid : n.in)
          if (!group.empty() && !produced_in_group(vid) && produced_in_group(root(vid))) flush_group();
        // a Reshape copy consumes its source by flat index: the source must have the group's element order
        if (n.kind == OpK::Reshape && produced_in_group(n.in[0]) && g.v(n.in[0]).shape != S) flush_group();
        if (!group.empty() && !group_fits_with((int)i)) flush_group();
        if (group.empty()) group_shape = S;
        group.push_back((int)i);
        continue;
      }
      flush_group();
      if (opk_is_reduce(n.kind)) add_reduce(n);
      else if (n.kind == OpK::Transpose) add_transpose(n);
      else if (n.kind == OpK::MatMul || n.kind == OpK::BatchMatMul) add_matmul(n, (int)i);
      else if (n.kind == OpK::Gather) add_gather(n);
      else if (n.kind == OpK::ArgMax) add_argmax(n);
      else if (n.kind == OpK::Pad) add_pad(n);
      else if (n.kind == OpK::UnsortedSegmentSum) add_segment_sum(n);
      else throw Unsupported(std::string("operator '") + n.name + "' is not supported");
    }
    flush_group();
    plan.workspace_bytes = ws;
    return std::move(plan);
  }
};

}  // namespace

Plan build_generic_plan(const Graph& g, int sm_count) {
  Builder b(g, sm_count);
  Plan p = b.run();
  if (p.steps.empty()) throw Unsupported("the region has no computing op");
  switch (g.op_class) {
    case OpClass::Elementwise: p.klass = "elementwise"; break;
    case OpClass::Broadcast: p.klass = "broadcast"; break;
    case OpClass::Reshape: p.klass = "reshape"; break;
    case OpClass::Transpose: p.klass = "transpose"; break;
    case OpClass::Matmul: p.klass = "matmul"; break;
    default:
      p.klass = g.reduce_dir == ReduceDir::All ? "reduce_all" : g.reduce_dir == ReduceDir::Y ? "reduce_y" : "reduce_x";
  }
  return p;
}

}  // namespace akgb
