// Recognises regions of the reduce-X class that can run as ONE generated kernel with a row kept in registers.
//
// The reference fuses such regions (elementwise ops around reductions along the last axis) into one kernel through its
// polyhedral schedule (reduce-X template: akg-mlir/lib/Dialect/Affine/Analysis/GpuTemplateTilingSolver.cpp:458-542,
// block-level combine: GpuUseAllReduceWithAtomicReturn.cpp:168-224).  The hand-written LayerNorm and softmax templates
// cover two spellings; this builder accepts any op list made of elementwise ops, BroadcastTo, view Reshapes and
// reductions over the last axis whose tensors are [rows, cols], [rows], [cols], scalars or a [m, cols] tensor shared by
// rows modulo m, and hands it to the run-time generator (ew_jit.cpp::row_jit_*).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <set>

#include "hostconv.hpp"
#include "plan.hpp"

namespace akgb {

bool ew_opcode_of(OpK k, EwOp* op);           // planner.cpp
uint32_t ew_const_bits(double v, DT d);       // planner.cpp
bool ew_type_ok(DT d);                        // planner.cpp

namespace {

EwClass cls_of(DT d) { return dt_is_float(d) ? EWC_FLOAT : (d == DT::Bool ? EWC_BOOL : EWC_INT); }

std::vector<int64_t> strip_leading_ones(std::vector<int64_t> s) {
  while (s.size() > 1 && s.front() == 1) s.erase(s.begin());
  return s;
}

}  // namespace

bool build_row_program(const Graph& g, RowProgram* out, std::vector<int>* in_values, std::vector<int>* out_values,
                       bool col_mode, const std::map<int, std::pair<int64_t, int64_t>>* row_index, bool allow_col_sums) {
  if (g.dynamic || g.nodes.empty()) return false;
  // the row shape comes from the first reduction
  const Node* first_red = nullptr;
  for (auto& n : g.nodes)
    if (opk_is_reduce(n.kind)) {
      first_red = &n;
      break;
    }
  if (!first_red) return false;
  const std::vector<int64_t>& S = g.v(first_red->in[0]).shape;
  if (S.empty()) return false;
  if (col_mode) {
    // column mode works on the caller's 2-D view [rows, cols]: from the first reduction on every op is a reduction over
    // the rows, and those are exactly the region's results
    if (S.size() != 2) return false;
    size_t n_red = 0;
    bool seen = false;
    for (auto& n : g.nodes) {
      seen = seen || &n == first_red;
      if (seen && !opk_is_reduce(n.kind)) return false;
      n_red += seen;
    }
    if (n_red != g.outputs.size() || n_red > 4) return false;
  }
  const int64_t C = S.back();
  int64_t R = 1;
  for (size_t i = 0; i + 1 < S.size(); ++i) R *= S[i];
  if (C < 2 || R < 1 || C > (1 << 20)) return false;
  const std::vector<int64_t> S_lead(S.begin(), S.end() - 1);

  RowProgram P;
  P.rows = R;
  P.cols = C;
  std::map<int, int> val_of;  // graph value -> program value
  std::map<int, int> col_sum_of;  // region result -> the per-element value it sums over all rows
  std::set<int> view_of_col_sum;  // re-views of such sums: no instruction of their own
  auto new_val = [&](bool full) {
    P.val_full.push_back(full ? 1 : 0);
    return P.n_val++;
  };
  // class of a tensor by its shape: 0 full, 1 row, 2 col, 3 scalar, 4 rowmod, -1 none
  auto shape_kind = [&](const std::vector<int64_t>& shp, int64_t* mod_rows) -> int {
    int64_t n = 1;
    for (auto e : shp) n *= e;
    if (shp.empty()) return RK_SCALAR;
    if (n == R * C && shp.back() == C) return RK_FULL;
    if (n == 1) return RK_SCALAR;
    if (n == C && shp.back() == C) return RK_COL;
    if (n == R && (shp.back() == 1 || shp.size() + 1 == S.size() || S.size() == 1)) {
      std::vector<int64_t> lead = shp;
      if (lead.back() == 1 && lead.size() > 1) lead.pop_back();
      if (strip_leading_ones(lead) == strip_leading_ones(S_lead) || lead == S_lead) return RK_ROW;
      return -1;
    }
    if (shp.back() == C && n % C == 0 && R % (n / C) == 0) {
      const std::vector<int64_t> t = strip_leading_ones(shp);
      if (t.size() > S.size()) return -1;
      for (size_t i = 0; i < t.size(); ++i)
        if (t[t.size() - 1 - i] != S[S.size() - 1 - i]) return -1;
      *mod_rows = n / C;
      return RK_ROWMOD;
    }
    return -1;
  };
  auto operand = [&](int vid, int* val) -> bool {
    auto it = val_of.find(vid);
    if (it != val_of.end()) {
      *val = it->second;
      return true;
    }
    const Value& v = g.v(vid);
    if (!ew_type_ok(v.dt)) return false;
    if (v.is_const) {
      if (v.cval.size() != 1) return false;
      const int id = new_val(false);
      P.const_val.push_back(id);
      P.const_bits.push_back(ew_const_bits(v.cval[0], v.dt));
      val_of[vid] = id;
      *val = id;
      return true;
    }
    if (v.input_index < 0) return false;  // produced by an op this builder did not take
    int64_t mod_rows = 0;
    int kind = shape_kind(v.shape, &mod_rows);
    RowOperand o;
    if (row_index && row_index->count(vid)) {  // the caller knows how the rows index this operand
      kind = RK_ROW;
      o.row_div = row_index->at(vid).first;
      o.row_mod = row_index->at(vid).second;
    }
    if (kind < 0) return false;
    o.dt = (int)v.dt;
    o.kind = kind;
    o.mod_rows = mod_rows;
    o.val = new_val(kind == RK_FULL || kind == RK_COL || kind == RK_ROWMOD);
    P.in.push_back(o);
    in_values->push_back(vid);
    val_of[vid] = o.val;
    *val = o.val;
    return true;
  };

  for (const Node& n : g.nodes) {
    const Value& ov = g.v(n.out);
    if (view_of_col_sum.count(n.out)) continue;
    if (!ew_type_ok(ov.dt)) return false;
    RowInstr ins;
    ins.dt = (uint8_t)ov.dt;
    ins.cls = cls_of(ov.dt);
    if (opk_is_reduce(n.kind) && col_mode) {
      const Value& x = g.v(n.in[0]);
      if (n.axes.size() != 1 || n.axes[0] != 0 || x.numel() != R * C || x.dt != DT::F32 || ov.dt != DT::F32 ||
          ov.numel() != C)
        return false;
      int src = 0;
      if (!operand(n.in[0], &src) || !P.val_full[src]) return false;
      RowOperand o;
      switch (n.kind) {
        case OpK::ReduceSum: o.red_op = 0; break;
        case OpK::ReduceMax: o.red_op = 1; break;
        case OpK::ReduceMin: o.red_op = 2; break;
        case OpK::ReduceProd: o.red_op = 3; break;
        default: return false;
      }
      if (ov.output_index < 0) return false;
      P.col_reduce = true;
      o.dt = (int)DT::F32;
      o.kind = RK_COL;
      o.val = src;
      P.out.push_back(o);
      out_values->push_back(n.out);
      continue;
    } else if (allow_col_sums && n.kind == OpK::ReduceSum && S.size() >= 2 && n.axes.size() + 1 == S.size() &&
               n.axes.front() == 0 && n.axes.back() == (int64_t)S.size() - 2 && g.v(n.in[0]).numel() == R * C &&
               g.v(n.in[0]).shape.back() == C) {
      // a sum over all rows of a per-element value: a result of its own, written per CTA and folded afterwards
      const Value& x = g.v(n.in[0]);
      int src = 0;
      if (x.dt != DT::F32 || ov.dt != DT::F32 || ov.numel() != C) return false;
      // the result itself, or what a chain of re-views ([1, cols] -> [cols]) makes of it, is a result of the region
      int result = n.out;
      for (int hops = 0; hops < 4 && g.v(result).output_index < 0; ++hops) {
        const Value& rv = g.v(result);
        if (rv.users.size() != 1 || g.nodes[rv.users[0]].kind != OpK::Reshape) return false;
        result = g.nodes[rv.users[0]].out;
        view_of_col_sum.insert(result);
      }
      if (g.v(result).output_index < 0 || !g.v(result).users.empty()) return false;
      if (!operand(n.in[0], &src) || !P.val_full[src] || col_sum_of.size() >= 4) return false;
      col_sum_of[result] = src;
      P.col_sums = true;
      continue;
    } else if (opk_is_reduce(n.kind)) {
      const Value& x = g.v(n.in[0]);
      if (n.axes.size() != 1 || n.axes[0] != (int64_t)x.shape.size() - 1 || x.shape.back() != C || x.numel() != R * C)
        return false;
      switch (n.kind) {
        case OpK::ReduceSum: ins.red_op = 0; break;
        case OpK::ReduceMax: ins.red_op = 1; break;
        case OpK::ReduceMin: ins.red_op = 2; break;
        case OpK::ReduceProd: ins.red_op = 3; break;
        default: return false;
      }
      if (!dt_is_float(x.dt) || ov.dt != x.dt || ov.numel() != R) return false;
      if (!operand(n.in[0], &ins.a) || !P.val_full[ins.a]) return false;
      ins.reduce = true;
      ins.full = false;
      ins.src_cls = EWC_FLOAT;
    } else if (n.kind == OpK::Reshape || n.kind == OpK::BroadcastTo) {
      if (!operand(n.in[0], &ins.a)) return false;
      const bool src_full = P.val_full[ins.a] != 0;
      int64_t dummy = 0;
      const int kind = shape_kind(ov.shape, &dummy);
      if (n.kind == OpK::Reshape) {
        // a view: the class must survive (full stays [.., cols], per-row stays per-row)
        if (src_full ? (ov.numel() != g.v(n.in[0]).numel() || ov.shape.back() != C) : (kind != RK_ROW && kind != RK_SCALAR))
          return false;
        ins.full = src_full;
      } else {
        if (kind != RK_FULL && kind != RK_ROW && kind != RK_SCALAR) return false;
        if (src_full && kind != RK_FULL) return false;
        ins.full = kind == RK_FULL;
      }
      ins.op = EW_COPY;
      ins.src_cls = cls_of(g.v(n.in[0]).dt);
      if (g.v(n.in[0]).dt != ov.dt) return false;
    } else if (opk_is_elementwise(n.kind)) {
      EwOp op;
      if (!ew_opcode_of(n.kind, &op) || n.in.empty() || n.in.size() > 3) return false;
      int regs[3] = {0, 0, 0};
      bool any_full = false;
      for (size_t j = 0; j < n.in.size(); ++j) {
        if (!operand(n.in[j], &regs[j])) return false;
        any_full |= P.val_full[regs[j]] != 0;
      }
      ins.op = (uint8_t)op;
      ins.a = regs[0];
      ins.b = regs[1];
      ins.c = regs[2];
      ins.src_cls = cls_of(g.v(n.in[op == EW_SELECT ? 1 : 0]).dt);
      if (op == EW_CAST && ins.src_cls == EWC_FLOAT && ins.cls == EWC_INT) return false;  // unpinned rounding
      ins.full = any_full;
      int64_t dummy = 0;
      const int kind = shape_kind(ov.shape, &dummy);
      if (kind < 0) return false;
      if (!any_full && kind != RK_ROW && kind != RK_SCALAR) return false;
    } else {
      return false;
    }
    ins.dst = new_val(ins.full);
    val_of[n.out] = ins.dst;
    P.instr.push_back(ins);
    if (P.instr.size() > 160) return false;
  }
  for (int vid : g.outputs) {
    if (col_mode) break;
    const Value& v = g.v(vid);
    if (col_sum_of.count(vid)) {
      RowOperand o;
      o.dt = (int)DT::F32;
      o.kind = RK_COL;
      o.val = col_sum_of[vid];
      o.red_op = 0;
      P.out.push_back(o);
      out_values->push_back(vid);
      continue;
    }
    auto it = val_of.find(vid);
    if (it == val_of.end() || v.producer < 0) return false;  // an input or constant passed through
    RowOperand o;
    o.dt = (int)v.dt;
    o.val = it->second;
    if (P.val_full[o.val]) {
      if (v.numel() != R * C) return false;  // a per-column value computed on the way cannot be a result
      o.kind = RK_FULL;
    } else {
      if (v.numel() != R) return false;
      o.kind = RK_ROW;
    }
    P.out.push_back(o);
    out_values->push_back(vid);
  }
  if (P.in.size() > 12 || P.out.size() > 8 || P.in.empty()) return false;
  bool any_full_in = false;
  for (auto& o : P.in) any_full_in |= o.kind == RK_FULL;
  if (!any_full_in) return false;
  if (P.col_sums) {
    // only next to row-wise work (sums over rows alone are the column kernels' job); the multi-pass schedule keeps the
    // sums of up to 16 384 columns
    bool any_row_reduction = false;
    for (auto& x : P.instr) any_row_reduction |= x.reduce;
    if (!any_row_reduction || (!row_jit_fits_registers(P) && P.cols > 16384)) return false;
  }
  *out = std::move(P);
  return true;
}

}  // namespace akgb
