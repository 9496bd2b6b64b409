// Pattern matcher over the fused region: decides which kernel template(s) run
// it.  Replaces the affine/GPU-dialect mapping of the reference's --gpu-opt
// pipeline (akg-mlir/lib/Pipelines/GPUPipelines/GPUOpt.cpp:45-132).
//
// LayerNorm, GELU and softmax do not arrive as single operators: the JSON
// factory has no entry for them (TranslateToMindsporeDialect.cpp:417-486), so
// they are recognised here from their primitive-op spellings, the same DAG
// shapes mfusion's fusion passes look for
// (mfusion/lib/Dialect/Mfuse/Transforms/Fusion/Passes/Norm/FuseLayerNorm.cc:131-192,
//  .../FuseGelu.cc:159-236, mfusion/include/mfusion/Analysis/DvmFusion/SafeSoftmax/SafeSoftmaxDvmUtils.h:29-41).
// Operand order of commutative ops is free; the association order is not,
// because every op rounds to its declared element type.
#include <algorithm>
#include <cmath>
#include <functional>
#include <set>

#include "hostconv.hpp"
#include "plan.hpp"

namespace akgb {
namespace {

struct M {
  const Graph& g;
  std::set<int> used;  // node indices consumed by the current pattern
  explicit M(const Graph& gr) : g(gr) {}
  M(const M&) = default;
  M& operator=(const M& o) {
    used = o.used;
    return *this;
  }

  int n_inputs() const { return (int)g.inputs.size(); }
  Ref ref_of(int vid) const {
    const Value& v = g.v(vid);
    Ref r;
    if (v.input_index >= 0) r.arg = v.input_index;
    else if (v.output_index >= 0) r.arg = n_inputs() + v.output_index;
    return r;
  }
  bool is_input(int vid) const { return g.v(vid).input_index >= 0; }
  // node producing vid if it has kind k
  const Node* prod(int vid, OpK k) {
    int p = g.v(vid).producer;
    if (p < 0 || g.nodes[p].kind != k) return nullptr;
    return &g.nodes[p];
  }
  void take(const Node* n) { used.insert((int)(n - &g.nodes[0])); }
  bool cst(int vid, double* val) const {
    const Value& v = g.v(vid);
    if (!v.is_const || v.cval.size() != 1) return false;
    *val = v.cval[0];
    return true;
  }
  // binary op with one constant operand (either side when commutative)
  bool bin_const(int vid, OpK k, bool commutative, int* other, double* c) {
    const Node* n = prod(vid, k);
    if (!n || n->in.size() != 2) return false;
    if (cst(n->in[1], c)) {
      *other = n->in[0];
      take(n);
      return true;
    }
    if (commutative && cst(n->in[0], c)) {
      *other = n->in[1];
      take(n);
      return true;
    }
    return false;
  }
  bool bin(int vid, OpK k, int* a, int* b) {
    const Node* n = prod(vid, k);
    if (!n || n->in.size() != 2) return false;
    *a = n->in[0];
    *b = n->in[1];
    take(n);
    return true;
  }
  bool un(int vid, OpK k, int* a) {
    const Node* n = prod(vid, k);
    if (!n || n->in.empty()) return false;
    *a = n->in[0];
    take(n);
    return true;
  }
  // skip view-only ops (Reshape) upwards
  int through_reshape(int vid) {
    for (;;) {
      const Node* n = prod(vid, OpK::Reshape);
      if (!n) return vid;
      take(n);
      vid = n->in[0];
    }
  }
  bool all_used() const { return used.size() == g.nodes.size(); }
};

int64_t prod_of(const std::vector<int64_t>& s, size_t b, size_t e) {
  int64_t n = 1;
  for (size_t i = b; i < e; ++i) n *= s[i];
  return n;
}

int64_t io_bytes(const Graph& g) {
  int64_t b = 0;
  for (int v : g.inputs) b += g.v(v).numel() * (int64_t)dt_size(g.v(v).dt);
  for (int v : g.outputs) b += g.v(v).numel() * (int64_t)dt_size(g.v(v).dt);
  return b;
}

// reduction over the last axis with keep_dims, returning its operand
bool row_reduce(M& m, int vid, OpK k, int* src) {
  const Node* n = m.prod(vid, k);
  if (!n) return false;
  const Value& in = m.g.v(n->in[0]);
  if (n->axes.size() != 1 || n->axes[0] != (int64_t)in.shape.size() - 1) return false;
  // keep_dims or not, the result has one value per row
  *src = n->in[0];
  m.take(n);
  return true;
}

// ---------------------------------------------------------------- LayerNorm --
bool match_layernorm(const Graph& g, Plan& plan) {
  if (g.outputs.empty()) return false;
  M m(g);
  int y = g.outputs[0];
  const Value& yv = g.v(y);
  if (yv.dt != DT::F32 || yv.shape.size() < 2) return false;
  const int64_t cols = yv.shape.back();
  const int64_t rows = yv.numel() / cols;
  auto is_row_vec = [&](int vid) {  // a [cols] (or [1,..,cols]) graph input
    const Value& v = g.v(vid);
    return m.is_input(vid) && v.dt == DT::F32 && v.numel() == cols && v.shape.back() == cols;
  };
  int cur = y, a, b, gamma = -1, beta = -1;
  {
    M probe = m;
    if (probe.bin(cur, OpK::Add, &a, &b) && (is_row_vec(a) || is_row_vec(b))) {
      m = probe;
      beta = is_row_vec(b) ? b : a;
      cur = is_row_vec(b) ? a : b;
    }
  }
  {
    M probe = m;
    if (probe.bin(cur, OpK::Mul, &a, &b) && (is_row_vec(a) || is_row_vec(b))) {
      m = probe;
      gamma = is_row_vec(b) ? b : a;
      cur = is_row_vec(b) ? a : b;
    }
  }
  if (!m.bin(cur, OpK::Mul, &a, &b)) return false;
  // one side is d [rows, cols], the other rstd [rows, 1]
  int d = a, rstd = b;
  if (g.v(a).numel() == rows && g.v(b).numel() == rows * cols) std::swap(d, rstd);
  if (g.v(d).numel() != rows * cols || g.v(rstd).numel() != rows) return false;
  int ve;
  if (!m.un(rstd, OpK::Rsqrt, &ve)) return false;
  int var;
  double eps;
  if (!m.bin_const(ve, OpK::Add, true, &var, &eps)) return false;
  // sum -> mean either as a multiplication by 1/N or as a division by N (the spelling PyTorch's mean decomposes to);
  // a power-of-two N makes the two identical, any other N keeps the division
  auto scaled = [&](int vid, int* src, double* inv, double* divn) {
    *divn = 0.0;
    if (m.bin_const(vid, OpK::Mul, true, src, inv)) return true;
    double c;
    if (!m.bin_const(vid, OpK::Div, false, src, &c) || c <= 0.0) return false;
    int e;
    if (std::frexp(c, &e) == 0.5) *inv = 1.0 / c;
    else *divn = c, *inv = 1.0 / c;
    return true;
  };
  int s2;
  double inv_n2, div_n2;
  if (!scaled(var, &s2, &inv_n2, &div_n2)) return false;
  int sq;
  if (!row_reduce(m, s2, OpK::ReduceSum, &sq)) return false;
  if (!m.bin(sq, OpK::Mul, &a, &b) || a != d || b != d) return false;
  int x, mean;
  if (!m.bin(d, OpK::Sub, &x, &mean)) return false;
  if (!m.is_input(x) || g.v(x).dt != DT::F32) return false;
  int s1;
  double inv_n1, div_n1;
  if (!scaled(mean, &s1, &inv_n1, &div_n1)) return false;
  int x2;
  if (!row_reduce(m, s1, OpK::ReduceSum, &x2) || x2 != x) return false;
  if ((float)inv_n1 != (float)inv_n2 || (float)div_n1 != (float)div_n2) return false;

  // optional extra outputs: mean and var, possibly through a Reshape
  Ref mean_ref, var_ref;
  for (size_t i = 1; i < g.outputs.size(); ++i) {
    int o = g.outputs[i];
    int src = m.through_reshape(o);
    if (src == mean && !mean_ref.valid()) mean_ref = m.ref_of(o);
    else if (src == var && !var_ref.valid()) var_ref = m.ref_of(o);
    else return false;
  }
  if (!m.all_used()) return false;
  // intermediate values other than mean/var must not be graph outputs
  Step st;
  st.kind = StepK::LayerNorm;
  st.kernel_name = "layernorm_rows_f32";
  st.a = m.ref_of(x);
  if (gamma >= 0) st.b = m.ref_of(gamma);
  if (beta >= 0) st.c = m.ref_of(beta);
  st.out = m.ref_of(y);
  st.out2 = mean_ref;
  st.out3 = var_ref;
  st.ln.rows = rows;
  st.ln.cols = cols;
  st.ln.inv_n = (float)inv_n1;
  st.ln.div_n = (float)div_n1;
  st.ln.eps = (float)eps;
  st.ln.has_gamma = gamma >= 0;
  st.ln.has_beta = beta >= 0;
  st.ln.write_mean = mean_ref.valid();
  st.ln.write_var = var_ref.valid();
  plan.klass = "layernorm";
  plan.steps.push_back(st);
  return true;
}

// ------------------------------------------------------------------ Softmax --
bool match_softmax(const Graph& g, Plan& plan) {
  if (g.outputs.size() != 1) return false;
  M m(g);
  int out = g.outputs[0];
  const Value& ov = g.v(out);
  if (ov.shape.empty()) return false;
  if (ov.dt != DT::F16 && ov.dt != DT::F32 && ov.dt != DT::BF16) return false;
  const int64_t cols = ov.shape.back();
  const int64_t rows = ov.numel() / cols;
  int cur = out, t;
  if (ov.dt != DT::F32) {
    if (!m.un(cur, OpK::Cast, &t)) return false;
    cur = t;
  }
  if (g.v(cur).dt != DT::F32) return false;
  int e, sum;
  if (!m.bin(cur, OpK::Div, &e, &sum)) return false;
  int e2;
  if (!row_reduce(m, sum, OpK::ReduceSum, &e2) || e2 != e) return false;
  int sh;
  if (!m.un(e, OpK::Exp, &sh)) return false;
  int s, mx;
  if (!m.bin(sh, OpK::Sub, &s, &mx)) return false;
  int s2;
  if (!row_reduce(m, mx, OpK::ReduceMax, &s2) || s2 != s) return false;
  if (g.v(s).numel() != rows * cols) return false;

  // pre-chain: s = [Add(., mask)]([Mul(., scale)]([Cast](x)))
  int mask = -1;
  DT mask_dt = DT::F32;
  int a, b;
  {
    M probe = m;
    if (probe.bin(s, OpK::Add, &a, &b)) {
      // the mask is a graph input (possibly behind a Cast) that broadcasts against the scores;
      // when both operands qualify, the smaller one is the mask, then the right-hand one
      auto mask_src = [&](int vid, M* trial, int* src) {
        int c = vid, q;
        if (trial->un(c, OpK::Cast, &q)) c = q;
        if (!trial->is_input(c)) return false;
        *src = c;
        return true;
      };
      M pa = probe, pb = probe;
      int sa = -1, sb = -1;
      const bool a_ok = mask_src(a, &pa, &sa), b_ok = mask_src(b, &pb, &sb);
      const bool pick_b = b_ok && (!a_ok || g.v(sb).numel() <= g.v(sa).numel());
      if (pick_b) {
        mask = sb;
        s = a;
        m = pb;
      } else if (a_ok) {
        mask = sa;
        s = b;
        m = pa;
      }
    }
  }
  double scale = 1.0;
  int has_scale = 0;
  {
    M probe = m;
    int other;
    double c;
    if (probe.bin_const(s, OpK::Mul, true, &other, &c)) {
      m = probe;
      s = other;
      scale = c;
      has_scale = 1;
    }
  }
  int x = s;
  if (!m.is_input(x)) {
    int q;
    if (!m.un(x, OpK::Cast, &q) || !m.is_input(q)) return false;
    x = q;
  }
  const Value& xv = g.v(x);
  if (xv.numel() != rows * cols) return false;
  if (xv.dt != DT::F16 && xv.dt != DT::F32 && xv.dt != DT::BF16) return false;
  int64_t mask_rows = 1;
  if (mask >= 0) {
    const Value& mv = g.v(mask);
    mask_dt = mv.dt;
    if (mask_dt != DT::F16 && mask_dt != DT::F32 && mask_dt != DT::BF16) return false;
    if (mv.shape.back() != cols) return false;
    // the mask's dims must be the trailing dims of x (leading 1s allowed)
    std::vector<int64_t> ms = mv.shape;
    while (ms.size() > 1 && ms.front() == 1) ms.erase(ms.begin());
    if (ms.size() > xv.shape.size()) return false;
    for (size_t i = 0; i < ms.size(); ++i)
      if (ms[ms.size() - 1 - i] != xv.shape[xv.shape.size() - 1 - i]) return false;
    mask_rows = mv.numel() / cols;
  }
  if (!m.all_used()) return false;

  Step st;
  st.kind = StepK::Softmax;
  st.kernel_name = "softmax_rows";
  st.a = m.ref_of(x);
  if (mask >= 0) st.b = m.ref_of(mask);
  st.out = m.ref_of(out);
  st.sm.rows = rows;
  st.sm.cols = cols;
  st.sm.in_dt = (int)xv.dt;
  st.sm.out_dt = (int)ov.dt;
  st.sm.mask_dt = (int)mask_dt;
  st.sm.has_scale = has_scale;
  st.sm.has_mask = mask >= 0;
  st.sm.scale = (float)scale;
  st.sm.mask_rows = mask_rows;
  plan.klass = "softmax";
  plan.steps.push_back(st);
  return true;
}

// --------------------------------------------------------------- reductions --
bool match_reduce(const Graph& g, Plan& plan, int sm_count) {
  M m(g);
  std::vector<Step> steps;
  size_t ws = 0;
  std::string klass;
  for (int o : g.outputs) {
    int src = m.through_reshape(o);
    int p = g.v(src).producer;
    if (p < 0) return false;
    const Node& n = g.nodes[p];
    RedOp op;
    switch (n.kind) {
      case OpK::ReduceSum: op = RedOp::Sum; break;
      case OpK::ReduceMax: op = RedOp::Max; break;
      case OpK::ReduceMin: op = RedOp::Min; break;
      case OpK::ReduceProd: op = RedOp::Prod; break;
      default: return false;
    }
    m.take(&n);
    int x = n.in[0];
    // a view change of the input is free
    x = m.through_reshape(x);
    if (!m.is_input(x) || g.v(x).dt != DT::F32 || g.v(o).dt != DT::F32) return false;
    const std::vector<int64_t>& xs = g.v(n.in[0]).shape;
    // reduced axes must form one contiguous range once extent-1 axes are ignored
    std::vector<bool> red(xs.size(), false);
    for (auto a : n.axes) red[a] = true;
    int64_t outer = 1, len = 1, inner = 1;
    int phase = 0;  // 0 outer, 1 reduce, 2 inner
    for (size_t i = 0; i < xs.size(); ++i) {
      if (xs[i] == 1) continue;
      if (red[i]) {
        if (phase == 2) return false;
        phase = 1;
        len *= xs[i];
      } else {
        if (phase == 1) phase = 2;
        if (phase == 0) outer *= xs[i];
        else inner *= xs[i];
      }
    }
    Step st;
    st.red_op = op;
    st.red_outer = outer;
    st.red_len = len;
    st.red_inner = inner;
    st.a = m.ref_of(x);
    st.out = m.ref_of(o);
    if (inner == 1 && outer == 1) {
      st.kind = StepK::ReduceAll;
      st.kernel_name = "reduce_all_f32";
      st.scratch.ws_off = (int64_t)ws;
      ws += (reduce_all_workspace(sm_count) + 255) / 256 * 256;
      if (klass.empty()) klass = "reduce_all";
    } else if (inner == 1) {
      st.kind = StepK::ReduceRow;
      st.kernel_name = "reduce_row_f32";
      if (klass.empty()) klass = "reduce_x";
    } else {
      st.kind = StepK::ReduceCol;
      st.kernel_name = "reduce_col_f32";
      if (outer != 1) return false;  // batched column reductions: not yet placed
      st.scratch.ws_off = (int64_t)ws;
      ws += (reduce_col_workspace(len, inner, sm_count) + 255) / 256 * 256;
      if (klass.empty()) klass = "reduce_y";
    }
    steps.push_back(st);
  }
  if (!m.all_used()) return false;
  // a column reduction and a reduction of all elements of the same tensor share one pass over it
  if (steps.size() == 2) {
    int ci = steps[0].kind == StepK::ReduceCol ? 0 : steps[1].kind == StepK::ReduceCol ? 1 : -1;
    int ai = steps[0].kind == StepK::ReduceAll ? 0 : steps[1].kind == StepK::ReduceAll ? 1 : -1;
    if (ci >= 0 && ai >= 0 && steps[ci].a.arg == steps[ai].a.arg && steps[ci].red_outer == 1 &&
        steps[ai].red_len == steps[ci].red_len * steps[ci].red_inner && reduce_col_dual_supported(steps[ci].red_inner, nullptr)) {
      Step st = steps[ci];
      st.kind = StepK::ReduceColDual;
      st.kernel_name = "reduce_col_dual_f32";
      st.red_op2 = steps[ai].red_op;
      st.out2 = steps[ai].out;
      st.scratch.ws_off = 0;
      ws = (std::max(reduce_col_dual_workspace(st.red_len, st.red_inner, sm_count),
                     reduce_col_workspace(st.red_len, st.red_inner, sm_count) + reduce_all_workspace(sm_count)) + 255) / 256 * 256;
      steps.assign(1, st);
    }
  }
  plan.klass = klass;
  plan.steps = steps;
  plan.workspace_bytes = ws;
  return true;
}

// ---------------------------------------------------------------- transpose --
bool match_transpose(const Graph& g, Plan& plan) {
  if (g.outputs.size() != 1) return false;
  M m(g);
  int o = m.through_reshape(g.outputs[0]);
  const Node* n = m.prod(o, OpK::Transpose);
  if (!n) return false;
  m.take(n);
  int x = m.through_reshape(n->in[0]);
  if (!m.is_input(x) || !m.all_used()) return false;
  const std::vector<int64_t>& xs = g.v(n->in[0]).shape;
  const size_t R = xs.size();
  std::vector<int64_t> xstride(R, 1);
  for (int i = (int)R - 2; i >= 0; --i) xstride[i] = xstride[i + 1] * xs[i + 1];
  // output dims in order, dropping extent-1 dims, merging dims that are also
  // adjacent (and in order) in the input
  std::vector<int64_t> oshape, istride;
  std::vector<int64_t> src_axis;
  for (size_t i = 0; i < R; ++i) {
    int64_t ax = n->perm[i];
    if (xs[ax] == 1) continue;
    if (!src_axis.empty() && src_axis.back() + 1 == ax) {
      // merge unless an extent-1 axis sits between them — extent-1 never breaks adjacency
      oshape.back() *= xs[ax];
      istride.back() = xstride[ax];
      src_axis.back() = ax;
    } else {
      oshape.push_back(xs[ax]);
      istride.push_back(xstride[ax]);
      src_axis.push_back(ax);
    }
  }
  // adjacency across dropped extent-1 axes
  if (oshape.empty()) {
    oshape.push_back(1);
    istride.push_back(1);
  }
  if (oshape.size() > 6) return false;
  Step st;
  st.kind = StepK::Transpose;
  st.kernel_name = "transpose_nd";
  st.a = m.ref_of(x);
  st.out = m.ref_of(g.outputs[0]);
  st.tp.rank = (int)oshape.size();
  for (size_t i = 0; i < oshape.size(); ++i) {
    st.tp.out_shape[i] = oshape[i];
    st.tp.in_stride[i] = istride[i];
  }
  st.tp.esize = (int)dt_size(g.v(x).dt);
  plan.klass = "transpose";
  plan.steps.push_back(st);
  return true;
}

// ------------------------------------------------------- matmul + epilogue --
bool match_matmul(const Graph& g, Plan& plan) {
  if (g.outputs.size() != 1) return false;
  M m(g);
  int out = g.outputs[0];
  int cur = out, t;
  DT out_dt = g.v(out).dt;
  if (out_dt == DT::BF16 || out_dt == DT::F16) {
    M probe = m;
    if (probe.un(cur, OpK::Cast, &t) && g.v(t).dt == DT::F32) {
      m = probe;
      cur = t;
    }
  } else if (out_dt != DT::F32) {
    return false;
  }
  int relu = 0;
  {
    M probe = m;
    int other;
    double c;
    if (probe.bin_const(cur, OpK::Maximum, true, &other, &c) && c == 0.0) {
      m = probe;
      relu = 1;
      cur = other;
    }
  }
  int bias = -1;
  DT bias_dt = DT::F32;
  {
    M probe = m;
    int a, b;
    if (probe.bin(cur, OpK::Add, &a, &b)) {
      auto bias_src = [&](int vid, int* src) {
        M p2 = probe;
        int c = vid, q;
        if (p2.un(c, OpK::Cast, &q)) c = q;
        if (!p2.is_input(c)) return false;
        probe = p2;
        *src = c;
        return true;
      };
      int src;
      bool a_mm = g.v(a).producer >= 0 && (g.nodes[g.v(a).producer].kind == OpK::MatMul);
      bool b_mm = g.v(b).producer >= 0 && (g.nodes[g.v(b).producer].kind == OpK::MatMul);
      if (a_mm && bias_src(b, &src)) {
        bias = src;
        cur = a;
        m = probe;
      } else if (b_mm && bias_src(a, &src)) {
        bias = src;
        cur = b;
        m = probe;
      }
    }
  }
  const Node* mmn = m.prod(cur, OpK::MatMul);
  if (!mmn) return false;
  m.take(mmn);
  if (mmn->transpose_a) throw Unsupported("MatMul with transpose_a is rejected (as by the reference lowering)");
  int A = mmn->in[0], B = mmn->in[1];
  if (!m.is_input(A) || !m.is_input(B) || !m.all_used()) return false;
  const Value& av = g.v(A);
  const Value& bv = g.v(B);
  if ((av.dt != DT::BF16 && av.dt != DT::F16 && av.dt != DT::F32) || bv.dt != av.dt) return false;
  if (out_dt != DT::F32 && out_dt != av.dt) return false;
  if (av.shape.size() != 2 || bv.shape.size() != 2) return false;
  // accumulation happens in the MatMul's declared result type; only f32 is placed
  if (g.v(cur).dt != DT::F32) return false;
  MatmulParams p;
  p.M = av.shape[0];
  p.K = av.shape[1];
  p.transpose_b = mmn->transpose_b;
  p.N = mmn->transpose_b ? bv.shape[0] : bv.shape[1];
  int64_t kb = mmn->transpose_b ? bv.shape[1] : bv.shape[0];
  if (kb != p.K) throw JsonError("MatMul inner extents disagree");
  if (bias >= 0) {
    const Value& biasv = g.v(bias);
    if (biasv.numel() != p.N || biasv.shape.back() != p.N) return false;
    bias_dt = biasv.dt;
    if (bias_dt != av.dt && bias_dt != DT::F32) return false;
    p.has_bias = 1;
  }
  p.bias_dt = (int)bias_dt;
  p.relu = relu;
  p.out_dt = (int)out_dt;
  p.in_dt = (int)av.dt;
  const char* why = nullptr;
  if (av.dt != DT::F32 && !matmul_bf16_supported(p, &why))
    throw Unsupported(std::string("matmul shape not placed: ") + why);
  Step st;
  st.kind = StepK::Matmul;
  st.kernel_name = av.dt == DT::F32 ? "sgemm_f32" : "matmul_bf16_tcgen05";
  st.a = m.ref_of(A);
  st.b = m.ref_of(B);
  if (bias >= 0) st.c = m.ref_of(bias);
  st.out = m.ref_of(out);
  st.mm = p;
  plan.klass = "matmul";
  plan.flops = 2 * p.M * p.N * p.K;
  plan.steps.push_back(st);
  return true;
}

// --------------------------------------------------------------- GELU chain --
bool match_gelu_chain(const Graph& g, Plan& plan) {
  if (g.outputs.size() != 1) return false;
  M m(g);
  int out = g.outputs[0];
  int cur = out, q;
  int out_f32 = 0;
  if (g.v(out).dt == DT::F32) {
    if (!m.un(cur, OpK::Cast, &q) || g.v(q).dt != DT::F16) return false;
    cur = q;
    out_f32 = 1;
  } else if (g.v(out).dt != DT::F16) {
    return false;
  }
  const int64_t n = g.v(out).numel();
  // k = Mul(h, y) with y a full-size graph input — optional
  int ymul = -1, a, b;
  {
    M probe = m;
    if (probe.bin(cur, OpK::Mul, &a, &b)) {
      if (probe.is_input(b) && g.v(b).numel() == n && g.v(b).dt == DT::F16 && !probe.is_input(a)) {
        ymul = b;
        cur = a;
        m = probe;
      } else if (probe.is_input(a) && g.v(a).numel() == n && g.v(a).dt == DT::F16 && !probe.is_input(b)) {
        ymul = a;
        cur = b;
        m = probe;
      }
    }
  }
  // h = Mul(g_, f); g_ = Mul(t, 0.5); f = Add(e, 1)
  int gh, f;
  if (!m.bin(cur, OpK::Mul, &gh, &f)) return false;
  double c2, c_one;
  int t_a, e;
  {
    M probe = m;
    if (!(probe.bin_const(gh, OpK::Mul, true, &t_a, &c2) && probe.bin_const(f, OpK::Add, true, &e, &c_one))) {
      probe = m;
      std::swap(gh, f);
      if (!(probe.bin_const(gh, OpK::Mul, true, &t_a, &c2) && probe.bin_const(f, OpK::Add, true, &e, &c_one)))
        return false;
    }
    m = probe;
  }
  int d;
  if (!m.un(e, OpK::Tanh, &d)) return false;
  int c;
  double c1;
  if (!m.bin_const(d, OpK::Mul, true, &c, &c1)) return false;
  int t_b, bb;
  if (!m.bin(c, OpK::Add, &t_b, &bb)) return false;
  if (t_b != t_a) std::swap(t_b, bb);
  if (t_b != t_a) return false;
  int t3;
  double c0;
  if (!m.bin_const(bb, OpK::Mul, true, &t3, &c0)) return false;
  int sq, t_c;
  if (!m.bin(t3, OpK::Mul, &sq, &t_c)) return false;
  if (t_c != t_a) std::swap(sq, t_c);
  if (t_c != t_a) return false;
  int s_a, s_b;
  if (!m.bin(sq, OpK::Mul, &s_a, &s_b) || s_a != t_a || s_b != t_a) return false;
  // t = Add(x, bias) or t = x
  int x = t_a, bias = -1;
  int64_t inner = 0;
  if (!m.is_input(x)) {
    if (!m.bin(t_a, OpK::Add, &a, &b)) return false;
    if (!m.is_input(a) || !m.is_input(b)) return false;
    if (g.v(a).numel() != n) std::swap(a, b);
    x = a;
    bias = b;
    const Value& bv = g.v(bias);
    const Value& xv = g.v(x);
    if (bv.dt != DT::F16 || bv.shape.back() != xv.shape.back() || bv.numel() != xv.shape.back()) return false;
    inner = bv.numel();
  }
  if (g.v(x).dt != DT::F16 || g.v(x).numel() != n) return false;
  if (g.v(d).dt != DT::F16 || g.v(e).dt != DT::F16) return false;
  if (!m.all_used()) return false;

  Step st;
  st.kind = StepK::GeluChain;
  st.kernel_name = "gelu_chain_f16";
  st.a = m.ref_of(x);
  if (bias >= 0) st.b = m.ref_of(bias);
  if (ymul >= 0) st.c = m.ref_of(ymul);
  st.out = m.ref_of(out);
  st.gelu.n = n;
  st.gelu.inner = inner;
  st.gelu.has_mul = ymul >= 0;
  st.gelu.out_f32 = out_f32;
  st.gelu.c0 = round_f64_to_f16(c0);
  st.gelu.c1 = round_f64_to_f16(c1);
  st.gelu.c2 = round_f64_to_f16(c2);
  st.gelu.c_one = round_f64_to_f16(c_one);
  plan.klass = inner ? "broadcast" : "elementwise";
  plan.needs_gelu_lut = true;
  plan.steps.push_back(st);
  return true;
}

}  // namespace

// An elementwise chain over equally shaped tensors that ends in a reduction over ALL axes reads its inputs once when
// the n elements are viewed as [n / c, c] rows: one generated row kernel folds every row (the chain runs in registers)
// and the hand-written global reduction folds the n / c row results.  Returns false when the region is not of that form.
bool fused_reduce_all_plan(const Graph& g, int sm_count, Plan* out) {
  if (g.dynamic || g.outputs.size() != 1 || g.nodes.empty()) return false;
  const Node& red = g.nodes.back();
  if (!opk_is_reduce(red.kind) || red.out != g.outputs[0]) return false;
  RedOp op;
  switch (red.kind) {
    case OpK::ReduceSum: op = RedOp::Sum; break;
    case OpK::ReduceMax: op = RedOp::Max; break;
    case OpK::ReduceMin: op = RedOp::Min; break;
    case OpK::ReduceProd: op = RedOp::Prod; break;
    default: return false;
  }
  const Value& x = g.v(red.in[0]);
  if (red.axes.size() != x.shape.size() || x.dt != DT::F32 || g.v(red.out).dt != DT::F32 || g.v(red.out).numel() != 1)
    return false;
  const int64_t n = x.numel();
  if (n < (1 << 16)) return false;  // small tensors: the extra pass is not worth a generated kernel
  for (size_t i = 0; i + 1 < g.nodes.size(); ++i) {
    const Node& nd = g.nodes[i];
    if (!opk_is_elementwise(nd.kind) || nd.kind == OpK::AddN) return false;
    if (g.v(nd.out).numel() != n || g.v(nd.out).output_index >= 0) return false;
    for (int vid : nd.in) {
      const Value& v = g.v(vid);
      if (!v.is_const && v.numel() != n) return false;  // broadcast operands would not survive the re-view
    }
  }
  // the widest row of at most 4096 elements, a multiple of 8, that divides n
  int64_t c = 0;
  for (int64_t cand = 4096; cand >= 32; cand -= 8)
    if (n % cand == 0) {
      c = cand;
      break;
    }
  // no such divisor: any divisor will do (element-wise accesses instead of 16-byte ones, still one pass)
  for (int64_t cand = 4096; c == 0 && cand >= 64; --cand)
    if (n % cand == 0) c = cand;
  if (c == 0) return false;
  const int64_t r = n / c;
  Graph g2 = g;
  for (auto& v : g2.values)
    if (!v.is_const && v.numel() == n) v.shape = {r, c};
  Node& red2 = g2.nodes.back();
  red2.axes = {1};
  red2.keep_dims = false;
  g2.v(red2.out).shape = {r};
  auto rp = std::make_shared<RowProgram>();
  std::vector<int> in_values, out_values;
  if (!build_row_program(g2, rp.get(), &in_values, &out_values) || out_values.size() != 1) return false;
  Plan p;
  p.klass = "reduce_all";
  Step st;
  st.kind = StepK::RowJit;
  st.kernel_name = "akgb_row_jit";
  st.row = rp;
  for (int vid : in_values) {
    Ref ref;
    ref.arg = g.v(vid).input_index;
    st.ew_in.push_back(ref);
  }
  Ref partial;
  partial.ws_off = 0;
  st.ew_out.push_back(partial);
  p.steps.push_back(std::move(st));
  size_t ws = ((size_t)r * sizeof(float) + 255) / 256 * 256;
  Step fin;
  fin.kind = StepK::ReduceAll;
  fin.kernel_name = "reduce_all_f32";
  fin.red_op = op;
  fin.red_len = r;
  fin.a = partial;
  fin.out.arg = (int)g.inputs.size();
  fin.scratch.ws_off = (int64_t)ws;
  ws += (reduce_all_workspace(sm_count) + 255) / 256 * 256;
  p.steps.push_back(std::move(fin));
  p.workspace_bytes = ws;
  *out = std::move(p);
  return true;
}

// An elementwise chain that ends in a reduction over the LEADING axes: with the tensors viewed as [rows, cols] one
// generated kernel walks the rows, runs the chain in registers and keeps column accumulators; partial results of the
// row splits are folded by the hand-written column reduction.  Returns false when the region is not of that form.
bool fused_reduce_col_plan(const Graph& g, int sm_count, Plan* out) {
  if (g.dynamic || g.outputs.empty() || g.outputs.size() > 4 || g.nodes.size() < 2) return false;
  // the tail of the op list: one reduction per result, all over the same leading axes of equally shaped tensors
  const size_t n_red = g.outputs.size();
  if (g.nodes.size() <= n_red) return false;
  const size_t first_red = g.nodes.size() - n_red;
  const Node& red0 = g.nodes[first_red];
  if (!opk_is_reduce(red0.kind)) return false;
  const Value& x = g.v(red0.in[0]);
  const size_t rank = x.shape.size(), k = red0.axes.size();
  if (k == 0 || k >= rank) return false;
  for (size_t i = 0; i < k; ++i)
    if (red0.axes[i] != (int64_t)i) return false;
  int64_t R = 1, C = 1;
  for (size_t i = 0; i < rank; ++i) (i < k ? R : C) *= x.shape[i];
  if (R < 2 || C < 2 || R * C < (1 << 16)) return false;
  std::vector<RedOp> ops;
  for (size_t i = first_red; i < g.nodes.size(); ++i) {
    const Node& red = g.nodes[i];
    const Value& xi = g.v(red.in[0]);
    if (!opk_is_reduce(red.kind) || red.axes != red0.axes || xi.shape != x.shape || xi.dt != DT::F32 ||
        g.v(red.out).dt != DT::F32 || g.v(red.out).numel() != C || g.v(red.out).output_index < 0)
      return false;
    switch (red.kind) {
      case OpK::ReduceSum: ops.push_back(RedOp::Sum); break;
      case OpK::ReduceMax: ops.push_back(RedOp::Max); break;
      case OpK::ReduceMin: ops.push_back(RedOp::Min); break;
      case OpK::ReduceProd: ops.push_back(RedOp::Prod); break;
      default: return false;
    }
  }
  const std::vector<int64_t> lead(x.shape.begin(), x.shape.begin() + k), trail(x.shape.begin() + k, x.shape.end());
  auto strip = [](std::vector<int64_t> s) {
    while (s.size() > 1 && s.front() == 1) s.erase(s.begin());
    return s;
  };
  Graph g2 = g;
  for (size_t vi = 0; vi < g2.values.size(); ++vi) {
    Value& v = g2.values[vi];
    if (v.is_const) continue;
    const int64_t n = v.numel();
    bool is_result = false;
    for (size_t i = first_red; i < g.nodes.size(); ++i) is_result |= g.nodes[i].out == (int)vi;
    if (is_result) {
      v.shape = {C};
    } else if (n == R * C && v.shape.size() == rank) {
      v.shape = {R, C};
    } else if (n == 1) {
      v.shape = {1};
    } else if (n == C && strip(v.shape) == strip(trail)) {
      v.shape = {C};
    } else if (n == R && v.shape.size() == rank && std::equal(lead.begin(), lead.end(), v.shape.begin())) {
      v.shape = {R, 1};
    } else {
      return false;
    }
  }
  for (size_t i = 0; i < first_red; ++i) {
    const Node& nd = g.nodes[i];
    if (!opk_is_elementwise(nd.kind) || nd.kind == OpK::AddN || g.v(nd.out).output_index >= 0) return false;
  }
  for (size_t i = first_red; i < g2.nodes.size(); ++i) {
    g2.nodes[i].axes = {0};
    g2.nodes[i].keep_dims = false;
  }
  auto rp = std::make_shared<RowProgram>();
  std::vector<int> in_values, out_values;
  if (!build_row_program(g2, rp.get(), &in_values, &out_values, true) || out_values.size() != n_red) return false;
  const int64_t splits = col_jit_splits(*rp, sm_count);
  Plan p;
  p.klass = "reduce_y";
  Step st;
  st.kind = StepK::ColJit;
  st.kernel_name = "akgb_col_jit";
  st.row = rp;
  st.red_len = splits;
  for (int vid : in_values) {
    Ref ref;
    ref.arg = g.v(vid).input_index;
    st.ew_in.push_back(ref);
  }
  size_t ws = 0;
  std::vector<Step> finishes;
  for (size_t i = 0; i < n_red; ++i) {
    Ref result;
    result.arg = (int)g.inputs.size() + g.v(out_values[i]).output_index;
    if (splits == 1) {
      st.ew_out.push_back(result);
      continue;
    }
    Ref partial;
    partial.ws_off = (int64_t)ws;
    ws += ((size_t)(splits * C) * sizeof(float) + 255) / 256 * 256;
    st.ew_out.push_back(partial);
    Step fin;
    fin.kind = StepK::ReduceCol;
    fin.kernel_name = "reduce_col_f32";
    fin.red_op = ops[i];
    fin.red_outer = 1;
    fin.red_len = splits;
    fin.red_inner = C;
    fin.a = partial;
    fin.out = result;
    finishes.push_back(std::move(fin));
  }
  p.steps.push_back(std::move(st));
  for (Step& fin : finishes) {
    fin.scratch.ws_off = (int64_t)ws;
    ws += (reduce_col_workspace(splits, C, sm_count) + 255) / 256 * 256;
    p.steps.push_back(std::move(fin));
  }
  p.workspace_bytes = ws;
  *out = std::move(p);
  return true;
}

// Re-views a region whose reductions all fold the same run of TRAILING axes (InstanceNorm on NCHW: mean / variance over
// (H, W)) as [rows, cols]: full tensors become [R, C], per-(row) values [R, 1] or [R], tensors that span only the
// trailing axes [C], and region inputs that vary along one block of the row axes only (a per-channel [1, C, 1, 1] scale)
// are recorded in `row_index` as (div, mod) of the row number.  Returns false when the region is not of that form.
bool view_trailing_run(const Graph& g, Graph* gv, std::map<int, std::pair<int64_t, int64_t>>* row_index) {
  const Node* red0 = nullptr;
  for (auto& n : g.nodes)
    if (opk_is_reduce(n.kind)) {
      red0 = &n;
      break;
    }
  if (!red0 || g.dynamic) return false;
  const std::vector<int64_t> S = g.v(red0->in[0]).shape;
  const size_t rank = S.size();
  if (rank < 2) return false;
  std::vector<bool> is_red(rank, false);
  for (auto a : red0->axes) is_red[a] = true;
  size_t first = rank;
  while (first > 0 && (is_red[first - 1] || S[first - 1] == 1)) --first;
  if (first == 0 || first == rank) return false;
  for (size_t d = 0; d < first; ++d)
    if (is_red[d] && S[d] != 1) return false;  // folds leading axes too: not a pure row region
  int64_t R = 1, C = 1;
  for (size_t d = 0; d < rank; ++d) (d < first ? R : C) *= S[d];
  *gv = g;
  for (auto& n : gv->nodes) {
    if (!opk_is_reduce(n.kind)) continue;
    if (g.v(n.in[0]).shape != S || n.axes != red0->axes) return false;
    n.axes = {1};
  }
  const std::vector<int64_t> lead(S.begin(), S.begin() + first), trail(S.begin() + first, S.end());
  auto strip = [](std::vector<int64_t> s) {
    while (s.size() > 1 && s.front() == 1) s.erase(s.begin());
    return s;
  };
  for (size_t vi = 0; vi < gv->values.size(); ++vi) {
    Value& v = gv->values[vi];
    if (v.is_const) continue;
    if (v.producer < 0 && v.users.empty() && v.input_index < 0 && v.output_index < 0) continue;  // not of this region
    std::vector<int64_t> shp = v.shape;
    int64_t n = 1;
    for (auto e : shp) n *= e;
    // a per-row vector on its way to the broadcastable shape (weight [R] -> [R, 1] -> [R, 1, 1]): only re-viewed here
    bool only_reshaped = n == R && n > 1 && v.output_index < 0 && !v.users.empty() && shp.size() < rank;
    for (int u : v.users) only_reshaped = only_reshaped && g.nodes[u].kind == OpK::Reshape;
    if (shp.size() < rank && n != C) shp.insert(shp.begin(), rank - shp.size(), 1);  // broadcasting aligns trailing axes
    bool trailing_ones = shp.size() == rank;
    for (size_t d = first; trailing_ones && d < rank; ++d) trailing_ones = shp[d] == 1;
    auto squeeze = [](const std::vector<int64_t>& s) {
      std::vector<int64_t> r;
      for (auto e : s)
        if (e != 1) r.push_back(e);
      return r;
    };
    // the same elements under another split of the row axes ([n, c, h, w] against [1, n * c, h, w])
    bool regrouped = n == R * C && shp.size() >= trail.size() &&
                     std::equal(trail.begin(), trail.end(), shp.end() - (std::ptrdiff_t)trail.size());
    if (!regrouped && n == R * C && v.shape != S) {
      // any other shape of the same elements (the [n, c, h, w] tensor in front of GroupNorm's [n, groups, rest] view):
      // fine as long as only re-views and elementwise ops between equally shaped tensors touch it
      auto plain = [&](const Node& nd) {
        if (nd.kind == OpK::Reshape) return true;
        if (!opk_is_elementwise(nd.kind) || nd.kind == OpK::AddN || g.v(nd.out).shape != v.shape) return false;
        for (int o : nd.in)
          if (!g.v(o).is_const && g.v(o).numel() != 1 && g.v(o).shape != v.shape) return false;
        return true;
      };
      regrouped = v.producer < 0 || plain(g.nodes[v.producer]);
      for (int u : v.users) regrouped = regrouped && plain(g.nodes[u]);
    }
    if (shp == S || regrouped) {
      v.shape = {R, C};
    } else if (n == 1) {
      v.shape = {1};
    } else if (only_reshaped && squeeze(shp) == squeeze(lead)) {
      v.shape = {R};
    } else if (trailing_ones && std::equal(lead.begin(), lead.end(), shp.begin())) {
      v.shape = {R, 1};
    } else if (shp == lead) {
      v.shape = {R};
    } else if (n == C && strip(shp) == strip(trail)) {
      v.shape = {C};
    } else if (trailing_ones && v.input_index >= 0) {
      size_t lo = rank, hi = 0;
      for (size_t d = 0; d < first; ++d) {
        if (shp[d] == 1) continue;
        if (shp[d] != S[d]) return false;
        lo = std::min(lo, d);
        hi = std::max(hi, d + 1);
      }
      int64_t div = 1, mod = 1;
      for (size_t d = lo; d < hi; ++d) {
        if (shp[d] != S[d]) return false;
        mod *= S[d];
      }
      for (size_t d = hi; d < first; ++d) div *= S[d];
      (*row_index)[(int)vi] = {div, mod};
    } else {
      return false;
    }
  }
  return true;
}

// producer / users links of every value, recomputed from the op list (after ops were removed or rewired)
void relink(Graph& g) {
  for (auto& v : g.values) {
    v.producer = -1;
    v.users.clear();
  }
  for (size_t i = 0; i < g.nodes.size(); ++i) {
    g.values[g.nodes[i].out].producer = (int)i;
    for (int vid : g.nodes[i].in) g.values[vid].users.push_back((int)i);
  }
}

void shift_ref(Ref& r, const std::vector<Ref>& args, int64_t ws_base) {
  if (r.arg >= 0) r = args[r.arg];
  else if (r.ws_off >= 0) r.ws_off += ws_base;
}

// Elementwise chains over equally shaped tensors, the reductions they feed (one to four, same axes, which include the
// trailing axes, none needing another's result), then anything on the reduced values (BatchNorm statistics on NCHW: Mul(x, x) -> ReduceSum over (0, 2, 3) -> Mul(1/n)).  The chain and
// the fold over the trailing axes run as one generated row kernel on the [rows, cols] view; what remains (a reduction
// over the other axes, the ops behind it) is planned on its own with the row results as its input.
bool fused_reduce_tail_plan(const Graph& g, int sm_count, bool allow_jit, Plan* out) {
  if (g.dynamic || g.nodes.size() < 2) return false;
  const int nn = (int)g.nodes.size();
  int ri = -1;
  for (int i = 0; i < nn; ++i)
    if (opk_is_reduce(g.nodes[i].kind)) {
      ri = i;
      break;
    }
  if (ri < 0) return false;
  const Node& red = g.nodes[ri];
  const Value& x = g.v(red.in[0]);
  const size_t rank = x.shape.size();
  if (rank == 0) return false;
  std::vector<bool> is_red(rank, false);
  for (auto a : red.axes) is_red[a] = true;
  // the trailing run: from the last axis backwards while the axis is reduced (extent-1 axes ride along)
  size_t first = rank;
  while (first > 0 && (is_red[first - 1] || x.shape[first - 1] == 1)) --first;
  int64_t C = 1, n = x.numel();
  for (size_t i = first; i < rank; ++i) C *= x.shape[i];
  if (first == 0 || C < 8 || C > (1 << 20) || n < (1 << 16)) return false;  // all axes: the re-viewed plan above
  const int64_t R = n / C;
  // Front: the ops that need no reduction result — elementwise ops over x's shape (the chains) and the reductions of
  // such values over the same axes (up to four share the pass).  Everything else is the rest.
  enum { REST = 0, CHAIN = 1, FOLD = 2 };
  std::vector<int> role(nn, REST);
  std::vector<char> dep(nn, 0);
  std::vector<int> folds;
  for (int i = 0; i < nn; ++i) {
    const Node& nd = g.nodes[i];
    for (int vid : nd.in) {
      const int p = g.v(vid).producer;
      if (p >= 0 && (dep[p] || opk_is_reduce(g.nodes[p].kind))) dep[i] = 1;
    }
    if (dep[i]) continue;
    const Value& ov = g.v(nd.out);
    if (opk_is_reduce(nd.kind)) {
      if (nd.kind != OpK::ReduceSum && nd.kind != OpK::ReduceMax && nd.kind != OpK::ReduceMin && nd.kind != OpK::ReduceProd)
        return false;
      if (g.v(nd.in[0]).shape != x.shape || nd.axes != red.axes || g.v(nd.in[0]).dt != DT::F32 || ov.dt != DT::F32) return false;
      role[i] = FOLD;
      folds.push_back(i);
    } else if (opk_is_elementwise(nd.kind) && nd.kind != OpK::AddN && ov.shape == x.shape) {
      role[i] = CHAIN;
    }
  }
  bool any_chain = false;
  for (int i = 0; i < nn; ++i) any_chain = any_chain || role[i] == CHAIN;
  // (a single reduction with no chain in front: the hand-written reductions do it)
  if (folds.empty() || folds.size() > 4 || !any_chain) return false;
  std::map<int, std::pair<int64_t, int64_t>> row_index;
  for (int i = 0; i < nn; ++i) {
    const Node& nd = g.nodes[i];
    if (role[i] == REST) {
      // the rest works on reduced values: nothing of x's size is read or made there
      if (opk_is_reduce(nd.kind) && g.v(nd.in[0]).numel() == n) return false;
      continue;
    }
    if (role[i] != CHAIN) continue;
    const Value& ov = g.v(nd.out);
    if (ov.output_index >= 0) return false;
    for (int vid : nd.in) {
      const Value& v = g.v(vid);
      if (v.is_const || v.shape == x.shape) continue;
      // a region input that varies along one block of the row axes only (a per-channel [1, C, 1, 1] value): read through
      // (row / div) % mod
      if (v.input_index < 0 || v.shape.size() != rank) return false;
      size_t lo = rank, hi = 0;
      for (size_t d = 0; d < rank; ++d) {
        if (v.shape[d] == 1) continue;
        if (d >= first || v.shape[d] != x.shape[d]) return false;
        lo = std::min(lo, d);
        hi = std::max(hi, d + 1);
      }
      if (lo >= hi) continue;  // one element: a scalar operand
      int64_t div = 1, mod = 1;
      for (size_t d = lo; d < hi; ++d) {
        if (v.shape[d] != x.shape[d]) return false;  // the block has no gaps
        mod *= x.shape[d];
      }
      for (size_t d = hi; d < first; ++d) div *= x.shape[d];
      row_index[vid] = {div, mod};
    }
    for (int u : ov.users)
      if (role[u] == REST) return false;  // the chain's values are not kept for the ops behind the reductions
  }
  // 1. the row program: chains + folds over the trailing run on the [R, C] view
  Graph g2 = g;
  g2.nodes.clear();
  for (int i = 0; i < nn; ++i)
    if (role[i] != REST) g2.nodes.push_back(g.nodes[i]);
  for (auto& v : g2.values) {
    v.output_index = -1;
    if (!v.is_const && v.shape == x.shape) v.shape = {R, C};
  }
  g2.outputs.clear();
  for (Node& nd : g2.nodes) {
    if (!opk_is_reduce(nd.kind)) continue;
    nd.axes = {1};
    nd.keep_dims = false;
    g2.v(nd.out).shape = {R};
    g2.v(nd.out).output_index = (int)g2.outputs.size();
    g2.outputs.push_back(nd.out);
  }
  relink(g2);
  auto rp = std::make_shared<RowProgram>();
  std::vector<int> in_values, out_values;
  if (!build_row_program(g2, rp.get(), &in_values, &out_values, false, &row_index) || out_values.size() != folds.size())
    return false;
  for (size_t j = 0; j < folds.size(); ++j)
    if (out_values[j] != g.nodes[folds[j]].out) return false;
  bool only_trailing = true;
  for (auto a : red.axes) only_trailing = only_trailing && ((size_t)a >= first || x.shape[a] == 1);
  if (only_trailing && folds.size() == 1 && (size_t)ri + 1 == g.nodes.size() && g.outputs.size() == 1 && g.outputs[0] == red.out) {
    // nothing behind the fold over the trailing axes: the row results are the region's result
    Plan p;
    p.klass = "reduce_x";
    Step st;
    st.kind = StepK::RowJit;
    st.kernel_name = "akgb_row_jit";
    st.row = rp;
    for (int vid : in_values) {
      Ref ref;
      ref.arg = g.v(vid).input_index;
      st.ew_in.push_back(ref);
    }
    Ref result;
    result.arg = (int)g.inputs.size();
    st.ew_out.push_back(result);
    p.steps.push_back(std::move(st));
    *out = std::move(p);
    return true;
  }
  // 2. the rest: the row results stand in for the reductions' operands, with the trailing run folded to extent 1
  const int64_t each = (int64_t)(((size_t)R * sizeof(float) + 255) / 256 * 256);
  Graph g3 = g;
  g3.nodes.clear();
  std::vector<Ref> arg_map;
  std::vector<int> new_inputs;
  std::vector<int64_t> rest_axes;
  for (auto a : red.axes)
    if ((size_t)a < first && x.shape[a] != 1) rest_axes.push_back(a);
  for (int i = 0; i < nn; ++i) {
    if (role[i] == CHAIN) continue;
    g3.nodes.push_back(g.nodes[i]);
    if (role[i] != FOLD) continue;
    Value part;
    part.name = "akgb_row_results" + std::to_string(new_inputs.size());
    part.shape = x.shape;
    for (size_t d = first; d < rank; ++d) part.shape[d] = 1;
    part.dt = DT::F32;
    part.input_index = (int)new_inputs.size();
    const int pid = (int)g3.values.size();
    g3.values.push_back(part);
    Ref partial;
    partial.ws_off = each * (int64_t)new_inputs.size();
    arg_map.push_back(partial);
    new_inputs.push_back(pid);
    Node& red3 = g3.nodes.back();
    red3.in[0] = pid;
    if (rest_axes.empty()) {
      red3.kind = OpK::Reshape;  // nothing left to fold: the row results are the reduction's result
      red3.name = "Reshape";
      red3.axes.clear();
    } else {
      red3.axes = rest_axes;
    }
  }
  relink(g3);
  // inputs of the rest: the row results first, then the region's inputs it still reads
  for (int vid : g.inputs) {
    if (g3.values[vid].users.empty()) {
      g3.values[vid].input_index = -1;
      continue;
    }
    Ref r;
    r.arg = g.v(vid).input_index;
    arg_map.push_back(r);
    g3.values[vid].input_index = (int)new_inputs.size();
    new_inputs.push_back(vid);
  }
  g3.inputs = new_inputs;
  for (int vid : g3.outputs)
    if (g3.values[vid].producer < 0) return false;  // a result that is not produced behind the reductions
  for (size_t i = 0; i < g.outputs.size(); ++i) {
    Ref r;
    r.arg = (int)g.inputs.size() + (int)i;
    arg_map.push_back(r);
  }
  classify(g3);
  Plan rest;
  try {
    rest = build_plan(g3, sm_count, allow_jit);
  } catch (const Unsupported&) {
    return false;
  }
  if (rest.fallback) return false;  // keep it to plans with one way of running
  const int64_t ws_base = each * (int64_t)folds.size();
  Plan p;
  p.klass = g.reduce_dir == ReduceDir::All ? "reduce_all" : g.reduce_dir == ReduceDir::Y ? "reduce_y" : "reduce_x";
  Step st;
  st.kind = StepK::RowJit;
  st.kernel_name = "akgb_row_jit";
  st.row = rp;
  for (int vid : in_values) {
    Ref ref;
    ref.arg = g.v(vid).input_index;
    st.ew_in.push_back(ref);
  }
  for (size_t j = 0; j < folds.size(); ++j) st.ew_out.push_back(arg_map[j]);
  p.steps.push_back(std::move(st));
  for (Step& s2 : rest.steps) {
    for (Ref* r : {&s2.a, &s2.b, &s2.c, &s2.out, &s2.out2, &s2.out3, &s2.scratch}) shift_ref(*r, arg_map, ws_base);
    for (Ref& r : s2.ew_in) shift_ref(r, arg_map, ws_base);
    for (Ref& r : s2.ew_out) shift_ref(r, arg_map, ws_base);
    p.steps.push_back(std::move(s2));
  }
  p.workspace_bytes = (size_t)ws_base + rest.workspace_bytes;
  p.needs_gelu_lut = rest.needs_gelu_lut;
  *out = std::move(p);
  return true;
}

// ---- regions that are a row region only in part -----------------------------------------------------------------------
// Nodes [a, b) of the region as a region of its own: what it reads from outside becomes its inputs (first use order),
// what is read outside of it or is a result of the whole region becomes its outputs.
Graph subregion(const Graph& g, int a, int b, std::vector<int>* in_vals, std::vector<int>* out_vals) {
  Graph gs = g;
  gs.nodes.assign(g.nodes.begin() + a, g.nodes.begin() + b);
  relink(gs);
  for (auto& v : gs.values) v.input_index = v.output_index = -1;
  in_vals->clear();
  out_vals->clear();
  for (const Node& n : gs.nodes)
    for (int vid : n.in) {
      const Value& v = gs.values[vid];
      if (v.is_const || v.producer >= 0 || v.input_index >= 0) continue;
      gs.values[vid].input_index = (int)in_vals->size();
      in_vals->push_back(vid);
    }
  for (const Node& n : gs.nodes) {
    const Value& ov = g.v(n.out);
    bool outside = ov.output_index >= 0;
    for (int u : ov.users) outside = outside || u >= b;
    if (!outside) continue;
    gs.values[n.out].output_index = (int)out_vals->size();
    out_vals->push_back(n.out);
  }
  gs.inputs = *in_vals;
  gs.outputs = *out_vals;
  classify(gs);
  return gs;
}

bool try_row_program(const Graph& gs, std::shared_ptr<RowProgram>* rp, std::vector<int>* in_values,
                     std::vector<int>* out_values) {
  *rp = std::make_shared<RowProgram>();
  in_values->clear();
  out_values->clear();
  if (build_row_program(gs, rp->get(), in_values, out_values)) return true;
  Graph gv;
  std::map<int, std::pair<int64_t, int64_t>> row_index;
  *rp = std::make_shared<RowProgram>();
  in_values->clear();
  out_values->clear();
  return view_trailing_run(gs, &gv, &row_index) && build_row_program(gv, rp->get(), in_values, out_values, false, &row_index);
}

// Cuts the op list into pieces: the longest runs of ops that form a row region of their own (at least one reduction
// inside) become one generated row kernel each, the ops in between are planned as separate launches; values that cross
// pieces live in the workspace.  GroupNorm (statistics on the [n, groups, rest] view, scale and shift per channel on
// another view) or a LayerNorm followed by a transpose run as two launches this way.  Returns false when no piece is
// a row region.
struct Piece {
  int a, b;
  bool row;
  std::shared_ptr<RowProgram> rp;
  std::vector<int> in_vals, out_vals;  // graph values, in the order the piece's kernel(s) take them
};
bool assemble_pieces(const Graph& g, std::vector<Piece>& pieces, int sm_count, Plan* out);

bool segmented_plan(const Graph& g, int sm_count, Plan* out) {
  const int n = (int)g.nodes.size();
  if (g.dynamic || n < 3 || n > 200) return false;
  for (auto& nd : g.nodes)
    if (nd.kind == OpK::Assign) return false;  // stores into inputs: keep the whole-region planner
  std::vector<Piece> pieces;
  bool any_row = false;
  int a = 0;
  while (a < n) {
    // the longest [a, b) with a reduction inside that is a row region
    int best = -1;
    Piece cand;
    for (int b = n; b > a + 1; --b) {
      bool has_red = false;
      for (int i = a; i < b; ++i) has_red = has_red || opk_is_reduce(g.nodes[i].kind);
      if (!has_red) break;
      std::vector<int> iv, ov, riv, rov;
      Graph gs = subregion(g, a, b, &iv, &ov);
      std::shared_ptr<RowProgram> rp;
      if (ov.empty() || !try_row_program(gs, &rp, &riv, &rov)) continue;
      best = b;
      cand.a = a;
      cand.b = b;
      cand.row = true;
      cand.rp = rp;
      cand.in_vals = riv;
      cand.out_vals = rov;
      break;
    }
    if (best > 0) {
      pieces.push_back(std::move(cand));
      any_row = true;
      a = best;
    } else {
      if (!pieces.empty() && !pieces.back().row) pieces.back().b = a + 1;  // extend the open run of other ops
      else pieces.push_back(Piece{a, a + 1, false, nullptr, {}, {}});
      ++a;
    }
  }
  if (!any_row || pieces.size() < 2) return false;
  return assemble_pieces(g, pieces, sm_count, out);
}

// Cuts the op list behind every reduction and the per-result ops that follow it: a piece is an elementwise chain, the
// reduction it feeds and the small ops on the reduced values, so each piece is planned as a region of its own (chain
// folded into the reduction pass) and only reduced values cross pieces.  Batch normalisation in training mode (mean
// over n, h, w; variance of the centred values; scale and shift) becomes three such pieces instead of materialising
// the centred squares.  Returns false when nothing is cut.
// Op order by stage: a value's stage counts the reductions whose results it needs.  Independent reductions (the two
// sums of a batch-norm backward pass) share a stage and therefore a pass over their operands; the small ops on reduced
// values stay with the reduction that feeds them.  Returns the end of each stage in the new op list.
std::vector<int> order_by_stage(Graph& g) {
  const int n = (int)g.nodes.size();
  int64_t large = 0;
  for (auto& nd : g.nodes) large = std::max(large, g.v(nd.out).numel());
  std::vector<int> stage(n, 0);
  std::vector<char> reduced(n, 0);  // the op works on reduced values only
  for (int i = 0; i < n; ++i) {
    const Node& nd = g.nodes[i];
    const bool red = opk_is_reduce(nd.kind);
    bool all_small = !red && g.v(nd.out).numel() < large;
    int st = 0;
    for (int vid : nd.in) {
      const Value& v = g.v(vid);
      if (v.is_const || v.producer < 0) {
        all_small = all_small && v.numel() < large;
        continue;
      }
      all_small = all_small && reduced[v.producer];
    }
    for (int vid : nd.in) {
      const int p = g.v(vid).producer;
      if (p < 0) continue;
      st = std::max(st, stage[p] + ((reduced[p] && !all_small) ? 1 : 0));
    }
    stage[i] = st;
    reduced[i] = red || all_small;
  }
  std::vector<int> idx(n);
  for (int i = 0; i < n; ++i) idx[i] = i;
  std::stable_sort(idx.begin(), idx.end(), [&](int x, int y) { return stage[x] < stage[y]; });
  std::vector<Node> sorted;
  std::vector<int> ends;
  for (int k = 0; k < n; ++k) {
    if (k && stage[idx[k]] != stage[idx[k - 1]]) ends.push_back(k);
    sorted.push_back(g.nodes[idx[k]]);
  }
  ends.push_back(n);
  g.nodes = std::move(sorted);
  relink(g);
  return ends;
}

bool reduction_cut_plan(const Graph& g0, int sm_count, bool by_stage, Plan* out) {
  const int n = (int)g0.nodes.size();
  if (g0.dynamic || n < 3 || n > 200) return false;
  for (auto& nd : g0.nodes)
    if (nd.kind == OpK::Assign) return false;
  Graph g = g0;
  std::vector<std::pair<int, int>> ranges;
  int a = 0;
  int64_t large = 0;
  for (auto& nd : g.nodes) large = std::max(large, g.v(nd.out).numel());
  if (by_stage) {
    for (int e : order_by_stage(g)) {
      ranges.push_back({a, e});
      a = e;
    }
    a = n;
  } else {
    bool seen_reduce = false;
    int64_t reduced_numel = 0;
    for (int i = 0; i < n; ++i) {
      const Node& nd = g.nodes[i];
      const bool red = opk_is_reduce(nd.kind);
      if (seen_reduce && (red || g.v(nd.out).numel() > reduced_numel)) {
        ranges.push_back({a, i});
        a = i;
        seen_reduce = false;
      }
      if (red) {
        seen_reduce = true;
        reduced_numel = g.v(nd.out).numel();
      }
    }
  }
  if (a < n) ranges.push_back({a, n});
  if (ranges.size() < 2) return false;
  // A full-size elementwise value of an earlier piece (the centred values x - mean, read again by the scale and
  // shift) is computed again in the piece that reads it instead of crossing through memory: its operands are read
  // there anyway or are small.
  Graph g2 = g;
  std::vector<Node> order;
  std::vector<Piece> pieces;
  for (size_t k = 0; k < ranges.size(); ++k) {
    const int pa = ranges[k].first, pb = ranges[k].second;
    const int start = (int)order.size();
    std::map<int, int> again;  // value of an earlier piece -> its copy in this piece
    int steps_left = 16;
    std::function<int(int)> here = [&](int vid) -> int {
      const Value& v = g.v(vid);
      if (v.is_const || v.producer < 0 || v.producer >= pa || v.output_index >= 0 || v.numel() < large) return vid;
      const Node& pn = g.nodes[v.producer];
      if (!opk_is_elementwise(pn.kind)) return vid;
      auto it = again.find(vid);
      if (it != again.end()) return it->second;
      if (--steps_left < 0) return vid;
      Node c = pn;
      for (int& u : c.in) u = here(u);
      Value nv = v;
      nv.name += "_again" + std::to_string(k);
      nv.users.clear();
      g2.values.push_back(nv);
      c.out = (int)g2.values.size() - 1;
      order.push_back(c);
      again[vid] = c.out;
      return c.out;
    };
    for (int i = pa; i < pb; ++i) {
      Node nd = g.nodes[i];
      for (int& u : nd.in) u = here(u);
      order.push_back(std::move(nd));
    }
    pieces.push_back(Piece{start, (int)order.size(), false, nullptr, {}, {}});
  }
  g2.nodes = std::move(order);
  relink(g2);
  return assemble_pieces(g2, pieces, sm_count, out);
}

bool assemble_pieces(const Graph& g, std::vector<Piece>& pieces, int sm_count, Plan* out) {
  // A piece made of Reshape ops only is a change of view: its result shares the buffer of its operand (the producer
  // writes into the region's output directly when the view is one).
  std::map<int, int> same_buffer;  // value -> value whose buffer it uses
  for (Piece& pc : pieces) {
    if (pc.row) continue;
    bool views = true;
    for (int i = pc.a; i < pc.b; ++i) {
      const Node& nd = g.nodes[i];
      const Value& src = g.v(nd.in[0]);
      // (two buffers of the caller cannot be one: a view of an input or output that is itself a result needs a copy)
      views = views && nd.kind == OpK::Reshape && src.numel() == g.v(nd.out).numel() &&
              !((src.input_index >= 0 || src.output_index >= 0) && g.v(nd.out).output_index >= 0);
    }
    if (!views) continue;
    for (int i = pc.a; i < pc.b; ++i) {
      const Node& nd = g.nodes[i];
      if (g.v(nd.out).output_index >= 0) same_buffer[nd.in[0]] = nd.out;  // the output's buffer holds both
      else same_buffer[nd.out] = nd.in[0];
    }
    pc.a = pc.b;  // nothing left to launch
  }
  auto root_of = [&](int vid) {
    for (int hops = 0; hops < 64; ++hops) {
      auto it = same_buffer.find(vid);
      if (it == same_buffer.end()) break;
      vid = it->second;
    }
    return vid;
  };
  // buffers of the values that cross pieces
  std::map<int, Ref> where;
  size_t ws = 0;
  auto ref_of = [&](int vid) {
    vid = root_of(vid);
    auto it = where.find(vid);
    if (it != where.end()) return it->second;
    const Value& v = g.v(vid);
    Ref r;
    if (v.input_index >= 0) r.arg = v.input_index;
    else if (v.output_index >= 0) r.arg = (int)g.inputs.size() + v.output_index;
    else {
      r.ws_off = (int64_t)ws;
      ws += ((size_t)v.numel() * dt_size(v.dt) + 255) / 256 * 256;
    }
    where[vid] = r;
    return r;
  };
  Plan p;
  p.klass = g.reduce_dir == ReduceDir::All ? "reduce_all" : g.reduce_dir == ReduceDir::Y ? "reduce_y" : "reduce_x";
  struct Pending {
    size_t first_step, n_steps;
  };
  std::vector<Pending> generic_runs;
  size_t sub_ws = 0;
  for (Piece& pc : pieces) {
    if (pc.row) {
      Step st;
      st.kind = StepK::RowJit;
      st.kernel_name = "akgb_row_jit";
      st.row = pc.rp;
      for (int vid : pc.in_vals) st.ew_in.push_back(ref_of(vid));
      for (int vid : pc.out_vals) st.ew_out.push_back(ref_of(vid));
      p.steps.push_back(std::move(st));
      continue;
    }
    if (pc.a >= pc.b) continue;  // a change of view
    std::vector<int> iv, ov;
    Graph gs = subregion(g, pc.a, pc.b, &iv, &ov);
    if (ov.empty()) continue;  // nothing of it is used
    // the piece is a region of its own: templates and generated reductions apply to it like to any region (should a
    // generated kernel fail to compile at launch, the whole region falls back, so the piece's own fallback is dropped)
    Plan sub;
    try {
      sub = build_plan(gs, sm_count, true);
    } catch (const Unsupported&) {
      return false;
    }
    sub.fallback.reset();
    std::vector<Ref> arg_map;
    for (int vid : iv) arg_map.push_back(ref_of(vid));
    for (int vid : ov) arg_map.push_back(ref_of(vid));
    generic_runs.push_back({p.steps.size(), sub.steps.size()});
    for (Step& s2 : sub.steps) {
      // workspace offsets of the piece are made absolute once all crossing buffers are known (marked by +1 below)
      for (Ref* r : {&s2.a, &s2.b, &s2.c, &s2.out, &s2.out2, &s2.out3, &s2.scratch}) {
        if (r->arg >= 0) *r = arg_map[r->arg];
        else if (r->ws_off >= 0) r->ws_off = -2 - r->ws_off;
      }
      for (auto* vec : {&s2.ew_in, &s2.ew_out})
        for (Ref& r : *vec) {
          if (r.arg >= 0) r = arg_map[r.arg];
          else if (r.ws_off >= 0) r.ws_off = -2 - r.ws_off;
        }
      p.steps.push_back(std::move(s2));
    }
    sub_ws = std::max(sub_ws, sub.workspace_bytes);
    p.flops += sub.flops;
    p.needs_gelu_lut = p.needs_gelu_lut || sub.needs_gelu_lut;
  }
  // the pieces' own scratch shares one area behind the crossing buffers (pieces run one after the other)
  const int64_t base = (int64_t)ws;
  for (Step& st : p.steps) {
    for (Ref* r : {&st.a, &st.b, &st.c, &st.out, &st.out2, &st.out3, &st.scratch})
      if (r->arg < 0 && r->ws_off <= -2) r->ws_off = base + (-2 - r->ws_off);
    for (auto* vec : {&st.ew_in, &st.ew_out})
      for (Ref& r : *vec)
        if (r.arg < 0 && r.ws_off <= -2) r.ws_off = base + (-2 - r.ws_off);
  }
  p.workspace_bytes = ws + sub_ws;
  *out = std::move(p);
  return true;
}

// Ops behind a sum over all rows (the cast of a weight gradient to the parameter type) are split off: the region in
// front of them is planned on its own, so that its sums can stay inside a row kernel, and the few small ops run after
// the partial sums have been folded.
bool tail_split_plan(const Graph& g0, int sm_count, Plan* out) {
  const int n = (int)g0.nodes.size();
  if (g0.dynamic || n < 3 || n > 200) return false;
  int64_t large = 0;
  for (auto& nd : g0.nodes) {
    if (nd.kind == OpK::Assign) return false;
    large = std::max(large, g0.v(nd.out).numel());
  }
  std::vector<char> tail(n, 0), view_of_sum(n, 0);
  bool any = false;
  for (int i = 0; i < n; ++i) {
    const Node& nd = g0.nodes[i];
    for (int vid : nd.in) {
      const int p = g0.v(vid).producer;
      if (p < 0) continue;
      const Node& pn = g0.nodes[p];
      const bool sum_over_rows = pn.kind == OpK::ReduceSum && !pn.axes.empty() && pn.axes.front() == 0 &&
                                 g0.v(pn.in[0]).shape.size() >= 2 && pn.axes.size() + 1 == g0.v(pn.in[0]).shape.size() &&
                                 pn.axes.back() == (int64_t)g0.v(pn.in[0]).shape.size() - 2;
      const bool of_sum = sum_over_rows || view_of_sum[p];
      if (of_sum && nd.kind == OpK::Reshape) view_of_sum[i] = 1;  // still the sum itself
      else if (tail[p] || of_sum) tail[i] = 1;
    }
    if (tail[i]) {
      if (g0.v(nd.out).numel() >= large) return false;  // the tail works on column vectors only
      any = true;
    }
  }
  if (!any) return false;
  Graph g = g0;
  std::vector<Node> order;
  for (int i = 0; i < n; ++i)
    if (!tail[i]) order.push_back(g0.nodes[i]);
  const int n_main = (int)order.size();
  for (int i = 0; i < n; ++i)
    if (tail[i]) order.push_back(g0.nodes[i]);
  if (n_main < 2 || n_main == n) return false;
  g.nodes = std::move(order);
  relink(g);
  std::vector<Piece> pieces = {Piece{0, n_main, false, nullptr, {}, {}}, Piece{n_main, n, false, nullptr, {}, {}}};
  return assemble_pieces(g, pieces, sm_count, out);
}

Plan build_plan(const Graph& g, int sm_count, bool allow_jit) {
  for (auto& n : g.nodes)
    if (n.kind == OpK::Unknown)
      throw Unsupported("operator '" + n.name + "' is not supported");
  Plan plan;
  bool ok = false;
  switch (g.op_class) {
    case OpClass::Matmul:
      ok = match_matmul(g, plan);
      break;
    case OpClass::Reduction:
      ok = match_layernorm(g, plan) || match_softmax(g, plan) || match_reduce(g, plan, sm_count);
      break;
    case OpClass::Transpose:
      ok = match_transpose(g, plan);
      break;
    default:
      ok = match_gelu_chain(g, plan);
      break;
  }
  if (!ok) {
    plan = build_generic_plan(g, sm_count);
    // a reduce-X region that would take several launches: one generated row kernel, the launches as its fallback
    auto rp = std::make_shared<RowProgram>();
    std::vector<int> in_values, out_values;
    Graph gv;
    std::map<int, std::pair<int64_t, int64_t>> row_index;
    const bool row_region =
        allow_jit && plan.steps.size() > 1 && g.op_class == OpClass::Reduction &&
        (build_row_program(g, rp.get(), &in_values, &out_values, false, nullptr, true) ||
         (in_values.clear(), out_values.clear(), *rp = RowProgram(), view_trailing_run(g, &gv, &row_index) &&
          build_row_program(gv, rp.get(), &in_values, &out_values, false, &row_index)));
    if (row_region) {
      Plan fused;
      fused.klass = plan.klass;
      fused.workspace_bytes = 0;  // one kernel, nothing crosses launches
      fused.flops = plan.flops;
      Step st;
      st.kind = StepK::RowJit;
      st.kernel_name = "akgb_row_jit";
      st.row = rp;
      for (int vid : in_values) {
        Ref r;
        r.arg = g.v(vid).input_index;
        st.ew_in.push_back(r);
      }
      // sums over all rows: the kernel writes one partial vector per CTA, a column reduction folds them
      std::vector<Step> finishes;
      size_t fws = 0;
      const int64_t parts = rp->col_sums ? row_jit_col_sum_ctas(*rp) : 0;
      for (size_t i = 0; i < out_values.size(); ++i) {
        Ref r;
        r.arg = (int)g.inputs.size() + g.v(out_values[i]).output_index;
        if (rp->out[i].kind != RK_COL) {
          st.ew_out.push_back(r);
          continue;
        }
        Ref partial;
        partial.ws_off = (int64_t)fws;
        fws += ((size_t)(parts * rp->cols) * sizeof(float) + 255) / 256 * 256;
        st.ew_out.push_back(partial);
        Step fin;
        fin.kind = StepK::ReduceCol;
        fin.kernel_name = "reduce_col_f32";
        fin.red_op = RedOp::Sum;
        fin.red_outer = 1;
        fin.red_len = parts;
        fin.red_inner = rp->cols;
        fin.a = partial;
        fin.out = r;
        finishes.push_back(std::move(fin));
      }
      fused.steps.push_back(std::move(st));
      for (Step& fin : finishes) {
        fin.scratch.ws_off = (int64_t)fws;
        fws += (reduce_col_workspace(parts, rp->cols, sm_count) + 255) / 256 * 256;
        fused.steps.push_back(std::move(fin));
      }
      fused.workspace_bytes = fws;
      fused.fallback = std::make_shared<Plan>(std::move(plan));
      plan = std::move(fused);
    } else if (Plan fused; allow_jit && plan.steps.size() >= 2 &&
               (fused_reduce_all_plan(g, sm_count, &fused) || fused_reduce_col_plan(g, sm_count, &fused) ||
                fused_reduce_tail_plan(g, sm_count, allow_jit, &fused))) {
      fused.flops = plan.flops;
      fused.fallback = std::make_shared<Plan>(std::move(plan));
      plan = std::move(fused);
    } else if (allow_jit && plan.steps.size() > 2) {
      // Other ways to run the region in fewer passes over its tensors: cut into row-kernel pieces and other ops; cut at
      // the reductions, in the given op order or stage by stage; the small ops behind sums over all rows split off.
      // The candidate with the smallest workspace (fewest full-size values crossing launches) wins, then the one with
      // the fewest launches.
      std::vector<Plan> cands;
      Plan c;
      if (segmented_plan(g, sm_count, &c)) cands.push_back(std::move(c));
      if (g.op_class == OpClass::Reduction) {
        if (c = Plan(); reduction_cut_plan(g, sm_count, false, &c)) cands.push_back(std::move(c));
        if (c = Plan(); reduction_cut_plan(g, sm_count, true, &c)) cands.push_back(std::move(c));
        if (c = Plan(); tail_split_plan(g, sm_count, &c)) cands.push_back(std::move(c));
      }
      Plan* best = nullptr;
      for (Plan& x : cands) {
        // taken with fewer launches, or far less workspace (no full-size intermediate is written)
        if (!(x.steps.size() < plan.steps.size() ||
              (x.steps.size() <= plan.steps.size() + 2 && x.workspace_bytes * 2 < plan.workspace_bytes)))
          continue;
        // (workspace counted in eighths of the region's own tensors: partial sums and per-channel values do not matter)
        const size_t quantum = std::max<size_t>((size_t)8 << 20, (size_t)io_bytes(g) / 8);
        const size_t wx = x.workspace_bytes / quantum, wb = best ? best->workspace_bytes / quantum : 0;
        if (!best || (wx != wb ? wx < wb : x.steps.size() < best->steps.size())) best = &x;
      }
      if (best) {
        best->flops = plan.flops;
        best->fallback = std::make_shared<Plan>(std::move(plan));
        plan = std::move(*best);
      }
    }
  }
  plan.bytes = io_bytes(g);
  if (plan.fallback) plan.fallback->bytes = plan.bytes;
  return plan;
}

}  // namespace akgb
