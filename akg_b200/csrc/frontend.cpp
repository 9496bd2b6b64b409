// JSON front end, class tagging and leading-axis shard inference.
#include <algorithm>
#include <cctype>
#include <cstring>
#include <set>

#include "graph.hpp"

namespace akgb {

const char* dt_name(DT d) {
  switch (d) {
    case DT::Bool: return "bool";
    case DT::I8: return "int8";
    case DT::I16: return "int16";
    case DT::I32: return "int32";
    case DT::I64: return "int64";
    case DT::F16: return "float16";
    case DT::F32: return "float32";
    case DT::F64: return "float64";
    case DT::BF16: return "bfloat16";
    default: return "invalid";
  }
}

DT dt_from_name(const std::string& s) {
  if (s == "bool" || s == "int1") return DT::Bool;
  if (s == "int8" || s == "uint8" || s == "sint8") return DT::I8;
  if (s == "int16") return DT::I16;
  if (s == "int32") return DT::I32;
  if (s == "int64") return DT::I64;
  if (s == "float16") return DT::F16;
  if (s == "float32") return DT::F32;
  if (s == "float64") return DT::F64;
  if (s == "bfloat16") return DT::BF16;
  return DT::Invalid;
}

namespace {
struct OpEntry {
  const char* name;
  OpK kind;
};
// JSON operator names the reference's factory knows
// (TranslateToMindsporeDialect.cpp:417-486) that this library places on
// kernels; every other name is kept as OpK::Unknown, like the reference's
// UnknownOp (:939-946), and rejected by the matcher.
const OpEntry kOps[] = {
    {"Abs", OpK::Abs},           {"Neg", OpK::Neg},           {"Exp", OpK::Exp},
    {"Log", OpK::Log},           {"Tanh", OpK::Tanh},         {"Rsqrt", OpK::Rsqrt},
    {"Sqrt", OpK::Sqrt},         {"Reciprocal", OpK::Reciprocal}, {"Floor", OpK::Floor},
    {"Square", OpK::Square},     {"Sin", OpK::Sin},           {"Cos", OpK::Cos},
    {"Asinh", OpK::Asinh},       {"Acosh", OpK::Acosh},       {"Atan", OpK::Atan},
    {"ASin", OpK::ASin},         {"ACos", OpK::ACos},         {"IsInf", OpK::IsInf},
    {"IsFinite", OpK::IsFinite}, {"IsNan", OpK::IsNan},       {"LogicalNot", OpK::LogicalNot},
    {"Cast", OpK::Cast},         {"Add", OpK::Add},           {"TensorAdd", OpK::Add},
    {"Sub", OpK::Sub},           {"Mul", OpK::Mul},           {"Div", OpK::Div},
    {"RealDiv", OpK::Div},       {"Maximum", OpK::Maximum},   {"Minimum", OpK::Minimum},
    {"Pow", OpK::Pow},           {"Atan2", OpK::Atan2},       {"Equal", OpK::Equal},
    {"NotEqual", OpK::NotEqual}, {"Greater", OpK::Greater},   {"GreaterEqual", OpK::GreaterEqual},
    {"Less", OpK::Less},         {"LessEqual", OpK::LessEqual}, {"LogicalAnd", OpK::LogicalAnd},
    {"LogicalOr", OpK::LogicalOr}, {"Select", OpK::Select},   {"BroadcastTo", OpK::BroadcastTo},
    {"Reshape", OpK::Reshape},   {"Transpose", OpK::Transpose}, {"ReduceSum", OpK::ReduceSum},
    {"ReduceMax", OpK::ReduceMax}, {"ReduceMin", OpK::ReduceMin}, {"ReducePrd", OpK::ReduceProd},
    {"ReduceProd", OpK::ReduceProd}, {"ReduceAll", OpK::ReduceAll}, {"ReduceAny", OpK::ReduceAny},
    {"ElemAny", OpK::ReduceAny}, {"MatMul", OpK::MatMul},     {"BatchMatMul", OpK::BatchMatMul},
    {"Assign", OpK::Assign},     {"InplaceAssign", OpK::Assign}, {"AddN", OpK::AddN},
    {"Tile", OpK::Tile},         {"Slice", OpK::Slice},       {"StridedSlice", OpK::StridedSlice},
    {"Concat", OpK::Concat},     {"Gather", OpK::Gather},     {"UnsortedSegmentSum", OpK::UnsortedSegmentSum},
    {"ArgMax", OpK::ArgMax},     {"Pad", OpK::Pad},
};
}  // namespace

const char* opk_name(OpK k) {
  for (auto& e : kOps)
    if (e.kind == k) return e.name;
  return "Unknown";
}
bool opk_is_unary(OpK k) { return (int)k >= (int)OpK::Abs && (int)k <= (int)OpK::Cast; }
bool opk_is_binary(OpK k) { return (int)k >= (int)OpK::Add && (int)k <= (int)OpK::LogicalOr; }
bool opk_is_reduce(OpK k) { return (int)k >= (int)OpK::ReduceSum && (int)k <= (int)OpK::ReduceAny; }
bool opk_is_elementwise(OpK k) { return opk_is_unary(k) || opk_is_binary(k) || k == OpK::Select || k == OpK::AddN; }

namespace {

std::vector<int64_t> shape_of(const Json& d) {
  // a missing "shape" means [1] (TranslateToMindsporeDialect.cpp:322-325)
  if (!d.contains("shape")) return {1};
  std::vector<int64_t> s = d.at("shape").as_int_list();
  if (s.empty()) s.push_back(1);
  // element counts are 64-bit throughout: a tensor of more than 2^46 elements (0.5 PB of float64) is refused here, so
  // that no product of extents overflows further down
  long double n = 1;
  for (auto x : s) {
    if (x < -1) throw JsonError("negative extent");
    if (x > 0) n *= (long double)x;
  }
  if (n > 70368744177664.0L) throw Unsupported("tensor of more than 2^46 elements");
  return s;
}

// "symbolic_shape": a list with one entry per dim, symbols ("s0") or numbers, as strings or integers
// (TranslateToMindsporeDialect.cpp:64, :322-335)
std::vector<std::string> symbols_of(const Json& d) {
  std::vector<std::string> out;
  const Json* s = d.find("symbolic_shape");
  if (!s || !s->is_array()) return out;
  for (auto& e : s->arr) {
    if (e.is_string()) out.push_back(e.str);
    else if (e.is_number()) out.push_back(std::to_string(e.as_int()));
    else out.push_back("");
  }
  return out;
}

// Integer expression over symbols: + - * / (floor division of non-negative values), parentheses, integer literals.
// `lookup` returns false for a symbol without a value yet, which makes the whole evaluation fail (return false).
struct SymExpr {
  const std::string& t;
  size_t i = 0;
  const std::map<std::string, int64_t>& env;
  bool ok = true;
  void ws() {
    while (i < t.size() && (t[i] == ' ' || t[i] == '\t')) ++i;
  }
  int64_t atom() {
    ws();
    if (i < t.size() && t[i] == '(') {
      ++i;
      const int64_t v = sum();
      ws();
      if (i < t.size() && t[i] == ')') ++i;
      else ok = false;
      return v;
    }
    if (i < t.size() && t[i] == '-') {
      ++i;
      return -atom();
    }
    if (i < t.size() && t[i] >= '0' && t[i] <= '9') {
      int64_t v = 0;
      while (i < t.size() && t[i] >= '0' && t[i] <= '9') v = v * 10 + (t[i++] - '0');
      return v;
    }
    std::string name;
    while (i < t.size() && (std::isalnum((unsigned char)t[i]) || t[i] == '_')) name += t[i++];
    auto it = env.find(name);
    if (name.empty() || it == env.end()) {
      ok = false;
      return 0;
    }
    return it->second;
  }
  int64_t product() {
    int64_t v = atom();
    for (;;) {
      ws();
      if (i < t.size() && t[i] == '*') {
        ++i;
        v *= atom();
      } else if (i < t.size() && t[i] == '/') {
        ++i;
        if (i < t.size() && t[i] == '/') ++i;  // "//"
        const int64_t d = atom();
        if (d == 0) {
          ok = false;
          return 0;
        }
        v = v / d;
      } else {
        return v;
      }
    }
  }
  int64_t sum() {
    int64_t v = product();
    for (;;) {
      ws();
      if (i < t.size() && t[i] == '+') {
        ++i;
        v += product();
      } else if (i < t.size() && t[i] == '-') {
        ++i;
        v -= product();
      } else {
        return v;
      }
    }
  }
};
bool eval_symbol_expr(const std::string& text, const std::map<std::string, int64_t>& env, int64_t* out) {
  SymExpr e{text, 0, env};
  const int64_t v = e.sum();
  e.ws();
  if (!e.ok || e.i != text.size()) return false;
  *out = v;
  return true;
}

const Json* find_attr(const Json& attrs, const char* name) {
  if (!attrs.is_array()) return nullptr;
  for (auto& a : attrs.arr) {
    if (a.is_object() && a.contains("name") && a.at("name").is_string() && a.at("name").str == name &&
        a.contains("value"))
      return &a.at("value");
  }
  return nullptr;
}

// Ops whose second operand carries an attribute as a 1-D constant
// (TranslateToMindsporeDialect.cpp:123-125).
bool attr_as_second_input(const std::string& op) {
  static const char* k[] = {"Reshape",   "BroadcastTo", "ReduceMax", "ReduceMin", "ReduceSum", "ReducePrd",
                            "ReduceAll", "ReduceAny",   "ArgMax",    "Transpose", "Tile"};
  for (auto s : k)
    if (op == s) return true;
  return false;
}

}  // namespace

Graph parse_info(const char* text, size_t len) {
  Json root = Json::parse(text, len);
  if (!root.is_object()) throw JsonError("top level must be an object");
  Graph g;
  g.sha256_hex = sha256_hex(text, len);
  g.kernel_name = root.at("op").as_string();
  g.process = root.at("process").as_string();
  if (const Json* ti = root.find("target_info")) {
    if (ti->is_object() && ti->contains("compute_capability") && ti->at("compute_capability").is_string())
      g.compute_capability = ti->at("compute_capability").str;
  }
  // symbol_calc_expr (TranslateToMindsporeDialect.cpp:59, :575-580): symbol -> expression, kept for bind_shapes
  if (const Json* sc = root.find("symbol_calc_expr")) {
    if (sc->is_object())
      for (auto& kv : sc->obj) {
        if (kv.second.is_string()) g.symbol_expr.emplace_back(kv.first, kv.second.str);
        else if (kv.second.is_number()) g.symbol_expr.emplace_back(kv.first, std::to_string(kv.second.as_int()));
        else if (kv.second.is_array() && kv.second.size() == 1 && kv.second[0].is_string())
          g.symbol_expr.emplace_back(kv.first, kv.second[0].str);
      }
  }

  std::map<std::string, int> by_name;
  auto new_value = [&](const std::string& name, std::vector<int64_t> shape, DT dt) {
    Value v;
    v.name = name;
    v.shape = std::move(shape);
    v.dt = dt;
    g.values.push_back(std::move(v));
    return (int)g.values.size() - 1;
  };

  // inputs: a list of one-element lists
  const Json& ind = root.at("input_desc");
  if (!ind.is_null()) {
    if (!ind.is_array()) throw JsonError("input_desc must be a list");
    for (size_t i = 0; i < ind.size(); ++i) {
      const Json& d = ind[i].is_array() ? ind[i][0] : ind[i];
      DT dt = dt_from_name(d.at("data_type").as_string());
      if (dt == DT::Invalid) throw Unsupported("data type '" + d.at("data_type").str + "' is not supported");
      const std::string& name = d.at("tensor_name").as_string();
      int id = new_value(name, shape_of(d), dt);
      g.values[id].input_index = (int)i;
      g.values[id].sym = symbols_of(d);
      if (d.contains("value") && d.at("value").is_number()) {
        // a graph input with a literal value stays a runtime argument (the
        // harness materialises it with np.full) — keep the value for matching
        g.values[id].cval = {d.at("value").as_double()};
      }
      by_name[name] = id;
      g.inputs.push_back(id);
    }
  }

  const Json& ops = root.at("op_desc");
  if (!ops.is_array()) throw JsonError("op_desc must be a list");
  for (size_t i = 0; i < ops.size(); ++i) {
    const Json& od = ops[i];
    Node n;
    n.name = od.at("name").as_string();
    n.kind = OpK::Unknown;
    for (auto& e : kOps)
      if (n.name == e.name) n.kind = e.kind;
    static const Json kNull;
    const Json& attrs = od.contains("attr") ? od.at("attr") : kNull;
    const Json& ins = od.at("input_desc");
    const Json& outs = od.at("output_desc");
    if (!ins.is_array() || ins.size() == 0) throw JsonError("op '" + n.name + "' has no input_desc");
    if (!outs.is_array() || outs.size() == 0) throw JsonError("op '" + n.name + "' has no output_desc");
    // fake_output: the result takes shape and type of the first operand and only the name of the declared output
    // (TranslateToMindsporeDialect.cpp:348-365)
    bool fake_output = false;
    if (const Json* fo = find_attr(attrs, "fake_output")) fake_output = fo->is_bool() && fo->b;

    // Concat and AddN list all their tensors inside the first input entry
    // (TranslateToMindsporeDialect.cpp:719-727, :766-783); StridedSlice may carry begin/end/strides as inputs 1..3
    std::vector<const Json*> operand_descs;
    if ((n.kind == OpK::Concat || n.kind == OpK::AddN) && ins[0].is_array()) {
      for (auto& e : ins[0].arr) operand_descs.push_back(&e);
    } else {
      for (size_t j = 0; j < ins.size(); ++j) {
        if (j == 1 && attr_as_second_input(n.name)) continue;  // attribute operand, read below
        if (j >= 1 && n.kind == OpK::StridedSlice) continue;
        if (j >= 2 && (n.kind == OpK::Gather || n.kind == OpK::UnsortedSegmentSum)) continue;  // axis / num_segments
        if (j >= 1 && n.kind == OpK::Cast) continue;  // a type id some producers append; the result type decides
        operand_descs.push_back(ins[j].is_array() ? &ins[j][0] : &ins[j]);
      }
    }
    for (const Json* dp : operand_descs) {
      const Json& d = *dp;
      const std::string& tn = d.at("tensor_name").as_string();
      auto it = by_name.find(tn);
      bool has_value = d.contains("value") && !d.at("value").is_null();
      if (it != by_name.end() && !(has_value && g.values[it->second].is_const)) {
        n.in.push_back(it->second);
        continue;
      }
      // an operand no earlier op or input defines is a constant (:776-789)
      if (!has_value) throw JsonError("operand '" + tn + "' of op '" + n.name + "' is undefined");
      DT dt = dt_from_name(d.at("data_type").as_string());
      if (dt == DT::Invalid) throw Unsupported("data type '" + d.at("data_type").str + "' is not supported");
      int id = new_value(tn, shape_of(d), dt);
      g.values[id].is_const = true;
      const Json& val = d.at("value");
      if (val.is_number() || val.is_bool()) g.values[id].cval = {val.as_double()};
      else if (val.is_array())
        for (auto& e : val.arr) g.values[id].cval.push_back(e.as_double());
      else throw JsonError("constant operand '" + tn + "' has a non-numeric value");
      // constants are not entered in by_name: two ops may reuse a name with different literals
      n.in.push_back(id);
    }

    const Json& o0 = outs[0];
    const Json& first_in = ins[0].is_array() ? ins[0][0] : ins[0];
    const Json& otype = fake_output ? first_in : o0;
    DT odt = dt_from_name(otype.at("data_type").as_string());
    if (odt == DT::Invalid) throw Unsupported("data type '" + otype.at("data_type").str + "' is not supported");
    int out_id = new_value(o0.at("tensor_name").as_string(), shape_of(otype), odt);
    g.values[out_id].producer = (int)g.nodes.size();
    n.out = out_id;

    const Json& in0 = ins[0].is_array() ? ins[0][0] : ins[0];
    int64_t in_rank = (int64_t)shape_of(in0).size();
    if (opk_is_reduce(n.kind) || n.kind == OpK::ArgMax) {
      // axes from the second operand or the "axis" attribute; negatives wrap
      // (TranslateToMindsporeDialect.cpp:1282-1300); keep_dims defaults to false (:1302)
      std::vector<int64_t> ax;
      if (ins.size() == 2) {
        const Json& d1 = ins[1].is_array() ? ins[1][0] : ins[1];
        ax = d1.at("value").as_int_list();
      } else if (n.name == "ElemAny") {
        for (int64_t a = 0; a < in_rank; ++a) ax.push_back(a);
      } else if (const Json* a = find_attr(attrs, "axis")) {
        ax = a->as_int_list();
      } else {
        throw JsonError("reduction '" + n.name + "' has no axis");
      }
      if (ax.empty())
        for (int64_t a = 0; a < in_rank; ++a) ax.push_back(a);
      for (auto& a : ax) {
        if (a < 0) a += in_rank;
        if (a < 0 || a >= in_rank) throw JsonError("reduction axis out of range");
      }
      std::sort(ax.begin(), ax.end());
      ax.erase(std::unique(ax.begin(), ax.end()), ax.end());
      n.axes = ax;
      const Json* kd = find_attr(attrs, "keep_dims");
      n.keep_dims = (n.name == "ElemAny") ? true : (kd ? kd->as_bool() : false);
      const Json* at = find_attr(attrs, "enable_atomic_add");
      n.enable_atomic_add = at ? at->as_bool() : false;
      if (n.kind == OpK::ArgMax) {
        if (n.axes.size() != 1) throw Unsupported("ArgMax over more than one axis");
        n.axis = n.axes[0];
      }
    } else if (n.kind == OpK::Transpose) {
      // perm from the second operand or the "perm" attribute (:965-978)
      if (ins.size() == 2) {
        const Json& d1 = ins[1].is_array() ? ins[1][0] : ins[1];
        n.perm = d1.at("value").as_int_list();
      } else if (const Json* p = find_attr(attrs, "perm")) {
        n.perm = p->as_int_list();
      } else {
        throw JsonError("Transpose has no perm");
      }
      if ((int64_t)n.perm.size() != in_rank) throw JsonError("Transpose perm rank mismatch");
      std::vector<bool> seen(in_rank, false);
      for (auto& p : n.perm) {
        if (p < 0) p += in_rank;
        if (p < 0 || p >= in_rank || seen[p]) throw JsonError("Transpose perm is not a permutation");
        seen[p] = true;
      }
    } else if (n.kind == OpK::MatMul || n.kind == OpK::BatchMatMul) {
      // transpose_a / transpose_b default to false (:1331-1349)
      const Json* ta = find_attr(attrs, "transpose_a");
      const Json* tb = find_attr(attrs, "transpose_b");
      n.transpose_a = ta ? ta->as_bool() : false;
      n.transpose_b = tb ? tb->as_bool() : false;
    } else if (n.kind == OpK::Tile) {
      // multiples from the second operand or the attribute (:1151-1160)
      if (ins.size() == 2) {
        const Json& d1 = ins[1].is_array() ? ins[1][0] : ins[1];
        n.multiples = d1.at("value").as_int_list();
      } else if (const Json* m = find_attr(attrs, "multiples")) {
        n.multiples = m->as_int_list();
      } else {
        throw JsonError("Tile has no multiples");
      }
    } else if (n.kind == OpK::Slice) {
      const Json* b = find_attr(attrs, "begin");
      const Json* sz = find_attr(attrs, "size");
      if (!b || !sz) throw JsonError("Slice needs begin and size");
      n.begin = b->as_int_list();
      n.size = sz->as_int_list();
    } else if (n.kind == OpK::StridedSlice) {
      // begin/end/strides from attributes or inputs 1..3 (:1037-1049); negative ends wrap (:1051-1055)
      auto from = [&](const char* attr_name, size_t idx) {
        if (ins.size() == 1) {
          const Json* a = find_attr(attrs, attr_name);
          if (!a) throw JsonError(std::string("StridedSlice needs ") + attr_name);
          return a->as_int_list();
        }
        if (ins.size() <= idx) throw JsonError("StridedSlice needs begin, end and strides");
        const Json& d = ins[idx].is_array() ? ins[idx][0] : ins[idx];
        return d.at("value").as_int_list();
      };
      n.begin = from("begin", 1);
      n.end = from("end", 2);
      n.strides = from("strides", 3);
      for (const char* mk : {"ellipsis_mask", "new_axis_mask", "shrink_axis_mask", "ellipsisMask", "newAxisMask",
                             "shrinkAxisMask"}) {
        const Json* m = find_attr(attrs, mk);
        if (m && m->as_int() != 0) throw Unsupported("StridedSlice with ellipsis/new-axis/shrink masks");
      }
      auto mask_of = [&](const char* a, const char* b2) {
        const Json* m = find_attr(attrs, a);
        if (!m) m = find_attr(attrs, b2);
        return m ? m->as_int() : (int64_t)0;
      };
      const int64_t bm = mask_of("begin_mask", "beginMask"), em = mask_of("end_mask", "endMask");
      const std::vector<int64_t> xs = shape_of(in0);
      if (n.begin.size() > xs.size() || n.end.size() != n.begin.size() || n.strides.size() != n.begin.size())
        throw JsonError("StridedSlice begin/end/strides disagree");
      for (size_t i = 0; i < n.begin.size(); ++i) {
        if (n.strides[i] <= 0) throw Unsupported("StridedSlice with non-positive strides");
        if (n.begin[i] < 0) n.begin[i] += xs[i];
        if (n.end[i] < 0) n.end[i] += xs[i];
        if ((bm >> i) & 1) n.begin[i] = 0;
        if ((em >> i) & 1) n.end[i] = xs[i];
        n.end[i] = std::min(n.end[i], xs[i]);
      }
      for (size_t i = n.begin.size(); i < xs.size(); ++i) {
        n.begin.push_back(0);
        n.end.push_back(xs[i]);
        n.strides.push_back(1);
      }
    } else if (n.kind == OpK::Gather) {
      // axis from a constant third operand or the attribute; batch_dims must be 0 (MindSporeToLinalg.cpp:543-550)
      if (ins.size() > 2) {
        const Json& d2 = ins[2].is_array() ? ins[2][0] : ins[2];
        n.axis = d2.at("value").as_int();
      } else if (const Json* a = find_attr(attrs, "axis")) {
        n.axis = a->as_int();
      }
      if (n.axis < 0) n.axis += in_rank;
      const Json* bd = find_attr(attrs, "batch_dims");
      if (bd && bd->as_int() != 0) throw Unsupported("Gather with batch_dims != 0");
    } else if (n.kind == OpK::UnsortedSegmentSum) {
      if (ins.size() > 2) {
        const Json& d2 = ins[2].is_array() ? ins[2][0] : ins[2];
        n.num_segments = d2.at("value").as_int();
      } else if (const Json* a = find_attr(attrs, "num_segments")) {
        n.num_segments = a->as_int();
      } else if (const Json* a2 = find_attr(attrs, "numSegments")) {
        n.num_segments = a2->as_int();
      }
      if (n.num_segments <= 0) throw JsonError("UnsortedSegmentSum needs num_segments");
    } else if (n.kind == OpK::Concat) {
      const Json* a = find_attr(attrs, "axis");
      n.axis = a ? a->as_int() : 0;
      if (n.axis < 0) n.axis += in_rank;
    } else if (n.kind == OpK::Pad) {
      // Two spellings: the factory reads "padding" = [low, high] pairs starting at the LAST dimension and an integer
      // "value" (TranslateToMindsporeDialect.cpp:1168-1180, MindSporeToTosa.cpp:339-357); the expected-value generator
      // reads "head"/"tail" per dimension and "pad_val" (op_dsl.py:623-634). Mode is constant in both.
      n.pad_low.assign(in_rank, 0);
      n.pad_high.assign(in_rank, 0);
      if (const Json* pd = find_attr(attrs, "padding")) {
        std::vector<int64_t> v = pd->as_int_list();
        if (v.size() % 2 || (int64_t)v.size() / 2 > in_rank) throw JsonError("Pad: bad padding list");
        for (size_t i = 0; i < v.size() / 2; ++i) {
          n.pad_low[in_rank - 1 - i] = v[2 * i];
          n.pad_high[in_rank - 1 - i] = v[2 * i + 1];
        }
        if (const Json* pv = find_attr(attrs, "value")) n.pad_value = pv->as_double();
      } else {
        const Json* hd = find_attr(attrs, "head");
        const Json* tl = find_attr(attrs, "tail");
        if (!hd || !tl) throw JsonError("Pad needs padding, or head and tail");
        n.pad_low = hd->as_int_list();
        n.pad_high = tl->as_int_list();
        if ((int64_t)n.pad_low.size() != in_rank || (int64_t)n.pad_high.size() != in_rank)
          throw JsonError("Pad: head/tail rank differs from the input");
        if (const Json* pv = find_attr(attrs, "pad_val")) n.pad_value = pv->as_double();
      }
      if (const Json* md = find_attr(attrs, "mode"))
        if (md->is_string() && md->str != "constant") throw Unsupported("Pad mode '" + md->str + "'");
      for (int64_t i = 0; i < in_rank; ++i)
        if (n.pad_low[i] < 0 || n.pad_high[i] < 0) throw Unsupported("Pad with negative widths");
    }
    if (n.name == "Split") {
      // One Slice per entry of output_desc; the extents along the axis come from the declared output shapes, which both
      // attribute spellings ("split_size_or_sections", :1206-1233; "output_num", op_dsl.py:416-425) must agree with.
      if (n.in.size() != 1) throw JsonError("Split takes one tensor");
      const Json* a = find_attr(attrs, "axis");
      int64_t axis = a ? a->as_int() : 0;
      if (axis < 0) axis += in_rank;
      if (axis < 0 || axis >= in_rank) throw JsonError("Split axis out of range");
      const std::vector<int64_t> xs = shape_of(in0);
      int64_t pos = 0;
      for (size_t k = 0; k < outs.size(); ++k) {
        Node sl;
        sl.name = "Slice";
        sl.kind = OpK::Slice;
        sl.in = n.in;
        int oid = out_id;
        if (k > 0) {
          DT kdt = dt_from_name(outs[k].at("data_type").as_string());
          if (kdt != odt) throw JsonError("Split outputs must share the input type");
          oid = new_value(outs[k].at("tensor_name").as_string(), shape_of(outs[k]), kdt);
        }
        const std::vector<int64_t>& os = g.values[oid].shape;
        if ((int64_t)os.size() != in_rank) throw JsonError("Split output rank differs from the input");
        sl.begin.assign(in_rank, 0);
        sl.begin[axis] = pos;
        sl.size = os;
        pos += os[axis];
        g.values[oid].producer = (int)g.nodes.size();
        sl.out = oid;
        by_name[g.values[oid].name] = oid;
        for (int vid : sl.in) g.values[vid].users.push_back((int)g.nodes.size());
        g.nodes.push_back(std::move(sl));
      }
      if (pos != xs[axis]) throw JsonError("Split extents do not add up to the input");
      continue;
    }
    by_name[g.values[out_id].name] = out_id;
    for (int vid : n.in) g.values[vid].users.push_back((int)g.nodes.size());
    g.nodes.push_back(std::move(n));
  }

  const Json& outd = root.at("output_desc");
  if (!outd.is_array() || outd.size() == 0) throw JsonError("output_desc must be a non-empty list");
  for (size_t i = 0; i < outd.size(); ++i) {
    const Json& d = outd[i];
    const std::string& name = d.at("tensor_name").as_string();
    auto it = by_name.find(name);
    if (it == by_name.end()) throw JsonError("output '" + name + "' is not produced by any op");
    if (g.values[it->second].output_index >= 0) {
      // listed twice: the second caller buffer receives a copy (a Reshape to the same shape, planned as a copy)
      const int src = it->second;
      Node cp;
      cp.name = "Reshape";
      cp.kind = OpK::Reshape;
      cp.in = {src};
      const int dup = new_value(name + "#" + std::to_string(i), g.values[src].shape, g.values[src].dt);
      g.values[dup].producer = (int)g.nodes.size();
      cp.out = dup;
      g.values[src].users.push_back((int)g.nodes.size());
      g.nodes.push_back(std::move(cp));
      g.values[dup].output_index = (int)i;
      g.outputs.push_back(dup);
      continue;
    }
    Value& v = g.values[it->second];
    v.output_index = (int)i;
    v.sym = symbols_of(d);
    // the declared output shape may differ from the op's by a trailing view
    // change only; keep the op's shape when the element counts agree
    std::vector<int64_t> s = shape_of(d);
    int64_t n = 1;
    bool unknown = false;
    for (auto x : s) {
      n *= x;
      unknown |= x < 0;
    }
    for (auto x : v.shape) unknown |= x < 0;
    if (!unknown && n != v.numel()) throw JsonError("output '" + name + "' shape disagrees with its producer");
    g.outputs.push_back(it->second);
  }
  for (auto& v : g.values)
    for (auto x : v.shape)
      if (x < 0) g.dynamic = true;
  classify(g);
  return g;
}

void classify(Graph& g) {
  OpClass c = OpClass::Elementwise;
  ReduceDir dir = ReduceDir::None;
  for (auto& n : g.nodes) {
    OpClass oc = OpClass::Elementwise;
    if (opk_is_elementwise(n.kind)) {
      // Elementwise when every operand has the result's shape, else Broadcast
      // (OperatorIdentify.cpp:38-60)
      bool same = true;
      for (int vid : n.in)
        if (g.v(vid).shape != g.v(n.out).shape) same = false;
      oc = same ? OpClass::Elementwise : OpClass::Broadcast;
    } else if (n.kind == OpK::BroadcastTo || n.kind == OpK::Tile) {
      oc = OpClass::Broadcast;  // tosa.tile counts as Broadcast (OperatorIdentify.cpp:61-62)
    } else if (n.kind == OpK::Reshape) {
      oc = OpClass::Reshape;
    } else if (n.kind == OpK::Transpose) {
      oc = OpClass::Transpose;
    } else if (opk_is_reduce(n.kind)) {
      oc = OpClass::Reduction;
      int64_t rank = (int64_t)g.v(n.in[0]).shape.size();
      ReduceDir d;
      if ((int64_t)n.axes.size() == rank) d = ReduceDir::All;
      else if (!n.axes.empty() && n.axes.back() == rank - 1) d = ReduceDir::X;
      else d = ReduceDir::Y;
      // the last reduction walked wins, as in the reference's global setter
      dir = d;
    } else if (n.kind == OpK::MatMul || n.kind == OpK::BatchMatMul) {
      oc = OpClass::Matmul;
    }
    if ((int)oc > (int)c) c = oc;
  }
  g.op_class = c;
  g.reduce_dir = dir;
}

void infer_sharding(Graph& g, int rank, int world) {
  if (world <= 1) return;
  if (rank < 0 || rank >= world) throw Unsupported("shard_rank outside [0, shard_world)");
  // The split extent S is axis 0 of the highest-rank, largest graph input.
  int lead = -1;
  for (int vid : g.inputs) {
    const Value& v = g.v(vid);
    if (lead < 0 || v.shape.size() > g.v(lead).shape.size() ||
        (v.shape.size() == g.v(lead).shape.size() && v.numel() > g.v(lead).numel()))
      lead = vid;
  }
  if (lead < 0) throw Unsupported("sharding needs at least one tensor input");
  int64_t S = g.v(lead).shape[0];
  size_t R = g.v(lead).shape.size();

  // With a (Batch)MatMul in the region the split axis is axis 0 of its LEFT operand: the rows of a MatMul, the batch
  // of a BatchMatMul.  Values that reach a right operand which does not carry that batch (the 2-D weight of a MatMul,
  // a BatchMatMul's shared right operand) stay whole on every rank, whatever their extents happen to be.
  bool has_matmul = false;
  std::vector<char> shared_rhs(g.values.size(), 0);
  for (auto& n : g.nodes) {
    if (n.kind != OpK::MatMul && n.kind != OpK::BatchMatMul) continue;
    if (!has_matmul) {
      S = g.v(n.in[0]).shape[0];
      R = g.v(n.in[0]).shape.size();
      has_matmul = true;
    }
    const Value& b = g.v(n.in[1]);
    const bool batched_rhs = n.kind == OpK::BatchMatMul && b.shape.size() >= 3 && b.shape.size() == R && b.shape[0] == S;
    if (!batched_rhs) shared_rhs[n.in[1]] = 1;
  }
  if (has_matmul)
    for (size_t i = g.nodes.size(); i-- > 0;)
      if (shared_rhs[g.nodes[i].out])
        for (int vid : g.nodes[i].in) shared_rhs[vid] = 1;
  if (S % world != 0) throw Unsupported("leading extent is not divisible by shard_world");
  const int64_t Sl = S / world;

  auto mark = [&](Value& v) {
    v.split0 = true;
    v.shape[0] = Sl;
  };
  for (int vid : g.inputs) {
    Value& v = g.v(vid);
    if (has_matmul && shared_rhs[vid]) continue;
    if (v.shape.size() == R && v.shape[0] == S) mark(v);
  }
  for (auto& n : g.nodes) {
    Value& out = g.v(n.out);
    bool any_split = false;
    for (int vid : n.in) {
      if (g.v(vid).partial) throw Unsupported("a reduction over the sharded axis feeds another op: replicas only");
      any_split |= g.v(vid).split0;
    }
    if (!any_split) continue;
    if (opk_is_elementwise(n.kind)) {
      // a replicated operand of full rank with S leading rows would need slicing
      for (int vid : n.in) {
        const Value& v = g.v(vid);
        if (!v.split0 && !v.is_const && v.shape.size() == out.shape.size() && v.shape[0] == S && S != 1)
          throw Unsupported("replicated operand spans the sharded axis");
      }
      mark(out);
    } else if (opk_is_reduce(n.kind)) {
      bool over0 = !n.axes.empty() && n.axes[0] == 0;
      if (!over0) {
        mark(out);
      } else {
        switch (n.kind) {
          case OpK::ReduceSum: out.partial = 2; break;
          case OpK::ReduceMax: out.partial = 3; break;
          case OpK::ReduceMin: out.partial = 4; break;
          case OpK::ReduceProd: out.partial = 5; break;
          default: throw Unsupported("this reduction cannot be split over ranks");
        }
        if (out.output_index < 0)
          throw Unsupported("a reduction over the sharded axis feeds another op: replicas only");
      }
    } else if (n.kind == OpK::Transpose) {
      if (n.perm[0] != 0) throw Unsupported("transpose moves the sharded axis");
      mark(out);
    } else if (n.kind == OpK::Reshape) {
      // a view change that keeps the leading extent keeps the split
      if (out.shape[0] != S) {
        // allow merging/splitting that keeps S as a factor of the leading extent
        if (out.shape[0] % S != 0 && S % out.shape[0] != 0) throw Unsupported("reshape mixes the sharded axis");
        if (out.shape[0] % world != 0) throw Unsupported("reshape mixes the sharded axis");
        out.split0 = true;
        out.shape[0] /= world;
      } else {
        mark(out);
      }
    } else if (n.kind == OpK::MatMul || n.kind == OpK::BatchMatMul) {
      if (n.transpose_a) throw Unsupported("transpose_a matmul cannot be split on rows");
      const Value& lhs = g.v(n.in[0]);
      const Value& rhs = g.v(n.in[1]);
      if (!lhs.split0) throw Unsupported("the left matmul operand is not split over the ranks");
      if (rhs.split0 && n.kind == OpK::MatMul) throw Unsupported("right matmul operand is split");
      if (n.kind == OpK::BatchMatMul && rhs.shape.size() >= 3) {
        // a batched right operand must carry this rank's batch entries, like the left one
        if (!rhs.split0 || rhs.shape[0] != lhs.shape[0])
          throw Unsupported("the batched right operand of a BatchMatMul is not split like the left one");
      }
      mark(out);
    } else if (n.kind == OpK::BroadcastTo) {
      mark(out);
    } else {
      throw Unsupported(std::string("op '") + n.name + "' cannot be sharded");
    }
  }
  (void)rank;
}

namespace {
void merge_shape(std::vector<int64_t>& have, const std::vector<int64_t>& inferred, const std::string& what) {
  if (have.size() != inferred.size()) {
    // a declared shape of another rank wins only when it is fully known (e.g. Reshape targets)
    for (auto x : have)
      if (x < 0) throw JsonError("cannot infer the shape of '" + what + "'");
    return;
  }
  for (size_t i = 0; i < have.size(); ++i) {
    if (have[i] < 0) have[i] = inferred[i];
    else if (inferred[i] >= 0 && have[i] != inferred[i])
      throw JsonError("shape of '" + what + "' contradicts the launch-time extents");
  }
}
}  // namespace

Graph bind_shapes(const Graph& src, const std::vector<std::vector<int64_t>>& shapes) {
  Graph g = src;
  if (shapes.size() != g.inputs.size() + g.outputs.size()) throw JsonError("bind_shapes: wrong number of arguments");
  auto bind_arg = [&](int vid, const std::vector<int64_t>& given) {
    Value& v = g.v(vid);
    if (given.size() != v.shape.size()) throw JsonError("argument '" + v.name + "': rank differs from the description");
    for (size_t i = 0; i < given.size(); ++i) {
      if (given[i] < 0) throw JsonError("argument '" + v.name + "': negative extent");
      if (v.shape[i] >= 0 && v.shape[i] != given[i])
        throw JsonError("argument '" + v.name + "': extent differs from the static extent of the description");
      v.shape[i] = given[i];
    }
  };
  for (size_t i = 0; i < g.inputs.size(); ++i) bind_arg(g.inputs[i], shapes[i]);
  for (size_t i = 0; i < g.outputs.size(); ++i) bind_arg(g.outputs[i], shapes[g.inputs.size() + i]);
  // Symbols: a symbol names ONE extent.  The inputs define them, symbol_calc_expr derives further ones (an output
  // extent as an expression of input extents), and every argument dim that carries a symbol must agree.
  {
    std::map<std::string, int64_t> env;
    auto is_number = [](const std::string& t) {
      if (t.empty()) return false;
      for (char ch : t)
        if (ch < '0' || ch > '9') return false;
      return true;
    };
    auto visit = [&](int vid, bool define) {
      const Value& v = g.v(vid);
      if (v.sym.size() != v.shape.size()) return;  // no (or a malformed) symbolic_shape: nothing to check
      for (size_t d = 0; d < v.sym.size(); ++d) {
        const std::string& t = v.sym[d];
        if (t.empty()) continue;
        if (is_number(t)) {
          if (std::stoll(t) != v.shape[d])
            throw JsonError("argument '" + v.name + "': dim " + std::to_string(d) + " is declared as " + t);
          continue;
        }
        auto it = env.find(t);
        if (it == env.end()) {
          if (define) env[t] = v.shape[d];
        } else if (it->second != v.shape[d]) {
          throw JsonError("argument '" + v.name + "': symbol '" + t + "' is bound to " + std::to_string(it->second) +
                          " by another dim but this dim has " + std::to_string(v.shape[d]));
        }
      }
    };
    for (int vid : g.inputs) visit(vid, true);
    bool progress = true;
    while (progress) {  // expressions may build on one another, in any order
      progress = false;
      for (auto& kv : g.symbol_expr) {
        if (env.count(kv.first)) continue;
        int64_t val = 0;
        if (eval_symbol_expr(kv.second, env, &val)) {
          env[kv.first] = val;
          progress = true;
        }
      }
    }
    for (auto& kv : g.symbol_expr) {  // a symbol that an input also carries must agree with its expression
      int64_t val = 0;
      auto it = env.find(kv.first);
      if (it != env.end() && eval_symbol_expr(kv.second, env, &val) && val != it->second)
        throw JsonError("symbol '" + kv.first + "' = " + kv.second + " evaluates to " + std::to_string(val) +
                        " but is bound to " + std::to_string(it->second));
    }
    for (int vid : g.outputs) visit(vid, true);
  }
  for (auto& n : g.nodes) {
    Value& out = g.v(n.out);
    std::vector<int64_t> inf;
    const std::vector<int64_t>& x = g.v(n.in[0]).shape;
    for (int vid : n.in)
      for (auto e : g.v(vid).shape)
        if (e < 0) throw JsonError("cannot infer the shape of operand '" + g.v(vid).name + "'");
    if (opk_is_elementwise(n.kind)) {
      size_t rank = 0;
      for (int vid : n.in) rank = std::max(rank, g.v(vid).shape.size());
      inf.assign(rank, 1);
      for (int vid : n.in) {
        const auto& s = g.v(vid).shape;
        for (size_t i = 0; i < s.size(); ++i) {
          int64_t& d = inf[rank - s.size() + i];
          if (d == 1) d = s[i];
          else if (s[i] != 1 && s[i] != d) throw JsonError("operands of '" + n.name + "' do not broadcast");
        }
      }
    } else if (opk_is_reduce(n.kind)) {
      std::vector<bool> red(x.size(), false);
      for (auto a : n.axes) red[a] = true;
      for (size_t i = 0; i < x.size(); ++i) {
        if (!red[i]) inf.push_back(x[i]);
        else if (n.keep_dims) inf.push_back(1);
      }
      if (inf.empty()) inf.push_back(1);
    } else if (n.kind == OpK::ArgMax) {
      for (size_t i = 0; i < x.size(); ++i) {
        if ((int64_t)i != n.axis) inf.push_back(x[i]);
        else if (n.keep_dims) inf.push_back(1);
      }
      if (inf.empty()) inf.push_back(1);
    } else if (n.kind == OpK::Pad) {
      for (size_t i = 0; i < x.size(); ++i) inf.push_back(x[i] + n.pad_low[i] + n.pad_high[i]);
    } else if (n.kind == OpK::Transpose) {
      for (auto p : n.perm) inf.push_back(x[p]);
    } else if (n.kind == OpK::MatMul || n.kind == OpK::BatchMatMul) {
      const auto& b = g.v(n.in[1]).shape;
      inf.assign(x.begin(), x.end() - 1);
      inf.push_back(n.transpose_b ? b[b.size() - 2] : b[b.size() - 1]);
    } else if (n.kind == OpK::Tile) {
      for (size_t i = 0; i < x.size(); ++i) inf.push_back(x[i] * (i < n.multiples.size() ? n.multiples[i] : 1));
    } else if (n.kind == OpK::Gather) {
      const auto& ix = g.v(n.in[1]).shape;
      inf.assign(x.begin(), x.begin() + n.axis);
      inf.insert(inf.end(), ix.begin(), ix.end());
      inf.insert(inf.end(), x.begin() + n.axis + 1, x.end());
    } else if (n.kind == OpK::UnsortedSegmentSum) {
      const auto& ix = g.v(n.in[1]).shape;
      inf.push_back(n.num_segments);
      inf.insert(inf.end(), x.begin() + ix.size(), x.end());
    } else if (n.kind == OpK::Concat) {
      inf = x;
      inf[n.axis] = 0;
      for (int vid : n.in) inf[n.axis] += g.v(vid).shape[n.axis];
    } else if (n.kind == OpK::Reshape || n.kind == OpK::BroadcastTo) {
      // the target is the declared output shape; one unknown extent follows from the element count
      inf = out.shape;
      int unknown = -1;
      int64_t known = 1;
      for (size_t i = 0; i < inf.size(); ++i) {
        if (inf[i] < 0) {
          if (unknown >= 0) throw JsonError("cannot infer the shape of '" + out.name + "'");
          unknown = (int)i;
        } else {
          known *= inf[i];
        }
      }
      if (unknown >= 0) {
        if (n.kind != OpK::Reshape || known == 0) throw JsonError("cannot infer the shape of '" + out.name + "'");
        int64_t total = 1;
        for (auto e : x) total *= e;
        inf[unknown] = total / known;
      }
    } else {
      inf = out.shape;  // Slice / StridedSlice and the rest: static extents only
    }
    merge_shape(out.shape, inf, out.name);
    for (auto e : out.shape)
      if (e < 0) throw JsonError("cannot infer the shape of '" + out.name + "'");
  }
  g.dynamic = false;
  classify(g);
  return g;
}

// ----------------------------------------------------------------------------
// SHA-256 (FIPS 180-4) of the description text; the reference stamps the same
// digest of its kernel file into the metadata JSON (mlir_driver.py:776-815).
namespace {
inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
}  // namespace

std::string sha256_hex(const char* data, size_t len) {
  static const uint32_t K[64] = {
      0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5,
      0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174,
      0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da,
      0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967,
      0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
      0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070,
      0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
      0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
  uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  std::vector<uint8_t> msg(data, data + len);
  msg.push_back(0x80);
  while (msg.size() % 64 != 56) msg.push_back(0);
  uint64_t bits = (uint64_t)len * 8;
  for (int i = 7; i >= 0; --i) msg.push_back((uint8_t)(bits >> (8 * i)));
  for (size_t off = 0; off < msg.size(); off += 64) {
    uint32_t w[64];
    for (int i = 0; i < 16; ++i)
      w[i] = (uint32_t)msg[off + 4 * i] << 24 | (uint32_t)msg[off + 4 * i + 1] << 16 |
             (uint32_t)msg[off + 4 * i + 2] << 8 | (uint32_t)msg[off + 4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], gg = h[6], hh = h[7];
    for (int i = 0; i < 64; ++i) {
      uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25);
      uint32_t ch = (e & f) ^ (~e & gg);
      uint32_t t1 = hh + S1 + ch + K[i] + w[i];
      uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22);
      uint32_t mj = (a & b) ^ (a & c) ^ (b & c);
      uint32_t t2 = S0 + mj;
      hh = gg; gg = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += gg; h[7] += hh;
  }
  static const char* hex = "0123456789abcdef";
  std::string out;
  for (int i = 0; i < 8; ++i)
    for (int j = 28; j >= 0; j -= 4) out.push_back(hex[(h[i] >> j) & 0xF]);
  return out;
}

}  // namespace akgb
