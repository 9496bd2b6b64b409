// Regions in which a reduction over the sharded (leading) axis feeds later ops -- batch-norm statistics, a LayerNorm
// over axis 0, a global scale taken from the tensor itself -- cannot run as one data-parallel kernel: the reduced value
// must be complete on every rank before the ops behind it run.  This file cuts such a region into STAGES at those
// reductions.  A stage is a region of its own whose partial results are outputs; the exchange step (an all-reduce of
// those outputs) runs between stages, and the next stage reads the completed values as ordinary, replicated inputs.
// Full-size elementwise values of an earlier stage that a later stage needs (the centred values x - mean) are computed
// again there instead of crossing through memory, exactly as the single-GPU planner does when it cuts a region at its
// reductions.
//
// The reference has no counterpart: it compiles a fused region for one device
// (akg-mlir/python/akg_mlir/utils/code_template.py:181).  The shapes of the chains handled here are the reference's own
// (reduce, then broadcast back: akg-mlir/lib/Conversion/MindSporeToLinalg/MindSporeToLinalg.cpp:1333-1451, :432-459).
#include <algorithm>
#include <set>

#include "graph.hpp"

namespace akgb {
namespace {

void relink_values(Graph& g) {
  for (auto& v : g.values) {
    v.producer = -1;
    v.users.clear();
  }
  for (size_t i = 0; i < g.nodes.size(); ++i) {
    g.values[g.nodes[i].out].producer = (int)i;
    for (int vid : g.nodes[i].in) g.values[vid].users.push_back((int)i);
  }
}

// Drops the values the stage does not touch (the rest of the region, still at its unsplit shape: the planners look at
// every value of a graph) and renumbers the others.
void drop_unused_values(Graph& g) {
  std::vector<int> remap(g.values.size(), -1);
  std::vector<Value> kept;
  auto keep = [&](int vid) {
    if (remap[vid] < 0) {
      remap[vid] = (int)kept.size();
      kept.push_back(g.values[vid]);
    }
  };
  for (int vid : g.inputs) keep(vid);
  for (auto& nd : g.nodes) {
    for (int vid : nd.in) keep(vid);
    keep(nd.out);
  }
  for (int vid : g.outputs) keep(vid);
  for (auto& nd : g.nodes) {
    for (int& vid : nd.in) vid = remap[vid];
    nd.out = remap[nd.out];
  }
  for (int& vid : g.inputs) vid = remap[vid];
  for (int& vid : g.outputs) vid = remap[vid];
  g.values = std::move(kept);
  relink_values(g);
}

}  // namespace

bool split_at_sharded_reductions(const Graph& g, StagePlan* out) {
  const int n = (int)g.nodes.size();
  if (g.dynamic || n == 0) return false;
  for (auto& nd : g.nodes)
    if (nd.kind == OpK::Assign || nd.kind == OpK::MatMul || nd.kind == OpK::BatchMatMul || nd.kind == OpK::Unknown) return false;
  // the split extent: axis 0 of the highest-rank, largest input (as infer_sharding)
  int lead = -1;
  for (int vid : g.inputs) {
    const Value& v = g.v(vid);
    if (lead < 0 || v.shape.size() > g.v(lead).shape.size() ||
        (v.shape.size() == g.v(lead).shape.size() && v.numel() > g.v(lead).numel()))
      lead = vid;
  }
  if (lead < 0 || g.v(lead).shape.empty()) return false;
  const int64_t S = g.v(lead).shape[0];
  const size_t R = g.v(lead).shape.size();
  // which values carry the split axis, which reductions fold it
  std::vector<char> spans(g.values.size(), 0), cut(n, 0);
  for (int vid : g.inputs) {
    const Value& v = g.v(vid);
    spans[vid] = v.shape.size() == R && v.shape[0] == S;
  }
  for (int i = 0; i < n; ++i) {
    const Node& nd = g.nodes[i];
    bool any = false;
    for (int vid : nd.in) any = any || spans[vid];
    if (!any) continue;
    if (opk_is_reduce(nd.kind) && !nd.axes.empty() && nd.axes[0] == 0 && spans[nd.in[0]]) {
      cut[i] = 1;  // folds the split axis: its result is a per-rank partial
      continue;
    }
    spans[nd.out] = 1;
  }
  // a value's stage counts the cuts on the longest path that leads to it
  std::vector<int> stage(n, 0);
  int last_stage = 0;
  bool feeds = false;
  for (int i = 0; i < n; ++i) {
    int st = 0;
    for (int vid : g.nodes[i].in) {
      const int p = g.v(vid).producer;
      if (p < 0) continue;
      st = std::max(st, stage[p] + (cut[p] ? 1 : 0));
      feeds = feeds || cut[p];
    }
    stage[i] = st;
    last_stage = std::max(last_stage, st);
  }
  if (!feeds) return false;  // nothing reads a partial: the ordinary sharded kernel handles the region
  out->stages.clear();
  out->carried.clear();
  std::map<int, int> carried_index;  // parent value id -> index in out->carried
  for (int t = 0; t <= last_stage; ++t) {
    // what this stage must produce: the partials of its cuts and the region's results that become known here
    std::vector<int> targets;
    for (int i = 0; i < n; ++i) {
      if (stage[i] != t) continue;
      const Value& ov = g.v(g.nodes[i].out);
      if (cut[i] && (!ov.users.empty() || ov.output_index >= 0)) targets.push_back(g.nodes[i].out);
      else if (!cut[i] && ov.output_index >= 0) targets.push_back(g.nodes[i].out);
    }
    if (targets.empty()) continue;
    // ancestors of the targets; completed partials of earlier stages are inputs of this stage
    std::set<int> take;           // node indices
    std::vector<int> stack(targets.begin(), targets.end());
    std::set<int> seen;
    while (!stack.empty()) {
      const int vid = stack.back();
      stack.pop_back();
      if (!seen.insert(vid).second) continue;
      const Value& v = g.v(vid);
      if (v.is_const || v.producer < 0) continue;
      const int p = v.producer;
      if (cut[p] && stage[p] < t) continue;  // arrives completed
      take.insert(p);
      for (int in : g.nodes[p].in) stack.push_back(in);
    }
    StageGraph sg;
    sg.g = g;
    sg.g.nodes.clear();
    // Small elementwise ops that depend only on inputs, completed partials and one another (mean = sum / n, the
    // reciprocal standard deviation from the completed sum of squares) go first, in op order; then the rest, in op
    // order.  In the description they sit between the full-size ops that use them, which would cut the stage into
    // alternating small and large launches; hoisted, the stage is one small launch and one large one.
    int64_t largest = 1;
    for (int i : take) largest = std::max(largest, g.v(g.nodes[i].out).numel());
    std::set<int> hoisted;
    for (int i : take) {  // std::set iterates in op order, so producers are seen before their users
      const Node& nd = g.nodes[i];
      if (!opk_is_elementwise(nd.kind) || g.v(nd.out).numel() * 16 > largest) continue;
      bool ok = true;
      for (int vid : nd.in) {
        const Value& v = g.v(vid);
        if (v.is_const || v.producer < 0) continue;
        const int p = v.producer;
        if (cut[p] && stage[p] < t) continue;  // arrives completed
        ok = ok && hoisted.count(p) != 0;
      }
      if (ok) hoisted.insert(i);
    }
    for (int i : take)
      if (hoisted.count(i)) sg.g.nodes.push_back(g.nodes[i]);
    for (int i : take)
      if (!hoisted.count(i)) sg.g.nodes.push_back(g.nodes[i]);
    relink_values(sg.g);
    for (auto& v : sg.g.values) v.input_index = v.output_index = -1;
    sg.g.inputs.clear();
    sg.g.outputs.clear();
    // inputs: the parent's inputs this stage reads, in the parent's order, then the completed partials
    for (size_t k = 0; k < g.inputs.size(); ++k) {
      const int vid = g.inputs[k];
      if (sg.g.values[vid].users.empty()) continue;
      sg.g.values[vid].input_index = (int)sg.g.inputs.size();
      sg.g.inputs.push_back(vid);
      sg.in_parent.push_back((int)k);
      sg.in_carried.push_back(-1);
    }
    for (int i : take)
      for (int vid : g.nodes[i].in) {
        const Value& v = g.v(vid);
        if (v.is_const || v.producer < 0) continue;
        const int p = v.producer;
        if (!(cut[p] && stage[p] < t) || sg.g.values[vid].input_index >= 0) continue;
        auto it = carried_index.find(vid);
        if (it == carried_index.end()) return false;  // cannot happen: earlier stages produced it
        sg.g.values[vid].input_index = (int)sg.g.inputs.size();
        sg.g.values[vid].producer = -1;
        sg.g.inputs.push_back(vid);
        sg.in_parent.push_back(-1);
        sg.in_carried.push_back(it->second);
      }
    for (int vid : targets) {
      sg.g.values[vid].output_index = (int)sg.g.outputs.size();
      sg.g.outputs.push_back(vid);
      sg.out_parent.push_back(g.v(vid).output_index);
      int ci = -1;
      if (cut[g.v(vid).producer] && !g.v(vid).users.empty()) {
        ci = (int)out->carried.size();
        carried_index[vid] = ci;
        out->carried.push_back(vid);
      }
      sg.out_carried.push_back(ci);
    }
    sg.g.kernel_name = g.kernel_name + "_stage" + std::to_string(out->stages.size());
    drop_unused_values(sg.g);
    classify(sg.g);
    out->stages.push_back(std::move(sg));
  }
  return out->stages.size() >= 2;
}

}  // namespace akgb
