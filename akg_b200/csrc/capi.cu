// C ABI + runtime launcher.  Replaces the generated CUDA-driver launcher of the
// reference (akg-mlir/python/akg_mlir/utils/code_template.py:16-211): instead of
// creating a context, JIT-ing PTX and allocating per call, a compiled kernel
// object keeps its plan and (for the host-pointer entry points) its device
// staging buffers, and launches are asynchronous on the caller's stream.
#include <cuda_runtime.h>

#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/akgb.h"
#include "graph.hpp"
#include "kernels.hpp"
#include "plan.hpp"

using namespace akgb;

namespace {
thread_local std::string g_err;
}
void akgb::set_last_error(const char* text) { g_err = text ? text : ""; }

namespace {
akgb_status fail(akgb_status st, const std::string& msg) {
  g_err = msg;
  return st;
}
akgb_status cuda_fail(cudaError_t e, const char* what) {
  return fail(AKGB_CUDA_ERROR, std::string(what) + ": " + cudaGetErrorString(e));
}

constexpr int kMaxDevices = 64;
struct DeviceState {
  std::mutex mu;
  void* gelu_lut = nullptr;   // device copy of the f16 tanh table
  uint32_t* err_word = nullptr;
  int sm_count = 0;
  bool exchange_failed = false;  // sticky: see device_exchange_failed()
};
DeviceState g_dev[kMaxDevices];

int query_sm_count(int device) {
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    return 148;  // planning without a device: a B200 has 148 SMs
  }
  return n;
}
}  // namespace

struct akgb_kernel {
  Graph graph;
  Plan plan;
  int device = 0;
  int sm_count = 148;
  int shard_rank = 0, shard_world = 1;
  bool no_jit = false;  // AKGB_FLAG_NO_JIT
  bool fold_in_launch = false;  // AKGB_FLAG_FOLD_IN_LAUNCH
  bool stage_long_rows = false;  // AKGB_FLAG_STAGE_LONG_ROWS
  bool checked = false;  // AKGB_FLAG_CHECKED
  // dynamic-shape regions: one plan per set of launch-time extents
  struct Bound {
    Graph graph;
    Plan plan;
  };
  std::map<std::vector<int64_t>, std::unique_ptr<Bound>> bound;
  std::mutex bound_mu;
  std::vector<akgb_tensor_desc> descs;
  int n_inputs = 0;
  // host-pointer entry points: staging buffers kept between calls
  std::vector<void*> d_tensors;
  void* d_workspace = nullptr;
  size_t d_workspace_bytes = 0;
  cudaStream_t stream = nullptr;
  bool staged = false;
  // chunked pipeline of akgb_run_host: the same region planned on 1/nchunks of axis 0, so that the
  // host->device copy of chunk c+1, the kernels of chunk c and the device->host copy of chunk c-1 overlap
  std::string json_text;
  int nchunks = 0;  // 0 = not pipelined
  Plan chunk_plan;
  std::vector<char> chunk_split;     // per argument: 1 = axis 0 is cut into chunks
  std::vector<size_t> chunk_bytes;   // per argument: bytes of one chunk
  cudaStream_t s_in = nullptr, s_out = nullptr;
  std::vector<cudaEvent_t> ev_in, ev_done;
  // arrival counters of the reductions that fold their partials in the launch that produced them (k_reduce.cu);
  // allocated zeroed on the first launch of a plan with such a step, left at zero by every launch
  uint32_t* d_tickets = nullptr;
  // a sharded region cut into stages at the reductions over the split axis that feed later ops (stages.cpp): every
  // stage is a kernel of its own; a stage argument is one of this kernel's arguments (`arg` >= 0) or a carried value
  // (a completed partial of an earlier stage) at `ws_off` of the workspace
  struct StageArg {
    int arg = -1;
    int64_t ws_off = -1;
  };
  struct Stage {
    akgb_kernel* k = nullptr;
    std::vector<StageArg> args;  // the stage kernel's inputs then outputs
  };
  std::vector<Stage> stages;
  size_t stage_ws_off = 0;  // the stages' own workspace starts here (after the carried values)
  ~akgb_kernel();
};

namespace {

bool plan_has_reduction(const Plan& p) {
  for (const Step& st : p.steps)
    if (st.kind == StepK::ReduceCol || st.kind == StepK::ReduceAll || st.kind == StepK::ReduceColDual) return true;
  return p.fallback && plan_has_reduction(*p.fallback);
}

// The calling thread's current device must be the kernel's: device state is cached per ordinal and generated kernels are
// loaded into the current context, so a launch issued with another device current would mix the two.
akgb_status check_current_device(const akgb_kernel* k, const char* who) {
  int cur = -1;
  if (cudaGetDevice(&cur) != cudaSuccess) {
    cudaGetLastError();
    return fail(AKGB_CUDA_ERROR, std::string(who) + ": no current CUDA device");
  }
  if (cur != k->device)
    return fail(AKGB_INVALID_ARG, std::string(who) + ": the kernel was compiled for device " + std::to_string(k->device) +
                                      " but device " + std::to_string(cur) + " is current on this thread");
  return AKGB_OK;
}

akgb_status ensure_device_state(akgb_kernel* k, bool need_lut, const Plan* plan = nullptr) {
  int dev = k->device;
  if (dev < 0 || dev >= kMaxDevices) return fail(AKGB_INVALID_ARG, "device ordinal out of range");
  akgb_status cs = check_current_device(k, "akgb");
  if (cs != AKGB_OK) return cs;
  DeviceState& ds = g_dev[dev];
  std::lock_guard<std::mutex> lock(ds.mu);
  if (!k->d_tickets && plan_has_reduction(plan ? *plan : k->plan)) {
    void* d = nullptr;
    cudaError_t e = cudaMalloc(&d, kReduceTicketWords * sizeof(uint32_t));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(arrival counters)");
    e = cudaMemset(d, 0, kReduceTicketWords * sizeof(uint32_t));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemset(arrival counters)");
    k->d_tickets = reinterpret_cast<uint32_t*>(d);
  }
  if (need_lut && !ds.gelu_lut) {
    std::vector<uint16_t> h(gelu_lut_entries());
    gelu_lut_build(h.data());
    void* d = nullptr;
    cudaError_t e = cudaMalloc(&d, h.size() * sizeof(uint16_t));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(tanh table)");
    e = cudaMemcpy(d, h.data(), h.size() * sizeof(uint16_t), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(tanh table)");
    ds.gelu_lut = d;
  }
  if (!ds.err_word) {
    void* d = nullptr;
    cudaError_t e = cudaMalloc(&d, 256);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(error word)");
    e = cudaMemset(d, 0, 256);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemset(error word)");
    ds.err_word = reinterpret_cast<uint32_t*>(d);
  }
  return AKGB_OK;
}

void* resolve(const Ref& r, void* const* tensors, void* ws) {
  if (r.arg >= 0) return tensors[r.arg];
  if (r.ws_off >= 0) return reinterpret_cast<char*>(ws) + r.ws_off;
  return nullptr;
}

// switches a plan whose generated kernel cannot be built on this host to its separate launches, if the caller's
// workspace is large enough for them (akgb_workspace_size reports what the generated kernel needs)
akgb_status enter_fallback(Plan& plan, size_t ws_bytes) {
  if (ws_bytes < plan.fallback->workspace_bytes)
    return fail(AKGB_UNSUPPORTED,
                "the kernel generated for this region could not be compiled on this host and the workspace is too small "
                "for the separate launches (" + std::to_string(plan.fallback->workspace_bytes) +
                " bytes): compile the region with AKGB_FLAG_NO_JIT");
  plan.use_fallback = true;
  return AKGB_OK;
}

// `fx` / `fx_step`: the exchange that step `fx_step` of the plan completes inside its own launch (sharded reductions)
void fill_arg_bytes(Plan& p, const Graph& g) {
  p.arg_bytes.clear();
  for (int vid : g.inputs) p.arg_bytes.push_back((size_t)g.v(vid).numel() * dt_size(g.v(vid).dt));
  for (int vid : g.outputs) p.arg_bytes.push_back((size_t)g.v(vid).numel() * dt_size(g.v(vid).dt));
  if (p.fallback) p.fallback->arg_bytes = p.arg_bytes;
}

akgb_status run_plan_steps(akgb_kernel* k, Plan& plan, void* const* tensors, void* ws, size_t ws_bytes, cudaStream_t s,
                           const FinishExchange* fx, int fx_step);

// Bytes taken off the end of every range of a checked launch: a test of the checker itself (the accesses it then
// reports and skips are inside the real tensors).
int g_checked_shrink = 0;

akgb_status run_plan(akgb_kernel* k, Plan& plan, void* const* tensors, void* ws, size_t ws_bytes, cudaStream_t s,
                     const FinishExchange* fx = nullptr, int fx_step = -1) {
  if (!k->checked) return run_plan_steps(k, plan, tensors, ws, ws_bytes, s, fx, fx_step);
  // checked launch: generated kernels test every global access against these ranges
  CheckedRanges r;
  for (size_t i = 0; i < plan.arg_bytes.size() && r.n < 31; ++i) {
    if (!tensors[i] || !plan.arg_bytes[i]) continue;
    r.lo[r.n] = reinterpret_cast<unsigned long long>(tensors[i]);
    r.hi[r.n] = r.lo[r.n] + plan.arg_bytes[i] - std::min<size_t>(plan.arg_bytes[i], (size_t)g_checked_shrink);
    ++r.n;
  }
  if (ws && ws_bytes) {
    r.lo[r.n] = reinterpret_cast<unsigned long long>(ws);
    r.hi[r.n] = r.lo[r.n] + ws_bytes;
    ++r.n;
  }
  r.err = g_dev[k->device].err_word;
  if (plan.arg_bytes.size() > 31) return fail(AKGB_UNSUPPORTED, "checked launches take at most 31 tensors");
  struct Scope {  // the table is gone from the thread again however the launches end
    explicit Scope(const CheckedRanges* t) { jit_set_checked_ranges(t); }
    ~Scope() { jit_set_checked_ranges(nullptr); }
  } scope(&r);
  return run_plan_steps(k, plan, tensors, ws, ws_bytes, s, fx, fx_step);
}

akgb_status run_plan_steps(akgb_kernel* k, Plan& plan, void* const* tensors, void* ws, size_t ws_bytes, cudaStream_t s,
                           const FinishExchange* fx, int fx_step) {
  if (plan.fallback && plan.use_fallback) return run_plan_steps(k, *plan.fallback, tensors, ws, ws_bytes, s, nullptr, -1);
  DeviceState& ds = g_dev[k->device];
  for (size_t si = 0; si < plan.steps.size(); ++si) {
    Step& st = plan.steps[si];
    const FinishExchange* sfx = ((int)si == fx_step) ? fx : nullptr;
    // arrival counters: the last CTA of a reduction folds its partials (AKGB_FLAG_FOLD_IN_LAUNCH); else a fold launch
    uint32_t* tickets = k->fold_in_launch ? k->d_tickets : nullptr;
    cudaError_t e = cudaSuccess;
    void* a = resolve(st.a, tensors, ws);
    void* b = resolve(st.b, tensors, ws);
    void* c = resolve(st.c, tensors, ws);
    void* o = resolve(st.out, tensors, ws);
    void* o2 = resolve(st.out2, tensors, ws);
    void* o3 = resolve(st.out3, tensors, ws);
    void* scratch = resolve(st.scratch, tensors, ws);
    switch (st.kind) {
      case StepK::GeluChain:
        e = gelu_chain_f16(st.gelu, a, b, c, o, ds.gelu_lut, ds.err_word, s, &st.dims);
        break;
      case StepK::LayerNorm:
        e = layernorm_f32(st.ln, (const float*)a, (const float*)b, (const float*)c, (float*)o, (float*)o2, (float*)o3,
                          ds.err_word, s, &st.dims);
        break;
      case StepK::Softmax:
        e = softmax_rows(st.sm, a, b, o, ds.err_word, s, &st.dims);
        break;
      case StepK::ReduceCol:
        for (int64_t bi = 0; bi < st.red_outer && e == cudaSuccess; ++bi)
          e = reduce_col_f32(st.red_op, (const float*)a + bi * st.red_batch_in, (float*)o + bi * st.red_batch_out,
                             st.red_len, st.red_inner, scratch, k->sm_count, s, &st.dims, tickets, sfx);
        break;
      case StepK::Gather:
        e = gather_rows(a, b, o, st.ix_outer, st.ix_dim, st.ix_n, st.ix_inner, st.ix_esize, st.ix_idx64, s, &st.dims);
        break;
      case StepK::ArgMax:
        e = argmax_axis(a, o, st.ix_outer, st.ix_dim, st.ix_inner, st.ix_esize, st.ix_idx64, s, &st.dims);
        break;
      case StepK::SegmentSum:
        e = segment_sum(a, b, o, st.ix_n, st.ix_inner, st.ix_segments, st.ix_idx64, st.ix_esize, s, &st.dims);
        break;
      case StepK::RowJit: {
        const void* ins[16];
        void* outs[16];
        for (size_t i = 0; i < st.ew_in.size(); ++i) ins[i] = resolve(st.ew_in[i], tensors, ws);
        for (size_t i = 0; i < st.ew_out.size(); ++i) outs[i] = resolve(st.ew_out[i], tensors, ws);
        e = row_jit_launch(*st.row, ins, outs, s, &st.dims);
        if (e == cudaErrorNotSupported && plan.fallback) {  // no run-time compiler here: the separate launches
          // (the generated kernel is always the plan's first step, so nothing has been enqueued yet)
          const akgb_status fs = enter_fallback(plan, ws_bytes);
          if (fs != AKGB_OK) return fs;
          return run_plan_steps(k, *plan.fallback, tensors, ws, ws_bytes, s, nullptr, -1);
        }
        break;
      }
      case StepK::ColJit: {
        const void* ins[16];
        for (size_t i = 0; i < st.ew_in.size(); ++i) ins[i] = resolve(st.ew_in[i], tensors, ws);
        float* parts[4] = {nullptr, nullptr, nullptr, nullptr};
        for (size_t i = 0; i < st.ew_out.size() && i < 4; ++i) parts[i] = (float*)resolve(st.ew_out[i], tensors, ws);
        e = col_jit_launch(*st.row, ins, parts, st.red_len, s, &st.dims);
        if (e == cudaErrorNotSupported && plan.fallback) {
          const akgb_status fs = enter_fallback(plan, ws_bytes);
          if (fs != AKGB_OK) return fs;
          return run_plan_steps(k, *plan.fallback, tensors, ws, ws_bytes, s, nullptr, -1);
        }
        break;
      }
      case StepK::Ew: {
        const void* ins[kEwMaxIn];
        void* outs[kEwMaxOut];
        for (size_t i = 0; i < st.ew_in.size(); ++i) ins[i] = resolve(st.ew_in[i], tensors, ws);
        for (size_t i = 0; i < st.ew_out.size(); ++i) outs[i] = resolve(st.ew_out[i], tensors, ws);
        e = ew_generic(st.ew, ins, outs, !k->no_jit, s, &st.dims);
        if (e == cudaErrorNotSupported)
          return fail(AKGB_UNSUPPORTED, "this region holds 64-bit integer values and needs the run-time compiler, which is "
                                        "switched off (AKGB_FLAG_NO_JIT) or not available on this host");
        break;
      }
      case StepK::ReduceColDual:
        if (reduce_col_dual_supported(st.red_inner, a)) {
          e = reduce_col_dual_f32(st.red_op, st.red_op2, (const float*)a, (float*)o, (float*)o2, st.red_len, st.red_inner,
                                  scratch, k->sm_count, s, &st.dims, tickets, sfx);
        } else if (sfx) {
          e = cudaErrorNotSupported;  // fused_exchange_step() only picks aligned inputs
        } else {  // unaligned input: the two single reductions, one after the other
          e = reduce_col_f32(st.red_op, (const float*)a, (float*)o, st.red_len, st.red_inner, scratch, k->sm_count, s,
                             &st.dims, tickets);
          if (e == cudaSuccess)
            e = reduce_all_f32(st.red_op2, (const float*)a, (float*)o2, st.red_len * st.red_inner, scratch, k->sm_count, s,
                               nullptr, tickets);
        }
        break;
      case StepK::ReduceAll:
        e = reduce_all_f32(st.red_op, (const float*)a, (float*)o, st.red_len, scratch, k->sm_count, s, &st.dims,
                           tickets, sfx);
        break;
      case StepK::ReduceRow:
        e = reduce_row_f32(st.red_op, (const float*)a, (float*)o, st.red_outer, st.red_len, s, &st.dims);
        break;
      case StepK::Transpose:
        e = transpose_nd(st.tp, a, o, s, &st.dims);
        break;
      case StepK::Matmul:
        if (st.mm.in_dt == (int)DT::F32) {
          e = matmul_f32(st.mm, a, b, c, o, st.mm_batch, st.mm_stride_a / 4, st.mm_stride_b / 4, st.mm_stride_o / 4, s,
                         &st.dims);
          break;
        }
        e = matmul_bf16(st.mm, a, b, c, o, st.mm_batch, st.mm_stride_b != 0, ds.err_word, k->sm_count, s, &st.dims);
        break;
    }
    if (e != cudaSuccess) return cuda_fail(e, st.kernel_name.c_str());
  }
  return AKGB_OK;
}

// the plan launches go through: the generated row kernel, or the separate launches once it has been given up
const Plan& active_plan(const akgb_kernel* k) {
  return (k->plan.fallback && k->plan.use_fallback) ? *k->plan.fallback : k->plan;
}

int launches_of(const akgb_kernel* k) {
  int n = 0;
  for (auto& st : k->stages) n += launches_of(st.k);
  for (const Step& st : active_plan(k).steps) {
    switch (st.kind) {
      case StepK::ReduceCol:  // the fold of the row splits happens in the launch that produced them
        n += (int)st.red_outer * reduce_col_launches(st.red_len, st.red_inner, k->sm_count, k->fold_in_launch);
        break;
      case StepK::ReduceAll:
        n += k->fold_in_launch ? 1 : 2;
        break;
      case StepK::ReduceColDual:
        n += (k->fold_in_launch && (st.red_inner + 127) / 128 <= kReduceMaxTicketTiles) ? 1 : 2;
        break;
      case StepK::GeluChain:
        n += (st.gelu.n % 8) ? 2 : 1;
        break;
      case StepK::Matmul:
        n += 1;
        break;
      default:
        n += 1;
    }
  }
  return n;
}

// Tries to plan the region on a fraction of axis 0.  Any failure simply leaves nchunks at 0 (one-shot path).
void plan_chunks(akgb_kernel* k) {
  k->nchunks = 0;
  int64_t moved = 0;
  for (auto& d : k->descs) moved += d.nbytes;
  if (moved < (int64_t)64 << 20) return;  // too small to be worth several copies
  for (auto& d : k->descs)
    if (d.written_in_place) return;
  // measured on the 1.07 GB benchmark chain (537 MB each way): 2 / 4 / 8 / 16 / 32 / 64 chunks -> 15.1 / 13.0 / 12.1 /
  // 11.9 / 12.6 / 14.2 ms per call: every chunk costs some tens of microseconds of copy and event set-up, fewer chunks
  // leave more of the first copy-in and the last copy-out uncovered
  for (int n : {16, 8, 4, 2}) {
    if (moved / n < ((int64_t)8 << 20)) continue;  // keep every copy large enough to run at full PCIe rate
    try {
      Graph g = parse_info(k->json_text.data(), k->json_text.size());
      infer_sharding(g, 0, k->shard_world * n);
      bool ok = true;
      std::vector<char> split;
      std::vector<size_t> bytes;
      auto visit = [&](int vid) {
        const Value& v = g.v(vid);
        if (v.partial) ok = false;
        split.push_back(v.split0 ? 1 : 0);
        bytes.push_back((size_t)v.numel() * dt_size(v.dt));
      };
      for (int vid : g.inputs) visit(vid);
      for (int vid : g.outputs) {
        visit(vid);
        if (!g.v(vid).split0) ok = false;  // every output must be produced chunk by chunk
      }
      if (!ok) return;
      Plan p = build_plan(g, k->sm_count, !k->no_jit);
      fill_arg_bytes(p, g);
      if (p.workspace_bytes > k->plan.workspace_bytes) return;
      if (cudaStreamCreateWithFlags(&k->s_in, cudaStreamNonBlocking) != cudaSuccess) return;
      if (cudaStreamCreateWithFlags(&k->s_out, cudaStreamNonBlocking) != cudaSuccess) return;
      k->ev_in.assign(n, nullptr);
      k->ev_done.assign(n, nullptr);
      for (int i = 0; i < n; ++i) {
        if (cudaEventCreateWithFlags(&k->ev_in[i], cudaEventDisableTiming) != cudaSuccess) return;
        if (cudaEventCreateWithFlags(&k->ev_done[i], cudaEventDisableTiming) != cudaSuccess) return;
      }
      k->chunk_plan = std::move(p);
      k->chunk_split = std::move(split);
      k->chunk_bytes = std::move(bytes);
      k->nchunks = n;
      return;
    } catch (const std::exception&) {
      // not divisible by this chunk count, or the region does not split on axis 0: try fewer chunks
    }
  }
}

akgb_status run_host_chunked(akgb_kernel* k, void* const* host) {
  const int n = k->nchunks;
  const size_t nt = k->descs.size();
  cudaError_t e;
  // operands that are not cut (bias, gamma, mask, the right matmul operand) go first, whole
  for (int i = 0; i < k->n_inputs; ++i) {
    if (k->chunk_split[i] || !k->descs[i].nbytes) continue;
    e = cudaMemcpyAsync(k->d_tensors[i], host[i], (size_t)k->descs[i].nbytes, cudaMemcpyHostToDevice, k->s_in);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(H2D)");
  }
  std::vector<void*> ptrs(nt);
  for (int c = 0; c < n; ++c) {
    for (int i = 0; i < k->n_inputs; ++i) {
      if (!k->chunk_split[i]) continue;
      const size_t off = (size_t)c * k->chunk_bytes[i];
      e = cudaMemcpyAsync((char*)k->d_tensors[i] + off, (const char*)host[i] + off, k->chunk_bytes[i],
                          cudaMemcpyHostToDevice, k->s_in);
      if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(H2D chunk)");
    }
    cudaEventRecord(k->ev_in[c], k->s_in);
    cudaStreamWaitEvent(k->stream, k->ev_in[c], 0);
    for (size_t i = 0; i < nt; ++i)
      ptrs[i] = k->chunk_split[i] ? (void*)((char*)k->d_tensors[i] + (size_t)c * k->chunk_bytes[i]) : k->d_tensors[i];
    akgb_status st = run_plan(k, k->chunk_plan, ptrs.data(), k->d_workspace, k->d_workspace_bytes, k->stream);
    if (st != AKGB_OK) return st;
    cudaEventRecord(k->ev_done[c], k->stream);
    cudaStreamWaitEvent(k->s_out, k->ev_done[c], 0);
    for (size_t i = k->n_inputs; i < nt; ++i) {
      const size_t off = (size_t)c * k->chunk_bytes[i];
      e = cudaMemcpyAsync((char*)host[i] + off, (const char*)k->d_tensors[i] + off, k->chunk_bytes[i],
                          cudaMemcpyDeviceToHost, k->s_out);
      if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(D2H chunk)");
    }
  }
  e = cudaStreamSynchronize(k->s_out);
  if (e == cudaSuccess) e = cudaStreamSynchronize(k->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(k->s_in);
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
  return AKGB_OK;
}

akgb_status stage(akgb_kernel* k) {
  if (k->staged) return AKGB_OK;
  cudaError_t e = cudaSetDevice(k->device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  k->d_tensors.assign(k->descs.size(), nullptr);
  for (size_t i = 0; i < k->descs.size(); ++i) {
    size_t bytes = (size_t)std::max<int64_t>(k->descs[i].nbytes, 16);
    e = cudaMalloc(&k->d_tensors[i], bytes);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(staging tensor)");
  }
  // the host-pointer path owns its workspace: large enough for the separate launches too
  k->d_workspace_bytes = std::max(k->plan.workspace_bytes, k->plan.fallback ? k->plan.fallback->workspace_bytes : (size_t)0);
  if (k->d_workspace_bytes) {
    e = cudaMalloc(&k->d_workspace, k->d_workspace_bytes);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(workspace)");
  }
  e = cudaStreamCreateWithFlags(&k->stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamCreate");
  plan_chunks(k);
  k->staged = true;
  return AKGB_OK;
}

}  // namespace

bool akgb::device_exchange_failed(int device) {
  return device >= 0 && device < kMaxDevices && g_dev[device].exchange_failed;
}
void akgb::device_exchange_set_failed(int device, bool failed) {
  if (device >= 0 && device < kMaxDevices) g_dev[device].exchange_failed = failed;
}

// The step of the plan that produces ALL partial outputs of a sharded kernel, if there is exactly one and it is a
// reduction that can complete the exchange in its own launch; -1 otherwise.  Fills the slot positions.
namespace {
int fused_exchange_step(const akgb_kernel* k, const Plan& plan, FinishExchange* fx) {
  std::vector<int> partial;
  for (size_t i = 0; i < k->descs.size(); ++i)
    if (k->descs[i].shard_kind >= AKGB_PARTIAL_SUM) {
      if (k->descs[i].dtype != AKGB_FLOAT32) return -1;
      partial.push_back((int)i);
    }
  if (partial.empty() || partial.size() > 2) return -1;
  auto op_of = [](int kind) {
    return kind == AKGB_PARTIAL_SUM ? RedOp::Sum : kind == AKGB_PARTIAL_MAX ? RedOp::Max
         : kind == AKGB_PARTIAL_MIN ? RedOp::Min : RedOp::Prod;
  };
  for (size_t si = 0; si < plan.steps.size(); ++si) {
    const Step& st = plan.steps[si];
    if (st.out.arg != partial[0]) continue;
    // nothing after this step may touch the result (it is final once the finisher has written it)
    if (si + 1 != plan.steps.size()) return -1;
    if (st.kind == StepK::ReduceCol && partial.size() == 1) {
      if (st.red_outer != 1 || st.red_inner > kExchangeTaggedElems || st.red_op != op_of(k->descs[partial[0]].shard_kind))
        return -1;
      fx->slot_off = 0;
      fx->finishers = (int)((st.red_inner + 127) / 128);
      return (int)si;
    }
    if (st.kind == StepK::ReduceAll && partial.size() == 1) {
      if (st.red_op != op_of(k->descs[partial[0]].shard_kind)) return -1;
      fx->slot_off = 0;
      fx->finishers = 1;
      return (int)si;
    }
    if (st.kind == StepK::ReduceColDual && partial.size() == 2 && st.out2.arg == partial[1]) {
      if (st.red_inner + 1 > kExchangeTaggedElems || st.red_inner % 4 != 0 ||
          st.red_op != op_of(k->descs[partial[0]].shard_kind) || st.red_op2 != op_of(k->descs[partial[1]].shard_kind))
        return -1;
      fx->slot_off = 0;
      fx->slot_off2 = (int)st.red_inner;
      fx->finishers = (int)((st.red_inner + 127) / 128) + 1;
      return (int)si;
    }
    return -1;
  }
  return -1;
}
}  // namespace

bool akgb::kernel_exchange_fusable(const akgb_kernel* k) {
  if (!k || k->graph.dynamic) return false;
  FinishExchange fx;
  return fused_exchange_step(k, active_plan(k), &fx) >= 0;
}

akgb_status akgb::launch_with_exchange(akgb_kernel* k, const FinishExchange& base, void* const* tensors, void* workspace,
                                       size_t workspace_bytes, void* stream, bool* fused) {
  *fused = false;
  if (!k || !tensors) return fail(AKGB_INVALID_ARG, "null argument");
  if (k->graph.dynamic) return AKGB_OK;
  FinishExchange fx = base;
  Plan& plan = (k->plan.fallback && k->plan.use_fallback) ? *k->plan.fallback : k->plan;
  const int step = fused_exchange_step(k, plan, &fx);
  if (step < 0) return AKGB_OK;  // nothing launched: the caller runs the kernel and the exchange one after the other
  if (workspace_bytes < k->plan.workspace_bytes || (k->plan.workspace_bytes && !workspace))
    return fail(AKGB_INVALID_ARG, "workspace smaller than akgb_workspace_size()");
  if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 255))
    return fail(AKGB_MISALIGNED, "workspace must be 256-byte aligned");
  const Step& st = plan.steps[step];
  if (st.kind == StepK::ReduceColDual && (reinterpret_cast<uintptr_t>(resolve(st.a, tensors, workspace)) & 15))
    return AKGB_OK;  // unaligned input: the two-kernel form of this step cannot carry the exchange
  akgb_status s = ensure_device_state(k, plan.needs_gelu_lut);
  if (s != AKGB_OK) return s;
  fx.err = g_dev[k->device].err_word;
  *fused = true;
  return run_plan(k, plan, tensors, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream), &fx, step);
}

uint32_t* akgb::kernel_error_word(akgb_kernel* k) {
  if (!k || ensure_device_state(k, false) != AKGB_OK) return nullptr;
  return g_dev[k->device].err_word;
}

namespace {
void verify_generated_bounds(const akgb_kernel* k, const Plan& plan);
// plan + argument descriptions of k->graph (already parsed) for k's shard
void plan_and_describe(akgb_kernel* k) {
  if (k->graph.dynamic) {
    if (k->shard_world > 1) throw Unsupported("dynamic-shape regions cannot be sharded at compile time");
    for (auto& n : k->graph.nodes)
      if (n.kind == OpK::Unknown) throw Unsupported("operator '" + n.name + "' is not supported");
    k->plan.klass = "dynamic";
  } else {
    infer_sharding(k->graph, k->shard_rank, k->shard_world);
    k->plan = build_plan(k->graph, k->sm_count, !k->no_jit);
    fill_arg_bytes(k->plan, k->graph);
    if (k->stage_long_rows)
      for (Step& st : k->plan.steps)
        if (st.kind == StepK::RowJit && st.row) st.row->stage_long_rows = true;
  }
  const Graph& g = k->graph;
  k->n_inputs = (int)g.inputs.size();
  k->descs.clear();
  auto add = [&](int vid, bool is_out) {
    const Value& v = g.v(vid);
    akgb_tensor_desc d;
    std::memset(&d, 0, sizeof(d));
    std::snprintf(d.name, sizeof(d.name), "%s", v.name.c_str());
    d.dtype = (int32_t)v.dt;
    d.rank = (int32_t)std::min<size_t>(v.shape.size(), AKGB_MAX_RANK);
    if (v.shape.size() > AKGB_MAX_RANK) throw Unsupported("tensor rank above 8");
    for (int i = 0; i < d.rank; ++i) d.shape[i] = v.shape[i];
    d.nbytes = v.numel() * (int64_t)dt_size(v.dt);
    for (auto e : v.shape)
      if (e < 0) d.nbytes = -1;  // bound at launch
    d.is_output = is_out;
    d.shard_kind = v.partial ? v.partial : (v.split0 ? AKGB_SPLIT_AXIS0 : AKGB_REPLICATED);
    k->descs.push_back(d);
  };
  for (int vid : g.inputs) add(vid, false);
  for (int vid : g.outputs) add(vid, true);
  for (auto& n : g.nodes)
    if (n.kind == OpK::Assign && g.v(n.in[0]).input_index >= 0) k->descs[g.v(n.in[0]).input_index].written_in_place = 1;
  if (!k->graph.dynamic) verify_generated_bounds(k, k->plan);
}

// Host-side bounds check of the generated kernels' index maps: for every operand of a generated elementwise or row
// kernel that is one of the caller's tensors, the smallest and largest element the kernel's index arithmetic can
// produce must lie inside that tensor.  Run on every plan before it is accepted; a violation is a planner error and
// refuses the region instead of launching it.
void verify_generated_bounds(const akgb_kernel* k, const Plan& plan) {
  auto nbytes_of = [&](const Ref& r) -> int64_t { return r.arg >= 0 && r.arg < (int)k->descs.size() ? k->descs[r.arg].nbytes : -1; };
  auto esize = [](int dt) { return (int64_t)dt_size((DT)dt); };
  auto fail_with = [&](const std::string& what) { throw Unsupported("internal bounds check of a generated kernel failed: " + what); };
  for (const Step& st : plan.steps) {
    if (st.kind == StepK::Ew) {
      const EwProgram& P = st.ew;
      auto check = [&](const EwOperand& o, const Ref& r, const char* role) {
        const int64_t have = nbytes_of(r);
        if (have < 0 || P.n <= 0) return;
        int64_t lo = 0, hi = 0;
        if (o.kind == EWI_FULL) hi = P.n - 1;
        else if (o.kind == EWI_MOD) hi = std::min<int64_t>(P.n, o.mod) - 1;
        else if (o.kind == EWI_STRIDED) {
          lo = hi = o.offset;
          for (int d = 0; d < P.rank; ++d) {
            int64_t ext = P.shape[d];
            if (o.wrap[d] != 0) ext = std::min<int64_t>(ext, o.wrap[d]);
            const int64_t span = (ext - 1) * o.stride[d];
            if (span > 0) hi += span;
            else lo += span;
          }
        }
        if (lo < 0 || (hi + 1) * esize(o.dt) > have)
          fail_with(std::string(role) + " operand of '" + st.kernel_name + "' reaches element " + std::to_string(hi) +
                    " (from " + std::to_string(lo) + ") of a tensor of " + std::to_string(have) + " bytes");
      };
      for (int i = 0; i < P.n_in && i < (int)st.ew_in.size(); ++i) check(P.in[i], st.ew_in[i], "input");
      for (int i = 0; i < P.n_out && i < (int)st.ew_out.size(); ++i) check(P.out[i], st.ew_out[i], "output");
    } else if ((st.kind == StepK::RowJit || st.kind == StepK::ColJit) && st.row) {
      const RowProgram& P = *st.row;
      auto elems = [&](const RowOperand& o) -> int64_t {
        switch (o.kind) {
          case RK_FULL: return P.rows * P.cols;
          case RK_ROW: return o.row_mod != 0 ? o.row_mod : P.rows;
          case RK_COL: return P.cols;
          case RK_ROWMOD: return o.mod_rows * P.cols;
          default: return 1;
        }
      };
      for (size_t i = 0; i < P.in.size() && i < st.ew_in.size(); ++i) {
        const int64_t have = nbytes_of(st.ew_in[i]);
        if (have >= 0 && elems(P.in[i]) * esize(P.in[i].dt) > have)
          fail_with("input " + std::to_string(i) + " of '" + st.kernel_name + "' is read beyond its " + std::to_string(have) + " bytes");
      }
      if (st.kind == StepK::RowJit && !P.col_sums)
        for (size_t i = 0; i < P.out.size() && i < st.ew_out.size(); ++i) {
          const int64_t have = nbytes_of(st.ew_out[i]);
          if (have >= 0 && elems(P.out[i]) * esize(P.out[i].dt) > have)
            fail_with("output " + std::to_string(i) + " of '" + st.kernel_name + "' is written beyond its " + std::to_string(have) + " bytes");
        }
    }
  }
  if (plan.fallback) verify_generated_bounds(k, *plan.fallback);
}

// The region as stages (stages.cpp): every stage planned as a sharded kernel of its own.  On success k describes the
// whole region (its arguments as the caller passes them) and holds the stage kernels.
bool build_stages(akgb_kernel* k, const char* text, size_t len) {
  Graph whole = parse_info(text, len);  // global shapes (k->graph may be half rewritten by the failed attempt)
  StagePlan sp;
  if (!split_at_sharded_reductions(whole, &sp)) return false;
  std::vector<akgb_kernel::Stage> stages;
  auto drop = [&] {
    for (auto& st : stages) delete st.k;
  };
  try {
    // carried values: in the caller's output when they are results of the region, else in the workspace
    std::vector<akgb_kernel::StageArg> where(sp.carried.size());
    size_t ws = 0;
    const int n_in = (int)whole.inputs.size();
    for (size_t c = 0; c < sp.carried.size(); ++c) {
      const Value& v = whole.v(sp.carried[c]);
      if (v.output_index >= 0) {
        where[c].arg = n_in + v.output_index;
      } else {
        where[c].ws_off = (int64_t)ws;
        ws += ((size_t)v.numel() * dt_size(v.dt) + 255) / 256 * 256;
      }
    }
    k->stage_ws_off = ws;
    size_t stage_ws = 0;
    std::vector<akgb_tensor_desc> descs(whole.inputs.size() + whole.outputs.size());
    std::vector<char> have(descs.size(), 0);
    Plan summary;
    summary.klass = "sharded_stages";
    for (StageGraph& sg : sp.stages) {
      akgb_kernel::Stage st;
      st.k = new akgb_kernel();
      stages.push_back(st);
      akgb_kernel* sk = stages.back().k;
      sk->device = k->device;
      sk->sm_count = k->sm_count;
      sk->shard_rank = k->shard_rank;
      sk->shard_world = k->shard_world;
      sk->no_jit = k->no_jit;
      sk->fold_in_launch = k->fold_in_launch;
      sk->stage_long_rows = k->stage_long_rows;
      sk->checked = k->checked;
      sk->graph = std::move(sg.g);
      plan_and_describe(sk);
      stage_ws = std::max(stage_ws, sk->plan.workspace_bytes);
      summary.flops += sk->plan.flops;
      summary.needs_gelu_lut = summary.needs_gelu_lut || sk->plan.needs_gelu_lut;
      auto& args = stages.back().args;
      for (size_t i = 0; i < sg.in_parent.size(); ++i) {
        akgb_kernel::StageArg a;
        if (sg.in_parent[i] >= 0) {
          a.arg = sg.in_parent[i];
          if (!have[a.arg]) {
            descs[a.arg] = sk->descs[i];
            have[a.arg] = 1;
          }
        } else {
          a = where[sg.in_carried[i]];
        }
        args.push_back(a);
      }
      for (size_t i = 0; i < sg.out_parent.size(); ++i) {
        akgb_kernel::StageArg a;
        const akgb_tensor_desc& sd = sk->descs[sg.in_parent.size() + i];
        if (sg.out_parent[i] >= 0) {
          a.arg = n_in + sg.out_parent[i];
          descs[a.arg] = sd;
          // the exchange runs inside akgb_launch_sharded of this kernel: the caller gets the completed value
          if (descs[a.arg].shard_kind >= AKGB_PARTIAL_SUM) descs[a.arg].shard_kind = AKGB_REPLICATED;
          have[a.arg] = 1;
        } else if (sg.out_carried[i] >= 0) {
          a = where[sg.out_carried[i]];
        } else {
          throw Unsupported("a stage result is neither a result of the region nor read by a later stage");
        }
        if (sd.shard_kind >= AKGB_PARTIAL_SUM && sd.dtype != AKGB_FLOAT32 && sd.dtype != AKGB_FLOAT16 &&
            sd.dtype != AKGB_BFLOAT16 && sd.dtype != AKGB_INT32)
          throw Unsupported("partial result of a type the exchange step does not carry");
        args.push_back(a);
      }
    }
    // arguments no stage reads (dead inputs) are described whole
    for (size_t i = 0; i < descs.size(); ++i) {
      if (have[i]) continue;
      const bool is_out = (int)i >= n_in;
      const Value& v = whole.v(is_out ? whole.outputs[i - n_in] : whole.inputs[i]);
      if (is_out) throw Unsupported("a result of the region is produced by no stage");
      akgb_tensor_desc d;
      std::memset(&d, 0, sizeof(d));
      std::snprintf(d.name, sizeof(d.name), "%s", v.name.c_str());
      d.dtype = (int32_t)v.dt;
      d.rank = (int32_t)v.shape.size();
      for (int r = 0; r < d.rank; ++r) d.shape[r] = v.shape[r];
      d.nbytes = v.numel() * (int64_t)dt_size(v.dt);
      descs[i] = d;
    }
    summary.workspace_bytes = ws + stage_ws;
    for (auto& d : descs) summary.bytes += d.nbytes;  // algorithmic: every argument of the region once
    k->graph = std::move(whole);
    k->plan = std::move(summary);
    k->descs = std::move(descs);
    k->n_inputs = n_in;
    k->stages = std::move(stages);
    return true;
  } catch (const Unsupported&) {
    drop();
    return false;
  } catch (...) {
    drop();
    throw;
  }
}
}  // namespace

akgb_kernel::~akgb_kernel() {
  for (auto& st : stages) akgb_release(st.k);
}

bool akgb::kernel_is_staged(const akgb_kernel* k) { return k && !k->stages.empty(); }
const akgb_kernel* akgb::kernel_stage(const akgb_kernel* k, int i) {
  return (k && i >= 0 && i < (int)k->stages.size()) ? k->stages[i].k : nullptr;
}

akgb_status akgb::launch_staged(akgb_kernel* k, akgb_comm* c, void* const* tensors, void* workspace,
                                size_t workspace_bytes, void* stream) {
  if (workspace_bytes < k->plan.workspace_bytes || (k->plan.workspace_bytes && !workspace))
    return fail(AKGB_INVALID_ARG, "workspace smaller than akgb_workspace_size()");
  if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 255))
    return fail(AKGB_MISALIGNED, "workspace must be 256-byte aligned");
  std::vector<void*> args;
  char* ws = static_cast<char*>(workspace);
  for (auto& st : k->stages) {
    args.clear();
    for (auto& a : st.args) args.push_back(a.arg >= 0 ? tensors[a.arg] : (void*)(ws + a.ws_off));
    // the stage, then the exchange that completes its partial results, on the same stream
    const akgb_status s = akgb_launch_sharded(st.k, c, args.data(), ws ? ws + k->stage_ws_off : nullptr,
                                              workspace_bytes - k->stage_ws_off, stream);
    if (s != AKGB_OK) return s;
  }
  return AKGB_OK;
}

extern "C" {

const char* akgb_last_error(void) { return g_err.c_str(); }
const char* akgb_version(void) { return "akgb 0.1 (sm_100a)"; }

akgb_status akgb_compile(const char* info_json, size_t len, const akgb_options* opt, akgb_kernel** out) {
  if (!info_json || !out) return fail(AKGB_INVALID_ARG, "null argument");
  *out = nullptr;
  int device = -1, rank = 0, world = 1, flags = 0;
  if (opt) {
    if (opt->struct_size < (int32_t)sizeof(akgb_options)) return fail(AKGB_INVALID_ARG, "akgb_options.struct_size");
    device = opt->device;
    rank = opt->shard_rank;
    world = opt->shard_world <= 0 ? 1 : opt->shard_world;
    flags = opt->flags;
  }
  if (device < 0) {
    if (cudaGetDevice(&device) != cudaSuccess) {
      cudaGetLastError();
      device = 0;
    }
  }
  akgb_kernel* k = nullptr;
  try {
    k = new akgb_kernel();
    k->device = device;
    k->sm_count = query_sm_count(device);
    k->shard_rank = rank;
    k->shard_world = world;
    k->no_jit = (flags & AKGB_FLAG_NO_JIT) != 0;
    k->fold_in_launch = (flags & AKGB_FLAG_FOLD_IN_LAUNCH) != 0;
    k->stage_long_rows = (flags & AKGB_FLAG_STAGE_LONG_ROWS) != 0;
    k->checked = (flags & AKGB_FLAG_CHECKED) != 0;
    k->json_text.assign(info_json, len);
    k->graph = parse_info(info_json, len);
    try {
      plan_and_describe(k);
    } catch (const Unsupported&) {
      // a reduction over the split axis that feeds later ops: stages with the exchange step between them
      if (world <= 1 || k->graph.dynamic || !build_stages(k, info_json, len)) throw;
    }
  } catch (const JsonError& e) {
    delete k;
    return fail(AKGB_INVALID_JSON, e.what());
  } catch (const Unsupported& e) {
    delete k;
    return fail(AKGB_UNSUPPORTED, e.what());
  } catch (const std::exception& e) {
    delete k;
    return fail(AKGB_INVALID_ARG, e.what());
  }
  *out = k;
  return AKGB_OK;
}

void akgb_release(akgb_kernel* k) {
  if (!k) return;
  if (k->d_tickets) {
    int cur = -1;
    cudaGetDevice(&cur);
    cudaSetDevice(k->device);
    cudaFree(k->d_tickets);
    if (cur >= 0) cudaSetDevice(cur);
  }
  if (k->staged) {
    cudaSetDevice(k->device);
    for (void* p : k->d_tensors)
      if (p) cudaFree(p);
    if (k->d_workspace) cudaFree(k->d_workspace);
    if (k->stream) cudaStreamDestroy(k->stream);
    if (k->s_in) cudaStreamDestroy(k->s_in);
    if (k->s_out) cudaStreamDestroy(k->s_out);
    for (auto ev : k->ev_in)
      if (ev) cudaEventDestroy(ev);
    for (auto ev : k->ev_done)
      if (ev) cudaEventDestroy(ev);
  }
  delete k;
}

int32_t akgb_num_tensors(const akgb_kernel* k) { return k ? (int32_t)k->descs.size() : 0; }
int32_t akgb_num_inputs(const akgb_kernel* k) { return k ? k->n_inputs : 0; }

akgb_status akgb_tensor_info(const akgb_kernel* k, int32_t index, akgb_tensor_desc* out) {
  if (!k || !out) return fail(AKGB_INVALID_ARG, "null argument");
  if (index < 0 || index >= (int32_t)k->descs.size()) return fail(AKGB_INVALID_ARG, "tensor index out of range");
  *out = k->descs[index];
  return AKGB_OK;
}

size_t akgb_workspace_size(const akgb_kernel* k) { return k ? k->plan.workspace_bytes : 0; }
int32_t akgb_launch_count(const akgb_kernel* k) { return k ? launches_of(k) : 0; }
const char* akgb_kernel_class(const akgb_kernel* k) { return k ? k->plan.klass.c_str() : ""; }
int64_t akgb_kernel_bytes(const akgb_kernel* k) { return k ? k->plan.bytes : 0; }
int64_t akgb_kernel_flops(const akgb_kernel* k) { return k ? k->plan.flops : 0; }

namespace {
// plan of a dynamic-shape kernel for the given extents (flat: all extents of argument 0, then argument 1, ...)
akgb_status bound_plan(akgb_kernel* k, const int64_t* shapes, size_t count, akgb_kernel::Bound** out) {
  if (!k->graph.dynamic) return fail(AKGB_INVALID_ARG, "this kernel has static shapes: use akgb_launch");
  size_t need = 0;
  for (auto& d : k->descs) need += (size_t)d.rank;
  if (!shapes || count != need) return fail(AKGB_INVALID_ARG, "shapes must list every extent of every argument");
  std::vector<int64_t> key(shapes, shapes + count);
  std::lock_guard<std::mutex> lock(k->bound_mu);
  auto it = k->bound.find(key);
  if (it == k->bound.end()) {
    try {
      std::vector<std::vector<int64_t>> per;
      size_t pos = 0;
      for (auto& d : k->descs) {
        per.emplace_back(shapes + pos, shapes + pos + d.rank);
        pos += (size_t)d.rank;
      }
      std::unique_ptr<akgb_kernel::Bound> b(new akgb_kernel::Bound());
      b->graph = bind_shapes(k->graph, per);
      b->plan = build_plan(b->graph, k->sm_count, !k->no_jit);
      fill_arg_bytes(b->plan, b->graph);
      it = k->bound.emplace(std::move(key), std::move(b)).first;
    } catch (const JsonError& e) {
      return fail(AKGB_INVALID_ARG, e.what());
    } catch (const Unsupported& e) {
      return fail(AKGB_UNSUPPORTED, e.what());
    } catch (const std::exception& e) {
      return fail(AKGB_INVALID_ARG, e.what());
    }
  }
  *out = it->second.get();
  return AKGB_OK;
}
}  // namespace

extern "C" akgb_status akgb_bind_shapes(akgb_kernel* k, const int64_t* shapes, size_t count, size_t* workspace_bytes) {
  if (!k) return fail(AKGB_INVALID_ARG, "null argument");
  akgb_kernel::Bound* b = nullptr;
  akgb_status st = bound_plan(k, shapes, count, &b);
  if (st != AKGB_OK) return st;
  if (workspace_bytes) *workspace_bytes = b->plan.workspace_bytes;
  return AKGB_OK;
}

extern "C" akgb_status akgb_launch_dynamic(akgb_kernel* k, void* const* tensors, const int64_t* shapes, size_t count,
                                           void* workspace, size_t workspace_bytes, void* stream) {
  if (!k || !tensors) return fail(AKGB_INVALID_ARG, "null argument");
  akgb_kernel::Bound* b = nullptr;
  akgb_status st = bound_plan(k, shapes, count, &b);
  if (st != AKGB_OK) return st;
  if (workspace_bytes < b->plan.workspace_bytes || (b->plan.workspace_bytes && !workspace))
    return fail(AKGB_INVALID_ARG, "workspace smaller than akgb_bind_shapes() reported");
  if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 255))
    return fail(AKGB_MISALIGNED, "workspace must be 256-byte aligned");
  st = ensure_device_state(k, b->plan.needs_gelu_lut, &b->plan);
  if (st != AKGB_OK) return st;
  return run_plan(k, b->plan, tensors, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

akgb_status akgb_launch(akgb_kernel* k, void* const* tensors, void* workspace, size_t workspace_bytes, void* stream) {
  if (!k || !tensors) return fail(AKGB_INVALID_ARG, "null argument");
  if (!k->stages.empty())
    return fail(AKGB_INVALID_ARG, "this sharded region has an exchange step between its stages: use akgb_launch_sharded");
  if (k->graph.dynamic) return fail(AKGB_INVALID_ARG, "this kernel has dynamic shapes: use akgb_launch_dynamic");
  if (workspace_bytes < k->plan.workspace_bytes || (k->plan.workspace_bytes && !workspace))
    return fail(AKGB_INVALID_ARG, "workspace smaller than akgb_workspace_size()");
  for (size_t i = 0; i < k->descs.size(); ++i) {
    if (!tensors[i] && k->descs[i].nbytes) return fail(AKGB_INVALID_ARG, "null tensor pointer");
  }
  if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 255))
    return fail(AKGB_MISALIGNED, "workspace must be 256-byte aligned");
  akgb_status st = ensure_device_state(k, k->plan.needs_gelu_lut);
  if (st != AKGB_OK) return st;
  return run_plan(k, k->plan, tensors, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

akgb_status akgb_run_host(akgb_kernel* k, void* const* host) {
  if (!k || !host) return fail(AKGB_INVALID_ARG, "null argument");
  if (!k->stages.empty())
    return fail(AKGB_INVALID_ARG, "this sharded region has an exchange step between its stages: use akgb_launch_sharded");
  if (k->graph.dynamic) return fail(AKGB_INVALID_ARG, "this kernel has dynamic shapes: use akgb_launch_dynamic");
  // like the reference's launcher this entry point picks its device itself (and leaves it current)
  const cudaError_t se = cudaSetDevice(k->device);
  if (se != cudaSuccess) return cuda_fail(se, "cudaSetDevice");
  akgb_status st = stage(k);
  if (st != AKGB_OK) return st;
  st = ensure_device_state(k, k->plan.needs_gelu_lut);
  if (st != AKGB_OK) return st;
  if (k->nchunks > 1) return run_host_chunked(k, host);
  cudaError_t e;
  for (int i = 0; i < k->n_inputs; ++i) {
    if (!k->descs[i].nbytes) continue;
    e = cudaMemcpyAsync(k->d_tensors[i], host[i], (size_t)k->descs[i].nbytes, cudaMemcpyHostToDevice, k->stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(H2D)");
  }
  st = run_plan(k, k->plan, k->d_tensors.data(), k->d_workspace, k->d_workspace_bytes, k->stream);
  if (st != AKGB_OK) return st;
  for (size_t i = 0; i < k->descs.size(); ++i) {
    if (!k->descs[i].nbytes) continue;
    if ((int)i < k->n_inputs && !k->descs[i].written_in_place) continue;
    e = cudaMemcpyAsync(host[i], k->d_tensors[i], (size_t)k->descs[i].nbytes, cudaMemcpyDeviceToHost, k->stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(D2H)");
  }
  e = cudaStreamSynchronize(k->stream);
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
  return AKGB_OK;
}

akgb_status akgb_profile_host(akgb_kernel* k, void* const* host, int32_t number, int32_t repeat, double* avg_us) {
  if (!k || !host || !avg_us || number <= 0 || repeat <= 0) return fail(AKGB_INVALID_ARG, "bad argument");
  akgb_status st = akgb_run_host(k, host);  // stages, copies inputs, one warm-up launch
  if (st != AKGB_OK) return st;
  cudaEvent_t t0, t1;
  cudaEventCreate(&t0);
  cudaEventCreate(&t1);
  cudaEventRecord(t0, k->stream);
  for (int i = 0; i < number * repeat; ++i) {
    st = run_plan(k, k->plan, k->d_tensors.data(), k->d_workspace, k->d_workspace_bytes, k->stream);
    if (st != AKGB_OK) break;
  }
  cudaEventRecord(t1, k->stream);
  cudaError_t e = cudaEventSynchronize(t1);
  float ms = 0.f;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, t0, t1);
  cudaEventDestroy(t0);
  cudaEventDestroy(t1);
  if (st != AKGB_OK) return st;
  if (e != cudaSuccess) return cuda_fail(e, "profiling");
  *avg_us = (double)ms * 1000.0 / ((double)number * repeat);
  return AKGB_OK;
}

akgb_status akgb_check_device_error(akgb_kernel* k, uint32_t* word) {
  if (!k || !word) return fail(AKGB_INVALID_ARG, "null argument");
  *word = 0;
  DeviceState& ds = g_dev[k->device];
  if (!ds.err_word) return AKGB_OK;
  cudaError_t e = cudaMemcpy(word, ds.err_word, sizeof(uint32_t), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(error word)");
  if (*word) {
    cudaMemset(ds.err_word, 0, sizeof(uint32_t));
    if (*word & 256u) ds.exchange_failed = true;  // the ranks' exchange counters may disagree now
    if (*word == 512u) return fail(AKGB_OUT_OF_RANGE, "a checked launch reported an access outside its tensors (skipped)");
    return fail(AKGB_DEVICE_TIMEOUT, "a bounded device-side wait gave up");
  }
  return AKGB_OK;
}

akgb_status akgb_prepare(akgb_kernel* k) {
  if (!k) return fail(AKGB_INVALID_ARG, "null argument");
  for (auto& st : k->stages) {  // a region that runs as stages: every stage's tables, counters and generated kernels
    const akgb_status ss = akgb_prepare(st.k);
    if (ss != AKGB_OK) return ss;
  }
  if (!k->stages.empty()) return AKGB_OK;
  const cudaError_t e = cudaSetDevice(k->device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  akgb_status st = ensure_device_state(k, k->plan.needs_gelu_lut);
  if (st != AKGB_OK) return st;
  if (k->no_jit) return AKGB_OK;
  for (const Step& step : active_plan(k).steps) {
    if (step.kind == StepK::Ew) ew_jit_prepare(step.ew);
    else if (step.kind == StepK::RowJit || step.kind == StepK::ColJit) row_jit_prepare(*step.row);
  }
  return AKGB_OK;
}

akgb_status akgb_set_cache_dir(const char* dir) {
  jit_set_cache_dir(dir);
  return AKGB_OK;
}

akgb_status akgb_jit_cache_stats(uint64_t* compiled, uint64_t* loaded_from_disk) {
  jit_cache_stats(compiled, loaded_from_disk);
  return AKGB_OK;
}

akgb_status akgb_dump_jit_source(const akgb_kernel* k, int32_t vectorised, char* buf, size_t cap, size_t* needed) {
  if (!k) return fail(AKGB_INVALID_ARG, "null argument");
  std::string src;
  for (const Step& st : active_plan(k).steps) {
    if (st.kind == StepK::RowJit || st.kind == StepK::ColJit) src = row_jit_source(*st.row, vectorised != 0);
    else if (st.kind == StepK::Ew) src = ew_jit_source(st.ew, vectorised != 0);
    if (!src.empty()) break;
  }
  if (needed) *needed = src.size() + 1;
  if (!buf) return AKGB_OK;
  if (cap < src.size() + 1) return fail(AKGB_INVALID_ARG, "buffer too small");
  std::memcpy(buf, src.c_str(), src.size() + 1);
  return AKGB_OK;
}

akgb_status akgb_export_kernel(const akgb_kernel* k, const char* dir) {
  if (!k || !dir || !*dir) return fail(AKGB_INVALID_ARG, "null argument");
  if (k->graph.dynamic || !k->stages.empty())
    return fail(AKGB_UNSUPPORTED, "only static, single-kernel regions have a stand-alone binary");
  const Plan& ap = active_plan(k);
  if (ap.steps.size() != 1 || (ap.steps[0].kind != StepK::Ew && ap.steps[0].kind != StepK::RowJit))
    return fail(AKGB_UNSUPPORTED,
                "this region runs on kernel templates built into the library or in several launches: there is no "
                "stand-alone binary for it (launch it through akgb_launch)");
  const Step& st = ap.steps[0];
  // the kernel takes the caller's tensors directly only when every operand is one of them, in argument order
  const std::vector<Ref>& in = st.ew_in;
  const std::vector<Ref>& out = st.ew_out;
  if ((int)in.size() != k->n_inputs || in.size() + out.size() != k->descs.size())
    return fail(AKGB_UNSUPPORTED, "the generated kernel does not take exactly the region's arguments");
  for (size_t i = 0; i < in.size(); ++i)
    if (in[i].arg != (int)i) return fail(AKGB_UNSUPPORTED, "the generated kernel reorders the region's arguments");
  for (size_t i = 0; i < out.size(); ++i)
    if (out[i].arg != k->n_inputs + (int)i)
      return fail(AKGB_UNSUPPORTED, "the generated kernel reorders the region's arguments");
  const std::string entry = k->graph.kernel_name + "_kernel";
  for (char ch : entry)
    if (!(std::isalnum((unsigned char)ch) || ch == '_'))
      return fail(AKGB_UNSUPPORTED, "the kernel name is not usable as a symbol");
  std::vector<char> cubin;
  LaunchDims d;
  bool align16 = false;
  const bool ok = st.kind == StepK::Ew ? ew_jit_export(st.ew, entry, &cubin, &d, &align16)
                                       : row_jit_export(*st.row, entry, &cubin, &d, &align16);
  if (!ok) return fail(AKGB_UNSUPPORTED, "the kernel of this region could not be generated or compiled on this host: " + g_err);
  const std::string base = std::string(dir) + "/" + k->graph.kernel_name;
  {
    FILE* f = std::fopen((base + ".cubin").c_str(), "wb");
    if (!f) return fail(AKGB_INVALID_ARG, "cannot write " + base + ".cubin");
    const bool w = std::fwrite(cubin.data(), 1, cubin.size(), f) == cubin.size();
    std::fclose(f);
    if (!w) return fail(AKGB_INVALID_ARG, "short write to " + base + ".cubin");
  }
  std::ostringstream o;
  o << "{\"kernelName\": \"" << entry << "\", \"blockIdx.x\": " << d.grid[0] << ", \"blockIdx.y\": " << d.grid[1]
    << ", \"blockIdx.z\": " << d.grid[2] << ", \"threadIdx.x\": " << d.block[0] << ", \"threadIdx.y\": " << d.block[1]
    << ", \"threadIdx.z\": " << d.block[2] << ", \"is_dynamic\": false, \"sha256\": \""
    << sha256_hex(cubin.data(), cubin.size()) << "\", \"binary\": \"" << k->graph.kernel_name
    << ".cubin\", \"arch\": \"sm_100a\", \"shared_mem_bytes\": " << d.smem
    << ", \"args\": \"device pointers of the inputs, then of the outputs\", \"pointer_alignment\": "
    << (align16 ? 16 : 1) << ", \"class\": \"" << k->plan.klass << "\"}";
  const std::string text = o.str();
  FILE* f = std::fopen((base + ".json").c_str(), "wb");
  if (!f) return fail(AKGB_INVALID_ARG, "cannot write " + base + ".json");
  std::fwrite(text.data(), 1, text.size(), f);
  std::fclose(f);
  return AKGB_OK;
}

akgb_status akgb_kernel_meta(const akgb_kernel* k, char* buf, size_t cap, size_t* needed) {
  if (!k) return fail(AKGB_INVALID_ARG, "null argument");
  // the keys the reference writes to <kernel>.json (GPUMapping.cpp:645-703,
  // mlir_driver.py:776-815); grid/block are those of the dominant (first) step
  static const Step kNoStep{};
  const Plan& ap = active_plan(k);
  const Step& st = ap.steps.empty() ? kNoStep : ap.steps.front();
  LaunchDims d = st.dims;
  std::ostringstream o;
  o << "{\"kernelName\": \"" << k->graph.kernel_name << "_kernel\", "
    << "\"blockIdx.x\": " << d.grid[0] << ", \"blockIdx.y\": " << d.grid[1] << ", \"blockIdx.z\": " << d.grid[2]
    << ", \"threadIdx.x\": " << d.block[0] << ", \"threadIdx.y\": " << d.block[1]
    << ", \"threadIdx.z\": " << d.block[2] << ", \"is_dynamic\": " << (k->graph.dynamic ? "true" : "false") << ", \"sha256\": \"" << k->graph.sha256_hex
    << "\", \"class\": \"" << k->plan.klass << "\", \"template\": \"" << st.kernel_name
    << "\", \"bytes\": " << k->plan.bytes << ", \"flops\": " << k->plan.flops << ", \"smem\": " << d.smem
    << ", \"workspace\": " << k->plan.workspace_bytes << ", \"launches\": " << launches_of(k) << ", \"steps\": [";
  for (size_t i = 0; i < ap.steps.size(); ++i) o << (i ? ", " : "") << "\"" << ap.steps[i].kernel_name << "\"";  // in launch order
  bool first = ap.steps.empty();
  for (auto& stg : k->stages)  // a staged region: the steps of every stage, "|" where an exchange separates two stages
    for (size_t i = 0; i < active_plan(stg.k).steps.size(); ++i) {
      o << (first ? "" : ", ") << "\"" << (i == 0 && &stg != &k->stages.front() ? "| " : "") << active_plan(stg.k).steps[i].kernel_name << "\"";
      first = false;
    }
  o << "]}";
  std::string s = o.str();
  if (needed) *needed = s.size() + 1;
  if (!buf || cap < s.size() + 1) return buf ? fail(AKGB_INVALID_ARG, "buffer too small") : AKGB_OK;
  std::memcpy(buf, s.c_str(), s.size() + 1);
  return AKGB_OK;
}

}  // extern "C"

extern "C" void akgb_checked_shrink_for_test(int bytes) { g_checked_shrink = bytes < 0 ? 0 : bytes; }
