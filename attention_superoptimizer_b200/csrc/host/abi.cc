// Graph-level C ABI (mugraph.h) over the C++ host library.  Nothing here computes: each entry
// validates its arguments, converts between the POD structs and the C++ objects, and forwards.
#include "mirage/kernel/device_memory_manager.h"
#include "mirage/kernel/graph.h"
#include "kernel_select.h"
#include "mirage/utils/json_utils.h"
#include "mugraph.h"
#include "status.h"
#include <cstring>
#include <cuda_runtime.h>
#include <new>

using namespace mirage;
using kernel::DeviceMemoryManager;
using kernel::DTensor;
using kernel::KNOperator;

// Side streams of the verification step: candidate graphs are independent of each other and a candidate's kernels
// fill a fraction of the GPU, so they are dealt over a few lanes that fork from and join the caller's stream.
constexpr int kVerifyLanes = 8;
struct mg_runtime {
  DeviceMemoryManager *dmm;
  cudaStream_t lanes[kVerifyLanes];
  cudaEvent_t lane_done[kVerifyLanes];
  cudaEvent_t fork;
  bool lanes_ready;
};
struct mg_graph {
  mg_runtime *rt;
  kernel::Graph graph;
  // Ticket counters of the batched entry points (one per (set, head) of every fused split-KV + merge pair): device
  // memory of the graph's own, zeroed when allocated; every launch leaves them zero.  Not in the caller's workspace,
  // so that no clearing copy sits between two launches of a stream and one launch can start under the other's tail.
  int *batch_tickets = nullptr;
  size_t batch_ticket_ints = 0;
  std::vector<int *> outgrown_tickets; // kept until the graph goes: a captured launch may still point at them
  ~mg_graph() {
    if (batch_tickets) cudaFree(batch_tickets);
    for (int *p : outgrown_tickets) cudaFree(p);
  }
};

namespace {
mg_runtime g_runtime{};

int fail(int code, char const *msg) {
  mg::set_error(msg);
  return code;
}

int op_index(mg_graph *g, KNOperator const *op) {
  for (size_t i = 0; i < g->graph.operators.size(); i++)
    if (g->graph.operators[i] == op) return (int)i;
  return -1;
}

void to_pod(mg_graph *g, DTensor const &t, mg_tensor *out) {
  std::memset(out, 0, sizeof(*out));
  out->data_type = (int)t.data_type;
  out->layout = (int)t.layout;
  out->num_dims = t.num_dims;
  for (int i = 0; i < t.num_dims; i++) out->dim[i] = t.dim[i];
  out->owner_op = op_index(g, t.owner_op);
  out->owner_ts_idx = t.owner_ts_idx;
  out->data_ptr = t.data_ptr;
  out->fp_ptr = t.fp_ptr;
}

// The authoritative descriptor lives in the graph; the POD only names it.
DTensor const *from_pod(mg_graph *g, mg_tensor const *t) {
  if (!t || t->owner_op < 0 || t->owner_op >= (int)g->graph.operators.size()) return nullptr;
  KNOperator *op = g->graph.operators[t->owner_op];
  if (t->owner_ts_idx < 0 || t->owner_ts_idx >= (int)op->output_tensors.size()) return nullptr;
  return &op->output_tensors[t->owner_ts_idx];
}

KNOperator *get_op(mg_graph *g, int idx) {
  if (!g || idx < 0 || idx >= (int)g->graph.operators.size()) return nullptr;
  return g->graph.operators[idx];
}

int push(mg_graph *g, KNOperator *op, mg_tensor *out, char const *what) {
  if (!op) return fail(MG_ERR_INVALID_GRAPH, what);
  g->graph.operators.push_back(op);
  if (out) to_pod(g, op->output_tensors[0], out);
  return MG_OK;
}

int refuse_dry(mg_runtime *rt) {
  if (rt && rt->dmm && rt->dmm->dry) return fail(MG_ERR_NO_DEVICE, "planning-only runtime (device < 0): no device memory");
  return MG_OK;
}

// Launch every operator of a graph in order; a split-KV attention operator directly followed by the merge
// operator that consumes it goes out as one launch.
int launch_all(mg_graph *g, bool fp, bool skip_inputs, void *stream) {
  auto &ops = g->graph.operators;
  for (size_t i = 0; i < ops.size(); i++) {
    KNOperator *op = ops[i];
    if (skip_inputs && op->op_type == type::KN_INPUT_OP) continue;
    int st;
    if (op->op_type == type::KN_CUSTOMIZED_OP && i + 1 < ops.size() &&
        static_cast<kernel::KNCustomizedOp *>(op)->can_fuse_with(ops[i + 1], fp)) {
      st = static_cast<kernel::KNCustomizedOp *>(op)->launch_fused(static_cast<kernel::KNCustomizedOp *>(ops[i + 1]), fp, stream);
      i++;
    } else {
      st = fp ? op->launch_fingerprint(stream) : op->launch_float(stream);
    }
    if (st != MG_OK) return st;
  }
  return MG_OK;
}

int synchronize_and_check() {
  if (g_runtime.dmm && g_runtime.dmm->dry) return fail(MG_ERR_NO_DEVICE, "planning-only runtime (device < 0)");
  MG_CUDA_TRY(cudaDeviceSynchronize());
  int32_t code = 0;
  int st = mgd_read_and_clear_device_error(&code);
  if (st != MG_OK) return fail(st, mgd_last_error());
  if (code != 0) return fail(MG_ERR_DEVICE_TIMEOUT, "a kernel gave up a bounded wait (device status word set)");
  return MG_OK;
}
} // namespace

extern "C" {

int mg_runtime_create(int device, size_t arena_bytes, mg_runtime **rt) {
  if (!rt) return fail(MG_ERR_INVALID_ARGUMENT, "rt is null");
  *rt = nullptr;
  char const *err = nullptr;
  int st = DeviceMemoryManager::create(device, arena_bytes, &err);
  if (st != MG_OK) return st;
  g_runtime.dmm = DeviceMemoryManager::singleton;
  *rt = &g_runtime;
  return MG_OK;
}

static bool ensure_lanes(mg_runtime *rt) {
  if (rt->lanes_ready) return true;
  for (int i = 0; i < kVerifyLanes; i++) {
    if (cudaStreamCreateWithFlags(&rt->lanes[i], cudaStreamNonBlocking) != cudaSuccess) return false;
    if (cudaEventCreateWithFlags(&rt->lane_done[i], cudaEventDisableTiming) != cudaSuccess) return false;
  }
  if (cudaEventCreateWithFlags(&rt->fork, cudaEventDisableTiming) != cudaSuccess) return false;
  rt->lanes_ready = true;
  return true;
}

int mg_runtime_destroy(mg_runtime *rt) {
  if (!rt || !rt->dmm) return fail(MG_ERR_INVALID_ARGUMENT, "no runtime");
  if (rt->lanes_ready) {
    for (int i = 0; i < kVerifyLanes; i++) {
      cudaStreamDestroy(rt->lanes[i]);
      cudaEventDestroy(rt->lane_done[i]);
    }
    cudaEventDestroy(rt->fork);
    rt->lanes_ready = false;
  }
  DeviceMemoryManager::destroy();
  mg::forget_streams();
  rt->dmm = nullptr;
  return MG_OK;
}

int mg_runtime_tables(mg_runtime *rt, const uint16_t **e, const uint16_t **p, const uint16_t **q) {
  if (!rt || !rt->dmm) return fail(MG_ERR_INVALID_ARGUMENT, "no runtime");
  if (e) *e = rt->dmm->exp_lookup_table;
  if (p) *p = rt->dmm->div_p_lookup_table;
  if (q) *q = rt->dmm->div_q_lookup_table;
  return MG_OK;
}

int mg_runtime_arena_usage(mg_runtime *rt, size_t *used, size_t *total) {
  if (!rt || !rt->dmm) return fail(MG_ERR_INVALID_ARGUMENT, "no runtime");
  if (used) *used = (size_t)rt->dmm->offset;
  if (total) *total = rt->dmm->total_size;
  return MG_OK;
}

int mg_runtime_set_max_smem(mg_runtime *rt, size_t bytes) {
  if (!rt || !rt->dmm) return fail(MG_ERR_INVALID_ARGUMENT, "no runtime");
  if (bytes == 0 || bytes > type::MAX_SMEM_SIZE) return fail(MG_ERR_INVALID_ARGUMENT, "shared-memory budget out of range");
  rt->dmm->max_smem = bytes;
  return MG_OK;
}

int mg_runtime_set_specialisation(mg_runtime *rt, int enabled) {
  if (!rt || !rt->dmm) return fail(MG_ERR_INVALID_ARGUMENT, "no runtime");
  rt->dmm->specialise = enabled < 0 ? 0 : (enabled > 2 ? 2 : enabled);
  return MG_OK;
}

int mg_runtime_set_launch_policy(mg_runtime *rt, int policy) {
  if (!rt || !rt->dmm) return fail(MG_ERR_INVALID_ARGUMENT, "no runtime");
  if (policy != MG_POLICY_LATENCY && policy != MG_POLICY_THROUGHPUT) return fail(MG_ERR_INVALID_ARGUMENT, "unknown launch policy");
  rt->dmm->launch_policy = policy;
  return MG_OK;
}

static_assert(MG_OPT_ATTN_STAGES == MGD_OPT_ATTN_STAGES && MG_OPT_ATTN_TILE_GROUPS == MGD_OPT_ATTN_TILE_GROUPS &&
                  MG_OPT_ATTN_ENGINE == MGD_OPT_ATTN_ENGINE && MG_OPT_ROWS_ENGINE == MGD_OPT_ROWS_ENGINE &&
                  MG_OPT_INTERP_THREADS == MGD_OPT_INTERP_THREADS && MG_OPT_WAIT_LIMIT == MGD_OPT_WAIT_LIMIT &&
                  MG_OPT_ATTN_PERSISTENT == MGD_OPT_ATTN_PERSISTENT && MG_OPT_KN_MATMUL_ENGINE == MGD_OPT_KN_MATMUL_ENGINE &&
                  MG_OPT_ATTN_DEPENDENT_LAUNCH == MGD_OPT_ATTN_DEPENDENT_LAUNCH,
              "the option keys of the two headers are the same numbers");

int mg_runtime_set_option(mg_runtime *rt, int32_t key, int32_t value) {
  if (!rt || !rt->dmm) return fail(MG_ERR_INVALID_ARGUMENT, "no runtime");
  int st = mgd_set_option(key, value);
  return st == MG_OK ? MG_OK : fail(st, mgd_last_error());
}

int mg_runtime_get_option(mg_runtime *rt, int32_t key, int32_t *value) {
  if (!rt || !rt->dmm) return fail(MG_ERR_INVALID_ARGUMENT, "no runtime");
  int st = mgd_get_option(key, value);
  return st == MG_OK ? MG_OK : fail(st, mgd_last_error());
}

int mg_stream_inputs_written(void *stream) {
  mg::stream_wrote_anything(stream);
  return MG_OK;
}

int mg_selftest_bounded_wait(mg_runtime *rt, int32_t poll_limit, void *stream) {
  if (int dry_st = refuse_dry(rt)) return dry_st;
  if (!rt || !rt->dmm) return fail(MG_ERR_INVALID_ARGUMENT, "no runtime");
  int st = mgd_selftest_bounded_wait(poll_limit, stream);
  return st == MG_OK ? MG_OK : fail(st, mgd_last_error());
}

int mg_graph_create(mg_runtime *rt, mg_graph **g) {
  if (!rt || !rt->dmm || !g) return fail(MG_ERR_INVALID_ARGUMENT, "no runtime");
  *g = new (std::nothrow) mg_graph{rt, {}};
  return *g ? MG_OK : fail(MG_ERR_OUT_OF_MEMORY, "host allocation failed");
}

int mg_graph_destroy(mg_graph *g) {
  if (!g) return fail(MG_ERR_INVALID_ARGUMENT, "graph is null");
  delete g;
  return MG_OK;
}

int mg_graph_new_input(mg_graph *g, const int32_t *dims, int32_t nd, int32_t dt, int32_t layout, mg_tensor *out) {
  if (!g || !dims || !out || nd <= 0 || nd > MG_MAX_TENSOR_DIMS) return fail(MG_ERR_INVALID_ARGUMENT, "bad input description");
  std::vector<int> d(dims, dims + nd);
  KNOperator *op = g->graph.create_input_op(d, (type::DataType)dt, (layout::DmemLayout)layout);
  if (!op) {
    kernel::DTensor probe;
    probe.num_dims = nd;
    bool positive = true;
    for (int i = 0; i < nd; i++) { probe.dim[i] = dims[i]; positive = positive && dims[i] > 0; }
    bool dtype_ok = dt == MG_DT_FLOAT16 || dt == MG_DT_BFLOAT16 || dt == MG_DT_FLOAT32;
    if (positive && dtype_ok) return fail(MG_ERR_OUT_OF_MEMORY, "device arena exhausted");
    return fail(MG_ERR_INVALID_ARGUMENT, "dims must be positive and the element type a float type");
  }
  return push(g, op, out, "");
}

int mg_graph_customized(mg_graph *g, const mg_tensor *inputs, int32_t n, const mg_plan *p, mg_tensor *outputs,
                        int32_t max_outputs, int32_t *num_outputs) {
  if (!g || !p || (n > 0 && !inputs) || !num_outputs) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  if (p->num_inputs != n) return fail(MG_ERR_INVALID_GRAPH, "plan lists a different number of inputs than were given");
  if (p->num_ops < 0 || (p->num_ops > 0 && (!p->op_types || !p->op_num_srcs || !p->op_srcs)))
    return fail(MG_ERR_INVALID_ARGUMENT, "plan operator arrays missing");
  if (n > 0 && (!p->input_map || !p->forloop_dim || !p->input_smem_layouts))
    return fail(MG_ERR_INVALID_ARGUMENT, "plan input arrays missing");
  std::vector<DTensor> ins;
  for (int i = 0; i < n; i++) {
    DTensor const *t = from_pod(g, &inputs[i]);
    if (!t) return fail(MG_ERR_INVALID_ARGUMENT, "input tensor does not belong to this graph");
    ins.push_back(*t);
  }
  threadblock::ExecutionPlan plan;
  int s = 0;
  for (int j = 0; j < p->num_ops; j++) {
    std::vector<std::pair<int, int>> srcs;
    if (p->op_num_srcs[j] < 0 || p->op_num_srcs[j] > 4) return fail(MG_ERR_INVALID_GRAPH, "operand count out of range");
    for (int t = 0; t < p->op_num_srcs[j]; t++, s++) srcs.push_back({p->op_srcs[2 * s], p->op_srcs[2 * s + 1]});
    plan.ops.push_back({(type::TBOperatorType)p->op_types[j], srcs});
  }
  for (int i = 0; i < n; i++) {
    plan.input_map.push_back({p->input_map[3 * i], p->input_map[3 * i + 1], p->input_map[3 * i + 2]});
    plan.forloop_dim.push_back(p->forloop_dim[i]);
    plan.input_smem_layouts.push_back((layout::SmemLayout)p->input_smem_layouts[i]);
  }
  plan.output_map = {p->output_map[0], p->output_map[1], p->output_map[2]};
  plan.forloop_range = p->forloop_range;
  plan.reduction_dimx = p->reduction_dimx;
  for (int a = 0; a < 3; a++)
    if (p->grid_dim[a] <= 0 || p->block_dim[a] <= 0) return fail(MG_ERR_INVALID_GRAPH, "grid_dim and block_dim must be positive");
  plan.grid_dim = dim3(p->grid_dim[0], p->grid_dim[1], p->grid_dim[2]);
  plan.block_dim = dim3(p->block_dim[0], p->block_dim[1], p->block_dim[2]);
  std::string err;
  int st = MG_ERR_INVALID_GRAPH;
  kernel::KNCustomizedOp *op = kernel::KNCustomizedOp::create(ins, plan, &err, &st);
  if (!op) return fail(st, err.c_str());
  if ((int)op->output_tensors.size() > max_outputs) {
    delete op;
    return fail(MG_ERR_INVALID_ARGUMENT, "more outputs than the caller made room for");
  }
  g->graph.operators.push_back(op);
  *num_outputs = (int)op->output_tensors.size();
  for (int i = 0; i < *num_outputs; i++) to_pod(g, op->output_tensors[i], &outputs[i]);
  return MG_OK;
}

#define MG_TWO(NAME, CALL)                                                                               \
  int NAME(mg_graph *g, const mg_tensor *a, const mg_tensor *b, mg_tensor *out) {                         \
    if (!g || !out) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");                                \
    DTensor const *A = from_pod(g, a), *B = from_pod(g, b);                                               \
    if (!A || !B) return fail(MG_ERR_INVALID_ARGUMENT, "tensor does not belong to this graph");           \
    return push(g, g->graph.CALL, out, #NAME ": shapes do not match or the arena is exhausted");          \
  }
MG_TWO(mg_graph_matmul, create_matmul_op(*A, *B))
MG_TWO(mg_graph_add, create_elementbinary_op(*A, *B, type::KN_ADD_OP))
MG_TWO(mg_graph_mul, create_elementbinary_op(*A, *B, type::KN_MUL_OP))
MG_TWO(mg_graph_div, create_elementbinary_op(*A, *B, type::KN_DIV_OP))
#undef MG_TWO

int mg_graph_exp(mg_graph *g, const mg_tensor *a, mg_tensor *out) {
  if (!g || !out) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  DTensor const *A = from_pod(g, a);
  if (!A) return fail(MG_ERR_INVALID_ARGUMENT, "tensor does not belong to this graph");
  return push(g, g->graph.create_elementunary_op(*A, type::KN_EXP_OP), out, "mg_graph_exp: arena exhausted");
}

int mg_graph_reduction(mg_graph *g, const mg_tensor *a, int32_t dim, int32_t size, mg_tensor *out) {
  if (!g || !out) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  DTensor const *A = from_pod(g, a);
  if (!A) return fail(MG_ERR_INVALID_ARGUMENT, "tensor does not belong to this graph");
  return push(g, g->graph.create_reduction_op(*A, dim, size), out, "mg_graph_reduction: bad dim/size or arena exhausted");
}

int mg_graph_num_operators(mg_graph *g, int32_t *n) {
  if (!g || !n) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  *n = (int)g->graph.operators.size();
  return MG_OK;
}

int mg_graph_to_json(mg_graph *g, char *buf, size_t capacity, size_t *length) {
  if (!g || !length) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  std::string text = kernel::to_json_string(g->graph);
  *length = text.size();
  if (!buf || capacity < text.size() + 1) return fail(MG_ERR_INVALID_ARGUMENT, "buffer too small for the JSON document");
  std::memcpy(buf, text.c_str(), text.size() + 1);
  return MG_OK;
}

int mg_graph_from_json(mg_runtime *rt, const char *text, mg_graph **out) {
  if (!rt || !rt->dmm || !text || !out) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  *out = nullptr;
  mg_graph *g = new (std::nothrow) mg_graph{rt, {}};
  if (!g) return fail(MG_ERR_OUT_OF_MEMORY, "host allocation failed");
  std::string err;
  if (!kernel::from_json_string(text, g->graph, &err)) {
    delete g; // releases what was built, in reverse order
    return fail(MG_ERR_INVALID_GRAPH, err.c_str());
  }
  *out = g;
  return MG_OK;
}

int mg_graph_operator_info(mg_graph *g, int32_t idx, int32_t *op_type, mg_tensor *outputs, int32_t max_outputs,
                           int32_t *num_outputs) {
  KNOperator *op = get_op(g, idx);
  if (!op) return fail(MG_ERR_INVALID_ARGUMENT, "operator index out of range");
  if (op_type) *op_type = (int32_t)op->op_type;
  if (num_outputs) *num_outputs = (int32_t)op->output_tensors.size();
  for (int i = 0; outputs && i < max_outputs && i < (int)op->output_tensors.size(); i++) to_pod(g, op->output_tensors[i], &outputs[i]);
  return MG_OK;
}

int mg_graph_customized_info(mg_graph *g, int32_t idx, int32_t *nops, int32_t *smem, int32_t *kfp, int32_t *kfl) {
  KNOperator *op = get_op(g, idx);
  if (!op || op->op_type != type::KN_CUSTOMIZED_OP) return fail(MG_ERR_INVALID_ARGUMENT, "not a customized operator");
  auto *c = static_cast<kernel::KNCustomizedOp *>(op);
  if (nops) *nops = (int)c->bgraph.operators.size();
  if (smem) *smem = (int)c->bgraph.smem_offset;
  if (kfp) *kfp = c->selected_kernel(true);
  if (kfl) *kfl = c->selected_kernel(false);
  return MG_OK;
}

int mg_graph_customized_program(mg_graph *g, int32_t idx, void *program_out, size_t program_bytes) {
  KNOperator *op = get_op(g, idx);
  if (!op || op->op_type != type::KN_CUSTOMIZED_OP || !program_out) return fail(MG_ERR_INVALID_ARGUMENT, "not a customized operator");
  if (program_bytes != sizeof(mgd_program)) return fail(MG_ERR_INVALID_ARGUMENT, "program_bytes must be sizeof(mgd_program)");
  auto *c = static_cast<kernel::KNCustomizedOp *>(op);
  char const *why = nullptr;
  if (!c->bgraph.lower(*static_cast<mgd_program *>(program_out), &why)) return fail(MG_ERR_UNSUPPORTED, why ? why : "cannot lower");
  return MG_OK;
}

int mg_graph_customized_set_causal_window(mg_graph *g, int32_t idx, int32_t window) {
  KNOperator *op = get_op(g, idx);
  if (!op || op->op_type != type::KN_CUSTOMIZED_OP || window < 0) return fail(MG_ERR_INVALID_ARGUMENT, "not a customized operator");
  static_cast<kernel::KNCustomizedOp *>(op)->set_causal_window(window);
  return MG_OK;
}

int mg_op_fingerprint(mg_graph *g, int32_t idx) {
  KNOperator *op = get_op(g, idx);
  if (!op) return fail(MG_ERR_INVALID_ARGUMENT, "operator index out of range");
  int st = op->launch_fingerprint(nullptr);
  if (st != MG_OK) return st;
  return synchronize_and_check();
}

int mg_graph_fingerprint(mg_graph *g) {
  if (!g) return fail(MG_ERR_INVALID_ARGUMENT, "graph is null");
  int st = launch_all(g, true, false, nullptr);
  return st != MG_OK ? st : synchronize_and_check();
}

int mg_graph_fingerprint_compute(mg_graph *g) {
  if (!g) return fail(MG_ERR_INVALID_ARGUMENT, "graph is null");
  int st = launch_all(g, true, true, nullptr);
  return st != MG_OK ? st : synchronize_and_check();
}

int mg_graph_fingerprint_enqueue(mg_graph *g, void *stream) {
  if (!g) return fail(MG_ERR_INVALID_ARGUMENT, "graph is null");
  return launch_all(g, true, true, stream);
}

int mg_op_run(mg_graph *g, int32_t idx, void *stream) {
  KNOperator *op = get_op(g, idx);
  if (!op) return fail(MG_ERR_INVALID_ARGUMENT, "operator index out of range");
  return op->launch_float(stream);
}

int mg_graph_run(mg_graph *g, void *stream) {
  if (!g) return fail(MG_ERR_INVALID_ARGUMENT, "graph is null");
  return launch_all(g, false, false, stream);
}

int mg_op_profile(mg_graph *g, int32_t idx, int32_t warmup, int32_t iters, float *ms) {
  KNOperator *op = get_op(g, idx);
  if (!op || !ms) return fail(MG_ERR_INVALID_ARGUMENT, "operator index out of range");
  if (warmup < 0 || iters < 0) return fail(MG_ERR_INVALID_ARGUMENT, "negative repetition count");
  if (warmup == 0 && iters == 0) {
    ProfileResult r;
    if (!op->profile(r)) return MG_ERR_CUDA;
    *ms = r.run_time;
    return synchronize_and_check();
  }
  cudaEvent_t ev[2];
  MG_CUDA_TRY(cudaDeviceSynchronize());
  MG_CUDA_TRY(cudaEventCreate(&ev[0]));
  MG_CUDA_TRY(cudaEventCreate(&ev[1]));
  int st = MG_OK;
  for (int i = 0; i < warmup && st == MG_OK; i++) st = op->launch_float(nullptr);
  cudaEventRecord(ev[0], nullptr);
  for (int i = 0; i < iters && st == MG_OK; i++) st = op->launch_float(nullptr);
  cudaEventRecord(ev[1], nullptr);
  cudaEventSynchronize(ev[1]);
  float t = 0.f;
  cudaEventElapsedTime(&t, ev[0], ev[1]);
  cudaEventDestroy(ev[0]);
  cudaEventDestroy(ev[1]);
  if (st != MG_OK) return st;
  *ms = t / (float)(iters > 0 ? iters : 1);
  return synchronize_and_check();
}

// Shared body of the two batched entry points.  Workspace layout: every customized-op output except the final one
// gets num_sets * elements 16-bit values (256-byte aligned).
static int run_batched(mg_graph *g, bool fp, int32_t num_sets, const void *const *in_ptrs, void *out_ptr, void *workspace,
                       size_t *workspace_bytes, void *stream) {
  if (!g || num_sets <= 0 || !workspace_bytes) return fail(MG_ERR_INVALID_ARGUMENT, "bad batched request");
  auto &ops = g->graph.operators;
  std::vector<KNOperator *> inputs, work;
  for (KNOperator *op : ops) {
    if (op->op_type == type::KN_INPUT_OP) inputs.push_back(op);
    else if (op->op_type == type::KN_CUSTOMIZED_OP) work.push_back(op);
    else return fail(MG_ERR_UNSUPPORTED, "batched evaluation handles graphs of inputs and customized operators");
  }
  if (work.empty()) return fail(MG_ERR_INVALID_GRAPH, "graph has no customized operator");
  struct Slot { KNOperator *op; int ts; size_t offset; long long elems; };
  std::vector<Slot> slots;
  size_t need = 0;
  for (size_t w = 0; w < work.size(); w++)
    for (size_t t = 0; t < work[w]->output_tensors.size(); t++) {
      bool final_out = (w + 1 == work.size()) && t == 0;
      long long e = (long long)work[w]->output_tensors[t].num_elements();
      if (final_out) { slots.push_back({work[w], (int)t, (size_t)-1, e}); continue; }
      slots.push_back({work[w], (int)t, need, e});
      need += ((size_t)e * 2 * (size_t)num_sets + 255) / 256 * 256;
    }
  // A split-KV operator and the merge that consumes it are issued as one launch.  The partials between them live in
  // the workspace and nobody else reads them, which lets the kernel sum consecutive splits of a head on the chip.
  std::vector<size_t> ticket_offset(work.size(), (size_t)-1); // in counters, into the graph's ticket array
  size_t ticket_ints = 0;
  for (size_t w = 0; w + 1 < work.size(); w++) {
    auto *c = static_cast<kernel::KNCustomizedOp *>(work[w]);
    if (c->selected_kernel(fp) == mg::KERNEL_ATTN_SPLIT && c->can_fuse_with(work[w + 1], fp)) {
      ticket_offset[w] = ticket_ints;
      ticket_ints += ((size_t)c->plan.grid_dim.x * (size_t)num_sets + 63) / 64 * 64;
      w++;
    }
  }
  if (!workspace) {
    *workspace_bytes = need;
    return MG_OK;
  }
  if (int dry_st = refuse_dry(g->rt)) return dry_st;
  if (*workspace_bytes < need) return fail(MG_ERR_INVALID_ARGUMENT, "workspace too small");
  if (!in_ptrs || !out_ptr) return fail(MG_ERR_INVALID_ARGUMENT, "null tensor pointers");
  if (ticket_ints > g->batch_ticket_ints) {
    // grown on the first call and when a call brings more sets (allocation synchronises the device: not for a stream
    // that is being captured - make the first call of a size outside the capture); the outgrown array stays alive
    size_t const want = ticket_ints > 2 * g->batch_ticket_ints ? ticket_ints : 2 * g->batch_ticket_ints;
    int *fresh = nullptr;
    MG_CUDA_TRY(cudaMalloc(&fresh, want * sizeof(int)));
    MG_CUDA_TRY(cudaMemset(fresh, 0, want * sizeof(int)));
    if (g->batch_tickets) g->outgrown_tickets.push_back(g->batch_tickets);
    g->batch_tickets = fresh;
    g->batch_ticket_ints = want;
  }
  auto locate = [&](DTensor const &t, void const **ptr, long long *stride) -> bool {
    for (size_t i = 0; i < inputs.size(); i++)
      if (inputs[i] == t.owner_op) {
        *ptr = in_ptrs[i];
        *stride = (long long)t.num_elements();
        return true;
      }
    for (Slot const &s : slots)
      if (s.op == t.owner_op && s.ts == t.owner_ts_idx) {
        *ptr = s.offset == (size_t)-1 ? (void const *)out_ptr : (void const *)((char *)workspace + s.offset);
        *stride = s.elems;
        return true;
      }
    return false;
  };
  for (size_t w = 0; w < work.size(); w++) {
    auto *c = static_cast<kernel::KNCustomizedOp *>(work[w]);
    void const *in[MGD_MAX_IO];
    void *out[MGD_MAX_IO];
    long long is[MGD_MAX_IO], os[MGD_MAX_IO];
    if (c->input_tensors.size() > MGD_MAX_IO || c->output_tensors.size() > MGD_MAX_IO) return fail(MG_ERR_UNSUPPORTED, "too many tensors");
    for (size_t i = 0; i < c->input_tensors.size(); i++)
      if (!locate(c->input_tensors[i], &in[i], &is[i])) return fail(MG_ERR_INVALID_GRAPH, "operand produced outside this graph");
    for (size_t i = 0; i < c->output_tensors.size(); i++) {
      void const *p;
      if (!locate(c->output_tensors[i], &p, &os[i])) return fail(MG_ERR_INVALID_GRAPH, "internal: output slot missing");
      out[i] = const_cast<void *>(p);
    }
    int st;
    if (ticket_offset[w] != (size_t)-1) {
      auto *m = static_cast<kernel::KNCustomizedOp *>(work[w + 1]);
      void const *mp;
      long long ms;
      if (!locate(m->output_tensors[0], &mp, &ms)) return fail(MG_ERR_INVALID_GRAPH, "internal: output slot missing");
      st = c->launch_fused_sets(m, fp, num_sets, in, is, out, os, const_cast<void *>(mp), ms,
                                g->batch_tickets + ticket_offset[w], stream,
                                /*partials_are_scratch=*/true); // the intermediates live in the caller's workspace
      w++;
    } else {
      st = fp ? c->launch_fingerprint_sets(num_sets, in, is, out, os, stream) : c->launch_float_sets(num_sets, in, is, out, os, stream);
    }
    if (st != MG_OK) return st;
  }
  return MG_OK;
}

int mg_graph_fingerprint_batched(mg_graph *g, int32_t num_sets, const uint16_t *const *in_fp, uint16_t *out_fp,
                                 void *workspace, size_t *workspace_bytes, void *stream) {
  return run_batched(g, true, num_sets, reinterpret_cast<const void *const *>(in_fp), out_fp, workspace, workspace_bytes, stream);
}

int mg_graph_run_batched(mg_graph *g, int32_t num_sets, const void *const *in_data, void *out_data, void *workspace,
                         size_t *workspace_bytes, void *stream) {
  return run_batched(g, false, num_sets, in_data, out_data, workspace, workspace_bytes, stream);
}

int mg_compare_fingerprint_rows(mg_runtime *rt, const uint16_t *a, const uint16_t *b, int64_t rows, int64_t row_elements,
                                int32_t *equal_flags, int32_t *mismatch_count, void *stream) {
  if (int dry_st = refuse_dry(rt)) return dry_st;
  if (!rt || !rt->dmm) return fail(MG_ERR_INVALID_ARGUMENT, "no runtime");
  int st = mgd_compare_rows_u16(a, b, rows, row_elements, equal_flags, mismatch_count, stream);
  return st == MG_OK ? MG_OK : fail(st, mgd_last_error());
}

int mg_tensor_has_same_fingerprint(mg_runtime *rt, const mg_tensor *a, const mg_tensor *b, int32_t *same) {
  if (int dry_st = refuse_dry(rt)) return dry_st;
  if (!rt || !rt->dmm || !a || !b || !same) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  *same = 0;
  if (a->num_dims != b->num_dims) return MG_OK;
  int64_t n = 1;
  for (int i = 0; i < a->num_dims; i++) {
    if (a->dim[i] != b->dim[i]) return MG_OK;
    n *= a->dim[i];
  }
  int st = mgd_compare_u16(a->fp_ptr, b->fp_ptr, n, rt->dmm->flag_word, nullptr);
  if (st != MG_OK) return fail(st, mgd_last_error());
  int flag = 0;
  MG_CUDA_TRY(cudaMemcpy(&flag, rt->dmm->flag_word, sizeof(int), cudaMemcpyDeviceToHost));
  *same = flag == 1;
  return MG_OK;
}

int mg_verify_candidates(mg_runtime *rt, const mg_tensor *reference, mg_graph *const *candidates,
                         const mg_tensor *outputs, int32_t n, int32_t *same, void *stream) {
  if (int dry_st = refuse_dry(rt)) return dry_st;
  if (!rt || !rt->dmm || !reference || !candidates || !outputs || !same || n < 0) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  if (n == 0) return MG_OK;
  // n result flags from the arena: taken here, given back (LIFO) before returning; nothing else allocates in between
  struct ArenaScratch {
    DeviceMemoryManager *dmm;
    void *p;
    ~ArenaScratch() { if (p) dmm->free_raw(p); }
  } scratch{rt->dmm, rt->dmm->allocate_raw(sizeof(int32_t) * (size_t)n)};
  if (!scratch.p) return fail(MG_ERR_OUT_OF_MEMORY, "device arena exhausted (verification flags)");
  int32_t *flags = static_cast<int32_t *>(scratch.p);
  MG_CUDA_TRY(cudaMemsetAsync(flags, 0, sizeof(int32_t) * (size_t)n, (cudaStream_t)stream));
  int64_t ref_elems = 1;
  for (int d = 0; d < reference->num_dims; d++) ref_elems *= reference->dim[d];
  for (int32_t i = 0; i < n; i++)
    if (!candidates[i]) return fail(MG_ERR_INVALID_ARGUMENT, "null candidate graph");
  // Candidate i runs on lane i % lanes: the lanes start after what the caller's stream holds so far (the inputs, the
  // reference's fingerprint, the cleared flags) and the caller's stream continues after all of them.
  int const lanes = n < kVerifyLanes ? n : kVerifyLanes;
  if (!ensure_lanes(rt)) return fail(MG_ERR_CUDA, "cannot create the verification streams");
  MG_CUDA_TRY(cudaEventRecord(rt->fork, (cudaStream_t)stream));
  for (int l = 0; l < lanes; l++) MG_CUDA_TRY(cudaStreamWaitEvent(rt->lanes[l], rt->fork, 0));
  int failed_st = MG_OK;
  for (int32_t i = 0; i < n && failed_st == MG_OK; i++) {
    void *lane = rt->lanes[i % lanes];
    int st = launch_all(candidates[i], true, true, lane);
    if (st != MG_OK) { failed_st = st; break; }
    bool same_shape = outputs[i].num_dims == reference->num_dims && outputs[i].fp_ptr != nullptr;
    for (int d = 0; same_shape && d < reference->num_dims; d++) same_shape = outputs[i].dim[d] == reference->dim[d];
    if (!same_shape) continue; // flag stays 0
    st = mgd_compare_u16(outputs[i].fp_ptr, reference->fp_ptr, ref_elems, flags + i, lane);
    if (st != MG_OK) failed_st = fail(st, mgd_last_error());
  }
  for (int l = 0; l < lanes; l++) { // joined also when a launch was refused: the flags go back to the arena below
    cudaEventRecord(rt->lane_done[l], rt->lanes[l]);
    cudaStreamWaitEvent((cudaStream_t)stream, rt->lane_done[l], 0);
  }
  if (failed_st != MG_OK) {
    cudaStreamSynchronize((cudaStream_t)stream);
    return failed_st;
  }
  MG_CUDA_TRY(cudaMemcpyAsync(same, flags, sizeof(int32_t) * (size_t)n, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  MG_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
  int32_t code = 0;
  int st = mgd_read_and_clear_device_error(&code);
  if (st != MG_OK) return fail(st, mgd_last_error());
  if (code != 0) return fail(MG_ERR_DEVICE_TIMEOUT, "a kernel gave up a bounded wait (device status word set)");
  for (int32_t i = 0; i < n; i++) same[i] = same[i] == 1;
  return MG_OK;
}

static int64_t pod_elements(const mg_tensor *t) {
  int64_t n = 1;
  for (int i = 0; i < t->num_dims; i++) n *= t->dim[i];
  return n;
}
static size_t pod_data_bytes(const mg_tensor *t) {
  return (size_t)pod_elements(t) * type::get_datatype_size((type::DataType)t->data_type);
}

int mg_tensor_fill_fingerprint_reference(mg_runtime *rt, const mg_tensor *t) {
  if (int dry_st = refuse_dry(rt)) return dry_st;
  mg::stream_wrote_anything(nullptr);
  if (!rt || !rt->dmm || !t || !t->fp_ptr) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  int st = mgd_fill_fingerprint_reference(t->fp_ptr, pod_elements(t), nullptr);
  return st == MG_OK ? synchronize_and_check() : fail(st, mgd_last_error());
}
int mg_tensor_fill_fingerprint_seeded(mg_runtime *rt, const mg_tensor *t, uint64_t seed, uint32_t modulus) {
  if (int dry_st = refuse_dry(rt)) return dry_st;
  mg::stream_wrote_anything(nullptr);
  if (!rt || !rt->dmm || !t || !t->fp_ptr || modulus == 0 || modulus > 65536) return fail(MG_ERR_INVALID_ARGUMENT, "bad fill request");
  int st = mgd_fill_fingerprint_seeded(t->fp_ptr, pod_elements(t), seed, modulus, nullptr);
  return st == MG_OK ? synchronize_and_check() : fail(st, mgd_last_error());
}
int mg_tensor_fill_data_seeded(mg_runtime *rt, const mg_tensor *t, uint64_t seed, float sigma) {
  if (int dry_st = refuse_dry(rt)) return dry_st;
  mg::stream_wrote_anything(nullptr);
  if (!rt || !rt->dmm || !t || !t->data_ptr) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  int st = mgd_fill_data_seeded(t->data_ptr, pod_elements(t), seed, sigma, t->data_type, nullptr);
  return st == MG_OK ? synchronize_and_check() : fail(st, mgd_last_error());
}
int mg_tensor_upload_fingerprint(mg_runtime *rt, const mg_tensor *t, const uint16_t *host) {
  if (int dry_st = refuse_dry(rt)) return dry_st;
  mg::stream_wrote_anything(nullptr);
  if (!rt || !t || !host || !t->fp_ptr) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  MG_CUDA_TRY(cudaMemcpy(t->fp_ptr, host, (size_t)pod_elements(t) * 2, cudaMemcpyHostToDevice));
  return MG_OK;
}
int mg_tensor_download_fingerprint(mg_runtime *rt, const mg_tensor *t, uint16_t *host) {
  if (int dry_st = refuse_dry(rt)) return dry_st;
  if (!rt || !t || !host || !t->fp_ptr) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  MG_CUDA_TRY(cudaMemcpy(host, t->fp_ptr, (size_t)pod_elements(t) * 2, cudaMemcpyDeviceToHost));
  return MG_OK;
}
int mg_tensor_upload_data(mg_runtime *rt, const mg_tensor *t, const void *host) {
  if (int dry_st = refuse_dry(rt)) return dry_st;
  mg::stream_wrote_anything(nullptr);
  if (!rt || !t || !host || !t->data_ptr) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  MG_CUDA_TRY(cudaMemcpy(t->data_ptr, host, pod_data_bytes(t), cudaMemcpyHostToDevice));
  return MG_OK;
}
int mg_tensor_download_data(mg_runtime *rt, const mg_tensor *t, void *host) {
  if (int dry_st = refuse_dry(rt)) return dry_st;
  if (!rt || !t || !host || !t->data_ptr) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  MG_CUDA_TRY(cudaMemcpy(host, t->data_ptr, pod_data_bytes(t), cudaMemcpyDeviceToHost));
  return MG_OK;
}
int mg_tensor_upload_data_async(mg_runtime *rt, const mg_tensor *t, const void *host, void *stream) {
  if (int dry_st = refuse_dry(rt)) return dry_st;
  mg::stream_wrote_anything(stream);
  if (!rt || !t || !host || !t->data_ptr) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  MG_CUDA_TRY(cudaMemcpyAsync(t->data_ptr, host, pod_data_bytes(t), cudaMemcpyHostToDevice, (cudaStream_t)stream));
  return MG_OK;
}
int mg_tensor_download_data_async(mg_runtime *rt, const mg_tensor *t, void *host, void *stream) {
  if (int dry_st = refuse_dry(rt)) return dry_st;
  if (!rt || !t || !host || !t->data_ptr) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  MG_CUDA_TRY(cudaMemcpyAsync(host, t->data_ptr, pod_data_bytes(t), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  return MG_OK;
}

int mg_graph_rebind_input(mg_graph *g, int32_t idx, void *data_ptr, uint16_t *fp_ptr) {
  KNOperator *op = get_op(g, idx);
  if (!op || op->op_type != type::KN_INPUT_OP) return fail(MG_ERR_INVALID_ARGUMENT, "not an input operator");
  DTensor &t = op->output_tensors[0];
  // Tensor descriptors are copied by value into their consumers: update every copy.  The arena keeps
  // owning the original buffers; the caller owns the ones bound here.
  for (KNOperator *o : g->graph.operators)
    for (DTensor &in : o->input_tensors)
      if (in.owner_op == op && in.owner_ts_idx == 0) {
        if (data_ptr) in.data_ptr = data_ptr;
        if (fp_ptr) in.fp_ptr = fp_ptr;
      }
  (void)t;
  mg::forget_streams(); // the new buffers may have been written by anything, on any stream
  static_cast<kernel::KNInputOp *>(op)->skip_fill = true;
  return MG_OK;
}

int mg_capture_begin(void *stream) {
  if (!stream) return fail(MG_ERR_INVALID_ARGUMENT, "capture needs a non-default stream");
  MG_CUDA_TRY(cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeThreadLocal));
  return MG_OK;
}
int mg_capture_end(void *stream, void **captured) {
  if (!stream || !captured) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  *captured = nullptr;
  cudaGraph_t graph = nullptr;
  MG_CUDA_TRY(cudaStreamEndCapture((cudaStream_t)stream, &graph));
  cudaGraphExec_t exec = nullptr;
  int st = mg::cuda_status((int)cudaGraphInstantiate(&exec, graph, 0), "cudaGraphInstantiate");
  cudaGraphDestroy(graph);
  if (st != MG_OK) return st;
  *captured = exec;
  return MG_OK;
}
int mg_captured_launch(void *captured, void *stream) {
  if (!captured) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  MG_CUDA_TRY(cudaGraphLaunch((cudaGraphExec_t)captured, (cudaStream_t)stream));
  return MG_OK;
}
int mg_captured_destroy(void *captured) {
  if (!captured) return fail(MG_ERR_INVALID_ARGUMENT, "null argument");
  MG_CUDA_TRY(cudaGraphExecDestroy((cudaGraphExec_t)captured));
  return MG_OK;
}

int mg_device_synchronize(void) { return synchronize_and_check(); }
const char *mg_last_error(void) { return mg::last_error(); }
const char *mg_version(void) { return "mugraph-b200 0.1 (sm_100a)"; }
uint64_t mg_launch_count(void) { return mgd_launch_count(); }

} // extern "C"
