// Host side of the kernel graph: device tensors, the arena, kernel-level operators and the
// customized operator that owns a threadblock graph.
//
// Reference behaviour followed: src/kernel/{graph,operator,customized,matmul,element_unary,
// element_binary,reduction,device_tensor}.cc and src/kernel/device_memory_manager.cu.  CUDA is
// reached only through the runtime API (memory, events) and the kernel-level C ABI
// (mugraph_device.h); no kernel is defined in this file.
#include "kernel_select.h"
#include "mirage/kernel/device_memory_manager.h"
#include "mirage/kernel/graph.h"
#include "mugraph.h"
#include "status.h"
#include <algorithm>
#include <cassert>
#include <cstdio>
#include <cstring>
#include <cuda_runtime.h>
#include <mutex>
#include <unordered_map>

namespace mg {
static thread_local std::string g_error;
void set_error(std::string const &m) { g_error = m; }
char const *last_error() { return g_error.c_str(); }
int cuda_status(int err, char const *what) {
  if (err == (int)cudaSuccess) return MG_OK;
  set_error(std::string(what) + ": " + cudaGetErrorString((cudaError_t)err));
  // leave the sticky error of this call behind so the next call starts clean
  cudaGetLastError();
  return (err == (int)cudaErrorNoDevice || err == (int)cudaErrorInsufficientDriver) ? MG_ERR_NO_DEVICE : MG_ERR_CUDA;
}
} // namespace mg

namespace mirage {
namespace kernel {

using namespace mirage::type;
using mirage::threadblock::ExecutionPlan;
using mirage::threadblock::STensor;

namespace {
void record_anything(void *stream); // defined with the stream bookkeeping below
}

// ---- DTensor ---------------------------------------------------------------------------------
int DTensor::next_guid = 10000000;

DTensor::DTensor()
    : data_type(DT_UNKNOWN), layout(mirage::layout::DmemUnknownLayout), num_dims(0), guid(0), owner_op(nullptr),
      owner_ts_idx(-1000), data_ptr(nullptr), fp_ptr(nullptr) {
  for (int &d : dim) d = 0;
}

bool DTensor::operator==(DTensor const &b) const {
  if (data_type != b.data_type || layout != b.layout || num_dims != b.num_dims) return false;
  for (int i = 0; i < num_dims; i++)
    if (dim[i] != b.dim[i]) return false;
  return owner_op == b.owner_op && owner_ts_idx == b.owner_ts_idx;
}

bool DTensor::has_same_fingerprint(DTensor const &ref) const {
  if (num_dims != ref.num_dims) return false;
  for (int i = 0; i < num_dims; i++)
    if (dim[i] != ref.dim[i]) return false;
  DeviceMemoryManager *dmm = DeviceMemoryManager::get_instance();
  if (!dmm || dmm->dry || !fp_ptr || !ref.fp_ptr) return false;
  if (mgd_compare_u16(fp_ptr, ref.fp_ptr, (int64_t)num_elements(), dmm->flag_word, nullptr) != MG_OK) return false;
  int flag = 0;
  if (cudaMemcpy(&flag, dmm->flag_word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return false;
  return flag == 1;
}

// ---- DeviceMemoryManager -----------------------------------------------------------------------
DeviceMemoryManager *DeviceMemoryManager::singleton = nullptr;
static constexpr size_t kAlign = 256;
static size_t round_up(size_t n) { return (n + kAlign - 1) / kAlign * kAlign; }

DeviceMemoryManager::DeviceMemoryManager(int dev, size_t arena_bytes)
    : base_ptr(nullptr), offset(0), total_size(arena_bytes), exp_lookup_table(nullptr), div_p_lookup_table(nullptr),
      div_q_lookup_table(nullptr), device(dev), max_smem(MAX_SMEM_SIZE), specialise(2), launch_policy(0), flag_word(nullptr),
      dry(dev < 0), ok_(false) {
  if (dry) {
    // Planning-only runtime: addresses are handed out from a range that is never dereferenced, so that
    // graph construction, validation, lowering and kernel selection can be exercised without a GPU.
    // Every launch and copy refuses to run on it.
    base_ptr = reinterpret_cast<char *>((uintptr_t)1 << 40);
  } else {
    if (mg::cuda_status(cudaSetDevice(dev), "cudaSetDevice")) return;
    if (mg::cuda_status(cudaMalloc((void **)&base_ptr, total_size), "cudaMalloc(arena)")) return;
  }
  // Tables, bit-identical to the reference's: powers of 3 modulo P (3 has order Q), and modular
  // inverses modulo P and Q where 0 (and 1) map to 1.
  FPType exp_table[FP_Q], div_p[FP_P], div_q[FP_Q];
  exp_table[0] = 1;
  for (int i = 1; i < FP_Q; i++) exp_table[i] = (FPType)((exp_table[i - 1] * FP_EXP_BASE) % FP_P);
  assert((exp_table[FP_Q - 1] * FP_EXP_BASE) % FP_P == 1);
  for (int i = 0; i < FP_P; i++) {
    div_p[i] = 1;
    for (int j = 1; j < FP_P; j++)
      if ((i * j) % FP_P == 1) div_p[i] = (FPType)j;
  }
  for (int i = 0; i < FP_Q; i++) {
    div_q[i] = 1;
    for (int j = 1; j < FP_Q; j++)
      if ((i * j) % FP_Q == 1) div_q[i] = (FPType)j;
  }
  exp_lookup_table = (FPType *)(base_ptr + offset);
  offset += (off_t)round_up(sizeof(exp_table));
  div_p_lookup_table = (FPType *)(base_ptr + offset);
  offset += (off_t)round_up(sizeof(div_p));
  div_q_lookup_table = (FPType *)(base_ptr + offset);
  offset += (off_t)round_up(sizeof(div_q));
  flag_word = (int *)(base_ptr + offset);
  offset += (off_t)kAlign;
  if (dry) {
    ok_ = mgd_tables_init(exp_table, div_p, div_q) == MG_OK;
    return;
  }
  if (mg::cuda_status(cudaMemcpy(exp_lookup_table, exp_table, sizeof(exp_table), cudaMemcpyHostToDevice), "tables"))
    return;
  if (mg::cuda_status(cudaMemcpy(div_p_lookup_table, div_p, sizeof(div_p), cudaMemcpyHostToDevice), "tables")) return;
  if (mg::cuda_status(cudaMemcpy(div_q_lookup_table, div_q, sizeof(div_q), cudaMemcpyHostToDevice), "tables")) return;
  if (mgd_tables_init(exp_table, div_p, div_q) != MG_OK) {
    mg::set_error(mgd_last_error());
    return;
  }
  ok_ = true;
}

DeviceMemoryManager::~DeviceMemoryManager() {
  if (base_ptr && !dry) cudaFree(base_ptr);
}

int DeviceMemoryManager::create(int dev, size_t arena_bytes, char const **error) {
  if (singleton) {
    mg::set_error("a device memory manager already exists in this process");
    if (error) *error = mg::last_error();
    return MG_ERR_INVALID_ARGUMENT;
  }
  if (arena_bytes == 0) arena_bytes = (size_t)10 << 30; // the reference's arena size
  if (dev >= 0) {
    int count = 0;
    int st = mg::cuda_status(cudaGetDeviceCount(&count), "cudaGetDeviceCount");
    if (st == MG_OK && count == 0) {
      mg::set_error("no CUDA device");
      st = MG_ERR_NO_DEVICE;
    }
    if (st != MG_OK) {
      if (error) *error = mg::last_error();
      return st == MG_ERR_CUDA ? MG_ERR_NO_DEVICE : st;
    }
  }
  auto *m = new DeviceMemoryManager(dev, arena_bytes);
  if (!m->ok_) {
    if (error) *error = mg::last_error();
    delete m;
    return MG_ERR_CUDA;
  }
  singleton = m;
  return MG_OK;
}

void DeviceMemoryManager::destroy() {
  delete singleton;
  singleton = nullptr;
}

DeviceMemoryManager *DeviceMemoryManager::get_instance() {
  if (singleton == nullptr) {
    char const *err = nullptr;
    if (create(0, 0, &err) != MG_OK) {
      // The reference terminates here (checkCUDA -> FatalError).  There is no CPU fallback.
      std::fprintf(stderr, "mugraph: cannot create the device memory manager: %s\n", err ? err : "?");
      std::abort();
    }
  }
  return singleton;
}

bool DeviceMemoryManager::can_allocate(size_t data_bytes, size_t fp_bytes) const {
  return (size_t)offset + round_up(data_bytes) + round_up(fp_bytes) <= total_size;
}

bool DeviceMemoryManager::allocate(DTensor &t, bool with_fp) {
  size_t db = round_up(t.data_size()), fb = with_fp ? round_up(t.fingerprint_size()) : 0;
  if ((size_t)offset + db + fb > total_size) return false;
  t.data_ptr = base_ptr + offset;
  allocated_tensors.push_back({t.data_ptr, db});
  offset += (off_t)db;
  t.fp_ptr = nullptr;
  if (with_fp) {
    t.fp_ptr = (FPType *)(base_ptr + offset);
    allocated_tensors.push_back({t.fp_ptr, fb});
    offset += (off_t)fb;
  }
  return true;
}

bool DeviceMemoryManager::free(DTensor &t) {
  if (t.fp_ptr != nullptr) {
    if (allocated_tensors.empty() || allocated_tensors.back().first != t.fp_ptr) return false;
    offset -= (off_t)allocated_tensors.back().second;
    allocated_tensors.pop_back();
  }
  if (allocated_tensors.empty() || allocated_tensors.back().first != t.data_ptr) return false;
  offset -= (off_t)allocated_tensors.back().second;
  allocated_tensors.pop_back();
  return true;
}

void *DeviceMemoryManager::allocate_raw(size_t bytes) {
  size_t b = round_up(bytes);
  if ((size_t)offset + b > total_size) return nullptr;
  void *p = base_ptr + offset;
  allocated_tensors.push_back({p, b});
  offset += (off_t)b;
  return p;
}
bool DeviceMemoryManager::free_raw(void *p) {
  if (allocated_tensors.empty() || allocated_tensors.back().first != p) return false;
  offset -= (off_t)allocated_tensors.back().second;
  allocated_tensors.pop_back();
  return true;
}

// ---- KNOperator ----------------------------------------------------------------------------------
KNOperator::KNOperator(KNOperatorType t) : op_type(t) {}
KNOperator::KNOperator(KNOperatorType t, DTensor const &a) : op_type(t) { input_tensors.push_back(a); }
KNOperator::KNOperator(KNOperatorType t, DTensor const &a, DTensor const &b) : op_type(t) {
  input_tensors.push_back(a);
  input_tensors.push_back(b);
}
KNOperator::KNOperator(KNOperatorType t, std::vector<DTensor> const &ins) : op_type(t), input_tensors(ins) {}
KNOperator::~KNOperator() {}

static void free_outputs(std::vector<DTensor> &outs) {
  DeviceMemoryManager *dmm = DeviceMemoryManager::get_instance();
  for (int i = (int)outs.size() - 1; i >= 0; i--) {
    bool ok = dmm->free(outs[i]);
    assert(ok && "device tensors must be released in reverse order of allocation");
    (void)ok;
  }
}

static int refuse_if_dry() {
  if (DeviceMemoryManager::get_instance()->dry) {
    mg::set_error("planning-only runtime (device < 0): nothing can be launched");
    return MG_ERR_NO_DEVICE;
  }
  return MG_OK;
}

static bool sync_ok(int st) {
  if (st != MG_OK) {
    if (!*mg::last_error()) mg::set_error(mgd_last_error());
    return false;
  }
  return mg::cuda_status(cudaDeviceSynchronize(), "cudaDeviceSynchronize") == MG_OK;
}

bool KNOperator::profile_with_events(ProfileResult &result, int warmup, int iters) {
  result.run_time = ProfileResult::infinity().run_time;
  if (refuse_if_dry()) return false;
  cudaEvent_t ev[2];
  if (mg::cuda_status(cudaDeviceSynchronize(), "cudaDeviceSynchronize")) return false;
  if (mg::cuda_status(cudaEventCreate(&ev[0]), "cudaEventCreate")) return false;
  if (mg::cuda_status(cudaEventCreate(&ev[1]), "cudaEventCreate")) return false;
  bool ok = true;
  for (int i = 0; i < warmup && ok; i++) ok = launch_float(nullptr) == MG_OK;
  cudaEventRecord(ev[0], nullptr);
  for (int i = 0; i < iters && ok; i++) ok = launch_float(nullptr) == MG_OK;
  cudaEventRecord(ev[1], nullptr);
  float ms = 0.f;
  if (mg::cuda_status(cudaEventSynchronize(ev[1]), "cudaEventSynchronize")) ok = false;
  if (ok && mg::cuda_status(cudaEventElapsedTime(&ms, ev[0], ev[1]), "cudaEventElapsedTime")) ok = false;
  cudaEventDestroy(ev[0]);
  cudaEventDestroy(ev[1]);
  if (ok) result.run_time = ms / (float)std::max(1, iters);
  return ok;
}

// ---- input ---------------------------------------------------------------------------------------
KNInputOp::KNInputOp(std::vector<int> const &dims, DataType dt, mirage::layout::DmemLayout lay)
    : KNOperator(KN_INPUT_OP) {
  DTensor t;
  t.num_dims = (int)dims.size();
  assert(t.num_dims <= MAX_TENSOR_DIMS);
  for (int i = 0; i < t.num_dims; i++) t.dim[i] = dims[i];
  t.data_type = dt;
  t.layout = lay;
  t.owner_op = this;
  t.owner_ts_idx = 0;
  t.guid = (size_t)DTensor::next_guid++;
  bool ok = DeviceMemoryManager::get_instance()->allocate(t);
  assert(ok && "device arena exhausted");
  (void)ok;
  output_tensors.push_back(t);
}
KNInputOp::~KNInputOp() { free_outputs(output_tensors); }
bool KNInputOp::profile(ProfileResult &r) {
  r.run_time = 0.f;
  return true;
}
int KNInputOp::launch_fingerprint(void *stream) {
  if (int dry_st = refuse_if_dry()) return dry_st;
  if (skip_fill) return MG_OK;
  record_anything(stream);
  return mgd_fill_fingerprint_reference(output_tensors[0].fp_ptr, (int64_t)output_tensors[0].num_elements(), stream);
}
int KNInputOp::launch_float(void *) { return MG_OK; }
bool KNInputOp::fingerprint(void) { return sync_ok(launch_fingerprint(nullptr)); }

// ---- un-fused operators ----------------------------------------------------------------------------
static DTensor owned_output(KNOperator *owner, DTensor proto) {
  proto.owner_op = owner;
  proto.owner_ts_idx = 0;
  proto.guid = (size_t)DTensor::next_guid++;
  bool ok = DeviceMemoryManager::get_instance()->allocate(proto);
  assert(ok && "device arena exhausted");
  (void)ok;
  return proto;
}

KNMatmulOp::KNMatmulOp(DTensor const &A, DTensor const &B) : KNOperator(KN_MATMUL_OP, A, B) {
  assert(A.num_dims == B.num_dims && A.dim[A.num_dims - 1] == B.dim[B.num_dims - 2]);
  DTensor C = A;
  C.dim[C.num_dims - 1] = B.dim[B.num_dims - 1];
  C.layout = mirage::layout::DmemRowMajor;
  output_tensors.push_back(owned_output(this, C));
}
KNMatmulOp::~KNMatmulOp() { free_outputs(output_tensors); }
int KNMatmulOp::launch_fingerprint(void *stream) {
  if (int dry_st = refuse_if_dry()) return dry_st;
  record_anything(stream);
  DTensor const &A = input_tensors[0], &B = input_tensors[1], &C = output_tensors[0];
  int nd = A.num_dims, batches = 1;
  for (int i = 0; i < nd - 2; i++) batches *= A.dim[i];
  return mgd_kn_matmul_fingerprint(A.fp_ptr, B.fp_ptr, C.fp_ptr, batches, C.dim[nd - 2], C.dim[nd - 1],
                                   A.dim[nd - 1], stream);
}
int KNMatmulOp::launch_float(void *stream) {
  if (int dry_st = refuse_if_dry()) return dry_st;
  record_anything(stream);
  DTensor const &A = input_tensors[0], &B = input_tensors[1], &C = output_tensors[0];
  int nd = A.num_dims, batches = 1;
  for (int i = 0; i < nd - 2; i++) batches *= A.dim[i];
  return mgd_kn_matmul_float(A.data_ptr, B.data_ptr, C.data_ptr, batches, C.dim[nd - 2], C.dim[nd - 1],
                             A.dim[nd - 1], (int)A.layout, (int)B.layout, (int)A.data_type, stream);
}
bool KNMatmulOp::fingerprint(void) { return sync_ok(launch_fingerprint(nullptr)); }
bool KNMatmulOp::profile(ProfileResult &r) { return profile_with_events(r, 16, 16); }

KNElementUnaryOp::KNElementUnaryOp(DTensor const &A, KNOperatorType t) : KNOperator(t, A) {
  output_tensors.push_back(owned_output(this, A));
}
KNElementUnaryOp::~KNElementUnaryOp() { free_outputs(output_tensors); }
int KNElementUnaryOp::launch_fingerprint(void *stream) {
  if (int dry_st = refuse_if_dry()) return dry_st;
  record_anything(stream);
  return mgd_kn_exp_fingerprint(input_tensors[0].fp_ptr, output_tensors[0].fp_ptr,
                                (int64_t)output_tensors[0].num_elements(), stream);
}
int KNElementUnaryOp::launch_float(void *stream) {
  if (int dry_st = refuse_if_dry()) return dry_st;
  record_anything(stream);
  return mgd_kn_exp_float(input_tensors[0].data_ptr, output_tensors[0].data_ptr,
                          (int64_t)output_tensors[0].num_elements(), (int)input_tensors[0].data_type, stream);
}
bool KNElementUnaryOp::fingerprint(void) { return sync_ok(launch_fingerprint(nullptr)); }
bool KNElementUnaryOp::profile(ProfileResult &r) { return profile_with_events(r, 16, 16); }

KNElementBinaryOp::KNElementBinaryOp(DTensor const &A, DTensor const &B, KNOperatorType t) : KNOperator(t, A, B) {
  assert(A.num_dims == B.num_dims);
  DTensor C = A;
  for (int i = 0; i < C.num_dims; i++) C.dim[i] = std::max(A.dim[i], B.dim[i]);
  output_tensors.push_back(owned_output(this, C));
}
KNElementBinaryOp::~KNElementBinaryOp() { free_outputs(output_tensors); }
static void right_aligned_dims(DTensor const &t, int32_t out[4]) {
  for (int i = 0; i < 4; i++) out[i] = 1;
  for (int i = 0; i < t.num_dims; i++) out[4 - t.num_dims + i] = t.dim[i];
}
int KNElementBinaryOp::launch_fingerprint(void *stream) {
  if (int dry_st = refuse_if_dry()) return dry_st;
  record_anything(stream);
  int32_t xd[4], yd[4], zd[4];
  right_aligned_dims(input_tensors[0], xd);
  right_aligned_dims(input_tensors[1], yd);
  right_aligned_dims(output_tensors[0], zd);
  return mgd_kn_binary_fingerprint((int)op_type, input_tensors[0].fp_ptr, xd, input_tensors[1].fp_ptr, yd,
                                   output_tensors[0].fp_ptr, zd, stream);
}
int KNElementBinaryOp::launch_float(void *stream) {
  if (int dry_st = refuse_if_dry()) return dry_st;
  record_anything(stream);
  int32_t xd[4], yd[4], zd[4];
  right_aligned_dims(input_tensors[0], xd);
  right_aligned_dims(input_tensors[1], yd);
  right_aligned_dims(output_tensors[0], zd);
  return mgd_kn_binary_float((int)op_type, input_tensors[0].data_ptr, xd, input_tensors[1].data_ptr, yd,
                             output_tensors[0].data_ptr, zd, (int)input_tensors[0].data_type, stream);
}
bool KNElementBinaryOp::fingerprint(void) { return sync_ok(launch_fingerprint(nullptr)); }
bool KNElementBinaryOp::profile(ProfileResult &r) { return profile_with_events(r, 16, 16); }

KNReductionOp::KNReductionOp(DTensor const &A, int dim, int size)
    : KNOperator((KNOperatorType)(KN_REDUCTION_0_OP + dim), A), reduction_dim_idx(dim), reduction_dim_size(size) {
  assert(dim < A.num_dims && A.dim[dim] % size == 0);
  DTensor out = A;
  out.dim[dim] = size;
  output_tensors.push_back(owned_output(this, out));
}
KNReductionOp::~KNReductionOp() { free_outputs(output_tensors); }
static void reduction_geometry(DTensor const &in, DTensor const &out, int dim, int64_t &is, int64_t &os, int &factor) {
  is = os = 1;
  for (int i = dim; i < out.num_dims; i++) {
    os *= out.dim[i];
    is *= in.dim[i];
  }
  factor = in.dim[dim] / out.dim[dim];
}
int KNReductionOp::launch_fingerprint(void *stream) {
  if (int dry_st = refuse_if_dry()) return dry_st;
  record_anything(stream);
  int64_t is, os;
  int factor;
  reduction_geometry(input_tensors[0], output_tensors[0], reduction_dim_idx, is, os, factor);
  return mgd_kn_reduction_fingerprint(input_tensors[0].fp_ptr, output_tensors[0].fp_ptr,
                                      (int64_t)output_tensors[0].num_elements(), factor, is, os, stream);
}
int KNReductionOp::launch_float(void *stream) {
  if (int dry_st = refuse_if_dry()) return dry_st;
  record_anything(stream);
  int64_t is, os;
  int factor;
  reduction_geometry(input_tensors[0], output_tensors[0], reduction_dim_idx, is, os, factor);
  return mgd_kn_reduction_float(input_tensors[0].data_ptr, output_tensors[0].data_ptr,
                                (int64_t)output_tensors[0].num_elements(), factor, is, os,
                                (int)input_tensors[0].data_type, stream);
}
bool KNReductionOp::fingerprint(void) { return sync_ok(launch_fingerprint(nullptr)); }
bool KNReductionOp::profile(ProfileResult &r) { return profile_with_events(r, 16, 16); }

// ---- what the previous launch on a stream wrote -------------------------------------------------------
// The split-KV attention kernel is launched with programmatic stream serialisation and may start loading its
// inputs while the previous kernel of the stream is still running.  That is only allowed when the library KNOWS
// that kernel and knows that it did not write those inputs.  Every launch through this file therefore records,
// per stream, what it wrote: a list of address ranges for the split-KV kernel, "anything" for every other kernel
// of the library and for copies and fills that go through the C ABI.  A stream the library has not launched on
// yet, and a stream on which the caller reported work of its own (mg_stream_inputs_written), count as
// "anything": the early loads are then left out for the next launch.
namespace {
struct Range { char const *lo, *hi; };
struct Written { std::vector<Range> last, before; }; // by the launch in front, and by the one in front of that
std::mutex g_track_mutex;
std::unordered_map<void *, Written> g_last_outputs;
constexpr size_t kMaxTrackedStreams = 4096; // the table is cleared beyond this: forgetting is the safe direction
Range const kAnything{(char const *)nullptr, (char const *)UINTPTR_MAX};

// Two launches deep: a kernel that is released as soon as its predecessor starts may run beside the launch in front of
// that one (never beside an older one: see the release rules in attn_split.cu and attn_rows_pp.cu).
void record_outputs(void *stream, std::vector<Range> const &r) {
  std::lock_guard<std::mutex> lock(g_track_mutex);
  if (g_last_outputs.size() > kMaxTrackedStreams) g_last_outputs.clear();
  auto it = g_last_outputs.find(stream);
  if (it == g_last_outputs.end()) {
    g_last_outputs[stream] = Written{r, {kAnything}}; // what ran before the first launch seen here is unknown
    return;
  }
  it->second.before = std::move(it->second.last);
  it->second.last = r;
}
void record_anything(void *stream) { record_outputs(stream, {kAnything}); }
bool inputs_untouched(void *stream, std::vector<Range> const &inputs) {
  std::lock_guard<std::mutex> lock(g_track_mutex);
  auto it = g_last_outputs.find(stream);
  if (it == g_last_outputs.end()) return false; // unknown predecessor
  for (std::vector<Range> const *written : {&it->second.last, &it->second.before})
    for (Range const &a : *written)
      for (Range const &b : inputs)
        if (a.lo < b.hi && b.lo < a.hi) return false;
  return true;
}
Range range_of(void const *p, size_t bytes) { return Range{(char const *)p, (char const *)p + bytes}; }
} // namespace

} // namespace kernel
} // namespace mirage
namespace mg {
void stream_wrote_anything(void *stream) { mirage::kernel::record_anything(stream); }
void forget_streams() {
  std::lock_guard<std::mutex> lock(mirage::kernel::g_track_mutex);
  mirage::kernel::g_last_outputs.clear();
}
} // namespace mg
namespace mirage {
namespace kernel {

// ---- customized operator -----------------------------------------------------------------------------
KNCustomizedOp::KNCustomizedOp(Deferred, std::vector<DTensor> const &ins, ExecutionPlan const &p)
    : KNOperator(KN_CUSTOMIZED_OP, ins), plan(p), bgraph(p.grid_dim, p.block_dim, p.forloop_range, p.reduction_dimx) {
  bgraph.max_smem = DeviceMemoryManager::get_instance()->max_smem;
}

KNCustomizedOp::KNCustomizedOp(std::vector<DTensor> const &ins, ExecutionPlan const &p)
    : KNCustomizedOp(Deferred{}, ins, p) {
  std::string err;
  int st = MG_OK;
  bool ok = build_from_plan(&err, &st);
  if (!ok) std::fprintf(stderr, "KNCustomizedOp: %s\n", err.c_str());
  assert(ok && "invalid execution plan");
  (void)ok;
  after_build();
}

// Decide the kernels now (the choice needs no device) and reserve what the fused launch needs.
void KNCustomizedOp::after_build() {
  if (!ensure_lowered()) return;
  DeviceMemoryManager *dmm = DeviceMemoryManager::get_instance();
  if (kernel_fp_ == mg::KERNEL_ATTN_SPLIT || kernel_float_ == mg::KERNEL_ATTN_SPLIT) {
    size_t bytes = (size_t)program_.grid[0] * sizeof(int);
    tickets_ = static_cast<int *>(dmm->allocate_raw(bytes));
    if (tickets_ && !dmm->dry && cudaMemset(tickets_, 0, bytes) != cudaSuccess) {
      cudaGetLastError();
      dmm->free_raw(tickets_);
      tickets_ = nullptr;
    }
  }
}

KNCustomizedOp *KNCustomizedOp::create(std::vector<DTensor> const &ins, ExecutionPlan const &p, std::string *error,
                                       int *status) {
  if (p.forloop_range <= 0 || p.reduction_dimx <= 0 || p.grid_dim.x == 0 || p.grid_dim.y == 0 || p.grid_dim.z == 0) {
    if (error) *error = "forloop_range, reduction_dimx and grid_dim must be positive";
    if (status) *status = MG_ERR_INVALID_GRAPH;
    return nullptr;
  }
  auto *op = new KNCustomizedOp(Deferred{}, ins, p);
  if (!op->build_from_plan(error, status)) {
    delete op;
    return nullptr;
  }
  op->after_build();
  return op;
}

// Replays the plan on the threadblock graph builder, then turns every operator result nobody
// consumes into an output (in operator order) and allocates it in the arena.
bool KNCustomizedOp::build_from_plan(std::string *error, int *status) {
  auto fail = [&](int st, std::string const &msg) {
    if (error) *error = msg;
    if (status) *status = st;
    return false;
  };
  size_t n = input_tensors.size();
  if (n != plan.input_map.size() || n != plan.forloop_dim.size() || n != plan.input_smem_layouts.size())
    return fail(MG_ERR_INVALID_GRAPH, "plan lists a different number of inputs than were given");
  for (size_t i = 0; i < n; i++) {
    auto *op = bgraph.create_input_op(input_tensors[i], plan.input_map[i], plan.forloop_dim[i],
                                      plan.input_smem_layouts[i]);
    if (!op) return fail(MG_ERR_INVALID_GRAPH, "input " + std::to_string(i) + ": tile shape invalid or shared memory exhausted");
    bgraph.operators.push_back(op);
  }
  for (auto const &entry : plan.ops) {
    std::vector<STensor> ins;
    for (auto const &src : entry.second) {
      if (src.first < 0 || src.first >= (int)bgraph.operators.size() || src.second < 0 ||
          src.second >= (int)bgraph.operators[src.first]->output_tensors.size())
        return fail(MG_ERR_INVALID_GRAPH, "operand refers to an operator that does not exist yet");
      ins.push_back(bgraph.operators[src.first]->output_tensors[src.second]);
    }
    threadblock::TBOperator *op = nullptr;
    TBOperatorType t = entry.first;
    size_t want = (t == TB_EXP_OP || (t >= TB_REDUCTION_0_OP && t <= TB_REDUCTION_2_TO_DIMX_OP)) ? 1 : 2;
    if (ins.size() != want) return fail(MG_ERR_INVALID_GRAPH, "wrong operand count for " + std::string(to_string(t)));
    if (t == TB_MATMUL_OP) op = bgraph.create_matmul_op(ins[0], ins[1]);
    else if (t == TB_EXP_OP) op = bgraph.create_elementunary_op(ins[0], t);
    else if (t == TB_ADD_OP || t == TB_MUL_OP || t == TB_DIV_OP) op = bgraph.create_elementbinary_op(ins[0], ins[1], t);
    else if (t >= TB_REDUCTION_0_OP && t <= TB_REDUCTION_2_OP) op = bgraph.create_reduction_op(ins[0], t - TB_REDUCTION_0_OP);
    else if (t >= TB_REDUCTION_0_TO_DIMX_OP && t <= TB_REDUCTION_2_TO_DIMX_OP)
      op = bgraph.create_reduction_to_dimx_op(ins[0], t - TB_REDUCTION_0_TO_DIMX_OP);
    else if (t >= TB_CONCAT_0_OP && t <= TB_CONCAT_2_OP) op = bgraph.create_concat_op(ins[0], ins[1], t - TB_CONCAT_0_OP);
    else return fail(MG_ERR_INVALID_GRAPH, "unsupported threadblock operator type " + std::to_string((int)t));
    if (!op) return fail(MG_ERR_INVALID_GRAPH, std::string(to_string(t)) + ": shapes do not fit or shared memory exhausted");
    bgraph.operators.push_back(op);
  }
  // outputs
  size_t num_ops = bgraph.operators.size();
  std::vector<STensor> results;
  for (size_t i = 0; i < num_ops; i++) {
    threadblock::TBOperator const *op = bgraph.operators[i];
    if (op->op_type == TB_INPUT_OP) continue;
    for (STensor const &t : op->output_tensors) {
      bool consumed = false;
      for (size_t j = i + 1; j < num_ops && !consumed; j++)
        for (STensor const &u : bgraph.operators[j]->input_tensors)
          if (u == t) consumed = true;
      if (!consumed) results.push_back(t);
    }
  }
  DeviceMemoryManager *dmm = DeviceMemoryManager::get_instance();
  for (STensor const &t : results) {
    auto *op = bgraph.create_output_op(t, plan.output_map);
    if (!op) return fail(MG_ERR_INVALID_GRAPH, "output tile does not fit in shared memory or output_map is out of range");
    bgraph.operators.push_back(op);
    auto *out = static_cast<threadblock::TBOutputOp *>(op);
    DTensor dt = out->dtensor;
    dt.owner_op = this;
    dt.owner_ts_idx = (int)output_tensors.size();
    dt.guid = (size_t)DTensor::next_guid++;
    if (!dmm->allocate(dt)) return fail(MG_ERR_OUT_OF_MEMORY, "device arena exhausted while allocating outputs");
    out->dtensor = dt;
    output_tensors.push_back(dt);
  }
  return true;
}

// Replays a template graph (the form the search produces) and re-derives the plan from it.
KNCustomizedOp::KNCustomizedOp(std::vector<DTensor> const &ins, threadblock::Graph const &g)
    : KNOperator(KN_CUSTOMIZED_OP, ins), bgraph(g.grid_dim, g.block_dim, g.forloop_range, g.reduction_dimx) {
  bgraph.max_smem = DeviceMemoryManager::get_instance()->max_smem;
  plan.grid_dim = g.grid_dim;
  plan.block_dim = g.block_dim;
  plan.forloop_range = g.forloop_range;
  plan.reduction_dimx = g.reduction_dimx;
  plan.output_map = {-1, -1, -1};
  DeviceMemoryManager *dmm = DeviceMemoryManager::get_instance();
  size_t next_input = 0;
  for (threadblock::TBOperator *src : g.operators) {
    std::vector<STensor> my_inputs;
    std::vector<std::pair<int, int>> where;
    for (STensor const &t : src->input_tensors) {
      int op_idx = -1;
      for (size_t l = 0; l < g.operators.size(); l++)
        if (g.operators[l] == t.owner_op) op_idx = (int)l;
      assert(op_idx >= 0 && op_idx < (int)bgraph.operators.size());
      my_inputs.push_back(bgraph.operators[op_idx]->output_tensors[t.owner_ts_idx]);
      where.push_back({op_idx, t.owner_ts_idx});
    }
    TBOperatorType t = src->op_type;
    if (t != TB_INPUT_OP && t != TB_OUTPUT_OP) plan.ops.push_back({t, where});
    if (t == TB_INPUT_OP) {
      auto *in = static_cast<threadblock::TBInputOp *>(src);
      // the template's own tensor descriptor gives the shape; the storage is the one passed in
      DTensor dt = next_input < ins.size() ? ins[next_input] : in->dtensor;
      next_input++;
      bgraph.new_input(dt, in->input_map, in->forloop_dim, in->output_tensors[0].layout);
      plan.input_map.push_back(in->input_map);
      plan.forloop_dim.push_back(in->forloop_dim);
      plan.input_smem_layouts.push_back(in->output_tensors[0].layout);
    } else if (t == TB_OUTPUT_OP) {
      auto *out = static_cast<threadblock::TBOutputOp *>(src);
      DTensor dt = bgraph.new_output(my_inputs[0], out->output_map);
      dt.owner_op = this;
      dt.owner_ts_idx = (int)output_tensors.size();
      dt.guid = (size_t)DTensor::next_guid++;
      bool ok = dmm->allocate(dt);
      assert(ok && "device arena exhausted");
      (void)ok;
      static_cast<threadblock::TBOutputOp *>(bgraph.operators.back())->dtensor = dt;
      output_tensors.push_back(dt);
      plan.output_map = out->output_map;
    } else if (t == TB_MATMUL_OP) bgraph.matmul(my_inputs[0], my_inputs[1]);
    else if (t == TB_EXP_OP) bgraph.exp(my_inputs[0]);
    else if (t == TB_ADD_OP) bgraph.add(my_inputs[0], my_inputs[1]);
    else if (t == TB_MUL_OP) bgraph.mul(my_inputs[0], my_inputs[1]);
    else if (t == TB_DIV_OP) bgraph.div(my_inputs[0], my_inputs[1]);
    else if (t >= TB_REDUCTION_0_OP && t <= TB_REDUCTION_2_OP) bgraph.reduction(my_inputs[0], t - TB_REDUCTION_0_OP);
    else if (t >= TB_REDUCTION_0_TO_DIMX_OP && t <= TB_REDUCTION_2_TO_DIMX_OP)
      bgraph.reduction_to_dimx(my_inputs[0], t - TB_REDUCTION_0_TO_DIMX_OP);
    else if (t >= TB_CONCAT_0_OP && t <= TB_CONCAT_2_OP) bgraph.concat(my_inputs[0], my_inputs[1], t - TB_CONCAT_0_OP);
    else assert(false && "unsupported threadblock operator");
  }
  after_build();
}

KNCustomizedOp::~KNCustomizedOp() {
  while (!bgraph.operators.empty()) {
    delete bgraph.operators.back();
    bgraph.operators.pop_back();
  }
  if (tickets_) DeviceMemoryManager::get_instance()->free_raw(tickets_);
  free_outputs(output_tensors);
}

bool KNCustomizedOp::ensure_lowered() {
  if (lowered_) return true;
  char const *why = nullptr;
  if (!bgraph.lower(program_, &why)) {
    mg::set_error(std::string("cannot lower threadblock graph: ") + (why ? why : "?"));
    return false;
  }
  lowered_ = true;
  kernel_fp_ = kernel_float_ = mg::KERNEL_INTERPRETER;
  o_output_ = o_input_ = 0;
  if (DeviceMemoryManager::get_instance()->specialise > 0) {
    mgd_attn_split sp;
    mgd_attn_merge mp;
    int h, r, d;
    if (mg::match_attn_split(program_, &sp, &o_output_)) {
      sp.data_type = (int)input_tensors[0].data_type;
      sp.causal_window = causal_window;
      if (mgd_attn_split_supported(&sp, 1)) kernel_fp_ = mg::KERNEL_ATTN_SPLIT;
      if (mgd_attn_split_supported(&sp, 0)) kernel_float_ = mg::KERNEL_ATTN_SPLIT;
    } else if (mgd_attn_rows rp; mg::match_attn_rows(program_, &rp, &o_output_)) {
      rp.data_type = (int)input_tensors[0].data_type;
      if (causal_window == 0 && mgd_attn_rows_supported(&rp)) kernel_float_ = mg::KERNEL_ATTN_ROWS;
    } else if (mgd_matmul_chain mc; mg::match_matmul_chain(program_, &mc)) {
      mc.data_type = (int)input_tensors[0].data_type;
      if (mgd_matmul_chain_supported(&mc, 1)) kernel_fp_ = mg::KERNEL_MATMUL_CHAIN;
      if (mgd_matmul_chain_supported(&mc, 0)) kernel_float_ = mg::KERNEL_MATMUL_CHAIN;
    } else if (mgd_tile_reduce tr; mg::match_tile_reduce(program_, &tr)) {
      tr.data_type = (int)input_tensors[0].data_type;
      if (mgd_tile_reduce_supported(&tr, 1)) kernel_fp_ = mg::KERNEL_TILE_REDUCE;
      if (mgd_tile_reduce_supported(&tr, 0)) kernel_float_ = mg::KERNEL_TILE_REDUCE;
    } else if (mg::match_attn_merge(program_, &mp, &o_input_)) {
      mp.data_type = (int)input_tensors[0].data_type;
      if (mgd_attn_merge_supported(&mp, 1)) kernel_fp_ = mg::KERNEL_ATTN_MERGE;
      if (mgd_attn_merge_supported(&mp, 0)) kernel_float_ = mg::KERNEL_ATTN_MERGE;
    } else {
      mg::match_div_rows(program_, &h, &r, &d, &o_input_); // only consulted by can_fuse_with of the producer
    }
  }
  return true;
}

int KNCustomizedOp::selected_kernel(bool fp) {
  if (!ensure_lowered()) return -1;
  return fp ? kernel_fp_ : kernel_float_;
}

static int finish(int st) {
  if (st != MG_OK) mg::set_error(mgd_last_error());
  return st;
}

int KNCustomizedOp::launch_fingerprint_sets(int num_sets, void const *const *in, long long const *in_stride,
                                            void *const *out, long long const *out_stride, void *stream) {
  return launch_sets(true, num_sets, in, in_stride, out, out_stride, stream);
}
int KNCustomizedOp::launch_float_sets(int num_sets, void const *const *in, long long const *in_stride,
                                      void *const *out, long long const *out_stride, void *stream) {
  return launch_sets(false, num_sets, in, in_stride, out, out_stride, stream);
}

// One launch of this operator over `num_sets` independent tensor sets, on whichever kernel was selected.
int KNCustomizedOp::launch_sets(bool fp, int num_sets, void const *const *in, long long const *in_stride,
                                void *const *out, long long const *out_stride, void *stream) {
  if (int dry_st = refuse_if_dry()) return dry_st;
  if (!ensure_lowered()) return MG_ERR_INVALID_GRAPH;
  if (num_sets <= 0) return MG_ERR_INVALID_ARGUMENT;
  int const kernel = fp ? kernel_fp_ : kernel_float_;
  int const dt = input_tensors.empty() ? (int)DT_FLOAT16 : (int)input_tensors[0].data_type;
  if (kernel == mg::KERNEL_ATTN_SPLIT) {
    void *o[2] = {out[o_output_], out[1 - o_output_]};
    long long os[2] = {out_stride[o_output_], out_stride[1 - o_output_]};
    return launch_split(fp, num_sets, in, in_stride, o, os, nullptr, stream);
  }
  if (kernel == mg::KERNEL_ATTN_ROWS) {
    if (num_sets != 1) {
      mg::set_error("the dense attention kernel takes one tensor set per launch");
      return MG_ERR_UNSUPPORTED;
    }
    mgd_attn_rows rp;
    mg::match_attn_rows(program_, &rp, nullptr);
    rp.data_type = dt;
    return launch_rows(&rp, in, out[o_output_], out[1 - o_output_], nullptr, stream);
  }
  if (kernel == mg::KERNEL_ATTN_MERGE) {
    mgd_attn_merge mp;
    mg::match_attn_merge(program_, &mp, nullptr);
    // the merge kernel writes its one output and nothing else
    record_outputs(stream, {range_of(out[0], ((size_t)(num_sets - 1) * (size_t)out_stride[0] + output_tensors[0].num_elements()) * 2)});
    mp.num_sets = num_sets;
    mp.data_type = dt;
    mp.o_part_set_stride = in_stride[o_input_]; mp.r_part_set_stride = in_stride[1 - o_input_]; mp.out_set_stride = out_stride[0];
    if (fp)
      return finish(mgd_launch_attn_merge_fingerprint(&mp, (uint16_t const *)in[o_input_], (uint16_t const *)in[1 - o_input_],
                                                      (uint16_t *)out[0], stream));
    return finish(mgd_launch_attn_merge_float(&mp, in[o_input_], in[1 - o_input_], out[0], stream));
  }
  if (!fp && causal_window != 0) {
    mg::set_error("the causal window is implemented by the split-KV attention kernel only");
    return MG_ERR_UNSUPPORTED;
  }
  record_anything(stream);
  mgd_bindings b;
  std::memset(&b, 0, sizeof(b));
  for (int i = 0; i < program_.num_inputs; i++) { b.in[i] = in[i]; b.in_set_stride[i] = in_stride[i]; }
  for (int i = 0; i < program_.num_outputs; i++) { b.out[i] = out[i]; b.out_set_stride[i] = out_stride[i]; }
  b.num_sets = num_sets;
  if (kernel == mg::KERNEL_TILE_REDUCE) {
    mgd_tile_reduce tr;
    mg::match_tile_reduce(program_, &tr);
    tr.data_type = dt;
    return finish(mgd_launch_tile_reduce(&tr, &b, fp ? 1 : 0, stream));
  }
  if (kernel == mg::KERNEL_MATMUL_CHAIN) {
    mgd_matmul_chain mc;
    mg::match_matmul_chain(program_, &mc);
    mc.data_type = dt;
    return finish(fp ? mgd_launch_matmul_chain_fingerprint(&mc, &b, stream) : mgd_launch_matmul_chain_float(&mc, &b, stream));
  }
  return finish(fp ? mgd_launch_fingerprint_interp(&program_, &b, stream) : mgd_launch_float_interp(&program_, &b, dt, stream));
}

int KNCustomizedOp::launch_fingerprint(void *stream) {
  void const *in[MGD_MAX_IO];
  void *out[MGD_MAX_IO];
  long long zs[MGD_MAX_IO] = {0};
  if (input_tensors.size() > MGD_MAX_IO || output_tensors.size() > MGD_MAX_IO) return MG_ERR_UNSUPPORTED;
  for (size_t i = 0; i < input_tensors.size(); i++) in[i] = input_tensors[i].fp_ptr;
  for (size_t i = 0; i < output_tensors.size(); i++) out[i] = output_tensors[i].fp_ptr;
  return launch_sets(true, 1, in, zs, out, zs, stream);
}

int KNCustomizedOp::launch_float(void *stream) {
  void const *in[MGD_MAX_IO];
  void *out[MGD_MAX_IO];
  long long zs[MGD_MAX_IO] = {0};
  if (input_tensors.size() > MGD_MAX_IO || output_tensors.size() > MGD_MAX_IO) return MG_ERR_UNSUPPORTED;
  for (size_t i = 0; i < input_tensors.size(); i++) in[i] = input_tensors[i].data_ptr;
  for (size_t i = 0; i < output_tensors.size(); i++) out[i] = output_tensors[i].data_ptr;
  return launch_sets(false, 1, in, zs, out, zs, stream);
}

// One launch of the split-KV attention kernel (out[0] = O', out[1] = R'); with `merge` the cross-split merge
// operator rides along.
int KNCustomizedOp::launch_split(bool fp, int num_sets, void const *const *in, long long const *in_stride,
                                 void *const *out, long long const *out_stride, FusedMerge const *merge, void *stream) {
  mgd_attn_split sp;
  mg::match_attn_split(program_, &sp, nullptr);
  sp.num_sets = num_sets;
  sp.q_set_stride = in_stride[0]; sp.k_set_stride = in_stride[1]; sp.v_set_stride = in_stride[2];
  sp.o_set_stride = out_stride[0]; sp.r_set_stride = out_stride[1];
  sp.data_type = (int)input_tensors[0].data_type;
  sp.causal_window = fp ? 0 : causal_window;
  mgd_attn_launch_opts opts;
  std::memset(&opts, 0, sizeof(opts));
  size_t elem = 2;
  std::vector<Range> ins, outs;
  for (int i = 0; i < 3; i++)
    ins.push_back(range_of(in[i], ((size_t)(num_sets - 1) * (size_t)in_stride[i] + input_tensors[i].num_elements()) * elem));
  for (int i = 0; i < 2; i++) { // out[0] = O', out[1] = R': output_tensors[o_output_] and the other one
    DTensor const &t = output_tensors[i == 0 ? o_output_ : 1 - o_output_];
    outs.push_back(range_of(out[i], ((size_t)(num_sets - 1) * (size_t)out_stride[i] + t.num_elements()) * elem));
  }
  if (merge != nullptr) {
    opts.merged_out = merge->out;
    opts.tickets = merge->tickets;
    opts.merged_set_stride = merge->set_stride;
    outs.push_back(range_of(merge->out, merge->bytes));
  }
  int32_t serial = 0;
  mgd_get_option(MGD_OPT_ATTN_DEPENDENT_LAUNCH, &serial); // 1 = plain stream order (no programmatic dependent launch)
  opts.overlap = (serial == 1 ? 0 : 1) | (inputs_untouched(stream, ins) && serial != 1 ? 2 : 0) | (DeviceMemoryManager::get_instance()->launch_policy == 1 ? 4 : 0) |
                 (merge != nullptr && merge->partials_are_scratch ? 8 : 0);
  int st = fp ? mgd_launch_attn_split_fingerprint_ex(&sp, (uint16_t const *)in[0], (uint16_t const *)in[1],
                                                     (uint16_t const *)in[2], (uint16_t *)out[0], (uint16_t *)out[1],
                                                     &opts, stream)
              : mgd_launch_attn_split_float_ex(&sp, in[0], in[1], in[2], out[0], out[1], &opts, stream);
  if (st == MG_OK) record_outputs(stream, outs);
  else record_anything(stream);
  return finish(st);
}

// Dense attention launch (with the division that follows fused in when `o_div` is given).  Like the split-KV launch
// it lets the next kernel of the stream start while it drains, and reads its inputs early when the library knows that
// the kernel in front of it did not write them.
int KNCustomizedOp::launch_rows(mgd_attn_rows const *rp, void const *const *in, void *o_acc, void *r_acc, void *o_div,
                                void *stream) {
  size_t const q_bytes = (size_t)rp->heads * rp->seq_q * rp->d * 2, kv_bytes = (size_t)rp->heads * rp->kv_len * rp->d * 2;
  std::vector<Range> ins = {range_of(in[0], q_bytes), range_of(in[1], kv_bytes), range_of(in[2], kv_bytes)};
  std::vector<Range> outs = {range_of(o_acc, q_bytes), range_of(r_acc, (size_t)rp->heads * rp->seq_q * 2)};
  if (o_div) outs.push_back(range_of(o_div, q_bytes));
  int32_t serial = 0;
  mgd_get_option(MGD_OPT_ATTN_DEPENDENT_LAUNCH, &serial); // 1 = plain stream order (no programmatic dependent launch)
  int32_t const overlap = serial == 1 ? 0 : (1 | (inputs_untouched(stream, ins) ? 2 : 0));
  int const st = mgd_launch_attn_rows_float_overlapped(rp, in[0], in[1], in[2], o_acc, r_acc, o_div, overlap, stream);
  if (st == MG_OK) record_outputs(stream, outs);
  else record_anything(stream);
  return finish(st);
}

bool KNCustomizedOp::can_fuse_with(KNOperator *next, bool fp) {
  if (DeviceMemoryManager::get_instance()->specialise < 2 || !next) return false;
  if (next->op_type != KN_CUSTOMIZED_OP || !ensure_lowered()) return false;
  auto *m = static_cast<KNCustomizedOp *>(next);
  if (!m->ensure_lowered()) return false;
  int mine = fp ? kernel_fp_ : kernel_float_;
  if (mine == mg::KERNEL_ATTN_ROWS) {
    // dense attention followed by the division of its two outputs
    int h, r, d;
    mgd_attn_rows rp;
    if (fp || !mg::match_div_rows(m->program_, &h, &r, &d, nullptr) || !mg::match_attn_rows(program_, &rp, nullptr)) return false;
    if (h != rp.heads || r != rp.seq_q || d != rp.d) return false;
  } else {
    if (mine != mg::KERNEL_ATTN_SPLIT || !tickets_) return false;
    if ((fp ? m->kernel_fp_ : m->kernel_float_) != mg::KERNEL_ATTN_MERGE) return false;
  }
  if (m->input_tensors.size() != 2 || output_tensors.size() != 2) return false;
  for (int i = 0; i < 2; i++) { // i = 0: the attention result, i = 1: the row sums
    DTensor const &a = output_tensors[i == 0 ? o_output_ : 1 - o_output_];
    DTensor const &b = m->input_tensors[i == 0 ? m->o_input_ : 1 - m->o_input_];
    if (a.data_ptr != b.data_ptr || a.fp_ptr != b.fp_ptr || a.num_elements() != b.num_elements()) return false;
  }
  return true;
}

int KNCustomizedOp::launch_fused(KNCustomizedOp *merge, bool fp, void *stream) {
  void const *in[3];
  void *out[2];
  long long zs[3] = {0, 0, 0};
  for (int i = 0; i < 3; i++) in[i] = fp ? (void const *)input_tensors[i].fp_ptr : input_tensors[i].data_ptr;
  for (int i = 0; i < 2; i++) out[i] = fp ? (void *)output_tensors[i].fp_ptr : output_tensors[i].data_ptr;
  DTensor const &o = merge->output_tensors[0];
  return launch_fused_sets(merge, fp, 1, in, zs, out, zs, fp ? (void *)o.fp_ptr : o.data_ptr, 0, tickets_, stream);
}

int KNCustomizedOp::launch_fused_sets(KNCustomizedOp *merge, bool fp, int num_sets, void const *const *in,
                                      long long const *in_stride, void *const *out, long long const *out_stride,
                                      void *merged_out, long long merged_stride, int *tickets, void *stream,
                                      bool partials_are_scratch) {
  if (int dry_st = refuse_if_dry()) return dry_st;
  if (!fp && kernel_float_ == mg::KERNEL_ATTN_ROWS) {
    if (num_sets != 1) {
      mg::set_error("the dense attention kernel takes one tensor set per launch");
      return MG_ERR_UNSUPPORTED;
    }
    mgd_attn_rows rp;
    mg::match_attn_rows(program_, &rp, nullptr);
    rp.data_type = (int)input_tensors[0].data_type;
    return launch_rows(&rp, in, out[o_output_], out[1 - o_output_], merged_out, stream);
  }
  void *o[2] = {out[o_output_], out[1 - o_output_]};
  long long os[2] = {out_stride[o_output_], out_stride[1 - o_output_]};
  FusedMerge fm{merged_out, merged_stride,
                ((size_t)(num_sets - 1) * (size_t)merged_stride + merge->output_tensors[0].num_elements()) * 2, tickets,
                partials_are_scratch};
  return launch_split(fp, num_sets, in, in_stride, o, os, &fm, stream);
}

bool KNCustomizedOp::fingerprint(void) { return sync_ok(launch_fingerprint(nullptr)); }
void KNCustomizedOp::run(void) {
  int st = launch_float(nullptr);
  if (st != MG_OK) std::fprintf(stderr, "KNCustomizedOp::run: %s\n", mg::last_error());
}
bool KNCustomizedOp::profile(ProfileResult &result) {
  return profile_with_events(result, ProfileResult::NUM_WARPUP_ITERATIONS, ProfileResult::NUM_ITERATIONS);
}

// ---- Graph ---------------------------------------------------------------------------------------
Graph::Graph(void) : owners_(std::make_shared<int>(0)) {}
Graph::Graph(Graph const &other) : operators(other.operators), owners_(other.owners_) {}
Graph &Graph::operator=(Graph const &other) {
  if (this != &other) {
    drop();
    operators = other.operators;
    owners_ = other.owners_;
  }
  return *this;
}
Graph::~Graph() { drop(); }
void Graph::release() { owners_.reset(); }
// Gives up this copy's share; the last copy deletes the operators in its list, newest first.
void Graph::drop() {
  bool const last = owners_ && owners_.use_count() == 1;
  owners_.reset();
  if (last)
    while (!operators.empty()) {
      delete operators.back();
      operators.pop_back();
    }
  operators.clear();
}

static bool fits_arena(DTensor const &t) {
  return DeviceMemoryManager::get_instance()->can_allocate(t.data_size(), t.fingerprint_size());
}

KNOperator *Graph::create_input_op(std::vector<int> const &dims, DataType dt, mirage::layout::DmemLayout lay) {
  if (dims.empty() || dims.size() > MAX_TENSOR_DIMS) return nullptr;
  DTensor t;
  t.num_dims = (int)dims.size();
  for (int i = 0; i < t.num_dims; i++) {
    if (dims[i] <= 0) return nullptr;
    t.dim[i] = dims[i];
  }
  t.data_type = dt;
  if (dt != DT_FLOAT16 && dt != DT_BFLOAT16 && dt != DT_FLOAT32) return nullptr;
  if (!fits_arena(t)) return nullptr;
  return new KNInputOp(dims, dt, lay);
}
DTensor Graph::new_input(std::vector<int> const &dims, DataType dt, mirage::layout::DmemLayout lay) {
  KNOperator *op = create_input_op(dims, dt, lay);
  assert(op != nullptr);
  operators.push_back(op);
  return op->output_tensors[0];
}
DTensor *Graph::new_input_ptr(std::vector<int> const &dims, DataType dt, mirage::layout::DmemLayout lay) {
  KNOperator *op = create_input_op(dims, dt, lay);
  assert(op != nullptr);
  operators.push_back(op);
  return &op->output_tensors[0];
}

KNOperator *Graph::create_matmul_op(DTensor const &A, DTensor const &B) {
  if (A.num_dims != B.num_dims || A.num_dims < 2) return nullptr;
  if (A.dim[A.num_dims - 1] != B.dim[B.num_dims - 2]) return nullptr;
  for (int i = 0; i < A.num_dims - 2; i++)
    if (A.dim[i] != B.dim[i]) return nullptr;
  DTensor C = A;
  C.dim[C.num_dims - 1] = B.dim[B.num_dims - 1];
  if (!fits_arena(C)) return nullptr;
  return new KNMatmulOp(A, B);
}
KNOperator *Graph::create_elementunary_op(DTensor const &A, KNOperatorType t) {
  if (t != KN_EXP_OP || !fits_arena(A)) return nullptr;
  return new KNElementUnaryOp(A, t);
}
KNOperator *Graph::create_elementbinary_op(DTensor const &A, DTensor const &B, KNOperatorType t) {
  if (A.num_dims != B.num_dims) return nullptr;
  if (t != KN_ADD_OP && t != KN_MUL_OP && t != KN_DIV_OP) return nullptr;
  DTensor C = A;
  for (int i = 0; i < A.num_dims; i++) {
    if (A.dim[i] != B.dim[i] && A.dim[i] > 1 && B.dim[i] > 1) return nullptr;
    C.dim[i] = std::max(A.dim[i], B.dim[i]);
  }
  if (!fits_arena(C)) return nullptr;
  return new KNElementBinaryOp(A, B, t);
}
KNOperator *Graph::create_reduction_op(DTensor const &A, int dim, int size) {
  if (dim < 0 || dim > 2 || A.num_dims <= dim || size <= 0 || A.dim[dim] % size != 0) return nullptr;
  if (!fits_arena(A)) return nullptr;
  return new KNReductionOp(A, dim, size);
}

#define MG_PUSH_RETURN(opexpr)            \
  KNOperator *op = (opexpr);              \
  assert(op != nullptr);                  \
  operators.push_back(op);
DTensor Graph::matmul(DTensor const &A, DTensor const &B) { MG_PUSH_RETURN(create_matmul_op(A, B)) return op->output_tensors[0]; }
DTensor *Graph::matmul(DTensor const *A, DTensor const *B) { MG_PUSH_RETURN(create_matmul_op(*A, *B)) return &op->output_tensors[0]; }
DTensor Graph::exp(DTensor const &A) { MG_PUSH_RETURN(create_elementunary_op(A, KN_EXP_OP)) return op->output_tensors[0]; }
DTensor *Graph::exp(DTensor const *A) { MG_PUSH_RETURN(create_elementunary_op(*A, KN_EXP_OP)) return &op->output_tensors[0]; }
DTensor Graph::add(DTensor const &a, DTensor const &b) { MG_PUSH_RETURN(create_elementbinary_op(a, b, KN_ADD_OP)) return op->output_tensors[0]; }
DTensor Graph::mul(DTensor const &a, DTensor const &b) { MG_PUSH_RETURN(create_elementbinary_op(a, b, KN_MUL_OP)) return op->output_tensors[0]; }
DTensor Graph::div(DTensor const &a, DTensor const &b) { MG_PUSH_RETURN(create_elementbinary_op(a, b, KN_DIV_OP)) return op->output_tensors[0]; }
DTensor *Graph::add(DTensor const *a, DTensor const *b) { MG_PUSH_RETURN(create_elementbinary_op(*a, *b, KN_ADD_OP)) return &op->output_tensors[0]; }
DTensor *Graph::mul(DTensor const *a, DTensor const *b) { MG_PUSH_RETURN(create_elementbinary_op(*a, *b, KN_MUL_OP)) return &op->output_tensors[0]; }
DTensor *Graph::div(DTensor const *a, DTensor const *b) { MG_PUSH_RETURN(create_elementbinary_op(*a, *b, KN_DIV_OP)) return &op->output_tensors[0]; }
DTensor Graph::reduction(DTensor const &A, int dim, int size) { MG_PUSH_RETURN(create_reduction_op(A, dim, size)) return op->output_tensors[0]; }
DTensor *Graph::reduction(DTensor const *A, int dim, int size) { MG_PUSH_RETURN(create_reduction_op(*A, dim, size)) return &op->output_tensors[0]; }
#undef MG_PUSH_RETURN

KNOperator *Graph::create_customized_op(std::vector<DTensor> const &ins, ExecutionPlan const &plan) {
  std::string err;
  int st = MG_OK;
  KNCustomizedOp *op = KNCustomizedOp::create(ins, plan, &err, &st);
  if (!op) mg::set_error(err);
  return op;
}
std::vector<DTensor> Graph::customized(std::vector<DTensor> const &ins, ExecutionPlan const &plan) {
  KNOperator *op = create_customized_op(ins, plan);
  if (!op) std::fprintf(stderr, "Graph::customized: %s\n", mg::last_error());
  assert(op != nullptr);
  operators.push_back(op);
  return op->output_tensors;
}
KNOperator *Graph::create_customized_op(std::vector<DTensor> const &ins, threadblock::Graph const &g) {
  size_t bytes = 0;
  for (threadblock::TBOperator *op : g.operators)
    if (op->op_type == TB_OUTPUT_OP) {
      DTensor const &t = static_cast<threadblock::TBOutputOp *>(op)->dtensor;
      bytes += ((t.data_size() + 255) / 256 + (t.fingerprint_size() + 255) / 256) * 256;
    }
  DeviceMemoryManager *dmm = DeviceMemoryManager::get_instance();
  if ((size_t)dmm->offset + bytes > dmm->total_size) return nullptr;
  return new KNCustomizedOp(ins, g);
}
std::vector<DTensor> Graph::customized(std::vector<DTensor> const &ins, threadblock::Graph const &g) {
  KNOperator *op = create_customized_op(ins, g);
  assert(op != nullptr);
  operators.push_back(op);
  return op->output_tensors;
}

} // namespace kernel
} // namespace mirage

namespace std {
size_t hash<mirage::kernel::DTensor>::operator()(mirage::kernel::DTensor const &t) const {
  size_t h = std::hash<int>()((int)t.data_type) * 31 + std::hash<int>()((int)t.layout);
  for (int i = 0; i < t.num_dims; i++) h = h * 1000003u + (size_t)t.dim[i];
  return h * 31 + std::hash<void *>()((void *)t.owner_op) + (size_t)t.owner_ts_idx;
}
size_t hash<mirage::threadblock::STensor>::operator()(mirage::threadblock::STensor const &t) const {
  size_t h = std::hash<int>()((int)t.data_type) * 31 + std::hash<int>()((int)t.layout);
  for (int i = 0; i < t.num_dims; i++) h = h * 1000003u + (size_t)t.dim[i];
  return h * 31 + std::hash<void *>()((void *)t.owner_op) + (size_t)t.owner_ts_idx * 7 + (size_t)t.smem_offset;
}
} // namespace std
