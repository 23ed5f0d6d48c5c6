/* mugraph.h - graph-level C ABI of the B200 muGraph executor.
 *
 * This is the boundary a foreign-language binding links against (ctypes,
 * Cython, cgo ...).  Every entry point is `extern "C"`, takes plain pointers
 * and sizes, returns an int status (0 = MG_OK) and never terminates the
 * process; `mg_last_error()` gives the message of the calling thread's last
 * failure.  The C++ facade in include/mirage/ (same class names as the
 * reference) sits on the same implementation.
 *
 * Each entry names the reference interface it stands in for (paths relative
 * to the reference project root).
 */
#ifndef MUGRAPH_H_
#define MUGRAPH_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes -------------------------------------------------------- */
enum {
  MG_OK = 0,
  MG_ERR_INVALID_ARGUMENT = 1,
  MG_ERR_INVALID_GRAPH = 2,   /* where the reference's create_*_op returns nullptr or asserts */
  MG_ERR_OUT_OF_MEMORY = 3,   /* device arena exhausted (reference: nullptr, customized.cc:56-59) */
  MG_ERR_CUDA = 4,            /* a CUDA runtime/driver call failed (reference: FatalError + exit) */
  MG_ERR_UNSUPPORTED = 5,     /* graph is valid but no kernel of this library can run it */
  MG_ERR_DEVICE_TIMEOUT = 6,  /* a bounded device-side wait gave up; the context stays usable */
  MG_ERR_NO_DEVICE = 7        /* no CUDA device / driver present */
};

/* ---- numeric codes: identical to the reference enums --------------------- */
/* include/mirage/type.h:38-46 (DataType), :79-103 (TBOperatorType), :50-62 (KNOperatorType),
 * include/mirage/layout.h:22-45 */
enum { MG_DT_BFLOAT16 = 920, MG_DT_FLOAT16 = 921, MG_DT_FLOAT32 = 930 };
enum { MG_DMEM_ROW_MAJOR = 100, MG_DMEM_COLUMN_MAJOR = 101 };
enum { MG_SMEM_ROW_MAJOR = 200, MG_SMEM_COLUMN_MAJOR = 201 };
enum {
  MG_TB_MATMUL_OP = 2003, MG_TB_EXP_OP = 2007, MG_TB_ADD_OP = 2008, MG_TB_MUL_OP = 2009, MG_TB_DIV_OP = 2010,
  MG_TB_REDUCTION_0_OP = 2101, MG_TB_REDUCTION_1_OP = 2102, MG_TB_REDUCTION_2_OP = 2103,
  MG_TB_REDUCTION_0_TO_DIMX_OP = 2104, MG_TB_REDUCTION_1_TO_DIMX_OP = 2105, MG_TB_REDUCTION_2_TO_DIMX_OP = 2106,
  MG_TB_CONCAT_0_OP = 2200, MG_TB_CONCAT_1_OP = 2201, MG_TB_CONCAT_2_OP = 2202
};
enum {
  MG_KN_INPUT_OP = 1001, MG_KN_MATMUL_OP = 1003, MG_KN_REDUCTION_0_OP = 1004, MG_KN_REDUCTION_1_OP = 1005,
  MG_KN_REDUCTION_2_OP = 1006, MG_KN_EXP_OP = 1007, MG_KN_ADD_OP = 1008, MG_KN_MUL_OP = 1009,
  MG_KN_DIV_OP = 1010, MG_KN_CUSTOMIZED_OP = 1999
};

/* finite-field constants, include/mirage/type.h:26-34 */
#define MG_FP_P 227
#define MG_FP_Q 113
#define MG_FP_PQ 25651
#define MG_FP_EXP_BASE 3
#define MG_FP_Q_MUL_P_MOD_1 25425
#define MG_FP_P_MUL_Q_MOD_1 227

#define MG_MAX_TENSOR_DIMS 4

/* Device tensor descriptor; the fields of kernel::DTensor
 * (include/mirage/kernel/device_tensor.h:31-124) a binding needs. */
typedef struct mg_tensor {
  int32_t data_type;
  int32_t layout;
  int32_t num_dims;
  int32_t dim[MG_MAX_TENSOR_DIMS];
  int32_t owner_op;      /* index of the producing operator in its graph */
  int32_t owner_ts_idx;
  void *data_ptr;        /* device pointer, 16-bit float storage */
  uint16_t *fp_ptr;      /* device pointer, uint16 fingerprints */
} mg_tensor;

/* threadblock::ExecutionPlan, include/mirage/threadblock/graph.h:28-42, flattened.
 * op_srcs holds (operator index, output index) pairs for all ops back to back;
 * operator indices count the plan's inputs first, as in the reference. */
typedef struct mg_plan {
  int32_t num_ops;
  const int32_t *op_types;          /* [num_ops]          MG_TB_* */
  const int32_t *op_num_srcs;       /* [num_ops] */
  const int32_t *op_srcs;           /* [2 * sum(op_num_srcs)] */
  int32_t num_inputs;
  const int32_t *input_map;         /* [3 * num_inputs]   tensor dim split by grid x,y,z; -1 = replicate */
  const int32_t *forloop_dim;       /* [num_inputs]       tensor dim tiled by the for-loop; -1 = none */
  const int32_t *input_smem_layouts;/* [num_inputs]       MG_SMEM_* (kept for drop-in; no effect on results) */
  int32_t output_map[3];
  int32_t forloop_range;
  int32_t reduction_dimx;
  int32_t grid_dim[3];
  int32_t block_dim[3];
} mg_plan;

typedef struct mg_runtime mg_runtime; /* kernel::DeviceMemoryManager, one per process */
typedef struct mg_graph mg_graph;     /* kernel::Graph */

/* ---- runtime / device memory manager -------------------------------------
 * replaces DeviceMemoryManager::get_instance() and its constructor
 * (src/kernel/device_memory_manager.cu:26-91,140-145): one arena cudaMalloc,
 * LIFO bump allocation, exp / inverse lookup tables at the arena base.
 * arena_bytes = 0 selects the reference's 10 GiB.  device < 0 creates a planning-only runtime:
 * graphs can be built, validated and lowered, every launch or copy returns MG_ERR_NO_DEVICE. */
int mg_runtime_create(int device, size_t arena_bytes, mg_runtime **rt);
int mg_runtime_destroy(mg_runtime *rt);
/* device pointers of DeviceMemoryManager::{exp,div_p,div_q}_lookup_table
 * (include/mirage/kernel/device_memory_manager.h:45-47) */
int mg_runtime_tables(mg_runtime *rt, const uint16_t **exp_tbl, const uint16_t **div_p_tbl,
                      const uint16_t **div_q_tbl);
/* DeviceMemoryManager::{offset,total_size} */
int mg_runtime_arena_usage(mg_runtime *rt, size_t *used_bytes, size_t *total_bytes);
/* per-SM shared-memory budget the graph builder validates against
 * (reference: MAX_SMEM_SIZE, include/mirage/type.h:35; here the sm_100 limit by default) */
int mg_runtime_set_max_smem(mg_runtime *rt, size_t bytes);
/* select which kernels may be chosen for operators created afterwards: 0 = generic interpreters only,
 * 1 = pattern-specialised kernels where a graph matches, 2 = also issue a split-KV attention operator and the
 * merge operator consuming it as one launch when a whole graph is run (default) */
int mg_runtime_set_specialisation(mg_runtime *rt, int level);
/* How launches are sized.  MG_POLICY_LATENCY (default): one call at a time is as fast as possible (a block keeps
 * its whole KV split in flight and works on its tiles side by side).  MG_POLICY_THROUGHPUT: the caller keeps
 * several independent calls in flight (streams, captured graphs); blocks are kept small so that blocks of
 * different launches share an SM and memory traffic of one call overlaps the arithmetic and tail of another.
 * The reference has no such knob (one kernel at a time on the default stream). */
enum { MG_POLICY_LATENCY = 0, MG_POLICY_THROUGHPUT = 1 };
int mg_runtime_set_launch_policy(mg_runtime *rt, int policy);

/* Tuning switches of the kernels (process-wide; 0 = let the library decide).  They are read when a launch is
 * configured: a captured sequence keeps the values it was recorded with.  The reference has no such knobs. */
enum {
  MG_OPT_ATTN_STAGES = 0,       /* split-KV attention: shared-memory ring depth, 1..6 */
  MG_OPT_ATTN_TILE_GROUPS = 1,  /* split-KV attention: KV tiles of the ring worked on side by side, 1..4 */
  MG_OPT_ATTN_ENGINE = 2,       /* split-KV attention, float mode: 1 = mma.sync kernel, 2 = tcgen05 kernel */
  MG_OPT_ROWS_ENGINE = 3,       /* dense attention: 1 = one query tile per block, 2 = two query tiles per block */
  MG_OPT_INTERP_THREADS = 4,    /* generic interpreters: threads per block, 256 / 512 / 1024 */
  MG_OPT_WAIT_LIMIT = 5,        /* split-KV attention: polls before a tile wait gives up; 1 = give up without polling
                                   (failure-path tests), n > 1 = n polls */
  MG_OPT_ATTN_PERSISTENT = 6,   /* split-KV attention with more blocks than fit at once: 1 = one block per work item,
                                   2 = resident blocks that walk the work items (the default where it fits) */
  MG_OPT_KN_MATMUL_ENGINE = 7,  /* kernel-level float matmul: 1 = CUDA cores, 2 = tcgen05 (the default where it applies) */
  MG_OPT_ATTN_DEPENDENT_LAUNCH = 8 /* split-KV and dense attention: 1 = plain stream order, 2 = programmatic dependent launch (default) */
};
int mg_runtime_set_option(mg_runtime *rt, int32_t key, int32_t value);
int mg_runtime_get_option(mg_runtime *rt, int32_t key, int32_t *value);
/* The split-KV and the dense attention kernels start fetching Q, K and V while the previous kernel of their stream is
 * still draining (the dense kernel's first blocks then run on the SMs that kernel's last round of blocks leaves idle),
 * when the library knows the two launches in front of it and knows they did not write them (a kernel may run beside
 * both, never beside an older one).  Launches, copies and fills that go through
 * this ABI are tracked.  A caller that writes a graph's input tensors with work of its own (a kernel given
 * data_ptr / fp_ptr) enqueued on `stream` says so with this call, after enqueueing that work and before the next
 * launch of this library on that stream; that launch then reads its inputs only after the stream's previous kernel
 * has completed.  No counterpart in the reference (one kernel at a time on the default stream). */
int mg_stream_inputs_written(void *stream);
/* Failure-path self-test (no counterpart in the reference, which exits on any CUDA error,
 * include/mirage/utils/cuda_helper.h:30-38): enqueues a one-block kernel that waits on an mbarrier nobody arrives
 * at, gives up after `poll_limit` polls and records a code in the device status word.  Nothing hangs or faults;
 * the next synchronising call (mg_device_synchronize, mg_graph_fingerprint ...) returns MG_ERR_DEVICE_TIMEOUT once,
 * and later launches run normally. */
int mg_selftest_bounded_wait(mg_runtime *rt, int32_t poll_limit, void *stream);

/* ---- kernel graph ---------------------------------------------------------
 * kernel::Graph, include/mirage/kernel/graph.h:28-85 */
int mg_graph_create(mg_runtime *rt, mg_graph **g);
/* destroys operators in reverse order (arena frees are LIFO, device_memory_manager.cu:124-138) */
int mg_graph_destroy(mg_graph *g);
/* Graph::new_input(dims, data_type, layout), src/kernel/operator.cc:52-60 */
int mg_graph_new_input(mg_graph *g, const int32_t *dims, int32_t num_dims, int32_t data_type, int32_t layout,
                       mg_tensor *out);
/* Graph::customized(inputs, plan), src/kernel/customized.cc:32-44; outputs in the
 * order the reference discovers them (customized.cc:144-185) */
int mg_graph_customized(mg_graph *g, const mg_tensor *inputs, int32_t num_inputs, const mg_plan *plan,
                        mg_tensor *outputs, int32_t max_outputs, int32_t *num_outputs);
/* un-fused kernel-level operators, Graph::{matmul,exp,add,mul,div,reduction}
 * (src/kernel/{matmul,element_unary,element_binary,reduction}.cc) */
int mg_graph_matmul(mg_graph *g, const mg_tensor *a, const mg_tensor *b, mg_tensor *out);
int mg_graph_exp(mg_graph *g, const mg_tensor *a, mg_tensor *out);
int mg_graph_add(mg_graph *g, const mg_tensor *a, const mg_tensor *b, mg_tensor *out);
int mg_graph_mul(mg_graph *g, const mg_tensor *a, const mg_tensor *b, mg_tensor *out);
int mg_graph_div(mg_graph *g, const mg_tensor *a, const mg_tensor *b, mg_tensor *out);
int mg_graph_reduction(mg_graph *g, const mg_tensor *a, int32_t dim, int32_t size, mg_tensor *out);

int mg_graph_num_operators(mg_graph *g, int32_t *n);
/* shared-memory bytes, operator count of the threadblock graph of a customized op
 * (threadblock::Graph::smem_offset / operators.size()) */
int mg_graph_customized_info(mg_graph *g, int32_t op_idx, int32_t *num_tb_operators, int32_t *smem_bytes,
                             int32_t *kernel_id_fingerprint, int32_t *kernel_id_float);

/* the lowered kernel-level program of a customized op (struct mgd_program of mugraph_device.h;
 * program_bytes = sizeof(mgd_program)); the counterpart of threadblock::Graph::get_new_kernel_params,
 * src/threadblock/graph.cc:68-432 */
int mg_graph_customized_program(mg_graph *g, int32_t op_idx, void *program_out, size_t program_bytes);
/* float-mode extension with no counterpart in the reference: query row r of the split-KV attention
 * operator belongs to draft token r / (rows / window) and sees KV positions <= kv_len - window + token;
 * 0 switches the mask off.  Fingerprint mode ignores it. */
int mg_graph_customized_set_causal_window(mg_graph *g, int32_t op_idx, int32_t window);

/* ---- batched verification ---------------------------------------------------
 * The search's verify step (src/search/search.cc:569-623: run every candidate's fingerprint kernels, then
 * DTensor::has_same_fingerprint against the computation graph, one device synchronisation and two blocking
 * copies per candidate) as one batch: the fingerprint kernels of all n candidate graphs (inputs already in place)
 * and the n comparisons of outputs[i] with `reference` are enqueued on `stream` back to back; one synchronisation
 * and one copy of n flags at the end.  same[i] = 1 when candidate i's output equals the reference bit for bit
 * (0 also when the shapes differ). */
int mg_verify_candidates(mg_runtime *rt, const mg_tensor *reference, mg_graph *const *candidates,
                         const mg_tensor *outputs, int32_t n, int32_t *same, void *stream);

/* ---- graph JSON wire format ------------------------------------------------
 * replaces to_json(json&, Graph const&) / from_json(json const&, Graph&) (src/kernel/graph.cc:33-159) and the
 * operators' `operator json()`; documents are exchanged as text (see include/mirage/utils/json_utils.h).
 * mg_graph_to_json: writes at most `capacity` bytes (NUL included) and always reports the length needed
 * (without NUL) in *length; MG_ERR_INVALID_ARGUMENT if the buffer is too small (call again with length + 1).
 * mg_graph_from_json: builds a new graph from a document the reference or this library wrote; on failure no
 * graph is left behind. */
int mg_graph_to_json(mg_graph *g, char *buf, size_t capacity, size_t *length);
int mg_graph_from_json(mg_runtime *rt, const char *text, mg_graph **g);
/* type (MG_KN_* code) and output tensors of operator op_idx; at most max_outputs tensors are written */
int mg_graph_operator_info(mg_graph *g, int32_t op_idx, int32_t *op_type, mg_tensor *outputs, int32_t max_outputs,
                           int32_t *num_outputs);

/* ---- the hot path ---------------------------------------------------------
 * KNOperator::fingerprint(), src/kernel/cuda/customized_kernel.cu:655-678 (and the
 * kernel-level ops' fingerprint()).  Synchronous like the reference. */
int mg_op_fingerprint(mg_graph *g, int32_t op_idx);
/* fingerprint every operator in order: `for (op : graph.operators) op->fingerprint()`
 * (cpp_examples/group_query_attn_inc_decode.cc:104-106), one stream, one final sync */
int mg_graph_fingerprint(mg_graph *g);
/* same, but input operators keep whatever their buffers hold (uploaded or seeded contents)
 * instead of being refilled with i % FP_PQ */
int mg_graph_fingerprint_compute(mg_graph *g);
/* mg_graph_fingerprint_compute without the synchronisation: the fingerprint kernels of every non-input operator
 * are enqueued on `stream` (a sequence a verifier captures and replays, or overlaps with other work); the caller
 * synchronises, e.g. with mg_device_synchronize, which also reports a bounded wait that gave up */
int mg_graph_fingerprint_enqueue(mg_graph *g, void *stream);
/* KNCustomizedOp::run(), customized_kernel.cu:605-613: asynchronous launch on `stream`
 * (a cudaStream_t; NULL = default stream) */
int mg_op_run(mg_graph *g, int32_t op_idx, void *stream);
/* KNOperator::profile(ProfileResult&), customized_kernel.cu:615-653: `warmup` untimed
 * then `iters` timed launches between two CUDA events; *ms = mean per launch.
 * warmup = iters = 0 selects the reference's 1024 + 1024. */
int mg_op_profile(mg_graph *g, int32_t op_idx, int32_t warmup, int32_t iters, float *ms);
/* run every operator of the graph in order on `stream` (asynchronous) */
int mg_graph_run(mg_graph *g, void *stream);
/* A graph owns the scratch of its fused launches (one ticket counter per head): two launches of the SAME graph
 * must not be in flight at the same time (different streams without an ordering between them).  Different graphs
 * are independent. */

/* Batched fingerprint evaluation: the same graph evaluated on `num_sets` independent
 * input sets in one pass.  Input i of set s is read at in_fp[i] + s * elements(input i);
 * the last operator's output 0 for set s is written to out_fp + s * elements(output).
 * Intermediate tensors of all sets live in `workspace` (device memory,
 * `*workspace_bytes` from the query call with workspace = NULL); what is in it when the call starts does not
 * matter, and nothing in it is meant for the caller.  The ticket counters of fused launches are device memory of the
 * graph's own: the first call, and a call with more sets than any before, allocates them (which synchronises the
 * device, so make that call outside a stream capture); after that consecutive calls on a stream run without any
 * copy or clearing between their kernels.
 * Stands in for `num_sets` repetitions of the verify loop, src/search/search.cc:601-603. */
int mg_graph_fingerprint_batched(mg_graph *g, int32_t num_sets, const uint16_t *const *in_fp, uint16_t *out_fp,
                                 void *workspace, size_t *workspace_bytes, void *stream);

/* The float-mode counterpart: `num_sets` independent calls of the same graph (KNCustomizedOp::run,
 * customized_kernel.cu:605-613, repeated) as one pass - one kernel per customized operator over all sets, and a
 * split-KV attention operator together with the merge operator consuming it as ONE kernel.  Input i of set s is
 * read at in_data[i] + s * elements(input i) 16-bit values, the last operator's output 0 of set s is written to
 * out_data + s * elements(output); same workspace protocol as above.  Asynchronous on `stream`. */
int mg_graph_run_batched(mg_graph *g, int32_t num_sets, const void *const *in_data, void *out_data, void *workspace,
                         size_t *workspace_bytes, void *stream);

/* Row-wise comparison of two fingerprint arrays [rows][row_elements] on the device, one pass over both:
 * equal_flags[r] = 1 when row r of `a` equals row r of `b` bit for bit, else 0; *mismatch_count (optional, device
 * memory, zeroed by this call) = rows that differ.  All pointers are device memory; asynchronous on `stream`.
 * The search's verify loop (src/search/search.cc:601-609: one DTensor::has_same_fingerprint with two blocking
 * copies per candidate) for a whole batch of gathered fingerprints. */
int mg_compare_fingerprint_rows(mg_runtime *rt, const uint16_t *a, const uint16_t *b, int64_t rows, int64_t row_elements,
                                int32_t *equal_flags, int32_t *mismatch_count, void *stream);

/* DTensor::has_same_fingerprint, src/kernel/cuda/device_tensor_kernel.cu:22-53;
 * compared on the device, one 4-byte result copied back */
int mg_tensor_has_same_fingerprint(mg_runtime *rt, const mg_tensor *a, const mg_tensor *b, int32_t *same);

/* ---- data movement and fills ---------------------------------------------- */
/* KNInputOp::fingerprint(), src/kernel/cuda/input_kernel.cu:56-73: fp[i] = i % FP_PQ */
int mg_tensor_fill_fingerprint_reference(mg_runtime *rt, const mg_tensor *t);
/* counter-based seeded fills (same generator as the host checker, see mugraph_rng.h):
 * fingerprints uniform in [0, modulus); 16-bit floats ~ N(0, sigma) rounded to storage type */
int mg_tensor_fill_fingerprint_seeded(mg_runtime *rt, const mg_tensor *t, uint64_t seed, uint32_t modulus);
int mg_tensor_fill_data_seeded(mg_runtime *rt, const mg_tensor *t, uint64_t seed, float sigma);
int mg_tensor_upload_fingerprint(mg_runtime *rt, const mg_tensor *t, const uint16_t *host);
int mg_tensor_download_fingerprint(mg_runtime *rt, const mg_tensor *t, uint16_t *host);
int mg_tensor_upload_data(mg_runtime *rt, const mg_tensor *t, const void *host_16bit);
int mg_tensor_download_data(mg_runtime *rt, const mg_tensor *t, void *host_16bit);
/* asynchronous variants for pinned host buffers (end-to-end paths) */
int mg_tensor_upload_data_async(mg_runtime *rt, const mg_tensor *t, const void *host_16bit, void *stream);
int mg_tensor_download_data_async(mg_runtime *rt, const mg_tensor *t, void *host_16bit, void *stream);
/* rebind a graph input to caller-owned device memory (e.g. one of several rotating buffers) */
int mg_graph_rebind_input(mg_graph *g, int32_t op_idx, void *data_ptr, uint16_t *fp_ptr);

/* ---- CUDA-graph capture of launch sequences ----------------------------------
 * At a few microseconds per customized op the CPU cost of a launch exceeds the kernel; a caller
 * that replays the same sequence (the reference's profile loop, customized_kernel.cu:631-647, or a
 * verification sweep) captures it once and replays it.  `stream` must be a non-default stream;
 * only asynchronous entry points (mg_op_run, mg_graph_run, mg_graph_fingerprint_batched, the
 * *_async copies) may be called between begin and end, after each was called once outside. */
int mg_capture_begin(void *stream);
int mg_capture_end(void *stream, void **captured);
int mg_captured_launch(void *captured, void *stream);
int mg_captured_destroy(void *captured);

/* ---- misc ------------------------------------------------------------------ */
int mg_device_synchronize(void);
const char *mg_last_error(void);
const char *mg_version(void);
/* number of kernels of this library launched by the calling process so far */
uint64_t mg_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* MUGRAPH_H_ */
