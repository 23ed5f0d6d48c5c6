/* mugraph_device.h - kernel-level C ABI: the only door between the host C++
 * (graph building, validation, planning, kernel selection) and the sm_100a
 * CUDA side.  Plain structs, pointers and sizes; every call returns an MG_*
 * status from mugraph.h and enqueues work on the given cudaStream_t without
 * synchronising unless stated.
 *
 * A threadblock graph travels as a `mgd_program`: the list of operators of one
 * customized op with all shapes, shared-memory offsets and block / for-loop
 * strides already resolved by the host.  It carries the information of the
 * reference's NewKernelParams (include/mirage/threadblock/serializer/kernel_params.h:25-35)
 * in a different container; the interpreters that consume it replace
 * compute_customizedop_fingerprint and customized_kernel_function
 * (src/kernel/cuda/customized_kernel.cu:39-603).
 */
#ifndef MUGRAPH_DEVICE_H_
#define MUGRAPH_DEVICE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MGD_MAX_OPS 24
#define MGD_MAX_IO 8
#define MGD_OP_ARGS 19

/* Operator record.  `type` is a MG_TB_* code (2001 = input, 2002 = output).
 * Shared-memory offsets are byte offsets in the reference's 2-byte-per-element plan.
 *  input   a[0..2] row block stride (x,y,z)   a[3..5] column block stride   a[6] row for-loop stride
 *          a[7] column for-loop stride   a[8..10] leading-dim block stride (elements)   a[11] leading-dim
 *          for-loop stride   a[12],a[13] tensor rows, cols   a[14],a[15] tile rows, cols   a[16] MG_DMEM_* layout
 *          a[17] tile offset   a[18] input slot
 *  output  a[0..2] row block stride   a[3..5] column block stride   a[6..8] leading-dim block stride
 *          a[9],a[10] tensor rows, cols   a[11],a[12] tile rows, cols   a[13] source tile offset
 *          a[14] accumulator tile offset   a[15] output slot
 *  matmul  a[0..2] m, n, k   a[3..5] offsets of A, B, C
 *  exp     a[0] offset   a[1] elements                      (in place)
 *  div/add/mul  a[0..2] shape of x (last three dims)   a[3..5] shape of y   a[6],a[7] offsets x, y   a[8] offset out
 *  reduction    a[0] output elements   a[1] degree   a[2] inner range   a[3] offset in   a[4] offset out
 *  concat  a[0] output elements   a[1],a[2] extents of A, B along the axis   a[3] inner size
 *          a[4],a[5] offsets A, B   a[6] offset out */
typedef struct mgd_op {
  int32_t type;
  int32_t a[MGD_OP_ARGS];
} mgd_op;

/* Names of the slots of mgd_op.a[] listed above ("+ axis" = three consecutive slots for grid x, y, z). */
enum {
  MGD_IN_ROW_BLOCK_STRIDE = 0 /* + axis */, MGD_IN_COL_BLOCK_STRIDE = 3 /* + axis */, MGD_IN_ROW_LOOP_STRIDE = 6,
  MGD_IN_COL_LOOP_STRIDE = 7, MGD_IN_LEAD_BLOCK_STRIDE = 8 /* + axis */, MGD_IN_LEAD_LOOP_STRIDE = 11,
  MGD_IN_ROWS = 12, MGD_IN_COLS = 13, MGD_IN_TILE_ROWS = 14, MGD_IN_TILE_COLS = 15, MGD_IN_LAYOUT = 16,
  MGD_IN_TILE_OFFSET = 17, MGD_IN_SLOT = 18
};
enum {
  MGD_OUT_ROW_BLOCK_STRIDE = 0 /* + axis */, MGD_OUT_COL_BLOCK_STRIDE = 3 /* + axis */,
  MGD_OUT_LEAD_BLOCK_STRIDE = 6 /* + axis */, MGD_OUT_ROWS = 9, MGD_OUT_COLS = 10, MGD_OUT_TILE_ROWS = 11,
  MGD_OUT_TILE_COLS = 12, MGD_OUT_SOURCE_OFFSET = 13, MGD_OUT_ACCUM_OFFSET = 14, MGD_OUT_SLOT = 15
};
enum { MGD_MM_M = 0, MGD_MM_N = 1, MGD_MM_K = 2, MGD_MM_A_OFFSET = 3, MGD_MM_B_OFFSET = 4, MGD_MM_C_OFFSET = 5 };
enum { MGD_EXP_OFFSET = 0, MGD_EXP_ELEMENTS = 1 };
enum { MGD_BIN_X_SHAPE = 0 /* + 0..2 */, MGD_BIN_Y_SHAPE = 3 /* + 0..2 */, MGD_BIN_X_OFFSET = 6, MGD_BIN_Y_OFFSET = 7,
       MGD_BIN_OUT_OFFSET = 8 };
enum { MGD_RED_OUT_ELEMENTS = 0, MGD_RED_DEGREE = 1, MGD_RED_INNER = 2, MGD_RED_IN_OFFSET = 3, MGD_RED_OUT_OFFSET = 4 };

typedef struct mgd_program {
  int32_t grid[3];
  int32_t threads;        /* threads per block the host asks for (plan.block_dim.x) */
  int32_t forloop_range;
  int32_t num_ops;
  int32_t num_inputs;
  int32_t num_outputs;
  int32_t smem_bytes;     /* reference plan size: 2 bytes per tile element */
  int32_t reserved[3];
  mgd_op ops[MGD_MAX_OPS];
} mgd_program;

/* Where the tensors of one launch live.  With num_sets > 1 the launch evaluates the
 * program on num_sets independent tensor sets: set s reads in[i] + s*in_set_stride[i]
 * elements and writes out[j] + s*out_set_stride[j]. */
typedef struct mgd_bindings {
  const void *in[MGD_MAX_IO];
  void *out[MGD_MAX_IO];
  int64_t in_set_stride[MGD_MAX_IO];
  int64_t out_set_stride[MGD_MAX_IO];
  int32_t num_sets;
  int32_t reserved;
} mgd_bindings;

/* ---- generic interpreters (any valid threadblock graph) -------------------- */
/* replaces compute_customizedop_fingerprint<<<grid, block, smem>>> (customized_kernel.cu:307-603) */
int mgd_launch_fingerprint_interp(const mgd_program *prog, const mgd_bindings *bind, void *stream);
/* replaces customized_kernel_function<<<grid, block, smem>>> (customized_kernel.cu:39-305);
 * data_type MG_DT_FLOAT16 or MG_DT_BFLOAT16; tiles are held in fp32 shared memory */
int mgd_launch_float_interp(const mgd_program *prog, const mgd_bindings *bind, int32_t data_type, void *stream);
/* shared memory the float interpreter needs for `prog`; *fits = 0 when above the device limit */
int mgd_float_interp_smem(const mgd_program *prog, size_t *bytes, int32_t *fits);

/* ---- split-KV attention, the pattern of cpp_examples/group_query_attn_inc_decode.cc:46-79 ---
 * op1: S = Q K, E = exp(S), O' = E V, R' = rowsum(E), both summed over the for-loop, one partial
 * per grid.y split.  Shapes: Q[heads, m, d], K[heads, d, kv], V[heads, kv, d];
 * O_part[heads, m, splits*d], R_part[heads, m, splits]. */
typedef struct mgd_attn_split {
  int32_t heads, m, d, kv_len;
  int32_t splits;         /* grid.y */
  int32_t forloop_range;  /* KV tiles per split */
  int32_t k_layout;       /* MG_DMEM_*: row-major = memory [d][kv]; column-major = memory [kv][d] */
  int32_t v_layout;       /* row-major = memory [kv][d]; column-major = memory [d][kv] */
  int32_t data_type;      /* float mode only */
  int32_t causal_window;  /* float mode only: 0 = none; w > 0 masks, for query row r (token r / (m / w)),
                             KV positions > kv_len - w + token */
  int32_t num_sets;
  int32_t reserved;
  int64_t q_set_stride, k_set_stride, v_set_stride, o_set_stride, r_set_stride; /* elements */
} mgd_attn_split;
int mgd_attn_split_supported(const mgd_attn_split *p, int32_t fingerprint_mode);
/* Optional extras of one split-KV launch.
 *  merged_out / tickets: also perform the second customized op of the example (:80-103) in the same launch -
 *    the last block of a head to finish sums the head's partials and divides ("last block done" ticket).
 *    tickets = heads * num_sets int32 in device memory, zero before the first use; the kernel leaves them zero
 *    (also when a block's bounded wait gave up: such a block still takes its ticket).
 *  overlap: bit 0 = launch with programmatic stream serialisation, so that this kernel's blocks may be scheduled
 *    while the previous kernel of the stream drains (every global write still waits for that kernel's completion);
 *    bit 1 = none of the inputs was written by the previous kernel of this library on this stream, so the tile
 *    loads may be issued before that wait;
 *    bit 2 = size the blocks for throughput (two-stage ring, four warps): blocks of several launches in flight
 *    then share an SM.  Without it a launch that fits one wave keeps its whole KV split in flight per block,
 *    which gives the lowest latency for one launch at a time;
 *    bit 3 (with merged_out) = o_part / r_part are scratch that nobody reads after the launch: a launch with more
 *    blocks than fit at once then sums consecutive splits of a head on the chip and writes only the partial sums the
 *    merge needs (some slots of o_part / r_part stay untouched). */
typedef struct mgd_attn_launch_opts {
  void *merged_out;          /* [num_sets][heads][m][d], NULL = partials only */
  int32_t *tickets;
  int64_t merged_set_stride;
  int32_t overlap;
  int32_t reserved;
} mgd_attn_launch_opts;
int mgd_launch_attn_split_float_ex(const mgd_attn_split *p, const void *q, const void *k, const void *v, void *o_part,
                                   void *r_part, const mgd_attn_launch_opts *opts, void *stream);
int mgd_launch_attn_split_fingerprint_ex(const mgd_attn_split *p, const uint16_t *q, const uint16_t *k,
                                         const uint16_t *v, uint16_t *o_part, uint16_t *r_part,
                                         const mgd_attn_launch_opts *opts, void *stream);
int mgd_launch_attn_split_float(const mgd_attn_split *p, const void *q, const void *k, const void *v, void *o_part,
                                void *r_part, void *stream);
int mgd_launch_attn_split_fingerprint(const mgd_attn_split *p, const uint16_t *q, const uint16_t *k,
                                      const uint16_t *v, uint16_t *o_part, uint16_t *r_part, void *stream);

/* ---- dense attention over query-row tiles, the pattern of cpp_examples/multi_head_attn_prefill.cc:43-98 ---
 * A block owns tile_m query rows of one head and walks the KV axis in for-loop tiles of tile_kv:
 * S = Q K, E = exp(S), O' += E V, R' += rowsum(E).  Q[heads, seq_q, d], K[heads, d, kv_len], V[heads, kv_len, d];
 * outputs O_acc[heads, seq_q, d] (not normalised) and R[heads, seq_q, 1].  Runs on tcgen05 tensor cores with
 * accumulators in tensor memory; float mode only (fingerprints of such graphs use the interpreter). */
typedef struct mgd_attn_rows {
  int32_t heads, seq_q, d, kv_len;
  int32_t tile_m, tile_kv, forloop_range;
  int32_t k_layout, v_layout, data_type;
} mgd_attn_rows;
int mgd_attn_rows_supported(const mgd_attn_rows *p);
int mgd_launch_attn_rows_float(const mgd_attn_rows *p, const void *q, const void *k, const void *v, void *o_acc,
                               void *r_acc, void *stream);
/* same launch that also performs the division operator that follows in the example (:88-98):
 * o_div[heads, seq_q, d] = O_acc / R, from the fp32 accumulators; NULL = none */
int mgd_launch_attn_rows_float_ex(const mgd_attn_rows *p, const void *q, const void *k, const void *v, void *o_acc,
                                  void *r_acc, void *o_div, void *stream);
/* the same with the `overlap` bits of mgd_attn_launch_opts (bits 0 and 1; the others are ignored): bit 0 launches with
 * programmatic stream serialisation, so that the NEXT kernel of the stream may start on the SMs this one leaves idle in
 * its last round of blocks; bit 1 says that the kernel in front of this one did not write Q, K or V, so this one may
 * read them before that kernel has finished.  Global memory is only written after it has.  The one-tile-per-block
 * kernel (query lengths that are not a multiple of 256) ignores the bits. */
int mgd_launch_attn_rows_float_overlapped(const mgd_attn_rows *p, const void *q, const void *k, const void *v, void *o_acc,
                                          void *r_acc, void *o_div, int32_t overlap, void *stream);

/* Allocation-free variant of the fused decode launch (split-KV partials + cross-split merge in one kernel).
 * It has no counterpart in the reference.
 *
 * Who needs it: a host that has already handed the GPU's memory to its own pool (a serving process whose
 * allocator owns the device, or an embedding of this library next to another arena like the reference's
 * 10 GiB slab) cannot count on a cudaMalloc inside a library succeeding, and a latency-critical loop cannot
 * afford one, because cudaMalloc / cudaFree synchronise the device.  This entry point therefore calls no
 * cudaMalloc, cudaFree or any allocating routine: the "last block done" ticket counters and the status word
 * live in a file-scope device array of the library (16.6 KB per GPU that loads the library, held until exit).
 *
 * Limit: heads * num_sets <= 4096 counters; larger requests are rejected with MG_ERR_INVALID_ARGUMENT.
 * The caller passes every tensor: q, k, v (inputs), o_part, r_part (partials, also outputs) and out
 * ([num_sets][heads][m][d], dense).  p->o_set_stride / r_set_stride / q_set_stride describe the set pitch of
 * those buffers as in mgd_attn_split.
 *
 * First call on a device: looks up the device address of the array (cudaGetSymbolAddress, with that device
 * current) and configures the kernel's shared-memory limit; make that first call before any stream capture.
 * Every call shares the one array: the counters are cleared on `stream` at the start of each call, so two calls
 * that overlap on the GPU (different streams, or anything else that lets them run concurrently) race on them
 * and must be serialised by the caller.
 * check_status != 0: synchronise `stream` after the launch and return MG_ERR_DEVICE_TIMEOUT if a bounded device
 * wait gave up (4-byte copy, still no allocation); 0: fully asynchronous, nothing is reported.  The status word is
 * cleared on `stream` at the start of every call, so a call reports only its own launch: a timeout of an earlier
 * call made with check_status = 0 is lost once the next call starts.
 * The shared-memory limit of the kernel is configured per device, on the first call on that device. */
int mgd_attn_decode_fused_noalloc(const mgd_attn_split *p, const void *q, const void *k, const void *v, void *o_part,
                                  void *r_part, void *out, int32_t fingerprint_mode, int32_t check_status,
                                  void *stream);

/* op2 of the same example (:80-103): O = (sum over splits of O_part) / (sum over splits of R_part) */
typedef struct mgd_attn_merge {
  int32_t heads, m, d, splits;
  int32_t data_type;
  int32_t num_sets;
  int64_t o_part_set_stride, r_part_set_stride, out_set_stride;
} mgd_attn_merge;
int mgd_attn_merge_supported(const mgd_attn_merge *p, int32_t fingerprint_mode);
int mgd_launch_attn_merge_float(const mgd_attn_merge *p, const void *o_part, const void *r_part, void *out,
                                void *stream);
int mgd_launch_attn_merge_fingerprint(const mgd_attn_merge *p, const uint16_t *o_part, const uint16_t *r_part,
                                      uint16_t *out, void *stream);

/* ---- two chained threadblock matmuls with for-loop accumulation ---------------------------------
 * out = sum over the for-loop of (X_i W1_i) W2 with a loop-invariant W2: the customized operator made of two
 * tb_matmul_op and an accumulating tb_output_op (the pattern of cpp_examples/mlp.cc).  x / w1 / w2 / out are the
 * program's records of the three inputs and of the output (coordinates per block and iteration as in mgd_op). */
typedef struct mgd_matmul_chain {
  int32_t grid[3];
  int32_t forloop_range;
  int32_t m, kt, n1, n2; /* X_i [m x kt], W1_i [kt x n1], W2 [n1 x n2], out [m x n2] */
  int32_t data_type;
  int32_t reserved;
  mgd_op x, w1, w2, out;
} mgd_matmul_chain;
int mgd_matmul_chain_supported(const mgd_matmul_chain *c, int32_t fingerprint_mode);
int mgd_launch_matmul_chain_float(const mgd_matmul_chain *c, const mgd_bindings *bind, void *stream);
int mgd_launch_matmul_chain_fingerprint(const mgd_matmul_chain *c, const mgd_bindings *bind, void *stream);

/* ---- a customized operator that is one threadblock reduction ----------------------------------------
 * input tile -> tb_reduction_*_op (plain or "to dimx") -> output tile, for-loop of one: the cross-block reduction
 * behind a split operator.  in / out are the program's records of the input and the output; out element i of a tile
 * = sum over k < degree of in_tile[(i / inner) * inner * degree + i % inner + k * inner] (dense row-major tile). */
typedef struct mgd_tile_reduce {
  int32_t grid[3];
  int32_t out_elements, degree, inner;
  int32_t data_type;
  int32_t chunks; /* set by the launch */
  mgd_op in, out;
} mgd_tile_reduce;
int mgd_tile_reduce_supported(const mgd_tile_reduce *c, int32_t fingerprint_mode);
int mgd_launch_tile_reduce(const mgd_tile_reduce *c, const mgd_bindings *bind, int32_t fingerprint_mode, void *stream);

/* ---- un-fused kernel-level operators, fingerprint mode ----------------------
 * replace compute_matmul_fingerprint (src/kernel/cuda/matmul_kernel.cu:145-173),
 * compute_elementunary_fingerprint (element_unary_kernel.cu:77-94),
 * compute_elementbinary_fingerprint (element_binary_kernel.cu:97-168),
 * compute_reduction_fingerprint (reduction_kernel.cu:80-108) */
int mgd_kn_matmul_fingerprint(const uint16_t *a, const uint16_t *b, uint16_t *c, int32_t batches, int32_t m,
                              int32_t n, int32_t k, void *stream);
int mgd_kn_exp_fingerprint(const uint16_t *x, uint16_t *y, int64_t n, void *stream);
/* op = MG_KN_ADD_OP / MG_KN_MUL_OP / MG_KN_DIV_OP; dims are the 4 (right-aligned) extents */
int mgd_kn_binary_fingerprint(int32_t op, const uint16_t *x, const int32_t *xdim, const uint16_t *y,
                              const int32_t *ydim, uint16_t *z, const int32_t *zdim, void *stream);
int mgd_kn_reduction_fingerprint(const uint16_t *x, uint16_t *y, int64_t out_elements, int32_t factor,
                                 int64_t input_stride, int64_t output_stride, void *stream);
/* float-mode counterparts (16-bit storage, fp32 arithmetic) */
int mgd_kn_matmul_float(const void *a, const void *b, void *c, int32_t batches, int32_t m, int32_t n, int32_t k,
                        int32_t a_layout, int32_t b_layout, int32_t data_type, void *stream);
int mgd_kn_exp_float(const void *x, void *y, int64_t n, int32_t data_type, void *stream);
int mgd_kn_binary_float(int32_t op, const void *x, const int32_t *xdim, const void *y, const int32_t *ydim, void *z,
                        const int32_t *zdim, int32_t data_type, void *stream);
int mgd_kn_reduction_float(const void *x, void *y, int64_t out_elements, int32_t factor, int64_t input_stride,
                           int64_t output_stride, int32_t data_type, void *stream);

/* ---- fills, compare, tables -------------------------------------------------- */
/* init_input_fingerprint, src/kernel/cuda/input_kernel.cu:56-62 */
int mgd_fill_fingerprint_reference(uint16_t *p, int64_t n, void *stream);
int mgd_fill_fingerprint_seeded(uint16_t *p, int64_t n, uint64_t seed, uint32_t modulus, void *stream);
int mgd_fill_data_seeded(void *p, int64_t n, uint64_t seed, float sigma, int32_t data_type, void *stream);
/* *device_flag (4 bytes, device memory) <- 1 if equal else 0 */
int mgd_compare_u16(const uint16_t *a, const uint16_t *b, int64_t n, int32_t *device_flag, void *stream);
/* row-wise: equal_flags[r] <- 1 if a[r][:] == b[r][:] else 0; *mismatch_count (optional) <- rows that differ */
int mgd_compare_rows_u16(const uint16_t *a, const uint16_t *b, int64_t rows, int64_t row_elements, int32_t *equal_flags,
                         int32_t *mismatch_count, void *stream);
/* copies the lookup tables of src/kernel/device_memory_manager.cu:41-90 into constant memory
 * of the current device; idempotent */
int mgd_tables_init(const uint16_t *exp_tbl, const uint16_t *div_p_tbl, const uint16_t *div_q_tbl);
/* device status word written by kernels whose bounded waits gave up; 0 = none. Synchronises. */
int mgd_read_and_clear_device_error(int32_t *code);

/* ---- tuning switches ----------------------------------------------------------
 * Process-wide launch options of the kernels (the reference has none: its launch shapes are the plan's).
 * Read when a launch is configured, so a captured sequence keeps the values it was recorded with.
 * 0 always means "let the library decide". */
enum {
  MGD_OPT_ATTN_STAGES = 0,        /* split-KV attention: shared-memory ring depth, 1..6 */
  MGD_OPT_ATTN_TILE_GROUPS = 1,   /* split-KV attention: KV tiles of the ring worked on side by side, 1..4 */
  MGD_OPT_ATTN_ENGINE = 2,        /* split-KV attention, float mode: 1 = mma.sync kernel, 2 = tcgen05 kernel */
  MGD_OPT_ROWS_ENGINE = 3,        /* dense attention: 1 = one query tile per block, 2 = two query tiles per block */
  MGD_OPT_INTERP_THREADS = 4,     /* generic interpreters: threads per block, 256 / 512 / 1024 */
  MGD_OPT_WAIT_LIMIT = 5,         /* split-KV attention: polls before a tile wait gives up; 1 = give up without
                                     polling (failure-path tests), n > 1 = n polls */
  MGD_OPT_ATTN_PERSISTENT = 6,    /* split-KV attention with more blocks than fit at once: 1 = one block per work item,
                                     2 = resident blocks that walk the work items (the default where it fits) */
  MGD_OPT_KN_MATMUL_ENGINE = 7,   /* kernel-level float matmul: 1 = CUDA cores, 2 = tcgen05 (the default where the
                                     operands are 16-byte aligned with rows of a multiple of 8 elements) */
  MGD_OPT_ATTN_DEPENDENT_LAUNCH = 8, /* split-KV and dense attention: 1 = plain stream order, 2 = programmatic dependent launch (default) */
  MGD_OPT_COUNT = 9
};
int mgd_set_option(int32_t key, int32_t value);
int mgd_get_option(int32_t key, int32_t *value);
/* Failure-path self-test: one block waits on an mbarrier nobody arrives at, for `poll_limit` polls, then records
 * code 2 in the device status word and returns - the GPU neither hangs nor faults.  The next call that reads the
 * status word (mgd_read_and_clear_device_error, mg_device_synchronize) reports it. */
int mgd_selftest_bounded_wait(int32_t poll_limit, void *stream);
uint64_t mgd_launch_count(void);
const char *mgd_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* MUGRAPH_DEVICE_H_ */
