// What the two generic interpreters (fingerprint and float) share:
//
//  * the tile loader: input tiles are fetched by the TMA engine, completion counted in bytes on an mbarrier, into a
//    ring of `stages` shared-memory copies of the tiles that move with the for-loop, so the tiles of the next
//    iterations are in flight while the operators of this one run; tiles that do not move are fetched once, up
//    front.  Three forms, chosen per input on the host:
//      - a tile that only matmuls read as their B operand: cp.async.bulk.tensor in 64-column boxes with the 128-byte
//        swizzle, so that the transposed ldmatrix of the tensor-core matmuls is conflict-free without row padding;
//      - any other tile of at most 256 x 256: one cp.async.bulk.tensor box, dense;
//      - wider tiles: cp.async.bulk, one copy per (long) tile row.
//    This replaces the reference's input loaders, which issue cp.async and wait for it at once
//    (include/mirage/threadblock/cuda/input_loader.h:190-247).  A tile whose rows are not 16-byte aligned, a
//    column-major tensor, and a tile that is converted while it is loaded stay on plain loads.
//
//  * a rewrite of the program before it is planned: a matmul  C = A B  whose B is a loop-invariant input tile and
//    whose result only feeds an output operator (which sums it over the for-loop) is hoisted out of the loop -
//    sum_i (A_i B) = (sum_i A_i) B - so the loop accumulates A and the product is taken once, after the last
//    iteration.  Exact in the finite ring of the fingerprints; within rounding (and closer to the exact product)
//    in float mode.
#pragma once
#include "common.cuh"
#include "ptx.cuh"

namespace mgk {
namespace interp {

constexpr int kOpInput = 2001, kOpOutput = 2002;
constexpr int kOpAccumulate = 2990; // internal: acc = first ? x : acc + x   a[0] elements, a[1] source, a[2] accumulator
constexpr int kPhaseSlot = 18;      // non-input operators: a[18] = 1 -> runs once, after the last for-loop iteration
constexpr int kMaxStages = 4;
constexpr int kDynSmemLimit = kSmemLimit - 768; // dynamic shared memory: the kernels also hold a few barriers statically

inline bool is_reduction(int type) { return type >= MG_TB_REDUCTION_0_OP && type <= MG_TB_REDUCTION_2_TO_DIMX_OP; }
inline bool is_concat(int type) { return type == MG_TB_CONCAT_0_OP || type == MG_TB_CONCAT_1_OP || type == MG_TB_CONCAT_2_OP; }
inline bool is_binary(int type) { return type == MG_TB_DIV_OP || type == MG_TB_ADD_OP || type == MG_TB_MUL_OP; }

// number of operand reads of tile `planned` by `op` (an in-place exp counts as a read)
inline int reads_of(mgd_op const &op, int planned) {
  int32_t const *a = op.a;
  if (op.type == MG_TB_MATMUL_OP) return (a[3] == planned) + (a[4] == planned);
  if (op.type == MG_TB_EXP_OP) return a[0] == planned;
  if (is_binary(op.type)) return (a[6] == planned) + (a[7] == planned);
  if (is_reduction(op.type)) return a[3] == planned;
  if (is_concat(op.type)) return (a[4] == planned) + (a[5] == planned);
  if (op.type == kOpOutput) return a[13] == planned;
  if (op.type == kOpAccumulate) return a[1] == planned;
  return 0;
}
// tile written by `op`, or -1
inline int written_by(mgd_op const &op) {
  int32_t const *a = op.a;
  if (op.type == kOpInput) return a[17];
  if (op.type == MG_TB_MATMUL_OP) return a[5];
  if (op.type == MG_TB_EXP_OP) return a[0];
  if (is_binary(op.type)) return a[8];
  if (is_reduction(op.type)) return a[4];
  if (is_concat(op.type)) return a[6];
  if (op.type == kOpOutput) return a[14];
  if (op.type == kOpAccumulate) return a[2];
  return -1;
}
inline bool input_moves(mgd_op const &op) { return op.a[6] != 0 || op.a[7] != 0 || op.a[11] != 0; }

// Hoists loop-invariant right-multiplications out of the for-loop (see the header comment).  `p` is rewritten in
// place; new tiles are appended to the reference's two-bytes-per-element plan (p.smem_bytes grows).
inline void hoist_invariant_products(mgd_program &p) {
  if (p.forloop_range <= 1) return;
  for (int mi = 0; mi < p.num_ops; mi++) {
    mgd_op &mm = p.ops[mi];
    if (mm.type != MG_TB_MATMUL_OP || mm.a[kPhaseSlot] != 0 || p.num_ops + 1 > MGD_MAX_OPS) continue;
    int const a_tile = mm.a[3], b_tile = mm.a[4], c_tile = mm.a[5];
    if (a_tile == b_tile) continue;
    // B: written by exactly one operator, an input that does not move; nothing else touches it but matmuls reading it
    int b_writer = -1, b_writers = 0;
    bool b_clean = true;
    for (int i = 0; i < p.num_ops; i++) {
      if (written_by(p.ops[i]) == b_tile) { b_writers++; b_writer = i; }
      if (p.ops[i].type == MG_TB_EXP_OP && p.ops[i].a[0] == b_tile) b_clean = false;
    }
    if (b_writers != 1 || !b_clean || p.ops[b_writer].type != kOpInput || input_moves(p.ops[b_writer])) continue;
    // C: written by this matmul only, read by exactly one operator, an output that comes later
    int c_writers = 0, c_reads = 0, out_op = -1;
    for (int i = 0; i < p.num_ops; i++) {
      if (written_by(p.ops[i]) == c_tile) c_writers++;
      int const r = reads_of(p.ops[i], c_tile);
      c_reads += r;
      if (r && p.ops[i].type == kOpOutput) out_op = i;
    }
    if (c_writers != 1 || c_reads != 1 || out_op < mi) continue;
    // the output's accumulator must be private to it
    int const acc_tile = p.ops[out_op].a[14];
    bool acc_private = true;
    for (int i = 0; i < p.num_ops; i++)
      if (i != out_op && (written_by(p.ops[i]) == acc_tile || reads_of(p.ops[i], acc_tile))) acc_private = false;
    if (!acc_private) continue;
    // A must still hold this iteration's value when the accumulate operator runs in the matmul's place: fine, it
    // takes the matmul's position.  New tile for the running sum of A.
    int const m = mm.a[0], k = mm.a[2];
    int const sum_tile = (p.smem_bytes + 15) & ~15;
    p.smem_bytes = sum_tile + m * k * 2;
    mgd_op acc{};
    acc.type = kOpAccumulate;
    acc.a[0] = m * k; acc.a[1] = a_tile; acc.a[2] = sum_tile;
    mgd_op post_mm = mm;
    post_mm.a[3] = sum_tile;
    post_mm.a[kPhaseSlot] = 1;
    mgd_op post_out = p.ops[out_op];
    post_out.a[kPhaseSlot] = 1;
    // in-loop: the accumulate replaces the matmul; the output operator leaves its place; both post-loop operators
    // go to the end, in order
    p.ops[mi] = acc;
    for (int i = out_op; i + 1 < p.num_ops; i++) p.ops[i] = p.ops[i + 1];
    p.ops[p.num_ops - 1] = post_mm;
    p.ops[p.num_ops] = post_out;
    p.num_ops += 1;
    mi = -1; // the table changed: scan again (a hoisted matmul carries the phase mark and is skipped)
  }
}

// ---- TMA loader plan (host-built, read by the kernels from their parameters) -----------------------------------------
// One barrier for the tiles that are fetched once, one per ring stage for the moving tiles.
struct TmaPlan {
  int32_t stages;        // ring depth (0 = no moving tile is fetched by TMA)
  int32_t ring_lo;       // the moving TMA tiles occupy [ring_lo, ring_lo + ring_bytes) of the kernel's plan, stage s
  int32_t ring_bytes;    //   of all of them sits s * ring_bytes further
  uint32_t moving_mask;  // operator indices of the moving inputs fetched by TMA
  uint32_t once_mask;    // operator indices of the inputs fetched by TMA once
  int32_t moving_tx;     // bytes one stage receives
  int32_t once_tx;       // bytes the once-barrier receives
  uint32_t plain_once_mask; // inputs on plain loads whose tile is the same in every iteration: loaded in the first only
  uint32_t tiled_mask;      // of the TMA inputs: fetched as one dense tensor-map box
  uint32_t swizzled_mask;   // of the TMA inputs: fetched as 64-column tensor-map boxes with the 128-byte swizzle
  int32_t field_tables;     // fingerprint interpreter: byte offset + 1 (from the start of the dynamic shared memory) of
                            // a copy of the finite-field tables, 0 = none (the program has no exp or div, or no room)
};
constexpr int kFieldTableBytes = 1024; // exp lifted to Z_PQ [Q], inverses mod P [P], inverses mod Q [Q], 16 bits each

// tensor maps of the inputs fetched in a tiled form, by input slot: [matrices][rows][cols] of 16-bit elements
struct TmaMaps {
  CUtensorMap m[MGD_MAX_IO];
};

// `mats` matrices of rows x cols 16-bit elements (row pitch = cols), box = box_rows x box_cols
inline bool make_tile_map(CUtensorMap *map, void const *base, uint64_t cols, uint64_t rows, uint64_t mats, uint32_t box_cols,
                          uint32_t box_rows, bool swizzle128) {
  TensorMapEncodeFn fn = tensor_map_encoder();
  if (!fn) return false;
  cuuint64_t dims[3] = {cols, rows, mats};
  cuuint64_t strides[2] = {cols * 2, rows * cols * 2};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void *>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// matrices a launch can address through input `in`: the furthest leading-dim offset any block, iteration and set adds
inline uint64_t matrices_addressed(mgd_program const &p, mgd_op const &in, int64_t set_stride, int num_sets) {
  int32_t const *a = in.a;
  int64_t far = (int64_t)(p.grid[0] - 1) * a[8] + (int64_t)(p.grid[1] - 1) * a[9] + (int64_t)(p.grid[2] - 1) * a[10] +
                (int64_t)(p.forloop_range - 1) * a[11] + (int64_t)(num_sets - 1) * set_stride;
  int64_t const mat = (int64_t)a[12] * a[13];
  return (uint64_t)(far / mat + 1);
}

// Which tiled form (if any) suits a TMA-eligible input: 2 = swizzled 64-column boxes (`b_operand_only`: a tile the
// planner would otherwise store with padded rows), 1 = one dense box, 0 = per-row bulk copies.  The leading-dim
// offsets must address whole matrices.
inline int tiled_form(mgd_op const &in, int64_t set_stride, int num_sets, bool b_operand_only) {
  int32_t const *a = in.a;
  int64_t const mat = (int64_t)a[12] * a[13];
  for (int i = 8; i <= 11; i++) if (a[i] % mat != 0) return 0;
  if (num_sets > 1 && set_stride % mat != 0) return 0;
  int const rows = a[14], cols = a[15];
  if (rows > 256) return 0;
  // a tile stored with padded rows is either re-laid as swizzled boxes or keeps its padding (row copies)
  if (b_operand_only) return (cols % 64 == 0 && rows % 16 == 0) ? 2 : 0;
  if (cols <= 256) return 1;
  return 0;
}

// Can the rows of this input's tile be fetched with 16-byte aligned bulk copies?  `ld_elems` = elements between
// tensor rows; every offset a block or an iteration can add must keep the alignment.
inline bool tma_eligible(mgd_op const &in, void const *base, int64_t set_stride, int num_sets, int pitch_elems,
                         bool layout_matters) {
  int32_t const *a = in.a;
  if (layout_matters && (a[16] & 0xff) == MG_DMEM_COLUMN_MAJOR) return false; // fingerprints are row-major whatever the tag
  int const cols = a[15], ld = a[13];
  if (cols % 8 != 0 || ld % 8 != 0 || pitch_elems % 8 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return false;
  if (num_sets > 1 && set_stride % 8 != 0) return false;
  for (int i = 3; i <= 5; i++) if (a[i] % 8 != 0) return false;  // column origin per block
  if (a[7] % 8 != 0) return false;                                // column step per iteration
  for (int i = 8; i <= 11; i++) if (a[i] % 8 != 0) return false; // leading-dim offsets
  return a[14] > 0 && cols > 0;
}

#ifdef __CUDACC__
__device__ __forceinline__ void issue_tile_boxes(uint32_t dst, CUtensorMap const *map, int form, int rows, int cols, int col,
                                                 int row, int z, uint32_t bar, int lane);
__device__ __forceinline__ void issue_tile_rows(uint32_t dst, uint16_t const *first, int rows, int cols, int pitch, int ld,
                                                uint32_t bar, int lane);
__device__ __forceinline__ void bulk_load_row(uint32_t dst, void const *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// One input tile through its tensor map: `form` 2 = 64-column swizzled boxes (box c lands rows * 128 bytes after box
// c - 1), 1 = one dense box.  (col, row, z) = origin of the tile in the [matrices][rows][cols] view.
__device__ __forceinline__ void issue_tile_boxes(uint32_t dst, CUtensorMap const *map, int form, int rows, int cols, int col,
                                                 int row, int z, uint32_t bar, int lane) {
  if (form == 2) {
    for (int c = lane; c < (cols >> 6); c += 32)
      ptx::tma_load_3d(dst + (uint32_t)(c * rows * 128), map, bar, col + 64 * c, row, z);
  } else if (lane == 0) {
    ptx::tma_load_3d(dst, map, bar, col, row, z);
  }
}

// One TMA-fetched input, resolved once per block: where its tile goes, where it comes from in the first iteration
// and how far every iteration moves it.  Issuing a stage then is a walk over a few of these records.
struct TileFetch {
  CUtensorMap const *map;  // tiled forms
  uint16_t const *first;   // row copies: first element of the tile in iteration 0
  int64_t dfirst;          //   elements every iteration adds
  uint32_t dst;            // shared address of the tile (stage 0)
  int32_t stage_stride;    // bytes to the same tile in the next ring stage (0: fetched once)
  int32_t form, rows, cols, pitch, ld;
  int32_t col, row, z, dcol, drow, dz;
  int32_t moving;
};

// Called by thread `oi` < num_ops for operator record `a` of an input in the TMA masks: fills fetch[slot in mask order].
__device__ __forceinline__ void resolve_fetch(TileFetch &f, int32_t const *a, TmaPlan const &tma, TmaMaps const &maps, int oi,
                                              void const *base, int64_t set_offset, int bx, int by, int bz, int pitch,
                                              unsigned char *smem_base) {
  int const row = bx * a[0] + by * a[1] + bz * a[2], col = bx * a[3] + by * a[4] + bz * a[5];
  int64_t const lead = (int64_t)bx * a[8] + (int64_t)by * a[9] + (int64_t)bz * a[10];
  int64_t const mat = (int64_t)a[12] * a[13];
  f.map = &maps.m[a[18]];
  f.first = static_cast<uint16_t const *>(base) + set_offset + lead + (size_t)row * a[13] + col;
  f.dfirst = (int64_t)a[6] * a[13] + a[7] + a[11];
  f.moving = (int)((tma.moving_mask >> oi) & 1u);
  f.dst = ptx::smem_u32(smem_base + a[17]);
  f.stage_stride = f.moving ? tma.ring_bytes : 0;
  f.form = ((tma.swizzled_mask >> oi) & 1u) ? 2 : (int)((tma.tiled_mask >> oi) & 1u);
  f.rows = a[14]; f.cols = a[15]; f.pitch = pitch; f.ld = a[13];
  f.col = col; f.row = row; f.dcol = a[7]; f.drow = a[6];
  f.z = f.form ? (int)((set_offset + lead) / mat) : 0;
  f.dz = f.form ? (int)(a[11] / mat) : 0;
}

// Requests iteration `it` of every resolved input with `moving` == want_moving into ring stage `stage`, completing on
// `bar` after `tx` bytes; called by all lanes of one warp.
__device__ __forceinline__ void issue_fetches(TileFetch const *fetch, int n, int want_moving, int it, int stage, uint32_t bar,
                                              int tx, int lane) {
  if (lane == 0) ptx::mbar_expect_tx(bar, (uint32_t)tx);
  __syncwarp();
  for (int i = 0; i < n; i++) {
    TileFetch const &f = fetch[i];
    if (f.moving != want_moving) continue;
    uint32_t const dst = f.dst + (uint32_t)(stage * f.stage_stride);
    if (f.form) issue_tile_boxes(dst, f.map, f.form, f.rows, f.cols, f.col + it * f.dcol, f.row + it * f.drow, f.z + it * f.dz, bar, lane);
    else issue_tile_rows(dst, f.first + it * f.dfirst, f.rows, f.cols, f.pitch, f.ld, bar, lane);
  }
}

// Issue the row copies of one 16-bit input tile; the lanes of the calling warp split the rows.
// `dst` = shared address of the tile (of the right stage), `pitch` / `ld` in elements.
__device__ __forceinline__ void issue_tile_rows(uint32_t dst, uint16_t const *first, int rows, int cols, int pitch, int ld,
                                                uint32_t bar, int lane) {
  for (int r = lane; r < rows; r += 32)
    bulk_load_row(dst + (uint32_t)(r * pitch * 2), first + (size_t)r * ld, (uint32_t)(cols * 2), bar);
}
#endif

} // namespace interp
} // namespace mgk
