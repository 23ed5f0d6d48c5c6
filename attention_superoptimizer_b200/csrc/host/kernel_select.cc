// Matches a lowered threadblock program against the operator patterns the specialised sm_100a kernels implement.
// The records are read through typed views whose accessors carry the slot names of mugraph_device.h, so a change
// of the record layout is a change of one enum there.
#include "kernel_select.h"
#include "mugraph.h"
#include <cstring>
#include <initializer_list>

namespace mg {
namespace {
constexpr int kInputOp = 2001, kOutputOp = 2002; // TB_INPUT_OP, TB_OUTPUT_OP

struct InputView {
  mgd_op const &o;
  bool valid() const { return o.type == kInputOp; }
  int row_block_stride(int axis) const { return o.a[MGD_IN_ROW_BLOCK_STRIDE + axis]; }
  int col_block_stride(int axis) const { return o.a[MGD_IN_COL_BLOCK_STRIDE + axis]; }
  int lead_block_stride(int axis) const { return o.a[MGD_IN_LEAD_BLOCK_STRIDE + axis]; }
  int row_loop_stride() const { return o.a[MGD_IN_ROW_LOOP_STRIDE]; }
  int col_loop_stride() const { return o.a[MGD_IN_COL_LOOP_STRIDE]; }
  int lead_loop_stride() const { return o.a[MGD_IN_LEAD_LOOP_STRIDE]; }
  int rows() const { return o.a[MGD_IN_ROWS]; }
  int cols() const { return o.a[MGD_IN_COLS]; }
  int tile_rows() const { return o.a[MGD_IN_TILE_ROWS]; }
  int tile_cols() const { return o.a[MGD_IN_TILE_COLS]; }
  int layout() const { return o.a[MGD_IN_LAYOUT]; }
  int tile_offset() const { return o.a[MGD_IN_TILE_OFFSET]; }
  int slot() const { return o.a[MGD_IN_SLOT]; }
  // grid.x walks the leading (head) dimension one matrix at a time and nothing else; grid.z is unused
  bool head_on_x() const {
    return lead_block_stride(0) == rows() * cols() && lead_block_stride(1) == 0 && lead_block_stride(2) == 0 &&
           lead_loop_stride() == 0 && row_block_stride(0) == 0 && col_block_stride(0) == 0 && row_block_stride(2) == 0 &&
           col_block_stride(2) == 0;
  }
  bool y_and_loop_untouched() const {
    return row_block_stride(1) == 0 && col_block_stride(1) == 0 && row_loop_stride() == 0 && col_loop_stride() == 0;
  }
  // grid.y picks a run of `forloop_range` row tiles and the for-loop walks them
  bool rows_split_by_y_and_loop(int forloop_range) const {
    return row_block_stride(1) == tile_rows() * forloop_range && row_loop_stride() == tile_rows() &&
           col_block_stride(1) == 0 && col_loop_stride() == 0;
  }
  bool cols_split_by_y_and_loop(int forloop_range) const {
    return col_block_stride(1) == tile_cols() * forloop_range && col_loop_stride() == tile_cols() &&
           row_block_stride(1) == 0 && row_loop_stride() == 0;
  }
  bool whole_matrix_per_block() const { return rows() == tile_rows() && cols() == tile_cols(); }
};

struct OutputView {
  mgd_op const &o;
  bool valid() const { return o.type == kOutputOp; }
  int row_block_stride(int axis) const { return o.a[MGD_OUT_ROW_BLOCK_STRIDE + axis]; }
  int col_block_stride(int axis) const { return o.a[MGD_OUT_COL_BLOCK_STRIDE + axis]; }
  int lead_block_stride(int axis) const { return o.a[MGD_OUT_LEAD_BLOCK_STRIDE + axis]; }
  int rows() const { return o.a[MGD_OUT_ROWS]; }
  int cols() const { return o.a[MGD_OUT_COLS]; }
  int tile_rows() const { return o.a[MGD_OUT_TILE_ROWS]; }
  int tile_cols() const { return o.a[MGD_OUT_TILE_COLS]; }
  int source_offset() const { return o.a[MGD_OUT_SOURCE_OFFSET]; }
  int slot() const { return o.a[MGD_OUT_SLOT]; }
  // one [rows x cols] matrix per head (grid.x); `row_y` / `col_y` = how far grid.y moves the tile; z unused
  bool placed(int tile_r, int tile_c, int all_rows, int all_cols, int row_y, int col_y) const {
    return tile_rows() == tile_r && tile_cols() == tile_c && rows() == all_rows && cols() == all_cols &&
           lead_block_stride(0) == all_rows * all_cols && lead_block_stride(1) == 0 && lead_block_stride(2) == 0 &&
           row_block_stride(0) == 0 && row_block_stride(1) == row_y && row_block_stride(2) == 0 &&
           col_block_stride(0) == 0 && col_block_stride(1) == col_y && col_block_stride(2) == 0;
  }
};

struct MatmulView {
  mgd_op const &o;
  bool valid() const { return o.type == MG_TB_MATMUL_OP; }
  int m() const { return o.a[MGD_MM_M]; }
  int n() const { return o.a[MGD_MM_N]; }
  int k() const { return o.a[MGD_MM_K]; }
  int a_offset() const { return o.a[MGD_MM_A_OFFSET]; }
  int b_offset() const { return o.a[MGD_MM_B_OFFSET]; }
  int c_offset() const { return o.a[MGD_MM_C_OFFSET]; }
  bool is(int mm, int nn, int kk, int a_off, int b_off) const {
    return m() == mm && n() == nn && k() == kk && a_offset() == a_off && b_offset() == b_off;
  }
};

struct ExpView {
  mgd_op const &o;
  bool valid() const { return o.type == MG_TB_EXP_OP; }
  int offset() const { return o.a[MGD_EXP_OFFSET]; }
  int elements() const { return o.a[MGD_EXP_ELEMENTS]; }
};

struct ReductionView {
  mgd_op const &o;
  bool plain() const { return o.type >= MG_TB_REDUCTION_0_OP && o.type <= MG_TB_REDUCTION_2_OP; }
  bool to_dimx() const { return o.type >= MG_TB_REDUCTION_0_TO_DIMX_OP && o.type <= MG_TB_REDUCTION_2_TO_DIMX_OP; }
  int out_elements() const { return o.a[MGD_RED_OUT_ELEMENTS]; }
  int degree() const { return o.a[MGD_RED_DEGREE]; }
  int inner() const { return o.a[MGD_RED_INNER]; }
  int in_offset() const { return o.a[MGD_RED_IN_OFFSET]; }
  int out_offset() const { return o.a[MGD_RED_OUT_OFFSET]; }
  bool is(int out_n, int deg, int inner_range, int in_off) const {
    return out_elements() == out_n && degree() == deg && inner() == inner_range && in_offset() == in_off;
  }
};

struct DivView {
  mgd_op const &o;
  bool valid() const { return o.type == MG_TB_DIV_OP; }
  int x_shape(int i) const { return o.a[MGD_BIN_X_SHAPE + i]; }
  int y_shape(int i) const { return o.a[MGD_BIN_Y_SHAPE + i]; }
  int x_offset() const { return o.a[MGD_BIN_X_OFFSET]; }
  int y_offset() const { return o.a[MGD_BIN_Y_OFFSET]; }
  int out_offset() const { return o.a[MGD_BIN_OUT_OFFSET]; }
  // [1, m, d] / [1, m, 1]
  bool rows_by_column(int m, int d) const {
    return x_shape(0) == 1 && x_shape(1) == m && x_shape(2) == d && y_shape(0) == 1 && y_shape(1) == m && y_shape(2) == 1;
  }
};

// The chain S = Q K, E = exp(S) in place, O' = E V, R' = rowsum(E) over inputs 0..2 and operators 3..6; the last
// two may come in either order (searched candidates put the reduction first).  Fills the common sizes and says
// which of the two output operators (7, 8) stores O'.
struct Chain {
  int m, d, tile_kv, o_output; // o_output: 0 when the first output operator stores O', 1 when the second does
};
bool match_chain(mgd_program const &p, Chain *c) {
  if (p.num_ops != 9 || p.num_inputs != 3 || p.num_outputs != 2 || p.grid[2] != 1) return false;
  InputView q{p.ops[0]}, k{p.ops[1]}, v{p.ops[2]};
  MatmulView s{p.ops[3]};
  ExpView e{p.ops[4]};
  if (!q.valid() || !k.valid() || !v.valid() || !s.valid() || !e.valid()) return false;
  bool const reduction_first = ReductionView{p.ops[5]}.plain();
  MatmulView o{p.ops[reduction_first ? 6 : 5]};
  ReductionView r{p.ops[reduction_first ? 5 : 6]};
  OutputView out0{p.ops[7]}, out1{p.ops[8]};
  if (!o.valid() || !r.plain() || !out0.valid() || !out1.valid()) return false;
  int const m = q.tile_rows(), d = q.tile_cols(), tkv = k.tile_cols();
  if (!s.is(m, tkv, d, q.tile_offset(), k.tile_offset())) return false;
  if (e.offset() != s.c_offset() || e.elements() != m * tkv) return false;
  if (!o.is(m, d, tkv, s.c_offset(), v.tile_offset())) return false;
  if (!r.is(m, tkv, 1, s.c_offset())) return false;
  // which output operator stores which result
  int o_output;
  if (out0.source_offset() == o.c_offset() && out1.source_offset() == r.out_offset()) o_output = 0;
  else if (out1.source_offset() == o.c_offset() && out0.source_offset() == r.out_offset()) o_output = 1;
  else return false;
  c->m = m; c->d = d; c->tile_kv = tkv; c->o_output = o_output;
  return true;
}
} // namespace

bool match_attn_split(mgd_program const &p, mgd_attn_split *out, int *o_output) {
  Chain c;
  if (!match_chain(p, &c)) return false;
  InputView q{p.ops[0]}, k{p.ops[1]}, v{p.ops[2]};
  int const heads = p.grid[0], splits = p.grid[1], fr = p.forloop_range, m = c.m, d = c.d, tkv = c.tile_kv;
  if (!q.head_on_x() || !k.head_on_x() || !v.head_on_x()) return false;
  // Q: the whole [m, d] matrix of a head in every block; K[d, kv]: columns split; V[kv, d]: rows split
  if (!q.y_and_loop_untouched() || !q.whole_matrix_per_block()) return false;
  if (!k.cols_split_by_y_and_loop(fr) || k.tile_rows() != d || k.rows() != d) return false;
  if (!v.rows_split_by_y_and_loop(fr) || v.tile_rows() != tkv || v.tile_cols() != d || v.cols() != d) return false;
  int const kv_len = k.cols();
  if (v.rows() != kv_len || kv_len != tkv * fr * splits) return false;
  // O' tile [m, d] at column block y * d of [heads, m, splits * d]; R' [m, 1] at column y of [heads, m, splits]
  OutputView oo{p.ops[7 + c.o_output]}, ro{p.ops[8 - c.o_output]};
  if (!oo.placed(m, d, m, splits * d, 0, d) || !ro.placed(m, 1, m, splits, 0, 1)) return false;
  std::memset(out, 0, sizeof(*out));
  out->heads = heads; out->m = m; out->d = d; out->kv_len = kv_len;
  out->splits = splits; out->forloop_range = fr;
  out->k_layout = k.layout(); out->v_layout = v.layout();
  out->num_sets = 1;
  if (o_output) *o_output = c.o_output;
  return true;
}

bool match_attn_rows(mgd_program const &p, mgd_attn_rows *out, int *o_output) {
  Chain c;
  if (!match_chain(p, &c)) return false;
  InputView q{p.ops[0]}, k{p.ops[1]}, v{p.ops[2]};
  int const fr = p.forloop_range, gy = p.grid[1], m = c.m, d = c.d, tkv = c.tile_kv;
  if (!q.head_on_x() || !k.head_on_x() || !v.head_on_x()) return false;
  // Q: rows tiled by grid.y only; K[d, kv]: columns tiled by the for-loop only; V[kv, d]: rows by the for-loop only
  if (q.row_block_stride(1) != m || q.col_block_stride(1) != 0 || q.row_loop_stride() != 0 || q.col_loop_stride() != 0 ||
      q.rows() != m * gy || q.cols() != d)
    return false;
  if (k.row_block_stride(1) != 0 || k.col_block_stride(1) != 0 || k.row_loop_stride() != 0 || k.col_loop_stride() != tkv ||
      k.tile_rows() != d || k.rows() != d || k.cols() != tkv * fr)
    return false;
  if (v.row_block_stride(1) != 0 || v.col_block_stride(1) != 0 || v.col_loop_stride() != 0 || v.row_loop_stride() != tkv ||
      v.tile_rows() != tkv || v.tile_cols() != d || v.cols() != d || v.rows() != tkv * fr)
    return false;
  OutputView oo{p.ops[7 + c.o_output]}, ro{p.ops[8 - c.o_output]};
  if (!oo.placed(m, d, m * gy, d, m, 0) || !ro.placed(m, 1, m * gy, 1, m, 0)) return false;
  std::memset(out, 0, sizeof(*out));
  out->heads = p.grid[0]; out->seq_q = m * gy; out->d = d; out->kv_len = tkv * fr;
  out->tile_m = m; out->tile_kv = tkv; out->forloop_range = fr;
  out->k_layout = k.layout(); out->v_layout = v.layout();
  if (o_output) *o_output = c.o_output;
  return true;
}

bool match_div_rows(mgd_program const &p, int *heads, int *rows, int *d, int *numerator_input) {
  if (p.num_ops != 4 || p.num_inputs != 2 || p.num_outputs != 1 || p.grid[2] != 1 || p.forloop_range != 1) return false;
  InputView in0{p.ops[0]}, in1{p.ops[1]};
  DivView div{p.ops[2]};
  OutputView out{p.ops[3]};
  if (!in0.valid() || !in1.valid() || !div.valid() || !out.valid()) return false;
  // the numerator is the input the division reads as x; the other one holds one value per row
  int num;
  if (div.x_offset() == in0.tile_offset() && div.y_offset() == in1.tile_offset()) num = 0;
  else if (div.x_offset() == in1.tile_offset() && div.y_offset() == in0.tile_offset()) num = 1;
  else return false;
  InputView a = num == 0 ? in0 : in1, r = num == 0 ? in1 : in0;
  int const m = a.tile_rows(), dd = a.tile_cols(), gy = p.grid[1];
  if (r.tile_rows() != m || r.tile_cols() != 1 || a.cols() != dd || r.cols() != 1) return false;
  for (InputView const &in : {a, r}) {
    if (!in.head_on_x() || in.rows() != m * gy) return false;
    if (in.row_block_stride(1) != m || in.col_block_stride(1) != 0 || in.row_loop_stride() != 0 || in.col_loop_stride() != 0)
      return false;
  }
  if (!div.rows_by_column(m, dd)) return false;
  if (out.source_offset() != div.out_offset() || !out.placed(m, dd, m * gy, dd, m, 0)) return false;
  *heads = p.grid[0]; *rows = m * gy; *d = dd;
  if (numerator_input) *numerator_input = num;
  return true;
}

bool match_attn_merge(mgd_program const &p, mgd_attn_merge *out, int *o_part_input) {
  // ops: two inputs, reduction_to_dimx(O_part), reduction(R_part) (either order), div, output
  if (p.num_ops != 6 || p.num_inputs != 2 || p.num_outputs != 1) return false;
  if (p.grid[1] != 1 || p.grid[2] != 1 || p.forloop_range != 1) return false;
  InputView in0{p.ops[0]}, in1{p.ops[1]};
  DivView div{p.ops[4]};
  OutputView so{p.ops[5]};
  if (!in0.valid() || !in1.valid() || !div.valid() || !so.valid()) return false;
  bool const wide_first = ReductionView{p.ops[2]}.to_dimx();
  ReductionView wide{p.ops[wide_first ? 2 : 3]}, narrow{p.ops[wide_first ? 3 : 2]};
  if (!wide.to_dimx() || !narrow.plain()) return false;
  int o_in;
  if (wide.in_offset() == in0.tile_offset() && narrow.in_offset() == in1.tile_offset()) o_in = 0;
  else if (wide.in_offset() == in1.tile_offset() && narrow.in_offset() == in0.tile_offset()) o_in = 1;
  else return false;
  InputView op = o_in == 0 ? in0 : in1, rp = o_in == 0 ? in1 : in0;
  int const m = op.tile_rows(), width = op.tile_cols(), splits = rp.tile_cols();
  if (rp.tile_rows() != m || splits <= 0 || width % splits != 0) return false;
  int const d = width / splits;
  for (InputView const &in : {op, rp})
    if (!in.whole_matrix_per_block() || !in.head_on_x() || !in.y_and_loop_untouched()) return false;
  // sum over the splits: [m, splits * d] -> [m, d] (stride d), [m, splits] -> [m, 1]; then the division
  if (!wide.is(m * d, splits, d, op.tile_offset()) || !narrow.is(m, splits, 1, rp.tile_offset())) return false;
  if (div.x_offset() != wide.out_offset() || div.y_offset() != narrow.out_offset() || !div.rows_by_column(m, d)) return false;
  if (so.source_offset() != div.out_offset() || !so.placed(m, d, m, d, 0, 0)) return false;
  std::memset(out, 0, sizeof(*out));
  out->heads = p.grid[0]; out->m = m; out->d = d; out->splits = splits; out->num_sets = 1;
  if (o_part_input) *o_part_input = o_in;
  return true;
}
bool match_matmul_chain(mgd_program const &p, mgd_matmul_chain *out) {
  // ops: three inputs, matmul(in_a, in_b) -> t, matmul(t, in_c) -> u, output(u)
  if (p.num_ops != 6 || p.num_inputs != 3 || p.num_outputs != 1) return false;
  InputView in[3] = {InputView{p.ops[0]}, InputView{p.ops[1]}, InputView{p.ops[2]}};
  MatmulView first{p.ops[3]}, second{p.ops[4]};
  OutputView so{p.ops[5]};
  if (!in[0].valid() || !in[1].valid() || !in[2].valid() || !first.valid() || !second.valid() || !so.valid()) return false;
  auto input_at = [&](int offset) {
    for (int i = 0; i < 3; i++)
      if (in[i].tile_offset() == offset) return i;
    return -1;
  };
  int const ix = input_at(first.a_offset()), iw1 = input_at(first.b_offset()), iw2 = input_at(second.b_offset());
  if (ix < 0 || iw1 < 0 || iw2 < 0 || ix == iw1 || ix == iw2 || iw1 == iw2) return false;
  if (second.a_offset() != first.c_offset() || so.source_offset() != second.c_offset()) return false;
  int const m = first.m(), n1 = first.n(), kt = first.k(), n2 = second.n();
  if (second.m() != m || second.k() != n1) return false;
  if (in[ix].tile_rows() != m || in[ix].tile_cols() != kt || in[iw1].tile_rows() != kt || in[iw1].tile_cols() != n1 ||
      in[iw2].tile_rows() != n1 || in[iw2].tile_cols() != n2)
    return false;
  mgd_op const &w2 = p.ops[iw2];
  if (w2.a[MGD_IN_ROW_LOOP_STRIDE] != 0 || w2.a[MGD_IN_COL_LOOP_STRIDE] != 0 || w2.a[MGD_IN_LEAD_LOOP_STRIDE] != 0) return false;
  if (p.ops[5].a[MGD_OUT_TILE_ROWS] != m || p.ops[5].a[MGD_OUT_TILE_COLS] != n2) return false;
  std::memset(out, 0, sizeof(*out));
  for (int i = 0; i < 3; i++) out->grid[i] = p.grid[i];
  out->forloop_range = p.forloop_range;
  out->m = m; out->kt = kt; out->n1 = n1; out->n2 = n2;
  out->x = p.ops[ix]; out->w1 = p.ops[iw1]; out->w2 = w2; out->out = p.ops[5];
  return true;
}
bool match_tile_reduce(mgd_program const &p, mgd_tile_reduce *out) {
  if (p.num_ops != 3 || p.num_inputs != 1 || p.num_outputs != 1 || p.forloop_range != 1) return false;
  InputView in{p.ops[0]};
  ReductionView red{p.ops[1]};
  OutputView so{p.ops[2]};
  if (!in.valid() || !(red.plain() || red.to_dimx()) || !so.valid()) return false;
  if (red.in_offset() != in.tile_offset() || so.source_offset() != red.out_offset()) return false;
  if (red.out_elements() != so.tile_rows() * so.tile_cols()) return false;
  if ((long long)red.out_elements() * red.degree() != (long long)in.tile_rows() * in.tile_cols()) return false;
  std::memset(out, 0, sizeof(*out));
  for (int i = 0; i < 3; i++) out->grid[i] = p.grid[i];
  out->out_elements = red.out_elements(); out->degree = red.degree(); out->inner = red.inner();
  out->in = p.ops[0]; out->out = p.ops[2];
  return true;
}
} // namespace mg
