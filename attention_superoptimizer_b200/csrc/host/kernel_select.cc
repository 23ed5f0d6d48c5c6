#include "kernel_select.h"
#include "mugraph.h"
#include <cstring>

namespace mg {
namespace {
bool is_input(mgd_op const &o) { return o.type == 2001; }
bool is_output(mgd_op const &o) { return o.type == 2002; }
// An input whose tile is selected by blockIdx.x along the leading (head) dimension only,
// optionally tiled along rows or columns by blockIdx.y and the for-loop.
struct InputShape {
  bool ok;
  int tile_rows, tile_cols, rows, cols;
  bool split_rows, split_cols; // grid.y + for-loop walk this dim
};
InputShape classify(mgd_op const &o, int forloop_range, int lead_elems_expected) {
  InputShape s{};
  s.tile_rows = o.a[14]; s.tile_cols = o.a[15]; s.rows = o.a[12]; s.cols = o.a[13];
  bool head_on_x = o.a[8] == lead_elems_expected && o.a[9] == 0 && o.a[10] == 0 && o.a[11] == 0;
  bool x_clean = o.a[0] == 0 && o.a[3] == 0 && o.a[2] == 0 && o.a[5] == 0; // x,z do not move rows/cols
  s.split_rows = o.a[1] == s.tile_rows * forloop_range && o.a[6] == s.tile_rows && o.a[4] == 0 && o.a[7] == 0;
  s.split_cols = o.a[4] == s.tile_cols * forloop_range && o.a[7] == s.tile_cols && o.a[1] == 0 && o.a[6] == 0;
  bool whole = o.a[1] == 0 && o.a[4] == 0 && o.a[6] == 0 && o.a[7] == 0;
  s.ok = head_on_x && x_clean && (s.split_rows || s.split_cols || whole);
  if (whole) s.split_rows = s.split_cols = false;
  return s;
}
} // namespace

bool match_attn_split(mgd_program const &p, int, mgd_attn_split *out) {
  // ops: in Q, in K, in V, matmul(Q,K)->S, exp(S), matmul(E,V)->O', reduction(E)->R', out O', out R'
  if (p.num_ops != 9 || p.num_inputs != 3 || p.num_outputs != 2 || p.grid[2] != 1) return false;
  mgd_op const *o = p.ops;
  if (!is_input(o[0]) || !is_input(o[1]) || !is_input(o[2])) return false;
  if (o[3].type != MG_TB_MATMUL_OP || o[4].type != MG_TB_EXP_OP || o[5].type != MG_TB_MATMUL_OP) return false;
  if (o[6].type != MG_TB_REDUCTION_0_OP && o[6].type != MG_TB_REDUCTION_1_OP && o[6].type != MG_TB_REDUCTION_2_OP)
    return false;
  if (!is_output(o[7]) || !is_output(o[8])) return false;
  int m = o[0].a[14], d = o[0].a[15], tkv = o[1].a[15];
  int heads = p.grid[0], splits = p.grid[1], fr = p.forloop_range;
  InputShape q = classify(o[0], fr, o[0].a[12] * o[0].a[13]);
  InputShape k = classify(o[1], fr, o[1].a[12] * o[1].a[13]);
  InputShape v = classify(o[2], fr, o[2].a[12] * o[2].a[13]);
  if (!q.ok || !k.ok || !v.ok) return false;
  if (q.split_rows || q.split_cols || q.rows != m || q.cols != d) return false;
  if (!k.split_cols || k.tile_rows != d || k.rows != d) return false;
  if (!v.split_rows || v.tile_rows != tkv || v.tile_cols != d || v.cols != d) return false;
  int kv_len = k.cols;
  if (v.rows != kv_len || kv_len != tkv * fr * splits) return false;
  // dataflow: S = Q K in o[3]; exp in place on S; O' = E V; R' = row sums of E (last dim)
  if (o[3].a[0] != m || o[3].a[1] != tkv || o[3].a[2] != d) return false;
  if (o[3].a[3] != o[0].a[17] || o[3].a[4] != o[1].a[17]) return false;
  if (o[4].a[0] != o[3].a[5] || o[4].a[1] != m * tkv) return false;
  if (o[5].a[0] != m || o[5].a[1] != d || o[5].a[2] != tkv) return false;
  if (o[5].a[3] != o[3].a[5] || o[5].a[4] != o[2].a[17]) return false;
  if (o[6].a[3] != o[3].a[5] || o[6].a[0] != m || o[6].a[1] != tkv || o[6].a[2] != 1) return false;
  // outputs: O' tile [m,d] placed at column block y*d of [heads, m, splits*d]; R' [m,1] at column y
  if (o[7].a[13] != o[5].a[5] || o[8].a[13] != o[6].a[4]) return false;
  if (o[7].a[11] != m || o[7].a[12] != d || o[7].a[9] != m || o[7].a[10] != splits * d) return false;
  if (o[8].a[11] != m || o[8].a[12] != 1 || o[8].a[9] != m || o[8].a[10] != splits) return false;
  if (o[7].a[6] != m * splits * d || o[7].a[4] != d || o[7].a[0] || o[7].a[1] || o[7].a[2] || o[7].a[3] ||
      o[7].a[5] || o[7].a[7] || o[7].a[8])
    return false;
  if (o[8].a[6] != m * splits || o[8].a[4] != 1 || o[8].a[0] || o[8].a[1] || o[8].a[2] || o[8].a[3] ||
      o[8].a[5] || o[8].a[7] || o[8].a[8])
    return false;
  std::memset(out, 0, sizeof(*out));
  out->heads = heads; out->m = m; out->d = d; out->kv_len = kv_len;
  out->splits = splits; out->forloop_range = fr;
  out->k_layout = o[1].a[16]; out->v_layout = o[2].a[16];
  out->num_sets = 1;
  return true;
}

bool match_attn_rows(mgd_program const &p, mgd_attn_rows *out) {
  if (p.num_ops != 9 || p.num_inputs != 3 || p.num_outputs != 2 || p.grid[2] != 1) return false;
  mgd_op const *o = p.ops;
  if (!is_input(o[0]) || !is_input(o[1]) || !is_input(o[2])) return false;
  if (o[3].type != MG_TB_MATMUL_OP || o[4].type != MG_TB_EXP_OP || o[5].type != MG_TB_MATMUL_OP) return false;
  if (o[6].type != MG_TB_REDUCTION_0_OP && o[6].type != MG_TB_REDUCTION_1_OP && o[6].type != MG_TB_REDUCTION_2_OP)
    return false;
  if (!is_output(o[7]) || !is_output(o[8])) return false;
  int m = o[0].a[14], d = o[0].a[15], tkv = o[1].a[15], fr = p.forloop_range, gy = p.grid[1];
  auto head_only = [](mgd_op const &in) {
    return in.a[8] == in.a[12] * in.a[13] && in.a[9] == 0 && in.a[10] == 0 && in.a[11] == 0 && in.a[0] == 0 &&
           in.a[2] == 0 && in.a[3] == 0 && in.a[5] == 0;
  };
  if (!head_only(o[0]) || !head_only(o[1]) || !head_only(o[2])) return false;
  // Q: rows tiled by grid.y only
  if (o[0].a[1] != m || o[0].a[4] || o[0].a[6] || o[0].a[7] || o[0].a[12] != m * gy || o[0].a[13] != d) return false;
  // K[d, kv]: columns tiled by the for-loop only;  V[kv, d]: rows tiled by the for-loop only
  if (o[1].a[1] || o[1].a[4] || o[1].a[6] || o[1].a[7] != tkv || o[1].a[14] != d || o[1].a[12] != d || o[1].a[13] != tkv * fr) return false;
  if (o[2].a[1] || o[2].a[4] || o[2].a[7] || o[2].a[6] != tkv || o[2].a[14] != tkv || o[2].a[15] != d || o[2].a[13] != d ||
      o[2].a[12] != tkv * fr)
    return false;
  if (o[3].a[0] != m || o[3].a[1] != tkv || o[3].a[2] != d || o[3].a[3] != o[0].a[17] || o[3].a[4] != o[1].a[17]) return false;
  if (o[4].a[0] != o[3].a[5] || o[4].a[1] != m * tkv) return false;
  if (o[5].a[0] != m || o[5].a[1] != d || o[5].a[2] != tkv || o[5].a[3] != o[3].a[5] || o[5].a[4] != o[2].a[17]) return false;
  if (o[6].a[3] != o[3].a[5] || o[6].a[0] != m || o[6].a[1] != tkv || o[6].a[2] != 1) return false;
  if (o[7].a[13] != o[5].a[5] || o[8].a[13] != o[6].a[4]) return false;
  // outputs: rows placed by grid.y, heads by grid.x
  if (o[7].a[11] != m || o[7].a[12] != d || o[7].a[9] != m * gy || o[7].a[10] != d || o[7].a[1] != m || o[7].a[6] != m * gy * d ||
      o[7].a[0] || o[7].a[2] || o[7].a[3] || o[7].a[4] || o[7].a[5] || o[7].a[7] || o[7].a[8])
    return false;
  if (o[8].a[11] != m || o[8].a[12] != 1 || o[8].a[9] != m * gy || o[8].a[10] != 1 || o[8].a[1] != m || o[8].a[6] != m * gy ||
      o[8].a[0] || o[8].a[2] || o[8].a[3] || o[8].a[4] || o[8].a[5] || o[8].a[7] || o[8].a[8])
    return false;
  std::memset(out, 0, sizeof(*out));
  out->heads = p.grid[0]; out->seq_q = m * gy; out->d = d; out->kv_len = tkv * fr;
  out->tile_m = m; out->tile_kv = tkv; out->forloop_range = fr;
  out->k_layout = o[1].a[16]; out->v_layout = o[2].a[16];
  return true;
}

bool match_div_rows(mgd_program const &p, int *heads, int *rows, int *d) {
  if (p.num_ops != 4 || p.num_inputs != 2 || p.num_outputs != 1 || p.grid[2] != 1 || p.forloop_range != 1) return false;
  mgd_op const *o = p.ops;
  if (!is_input(o[0]) || !is_input(o[1]) || o[2].type != MG_TB_DIV_OP || !is_output(o[3])) return false;
  int m = o[0].a[14], dd = o[0].a[15], gy = p.grid[1];
  if (o[1].a[14] != m || o[1].a[15] != 1) return false;
  for (int i = 0; i < 2; i++) {
    mgd_op const &in = o[i];
    if (in.a[8] != in.a[12] * in.a[13] || in.a[9] || in.a[10] || in.a[11]) return false;
    if (in.a[1] != m || in.a[0] || in.a[2] || in.a[3] || in.a[4] || in.a[5] || in.a[6] || in.a[7]) return false;
    if (in.a[12] != m * gy) return false;
  }
  if (o[0].a[13] != dd || o[1].a[13] != 1) return false;
  if (o[2].a[6] != o[0].a[17] || o[2].a[7] != o[1].a[17]) return false;
  if (o[2].a[0] != 1 || o[2].a[1] != m || o[2].a[2] != dd || o[2].a[3] != 1 || o[2].a[4] != m || o[2].a[5] != 1) return false;
  mgd_op const &so = o[3];
  if (so.a[13] != o[2].a[8] || so.a[11] != m || so.a[12] != dd || so.a[9] != m * gy || so.a[10] != dd || so.a[1] != m ||
      so.a[6] != m * gy * dd || so.a[0] || so.a[2] || so.a[3] || so.a[4] || so.a[5] || so.a[7] || so.a[8])
    return false;
  *heads = p.grid[0]; *rows = m * gy; *d = dd;
  return true;
}

bool match_attn_merge(mgd_program const &p, mgd_attn_merge *out) {
  // ops: in O_part, in R_part, reduction_to_dimx(O_part), reduction(R_part), div, out
  if (p.num_ops != 6 || p.num_inputs != 2 || p.num_outputs != 1) return false;
  if (p.grid[1] != 1 || p.grid[2] != 1 || p.forloop_range != 1) return false;
  mgd_op const *o = p.ops;
  if (!is_input(o[0]) || !is_input(o[1]) || !is_output(o[5])) return false;
  bool r0 = o[2].type >= MG_TB_REDUCTION_0_TO_DIMX_OP && o[2].type <= MG_TB_REDUCTION_2_TO_DIMX_OP;
  bool r1 = o[3].type >= MG_TB_REDUCTION_0_OP && o[3].type <= MG_TB_REDUCTION_2_OP;
  if (!r0 || !r1 || o[4].type != MG_TB_DIV_OP) return false;
  int m = o[0].a[14], wide = o[0].a[15], splits = o[1].a[15];
  if (o[1].a[14] != m || splits <= 0 || wide % splits != 0) return false;
  int d = wide / splits;
  for (int i = 0; i < 2; i++) {
    mgd_op const &in = o[i];
    if (in.a[12] != in.a[14] || in.a[13] != in.a[15]) return false; // whole matrix per block
    if (in.a[8] != in.a[12] * in.a[13] || in.a[9] || in.a[10] || in.a[11]) return false;
    for (int j = 0; j < 8; j++)
      if (in.a[j]) return false;
  }
  // reduction_to_dimx over the last dim: out [m,d], degree = splits, inner = d
  if (o[2].a[3] != o[0].a[17] || o[2].a[0] != m * d || o[2].a[1] != splits || o[2].a[2] != d) return false;
  if (o[3].a[3] != o[1].a[17] || o[3].a[0] != m || o[3].a[1] != splits || o[3].a[2] != 1) return false;
  if (o[4].a[6] != o[2].a[4] || o[4].a[7] != o[3].a[4]) return false;
  if (o[4].a[0] != 1 || o[4].a[1] != m || o[4].a[2] != d || o[4].a[3] != 1 || o[4].a[4] != m || o[4].a[5] != 1)
    return false;
  mgd_op const &so = o[5];
  if (so.a[13] != o[4].a[8] || so.a[11] != m || so.a[12] != d || so.a[9] != m || so.a[10] != d) return false;
  if (so.a[6] != m * d || so.a[0] || so.a[1] || so.a[2] || so.a[3] || so.a[4] || so.a[5] || so.a[7] || so.a[8])
    return false;
  std::memset(out, 0, sizeof(*out));
  out->heads = p.grid[0]; out->m = m; out->d = d; out->splits = splits; out->num_sets = 1;
  return true;
}
} // namespace mg
