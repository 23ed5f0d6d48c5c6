// Host-side matcher from a lowered threadblock program to the specialised sm_100a kernels.
// A program that matches no pattern runs on the generic interpreters.
#pragma once
#include "mugraph_device.h"
namespace mg {
enum KernelId {
  KERNEL_INTERPRETER = 0,  // generic interpreter (any valid graph)
  KERNEL_ATTN_SPLIT = 1,   // S=QK, E=exp(S), O'=EV, R'=rowsum(E) summed over the for-loop, per KV split
  KERNEL_ATTN_MERGE = 2,   // O = sum_splits(O_part) / sum_splits(R_part)
  KERNEL_ATTN_ROWS = 3,    // same chain with query rows split over grid.y and the whole KV axis in the for-loop
  KERNEL_MATMUL_CHAIN = 4, // out = sum over the for-loop of (X_i W1_i) W2, W2 loop-invariant
  KERNEL_TILE_REDUCE = 5,  // one threadblock reduction between an input and an output, for-loop of one
};
// Recognise the split-KV attention operator (pattern of the reference's
// cpp_examples/group_query_attn_inc_decode.cc:46-79); fills `out` on success.  The second matmul and the row
// reduction may come in either order; *o_output = which of the operator's two outputs (0 or 1) is O'.
bool match_attn_split(mgd_program const &p, mgd_attn_split *out, int *o_output);
// Recognise the cross-split reduction + division (same file, :80-103); *o_part_input = which input is O_part.
bool match_attn_merge(mgd_program const &p, mgd_attn_merge *out, int *o_part_input);
// Recognise the dense (prefill) form: pattern of cpp_examples/multi_head_attn_prefill.cc:43-98.
bool match_attn_rows(mgd_program const &p, mgd_attn_rows *out, int *o_output);
// Recognise O = A / R with A[heads, rows, d], R[heads, rows, 1] tiled like match_attn_rows' outputs (same example,
// :88-98); *numerator_input = which input is A.
bool match_div_rows(mgd_program const &p, int *heads, int *rows, int *d, int *numerator_input);
// Recognise two chained matmuls whose result an output operator accumulates over the for-loop, with a
// loop-invariant right operand of the second one (pattern of cpp_examples/mlp.cc's fused block).
bool match_matmul_chain(mgd_program const &p, mgd_matmul_chain *out);
// Recognise input -> reduction -> output with a for-loop of one (the cross-block sums behind a split operator).
bool match_tile_reduce(mgd_program const &p, mgd_tile_reduce *out);
} // namespace mg
