// Host side of the threadblock graph: tile-shape inference, the shared-memory plan and the
// lowering into the flat kernel-level program.
//
// Behaviour follows the reference's builders (src/threadblock/{graph,input_loader,output,matmul,
// element_unary,element_binary,reduction,concat}.cc); conditions the reference asserts inside
// constructors are checked in the create_*_op functions here so that an invalid request yields
// nullptr instead of aborting.
#include "mirage/threadblock/graph.h"
#include "mugraph.h"
#include <algorithm>
#include <cassert>
#include <cstring>

namespace mirage {
namespace type {
size_t get_datatype_size(DataType t) {
  switch (t) {
    case DT_INT8: return 1;
    case DT_UINT16: case DT_BFLOAT16: case DT_FLOAT16: return 2;
    case DT_FLOAT32: return 4;
    case DT_DOUBLE: return 8;
    default: assert(false && "unknown element type"); return 0;
  }
}
char const *to_string(KNOperatorType t) {
  switch (t) {
    case KN_INPUT_OP: return "kn_input_op";
    case KN_MATMUL_OP: return "kn_matmul_op";
    case KN_REDUCTION_0_OP: return "kn_reduction_0_op";
    case KN_REDUCTION_1_OP: return "kn_reduction_1_op";
    case KN_REDUCTION_2_OP: return "kn_reduction_2_op";
    case KN_EXP_OP: return "kn_exp_op";
    case KN_ADD_OP: return "kn_add_op";
    case KN_MUL_OP: return "kn_mul_op";
    case KN_DIV_OP: return "kn_div_op";
    case KN_CUSTOMIZED_OP: return "kn_customized_op";
    default: return "kn_unkown";
  }
}
char const *to_string(TBOperatorType t) {
  switch (t) {
    case TB_INPUT_OP: return "tb_input_op";
    case TB_OUTPUT_OP: return "tb_output_op";
    case TB_MATMUL_OP: return "tb_matmul_op";
    case TB_EXP_OP: return "tb_exp_op";
    case TB_ADD_OP: return "tb_add_op";
    case TB_MUL_OP: return "tb_mul_op";
    case TB_DIV_OP: return "tb_div_op";
    case TB_REDUCTION_0_OP: return "tb_reduction_0_op";
    case TB_REDUCTION_1_OP: return "tb_reduction_1_op";
    case TB_REDUCTION_2_OP: return "tb_reduction_2_op";
    case TB_REDUCTION_0_TO_DIMX_OP: return "tb_reduction_0_to_dimx_op";
    case TB_REDUCTION_1_TO_DIMX_OP: return "tb_reduction_1_to_dimx_op";
    case TB_REDUCTION_2_TO_DIMX_OP: return "tb_reduction_2_to_dimx_op";
    case TB_CONCAT_0_OP: return "tb_concat_0_op";
    case TB_CONCAT_1_OP: return "tb_concat_1_op";
    case TB_CONCAT_2_OP: return "tb_concat_2_op";
    case TB_CUSTOMIZED_OP: return "tb_customized_op";
    default: return "tb_unkown";
  }
}
} // namespace type

namespace layout {
char const *to_string(DmemLayout l) {
  return l == DmemRowMajor ? "DmemRowMajor" : l == DmemColumnMajor ? "DmemColumnMajor" : "DmemUnknownLayout";
}
char const *to_string(SmemLayout l) {
  static char const *names[] = {"SmemRowMajor", "SmemColumnMajor",
                                "SmemRowMajorTensorOpMultiplicand_Crosswise16",
                                "SmemRowMajorTensorOpMultiplicand_Crosswise32",
                                "SmemRowMajorTensorOpMultiplicand_Crosswise64",
                                "SmemColumnMajorTensorOpMultiplicand_Crosswise16",
                                "SmemColumnMajorTensorOpMultiplicand_Crosswise32",
                                "SmemColumnMajorTensorOpMultiplicand_Crosswise64"};
  int i = (int)l - (int)SmemRowMajor;
  return (i >= 0 && i < 8) ? names[i] : "SmemUnknownLayout";
}
} // namespace layout

namespace threadblock {

using mirage::kernel::DTensor;
using namespace mirage::type;

int STensor::next_guid = 10000000;

STensor::STensor()
    : data_type(DT_UNKNOWN), layout(mirage::layout::SmemUnknownLayout), num_dims(0), guid(0), owner_op(nullptr),
      owner_ts_idx(-1000), smem_offset(128) {
  for (int &d : dim) d = 0;
}

bool STensor::operator==(STensor const &b) const {
  if (data_type != b.data_type || layout != b.layout || num_dims != b.num_dims) return false;
  for (int i = 0; i < num_dims; i++)
    if (dim[i] != b.dim[i]) return false;
  return owner_op == b.owner_op && owner_ts_idx == b.owner_ts_idx && smem_offset == b.smem_offset;
}

size_t STensor::size() const {
  size_t elem = 0;
  switch (data_type) {
    case DT_INT8: elem = 1; break;
    case DT_BFLOAT16: case DT_FLOAT16: case DT_UINT16: elem = 2; break;
    case DT_FLOAT32: elem = 4; break;
    default: assert(false && "tile of unknown element type");
  }
  return num_elements() * elem;
}

// ---- operators --------------------------------------------------------------------------------
TBOperator::TBOperator(Graph *g, TBOperatorType t) : bgraph(g), op_type(t) {}
TBOperator::TBOperator(Graph *g, TBOperatorType t, STensor const &a) : bgraph(g), op_type(t) {
  input_tensors.push_back(a);
}
TBOperator::TBOperator(Graph *g, TBOperatorType t, STensor const &a, STensor const &b) : bgraph(g), op_type(t) {
  input_tensors.push_back(a);
  input_tensors.push_back(b);
}
TBOperator::~TBOperator() {}

namespace {
// Tile extents of a device tensor under a grid partition and a for-loop tiling; false when a
// mapped dimension is not evenly divisible (input_loader.cc:44-70 asserts these).
bool partitioned_dims(Graph const &g, DTensor const &t, int3 map, int forloop_dim, int out[MAX_TENSOR_DIMS]) {
  for (int i = 0; i < t.num_dims; i++) out[i] = t.dim[i];
  int const idx[3] = {map.x, map.y, map.z};
  unsigned const div[3] = {g.grid_dim.x, g.grid_dim.y, g.grid_dim.z};
  for (int a = 0; a < 3; a++) {
    if (div[a] > 1 && idx[a] >= 0) {
      if (idx[a] >= t.num_dims || out[idx[a]] <= 0 || out[idx[a]] % (int)div[a] != 0) return false;
      out[idx[a]] /= (int)div[a];
    }
  }
  if (forloop_dim >= 0) {
    if (forloop_dim >= t.num_dims || out[forloop_dim] <= 0 || out[forloop_dim] % g.forloop_range != 0) return false;
    out[forloop_dim] /= g.forloop_range;
  }
  return true;
}

STensor make_output_like(TBOperator *owner, STensor const &proto) {
  STensor t = proto;
  t.owner_op = owner;
  t.owner_ts_idx = 0;
  t.guid = STensor::next_guid++;
  return t;
}
} // namespace

TBInputOp::TBInputOp(Graph *g, DTensor const &dt, int3 map, int fdim, mirage::layout::SmemLayout lay)
    : TBOperator(g, TB_INPUT_OP), dtensor(dt), input_map(map), forloop_dim(fdim) {
  STensor t;
  t.layout = lay;
  t.num_dims = dt.num_dims;
  t.data_type = dt.data_type;
  bool ok = partitioned_dims(*g, dt, map, fdim, t.dim);
  assert(ok && "input dimension not divisible by grid / for-loop");
  (void)ok;
  for (int i = 0; i < t.num_dims - 2; i++) assert(t.dim[i] == 1);
  t = make_output_like(this, t);
  t.smem_offset = (int)g->allocate(t);
  output_tensors.push_back(t);
}
TBInputOp::~TBInputOp() { bgraph->free(output_tensors[0]); }

TBOutputOp::TBOutputOp(Graph *g, STensor const &in, int3 map) : TBOperator(g, TB_OUTPUT_OP, in), output_map(map) {
  STensor acc = make_output_like(this, in); // accumulator tile carried across for-loop iterations
  acc.smem_offset = (int)g->allocate(acc);
  output_tensors.push_back(acc);
  dtensor.num_dims = acc.num_dims;
  dtensor.data_type = acc.data_type;
  dtensor.layout = mirage::layout::DmemRowMajor;
  for (int i = 0; i < acc.num_dims; i++) dtensor.dim[i] = acc.dim[i];
  int const idx[3] = {map.x, map.y, map.z};
  unsigned const mul[3] = {g->grid_dim.x, g->grid_dim.y, g->grid_dim.z};
  for (int a = 0; a < 3; a++)
    if (mul[a] > 1 && idx[a] >= 0) {
      assert(idx[a] < dtensor.num_dims && dtensor.dim[idx[a]] > 0);
      dtensor.dim[idx[a]] *= (int)mul[a];
    }
}
TBOutputOp::~TBOutputOp() { bgraph->free(output_tensors); }

TBMatmulOp::TBMatmulOp(Graph *g, STensor const &A, STensor const &B) : TBOperator(g, TB_MATMUL_OP, A, B) {
  assert(A.num_dims == B.num_dims);
  STensor C = A;
  C.layout = mirage::layout::SmemRowMajor; // matmul results are always planned row-major
  C.dim[C.num_dims - 1] = B.dim[B.num_dims - 1];
  C = make_output_like(this, C);
  C.smem_offset = (int)g->allocate(C);
  output_tensors.push_back(C);
}
TBMatmulOp::~TBMatmulOp() { bgraph->free(output_tensors); }

TBElementUnaryOp::TBElementUnaryOp(Graph *g, STensor const &A, TBOperatorType t) : TBOperator(g, t, A) {
  // in place: the result tile aliases the operand tile (element_unary.cc:44-46)
  STensor out = make_output_like(this, A);
  out.smem_offset = A.smem_offset;
  output_tensors.push_back(out);
}
TBElementUnaryOp::~TBElementUnaryOp() {}

TBElementBinaryOp::TBElementBinaryOp(Graph *g, STensor const &A, STensor const &B, TBOperatorType t)
    : TBOperator(g, t, A, B) {
  assert(A.num_dims == B.num_dims);
  STensor out = A;
  for (int i = 0; i < out.num_dims; i++) out.dim[i] = std::max(A.dim[i], B.dim[i]);
  out = make_output_like(this, out);
  out.smem_offset = (int)g->allocate(out);
  output_tensors.push_back(out);
}
TBElementBinaryOp::~TBElementBinaryOp() { bgraph->free(output_tensors); }

TBReductionOp::TBReductionOp(Graph *g, STensor const &A, int dim, int size)
    : TBOperator(g, (TBOperatorType)((size == 1 ? TB_REDUCTION_0_OP : TB_REDUCTION_0_TO_DIMX_OP) + dim), A),
      reduce_dim(dim), reduce_size(size) {
  STensor out = A;
  assert(out.num_dims > dim);
  out.dim[dim] = size;
  out = make_output_like(this, out);
  out.smem_offset = (int)g->allocate(out);
  output_tensors.push_back(out);
}
TBReductionOp::~TBReductionOp() { bgraph->free(output_tensors[0]); }

TBConcatOp::TBConcatOp(Graph *g, STensor const &A, STensor const &B, int dim)
    : TBOperator(g, (TBOperatorType)(TB_CONCAT_0_OP + dim), A, B), concat_dim(dim) {
  STensor out = A;
  out.dim[dim] = A.dim[dim] + B.dim[dim];
  out = make_output_like(this, out);
  out.smem_offset = (int)g->allocate(out);
  output_tensors.push_back(out);
}
TBConcatOp::~TBConcatOp() { bgraph->free(output_tensors[0]); }

// ---- graph -------------------------------------------------------------------------------------
Graph::Graph(dim3 grid, dim3 block, int frange, int dimx)
    : grid_dim(grid), block_dim(block), forloop_range(frange), reduction_dimx(dimx), smem_offset(0),
      max_smem(mirage::type::MAX_SMEM_SIZE) {
  assert(reduction_dimx > 0);
  assert(forloop_range > 0);
}

off_t Graph::allocate(STensor const &t) {
  off_t at = smem_offset;
  off_t bytes = (off_t)((t.size() + 15) & ~(size_t)15);
  smem_offset += bytes;
  assert(smem_offset <= (off_t)max_smem);
  allocated_tensors.push_back({at, (size_t)bytes});
  return at;
}
void Graph::free(STensor const &t) {
  assert(!allocated_tensors.empty());
  assert(allocated_tensors.back().first == t.smem_offset);
  smem_offset -= (off_t)allocated_tensors.back().second;
  allocated_tensors.pop_back();
}
void Graph::free(std::vector<STensor> const &ts) {
  for (int i = (int)ts.size() - 1; i >= 0; i--) free(ts[i]);
}
bool Graph::fits(size_t extra, bool strict) const {
  size_t need = (size_t)smem_offset + extra;
  return strict ? need < max_smem : need <= max_smem;
}

TBOperator *Graph::create_input_op(DTensor const &dt, int3 map, int fdim, mirage::layout::SmemLayout lay) {
  if (dt.num_dims < 2 || dt.num_dims > MAX_TENSOR_DIMS) return nullptr;
  if (dt.data_type != DT_FLOAT16 && dt.data_type != DT_BFLOAT16) return nullptr; // 16-bit tiles only
  STensor probe;
  probe.num_dims = dt.num_dims;
  probe.data_type = dt.data_type;
  if (!partitioned_dims(*this, dt, map, fdim, probe.dim)) return nullptr;
  for (int i = 0; i < probe.num_dims - 2; i++)
    if (probe.dim[i] != 1) return nullptr; // loaders move 2-D tiles
  if (!fits(probe.size())) return nullptr;
  return new TBInputOp(this, dt, map, fdim, lay);
}
STensor Graph::new_input(DTensor const &dt, int3 map, int fdim, mirage::layout::SmemLayout lay) {
  TBOperator *op = create_input_op(dt, map, fdim, lay);
  assert(op != nullptr);
  operators.push_back(op);
  return op->output_tensors[0];
}

TBOperator *Graph::create_output_op(STensor const &s, int3 map) {
  if (!fits(s.size(), /*strict=*/true)) return nullptr; // output.cc:33 uses >=
  int const idx[3] = {map.x, map.y, map.z};
  for (int a = 0; a < 3; a++)
    if (idx[a] >= s.num_dims) return nullptr;
  return new TBOutputOp(this, s, map);
}
DTensor Graph::new_output(STensor const &s, int3 map) {
  TBOperator *op = create_output_op(s, map);
  assert(op != nullptr);
  operators.push_back(op);
  return static_cast<TBOutputOp *>(op)->dtensor;
}

TBOperator *Graph::create_matmul_op(STensor const &A, STensor const &B) {
  if (A.num_dims != B.num_dims || A.num_dims < 2) return nullptr;
  if (A.dim[A.num_dims - 1] != B.dim[B.num_dims - 2]) return nullptr;
  for (int i = 0; i < A.num_dims - 2; i++)
    if (A.dim[i] != 1 || B.dim[i] != 1) return nullptr; // no batched matmul inside a block
  STensor C = A;
  C.dim[C.num_dims - 1] = B.dim[B.num_dims - 1];
  if (!fits(C.size())) return nullptr;
  return new TBMatmulOp(this, A, B);
}
STensor Graph::matmul(STensor const &A, STensor const &B) {
  TBOperator *op = create_matmul_op(A, B);
  assert(op != nullptr);
  operators.push_back(op);
  return op->output_tensors[0];
}

TBOperator *Graph::create_elementunary_op(STensor const &A, TBOperatorType t) {
  if (t != TB_EXP_OP) return nullptr;
  return new TBElementUnaryOp(this, A, t);
}
STensor Graph::exp(STensor const &A) {
  TBOperator *op = create_elementunary_op(A, TB_EXP_OP);
  assert(op != nullptr);
  operators.push_back(op);
  return op->output_tensors[0];
}

TBOperator *Graph::create_elementbinary_op(STensor const &A, STensor const &B, TBOperatorType t) {
  if (A.num_dims != B.num_dims) return nullptr;
  STensor out = A;
  for (int i = 0; i < A.num_dims; i++) {
    if (A.dim[i] != B.dim[i] && A.dim[i] > 1 && B.dim[i] > 1) return nullptr;
    out.dim[i] = std::max(A.dim[i], B.dim[i]);
  }
  if (!fits(out.size())) return nullptr;
  return new TBElementBinaryOp(this, A, B, t);
}
#define MG_BINARY(NAME, TYPE)                                         \
  STensor Graph::NAME(STensor const &A, STensor const &B) {           \
    TBOperator *op = create_elementbinary_op(A, B, TYPE);             \
    assert(op != nullptr);                                            \
    operators.push_back(op);                                          \
    return op->output_tensors[0];                                     \
  }
MG_BINARY(add, TB_ADD_OP)
MG_BINARY(mul, TB_MUL_OP)
MG_BINARY(div, TB_DIV_OP)
#undef MG_BINARY

TBOperator *Graph::create_reduction_op(STensor const &A, int dim) {
  if (dim < 0 || dim >= A.num_dims || dim > 2) return nullptr;
  if (A.layout != mirage::layout::SmemRowMajor) return nullptr; // reduction.cc:33 asserts this
  if (dim < A.num_dims - 2) return nullptr;
  STensor out = A;
  out.dim[dim] = 1;
  if (!fits(out.size())) return nullptr;
  return new TBReductionOp(this, A, dim, 1);
}
STensor Graph::reduction(STensor const &A, int dim) {
  TBOperator *op = create_reduction_op(A, dim);
  assert(op != nullptr);
  operators.push_back(op);
  return op->output_tensors[0];
}
TBOperator *Graph::create_reduction_to_dimx_op(STensor const &A, int dim) {
  if (dim < 0 || dim >= A.num_dims || dim > 2) return nullptr;
  if (A.layout != mirage::layout::SmemRowMajor) return nullptr;
  if (A.dim[dim] % reduction_dimx != 0) return nullptr;
  STensor out = A;
  out.dim[dim] = reduction_dimx;
  if (!fits(out.size())) return nullptr;
  return new TBReductionOp(this, A, dim, reduction_dimx);
}
STensor Graph::reduction_to_dimx(STensor const &A, int dim) {
  TBOperator *op = create_reduction_to_dimx_op(A, dim);
  assert(op != nullptr);
  operators.push_back(op);
  return op->output_tensors[0];
}

TBOperator *Graph::create_concat_op(STensor const &A, STensor const &B, int dim) {
  if (A.num_dims != B.num_dims || dim < 0 || A.num_dims <= dim || dim > 2) return nullptr;
  for (int i = 0; i < A.num_dims; i++)
    if (i != dim && A.dim[i] != B.dim[i]) return nullptr;
  if (A.layout != B.layout) return nullptr;
  if (!fits(A.size() + B.size())) return nullptr;
  return new TBConcatOp(this, A, B, dim);
}
STensor Graph::concat(STensor const &A, STensor const &B, int dim) {
  TBOperator *op = create_concat_op(A, B, dim);
  assert(op != nullptr);
  operators.push_back(op);
  return op->output_tensors[0];
}

// ---- lowering ------------------------------------------------------------------------------------
namespace {
void leading_strides(DTensor const &t, int strides[MAX_TENSOR_DIMS]) {
  int nd = t.num_dims;
  for (int i = 0; i < MAX_TENSOR_DIMS; i++) strides[i] = 0;
  if (nd > 2) {
    strides[nd - 3] = t.dim[nd - 2] * t.dim[nd - 1];
    for (int j = nd - 4; j >= 0; j--) strides[j] = strides[j + 1] * t.dim[j + 1];
  }
}
void last3(STensor const &t, int32_t out[3]) {
  out[2] = t.num_dims > 0 ? t.dim[t.num_dims - 1] : 1;
  out[1] = t.num_dims > 1 ? t.dim[t.num_dims - 2] : 1;
  out[0] = t.num_dims > 2 ? t.dim[t.num_dims - 3] : 1;
}
} // namespace

bool Graph::lower(mgd_program &P, char const **why) const {
  char const *dummy;
  if (!why) why = &dummy;
  std::memset(&P, 0, sizeof(P));
  if (operators.size() > MGD_MAX_OPS) { *why = "too many threadblock operators"; return false; }
  if (block_dim.y != 1 || block_dim.z != 1) { *why = "block_dim must be (n,1,1)"; return false; }
  P.grid[0] = (int)grid_dim.x; P.grid[1] = (int)grid_dim.y; P.grid[2] = (int)grid_dim.z;
  P.threads = (int)block_dim.x;
  P.forloop_range = forloop_range;
  P.num_ops = (int)operators.size();
  P.smem_bytes = (int)smem_offset;
  bool seen_non_input = false, seen_output = false;
  for (size_t i = 0; i < operators.size(); i++) {
    TBOperator const *op = operators[i];
    mgd_op &o = P.ops[i];
    o.type = (int)op->op_type;
    if (op->op_type != TB_INPUT_OP) seen_non_input = true;
    if (op->op_type == TB_OUTPUT_OP) seen_output = true;
    else if (seen_output) { *why = "output operators must come last"; return false; }
    switch (op->op_type) {
      case TB_INPUT_OP: {
        if (seen_non_input) { *why = "input operators must come first"; return false; }
        if (P.num_inputs >= MGD_MAX_IO) { *why = "too many inputs"; return false; }
        auto const *in = static_cast<TBInputOp const *>(op);
        STensor const &st = op->output_tensors[0];
        DTensor const &dt = in->dtensor;
        int nd = st.num_dims, rd = nd - 2, cd = nd - 1;
        int const map[3] = {in->input_map.x, in->input_map.y, in->input_map.z};
        // A block's tile origin: grid index times tile extent along the mapped dim; when that dim is
        // also tiled by the for-loop each block owns forloop_range consecutive tiles.
        for (int a = 0; a < 3; a++) {
          o.a[0 + a] = (map[a] == rd ? st.dim[rd] : 0) * (in->forloop_dim == rd ? forloop_range : 1);
          o.a[3 + a] = (map[a] == cd ? st.dim[cd] : 0) * (in->forloop_dim == cd ? forloop_range : 1);
        }
        o.a[6] = in->forloop_dim == rd ? st.dim[rd] : 0;
        o.a[7] = in->forloop_dim == cd ? st.dim[cd] : 0;
        int strides[MAX_TENSOR_DIMS];
        leading_strides(dt, strides);
        for (int a = 0; a < 3; a++) o.a[8 + a] = (map[a] >= 0 && map[a] < nd - 2) ? strides[map[a]] : 0;
        o.a[11] = (in->forloop_dim >= 0 && in->forloop_dim < nd - 2) ? st.dim[in->forloop_dim] * strides[in->forloop_dim] : 0;
        o.a[12] = dt.dim[rd]; o.a[13] = dt.dim[cd];
        o.a[14] = st.dim[rd]; o.a[15] = st.dim[cd];
        o.a[16] = (int)dt.layout;
        o.a[17] = st.smem_offset;
        o.a[18] = P.num_inputs++;
        break;
      }
      case TB_OUTPUT_OP: {
        if (P.num_outputs >= MGD_MAX_IO) { *why = "too many outputs"; return false; }
        auto const *out = static_cast<TBOutputOp const *>(op);
        STensor const &src = op->input_tensors[0];
        STensor const &acc = op->output_tensors[0];
        DTensor const &dt = out->dtensor;
        int nd = src.num_dims, rd = nd - 2, cd = nd - 1;
        int const map[3] = {out->output_map.x, out->output_map.y, out->output_map.z};
        int strides[MAX_TENSOR_DIMS];
        leading_strides(dt, strides);
        for (int a = 0; a < 3; a++) {
          o.a[0 + a] = map[a] == rd ? src.dim[rd] : 0;
          o.a[3 + a] = map[a] == cd ? src.dim[cd] : 0;
          o.a[6 + a] = (map[a] >= 0 && map[a] < nd - 2) ? strides[map[a]] : 0;
        }
        o.a[9] = dt.dim[rd]; o.a[10] = dt.dim[cd];
        o.a[11] = src.dim[rd]; o.a[12] = src.dim[cd];
        o.a[13] = src.smem_offset;
        o.a[14] = acc.smem_offset;
        o.a[15] = P.num_outputs++;
        break;
      }
      case TB_MATMUL_OP: {
        STensor const &A = op->input_tensors[0], &B = op->input_tensors[1], &C = op->output_tensors[0];
        int nd = A.num_dims;
        o.a[0] = A.dim[nd - 2]; o.a[1] = B.dim[nd - 1]; o.a[2] = A.dim[nd - 1];
        o.a[3] = A.smem_offset; o.a[4] = B.smem_offset; o.a[5] = C.smem_offset;
        break;
      }
      case TB_EXP_OP: {
        o.a[0] = op->input_tensors[0].smem_offset;
        o.a[1] = (int)op->input_tensors[0].num_elements();
        break;
      }
      case TB_DIV_OP: case TB_ADD_OP: case TB_MUL_OP: {
        STensor const &x = op->input_tensors[0], &y = op->input_tensors[1];
        for (int d = 0; d < x.num_dims - 3; d++)
          if (x.dim[d] != 1 || y.dim[d] != 1) { *why = "only the last three dims may exceed 1"; return false; }
        last3(x, &o.a[0]);
        last3(y, &o.a[3]);
        o.a[6] = x.smem_offset; o.a[7] = y.smem_offset; o.a[8] = op->output_tensors[0].smem_offset;
        break;
      }
      case TB_REDUCTION_0_OP: case TB_REDUCTION_1_OP: case TB_REDUCTION_2_OP:
      case TB_REDUCTION_0_TO_DIMX_OP: case TB_REDUCTION_1_TO_DIMX_OP: case TB_REDUCTION_2_TO_DIMX_OP: {
        STensor const &in = op->input_tensors[0], &out = op->output_tensors[0];
        int rdim = op->op_type >= TB_REDUCTION_0_TO_DIMX_OP ? op->op_type - TB_REDUCTION_0_TO_DIMX_OP
                                                            : op->op_type - TB_REDUCTION_0_OP;
        int inner = 1;
        for (int d = rdim; d < out.num_dims; d++) inner *= out.dim[d];
        o.a[0] = (int)out.num_elements();
        o.a[1] = (int)(in.num_elements() / out.num_elements());
        o.a[2] = inner;
        o.a[3] = in.smem_offset; o.a[4] = out.smem_offset;
        break;
      }
      case TB_CONCAT_0_OP: case TB_CONCAT_1_OP: case TB_CONCAT_2_OP: {
        STensor const &A = op->input_tensors[0], &B = op->input_tensors[1], &out = op->output_tensors[0];
        int cdim = op->op_type - TB_CONCAT_0_OP, inner = 1;
        for (int d = cdim + 1; d < out.num_dims; d++) inner *= out.dim[d];
        o.a[0] = (int)out.num_elements();
        o.a[1] = A.dim[cdim]; o.a[2] = B.dim[cdim]; o.a[3] = inner;
        o.a[4] = A.smem_offset; o.a[5] = B.smem_offset; o.a[6] = out.smem_offset;
        break;
      }
      default: *why = "operator has no kernel"; return false;
    }
  }
  return true;
}

} // namespace threadblock
} // namespace mirage
