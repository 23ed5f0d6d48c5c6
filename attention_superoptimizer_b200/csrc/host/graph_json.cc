// Graph JSON wire format: see include/mirage/utils/json_utils.h for the contract and the reference locations.
// A small JSON reader/writer lives here so that the library keeps zero third-party dependencies.
#include "mirage/utils/json_utils.h"
#include "status.h"
#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <unordered_map>
#include <vector>

namespace {
using namespace mirage;

// ---- a JSON value -----------------------------------------------------------------------------------------------
struct JValue {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<JValue> arr;
  std::map<std::string, JValue> obj; // ordered: dump() prints keys alphabetically like the reference's library

  JValue const *find(char const *key) const {
    if (kind != Object) return nullptr;
    auto it = obj.find(key);
    return it == obj.end() ? nullptr : &it->second;
  }
};

struct Parser {
  char const *p, *end;
  std::string err;
  int depth = 0;

  void skip() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++;
  }
  bool fail(char const *what) {
    if (err.empty()) err = std::string("JSON: ") + what + " at byte " + std::to_string((long long)(p - (end - len)));
    return false;
  }
  size_t len = 0;

  bool parse_string(std::string &out) {
    if (p >= end || *p != '"') return fail("expected a string");
    p++;
    out.clear();
    while (p < end && *p != '"') {
      if (*p == '\\') {
        if (++p >= end) return fail("unterminated escape");
        switch (*p) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'r': out += '\r'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'u': { // basic multilingual plane only; names in this format are ASCII
            if (end - p < 5) return fail("short \\u escape");
            unsigned code = (unsigned)std::strtoul(std::string(p + 1, p + 5).c_str(), nullptr, 16);
            if (code < 0x80) out += (char)code;
            else if (code < 0x800) { out += (char)(0xC0 | (code >> 6)); out += (char)(0x80 | (code & 0x3F)); }
            else { out += (char)(0xE0 | (code >> 12)); out += (char)(0x80 | ((code >> 6) & 0x3F)); out += (char)(0x80 | (code & 0x3F)); }
            p += 4;
            break;
          }
          default: out += *p; break; // \" \\ \/
        }
        p++;
      } else {
        out += *p++;
      }
    }
    if (p >= end) return fail("unterminated string");
    p++;
    return true;
  }

  bool parse(JValue &v) {
    if (++depth > 64) return fail("nesting too deep");
    skip();
    if (p >= end) return fail("unexpected end");
    bool ok = true;
    if (*p == '{') {
      v.kind = JValue::Object;
      p++;
      skip();
      if (p < end && *p == '}') p++;
      else
        for (;;) {
          skip();
          std::string key;
          if (!parse_string(key)) { ok = false; break; }
          skip();
          if (p >= end || *p != ':') { ok = fail("expected ':'"); break; }
          p++;
          if (!parse(v.obj[key])) { ok = false; break; }
          skip();
          if (p < end && *p == ',') { p++; continue; }
          if (p < end && *p == '}') { p++; break; }
          ok = fail("expected ',' or '}'");
          break;
        }
    } else if (*p == '[') {
      v.kind = JValue::Array;
      p++;
      skip();
      if (p < end && *p == ']') p++;
      else
        for (;;) {
          v.arr.emplace_back();
          if (!parse(v.arr.back())) { ok = false; break; }
          skip();
          if (p < end && *p == ',') { p++; continue; }
          if (p < end && *p == ']') { p++; break; }
          ok = fail("expected ',' or ']'");
          break;
        }
    } else if (*p == '"') {
      v.kind = JValue::String;
      ok = parse_string(v.str);
    } else if (end - p >= 4 && std::string(p, p + 4) == "true") {
      v.kind = JValue::Bool; v.b = true; p += 4;
    } else if (end - p >= 5 && std::string(p, p + 5) == "false") {
      v.kind = JValue::Bool; v.b = false; p += 5;
    } else if (end - p >= 4 && std::string(p, p + 4) == "null") {
      v.kind = JValue::Null; p += 4;
    } else if (*p == '-' || std::isdigit((unsigned char)*p)) {
      char const *q = p;
      while (q < end && (std::isdigit((unsigned char)*q) || *q == '-' || *q == '+' || *q == '.' || *q == 'e' || *q == 'E')) q++;
      std::string tok(p, q);
      char *stop = nullptr;
      v.kind = JValue::Number;
      v.num = std::strtod(tok.c_str(), &stop);
      if (stop == tok.c_str() || *stop != 0) ok = fail("bad number");
      p = q;
    } else {
      ok = fail("unexpected character");
    }
    depth--;
    return ok;
  }
};

bool parse_json(std::string const &text, JValue &v, std::string *err) {
  Parser ps;
  ps.p = text.data();
  ps.end = text.data() + text.size();
  ps.len = text.size();
  if (!ps.parse(v)) {
    if (err) *err = ps.err;
    return false;
  }
  ps.skip();
  if (ps.p != ps.end) {
    if (err) *err = "JSON: trailing characters after the document";
    return false;
  }
  return true;
}

void dump(JValue const &v, std::string &out) {
  switch (v.kind) {
    case JValue::Null: out += "null"; break;
    case JValue::Bool: out += v.b ? "true" : "false"; break;
    case JValue::Number: {
      char buf[40];
      if (v.num == (double)(long long)v.num && v.num > -9.0e15 && v.num < 9.0e15) std::snprintf(buf, sizeof buf, "%lld", (long long)v.num);
      else std::snprintf(buf, sizeof buf, "%.17g", v.num);
      out += buf;
      break;
    }
    case JValue::String:
      out += '"';
      for (char c : v.str) {
        if (c == '"' || c == '\\') { out += '\\'; out += c; }
        else if (c == '\n') out += "\\n";
        else if (c == '\t') out += "\\t";
        else if ((unsigned char)c < 0x20) { char b[8]; std::snprintf(b, sizeof b, "\\u%04x", c); out += b; }
        else out += c;
      }
      out += '"';
      break;
    case JValue::Array:
      out += '[';
      for (size_t i = 0; i < v.arr.size(); i++) {
        if (i) out += ',';
        dump(v.arr[i], out);
      }
      out += ']';
      break;
    case JValue::Object: {
      out += '{';
      bool first = true;
      for (auto const &kv : v.obj) {
        if (!first) out += ',';
        first = false;
        JValue k;
        k.kind = JValue::String;
        k.str = kv.first;
        dump(k, out);
        out += ':';
        dump(kv.second, out);
      }
      out += '}';
      break;
    }
  }
}

JValue jnum(double x) { JValue v; v.kind = JValue::Number; v.num = x; return v; }
JValue jstr(std::string const &s) { JValue v; v.kind = JValue::String; v.str = s; return v; }
JValue jarr() { JValue v; v.kind = JValue::Array; return v; }
JValue jobj() { JValue v; v.kind = JValue::Object; return v; }

// ---- enum names -------------------------------------------------------------------------------------------------
template <typename E> bool enum_from_name(std::string const &name, std::initializer_list<E> all, E *out) {
  for (E e : all)
    if (name == to_string(e)) { *out = e; return true; }
  return false;
}

bool parse_kn_type(JValue const &v, type::KNOperatorType *t) {
  using namespace type;
  return v.kind == JValue::String &&
         enum_from_name<KNOperatorType>(v.str, {KN_INPUT_OP, KN_MATMUL_OP, KN_REDUCTION_0_OP, KN_REDUCTION_1_OP, KN_REDUCTION_2_OP,
                                                KN_EXP_OP, KN_ADD_OP, KN_MUL_OP, KN_DIV_OP, KN_CUSTOMIZED_OP}, t);
}
bool parse_tb_type(JValue const &v, type::TBOperatorType *t) {
  using namespace type;
  return v.kind == JValue::String &&
         enum_from_name<TBOperatorType>(v.str, {TB_INPUT_OP, TB_OUTPUT_OP, TB_MATMUL_OP, TB_EXP_OP, TB_ADD_OP, TB_MUL_OP, TB_DIV_OP,
                                                TB_REDUCTION_0_OP, TB_REDUCTION_1_OP, TB_REDUCTION_2_OP,
                                                TB_REDUCTION_0_TO_DIMX_OP, TB_REDUCTION_1_TO_DIMX_OP, TB_REDUCTION_2_TO_DIMX_OP,
                                                TB_CONCAT_0_OP, TB_CONCAT_1_OP, TB_CONCAT_2_OP, TB_CUSTOMIZED_OP}, t);
}
bool parse_dmem(JValue const &v, layout::DmemLayout *l) {
  using namespace layout;
  return v.kind == JValue::String && enum_from_name<DmemLayout>(v.str, {DmemRowMajor, DmemColumnMajor, DmemUnknownLayout}, l);
}
bool parse_smem(JValue const &v, layout::SmemLayout *l) {
  using namespace layout;
  return v.kind == JValue::String &&
         enum_from_name<SmemLayout>(v.str, {SmemRowMajor, SmemColumnMajor, SmemRowMajorTensorOpMultiplicand_Crosswise16,
                                            SmemRowMajorTensorOpMultiplicand_Crosswise32, SmemRowMajorTensorOpMultiplicand_Crosswise64,
                                            SmemColumnMajorTensorOpMultiplicand_Crosswise16, SmemColumnMajorTensorOpMultiplicand_Crosswise32,
                                            SmemColumnMajorTensorOpMultiplicand_Crosswise64, SmemUnknownLayout}, l);
}

// ---- writers ----------------------------------------------------------------------------------------------------
JValue xyz(long long x, long long y, long long z) {
  JValue v = jobj();
  v.obj["x"] = jnum((double)x); v.obj["y"] = jnum((double)y); v.obj["z"] = jnum((double)z);
  return v;
}

// DTensor: data_type (number), layout (name), num_dims, dim (all MAX_TENSOR_DIMS entries), guid
JValue to_value(kernel::DTensor const &t) {
  JValue v = jobj();
  v.obj["data_type"] = jnum((double)t.data_type);
  v.obj["layout"] = jstr(to_string(t.layout));
  v.obj["num_dims"] = jnum(t.num_dims);
  JValue d = jarr();
  for (int i = 0; i < MAX_TENSOR_DIMS; i++) d.arr.push_back(jnum(i < t.num_dims ? t.dim[i] : 0));
  v.obj["dim"] = d;
  v.obj["guid"] = jnum((double)t.guid);
  return v;
}

JValue to_value(threadblock::STensor const &t) {
  JValue v = jobj();
  v.obj["data_type"] = jnum((double)t.data_type);
  v.obj["layout"] = jstr(to_string(t.layout));
  v.obj["num_dims"] = jnum(t.num_dims);
  JValue d = jarr();
  for (int i = 0; i < MAX_TENSOR_DIMS; i++) d.arr.push_back(jnum(i < t.num_dims ? t.dim[i] : 0));
  v.obj["dim"] = d;
  v.obj["smem_offset"] = jnum(t.smem_offset);
  v.obj["guid"] = jnum(t.guid);
  return v;
}

template <typename T> JValue to_array(std::vector<T> const &ts) {
  JValue a = jarr();
  for (T const &t : ts) a.arr.push_back(to_value(t));
  return a;
}

JValue to_value(threadblock::ExecutionPlan const &plan) {
  JValue v = jobj();
  JValue ops = jarr();
  for (auto const &op : plan.ops) { // std::pair serialises as a two-element array
    JValue pair = jarr(), ins = jarr();
    pair.arr.push_back(jstr(to_string(op.first)));
    for (auto const &in : op.second) {
      JValue ij = jarr();
      ij.arr.push_back(jnum(in.first));
      ij.arr.push_back(jnum(in.second));
      ins.arr.push_back(ij);
    }
    pair.arr.push_back(ins);
    ops.arr.push_back(pair);
  }
  v.obj["ops"] = ops;
  JValue imap = jarr(), fdim = jarr(), lay = jarr();
  for (int3 const &m : plan.input_map) imap.arr.push_back(xyz(m.x, m.y, m.z));
  for (int f : plan.forloop_dim) fdim.arr.push_back(jnum(f));
  for (auto l : plan.input_smem_layouts) lay.arr.push_back(jstr(to_string(l)));
  v.obj["input_map"] = imap;
  v.obj["forloop_dim"] = fdim;
  v.obj["input_smem_layouts"] = lay;
  v.obj["output_map"] = xyz(plan.output_map.x, plan.output_map.y, plan.output_map.z);
  v.obj["forloop_range"] = jnum(plan.forloop_range);
  v.obj["reduction_dimx"] = jnum(plan.reduction_dimx);
  v.obj["grid_dim"] = xyz(plan.grid_dim.x, plan.grid_dim.y, plan.grid_dim.z);
  v.obj["block_dim"] = xyz(plan.block_dim.x, plan.block_dim.y, plan.block_dim.z);
  return v;
}

// threadblock operator: op_type, input_tensors, output_tensors plus the per-class members
JValue to_value(threadblock::TBOperator const *op) {
  using namespace threadblock;
  JValue v = jobj();
  v.obj["op_type"] = jstr(to_string(op->op_type));
  v.obj["input_tensors"] = to_array(op->input_tensors);
  v.obj["output_tensors"] = to_array(op->output_tensors);
  if (auto in = dynamic_cast<TBInputOp const *>(op)) {
    v.obj["dtensor"] = to_value(in->dtensor);
    v.obj["input_map"] = xyz(in->input_map.x, in->input_map.y, in->input_map.z);
    v.obj["forloop_dim"] = jnum(in->forloop_dim);
  } else if (auto out = dynamic_cast<TBOutputOp const *>(op)) {
    v.obj["dtensor"] = to_value(out->dtensor);
    v.obj["output_map"] = xyz(out->output_map.x, out->output_map.y, out->output_map.z);
  } else if (auto red = dynamic_cast<TBReductionOp const *>(op)) {
    v.obj["reduce_dim"] = jnum(red->reduce_dim);
    v.obj["reduce_size"] = jnum(red->reduce_size);
  } else if (auto cat = dynamic_cast<TBConcatOp const *>(op)) {
    v.obj["concat_dim"] = jnum(cat->concat_dim);
  }
  return v;
}

JValue to_value(threadblock::Graph const &g) {
  JValue v = jobj();
  v.obj["graph_level"] = jstr("thread_block_graph");
  v.obj["grid_dim"] = xyz(g.grid_dim.x, g.grid_dim.y, g.grid_dim.z);
  v.obj["block_dim"] = xyz(g.block_dim.x, g.block_dim.y, g.block_dim.z);
  v.obj["forloop_range"] = jnum(g.forloop_range);
  v.obj["reduction_dimx"] = jnum(g.reduction_dimx);
  v.obj["smem_offset"] = jnum((double)g.smem_offset);
  JValue ops = jarr();
  for (threadblock::TBOperator const *op : g.operators) ops.arr.push_back(to_value(op));
  v.obj["operators"] = ops;
  return v;
}

JValue to_value(kernel::KNOperator const *op) {
  JValue v = jobj();
  v.obj["op_type"] = jstr(to_string(op->op_type));
  v.obj["input_tensors"] = to_array(op->input_tensors);
  v.obj["output_tensors"] = to_array(op->output_tensors);
  if (auto c = dynamic_cast<kernel::KNCustomizedOp const *>(op)) {
    v.obj["bgraph"] = to_value(c->bgraph);
    v.obj["plan"] = to_value(c->plan);
  }
  return v;
}

// ---- readers ----------------------------------------------------------------------------------------------------
struct Reader {
  std::string err;
  bool fail(std::string const &what) {
    if (err.empty()) err = what;
    return false;
  }
  bool integer(JValue const *v, long long *out, char const *what) {
    if (!v || v->kind != JValue::Number || v->num != (double)(long long)v->num) return fail(std::string("missing or non-integer \"") + what + "\"");
    *out = (long long)v->num;
    return true;
  }
  bool integer(JValue const *v, int *out, char const *what) {
    long long x;
    if (!integer(v, &x, what)) return false;
    *out = (int)x;
    return true;
  }
  bool xyz_of(JValue const *v, long long *x, long long *y, long long *z, char const *what) {
    if (!v || v->kind != JValue::Object) return fail(std::string("missing {x,y,z} object \"") + what + "\"");
    return integer(v->find("x"), x, "x") && integer(v->find("y"), y, "y") && integer(v->find("z"), z, "z");
  }
  bool int3_of(JValue const *v, int3 *out, char const *what) {
    long long x, y, z;
    if (!xyz_of(v, &x, &y, &z, what)) return false;
    out->x = (int)x; out->y = (int)y; out->z = (int)z;
    return true;
  }
  bool dim3_of(JValue const *v, dim3 *out, char const *what) {
    long long x, y, z;
    if (!xyz_of(v, &x, &y, &z, what)) return false;
    if (x <= 0 || y <= 0 || z <= 0) return fail(std::string("non-positive extent in \"") + what + "\"");
    *out = dim3((unsigned)x, (unsigned)y, (unsigned)z);
    return true;
  }
  JValue const *array_of(JValue const *v, char const *what) {
    if (!v || v->kind != JValue::Array) {
      fail(std::string("missing array \"") + what + "\"");
      return nullptr;
    }
    return v;
  }
  bool guid_of(JValue const &tensor, size_t *guid) {
    long long g;
    if (!integer(tensor.find("guid"), &g, "guid")) return false;
    *guid = (size_t)g;
    return true;
  }

  bool plan_of(JValue const *v, threadblock::ExecutionPlan *plan) {
    if (!v || v->kind != JValue::Object) return fail("customized operator without a \"plan\" object");
    JValue const *ops = array_of(v->find("ops"), "plan.ops");
    if (!ops) return false;
    for (JValue const &jop : ops->arr) {
      if (jop.kind != JValue::Array || jop.arr.size() != 2 || jop.arr[1].kind != JValue::Array) return fail("plan.ops entry is not [type, inputs]");
      type::TBOperatorType t;
      if (!parse_tb_type(jop.arr[0], &t)) return fail("plan.ops: unknown threadblock operator type");
      std::vector<std::pair<int, int>> ins;
      for (JValue const &ji : jop.arr[1].arr) {
        int a, b;
        if (ji.kind != JValue::Array || ji.arr.size() != 2) return fail("plan.ops input is not [operator, output]");
        if (!integer(&ji.arr[0], &a, "operator index") || !integer(&ji.arr[1], &b, "output index")) return false;
        ins.emplace_back(a, b);
      }
      plan->ops.emplace_back(t, ins);
    }
    JValue const *imap = array_of(v->find("input_map"), "plan.input_map");
    JValue const *fdim = array_of(v->find("forloop_dim"), "plan.forloop_dim");
    JValue const *lay = array_of(v->find("input_smem_layouts"), "plan.input_smem_layouts");
    if (!imap || !fdim || !lay) return false;
    for (JValue const &m : imap->arr) {
      int3 x;
      if (!int3_of(&m, &x, "input_map")) return false;
      plan->input_map.push_back(x);
    }
    for (JValue const &f : fdim->arr) {
      int x;
      if (!integer(&f, &x, "forloop_dim")) return false;
      plan->forloop_dim.push_back(x);
    }
    for (JValue const &l : lay->arr) {
      layout::SmemLayout x;
      if (!parse_smem(l, &x)) return fail("plan.input_smem_layouts: unknown layout name");
      plan->input_smem_layouts.push_back(x);
    }
    if (!int3_of(v->find("output_map"), &plan->output_map, "plan.output_map")) return false;
    if (!integer(v->find("forloop_range"), &plan->forloop_range, "plan.forloop_range")) return false;
    // checkpoints written before the reference grew `reduction_dimx` (its demo checkpoint is one) lack the key:
    // they get the default, where the reference's own reader would throw
    if (v->find("reduction_dimx") && !integer(v->find("reduction_dimx"), &plan->reduction_dimx, "plan.reduction_dimx")) return false;
    return dim3_of(v->find("grid_dim"), &plan->grid_dim, "plan.grid_dim") &&
           dim3_of(v->find("block_dim"), &plan->block_dim, "plan.block_dim");
  }
};
} // namespace

namespace mirage {
namespace kernel {

std::string to_json_string(KNOperator const &op) {
  std::string out;
  dump(to_value(&op), out);
  return out;
}

std::string to_json_string(Graph const &g) {
  JValue root = jarr();
  for (KNOperator const *op : g.operators) root.arr.push_back(to_value(op));
  std::string out;
  dump(root, out);
  return out;
}

bool from_json_string(std::string const &text, Graph &g, std::string *error) {
  JValue root;
  Reader rd;
  auto give_up = [&](std::string const &what) {
    if (error) *error = what;
    mg::set_error(what);
    return false;
  };
  {
    std::string perr;
    if (!parse_json(text, root, &perr)) return give_up(perr);
  }
  if (root.kind != JValue::Array) return give_up("graph JSON: the document is not an array of operators");

  // guid in the document -> tensor built here (the reference keeps the inverse map and searches the graph)
  std::unordered_map<size_t, DTensor> by_guid;
  auto operand = [&](JValue const *inputs, size_t i, DTensor *out) {
    if (!inputs || inputs->kind != JValue::Array || inputs->arr.size() <= i) return rd.fail("operator with too few input_tensors");
    size_t guid;
    if (!rd.guid_of(inputs->arr[i], &guid)) return false;
    auto it = by_guid.find(guid);
    if (it == by_guid.end()) return rd.fail("operand guid " + std::to_string(guid) + " was not produced by an earlier operator");
    *out = it->second;
    return true;
  };

  for (size_t n = 0; n < root.arr.size(); n++) {
    JValue const &jop = root.arr[n];
    std::string const where = "graph JSON, operator " + std::to_string(n) + ": ";
    type::KNOperatorType op_type;
    if (jop.kind != JValue::Object || !jop.find("op_type") || !parse_kn_type(*jop.find("op_type"), &op_type))
      return give_up(where + "missing or unknown \"op_type\"");
    JValue const *ins = jop.find("input_tensors");
    JValue const *outs = rd.array_of(jop.find("output_tensors"), "output_tensors");
    if (!outs || outs->arr.empty()) return give_up(where + "no output_tensors");
    KNOperator *op = nullptr;
    switch (op_type) {
      case type::KN_INPUT_OP: {
        JValue const &t = outs->arr[0];
        int num_dims = 0;
        long long dt = 0;
        layout::DmemLayout lay;
        if (!rd.integer(t.find("num_dims"), &num_dims, "num_dims") || !rd.integer(t.find("data_type"), &dt, "data_type"))
          return give_up(where + rd.err);
        if (!t.find("layout") || !parse_dmem(*t.find("layout"), &lay)) return give_up(where + "unknown layout name");
        JValue const *dim = rd.array_of(t.find("dim"), "dim");
        if (!dim || num_dims < 1 || num_dims > MAX_TENSOR_DIMS || (int)dim->arr.size() < num_dims) return give_up(where + "bad dim / num_dims");
        std::vector<int> dims(num_dims);
        for (int i = 0; i < num_dims; i++)
          if (!rd.integer(&dim->arr[i], &dims[i], "dim")) return give_up(where + rd.err);
        op = g.create_input_op(dims, (type::DataType)dt, lay);
        break;
      }
      case type::KN_MATMUL_OP:
      case type::KN_ADD_OP:
      case type::KN_MUL_OP:
      case type::KN_DIV_OP: {
        DTensor a, b;
        if (!operand(ins, 0, &a) || !operand(ins, 1, &b)) return give_up(where + rd.err);
        op = op_type == type::KN_MATMUL_OP ? g.create_matmul_op(a, b) : g.create_elementbinary_op(a, b, op_type);
        break;
      }
      case type::KN_EXP_OP: {
        DTensor a;
        if (!operand(ins, 0, &a)) return give_up(where + rd.err);
        op = g.create_elementunary_op(a, op_type);
        break;
      }
      case type::KN_REDUCTION_0_OP:
      case type::KN_REDUCTION_1_OP:
      case type::KN_REDUCTION_2_OP: {
        DTensor a;
        if (!operand(ins, 0, &a)) return give_up(where + rd.err);
        // the document does not carry the reduced size; like the reference, the dimension goes to 1
        op = g.create_reduction_op(a, op_type - type::KN_REDUCTION_0_OP, 1);
        break;
      }
      case type::KN_CUSTOMIZED_OP: {
        std::vector<DTensor> inputs;
        size_t count = ins && ins->kind == JValue::Array ? ins->arr.size() : 0;
        for (size_t i = 0; i < count; i++) {
          DTensor t;
          if (!operand(ins, i, &t)) return give_up(where + rd.err);
          inputs.push_back(t);
        }
        threadblock::ExecutionPlan plan;
        if (!rd.plan_of(jop.find("plan"), &plan)) return give_up(where + rd.err);
        op = g.create_customized_op(inputs, plan);
        if (op && op->output_tensors.size() != outs->arr.size()) {
          delete op;
          return give_up(where + "the plan produces a different number of outputs than the document lists");
        }
        // tile layouts recorded in "bgraph" replace the defaults the plan gave (results do not depend on them)
        if (op) {
          KNCustomizedOp *c = static_cast<KNCustomizedOp *>(op);
          JValue const *jb = jop.find("bgraph");
          JValue const *jops = jb ? jb->find("operators") : nullptr;
          if (jops && jops->kind == JValue::Array && jops->arr.size() == c->bgraph.operators.size()) {
            for (size_t i = 0; i < jops->arr.size(); i++) {
              threadblock::TBOperator *bop = c->bgraph.operators[i];
              for (int side = 0; side < 2; side++) {
                JValue const *list = jops->arr[i].find(side ? "output_tensors" : "input_tensors");
                auto &tensors = side ? bop->output_tensors : bop->input_tensors;
                if (!list || list->kind != JValue::Array || list->arr.size() != tensors.size()) continue;
                for (size_t j = 0; j < tensors.size(); j++) {
                  JValue const *l = list->arr[j].find("layout");
                  layout::SmemLayout sl;
                  if (l && parse_smem(*l, &sl)) tensors[j].layout = sl;
                }
              }
            }
          }
        }
        break;
      }
      default: return give_up(where + "operator type cannot be rebuilt");
    }
    if (!op) return give_up(where + "the builder refused the operator: " + mg::last_error());
    g.operators.push_back(op);
    for (size_t i = 0; i < op->output_tensors.size() && i < outs->arr.size(); i++) {
      size_t guid;
      if (!rd.guid_of(outs->arr[i], &guid)) return give_up(where + rd.err);
      by_guid[guid] = op->output_tensors[i];
    }
  }
  return true;
}

} // namespace kernel
} // namespace mirage
