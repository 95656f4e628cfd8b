// IntentIR planner and plan executor (host C++).
//
// ib200_plan_create(intent_json, bindings_json) lowers one IntentIR graph under concrete
// shape bindings to a short list of launches of the pre-compiled kernels in this library.
// It replaces the reference's source-emitting C++ codegen
// (backends/cuda/cpp_codegen/intentir_cuda_codegen.cpp:5777-5852) and its Python twin
// (backends/cuda/codegen/intentir_to_cuda.py:2131-2201): same role — pattern dispatch over
// the op list — but the result is a plan over fixed kernels, not CUDA source.
//
// Three phases:
//   A. build: every op becomes a node with a concrete shape, following the interpreter's
//      semantics (verify/interpreter.py:211-545): numpy broadcasting, the declared-symbol
//      alignment of rank-1 operands (:752-841), broadcast_in_dim (:594-608), reduce axis
//      resolution (:676-694), one-input binary ops whose second operand is an attribute
//      (:215-226), matmul epilogue trees (:567-591).
//   B. match: whole-graph patterns that map to one fused kernel — row softmax (single op
//      or the reduce_max/sub/exp/reduce_sum/div chain, with optional row_max / row_sum
//      outputs), layernorm / groupnorm (the centred-variance chain in any of its surface
//      forms, with optional mean / rstd outputs), matmul + bias + relu, and any(x != 0).
//      Matching is structural over the dataflow, looking through reshape /
//      broadcast_in_dim / identity views, and every broadcast is verified through strides.
//   C. general lowering for everything else: maximal elementwise/broadcast subgraphs
//      become single micro-op kernels (ew_program.h); reductions, softmax, matmul and
//      transposes become their kernels; intermediates live in a caller-provided workspace.
#include <algorithm>
#include <cstdlib>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <tuple>
#include <vector>

#include "common.cuh"
#include "ew_program.h"
#include "json.hpp"
#include "row_program.h"

namespace ib200 {
namespace {

struct Unsupported : std::runtime_error { using std::runtime_error::runtime_error; };
struct Invalid : std::runtime_error { using std::runtime_error::runtime_error; };

using Shape = std::vector<int64_t>;

int64_t numel(const Shape& s) { int64_t n = 1; for (auto d : s) n *= d; return n; }
Shape contiguous_strides(const Shape& s) {
  Shape st(s.size());
  int64_t acc = 1;
  for (int i = (int)s.size() - 1; i >= 0; --i) { st[i] = acc; acc *= s[i]; }
  return st;
}
std::string shape_str(const Shape& s) {
  std::string o = "[";
  for (size_t i = 0; i < s.size(); ++i) o += (i ? "," : "") + std::to_string(s[i]);
  return o + "]";
}

enum DClass { DC_FLOAT = 0, DC_BOOL = 1, DC_INT = 2 };

int dtype_code(const std::string& s) {
  static const std::map<std::string, int> m = {{"f32", IB200_F32}, {"bf16", IB200_BF16}, {"f16", IB200_F16}, {"i32", IB200_I32},
                                               {"i64", IB200_I64}, {"bool", IB200_BOOL}, {"i1", IB200_BOOL}, {"u8", IB200_U8},
                                               {"i8", IB200_I8}, {"i16", IB200_I16}, {"f64", IB200_F64}};
  auto it = m.find(s);
  if (it == m.end()) throw Invalid("unknown dtype '" + s + "'");
  return it->second;
}
const char* dtype_name(int c) {
  static const char* n[] = {"f32", "bf16", "f16", "i32", "i64", "bool", "u8", "i8", "i16", "f64"};
  return c >= 0 && c < 10 ? n[c] : "?";
}
int class_of_dtype(int c) {
  if (c == IB200_BOOL) return DC_BOOL;
  if (c == IB200_F32 || c == IB200_BF16 || c == IB200_F16 || c == IB200_F64) return DC_FLOAT;
  return DC_INT;
}
int storage_of_class(int dc) { return dc == DC_BOOL ? IB200_BOOL : dc == DC_INT ? IB200_I32 : IB200_F32; }

// ---- strided views -------------------------------------------------------------------------
struct View {
  int buffer = -1;
  Shape shape, strides;
  int64_t offset = 0;
  bool contiguous() const {
    int64_t acc = 1;
    for (int i = (int)shape.size() - 1; i >= 0; --i) {
      if (shape[i] != 1 && strides[i] != acc) return false;
      acc *= shape[i];
    }
    return offset == 0;
  }
};

// new strides for viewing (shape, strides) as `to` without copying; false if impossible.
// Dims are grouped into chunks that are contiguous among themselves (broadcast chunks have
// stride 0 throughout); each chunk must be covered by a run of target dims.
bool reshape_view(const Shape& shape, const Shape& strides, const Shape& to, Shape& out) {
  out.assign(to.size(), 0);
  if (numel(shape) != numel(to)) return false;
  if (numel(to) == 0) { out = contiguous_strides(to); return true; }
  if (shape.empty()) return true;  // a scalar viewed as [1,1,...]
  int view_d = (int)to.size() - 1;
  int64_t chunk_base = strides.back(), tensor_numel = 1, view_numel = 1;
  for (int d = (int)shape.size() - 1; d >= 0; --d) {
    tensor_numel *= shape[d];
    if (d == 0 || (shape[d - 1] != 1 && strides[d - 1] != tensor_numel * chunk_base)) {
      while (view_d >= 0 && (view_numel < tensor_numel || to[view_d] == 1)) {
        out[view_d] = view_numel * chunk_base;
        view_numel *= to[view_d];
        --view_d;
      }
      if (view_numel != tensor_numel) return false;
      if (d > 0) { chunk_base = strides[d - 1]; tensor_numel = 1; view_numel = 1; }
    }
  }
  return view_d == -1;
}

// ---- graph nodes -----------------------------------------------------------------------------
struct Node {
  std::string name, op;
  std::vector<int> in;
  Shape shape;
  int dclass = DC_FLOAT;
  int decl_dtype = -1;
  double cval = 0.0;
  std::vector<int> axes;  // reduce axes | transpose perm | broadcast dims
  bool keepdims = false;
  double scale = 1.0;
  int axis = 0;
  bool ta = false, tb = false;
  int cast_to = -1;
  // lowering state
  enum Repr { NONE, STRIDED, CONSTANT, IOTA, EXPR } repr = NONE;
  View view;
};

const std::set<std::string> kBinary = {"add", "sub", "mul", "div", "max", "min"};
const std::set<std::string> kUnary = {"relu", "exp", "rsqrt", "abs", "floor"};
const std::set<std::string> kCompare = {"ne", "lt", "le", "gt", "ge"};
const std::set<std::string> kLogic2 = {"and", "or"};
const std::set<std::string> kViews = {"reshape", "broadcast_in_dim", "identity", "layout_cast", "transpose"};

bool is_elementwise(const std::string& op) {
  return kBinary.count(op) || kUnary.count(op) || kCompare.count(op) || kLogic2.count(op) || op == "not" || op == "where" || op == "cast";
}

struct Buffer {
  bool is_arg = false;
  int arg_index = -1;
  size_t ws_offset = 0, bytes = 0;
  int dtype = IB200_F32;
  std::string name;
};

struct Step {
  enum Kind { REDUCE, SOFTMAX, NORM, GEMM, ELEMENTWISE, TRANSPOSE, GATHER, ROWFUSE, ROPE, DROPOUT, CORRELATION, RESIZE, WARP } kind;
  std::string label;
  int in[3] = {-1, -1, -1};
  int out[3] = {-1, -1, -1};
  // kernel extents.  REDUCE: outer, reduced, inner; SOFTMAX / NORM: rows, cols; GEMM: M, N, K; TRANSPOSE: rows, cols;
  // GATHER / DROPOUT: elements (DROPOUT d[1]: Philox rounds); ROPE: seq, batch*heads, D; image ops: C, H, W and
  // d[3] = output channels (correlation) or hw_fl (resize)
  int64_t d[4] = {0, 0, 0, 0};
  int64_t aff_inner = 1, aff_period = 1;  // NORM: weight index = (linear / aff_inner) % aff_period
  int reduce_kind = 0;  // REDUCE: IB200_REDUCE_*; SOFTMAX: 1 when in[1] is a mask applied on load (fill = other, mask row stride = aff_inner)
  float scale = 1.0f, eps = 0.0f;
  int dtype = IB200_F32, dtype2 = IB200_F32;  // element types of the main input and of the output (NORM: of w / b; DROPOUT: of p and seed)
  int transpose_b = 0;
  int act = 0;  // GEMM: IB200_ACT_*; NORM: 1 when the row mean is subtracted (0: rms-norm)
  int64_t batch = 1, batch_stride[3] = {0, 0, 0};  // batched matmul: elements between consecutive A / B / C matrices
  int scratch = -1;  // REDUCE: workspace buffer for the split-row kernel (few, long rows), or -1; GEMM: for the K-split tail tiles
  int flags = 0;     // GEMM: IB200_GEMM_* options
  bool wide = false;  // ELEMENTWISE: values are carried as doubles (f64 tensors, 32/64-bit integers): ew_imm holds the immediates
  std::vector<double> ew_imm;
  std::vector<int> idx_buf;  // GATHER: index buffers; NORM: {residual[, residual bias]} summed while the rows are loaded
  Shape g_dim, g_stride;
  double other = 0.0;     // gather: fill value; dropout: p when it is a constant
  long long seed = 0;     // dropout: the seed when it is a constant; correlation: out_shift when it is a constant
  EwProgram ew;
  std::vector<int> ew_in_buf, ew_out_buf;
  std::vector<int64_t> ew_in_off;  // element offsets into the input buffers
  // ROWFUSE: several of the steps above run as one row program
  RowProgram row;
  std::vector<int> row_in_buf, row_load_buf, row_out_buf;  // per RowInput / RowScalarLoad / RowOutput (-1: none)
  std::vector<int64_t> row_in_off, row_load_off;
};

}  // namespace
}  // namespace ib200

struct ib200_plan {
  std::string kernel_name;
  std::vector<ib200::Buffer> buffers;
  std::vector<ib200::Step> steps;
  std::vector<std::string> arg_names;
  std::vector<std::string> output_names;
  size_t workspace_bytes = 0;
  size_t status_offset = 0;
  bool uses_status = false;
  ib200::Json description;
};

namespace ib200 {
namespace {

class Planner {
 public:
  Planner(const Json& intent, const Json& bindings) : intent_(intent) {
    if (!intent.is_obj()) throw Invalid("intent must be a JSON object");
    if (bindings.is_obj())
      for (auto& kv : bindings.obj)
        if (kv.second.is_num()) bind_[kv.first] = kv.second.num;
  }

  std::unique_ptr<ib200_plan> run() {
    plan_.reset(new ib200_plan);
    const Json* nm = intent_.find("name");
    plan_->kernel_name = nm && nm->is_str() ? nm->s : "intent_fn";
    build();
    if (!match_fused()) lower_general();
    fuse_gemm_epilogues();
    fuse_softmax_masks();
    fuse_rows();
    add_long_row_scratch();
    finish();
    return std::move(plan_);
  }

 private:
  const Json& intent_;
  std::map<std::string, double> bind_;
  std::map<std::string, Json> decl_;       // declared tensors
  std::vector<std::string> decl_order_;
  std::deque<Node> nodes_;  // a deque: references stay valid while lowering appends nodes
  std::map<std::string, int> by_name_;
  std::vector<std::string> outputs_;
  std::vector<int> inputs_;                // node ids of external inputs, first-use order
  std::unique_ptr<ib200_plan> plan_;

  // =============================== phase A: build ==========================================
  int64_t dim_value(const Json& d, const std::string& where) const {
    if (d.is_num()) {
      if (!d.is_int() || d.num < -1 || d.num > (double)kMaxElements) throw Invalid("bad dim in " + where);
      return d.as_int();
    }
    if (d.is_str()) {
      auto it = bind_.find(d.s);
      if (it != bind_.end()) {
        if (!(it->second >= 0 && it->second <= (double)kMaxElements) || std::floor(it->second) != it->second)
          throw Invalid("symbol '" + d.s + "' is bound to something that is not an extent, in " + where);
        return (int64_t)it->second;
      }
      char* end = nullptr;
      long long v = std::strtoll(d.s.c_str(), &end, 10);
      if (end && *end == 0 && !d.s.empty()) return v;
      throw Invalid("unbound symbolic dim '" + d.s + "' in " + where);
    }
    throw Invalid("bad dim in " + where);
  }
  // an axis, a position or a small count: an integral literal that fits an int
  static int small_int(const Json& j, const std::string& where) {
    if (!j.is_int() || std::fabs(j.num) > 2147483647.0) throw Invalid(where + ": expected an integer");
    return (int)j.as_int();
  }
  Shape shape_of(const Json& arr, const std::string& where) const {
    Shape s;
    if (!arr.is_arr()) throw Invalid(where + " must be a list");
    for (auto& d : arr.arr) s.push_back(dim_value(d, where));
    return s;
  }

  // Extents are final when a node is added (reshape has resolved its -1 by then): none negative, and a
  // product that neither wraps nor exceeds what any device holds.
  static constexpr int64_t kMaxElements = (int64_t)1 << 40;
  int add(Node n) {
    int64_t total = 1;
    for (int64_t d : n.shape) {
      if (d < 0) throw Invalid("negative extent in the shape of '" + (n.name.empty() ? n.op : n.name) + "': " + shape_str(n.shape));
      if (__builtin_mul_overflow(total, d, &total) || total > kMaxElements)
        throw Unsupported("tensor '" + (n.name.empty() ? n.op : n.name) + "' is larger than 2^40 elements: " + shape_str(n.shape));
    }
    nodes_.push_back(std::move(n));
    int id = (int)nodes_.size() - 1;
    if (!nodes_[id].name.empty()) by_name_[nodes_[id].name] = id;
    return id;
  }
  int add_const(double v) {
    Node n;
    n.op = "const";
    n.cval = v;
    return add(n);
  }

  int lookup(const std::string& name) {
    auto it = by_name_.find(name);
    if (it != by_name_.end()) return it->second;
    auto d = decl_.find(name);
    if (d == decl_.end()) throw Invalid("undefined value referenced: " + name);
    Node n;
    n.name = name;
    n.op = "input";
    const Json* dt = d->second.find("dtype");
    n.decl_dtype = dtype_code(dt && dt->is_str() ? dt->s : "f32");
    n.dclass = class_of_dtype(n.decl_dtype);
    const Json* sh = d->second.find("shape");
    n.shape = sh ? shape_of(*sh, "tensors." + name + ".shape") : Shape{};
    int id = add(n);
    inputs_.push_back(id);
    return id;
  }

  // declared shape tokens, as the interpreter's match_axis sees them
  bool decl_tokens(const std::string& name, std::vector<const Json*>& toks) const {
    auto d = decl_.find(name);
    if (d == decl_.end()) return false;
    const Json* sh = d->second.find("shape");
    if (!sh || !sh->is_arr()) return false;
    for (auto& t : sh->arr) toks.push_back(&t);
    return true;
  }
  bool token_value(const Json& t, int64_t& v) const {
    if (t.is_num()) { if (!t.is_int()) return false; v = t.as_int(); return true; }
    if (t.is_str()) {
      auto it = bind_.find(t.s);
      if (it != bind_.end() && std::fabs(it->second) < 9e15) { v = (int64_t)it->second; return true; }
    }
    return false;
  }
  // interpreter.py:803-821
  int match_axis(const std::string& vec, const std::string& ten, int ten_rank) const {
    std::vector<const Json*> v, t;
    if (vec.empty() || ten.empty() || !decl_tokens(vec, v) || !decl_tokens(ten, t)) return -1;
    if (v.size() != 1 || (int)t.size() != ten_rank) return -1;
    if (v[0]->is_str()) {
      int hit = -1, n = 0;
      for (int i = 0; i < ten_rank; ++i)
        if (t[i]->is_str() && t[i]->s == v[0]->s) { hit = i; ++n; }
      if (n == 1) return hit;
    }
    int64_t want;
    if (!token_value(*v[0], want)) return -1;
    int hit = -1, n = 0;
    for (int i = 0; i < ten_rank; ++i) {
      int64_t x;
      if (token_value(*t[i], x) && x == want) { hit = i; ++n; }
    }
    return n == 1 ? hit : -1;
  }
  // interpreter.py:832-841: lift a rank-1 operand onto the axis its declared symbol names
  void align(const std::string& an, int& a, const std::string& bn, int& b) {
    auto lift = [&](int vec, const std::string& vn, int ten, const std::string& tn) {
      const int rank = (int)nodes_[ten].shape.size();
      int ax = match_axis(vn, tn, rank);
      if (ax < 0 || nodes_[vec].shape[0] != nodes_[ten].shape[ax]) return vec;
      Node n;
      n.op = "reshape";
      n.in = {vec};
      n.shape.assign(rank, 1);
      n.shape[ax] = nodes_[vec].shape[0];
      n.dclass = nodes_[vec].dclass;
      return add(n);
    };
    if (nodes_[a].shape.size() == 1 && nodes_[b].shape.size() >= 2) a = lift(a, an, b, bn);
    if (nodes_[b].shape.size() == 1 && nodes_[a].shape.size() >= 2) b = lift(b, bn, a, an);
  }
  static Shape broadcast(const Shape& a, const Shape& b, const std::string& what) {
    Shape o(std::max(a.size(), b.size()), 1);
    for (size_t i = 0; i < o.size(); ++i) {
      int64_t x = i < o.size() - a.size() ? 1 : a[i - (o.size() - a.size())];
      int64_t y = i < o.size() - b.size() ? 1 : b[i - (o.size() - b.size())];
      if (x != y && x != 1 && y != 1) throw Invalid(what + ": operands could not be broadcast together: " + shape_str(a) + " vs " + shape_str(b));
      o[i] = x == 1 ? y : x;
    }
    return o;
  }

  // attribute operand: a value name, a bound symbol, or a number (interpreter.py:633-643)
  int scalar_operand(const Json& v, const std::string& where) {
    if (v.is_num()) return add_const(v.num);
    if (v.type == Json::Bool) return add_const(v.b ? 1.0 : 0.0);
    if (v.is_str()) {
      if (by_name_.count(v.s)) return by_name_[v.s];
      auto it = bind_.find(v.s);
      if (it != bind_.end()) return add_const(it->second);
      char* end = nullptr;
      double d = std::strtod(v.s.c_str(), &end);
      if (end && *end == 0 && !v.s.empty()) return add_const(d);
      throw Unsupported(where + ": unresolved scalar value '" + v.s + "' (expression strings must be resolved by the host)");
    }
    throw Invalid(where + ": bad scalar attribute");
  }
  double number_attr(const Json& v, const std::string& where) const {
    if (v.is_num()) return v.num;
    if (v.is_str()) {
      auto it = bind_.find(v.s);
      if (it != bind_.end()) return it->second;
      if (v.s == "eps") return 1e-5;
      char* end = nullptr;
      double d = std::strtod(v.s.c_str(), &end);
      if (end && *end == 0 && !v.s.empty()) return d;
      throw Unsupported(where + ": '" + v.s + "' is an expression; the host must resolve it to a number");
    }
    throw Invalid(where + ": expected a number");
  }

  int build_epilogue(const Json& node, int acc) {
    if (node.is_str()) return node.s == "$x" ? acc : lookup(node.s);
    const Json* opj = node.find("op");
    const Json* ins = node.find("inputs");
    if (!opj || !opj->is_str() || !ins || !ins->is_arr()) throw Invalid("malformed matmul epilogue");
    std::vector<int> args;
    for (auto& i : ins->arr) args.push_back(build_epilogue(i, acc));
    return make_elementwise(opj->s, args, std::vector<std::string>(args.size()), "", nullptr);
  }

  int make_elementwise(const std::string& op, std::vector<int> args, const std::vector<std::string>& names, const std::string& out_name,
                       const Json* attrs) {
    Node n;
    n.name = out_name;
    n.op = op;
    if (kBinary.count(op) || kCompare.count(op) || kLogic2.count(op)) {
      if (args.size() != 2) throw Invalid(op + " requires 2 inputs (or 1+attrs)");
      align(names[0], args[0], names[1], args[1]);
      n.shape = broadcast(nodes_[args[0]].shape, nodes_[args[1]].shape, op);
      if (kBinary.count(op) && nodes_[args[0]].dclass == DC_BOOL && nodes_[args[1]].dclass == DC_BOOL && op != "div") {
        // numpy's arithmetic on two boolean arrays stays boolean: add and max are "or", mul and min are "and",
        // and it refuses to subtract them (verify/interpreter.py:17-23 calls np.add / np.multiply / ... as they are)
        if (op == "add" || op == "max") n.op = "or";
        else if (op == "mul" || op == "min") n.op = "and";
        else throw Unsupported(op + " of two boolean tensors (numpy refuses it)");
        n.dclass = DC_BOOL;
      } else if (kBinary.count(op)) {
        const int ca = nodes_[args[0]].dclass, cb = nodes_[args[1]].dclass;
        const bool a_const = nodes_[args[0]].op == "const", b_const = nodes_[args[1]].op == "const";
        n.dclass = (ca == DC_FLOAT || cb == DC_FLOAT || op == "div") ? DC_FLOAT : DC_INT;
        if (a_const && !b_const && cb == DC_INT && std::floor(nodes_[args[0]].cval) == nodes_[args[0]].cval && op != "div") n.dclass = DC_INT;
        if (b_const && !a_const && ca == DC_INT && std::floor(nodes_[args[1]].cval) == nodes_[args[1]].cval && op != "div") n.dclass = DC_INT;
      } else {
        n.dclass = DC_BOOL;
      }
    } else if (kUnary.count(op) || op == "not" || op == "cast" || op == "identity") {
      if (args.size() != 1) throw Invalid(op + " requires 1 input");
      n.shape = nodes_[args[0]].shape;
      n.dclass = op == "not" ? DC_BOOL : (op == "exp" || op == "rsqrt") ? DC_FLOAT : nodes_[args[0]].dclass;
      if (op == "relu" && n.dclass == DC_BOOL) n.dclass = DC_INT;  // np.maximum(booleans, 0) is an integer array; abs and floor of booleans stay boolean
      if (op == "cast") {
        const Json* to = attrs ? attrs->find("to") : nullptr;
        if (!to || !to->is_str()) throw Invalid("cast requires attrs.to");
        n.cast_to = dtype_code(to->s);
        n.dclass = class_of_dtype(n.cast_to);
      }
    } else if (op == "where") {
      if (args.size() != 3) throw Invalid("where requires 3 inputs (cond, x, y)");
      align(names[0], args[0], names[1], args[1]);
      align(names[0], args[0], names[2], args[2]);
      align(names[1], args[1], names[2], args[2]);
      n.shape = broadcast(broadcast(nodes_[args[0]].shape, nodes_[args[1]].shape, op), nodes_[args[2]].shape, op);
      n.dclass = (nodes_[args[1]].dclass == DC_FLOAT || nodes_[args[2]].dclass == DC_FLOAT) ? DC_FLOAT
                 : (nodes_[args[1]].dclass == DC_INT || nodes_[args[2]].dclass == DC_INT) ? DC_INT : DC_BOOL;
    } else {
      throw Unsupported("elementwise op '" + op + "' is not covered");
    }
    n.in = args;
    return add(n);
  }

  std::vector<int> reduce_axes(const Json* raw, int rank) const {
    std::vector<int> axes;
    if (!raw || raw->is_null()) {
      for (int i = 0; i < rank; ++i) axes.push_back(i);
      return axes;
    }
    std::vector<const Json*> items;
    if (raw->is_arr()) for (auto& j : raw->arr) items.push_back(&j);
    else items.push_back(raw);
    for (auto* j : items) {
      if (j->is_num()) axes.push_back(small_int(*j, "reduce axes"));
      else if (j->is_str() && !j->s.empty() && std::all_of(j->s.begin(), j->s.end(), ::isdigit)) axes.push_back(std::atoi(j->s.c_str()));
    }
    if (axes.empty()) for (int i = 1; i < rank; ++i) axes.push_back(i);
    for (auto& a : axes) {
      if (a < 0) a += rank;
      if (a < 0 || a >= rank) throw Invalid("reduce axis out of range");
    }
    std::sort(axes.begin(), axes.end());
    axes.erase(std::unique(axes.begin(), axes.end()), axes.end());
    return axes;
  }

  void build() {
    const Json* tensors = intent_.find("tensors");
    if (tensors && tensors->is_obj())
      for (auto& kv : tensors->obj) { decl_[kv.first] = kv.second; decl_order_.push_back(kv.first); }
    const Json* ops = intent_.find("ops");
    if (!ops || !ops->is_arr() || ops->arr.empty()) throw Invalid("ops must not be empty");
    for (size_t idx = 0; idx < ops->arr.size(); ++idx) {
      const Json& o = ops->arr[idx];
      const Json* opj = o.find("op");
      const Json* outj = o.find("output");
      if (!opj || !opj->is_str() || !outj || !outj->is_str()) throw Invalid("op[" + std::to_string(idx) + "] needs op and output strings");
      const std::string op = opj->s, out = outj->s, where = "op[" + std::to_string(idx) + "] " + op;
      static const Json empty_obj = Json::object();
      const Json* attrs = o.find("attrs");
      if (!attrs || !attrs->is_obj()) attrs = &empty_obj;
      std::vector<std::string> in_names;
      if (const Json* ins = o.find("inputs"))
        if (ins->is_arr()) for (auto& i : ins->arr) if (i.is_str()) in_names.push_back(i.s);
      std::vector<int> in;
      for (auto& nme : in_names) in.push_back(lookup(nme));
      int id = -1;

      if (is_elementwise(op)) {
        static const std::map<std::string, std::string> scalar_attr = {{"div", "divisor"}, {"add", "addend"}, {"sub", "subtract"},
                                                                       {"mul", "mul_factor"}, {"max", "other"}, {"min", "other"}};
        std::vector<std::string> names = in_names;
        if (kBinary.count(op) && in.size() == 1) {
          const Json* extra = attrs->find(scalar_attr.at(op));
          if (extra) { in.push_back(scalar_operand(*extra, where)); names.push_back(""); }
        }
        id = make_elementwise(op, in, names, out, attrs);
      } else if (op == "identity" || op == "layout_cast") {
        if (in.size() != 1) throw Invalid(where + " requires 1 input");
        Node n; n.name = out; n.op = op; n.in = in; n.shape = nodes_[in[0]].shape; n.dclass = nodes_[in[0]].dclass;
        id = add(n);
      } else if (op == "const") {
        const Json* v = attrs->find("value");
        if (!v) throw Invalid(where + " requires attrs.value");
        if (v->is_str() && by_name_.count(v->s)) {  // alias of an existing value (interpreter.py:527-528)
          Node n; n.name = out; n.op = "identity"; n.in = {by_name_[v->s]}; n.shape = nodes_[n.in[0]].shape; n.dclass = nodes_[n.in[0]].dclass;
          id = add(n);
        } else {
          Node n; n.name = out; n.op = "const";
          n.cval = v->type == Json::Bool ? (v->b ? 1.0 : 0.0) : number_attr(*v, where);
          const Json* dt = attrs->find("dtype");
          if (dt && dt->is_str()) {
            n.dclass = class_of_dtype(dtype_code(dt->s));
            const int code = dtype_code(dt->s);
            // np.array(value, dtype) rounds the literal to the const's dtype (bf16 is carried as f16)
            if (code == IB200_F32) n.cval = (double)(float)n.cval;
            else if (code == IB200_F16 || code == IB200_BF16) n.cval = (double)__half2float(__float2half_rn((float)n.cval));
            else if (n.dclass == DC_INT) n.cval = std::trunc(n.cval);
            else if (n.dclass == DC_BOOL) n.cval = n.cval != 0.0;
          } else {
            n.dclass = (v->type == Json::Bool) ? DC_BOOL : (v->is_num() && v->integral) ? DC_INT : DC_FLOAT;
          }
          id = add(n);
        }
      } else if (op == "iota") {
        Node n; n.name = out; n.op = "iota";
        const Json* sh = attrs->find("shape");
        if (!sh) throw Invalid(where + " requires attrs.shape");
        n.shape = shape_of(*sh, where);
        const Json* ax = attrs->find("axis");
        n.axis = ax && ax->is_num() ? small_int(*ax, where) : 0;
        if (n.axis < 0 || n.axis >= (int)n.shape.size()) throw Invalid(where + ": iota axis out of range");
        const Json* dt = attrs->find("dtype");
        n.dclass = class_of_dtype(dtype_code(dt && dt->is_str() ? dt->s : "i32"));
        id = add(n);
      } else if (op == "reshape") {
        if (in.size() != 1) throw Invalid(where + " requires 1 input");
        Node n; n.name = out; n.op = op; n.in = in; n.dclass = nodes_[in[0]].dclass;
        const Json* sh = attrs->find("shape");
        if (!sh) throw Invalid(where + " requires attrs.shape");
        n.shape = shape_of(*sh, where);
        int64_t known = 1; int infer = -1;
        for (size_t i = 0; i < n.shape.size(); ++i) { if (n.shape[i] == -1) infer = (int)i; else known *= n.shape[i]; }
        if (infer >= 0) n.shape[infer] = known ? numel(nodes_[in[0]].shape) / known : 0;
        if (numel(n.shape) != numel(nodes_[in[0]].shape))
          throw Invalid(where + ": cannot reshape " + shape_str(nodes_[in[0]].shape) + " into " + shape_str(n.shape));
        id = add(n);
      } else if (op == "broadcast_in_dim") {
        if (in.size() != 1) throw Invalid(where + " requires 1 input");
        Node n; n.name = out; n.op = op; n.in = in; n.dclass = nodes_[in[0]].dclass;
        const Json* sh = attrs->find("out_shape");
        const Json* bd = attrs->find("broadcast_dims");
        if (!sh || !bd || !bd->is_arr()) throw Invalid(where + " requires out_shape and broadcast_dims");
        n.shape = shape_of(*sh, where);
        for (auto& j : bd->arr) n.axes.push_back(small_int(j, where));
        for (int a : n.axes) if (a < 0 || a >= (int)n.shape.size()) throw Invalid(where + ": broadcast_dims out of range");
        id = add(n);
      } else if (op == "transpose") {
        if (in.size() != 1) throw Invalid(where + " requires 1 input");
        Node n; n.name = out; n.op = op; n.in = in; n.dclass = nodes_[in[0]].dclass;
        const Json* pj = attrs->find("perm");
        if (!pj || !pj->is_arr() || pj->arr.size() != nodes_[in[0]].shape.size()) throw Invalid(where + " requires attrs.perm of the input's rank");
        for (auto& j : pj->arr) {
          int a = small_int(j, where);
          if (a < 0) a += (int)pj->arr.size();
          if (a < 0 || a >= (int)pj->arr.size()) throw Invalid(where + ": perm out of range");
          if (std::find(n.axes.begin(), n.axes.end(), a) != n.axes.end()) throw Invalid(where + ": repeated axis in perm");
          n.axes.push_back(a);
          n.shape.push_back(nodes_[in[0]].shape[a]);
        }
        id = add(n);
      } else if (op == "reduce_sum" || op == "reduce_max" || op == "reduce_any") {
        if (in.size() != 1) throw Invalid(where + " requires 1 input");
        Node n; n.name = out; n.op = op; n.in = in;
        const Json* raw = attrs->find("axes");
        if (!raw) raw = attrs->find("dims");
        if (!raw) raw = attrs->find("axis");
        const Shape& xs = nodes_[in[0]].shape;
        n.axes = reduce_axes(raw, (int)xs.size());
        const Json* kd = attrs->find("keepdims");
        if (kd && kd->type != Json::Bool && !kd->is_num() && kd->type != Json::Null) throw Invalid(where + ": keepdims must be a boolean");
        n.keepdims = kd && ((kd->type == Json::Bool && kd->b) || (kd->is_num() && kd->num != 0));
        for (int i = 0; i < (int)xs.size(); ++i) {
          const bool red = std::binary_search(n.axes.begin(), n.axes.end(), i);
          if (!red) n.shape.push_back(xs[i]);
          else if (n.keepdims) n.shape.push_back(1);
        }
        const Json* rt = attrs->find("reduction_type");
        if (op == "reduce_sum" && rt && rt->is_str() && rt->s == "any") n.op = "reduce_any";
        n.dclass = n.op == "reduce_any" ? DC_BOOL : nodes_[in[0]].dclass;
        if (n.op == "reduce_sum" && n.dclass == DC_BOOL) n.dclass = DC_INT;  // numpy counts: the sum of booleans is an integer
        if (op == "reduce_sum") {
          const Json* sc = attrs->find("scale");
          if (sc && !sc->is_null()) {
            double f;
            if (sc->is_str() && sc->s == "num_elements" && !bind_.count("num_elements") && bind_.count("group_size") && bind_.count("HW"))
              f = bind_.at("group_size") * bind_.at("HW");
            else f = number_attr(*sc, where + ".scale");
            if (n.op == "reduce_any") {  // np.any(...) * factor is a float
              int rid = add(n);
              n = Node();
              n.op = "mul"; n.in = {rid, add_const(f)}; n.shape = nodes_[rid].shape; n.dclass = DC_FLOAT; n.name = out;
              nodes_[rid].name.clear();
            } else {
              n.scale = f;
              n.dclass = DC_FLOAT;
            }
          }
        }
        id = add(n);
      } else if (op == "softmax") {
        if (in.size() != 1) throw Invalid(where + " requires 1 input");
        Node n; n.name = out; n.op = op; n.in = in; n.shape = nodes_[in[0]].shape; n.dclass = DC_FLOAT;
        const Json* ax = attrs->find("axis");
        n.axis = ax && ax->is_num() ? small_int(*ax, where) : -1;
        if (n.axis < 0) n.axis += (int)n.shape.size();
        if (n.axis < 0 || n.axis >= (int)n.shape.size()) throw Invalid(where + ": axis out of range");
        id = add(n);
      } else if (op == "matmul") {
        if (in.size() != 2) throw Invalid(where + " requires 2 inputs (A, B)");
        Node n; n.op = op; n.in = in; n.dclass = DC_FLOAT;
        if (nodes_[in[0]].dclass == DC_BOOL && nodes_[in[1]].dclass == DC_BOOL)  // np.matmul of booleans is "any(and)", a boolean
          throw Unsupported(where + ": a product of two boolean tensors is not covered");
        auto flag = [&](const char* k) { const Json* j = attrs->find(k); return j && ((j->type == Json::Bool && j->b) || (j->is_num() && j->num != 0)); };
        n.ta = flag("transpose_a");
        n.tb = flag("transpose_b");
        Shape a = nodes_[in[0]].shape, b = nodes_[in[1]].shape;
        if (a.size() < 2 || b.size() < 2) throw Unsupported(where + ": rank-1 operands are not covered (got " + shape_str(a) + " x " + shape_str(b) + ")");
        if (n.ta) std::swap(a[a.size() - 1], a[a.size() - 2]);
        if (n.tb) std::swap(b[b.size() - 1], b[b.size() - 2]);
        if (a.back() != b[b.size() - 2]) throw Invalid(where + ": inner extents differ: " + shape_str(a) + " x " + shape_str(b));
        n.shape = broadcast(Shape(a.begin(), a.end() - 2), Shape(b.begin(), b.end() - 2), op);  // np.matmul broadcasts the batch axes
        n.shape.push_back(a[a.size() - 2]);
        n.shape.push_back(b.back());
        const Json* ep = attrs->find("epilogue");
        if (ep && !ep->is_null() && !(ep->is_str() && ep->s.empty()) && !(ep->is_obj() && ep->obj.empty())) {
          const int mm = add(n);
          const int e = build_epilogue(*ep, mm);
          if (nodes_[e].name.empty()) { nodes_[e].name = out; by_name_[out] = e; id = e; }
          else {  // the epilogue is just another named value: alias it
            Node al; al.op = "identity"; al.in = {e}; al.shape = nodes_[e].shape; al.dclass = nodes_[e].dclass; al.name = out;
            id = add(al);
          }
        } else {
          n.name = out;
          id = add(n);
        }
      } else if (op == "gather") {
        if (in.size() < 2) throw Invalid(where + " requires data + index tensors");
        Node n; n.name = out; n.op = op; n.in = in; n.dclass = nodes_[in[0]].dclass;
        if (in.size() - 1 != nodes_[in[0]].shape.size() || in.size() - 1 > 4)
          throw Unsupported(where + ": one index tensor per data axis (at most 4) is what the gather kernel covers");
        n.shape = nodes_[in[1]].shape;
        for (size_t k = 2; k < in.size(); ++k)
          if (nodes_[in[k]].shape != n.shape) throw Unsupported(where + ": index tensors of different shapes are not covered");
        const Json* ov = attrs->find("other_value");
        n.cval = ov && ov->is_num() ? ov->num : 0.0;
        id = add(n);
      } else if (op == "rope") {
        // x[SEQ, B, H, D even], cos / sin [SEQ, D/2]  (verify/interpreter.py:455-477)
        if (in.size() != 3) throw Invalid(where + " requires x, cos, sin");
        const Shape &xs = nodes_[in[0]].shape, &cs = nodes_[in[1]].shape, &ss = nodes_[in[2]].shape;
        if (xs.size() != 4 || cs.size() != 2 || ss.size() != 2 || xs[3] % 2)
          throw Invalid(where + ": rope expects x[SEQ,B,H,D even] and cos/sin[SEQ,D/2]; got " + shape_str(xs) + " " + shape_str(cs) + " " + shape_str(ss));
        if (cs[0] != xs[0] || cs[1] != xs[3] / 2 || ss != cs) throw Invalid(where + ": rope cos/sin shape mismatch");
        Node n; n.name = out; n.op = op; n.in = in; n.shape = xs; n.dclass = DC_FLOAT;
        id = add(n);
      } else if (op == "correlation" || op == "resize" || op == "warp") {
        // int8 image ops; the output shape is the declared one (verify/interpreter.py:330-454)
        auto dd = decl_.find(out);
        if (dd == decl_.end() || !dd->second.find("shape")) throw Invalid(where + ": the output tensor must be declared");
        Node n; n.name = out; n.op = op; n.in = in; n.dclass = DC_INT;
        n.shape = shape_of(*dd->second.find("shape"), where);
        if (n.shape.size() != 3) throw Invalid(where + ": " + op + " output must be rank-3, got " + shape_str(n.shape));
        const size_t want_in = op == "correlation" ? 3 : op == "resize" ? 1 : 2;
        if (in.size() != want_in) throw Invalid(where + ": " + op + " requires " + std::to_string(want_in) + " input(s)");
        const Shape& src = nodes_[in[0]].shape;
        if (src.size() != 3) throw Invalid(where + ": " + op + " input must be rank-3, got " + shape_str(src));
        if (op == "correlation") {
          if (nodes_[in[1]].shape != src) throw Invalid(where + ": correlation inputs shape mismatch: " + shape_str(src) + " vs " + shape_str(nodes_[in[1]].shape));
          if (src[1] != n.shape[1] || src[2] != n.shape[2]) throw Invalid(where + ": correlation spatial shape mismatch");
          if (numel(nodes_[in[2]].shape) != 1) throw Invalid(where + ": out_shift must be a scalar");
          if (numel(n.shape) > 0 && src[0] > 0 && n.shape[0] - 1 > n.shape[2]) throw Invalid(where + ": correlation output channels need shifts beyond the width");
        } else if (op == "resize") {
          if (n.shape[0] != src[0]) throw Invalid(where + ": resize channel mismatch");
          if (n.shape[1] != 2 * src[1] || n.shape[2] != 2 * src[2]) throw Invalid(where + ": resize currently expects 2x upsample: src=" + shape_str(src) + " out=" + shape_str(n.shape));
          const Json* fl = attrs->find("hw_fl");
          n.axis = fl && fl->is_num() ? small_int(*fl, where) : 7;
        } else {
          if (n.shape != src) throw Invalid(where + ": warp output shape mismatch: src=" + shape_str(src) + " out=" + shape_str(n.shape));
          if (nodes_[in[1]].shape != Shape{src[1], src[2]}) throw Invalid(where + ": warp offset shape mismatch");
        }
        id = add(n);
      } else if (op == "dropout") {
        // x, p (scalar), seed (scalar); attrs.n_rounds, default 10  (verify/interpreter.py:697-742)
        if (in.size() != 3) throw Invalid(where + " requires x, p, seed");
        if (numel(nodes_[in[1]].shape) != 1 || numel(nodes_[in[2]].shape) != 1) throw Invalid(where + ": p and seed must be scalars");
        Node n; n.name = out; n.op = op; n.in = in; n.shape = nodes_[in[0]].shape; n.dclass = DC_FLOAT;
        const Json* nr = attrs->find("n_rounds");
        n.axis = nr && nr->is_num() && small_int(*nr, where) > 0 ? small_int(*nr, where) : 10;
        id = add(n);
      } else {
        throw Unsupported("op '" + op + "' is not covered by the B200 kernels (name=" + plan_->kernel_name + ")");
      }
      // declared dtype of the produced tensor, if any
      auto d = decl_.find(out);
      if (d != decl_.end()) {
        const Json* dt = d->second.find("dtype");
        if (dt && dt->is_str()) nodes_[by_name_[out]].decl_dtype = dtype_code(dt->s);
      }
    }
    const Json* outs = intent_.find("outputs");
    if (outs && outs->is_arr()) for (auto& j : outs->arr) if (j.is_str()) outputs_.push_back(j.s);
    if (outputs_.empty()) outputs_.push_back(ops->arr.back().find("output")->s);
    for (size_t i = 0; i < outputs_.size(); ++i)
      for (size_t k = 0; k < i; ++k)
        if (outputs_[k] == outputs_[i]) throw Invalid("output '" + outputs_[i] + "' is listed twice");
    for (auto& o : outputs_) {
      if (!by_name_.count(o)) throw Invalid("output '" + o + "' is never produced");
      // an op consumed it before anything produced it, so it entered as an external input: the interpreter would stop
      // at that op with an undefined value unless the caller supplied the output as an input
      if (nodes_[by_name_[o]].op == "input") throw Invalid("output '" + o + "' is consumed but no op produces it");
      if (!decl_.count(o)) throw Invalid("outputs entry not found in tensors: " + o);
    }
    // argument list: external inputs in first-use order, then outputs
    for (int id : inputs_) {
      Buffer b; b.is_arg = true; b.arg_index = (int)plan_->arg_names.size(); b.dtype = nodes_[id].decl_dtype; b.name = nodes_[id].name;
      b.bytes = (size_t)numel(nodes_[id].shape) * dtype_size(b.dtype);
      plan_->buffers.push_back(b);
      plan_->arg_names.push_back(nodes_[id].name);
      nodes_[id].repr = Node::STRIDED;
      nodes_[id].view.buffer = (int)plan_->buffers.size() - 1;
      nodes_[id].view.shape = nodes_[id].shape;
      nodes_[id].view.strides = contiguous_strides(nodes_[id].shape);
    }
    for (auto& o : outputs_) {
      const int id = by_name_[o];
      Buffer b; b.is_arg = true; b.arg_index = (int)plan_->arg_names.size(); b.name = o;
      b.dtype = nodes_[id].decl_dtype >= 0 ? nodes_[id].decl_dtype : storage_of_class(nodes_[id].dclass);
      b.bytes = (size_t)numel(nodes_[id].shape) * dtype_size(b.dtype);
      plan_->buffers.push_back(b);
      out_buffer_[o] = (int)plan_->buffers.size() - 1;
      plan_->arg_names.push_back(o);
      plan_->output_names.push_back(o);
    }
  }
  std::map<std::string, int> out_buffer_;

  // =============================== helpers shared by B and C ================================
  int skip_views(int id) const {
    while (kViews.count(nodes_[id].op) && nodes_[id].op != "transpose") id = nodes_[id].in[0];
    return id;
  }
  int skip_reshapes(int id) const {
    while (nodes_[id].op == "reshape" || nodes_[id].op == "identity" || nodes_[id].op == "layout_cast") id = nodes_[id].in[0];
    return id;
  }
  bool const_value(int id, double& v) const {
    id = skip_views(id);
    if (nodes_[id].op != "const") return false;
    v = nodes_[id].cval;
    return true;
  }
  bool is_input(int id) const { return nodes_[id].op == "input"; }

  // strides of `id` (which must bottom out at an external input through view ops only)
  // expressed over id's own shape; false if it is not a pure view of an input
  bool input_view(int id, View& v) const {
    const Node& n = nodes_[id];
    if (n.op == "input") { v = n.view; return true; }
    if (!kViews.count(n.op)) return false;
    View src;
    if (!input_view(n.in[0], src)) return false;
    return apply_view(n, src, v);
  }
  bool apply_view(const Node& n, const View& src, View& v) const {
    v.buffer = src.buffer;
    v.offset = src.offset;
    v.shape = n.shape;
    if (n.op == "identity" || n.op == "layout_cast") { v.strides = src.strides; return true; }
    if (n.op == "reshape") return reshape_view(src.shape, src.strides, n.shape, v.strides);
    if (n.op == "transpose") {
      v.strides.resize(n.shape.size());
      for (size_t i = 0; i < n.axes.size(); ++i) v.strides[i] = src.strides[n.axes[i]];
      return true;
    }
    if (n.op == "broadcast_in_dim") {
      Shape staged(n.shape.size(), 1), st;
      for (size_t i = 0; i < n.axes.size(); ++i)
        if (i < src.shape.size()) staged[n.axes[i]] = src.shape[i];
      if (!reshape_view(src.shape, src.strides, staged, st)) return false;
      v.strides.resize(n.shape.size());
      for (size_t d = 0; d < n.shape.size(); ++d) {
        if (staged[d] == n.shape[d]) v.strides[d] = staged[d] == 1 ? 0 : st[d];
        else if (staged[d] == 1) v.strides[d] = 0;
        else throw Invalid("broadcast_in_dim: cannot broadcast " + shape_str(staged) + " to " + shape_str(n.shape));
      }
      return true;
    }
    return false;
  }
  // strides of a view `v` right-aligned and broadcast onto `target`
  static bool broadcast_strides(const View& v, const Shape& target, Shape& out) {
    out.assign(target.size(), 0);
    if (v.shape.size() > target.size()) return false;
    const size_t lead = target.size() - v.shape.size();
    for (size_t i = 0; i < v.shape.size(); ++i) {
      if (v.shape[i] == target[lead + i]) out[lead + i] = v.shape[i] == 1 ? 0 : v.strides[i];
      else if (v.shape[i] == 1) out[lead + i] = 0;
      else return false;
    }
    return true;
  }

  // softmax / normalisation over rows too long for the resident kernels and too few (or too large) for one streaming
  // CTA per row: the rows are cut into segments, whose statistics travel through the workspace
  void add_long_row_scratch() {
    for (Step& s : plan_->steps) {
      size_t bytes = 0;
      if (s.kind == Step::SOFTMAX && s.reduce_kind == 0) bytes = softmax_scratch_bytes(s.d[0], s.d[1], (int)dtype_size(s.dtype));
      else if (s.kind == Step::NORM && s.idx_buf.empty() && s.flags == 0) bytes = norm_scratch_bytes(s.d[0], s.d[1], (int)dtype_size(s.dtype));
      if (bytes == 0 || s.scratch >= 0) continue;
      s.scratch = new_workspace_buffer(IB200_U8, (int64_t)bytes, "row segment statistics");
      s.label += "(segmented)";
    }
  }

  // reductions whose results alone give too few CTAs are split along the reduced axis; the partial results go through the workspace
  void add_reduce_scratch(Step& s) {
    const size_t bytes = reduce_scratch_bytes(s.d[0], s.d[1], s.d[2]);
    if (bytes == 0) return;
    s.scratch = new_workspace_buffer(IB200_U8, (int64_t)bytes, "reduce scratch");
    s.label += s.d[2] == 1 ? "(split rows)" : "(split columns)";
  }

  int new_workspace_buffer(int dtype, int64_t elements, const std::string& name) {
    Buffer b;
    b.dtype = dtype;
    b.bytes = (size_t)elements * dtype_size(dtype);
    b.ws_offset = plan_->workspace_bytes;
    b.name = name;
    plan_->workspace_bytes += (b.bytes + 255) & ~(size_t)255;
    plan_->buffers.push_back(b);
    return (int)plan_->buffers.size() - 1;
  }
  // where a non-elementwise op writes its result: straight into the output argument when the
  // value is a declared graph output, else into the workspace
  int result_buffer(int id, int dtype_if_temp) {
    const Node& n = nodes_[id];
    auto it = out_buffer_.find(n.name);
    if (!n.name.empty() && it != out_buffer_.end() && !out_written_.count(n.name)) {
      out_written_.insert(n.name);
      return it->second;
    }
    return new_workspace_buffer(dtype_if_temp, numel(n.shape), n.name);
  }
  std::set<std::string> out_written_;
  void set_strided(int id, int buffer) {
    Node& n = nodes_[id];
    n.repr = Node::STRIDED;
    n.view = View();
    n.view.buffer = buffer;
    n.view.shape = n.shape;
    n.view.strides = contiguous_strides(n.shape);
  }

  // =============================== phase B: fused patterns ==================================
  static bool close(double a, double b) { return std::fabs(a - b) <= 1e-6 * std::max(1.0, std::fabs(b)); }

  // `id` == mean over `axes`-trailing elements of Z: div(sum, L) | mul(sum, 1/L) | sum{scale 1/L}
  bool match_mean(int id, int& z, int& red, int64_t& L) const {
    id = skip_views(id);
    const Node& n = nodes_[id];
    auto sum_of = [&](int s, double factor) {
      s = skip_views(s);
      const Node& r = nodes_[s];
      if (r.op != "reduce_sum") return false;
      const Shape& xs = nodes_[r.in[0]].shape;
      int64_t l = 1;
      for (int a : r.axes) l *= xs[a];
      // trailing, adjacent axes only
      for (size_t i = 0; i < r.axes.size(); ++i)
        if (r.axes[i] != (int)xs.size() - (int)r.axes.size() + (int)i) return false;
      if (l <= 0 || !close(r.scale * factor * (double)l, 1.0)) return false;
      z = r.in[0]; red = s; L = l;
      return true;
    };
    double c;
    if (n.op == "reduce_sum") return sum_of(id, 1.0);
    if (n.op == "div" && const_value(n.in[1], c) && c != 0) return sum_of(n.in[0], 1.0 / c);
    if (n.op == "mul") {
      if (const_value(n.in[1], c)) return sum_of(n.in[0], c);
      if (const_value(n.in[0], c)) return sum_of(n.in[1], c);
    }
    return false;
  }

  // is `id` (used as an operand against a full tensor of shape `full`, rows x L) a per-row
  // scalar, i.e. does its right-aligned broadcast have contiguous row strides and stride 0
  // along the reduced trailing elements?
  bool per_row_operand(int id, int base, const Shape& full, int64_t L) const {
    // walk the view chain from id down to base, composing views over base's own shape
    std::vector<int> chain;
    int cur = id;
    while (cur != base) {
      if (!kViews.count(nodes_[cur].op) || nodes_[cur].op == "transpose") return false;
      chain.push_back(cur);
      cur = nodes_[cur].in[0];
    }
    View v;
    v.shape = nodes_[base].shape;
    v.strides = contiguous_strides(v.shape);
    for (auto it = chain.rbegin(); it != chain.rend(); ++it) {
      View nv;
      if (!apply_view(nodes_[*it], v, nv)) return false;
      v = nv;
    }
    Shape st;
    if (!broadcast_strides(v, full, st)) return false;
    // linearise: element (row r, col j) must read base element r
    int64_t inner = 1;
    int d = (int)full.size() - 1;
    for (; d >= 0 && inner < L; --d) {
      if (full[d] != 1 && st[d] != 0) return false;
      inner *= full[d];
    }
    if (inner != L) return false;
    int64_t acc = 1;
    for (; d >= 0; --d) {
      if (full[d] != 1 && st[d] != acc) return false;
      acc *= full[d];
    }
    return acc == numel(nodes_[base].shape);
  }

  // affine operand W used against a full tensor: widx = (linear / inner) % period
  bool affine_operand(int id, const Shape& full, int& input_id, int64_t& inner, int64_t& period) const {
    View v;
    if (!input_view(id, v)) return false;
    input_id = -1;
    for (int i : inputs_) if (nodes_[i].view.buffer == v.buffer) input_id = i;
    if (input_id < 0 || v.offset != 0) return false;
    Shape st;
    if (!broadcast_strides(v, full, st)) return false;
    period = numel(nodes_[input_id].shape);
    inner = 1;
    int d = (int)full.size() - 1;
    for (; d >= 0 && (full[d] == 1 || st[d] == 0); --d) inner *= full[d];
    int64_t acc = 1;
    for (; d >= 0 && acc < period; --d) {
      if (full[d] != 1 && st[d] != acc) return false;
      acc *= full[d];
    }
    if (acc != period) return false;
    for (; d >= 0; --d)
      if (full[d] != 1 && st[d] != 0) return false;
    return true;
  }

  bool all_outputs_in(const std::map<std::string, int>& covered) const {
    for (auto& o : outputs_) if (!covered.count(o)) return false;
    return true;
  }
  int float_dtype_of_input(int id) const {
    const int dt = nodes_[id].decl_dtype;
    return (dt == IB200_F32 || dt == IB200_BF16 || dt == IB200_F16) ? dt : -1;
  }

  bool match_fused() { return match_softmax() || match_norm() || match_gemm() || match_any(); }

  bool match_any() {
    if (outputs_.size() != 1) return false;
    const int out = by_name_[outputs_[0]];
    const Node& r = nodes_[out];
    if (r.op != "reduce_any") return false;
    int x = skip_reshapes(r.in[0]);
    const Node& c = nodes_[x];
    if (c.op == "ne") {
      double z;
      if (const_value(c.in[1], z) && z == 0.0) x = skip_reshapes(c.in[0]);
      else if (const_value(c.in[0], z) && z == 0.0) x = skip_reshapes(c.in[1]);
      else return false;
      if (nodes_[x].shape != nodes_[r.in[0]].shape && numel(nodes_[x].shape) != numel(nodes_[r.in[0]].shape)) return false;
    }
    if (!is_input(x) || numel(nodes_[x].shape) != numel(nodes_[r.in[0]].shape)) return false;
    const int xd = nodes_[x].decl_dtype;
    if (!(xd == IB200_F32 || xd == IB200_BF16 || xd == IB200_F16 || xd == IB200_BOOL)) return false;
    const Shape& xs = nodes_[r.in[0]].shape;
    if (r.axes.empty()) return false;
    for (size_t i = 1; i < r.axes.size(); ++i) if (r.axes[i] != r.axes[i - 1] + 1) return false;
    Step s;
    s.kind = Step::REDUCE;
    s.label = "reduce_any";
    s.reduce_kind = IB200_REDUCE_ANY;
    s.d[0] = s.d[1] = s.d[2] = 1;
    for (int i = 0; i < (int)xs.size(); ++i) (i < r.axes.front() ? s.d[0] : i > r.axes.back() ? s.d[2] : s.d[1]) *= xs[i];
    s.in[0] = nodes_[x].view.buffer;
    s.out[0] = out_buffer_[outputs_[0]];
    s.dtype = xd;
    s.dtype2 = plan_->buffers[s.out[0]].dtype;
    if (s.dtype2 != IB200_BOOL) return false;
    add_reduce_scratch(s);
    plan_->steps.push_back(s);
    return true;
  }

  bool match_softmax() {
    // locate the main output: softmax(X) or div(E, S)
    for (auto& oname : outputs_) {
      const int out = skip_reshapes(by_name_[oname]);
      const Node& y = nodes_[out];
      int x = -1, rmax = -1, rsum = -1;
      if (y.op == "softmax") {
        x = skip_reshapes(y.in[0]);
        if (y.axis != (int)y.shape.size() - 1) continue;
      } else if (y.op == "div") {
        const int e = skip_views(y.in[0]);
        const Node& en = nodes_[e];
        if (en.op != "exp") continue;
        const int sub = skip_views(en.in[0]);
        if (nodes_[sub].op != "sub") continue;
        x = skip_reshapes(nodes_[sub].in[0]);
        rmax = skip_views(nodes_[sub].in[1]);
        rsum = skip_views(y.in[1]);
        const Node &mx = nodes_[rmax], &sm = nodes_[rsum];
        if (mx.op != "reduce_max" || sm.op != "reduce_sum" || sm.scale != 1.0) continue;
        if (skip_reshapes(mx.in[0]) != x || skip_views(sm.in[0]) != e) continue;
        const int rank = (int)nodes_[mx.in[0]].shape.size();
        if (mx.axes != std::vector<int>{rank - 1} || sm.axes != std::vector<int>{(int)nodes_[sm.in[0]].shape.size() - 1}) continue;
        const int64_t L = nodes_[mx.in[0]].shape.back();
        if (nodes_[e].shape.empty() || nodes_[e].shape.back() != L || y.shape != nodes_[e].shape) continue;
        if (!per_row_operand(nodes_[sub].in[1], rmax, nodes_[sub].shape, L)) continue;
        if (!per_row_operand(y.in[1], rsum, y.shape, L)) continue;
      } else {
        continue;
      }
      if (x < 0 || !is_input(x) || float_dtype_of_input(x) < 0) continue;
      if (numel(nodes_[x].shape) != numel(y.shape) || y.shape.empty()) continue;
      std::map<std::string, int> covered;
      covered[oname] = 0;
      Step s;
      s.kind = Step::SOFTMAX;
      s.label = "softmax";
      s.d[1] = y.shape.back();
      s.d[0] = s.d[1] ? numel(y.shape) / s.d[1] : 0;
      s.in[0] = nodes_[x].view.buffer;
      s.out[0] = out_buffer_[oname];
      s.dtype = nodes_[x].decl_dtype;
      s.dtype2 = plan_->buffers[s.out[0]].dtype;
      if (s.dtype2 != s.dtype && !(s.dtype2 == IB200_F32 && s.dtype != IB200_F32)) continue;
      for (auto& other : outputs_) {
        if (other == oname) continue;
        const int o = skip_reshapes(by_name_[other]);
        const int buf = out_buffer_[other];
        if (plan_->buffers[buf].dtype != IB200_F32) continue;
        if (rmax >= 0 && o == rmax) { s.out[1] = buf; covered[other] = 1; }
        else if (rsum >= 0 && o == rsum) { s.out[2] = buf; covered[other] = 2; }
      }
      if (!all_outputs_in(covered)) continue;
      plan_->steps.push_back(s);
      return true;
    }
    return false;
  }

  // x = a + b, or (a + b) + v with v a vector along the row: a and b dense f32 views of inputs with x's
  // element count, v an f32 input of L elements.  The row kernels sum these as they load a row.
  bool residual_sum(int x, int64_t L, int& a_buf, int& b_buf, int& v_buf) const {
    auto dense_input = [&](int id, int& buf) {
      View v;
      if (!input_view(id, v) || !v.contiguous() || numel(v.shape) != numel(nodes_[x].shape)) return false;
      if (plan_->buffers[v.buffer].dtype != IB200_F32) return false;
      buf = v.buffer;
      return true;
    };
    auto pair = [&](int id) {
      id = skip_reshapes(id);
      const Node& n = nodes_[id];
      return n.op == "add" && n.in.size() == 2 && dense_input(n.in[0], a_buf) && dense_input(n.in[1], b_buf);
    };
    v_buf = -1;
    if (pair(x)) return true;
    const Node& n = nodes_[skip_reshapes(x)];
    if (n.op != "add" || n.in.size() != 2) return false;
    for (int k = 0; k < 2; ++k) {
      int vin = -1;
      int64_t inner = 0, period = 0;
      if (!pair(n.in[k])) continue;
      for (auto& o : outputs_) if (by_name_.at(o) == skip_reshapes(n.in[k])) return false;  // the inner sum is itself returned
      if (!affine_operand(n.in[1 - k], nodes_[x].shape, vin, inner, period) || inner != 1 || period != L) continue;
      if (nodes_[vin].decl_dtype != IB200_F32) continue;
      v_buf = nodes_[vin].view.buffer;
      return true;
    }
    return false;
  }

  bool match_norm() {
    for (auto& oname : outputs_) {
      int y = skip_reshapes(by_name_[oname]);
      int w = -1, b = -1;
      // Y = XH*W + B | XH*W | XH + B | XH
      auto is_xhat = [&](int id, int& d, int& rs) {
        id = skip_reshapes(id);
        const Node& n = nodes_[id];
        if (n.op != "mul") return false;
        for (int k = 0; k < 2; ++k) {
          const int cand_d = skip_reshapes(n.in[k]), cand_rs = skip_views(n.in[1 - k]);
          if (nodes_[cand_d].op == "sub" && nodes_[cand_rs].op == "rsqrt") { d = cand_d; rs = cand_rs; xh_rs_operand_ = n.in[1 - k]; xh_node_ = id; return true; }
        }
        // rms-norm: X * rsqrt(mean(X*X) + eps), nothing subtracted
        for (int k = 0; k < 2; ++k) {
          const int cand_d = skip_reshapes(n.in[k]), cand_rs = skip_views(n.in[1 - k]);
          if (nodes_[cand_rs].op == "rsqrt" && nodes_[cand_d].op != "rsqrt" && numel(nodes_[cand_d].shape) == numel(n.shape)) {
            d = cand_d; rs = cand_rs; xh_rs_operand_ = n.in[1 - k]; xh_node_ = id;
            return true;
          }
        }
        return false;
      };
      int d = -1, rs = -1, xh = -1;
      Shape w_full;
      // a ReLU inside the normalisation rides in the kernel: on the affine result (Y = relu(XH*W + B)) or on the
      // normalised value (Y = relu(XH)*W + B), as long as the value under it is not itself a graph output
      int act_pos = 0;
      auto through_relu = [&](int id, int pos) {
        id = skip_reshapes(id);
        if (nodes_[id].op != "relu" || act_pos != 0) return id;
        for (auto& other : outputs_)
          if (skip_reshapes(by_name_[other]) == skip_reshapes(nodes_[id].in[0])) return id;
        act_pos = pos;
        return skip_reshapes(nodes_[id].in[0]);
      };
      y = through_relu(y, 2);
      {
        const Node& n = nodes_[y];
        int scaled = y;
        if (n.op == "add") {
          for (int k = 0; k < 2; ++k) {
            View tmp;
            if (input_view(n.in[k], tmp) && !input_view(n.in[1 - k], tmp)) { b = n.in[k]; scaled = skip_reshapes(n.in[1 - k]); break; }
          }
          if (b < 0) continue;
        }
        const Node& m = nodes_[scaled];
        if (is_xhat(scaled, d, rs)) xh = scaled;
        else if (m.op == "mul") {
          for (int k = 0; k < 2; ++k) {
            View tmp;
            if (!input_view(m.in[k], tmp)) continue;
            const int saved = act_pos;
            const int cand = through_relu(m.in[1 - k], 1);
            if (is_xhat(cand, d, rs)) { w = m.in[k]; w_full = m.shape; xh = cand; break; }
            act_pos = saved;
          }
        } else if (m.op == "relu" && act_pos == 0) {  // Y = relu(XH) [+ B]
          const int cand = through_relu(scaled, 1);
          if (cand != scaled && is_xhat(cand, d, rs)) xh = cand;
        }
        if (xh < 0) continue;
      }
      // D = X - mean(X); for rms-norm D is X itself
      const bool centred = nodes_[d].op == "sub";
      const Node& dn = nodes_[d];
      // X is an external input, or any float value computed from inputs (a residual sum, say):
      // that value is then computed first, by the general lowering, into the workspace (or into
      // its own output buffer when the graph also returns it)
      const int x = centred ? skip_reshapes(dn.in[0]) : d;
      const bool x_is_input = is_input(x);
      int x_dtype = x_is_input ? float_dtype_of_input(x) : -1;
      if (!x_is_input) {
        if (nodes_[x].dclass != DC_FLOAT || nodes_[x].op == "const") continue;
        x_dtype = IB200_F32;
        for (auto& other : outputs_)
          if (by_name_[other] == x) x_dtype = plan_->buffers[out_buffer_[other]].dtype;
        if (!(x_dtype == IB200_F32 || x_dtype == IB200_BF16 || x_dtype == IB200_F16)) continue;
      }
      if (x_dtype < 0) continue;
      int z1, red1, z2, red2;
      int64_t L1 = -1, L2;
      if (centred && (!match_mean(dn.in[1], z1, red1, L1) || skip_reshapes(z1) != x)) continue;
      const int mu = centred ? skip_views(dn.in[1]) : -1;
      // RS = rsqrt(mean(D*D) + eps)
      const Node& rn = nodes_[rs];
      const int ve = skip_views(rn.in[0]);
      if (nodes_[ve].op != "add") continue;
      double eps = 0;
      int var = -1;
      if (const_value(nodes_[ve].in[1], eps)) var = nodes_[ve].in[0];
      else if (const_value(nodes_[ve].in[0], eps)) var = nodes_[ve].in[1];
      else continue;
      if (!match_mean(var, z2, red2, L2) || (centred && L2 != L1)) continue;
      if (!centred) L1 = L2;
      const int sq = skip_reshapes(z2);
      if (nodes_[sq].op != "mul" || skip_reshapes(nodes_[sq].in[0]) != d || skip_reshapes(nodes_[sq].in[1]) != d) continue;
      const int64_t L = L1, total = numel(nodes_[x].shape);
      if (L <= 0 || total % L != 0 || numel(dn.shape) != total || numel(nodes_[y].shape) != total) continue;
      // the mean and rstd operands must broadcast per row
      if (centred && !per_row_operand(dn.in[1], mu, dn.shape, L)) continue;
      if (!per_row_operand(xh_rs_operand_, rs, nodes_[xh_node_].shape, L)) continue;
      // row-major views only between X, D, XH and Y (no transposes): guaranteed by skip_reshapes
      int w_in = -1, b_in = -1;
      int64_t inner = 1, period = 1, inner2 = 1, period2 = 1;
      if (w >= 0 && !affine_operand(w, w_full, w_in, inner, period)) continue;
      if (b >= 0 && !affine_operand(b, nodes_[y].shape, b_in, inner2, period2)) continue;
      if (w >= 0 && b >= 0 && (inner != inner2 || period != period2)) continue;
      if (w < 0 && b >= 0) { inner = inner2; period = period2; }
      const int wd = w_in >= 0 ? nodes_[w_in].decl_dtype : b_in >= 0 ? nodes_[b_in].decl_dtype : x_dtype;
      if (w_in >= 0 && b_in >= 0 && nodes_[w_in].decl_dtype != nodes_[b_in].decl_dtype) continue;
      if (!(wd == x_dtype || wd == IB200_F32)) continue;

      std::map<std::string, int> covered;
      covered[oname] = 0;
      Step s;
      s.kind = Step::NORM;
      s.label = !centred ? "rmsnorm" : (inner == 1 && period == L) || (w < 0 && b < 0) ? "layernorm" : "groupnorm";
      if (act_pos) s.label += "+relu";
      s.flags = act_pos;        // NORM steps: where a ReLU sits (1: on the normalised value, 2: on the affine result)
      s.act = centred ? 1 : 0;  // NORM steps: whether the row mean is subtracted
      s.d[0] = total / L;
      s.d[1] = L;
      s.aff_inner = inner;
      s.aff_period = period;
      s.eps = (float)eps;
      s.in[1] = w_in >= 0 ? nodes_[w_in].view.buffer : -1;
      s.in[2] = b_in >= 0 ? nodes_[b_in].view.buffer : -1;
      s.out[0] = out_buffer_[oname];
      s.dtype = x_dtype;
      s.dtype2 = wd;
      if (plan_->buffers[s.out[0]].dtype != s.dtype) continue;
      for (auto& other : outputs_) {
        if (other == oname) continue;
        if (!x_is_input && by_name_[other] == x) { covered[other] = 3; continue; }  // written when X is computed
        const int o = skip_reshapes(by_name_[other]);
        const int buf = out_buffer_[other];
        if (plan_->buffers[buf].dtype != IB200_F32 || numel(nodes_[by_name_[other]].shape) != s.d[0]) continue;
        if (centred && o == mu) { s.out[1] = buf; covered[other] = 1; }
        else if (o == rs) { s.out[2] = buf; covered[other] = 2; }
      }
      if (!all_outputs_in(covered)) continue;
      int res_a = -1, res_b = -1, res_v = -1;
      bool x_is_output = false;
      for (auto& other : outputs_) x_is_output |= by_name_[other] == x;
      if (!x_is_input && !x_is_output && L <= 16384 && x_dtype == IB200_F32 && wd == IB200_F32 && residual_sum(x, L, res_a, res_b, res_v)) {
        // the residual sum is formed by the norm kernel itself while it loads the rows
        s.in[0] = res_a;
        s.idx_buf = {res_b};
        if (res_v >= 0) s.idx_buf.push_back(res_v);
        s.label = "residual+" + s.label;
        plan_->uses_status = true;
        plan_->steps.push_back(s);
        return true;
      }
      if (!x_is_input) {  // everything checked: now emit the kernel(s) that compute X
        std::function<void(int)> lower_deps = [&](int id) {
          if (nodes_[id].repr != Node::NONE) return;
          for (int c : nodes_[id].in) lower_deps(c);
          lower_node(id);
        };
        lower_deps(x);
        materialise_contiguous(x);
        if (plan_->buffers[nodes_[x].view.buffer].dtype != x_dtype) throw Unsupported("internal: normalised value landed in an unexpected dtype");
      }
      s.in[0] = nodes_[x].view.buffer;
      plan_->uses_status = true;
      plan_->steps.push_back(s);
      return true;
    }
    return false;
  }
  int xh_rs_operand_ = -1, xh_node_ = -1;
  bool match_gemm() {
    if (outputs_.size() != 1) return false;
    int cur = skip_reshapes(by_name_[outputs_[0]]);
    int act = IB200_ACT_NONE, bias = -1;
    if (nodes_[cur].op == "relu") { act = IB200_ACT_RELU; cur = skip_reshapes(nodes_[cur].in[0]); }
    int mm = -1;
    if (nodes_[cur].op == "add") {
      for (int k = 0; k < 2; ++k) {
        const int c = skip_reshapes(nodes_[cur].in[k]);
        View tmp;
        if (nodes_[c].op == "matmul" && input_view(nodes_[cur].in[1 - k], tmp)) { mm = c; bias = nodes_[cur].in[1 - k]; }
      }
      if (mm < 0) return false;
    } else if (nodes_[cur].op == "matmul") {
      mm = cur;
    } else {
      return false;
    }
    const Node& m = nodes_[mm];
    if (m.ta || m.shape.size() != 2) return false;  // A^T and batched products: left to the general path
    const int a = m.in[0], b = m.in[1];
    if (!is_input(a) || !is_input(b)) return false;
    const int in_dt = nodes_[a].decl_dtype;
    if (in_dt != nodes_[b].decl_dtype || !(in_dt == IB200_F32 || in_dt == IB200_BF16 || in_dt == IB200_F16)) return false;
    const int out_buf = out_buffer_[outputs_[0]];
    const int out_dt = plan_->buffers[out_buf].dtype;
    if (!(out_dt == IB200_F32 || (out_dt == in_dt && in_dt != IB200_F32))) return false;
    if (numel(nodes_[by_name_[outputs_[0]]].shape) != numel(m.shape)) return false;
    int bias_in = -1;
    if (bias >= 0) {
      int64_t inner, period;
      if (!affine_operand(bias, m.shape, bias_in, inner, period)) return false;
      if (inner != 1 || period != m.shape[1]) return false;
      if (nodes_[bias_in].decl_dtype != out_dt) return false;
    }
    Step s;
    s.kind = Step::GEMM;
    s.label = std::string("gemm") + (bias >= 0 ? "+bias" : "") + (act ? "+relu" : "");
    s.d[0] = m.shape[0];
    s.d[1] = m.shape[1];
    s.d[2] = m.tb ? nodes_[b].shape[1] : nodes_[b].shape[0];
    s.in[0] = nodes_[a].view.buffer;
    s.in[1] = nodes_[b].view.buffer;
    s.in[2] = bias_in >= 0 ? nodes_[bias_in].view.buffer : -1;
    s.out[0] = out_buf;
    s.dtype = in_dt;
    s.dtype2 = out_dt;
    s.transpose_b = m.tb;
    s.act = act;
    finish_gemm(s);
    plan_->uses_status = true;
    plan_->steps.push_back(s);
    return true;
  }

  // options from the bindings, and the scratch for the K-split tail of the tensor-core kernel
  void finish_gemm(Step& s) {
    const auto tf = bind_.find("ALLOW_TF32");
    if (tf != bind_.end() && tf->second != 0) s.flags |= IB200_GEMM_ALLOW_TF32;
    if (s.batch != 1) return;
    const size_t bytes = gemm_scratch_bytes(s.dtype, s.dtype2, s.d[0], s.d[1], s.d[2], s.flags, s.transpose_b);
    if (bytes) s.scratch = new_workspace_buffer(IB200_U8, (int64_t)bytes, "gemm scratch");
    s.label += gemm_suffix(s);
  }
  static std::string gemm_suffix(const Step& s) {
    std::string out;
    const bool tf32 = s.dtype == IB200_F32 && gemm_uses_tensor_cores(s.dtype, s.dtype2, s.d[1], s.d[2], s.flags);
    if (tf32) out += "(tf32)";
    if (gemm_uses_tensor_cores(s.dtype, s.dtype2, s.d[1], s.d[2], s.flags) && prefers_cta_pairs(s.d[0], s.d[1], s.flags)) out += "(cta pairs)";
    if (s.scratch >= 0 && gemm_scratch_bytes(s.dtype, s.dtype2, s.d[0], s.d[1], s.d[2], s.flags, 1) > 0) out += "(split tail)";
    return out;
  }

  // =============================== phase C: general lowering ================================
  // number of consumers of each node (ops + graph outputs)
  void lower_general() {
    for (size_t id = 0; id < nodes_.size(); ++id) lower_node((int)id);
    // graph outputs: whatever is not yet in its argument buffer is written by elementwise kernels
    std::vector<int> pending;
    for (auto& o : outputs_) {
      const int id = by_name_[o];
      const Node& n = nodes_[id];
      if (n.repr == Node::STRIDED && n.view.buffer == out_buffer_[o] && n.view.contiguous()) continue;
      if (n.repr == Node::STRIDED && n.shape.size() == 2 && n.view.offset == 0 && n.view.strides[0] == 1 &&
          n.view.strides[1] == n.shape[0] && n.shape[0] > 1 && n.shape[1] > 1 &&
          plan_->buffers[n.view.buffer].dtype == plan_->buffers[out_buffer_[o]].dtype) {
        Step s;  // the output is the transpose of a dense matrix: tiled transpose, no gather
        s.kind = Step::TRANSPOSE;
        s.label = "transpose2d";
        s.in[0] = n.view.buffer;
        s.out[0] = out_buffer_[o];
        s.d[0] = n.shape[1];
        s.d[1] = n.shape[0];
        s.dtype = plan_->buffers[n.view.buffer].dtype;
        plan_->steps.push_back(s);
        continue;
      }
      pending.push_back(id);
    }
    // group by shape so that sibling outputs share one pass over their operands
    while (!pending.empty()) {
      std::vector<int> group = {pending[0]};
      for (size_t i = 1; i < pending.size() && group.size() < (size_t)kEwMaxOutputs; ++i)
        if (nodes_[pending[i]].shape == nodes_[pending[0]].shape) group.push_back(pending[i]);
      std::vector<int> bufs;
      for (int id : group) bufs.push_back(out_buffer_[nodes_[id].name]);
      if (!emit_elementwise(group, bufs, /*may_fail=*/group.size() > 1)) {
        group.resize(1);
        bufs.resize(1);
        emit_elementwise(group, bufs, false);
      }
      for (int id : group) pending.erase(std::find(pending.begin(), pending.end(), id));
    }
  }

  void lower_node(int id) {
    Node& n = nodes_[id];
    if (n.repr != Node::NONE) return;
    const std::string& op = n.op;
    if (op == "const") { n.repr = Node::CONSTANT; return; }
    if (op == "iota") { n.repr = Node::IOTA; return; }
    if (is_elementwise(op)) { n.repr = Node::EXPR; return; }
    if (kViews.count(op)) {
      Node& src = nodes_[n.in[0]];
      if (src.repr == Node::CONSTANT) { n.repr = Node::CONSTANT; n.cval = src.cval; return; }
      if (src.repr == Node::EXPR && (op == "identity" || op == "layout_cast")) { n.repr = Node::EXPR; n.op = "identity"; return; }
      if (src.repr != Node::STRIDED) materialise(n.in[0]);
      View v;
      if (!apply_view(n, nodes_[n.in[0]].view, v)) {  // e.g. reshape of a transposed / broadcast view
        materialise_contiguous(n.in[0]);
        if (!apply_view(n, nodes_[n.in[0]].view, v)) throw Unsupported(op + ": cannot express as a view");
      }
      n.repr = Node::STRIDED;
      n.view = v;
      return;
    }
    if (op == "reduce_sum" || op == "reduce_max" || op == "reduce_any") {
      Shape xs = nodes_[n.in[0]].shape;
      if (n.axes.empty()) {  // nothing to reduce (rank-0 input): the value itself
        n.repr = Node::EXPR; n.op = op == "reduce_any" ? "cast" : "identity"; n.cast_to = IB200_BOOL;
        return;
      }
      // The kernels reduce one run of adjacent axes ([outer, reduced, inner]).  Axes that are not adjacent (gaps of
      // extent 1 do not count) are reduced run by run, the last run first, so that the indices of the earlier runs stay
      // valid: np.sum / np.max / np.any over several axes (verify/interpreter.py:478-500) is the same nested reduction.
      {
        std::vector<std::pair<int, int>> runs;
        for (int a : n.axes) {
          bool joins = !runs.empty();
          for (int g = joins ? runs.back().second + 1 : a; joins && g < a; ++g) joins = xs[g] == 1;
          if (joins) runs.back().second = a;
          else runs.emplace_back(a, a);
        }
        Shape cur = xs;
        while (runs.size() > 1) {
          const std::pair<int, int> run = runs.back();
          runs.pop_back();
          Node m;
          m.op = op;
          m.in = {nodes_[id].in[0]};
          m.dclass = op == "reduce_any" ? DC_BOOL : DC_FLOAT;
          for (int a = run.first; a <= run.second; ++a) m.axes.push_back(a);
          for (int a = 0; a < (int)cur.size(); ++a)
            if (a < run.first || a > run.second) m.shape.push_back(cur[a]);
          const int mid = add(m);
          lower_node(mid);
          Node& self = nodes_[id];
          self.in[0] = mid;
          self.axes.erase(std::remove_if(self.axes.begin(), self.axes.end(), [&](int a) { return a >= run.first; }), self.axes.end());
          cur = nodes_[mid].shape;
        }
        xs = cur;  // what is left: one run of adjacent axes of the partly reduced tensor
      }
      materialise_contiguous(n.in[0]);
      const Node& x = nodes_[n.in[0]];
      const int xdt = plan_->buffers[x.view.buffer].dtype;
      if (op != "reduce_any" && class_of_dtype(xdt) != DC_FLOAT) throw Unsupported(op + " over a non-float tensor is not covered");
      Step s;
      s.kind = Step::REDUCE;
      s.label = op;
      s.reduce_kind = op == "reduce_sum" ? IB200_REDUCE_SUM : op == "reduce_max" ? IB200_REDUCE_MAX : IB200_REDUCE_ANY;
      s.d[0] = s.d[1] = s.d[2] = 1;
      for (int i = 0; i < (int)xs.size(); ++i) (i < n.axes.front() ? s.d[0] : i > n.axes.back() ? s.d[2] : s.d[1]) *= xs[i];
      s.scale = (float)n.scale;
      s.in[0] = x.view.buffer;
      s.dtype = xdt;
      const int tmp_dt = op == "reduce_any" ? IB200_BOOL : IB200_F32;
      s.out[0] = result_buffer(id, tmp_dt);
      s.dtype2 = plan_->buffers[s.out[0]].dtype;
      if (op == "reduce_any" ? s.dtype2 != IB200_BOOL : class_of_dtype(s.dtype2) != DC_FLOAT || s.dtype2 == IB200_F64) {
        // the declared output type needs a conversion pass: reduce into the workspace instead
        out_written_.erase(n.name);
        s.out[0] = new_workspace_buffer(tmp_dt, numel(n.shape), n.name);
        s.dtype2 = tmp_dt;
      }
      add_reduce_scratch(s);
      plan_->steps.push_back(s);
      set_strided(id, s.out[0]);
      return;
    }
    if (op == "softmax") {
      if (n.axis != (int)n.shape.size() - 1) {
        bool trailing_units = true;
        for (int a = n.axis + 1; a < (int)n.shape.size(); ++a) trailing_units &= n.shape[a] == 1;
        if (!trailing_units) {
          // softmax along an axis that is not the innermost one (verify/interpreter.py:501-506 takes any axis): the
          // rows are strided, so it is computed as the interpreter writes it — max over the axis, exp(x - max), sum
          // over the axis, division — with the reduction kernels' [outer, reduced, inner] form and two elementwise passes
          const int x = n.in[0], ax = n.axis;
          const Shape full = n.shape;
          auto reduce_over_axis = [&](const char* rop, int src) {
            Node r;
            r.op = rop;
            r.in = {src};
            r.axes = {ax};
            r.keepdims = true;
            r.shape = full;
            r.shape[ax] = 1;
            r.dclass = DC_FLOAT;
            const int rid = add(r);
            lower_node(rid);
            return rid;
          };
          const int mx = reduce_over_axis("reduce_max", x);
          Node d;
          d.op = "sub"; d.in = {x, mx}; d.shape = full; d.dclass = DC_FLOAT;
          const int di = add(d);
          lower_node(di);
          Node e;
          e.op = "exp"; e.in = {di}; e.shape = full; e.dclass = DC_FLOAT;
          const int ei = add(e);
          lower_node(ei);
          const int sm = reduce_over_axis("reduce_sum", ei);  // materialises exp(x - max) once; the division reads it back
          Node& self = nodes_[id];
          self.op = "div";
          self.in = {ei, sm};
          self.repr = Node::EXPR;
          return;
        }
      }
      materialise_contiguous(n.in[0]);
      const Node& x = nodes_[n.in[0]];
      const int xdt = plan_->buffers[x.view.buffer].dtype;
      if (!(xdt == IB200_F32 || xdt == IB200_BF16 || xdt == IB200_F16)) throw Unsupported("softmax over a non-float tensor is not covered");
      Step s;
      s.kind = Step::SOFTMAX;
      s.label = "softmax";
      s.d[1] = n.shape[n.axis];
      s.d[0] = s.d[1] ? numel(n.shape) / s.d[1] : 0;
      s.in[0] = x.view.buffer;
      s.dtype = xdt;
      s.out[0] = result_buffer(id, IB200_F32);  // intermediates are kept in f32
      s.dtype2 = plan_->buffers[s.out[0]].dtype;
      if (s.dtype2 != xdt && s.dtype2 != IB200_F32) {
        out_written_.erase(n.name);
        s.out[0] = new_workspace_buffer(IB200_F32, numel(n.shape), n.name);
        s.dtype2 = IB200_F32;
      }
      plan_->steps.push_back(s);
      set_strided(id, s.out[0]);
      return;
    }
    if (op == "matmul") {
      int a = n.in[0], b = n.in[1];
      bool tb = n.tb;
      if (n.ta) a = transposed_copy(a);
      // a B that is a swapped-last-two-axes view of a dense tensor is consumed as stored
      materialise(b);
      {
        const View& v = nodes_[b].view;
        const size_t r = v.shape.size();
        View sw = v;
        std::swap(sw.shape[r - 1], sw.shape[r - 2]);
        std::swap(sw.strides[r - 1], sw.strides[r - 2]);
        if (!v.contiguous() && sw.contiguous()) {
          Node alias; alias.op = "identity"; alias.in = {b}; alias.shape = sw.shape; alias.dclass = nodes_[b].dclass;
          const int id2 = add(alias);
          nodes_[id2].repr = Node::STRIDED;
          nodes_[id2].view = sw;
          b = id2;
          tb = !tb;
        }
      }
      materialise_contiguous(a);
      materialise_contiguous(b);
      int adt = plan_->buffers[nodes_[a].view.buffer].dtype, bdt = plan_->buffers[nodes_[b].view.buffer].dtype;
      if (adt != bdt || !(adt == IB200_F32 || adt == IB200_BF16 || adt == IB200_F16)) {
        a = converted_copy(a, IB200_F32);
        b = converted_copy(b, IB200_F32);
        adt = IB200_F32;
      }
      const Shape &as = nodes_[a].shape, &bs = nodes_[b].shape;
      Step s;
      s.kind = Step::GEMM;
      s.label = "gemm";
      s.d[0] = n.shape[n.shape.size() - 2];
      s.d[1] = n.shape.back();
      s.d[2] = as.back();
      // batch counts are the products of the leading extents (not element counts over matrix sizes: K, M or N may be 0)
      auto leading = [](const Shape& sh) { int64_t n = 1; for (size_t i = 0; i + 2 < sh.size(); ++i) n *= sh[i]; return n; };
      s.batch = leading(n.shape);
      const int64_t abatch = leading(as), bbatch = leading(bs);
      if (s.d[0] * s.d[1] == 0) s.batch = 0;
      if ((abatch != s.batch && abatch != 1) || (bbatch != s.batch && bbatch != 1))
        throw Unsupported("matmul: partially broadcast batch axes are not covered (" + shape_str(as) + " x " + shape_str(bs) + ")");
      s.batch_stride[0] = abatch == 1 ? 0 : s.d[0] * s.d[2];
      s.batch_stride[1] = bbatch == 1 ? 0 : s.d[1] * s.d[2];
      s.batch_stride[2] = s.d[0] * s.d[1];
      if (s.batch > 1) s.label = "gemm x" + std::to_string(s.batch);
      s.in[0] = nodes_[a].view.buffer;
      s.in[1] = nodes_[b].view.buffer;
      s.dtype = adt;
      s.transpose_b = tb;
      s.out[0] = result_buffer(id, IB200_F32);
      s.dtype2 = plan_->buffers[s.out[0]].dtype;
      if (!(s.dtype2 == IB200_F32 || (s.dtype2 == adt && adt != IB200_F32))) {
        out_written_.erase(n.name);
        s.out[0] = new_workspace_buffer(IB200_F32, numel(n.shape), n.name);
        s.dtype2 = IB200_F32;
      }
      finish_gemm(s);
      plan_->uses_status = true;
      plan_->steps.push_back(s);
      set_strided(id, s.out[0]);
      return;
    }
    if (op == "gather") {
      materialise_contiguous(n.in[0]);
      const Node& data = nodes_[n.in[0]];
      Step s;
      s.kind = Step::GATHER;
      s.label = "gather";
      s.in[0] = data.view.buffer;
      s.dtype = plan_->buffers[s.in[0]].dtype;
      s.g_dim = data.shape;
      s.g_stride = contiguous_strides(data.shape);
      s.other = n.cval;
      s.d[0] = numel(n.shape);
      int idx_dtype = -1;
      for (size_t k = 1; k < n.in.size(); ++k) {
        materialise_contiguous(n.in[k]);
        const int buf = nodes_[n.in[k]].view.buffer;
        const int dt = plan_->buffers[buf].dtype;
        if (dt != IB200_I32 && dt != IB200_I64) throw Unsupported("gather: index tensors must be i32 or i64");
        if (idx_dtype >= 0 && dt != idx_dtype) throw Unsupported("gather: index tensors of mixed integer types are not covered");
        idx_dtype = dt;
        s.idx_buf.push_back(buf);
      }
      s.dtype2 = idx_dtype;
      s.out[0] = result_buffer(id, s.dtype);
      if (plan_->buffers[s.out[0]].dtype != s.dtype) {
        out_written_.erase(n.name);
        s.out[0] = new_workspace_buffer(s.dtype, numel(n.shape), n.name);
      }
      plan_->steps.push_back(s);
      set_strided(id, s.out[0]);
      return;
    }
    if (op == "rope" || op == "dropout") {
      Step s;
      s.kind = op == "rope" ? Step::ROPE : Step::DROPOUT;
      s.label = op;
      const int x = converted_copy(n.in[0], IB200_F32);  // the interpreter computes both in float32
      s.in[0] = nodes_[x].view.buffer;
      const Shape& xs = nodes_[id].shape;
      if (op == "rope") {
        const int c = converted_copy(nodes_[id].in[1], IB200_F32), sn = converted_copy(nodes_[id].in[2], IB200_F32);
        s.in[1] = nodes_[c].view.buffer;
        s.in[2] = nodes_[sn].view.buffer;
        s.d[0] = xs[0];
        s.d[1] = xs[1] * xs[2];
        s.d[2] = xs[3];
      } else {
        s.d[0] = numel(xs);
        s.d[1] = nodes_[id].axis;
        const int pn = nodes_[id].in[1], sd = nodes_[id].in[2];
        if (nodes_[pn].repr == Node::NONE) lower_node(pn);
        if (nodes_[sd].repr == Node::NONE) lower_node(sd);
        if (nodes_[pn].repr == Node::CONSTANT) {
          s.other = nodes_[pn].cval;
        } else {
          materialise_contiguous(pn);
          s.in[1] = nodes_[pn].view.buffer;
          s.dtype = plan_->buffers[s.in[1]].dtype;
          if (class_of_dtype(s.dtype) != DC_FLOAT) throw Unsupported("dropout: p must be a floating-point scalar");
        }
        if (nodes_[sd].repr == Node::CONSTANT) {
          s.seed = (long long)nodes_[sd].cval;
        } else {
          materialise_contiguous(sd);
          s.in[2] = nodes_[sd].view.buffer;
          s.dtype2 = plan_->buffers[s.in[2]].dtype;
          if (s.dtype2 != IB200_I32 && s.dtype2 != IB200_I64) throw Unsupported("dropout: seed must be an i32 or i64 scalar");
        }
      }
      s.out[0] = result_buffer(id, IB200_F32);
      if (plan_->buffers[s.out[0]].dtype != IB200_F32) {
        out_written_.erase(nodes_[id].name);
        s.out[0] = new_workspace_buffer(IB200_F32, numel(xs), nodes_[id].name);
      }
      plan_->steps.push_back(s);
      set_strided(id, s.out[0]);
      return;
    }
    if (op == "correlation" || op == "resize" || op == "warp") {
      Step s;
      s.kind = op == "correlation" ? Step::CORRELATION : op == "resize" ? Step::RESIZE : Step::WARP;
      s.label = op;
      auto dense_input = [&](int node, int dtype, const char* what) {
        if (nodes_[node].repr == Node::NONE) lower_node(node);
        materialise_contiguous(node);
        const int buf = nodes_[node].view.buffer;
        if (plan_->buffers[buf].dtype != dtype) throw Unsupported(op + ": " + what + " must be declared " + dtype_name(dtype));
        return buf;
      };
      const std::vector<int> ins = nodes_[id].in;
      const Shape src = nodes_[ins[0]].shape, os = nodes_[id].shape;
      s.in[0] = dense_input(ins[0], IB200_I8, "the source");
      s.d[0] = src[0]; s.d[1] = src[1]; s.d[2] = src[2]; s.d[3] = os[0];
      if (op == "correlation") {
        s.in[1] = dense_input(ins[1], IB200_I8, "the second source");
        const int sh = ins[2];
        if (nodes_[sh].repr == Node::NONE) lower_node(sh);
        if (nodes_[sh].repr == Node::CONSTANT) {
          s.seed = (long long)nodes_[sh].cval;
          if (s.seed < 0) throw Invalid("correlation: negative out_shift");
        } else {
          materialise_contiguous(sh);
          s.in[2] = nodes_[sh].view.buffer;
          s.dtype2 = plan_->buffers[s.in[2]].dtype;
          if (s.dtype2 != IB200_I32 && s.dtype2 != IB200_I64) throw Unsupported("correlation: out_shift must be an i32 or i64 scalar");
        }
      } else if (op == "resize") {
        s.d[3] = nodes_[id].axis;  // hw_fl
      } else {
        s.in[1] = dense_input(ins[1], IB200_I16, "the offset");
      }
      s.out[0] = result_buffer(id, IB200_I8);
      if (plan_->buffers[s.out[0]].dtype != IB200_I8) {
        out_written_.erase(nodes_[id].name);
        s.out[0] = new_workspace_buffer(IB200_I8, numel(os), nodes_[id].name);
      }
      plan_->steps.push_back(s);
      set_strided(id, s.out[0]);
      return;
    }
    if (op == "input") return;
    throw Unsupported("op '" + op + "' is not covered by the B200 kernels");
  }

  // make `id` a STRIDED value (any strides)
  void materialise(int id) {
    Node& n = nodes_[id];
    if (n.repr == Node::STRIDED) return;
    // a value that is also a graph output is computed straight into its argument buffer
    const int buf = result_buffer(id, storage_of_class(n.dclass));
    emit_elementwise({id}, {buf}, false);
  }
  // make `id` a STRIDED value that is dense row-major at offset 0
  void materialise_contiguous(int id) {
    materialise(id);
    Node& n = nodes_[id];
    if (n.view.contiguous()) return;
    const int dt = plan_->buffers[n.view.buffer].dtype;
    const int buf = new_workspace_buffer(dt, numel(n.shape), n.name + ".dense");
    if (n.shape.size() == 2 && n.view.offset == 0 && n.view.strides[1] == n.shape[0] && n.view.strides[0] == 1) {
      Step s;  // a plain 2-D transpose of a dense matrix
      s.kind = Step::TRANSPOSE;
      s.label = "transpose2d";
      s.in[0] = n.view.buffer;
      s.out[0] = buf;
      s.d[0] = n.shape[1];
      s.d[1] = n.shape[0];
      s.dtype = dt;
      plan_->steps.push_back(s);
      set_strided(id, buf);
    } else {
      emit_elementwise({id}, {buf}, false);
    }
  }
  int transposed_copy(int id) {
    Node t;
    t.op = "transpose";
    t.in = {id};
    t.axes = {1, 0};
    t.shape = {nodes_[id].shape[1], nodes_[id].shape[0]};
    t.dclass = nodes_[id].dclass;
    const int tid = add(t);
    lower_node(tid);
    return tid;
  }
  int converted_copy(int id, int dtype) {
    materialise(id);
    if (plan_->buffers[nodes_[id].view.buffer].dtype == dtype && nodes_[id].view.contiguous()) return id;
    Node c;
    c.op = "identity";
    c.in = {id};
    c.shape = nodes_[id].shape;
    c.dclass = class_of_dtype(dtype);
    const int cid = add(c);
    nodes_[cid].repr = Node::EXPR;
    const int buf = new_workspace_buffer(dtype, numel(c.shape), "");
    emit_elementwise({cid}, {buf}, false);
    return cid;
  }

  // ---- micro-op code generation ----------------------------------------------------------
  struct Gen {
    EwProgram prog{};
    std::vector<int> in_buf;
    std::vector<int64_t> in_off;
    std::map<int, int> leaf_slot;   // node id -> input slot
    std::map<int, int> value_slot;  // computed node id -> slot
    std::map<int, int> uses;        // remaining in-kernel uses of computed nodes
    std::vector<int> free_slots;
    int acc_holds = -1;
    bool failed = false;
    double imm_d[kEwMaxInstr] = {};  // every instruction's immediate at full precision (the wide kernel reads these)
    double last_imm_d = 0.0;
  };

  static uint8_t ew_opcode(const Node& n) {
    static const std::map<std::string, uint8_t> m = {
        {"add", EW_ADD}, {"sub", EW_SUB}, {"mul", EW_MUL}, {"div", EW_DIV}, {"max", EW_MAX}, {"min", EW_MIN}, {"relu", EW_RELU},
        {"exp", EW_EXP}, {"rsqrt", EW_RSQRT}, {"abs", EW_ABS}, {"floor", EW_FLOOR}, {"ne", EW_NE}, {"lt", EW_LT}, {"le", EW_LE},
        {"gt", EW_GT}, {"ge", EW_GE}, {"and", EW_AND}, {"or", EW_OR}, {"not", EW_NOT}, {"where", EW_WHERE}, {"identity", EW_MOV}};
    if (n.op == "cast") {
      switch (n.cast_to) {
        case IB200_BOOL: return EW_TO_BOOL;
        case IB200_BF16: case IB200_F16: return EW_ROUND_F16;  // the oracle carries bf16 as float16
        case IB200_F32: case IB200_F64: return EW_MOV;
        default: return EW_TO_INT;
      }
    }
    return m.at(n.op);
  }

  // count in-kernel uses of EXPR nodes reachable from `id`
  void count_uses(int id, Gen& g, std::set<int>& seen) {
    if (nodes_[id].repr != Node::EXPR) return;
    g.uses[id]++;
    if (!seen.insert(id).second) return;
    for (int c : nodes_[id].in) count_uses(c, g, seen);
  }

  int alloc_slot(Gen& g) {
    if (!g.free_slots.empty()) { int s = g.free_slots.back(); g.free_slots.pop_back(); return s; }
    if (g.prog.n_slots >= kEwMaxSlots) { g.failed = true; return 0; }
    return g.prog.n_slots++;
  }

  // operand code for node `id` as seen from a kernel over `root_shape`; emits code if needed
  uint8_t operand(int id, Gen& g, const Shape& root_shape, float& imm, bool& has_imm, bool force_slot) {
    Node& n = nodes_[id];
    if (n.repr == Node::CONSTANT) {
      if (has_imm && (imm != (float)n.cval || g.last_imm_d != n.cval)) {  // one immediate per instruction: stage this one through ACC/slot
        return stage_constant(n.cval, g, force_slot);
      }
      imm = (float)n.cval;
      g.last_imm_d = n.cval;
      has_imm = true;
      return EW_IMM;
    }
    if (n.repr == Node::STRIDED || n.repr == Node::IOTA) {
      auto it = g.leaf_slot.find(id);
      if (it != g.leaf_slot.end()) return (uint8_t)it->second;
      return (uint8_t)add_leaf(id, g, root_shape);
    }
    if (n.repr != Node::EXPR) throw Unsupported("internal: operand '" + n.name + "' has no representation");
    auto vs = g.value_slot.find(id);
    if (vs != g.value_slot.end()) return (uint8_t)vs->second;
    if (g.acc_holds == id && !force_slot) return EW_ACC;
    emit_node(id, g, root_shape, force_slot);
    auto vs2 = g.value_slot.find(id);
    if (vs2 != g.value_slot.end()) return (uint8_t)vs2->second;
    return EW_ACC;
  }

  uint8_t stage_constant(double v, Gen& g, bool force_slot) {
    if (g.prog.n_instr >= kEwMaxInstr) { g.failed = true; return EW_ACC; }
    g.imm_d[g.prog.n_instr] = v;
    EwInstr& ins = g.prog.instr[g.prog.n_instr++];
    ins = EwInstr{};
    ins.op = EW_MOV; ins.a = EW_IMM; ins.b = EW_IMM; ins.c = EW_IMM; ins.imm = (float)v; ins.dst = EW_NODST;
    g.acc_holds = -1;
    if (force_slot) { ins.dst = (uint8_t)alloc_slot(g); return ins.dst; }
    return EW_ACC;
  }

  int add_leaf(int id, Gen& g, const Shape& root_shape) {
    const Node& n = nodes_[id];
    if (g.prog.n_inputs >= kEwMaxInputs) { g.failed = true; return 0; }
    // inputs occupy the first slots: they must all be registered before temporaries, which
    // emit_elementwise guarantees by collecting leaves first
    EwInput& in = g.prog.in[g.prog.n_inputs];
    in = EwInput{};
    View v;
    if (n.repr == Node::IOTA) {
      in.kind = EW_IN_IOTA;
      v.shape = n.shape;
      v.strides.assign(n.shape.size(), 0);
      v.strides[n.axis] = 1;
      in.dtype = IB200_I32;
      g.in_buf.push_back(-1);
      g.in_off.push_back(0);
    } else {
      in.kind = EW_IN_TENSOR;
      v = n.view;
      in.dtype = plan_->buffers[v.buffer].dtype;
      g.in_buf.push_back(v.buffer);
      g.in_off.push_back(v.offset);
    }
    Shape st;
    if (!broadcast_strides(v, root_shape, st)) throw Invalid("cannot broadcast " + shape_str(v.shape) + " onto " + shape_str(root_shape));
    // the same memory seen through the same strides is one operand, however many view nodes name it
    for (int k = 0; k < g.prog.n_inputs; ++k)
      if (g.prog.in[k].kind == in.kind && g.in_buf[k] == g.in_buf.back() && g.in_off[k] == g.in_off.back() && leaf_strides_[k] == st &&
          (in.kind == EW_IN_TENSOR || true)) {
        g.in_buf.pop_back();
        g.in_off.pop_back();
        g.leaf_slot[id] = k;
        return k;
      }
    leaf_strides_.push_back(st);
    const int slot = g.prog.n_inputs++;
    g.leaf_slot[id] = slot;
    return slot;
  }
  std::vector<Shape> leaf_strides_;

  void emit_node(int id, Gen& g, const Shape& root_shape, bool force_slot) {
    Node& n = nodes_[id];
    // decide evaluation order: operands that still need instructions go first; all but the
    // last of them must be parked in slots because the next computation clobbers ACC
    std::vector<int> pending;
    for (int c : n.in)
      if (nodes_[c].repr == Node::EXPR && !g.value_slot.count(c) && g.acc_holds != c) pending.push_back(c);
    std::sort(pending.begin(), pending.end());
    pending.erase(std::unique(pending.begin(), pending.end()), pending.end());
    for (size_t i = 0; i < pending.size(); ++i) {
      const bool park = i + 1 < pending.size();
      emit_node(pending[i], g, root_shape, park);
      if (g.failed) return;
    }
    if (g.prog.n_instr >= kEwMaxInstr) { g.failed = true; return; }
    EwInstr ins{};
    ins.op = ew_opcode(n);
    ins.dst = EW_NODST;
    float imm = 0.0f;
    bool has_imm = false;
    uint8_t codes[3] = {EW_ACC, EW_ACC, EW_ACC};
    // a constant that cannot ride as the immediate is staged through a slot *before* the
    // other operands are resolved, so that ACC still holds what they expect
    int n_const = 0;
    for (size_t k = 0; k < n.in.size() && k < 3; ++k) n_const += nodes_[n.in[k]].repr == Node::CONSTANT;
    std::map<size_t, uint8_t> staged;
    if (n_const > 1) {
      bool first = true;
      for (size_t k = 0; k < n.in.size() && k < 3; ++k) {
        if (nodes_[n.in[k]].repr != Node::CONSTANT) continue;
        if (first) { first = false; continue; }
        if ((float)nodes_[n.in[k]].cval == (float)nodes_[n.in[0]].cval && nodes_[n.in[0]].repr == Node::CONSTANT) continue;
        // park whatever ACC holds if one of our operands lives there
        for (int c : n.in)
          if (g.acc_holds == c && !g.value_slot.count(c)) park_acc(c, g);
        staged[k] = stage_constant(nodes_[n.in[k]].cval, g, true);
        if (g.failed) return;
      }
    }
    for (size_t k = 0; k < n.in.size() && k < 3; ++k) {
      if (staged.count(k)) { codes[k] = staged[k]; continue; }
      codes[k] = operand(n.in[k], g, root_shape, imm, has_imm, false);
      if (g.failed) return;
    }
    ins.a = codes[0];
    ins.b = n.in.size() > 1 ? codes[1] : codes[0];
    ins.c = n.in.size() > 2 ? codes[2] : codes[0];
    ins.imm = imm;
    // release operand slots whose last use this was
    for (int c : n.in) {
      if (nodes_[c].repr != Node::EXPR) continue;
      if (--g.uses[c] == 0) {
        auto it = g.value_slot.find(c);
        if (it != g.value_slot.end()) { g.free_slots.push_back(it->second); g.value_slot.erase(it); }
      }
    }
    for (auto& kv : staged) g.free_slots.push_back(kv.second);
    if (force_slot || g.uses[id] > 1) {
      ins.dst = (uint8_t)alloc_slot(g);
      g.value_slot[id] = ins.dst;
    }
    if (g.prog.n_instr >= kEwMaxInstr) { g.failed = true; return; }
    g.imm_d[g.prog.n_instr] = has_imm ? g.last_imm_d : 0.0;
    g.prog.instr[g.prog.n_instr++] = ins;
    g.acc_holds = id;
  }

  void park_acc(int id, Gen& g) {
    if (g.prog.n_instr >= kEwMaxInstr) { g.failed = true; return; }
    EwInstr& ins = g.prog.instr[g.prog.n_instr++];
    ins = EwInstr{};
    ins.op = EW_MOV; ins.a = ins.b = ins.c = EW_ACC; ins.dst = (uint8_t)alloc_slot(g);
    g.value_slot[id] = ins.dst;
  }

  void collect_leaves(int id, Gen& g, const Shape& root_shape, std::set<int>& seen) {
    if (!seen.insert(id).second) return;
    Node& n = nodes_[id];
    if (n.repr == Node::NONE) lower_node(id);
    if (n.repr == Node::STRIDED || n.repr == Node::IOTA) {
      if (!g.leaf_slot.count(id)) add_leaf(id, g, root_shape);
      return;
    }
    if (n.repr == Node::EXPR)
      for (int c : n.in) collect_leaves(c, g, root_shape, seen);
  }

  // One kernel computing `roots` (same shape) into `bufs`.  Returns false (emitting nothing)
  // when may_fail and the program does not fit; otherwise splits by materialising operands.
  bool emit_elementwise(const std::vector<int>& roots, const std::vector<int>& bufs, bool may_fail) {
    const Shape root_shape = nodes_[roots[0]].shape;
    Gen g;
    leaf_strides_.clear();
    std::set<int> seen;
    for (int r : roots) collect_leaves(r, g, root_shape, seen);
    g.prog.n_slots = g.prog.n_inputs;
    std::set<int> seen2;
    for (int r : roots) { count_uses(r, g, seen2); }
    // every root but the last must be kept in a slot until the stores
    for (size_t i = 0; i < roots.size() && !g.failed; ++i) {
      Node& n = nodes_[roots[i]];
      EwOutput& o = g.prog.out[g.prog.n_outputs++];
      o = EwOutput{};
      o.dtype = plan_->buffers[bufs[i]].dtype;
      const bool last = i + 1 == roots.size();
      if (n.repr == Node::EXPR) {
        float imm; bool has_imm = false;
        o.src = operand(roots[i], g, root_shape, imm, has_imm, !last);
        if (o.src == EW_ACC && !last) g.failed = true;
      } else if (n.repr == Node::CONSTANT) {
        o.src = stage_constant(n.cval, g, !last);
      } else {
        o.src = (uint8_t)g.leaf_slot.at(roots[i]);
      }
    }
    if (g.failed) {
      if (may_fail) return false;
      if (roots.size() != 1) throw Unsupported("internal: multi-output kernel must be allowed to fail");
      // too big for one kernel: materialise the root's EXPR operands first, then retry
      bool progressed = false;
      for (int c : nodes_[roots[0]].in)
        if (nodes_[c].repr == Node::EXPR) { materialise(c); progressed = true; }
      if (!progressed) throw Unsupported("elementwise chain does not fit the micro-op program limits");
      return emit_elementwise(roots, bufs, false);
    }
    // collapse the output dims: drop unit dims, then merge adjacent dims wherever every
    // operand's strides allow it (the outputs are dense, so they always do)
    Shape dims = root_shape;
    std::vector<Shape> strides = leaf_strides_;
    for (int d = (int)dims.size() - 1; d >= 0; --d)
      if (dims[d] == 1) { dims.erase(dims.begin() + d); for (auto& st : strides) st.erase(st.begin() + d); }
    if (dims.empty()) { dims = {1}; for (auto& st : strides) st = {0}; }
    for (int d = (int)dims.size() - 2; d >= 0; --d) {
      bool ok = true;
      for (auto& st : strides) ok &= st[d] == st[d + 1] * dims[d + 1];
      if (!ok) continue;
      dims[d] *= dims[d + 1];
      dims.erase(dims.begin() + d + 1);
      for (auto& st : strides) { st[d] = st[d + 1]; st.erase(st.begin() + d + 1); }
    }
    if ((int)dims.size() > kEwMaxRank) throw Unsupported("elementwise kernel over more than 5 non-mergeable dims");
    EwProgram& p = g.prog;
    p.rank = (int)dims.size();
    p.total = numel(dims);
    for (int d = 0; d < p.rank; ++d) p.dim[d] = (uint32_t)dims[d];
    for (int k = 0; k < p.n_inputs; ++k)
      for (int d = 0; d < p.rank; ++d) p.in[k].stride[d] = strides[k][d];
    Step s;
    s.kind = Step::ELEMENTWISE;
    s.label = "elementwise(" + std::to_string(p.n_instr) + " ops, " + std::to_string(p.n_inputs) + " in, " + std::to_string(p.n_outputs) + " out)";
    s.ew = p;
    s.ew_in_buf = g.in_buf;
    s.ew_in_off = g.in_off;
    s.ew_out_buf = bufs;
    // f64 values and 32- / 64-bit integers do not fit the kernels' f32 registers (24 bits of mantissa): such programs run on
    // the double-valued kernel — exact for f64 and for integers up to 2^53
    auto needs_wide = [](int dt) { return dt == IB200_F64 || dt == IB200_I32 || dt == IB200_I64; };
    for (int k = 0; k < p.n_inputs; ++k) s.wide |= p.in[k].kind == EW_IN_TENSOR ? needs_wide(p.in[k].dtype) : p.total >= ((int64_t)1 << 24);
    for (int o = 0; o < p.n_outputs; ++o) s.wide |= needs_wide(p.out[o].dtype);
    if (s.wide) {
      s.ew_imm.assign(g.imm_d, g.imm_d + kEwMaxInstr);
      s.label += "(f64 lanes)";
    }
    plan_->steps.push_back(s);
    for (size_t i = 0; i < roots.size(); ++i) {
      set_strided(roots[i], bufs[i]);
      if (out_buffer_.count(nodes_[roots[i]].name) && out_buffer_[nodes_[roots[i]].name] == bufs[i]) out_written_.insert(nodes_[roots[i]].name);
    }
    return true;
  }

  // =============================== GEMM epilogues ===========================================
  // A GEMM whose only consumer is an elementwise step computing [relu](gemm [+ bias[col]])
  // takes that step into its epilogue: multi-matmul graphs (mlp, attention output) then run one
  // kernel per matmul, as the single-matmul pattern of phase B already does.
  void fuse_gemm_epilogues() {
    std::vector<Step>& steps = plan_->steps;
    std::vector<int> reads, writes;
    for (size_t i = 0; i + 1 < steps.size(); ++i) {
      Step& g = steps[i];
      const Step& e = steps[i + 1];
      if (g.kind != Step::GEMM || g.batch != 1 || g.in[2] >= 0 || g.act != IB200_ACT_NONE || e.kind != Step::ELEMENTWISE || e.wide) continue;
      const int gb = g.out[0];
      if (plan_->buffers[gb].is_arg) continue;
      bool used_elsewhere = false;
      for (size_t k = i + 2; k < steps.size() && !used_elsewhere; ++k) {
        step_io(steps[k], reads, writes);
        used_elsewhere = std::find(reads.begin(), reads.end(), gb) != reads.end();
      }
      if (used_elsewhere) continue;
      const EwProgram& q = e.ew;
      const int64_t M = g.d[0], N = g.d[1];
      if (q.n_outputs != 1 || q.total != M * N || q.n_inputs < 1 || q.n_inputs > 2 || M < 2 || N < 2) continue;
      // operand roles: the GEMM result (dense) and, optionally, a vector along N
      int slot_g = -1, slot_b = -1;
      bool ok = true;
      for (int k = 0; k < q.n_inputs && ok; ++k) {
        const EwInput& in = q.in[k];
        if (in.kind != EW_IN_TENSOR || e.ew_in_off[k] != 0) { ok = false; break; }
        const bool dense = q.rank == 1 ? in.stride[0] == 1 : (q.rank == 2 && (int64_t)q.dim[0] == M && (int64_t)q.dim[1] == N && in.stride[0] == N && in.stride[1] == 1);
        const bool colvec = q.rank == 2 && (int64_t)q.dim[0] == M && (int64_t)q.dim[1] == N && in.stride[0] == 0 && in.stride[1] == 1;
        if (e.ew_in_buf[k] == gb && dense && slot_g < 0) slot_g = k;
        else if (colvec && slot_b < 0) slot_b = k;
        else ok = false;
      }
      if (!ok || slot_g < 0 || (q.n_inputs == 2 && slot_b < 0)) continue;
      // program: [add(g, b)] [relu]
      int ip = 0, act = IB200_ACT_NONE;
      if (slot_b >= 0) {
        if (q.n_instr < 1 || q.instr[0].op != EW_ADD) continue;
        const uint8_t a = q.instr[0].a, b = q.instr[0].b;
        if (!((a == slot_g && b == slot_b) || (a == slot_b && b == slot_g))) continue;
        ip = 1;
      }
      if (ip < q.n_instr && q.instr[ip].op == EW_RELU && (ip == 0 ? q.instr[ip].a == slot_g : q.instr[ip].a == EW_ACC)) { act = IB200_ACT_RELU; ++ip; }
      if (ip != q.n_instr || ip == 0) continue;
      if (q.out[0].src != EW_ACC) continue;
      const int ob = e.ew_out_buf[0];
      const int out_dt = plan_->buffers[ob].dtype;
      if (!(out_dt == IB200_F32 || (out_dt == g.dtype && g.dtype != IB200_F32))) continue;
      if (slot_b >= 0 && plan_->buffers[e.ew_in_buf[slot_b]].dtype != out_dt) continue;
      g.in[2] = slot_b >= 0 ? e.ew_in_buf[slot_b] : -1;
      g.act = act;
      g.out[0] = ob;
      g.dtype2 = out_dt;
      g.label = std::string("gemm") + (slot_b >= 0 ? "+bias" : "") + (act ? "+relu" : "") + gemm_suffix(g);
      steps.erase(steps.begin() + i + 1);
    }
  }

  // =============================== masked softmax ===========================================
  // softmax(where(mask, x, constant)) over f32 rows of up to 16384 elements: the softmax kernel applies the
  // mask while it loads each row, so the masked scores never exist in HBM (pipeline/tilelang/core.py:1050-1076).
  void fuse_softmax_masks() {
    std::vector<Step>& steps = plan_->steps;
    std::vector<int> reads, writes;
    for (size_t i = 0; i + 1 < steps.size(); ++i) {
      const Step& e = steps[i];
      Step& sm = steps[i + 1];
      if (e.kind != Step::ELEMENTWISE || e.wide || sm.kind != Step::SOFTMAX || sm.reduce_kind != 0) continue;
      const EwProgram& q = e.ew;
      const int64_t R = sm.d[0], C = sm.d[1];
      if (q.n_outputs != 1 || q.n_inputs != 2 || q.n_instr != 1 || q.instr[0].op != EW_WHERE || q.out[0].src != EW_ACC) continue;
      if (e.ew_out_buf[0] != sm.in[0] || plan_->buffers[sm.in[0]].is_arg || sm.dtype != IB200_F32 || sm.dtype2 != IB200_F32) continue;
      if (q.total != R * C || C > 16384 || C < 1 || sm.out[1] >= 0 || sm.out[2] >= 0) continue;
      bool used_elsewhere = false;
      for (size_t k = i + 2; k < steps.size() && !used_elsewhere; ++k) {
        step_io(steps[k], reads, writes);
        used_elsewhere = std::find(reads.begin(), reads.end(), sm.in[0]) != reads.end();
      }
      if (used_elsewhere) continue;
      const EwInstr& w = q.instr[0];
      if (w.a >= q.n_inputs || w.b >= q.n_inputs || w.a == w.b || w.c != EW_IMM) continue;
      const EwInput &mask = q.in[w.a], &x = q.in[w.b];
      if (mask.kind != EW_IN_TENSOR || x.kind != EW_IN_TENSOR || e.ew_in_off[w.a] != 0 || e.ew_in_off[w.b] != 0) continue;
      if (!(mask.dtype == IB200_BOOL || mask.dtype == IB200_U8) || x.dtype != IB200_F32) continue;
      // strides over [R, C] (rank 2) or over the flat extent (rank 1: everything dense)
      int64_t mask_row_stride;
      if (q.rank <= 1) {  // dense operands, rows of one element, or a single row
        if (q.total == 1) mask_row_stride = 0;
        else if (x.stride[0] != 1) continue;
        else if (mask.stride[0] == 1) mask_row_stride = C;
        else if (mask.stride[0] == 0 && C == 1) mask_row_stride = 0;
        else continue;
      } else if (q.rank == 2 && (int64_t)q.dim[0] == R && (int64_t)q.dim[1] == C) {
        if (x.stride[0] != C || x.stride[1] != 1 || mask.stride[1] != 1 || !(mask.stride[0] == 0 || mask.stride[0] == C)) continue;
        mask_row_stride = mask.stride[0];
      } else {
        continue;
      }
      sm.in[0] = e.ew_in_buf[w.b];
      sm.in[1] = e.ew_in_buf[w.a];
      sm.reduce_kind = 1;  // SOFTMAX: a mask is applied on load
      sm.aff_inner = mask_row_stride;
      sm.other = w.imm;
      sm.label = "softmax+mask";
      steps.erase(steps.begin() + i);
    }
  }

  // =============================== row fusion ===============================================
  // Runs of steps that all work row by row on one [R, C] problem (elementwise chains over
  // [R, C] or over the R per-row results, reductions along the row, softmax) become one
  // ROWFUSE step: see row_program.h.  The pass works on the finished step list, so it reuses
  // every micro-op program the general lowering produced.
  static void step_io(const Step& s, std::vector<int>& reads, std::vector<int>& writes) {
    reads.clear();
    writes.clear();
    if (s.kind == Step::ELEMENTWISE) {
      for (int b : s.ew_in_buf) if (b >= 0) reads.push_back(b);
      writes = s.ew_out_buf;
      return;
    }
    if (s.kind == Step::ROWFUSE) {
      for (int b : s.row_in_buf) if (b >= 0) reads.push_back(b);
      for (int b : s.row_load_buf) if (b >= 0) reads.push_back(b);
      for (int b : s.row_out_buf) if (b >= 0) writes.push_back(b);
      return;
    }
    for (int k = 0; k < 3; ++k) {
      if (s.in[k] >= 0) reads.push_back(s.in[k]);
      if (s.out[k] >= 0) writes.push_back(s.out[k]);
    }
    for (int b : s.idx_buf) reads.push_back(b);
  }

  static bool row_anchor(const Step& s, int64_t& R, int64_t& C) {
    if (s.kind == Step::REDUCE && s.d[2] == 1) { R = s.d[0]; C = s.d[1]; }
    else if (s.kind == Step::SOFTMAX && s.out[1] < 0 && s.out[2] < 0) { R = s.d[0]; C = s.d[1]; }
    else return false;
    return R >= 1 && C >= 2 && C < (1 << 24) && R * C < ((int64_t)1 << 31);
  }
  static bool row_candidate(const Step& s, int64_t R, int64_t C) {
    int64_t r, c;
    if (row_anchor(s, r, c)) return r == R && c == C;
    if (s.kind != Step::ELEMENTWISE || s.wide) return false;  // row programs carry f32 values
    return s.ew.total == R * C || s.ew.total == R;
  }

  struct RowBuild {
    const std::vector<Step>& steps;
    size_t b, e;
    int64_t R, C;
    Step out;
    std::map<int, int> full_slot, scalar_of, last_read;
    std::set<int> written, needed_after;
    std::map<std::tuple<int, int64_t, int64_t, int64_t>, int> leaf_cache;
    std::map<std::tuple<int, int64_t, int64_t>, int> load_cache;
    bool busy[kRowMaxSlots] = {}, pinned[kRowMaxSlots] = {};
    int slot_last[kRowMaxSlots] = {};
    std::set<size_t> sunk;
    int saved = 0;  // HBM round trips the fusion removes
    RowBuild(const std::vector<Step>& st, size_t b_, size_t e_, int64_t r, int64_t c) : steps(st), b(b_), e(e_), R(r), C(c) {}

    RowProgram& p() { return out.row; }
    // a pinned slot (a row-invariant operand staged before the first row only) must be one no
    // other value has used or will use: it keeps its contents from row to row
    bool ever[kRowMaxSlots] = {};
    int n_slots = 0;
    int alloc(int last, bool pin = false) {
      for (int s = 0; s < kRowMaxSlots; ++s)
        if (!busy[s] && !(pin && ever[s])) {
          busy[s] = true; pinned[s] = pin; slot_last[s] = last; ever[s] = true;
          if (s + 1 > n_slots) n_slots = s + 1;
          return s;
        }
      return -1;
    }
    int new_scalar() { return p().n_scalars < kRowMaxScalars ? p().n_scalars++ : -1; }
    void release(int step) {
      for (int s = 0; s < kRowMaxSlots; ++s)
        if (busy[s] && !pinned[s] && slot_last[s] <= step) busy[s] = false;
    }
    RowPhase* begin_phase(uint8_t domain) {
      if (p().n_phases >= kRowMaxPhases) return nullptr;
      RowPhase& ph = p().phase[p().n_phases++];
      ph = RowPhase{};
      ph.domain = domain;
      ph.first_input = (uint16_t)p().n_inputs; ph.first_load = (uint16_t)p().n_loads;
      ph.first_output = (uint16_t)p().n_outputs; ph.first_instr = (uint16_t)p().n_instr;
      return &ph;
    }
    EwInstr* add_instr(RowPhase& ph) {
      if (p().n_instr >= kRowMaxInstr) return nullptr;
      ph.n_instr++;
      EwInstr& i = p().instr[p().n_instr++];
      i = EwInstr{};
      i.a = i.b = i.c = EW_ACC; i.dst = EW_NODST;
      return &i;
    }
    RowOutput* add_output(RowPhase& ph, int buf) {
      if (p().n_outputs >= kRowMaxOutputs || (ph.domain == ROW_FULL && ph.n_outputs >= kRowMaxSinks)) return nullptr;
      ph.n_outputs++;
      RowOutput& o = p().out[p().n_outputs++];
      o = RowOutput{};
      o.scalar = kRowNone; o.scale = 1.0f; o.src = EW_ACC;
      out.row_out_buf.push_back(buf);
      return &o;
    }
    // S[k] = buffer[off + row * stride], loaded once per row
    int scalar_load(RowPhase& ph, int buf, int64_t off, int64_t stride, int dtype) {
      auto key = std::make_tuple(buf, off, stride);
      auto it = load_cache.find(key);
      if (it != load_cache.end()) { ++saved; return it->second; }
      const int k = new_scalar();
      if (k < 0 || p().n_loads >= kRowMaxLoads) return -1;
      RowScalarLoad& ld = p().load[p().n_loads++];
      ld = RowScalarLoad{};
      ld.row_stride = stride; ld.dtype = dtype; ld.scalar = k;
      ph.n_loads++;
      out.row_load_buf.push_back(buf);
      out.row_load_off.push_back(off);
      load_cache[key] = k;
      return k;
    }
    // a slot holding buffer[off + row*rs + col*cs] for the current row
    int leaf(RowPhase& ph, int buf, int64_t off, int64_t rs, int64_t cs, int dtype, int kind) {
      auto key = std::make_tuple(buf, off, rs, cs);
      if (kind == EW_IN_TENSOR) {
        auto it = leaf_cache.find(key);
        if (it != leaf_cache.end()) { ++saved; return it->second; }
      }
      if (p().n_inputs >= kRowMaxInputs || cs > INT32_MAX || cs < INT32_MIN) return -1;
      const bool once = kind == EW_IN_TENSOR && rs == 0 && R > 1;
      const int slot = alloc(kind == EW_IN_TENSOR ? last_read[buf] : cur, once);
      if (slot < 0) return -1;
      RowInput& in = p().in[p().n_inputs++];
      in = RowInput{};
      in.row_stride = rs; in.col_stride = (int32_t)cs; in.dtype = dtype; in.kind = (uint8_t)kind; in.slot = (uint8_t)slot; in.once = once;
      ph.n_inputs++;
      out.row_in_buf.push_back(kind == EW_IN_TENSOR ? buf : -1);
      out.row_in_off.push_back(off);
      if (kind == EW_IN_TENSOR) leaf_cache[key] = slot;
      return slot;
    }
    int cur = 0;  // index of the step being translated

    bool read_later_in_run(int buf, size_t after, bool skip_sunk) const {
      std::vector<int> r, w;
      for (size_t k = after + 1; k < e; ++k) {
        if (skip_sunk && sunk.count(k)) continue;
        step_io(steps[k], r, w);
        if (std::find(r.begin(), r.end(), buf) != r.end()) return true;
      }
      return false;
    }
  };

  // FULL-phase instructions in accumulate form: every instruction but `where` is
  // acc = op(acc, b) (or acc = b for EW_LOADB), so the kernel never materialises a first
  // operand.  op(a, acc) becomes the reversed opcode; op(a, b) becomes a load and an op.
  static bool emit_accumulate_form(RowBuild& rb, RowPhase& ph, EwInstr ins) {
    auto push = [&](uint8_t op, uint8_t bcode, float imm, uint8_t dst) -> bool {
      EwInstr* o = rb.add_instr(ph);
      if (!o) return false;
      o->op = op; o->a = EW_ACC; o->b = bcode; o->c = EW_ACC; o->imm = imm; o->dst = dst;
      return true;
    };
    if (ins.op == EW_WHERE) {
      EwInstr* o = rb.add_instr(ph);
      if (!o) return false;
      *o = ins;
      return true;
    }
    const bool unary = ins.op == EW_MOV || ins.op == EW_RELU || ins.op == EW_EXP || ins.op == EW_RSQRT || ins.op == EW_ABS ||
                       ins.op == EW_FLOOR || ins.op == EW_NOT || ins.op == EW_TO_BOOL || ins.op == EW_TO_INT ||
                       ins.op == EW_ROUND_BF16 || ins.op == EW_ROUND_F16;
    if (unary) {
      if (ins.a != EW_ACC && !push(EW_LOADB, ins.a, ins.imm, EW_NODST)) return false;
      if (ins.op == EW_MOV && ins.a != EW_ACC) {  // the load is the whole instruction
        rb.p().instr[rb.p().n_instr - 1].dst = ins.dst;
        return true;
      }
      return push(ins.op, EW_ACC, 0.0f, ins.dst);
    }
    if (ins.a == EW_ACC) return push(ins.op, ins.b, ins.imm, ins.dst);
    if (ins.b == EW_ACC) {
      uint8_t r;
      switch (ins.op) {
        case EW_SUB: r = EW_RSUB; break;
        case EW_DIV: r = EW_RDIV; break;
        case EW_RSUB: r = EW_SUB; break;
        case EW_RDIV: r = EW_DIV; break;
        case EW_LT: r = EW_GT; break;
        case EW_GT: r = EW_LT; break;
        case EW_LE: r = EW_GE; break;
        case EW_GE: r = EW_LE; break;
        case EW_ADD: case EW_MUL: case EW_MAX: case EW_MIN: case EW_NE: case EW_AND: case EW_OR: r = ins.op; break;
        default: return false;
      }
      return push(r, ins.a, ins.imm, ins.dst);
    }
    return push(EW_LOADB, ins.a, ins.imm, EW_NODST) && push(ins.op, ins.b, ins.imm, ins.dst);
  }

  bool build_row_program(size_t b, size_t e, int64_t R, int64_t C, Step& fused) {
    const std::vector<Step>& steps = plan_->steps;
    RowBuild rb(steps, b, e, R, C);
    RowProgram& p = rb.p();
    p = RowProgram{};
    p.rows = R;
    p.cols = (int32_t)C;
    std::vector<int> reads, writes;
    for (size_t k = b; k < e; ++k) {
      step_io(steps[k], reads, writes);
      for (int r : reads) rb.last_read[r] = (int)k;
    }
    for (size_t k = e; k < steps.size(); ++k) {
      step_io(steps[k], reads, writes);
      for (int r : reads) rb.needed_after.insert(r);
    }
    auto goes_to_hbm = [&](int buf) { return plan_->buffers[buf].is_arg || rb.needed_after.count(buf) > 0; };
    auto dtype_of = [&](int buf) { return plan_->buffers[buf].dtype; };
    bool has_reduce = false;

    for (size_t k = b; k < e; ++k) {
      if (rb.sunk.count(k)) continue;
      const Step& st = steps[k];
      rb.cur = (int)k;
      if (st.kind == Step::ELEMENTWISE && st.ew.total == R * C) {
        // ---------------- an elementwise chain over the full [R, C] problem ----------------
        const EwProgram& q = st.ew;
        const bool split = q.rank == 1;
        if (!split && !(q.rank == 2 && (int64_t)q.dim[0] == R && (int64_t)q.dim[1] == C)) return false;
        RowPhase* ph = rb.begin_phase(ROW_FULL);
        if (!ph) return false;
        std::vector<uint8_t> code(q.n_slots, 0);
        for (int i = 0; i < q.n_inputs; ++i) {
          const EwInput& in = q.in[i];
          const int64_t rs = split ? in.stride[0] * C : in.stride[0], cs = split ? in.stride[0] : in.stride[1];
          if (in.kind == EW_IN_IOTA) {
            const int slot = rb.leaf(*ph, -1, 0, rs, cs, IB200_I32, EW_IN_IOTA);
            if (slot < 0) return false;
            code[i] = (uint8_t)slot;
            continue;
          }
          const int buf = st.ew_in_buf[i];
          const int64_t off = st.ew_in_off[i];
          if (rb.scalar_of.count(buf)) {
            if (off != 0 || cs != 0 || !(rs == 1 || R == 1)) return false;
            code[i] = (uint8_t)(EW_ROWSCALAR + rb.scalar_of[buf]);
          } else if (rb.full_slot.count(buf)) {
            if (off != 0 || cs != 1 || !(rs == C || R == 1)) return false;
            code[i] = (uint8_t)rb.full_slot[buf];
          } else if (rb.written.count(buf)) {
            return false;
          } else if (cs == 0) {
            const int sc = rb.scalar_load(*ph, buf, off, rs, in.dtype);
            if (sc < 0) return false;
            code[i] = (uint8_t)(EW_ROWSCALAR + sc);
          } else {
            if (rs < 0 || cs < 0) return false;
            const int slot = rb.leaf(*ph, buf, off, rs, cs, in.dtype, EW_IN_TENSOR);
            if (slot < 0) return false;
            code[i] = (uint8_t)slot;
          }
        }
        for (int i = q.n_inputs; i < q.n_slots; ++i) {
          const int slot = rb.alloc((int)k);
          if (slot < 0) return false;
          code[i] = (uint8_t)slot;
        }
        auto remap = [&](uint8_t c) -> uint8_t { return c < kEwMaxSlots ? code[c] : c; };
        for (int i = 0; i < q.n_instr; ++i) {
          EwInstr ins = q.instr[i];
          ins.a = remap(ins.a); ins.b = remap(ins.b); ins.c = remap(ins.c);
          if (ins.dst != EW_NODST) {
            ins.dst = remap(ins.dst);
            if (ins.dst >= kRowMaxSlots) return false;
          }
          if (!emit_accumulate_form(rb, *ph, ins)) return false;
        }
        for (int o = 0; o < q.n_outputs; ++o) {
          const int ob = st.ew_out_buf[o];
          uint8_t src = remap(q.out[o].src);
          // reductions of this value along the row fold into the phase that computes it
          for (size_t k2 = k + 1; k2 < e; ++k2) {
            const Step& r2 = steps[k2];
            if (r2.kind != Step::REDUCE || r2.in[0] != ob || rb.sunk.count(k2) || ph->n_outputs >= kRowMaxSinks - 1) continue;
            if (src == EW_ACC && o + 1 != q.n_outputs) continue;
            RowOutput* ro = rb.add_output(*ph, goes_to_hbm(r2.out[0]) ? r2.out[0] : -1);
            const int sc = rb.new_scalar();
            if (!ro || sc < 0) return false;
            ro->src = src; ro->reduce = (uint8_t)(r2.reduce_kind + 1); ro->scalar = (uint8_t)sc; ro->scale = r2.scale;
            ro->dtype = r2.dtype2; ro->row_stride = 1;
            rb.scalar_of[r2.out[0]] = sc;
            rb.written.insert(r2.out[0]);
            rb.sunk.insert(k2);
            has_reduce = true;
            ++rb.saved;
          }
          const bool resident = rb.read_later_in_run(ob, k, true);
          if (resident) {
            ++rb.saved;
            if (src < kRowMaxSlots) {
              rb.full_slot[ob] = src;
              rb.slot_last[src] = std::max(rb.slot_last[src], rb.last_read[ob]);
            } else if (src == EW_ACC) {
              if (q.n_instr == 0) return false;
              EwInstr& last = p.instr[p.n_instr - 1];
              if (last.dst == EW_NODST) {
                const int slot = rb.alloc(rb.last_read[ob]);
                if (slot < 0) return false;
                last.dst = (uint8_t)slot;
              } else {
                rb.slot_last[last.dst] = std::max(rb.slot_last[last.dst], rb.last_read[ob]);
              }
              rb.full_slot[ob] = last.dst;
            } else {
              return false;
            }
          }
          if (goes_to_hbm(ob)) {
            RowOutput* ro = rb.add_output(*ph, ob);
            if (!ro) return false;
            ro->src = src; ro->dtype = q.out[o].dtype; ro->row_stride = C;
          }
          rb.written.insert(ob);
        }
      } else if (st.kind == Step::ELEMENTWISE && st.ew.total == R) {
        // ---------------- a chain over the per-row results ----------------------------------------
        const EwProgram& q = st.ew;
        if (q.rank != 1) return false;
        RowPhase* ph = rb.begin_phase(ROW_SCALAR);
        if (!ph) return false;
        std::vector<uint8_t> code(q.n_slots, 0);
        for (int i = 0; i < q.n_inputs; ++i) {
          const EwInput& in = q.in[i];
          if (in.kind != EW_IN_TENSOR) return false;
          const int buf = st.ew_in_buf[i];
          const int64_t off = st.ew_in_off[i], rs = in.stride[0];
          int sc;
          if (rb.scalar_of.count(buf)) {
            if (off != 0 || !(rs == 1 || R == 1)) return false;
            sc = rb.scalar_of[buf];
          } else if (rb.written.count(buf)) {
            return false;
          } else {
            sc = rb.scalar_load(*ph, buf, off, rs, in.dtype);
            if (sc < 0) return false;
          }
          code[i] = (uint8_t)(EW_ROWSCALAR + sc);
        }
        for (int i = q.n_inputs; i < q.n_slots; ++i) {
          const int sc = rb.new_scalar();
          if (sc < 0) return false;
          code[i] = (uint8_t)(EW_ROWSCALAR + sc);
        }
        auto remap = [&](uint8_t c) -> uint8_t { return c < kEwMaxSlots ? code[c] : c; };
        for (int i = 0; i < q.n_instr; ++i) {
          EwInstr* ins = rb.add_instr(*ph);
          if (!ins) return false;
          *ins = q.instr[i];
          ins->a = remap(ins->a); ins->b = remap(ins->b); ins->c = remap(ins->c);
          if (ins->dst != EW_NODST) ins->dst = remap(ins->dst);
        }
        for (int o = 0; o < q.n_outputs; ++o) {
          const int ob = st.ew_out_buf[o];
          const uint8_t src = remap(q.out[o].src);
          const bool hbm = goes_to_hbm(ob);
          if (src == EW_ACC) {
            if (o + 1 != q.n_outputs) return false;
            const int sc = rb.new_scalar();
            RowOutput* ro = rb.add_output(*ph, hbm ? ob : -1);
            if (sc < 0 || !ro) return false;
            ro->src = src; ro->scalar = (uint8_t)sc; ro->dtype = q.out[o].dtype; ro->row_stride = 1;
            rb.scalar_of[ob] = sc;
          } else {
            if (src < EW_ROWSCALAR || src >= EW_ACC) return false;
            rb.scalar_of[ob] = src - EW_ROWSCALAR;
            if (hbm) {
              RowOutput* ro = rb.add_output(*ph, ob);
              if (!ro) return false;
              ro->src = src; ro->dtype = q.out[o].dtype; ro->row_stride = 1;
            }
          }
          if (rb.read_later_in_run(ob, k, false)) ++rb.saved;
          rb.written.insert(ob);
        }
      } else if (st.kind == Step::REDUCE) {
        // ---------------- a reduction whose operand was not produced by a chain in this run ----
        RowPhase* ph = rb.begin_phase(ROW_FULL);
        if (!ph) return false;
        const int xb = st.in[0];
        int slot;
        if (rb.full_slot.count(xb)) slot = rb.full_slot[xb];
        else if (rb.written.count(xb)) return false;
        else slot = rb.leaf(*ph, xb, 0, C, 1, st.dtype, EW_IN_TENSOR);
        if (slot < 0) return false;
        const int sc = rb.new_scalar();
        RowOutput* ro = rb.add_output(*ph, goes_to_hbm(st.out[0]) ? st.out[0] : -1);
        if (sc < 0 || !ro) return false;
        ro->src = (uint8_t)slot; ro->reduce = (uint8_t)(st.reduce_kind + 1); ro->scalar = (uint8_t)sc; ro->scale = st.scale;
        ro->dtype = st.dtype2; ro->row_stride = 1;
        rb.scalar_of[st.out[0]] = sc;
        rb.written.insert(st.out[0]);
        if (rb.read_later_in_run(st.out[0], k, false)) ++rb.saved;
        has_reduce = true;
      } else if (st.kind == Step::SOFTMAX) {
        // ---------------- softmax along the row: max, exp(x - max) and its sum, the quotient ----
        const int xb = st.in[0], ob = st.out[0];
        RowPhase* p1 = rb.begin_phase(ROW_FULL);
        if (!p1) return false;
        int sx;
        if (rb.full_slot.count(xb)) sx = rb.full_slot[xb];
        else if (rb.written.count(xb)) return false;
        else sx = rb.leaf(*p1, xb, 0, C, 1, st.dtype, EW_IN_TENSOR);
        if (sx < 0) return false;
        const int m = rb.new_scalar(), sum = rb.new_scalar();
        RowOutput* o1 = rb.add_output(*p1, -1);
        if (m < 0 || sum < 0 || !o1) return false;
        o1->src = (uint8_t)sx; o1->reduce = IB200_REDUCE_MAX + 1; o1->scalar = (uint8_t)m; o1->dtype = IB200_F32;
        const bool resident = rb.read_later_in_run(ob, k, false);
        const int se = rb.alloc(resident ? rb.last_read[ob] : (int)k);
        if (se < 0) return false;
        RowPhase* p2 = rb.begin_phase(ROW_FULL);
        if (!p2) return false;
        EwInstr i1{}, i2{};
        i1.op = EW_SUB; i1.a = (uint8_t)sx; i1.b = (uint8_t)(EW_ROWSCALAR + m); i1.c = EW_ACC; i1.dst = EW_NODST;
        i2.op = EW_EXP; i2.a = i2.b = i2.c = EW_ACC; i2.dst = (uint8_t)se;
        if (!emit_accumulate_form(rb, *p2, i1) || !emit_accumulate_form(rb, *p2, i2)) return false;
        RowOutput* o2 = rb.add_output(*p2, -1);
        if (!o2) return false;
        o2->src = EW_ACC; o2->reduce = IB200_REDUCE_SUM + 1; o2->scalar = (uint8_t)sum; o2->dtype = IB200_F32;
        RowPhase* p3 = rb.begin_phase(ROW_FULL);
        if (!p3) return false;
        EwInstr i3{};
        i3.op = EW_DIV; i3.a = (uint8_t)se; i3.b = (uint8_t)(EW_ROWSCALAR + sum); i3.c = EW_ACC;
        i3.dst = resident ? (uint8_t)se : EW_NODST;
        if (!emit_accumulate_form(rb, *p3, i3)) return false;
        if (resident) {
          rb.full_slot[ob] = se;
          ++rb.saved;
        }
        if (goes_to_hbm(ob)) {
          RowOutput* o3 = rb.add_output(*p3, ob);
          if (!o3) return false;
          o3->src = EW_ACC; o3->dtype = st.dtype2; o3->row_stride = C;
        }
        rb.written.insert(ob);
        has_reduce = true;
      } else {
        return false;
      }
      rb.release((int)k);
    }
    if (!has_reduce || rb.saved == 0 || p.n_phases == 0) return false;
    // Worth it?  Small problems are launch-bound: one launch beats several.  Large ones weigh the
    // HBM round trips saved against the row kernel's interpretive cost.  The constants are
    // microseconds per million elements measured on B200 (f32 [8192,4096] rms-norm, residual
    // layernorm and masked softmax, fused and unfused): 0.82 per full-size tensor read or written
    // by a separate kernel; in the row kernel 0.4 per micro-op, 1.2 more for exp / div / rsqrt,
    // 0.5 per row reduction and 0.3 per staged operand or stored result.
    const char* mode = std::getenv("IB200_ROWFUSE");  // "2": fuse whatever fits (for measurements)
    if (R * C > (1 << 20) && !(mode && mode[0] == '2')) {
      double fused_cost = 0.0, unfused_cost = 0.0;
      for (int ph = 0; ph < p.n_phases; ++ph) {
        const RowPhase& f = p.phase[ph];
        if (f.domain != ROW_FULL) continue;
        for (int i = f.first_instr; i < f.first_instr + f.n_instr; ++i) {
          const uint8_t op = p.instr[i].op;
          fused_cost += 0.4 + ((op == EW_EXP || op == EW_DIV || op == EW_RDIV || op == EW_RSQRT) ? 1.2 : 0.0);
        }
        for (int i = f.first_input; i < f.first_input + f.n_inputs; ++i) fused_cost += p.in[i].once ? 0.0 : 0.3 * dtype_size(p.in[i].dtype) / 4.0;
        for (int i = f.first_output; i < f.first_output + f.n_outputs; ++i)
          fused_cost += p.out[i].reduce ? 0.5 : (rb.out.row_out_buf[i] >= 0 ? 0.3 * dtype_size(p.out[i].dtype) / 4.0 : 0.0);
      }
      for (size_t k = b; k < e; ++k) {
        const Step& st = steps[k];
        double tensors = 0.0;
        if (st.kind == Step::ELEMENTWISE && st.ew.total == R * C) {
          for (int i = 0; i < st.ew.n_inputs; ++i) {
            bool full = st.ew.in[i].kind == EW_IN_TENSOR;
            for (int d = 0; d < st.ew.rank; ++d) full &= st.ew.in[i].stride[d] != 0;
            if (full) tensors += dtype_size(st.ew.in[i].dtype) / 4.0;
          }
          for (int o = 0; o < st.ew.n_outputs; ++o) tensors += dtype_size(st.ew.out[o].dtype) / 4.0;
        } else if (st.kind == Step::REDUCE) {
          tensors = dtype_size(st.dtype) / 4.0;
        } else if (st.kind == Step::SOFTMAX) {
          tensors = (dtype_size(st.dtype) + dtype_size(st.dtype2)) / 4.0;
        }
        unfused_cost += 0.82 * tensors;
      }
      if (fused_cost >= unfused_cost) return false;
    }
    // renumber the slots: the per-row ones first, then the row-invariant ones (one copy per CTA)
    uint8_t perm[kRowMaxSlots];
    int n_row = 0, n_once = 0;
    for (int sl = 0; sl < rb.n_slots; ++sl)
      if (!rb.pinned[sl]) perm[sl] = (uint8_t)n_row++;
    for (int sl = 0; sl < rb.n_slots; ++sl)
      if (rb.pinned[sl]) perm[sl] = (uint8_t)(n_row + n_once++);
    auto renum = [&](uint8_t& c) { if (c < kRowMaxSlots) c = perm[c]; };
    for (int i = 0; i < p.n_inputs; ++i) renum(p.in[i].slot);
    for (int ph = 0; ph < p.n_phases; ++ph) {
      const RowPhase& f = p.phase[ph];
      if (f.domain != ROW_FULL) continue;
      for (int i = f.first_instr; i < f.first_instr + f.n_instr; ++i) {
        renum(p.instr[i].a); renum(p.instr[i].b); renum(p.instr[i].c);
        if (p.instr[i].dst != EW_NODST) renum(p.instr[i].dst);
      }
      for (int i = f.first_output; i < f.first_output + f.n_outputs; ++i) renum(p.out[i].src);
    }
    p.n_row_slots = n_row;
    p.n_once_slots = n_once;
    if (!row_program_fits(n_row, n_once, (int)C)) return false;
    fused = rb.out;
    fused.kind = Step::ROWFUSE;
    fused.d[0] = R;
    fused.d[1] = C;
    fused.label = "rowfused(" + std::to_string(e - b) + " steps, " + std::to_string(p.n_phases) + " phases)";
    return true;
  }

  void fuse_rows() {
    if (const char* env = std::getenv("IB200_ROWFUSE"))
      if (env[0] == '0') return;
    std::vector<Step>& steps = plan_->steps;
    size_t floor = 0;  // steps before this index are final
    for (size_t a = 0; a < steps.size(); ++a) {
      int64_t R, C;
      if (a < floor || !row_anchor(steps[a], R, C)) continue;
      size_t b = a, e = a + 1;
      while (b > floor && row_candidate(steps[b - 1], R, C)) --b;
      while (e < steps.size() && row_candidate(steps[e], R, C)) ++e;
      bool done = false;
      for (size_t b2 = b; b2 <= a && !done; ++b2)
        for (size_t e2 = e; e2 > a && e2 - b2 >= 2 && !done; --e2) {
          Step fused;
          if (!build_row_program(b2, e2, R, C, fused)) continue;
          steps.erase(steps.begin() + b2, steps.begin() + e2);
          steps.insert(steps.begin() + b2, fused);
          floor = b2 + 1;
          a = b2;  // the loop's ++a moves past the fused step
          done = true;
        }
      if (!done) floor = std::max(floor, b);
    }
  }

  // =============================== description ==============================================
  // the row program in readable form, so that the host side (and its tests) can inspect what
  // a fused step does without a GPU
  static const char* op_name(int op) {
    static const char* kOps[] = {"mov", "add", "sub", "mul", "div", "max", "min", "relu", "exp", "rsqrt", "abs", "floor", "ne", "lt", "le",
                                 "gt", "ge", "and", "or", "not", "where", "to_bool", "to_int", "round_bf16", "round_f16", "rsub", "rdiv", "loadb"};
    return op >= 0 && op < EW_NUM_OPS ? kOps[op] : "?";
  }
  static Json describe_ew_program(const Step& s) {
    auto num = [](double v) { return Json::number(v); };
    const EwProgram& p = s.ew;
    Json r = Json::object(), ins = Json::array(), code = Json::array(), outs = Json::array();
    for (int k = 0; k < p.n_inputs; ++k) {
      Json j = Json::object(), st = Json::array();
      j.set("buffer", num(s.ew_in_buf[k])); j.set("offset", num((double)s.ew_in_off[k]));
      j.set("dtype", Json::string(dtype_name(p.in[k].dtype))); j.set("iota", num(p.in[k].kind == EW_IN_IOTA));
      for (int d = 0; d < p.rank; ++d) st.push(num((double)p.in[k].stride[d]));
      j.set("strides", st);
      ins.push(j);
    }
    for (int k = 0; k < p.n_instr; ++k) {
      const EwInstr& i = p.instr[k];
      Json j = Json::object();
      j.set("op", Json::string(op_name(i.op)));
      j.set("a", num(i.a)); j.set("b", num(i.b)); j.set("c", num(i.c)); j.set("dst", num(i.dst));
      j.set("imm", num(s.wide && k < (int)s.ew_imm.size() ? s.ew_imm[k] : (double)i.imm));  // what the kernel that runs is given
      code.push(j);
    }
    for (int k = 0; k < p.n_outputs; ++k) {
      Json j = Json::object();
      j.set("buffer", num(s.ew_out_buf[k])); j.set("dtype", Json::string(dtype_name(p.out[k].dtype))); j.set("src", num(p.out[k].src));
      outs.push(j);
    }
    r.set("inputs", ins); r.set("instr", code); r.set("outputs", outs); r.set("n_slots", num(p.n_slots));
    r.set("wide", num(s.wide));
    if (!s.wide) {
      bool compiled_in = false;
      const std::string sig = ew_register_signature(p, &compiled_in);
      r.set("register_code", Json::string(sig));
      r.set("compiled_in", num(compiled_in ? 1 : 0));
    }
    return r;
  }
  static Json describe_row_program(const Step& s) {
    static const char* kOps[] = {"mov", "add", "sub", "mul", "div", "max", "min", "relu", "exp", "rsqrt", "abs", "floor", "ne", "lt", "le",
                                 "gt", "ge", "and", "or", "not", "where", "to_bool", "to_int", "round_bf16", "round_f16", "rsub", "rdiv", "loadb"};
    auto num = [](double v) { return Json::number(v); };
    const RowProgram& p = s.row;
    Json r = Json::object();
    r.set("rows", num((double)p.rows));
    r.set("cols", num(p.cols));
    r.set("n_row_slots", num(p.n_row_slots));
    r.set("n_once_slots", num(p.n_once_slots));
    r.set("n_scalars", num(p.n_scalars));
    r.set("compiled_in", Json::boolean(row_program_compiled_in(p)));
    Json phases = Json::array();
    for (int ph = 0; ph < p.n_phases; ++ph) {
      const RowPhase& f = p.phase[ph];
      Json jp = Json::object(), ins = Json::array(), lds = Json::array(), code = Json::array(), outs = Json::array();
      jp.set("domain", Json::string(f.domain == ROW_FULL ? "full" : "scalar"));
      for (int k = f.first_input; k < f.first_input + f.n_inputs; ++k) {
        Json j = Json::object();
        j.set("buffer", num(s.row_in_buf[k])); j.set("offset", num((double)s.row_in_off[k]));
        j.set("row_stride", num((double)p.in[k].row_stride)); j.set("col_stride", num(p.in[k].col_stride));
        j.set("dtype", Json::string(dtype_name(p.in[k].dtype))); j.set("iota", num(p.in[k].kind == EW_IN_IOTA));
        j.set("slot", num(p.in[k].slot)); j.set("once", num(p.in[k].once));
        ins.push(j);
      }
      for (int k = f.first_load; k < f.first_load + f.n_loads; ++k) {
        Json j = Json::object();
        j.set("buffer", num(s.row_load_buf[k])); j.set("offset", num((double)s.row_load_off[k]));
        j.set("row_stride", num((double)p.load[k].row_stride)); j.set("dtype", Json::string(dtype_name(p.load[k].dtype)));
        j.set("scalar", num(p.load[k].scalar));
        lds.push(j);
      }
      for (int k = f.first_instr; k < f.first_instr + f.n_instr; ++k) {
        const EwInstr& i = p.instr[k];
        Json j = Json::object();
        j.set("op", Json::string(i.op < EW_NUM_OPS ? kOps[i.op] : "?"));
        j.set("a", num(i.a)); j.set("b", num(i.b)); j.set("c", num(i.c)); j.set("dst", num(i.dst)); j.set("imm", num(i.imm));
        code.push(j);
      }
      for (int k = f.first_output; k < f.first_output + f.n_outputs; ++k) {
        const RowOutput& o = p.out[k];
        Json j = Json::object();
        j.set("buffer", num(s.row_out_buf[k])); j.set("row_stride", num((double)o.row_stride));
        j.set("dtype", Json::string(dtype_name(o.dtype))); j.set("src", num(o.src)); j.set("reduce", num(o.reduce));
        j.set("scalar", num(o.scalar)); j.set("scale", num(o.scale));
        outs.push(j);
      }
      jp.set("inputs", ins); jp.set("loads", lds); jp.set("instr", code); jp.set("outputs", outs);
      phases.push(jp);
    }
    r.set("phases", phases);
    return r;
  }

  void finish() {
    if (plan_->uses_status) {
      plan_->status_offset = plan_->workspace_bytes;
      plan_->workspace_bytes += 256;
    }
    Json d = Json::object();
    d.set("kernel_name", Json::string(plan_->kernel_name));
    d.set("cuda_src", Json::string(""));
    Json io = Json::object(), names = Json::array(), tensors = Json::object();
    for (auto& a : plan_->arg_names) names.push(Json::string(a));
    for (size_t i = 0; i < plan_->arg_names.size(); ++i) {
      const Buffer& b = plan_->buffers[i];
      Json t = Json::object(), sh = Json::array();
      t.set("dtype", Json::string(dtype_name(b.dtype)));
      for (auto v : nodes_[by_name_[b.name]].shape) sh.push(Json::number((double)v));
      t.set("shape", sh);
      tensors.set(b.name, t);
    }
    io.set("arg_names", names);
    io.set("tensors", tensors);
    io.set("scalars", Json::object());
    d.set("io_spec", io);
    Json launch = Json::object(), g3 = Json::array(), b3 = Json::array();
    for (int i = 0; i < 3; ++i) { g3.push(Json::number(i == 0 ? (double)plan_->steps.size() : 1)); b3.push(Json::number(1)); }
    launch.set("grid", g3);  // informational: grids are chosen by the kernels' launchers
    launch.set("block", b3);
    launch.set("shared_mem", Json::number(0));
    d.set("launch", launch);
    Json outs = Json::array();
    for (auto& o : plan_->output_names) outs.push(Json::string(o));
    d.set("output_names", outs);
    Json binds = Json::object();
    for (auto& kv : bind_) binds.set(kv.first, Json::number(kv.second));
    d.set("bindings", binds);
    Json steps = Json::array();
    for (auto& s : plan_->steps) {
      Json j = Json::object();
      j.set("kernel", Json::string(s.label));
      Json ext = Json::array();
      for (int i = 0; i < 4; ++i) ext.push(Json::number((double)s.d[i]));
      if (s.kind == Step::ELEMENTWISE) { ext = Json::array(); for (int i = 0; i < s.ew.rank; ++i) ext.push(Json::number((double)s.ew.dim[i])); }
      j.set("extents", ext);
      if (s.kind == Step::ROWFUSE) j.set("row_program", describe_row_program(s));
      if (s.kind == Step::ELEMENTWISE) j.set("program", describe_ew_program(s));
      if (s.kind == Step::REDUCE || s.kind == Step::SOFTMAX || s.kind == Step::NORM || s.kind == Step::GEMM || s.kind == Step::TRANSPOSE ||
          s.kind == Step::GATHER) {
        // what the launcher of this step is given, buffer ids in place of pointers: a CPU restatement of the
        // kernels' contracts can then run the whole plan
        auto num = [](double v) { return Json::number(v); };
        auto ids = [&](const int* v, int n) { Json a = Json::array(); for (int k = 0; k < n; ++k) a.push(num(v[k])); return a; };
        Json a = Json::object(), res = Json::array(), bs = Json::array();
        static const char* kKinds[] = {"reduce", "softmax", "norm", "gemm", "elementwise", "transpose", "gather"};
        a.set("kind", Json::string(kKinds[s.kind]));
        a.set("in", ids(s.in, 3)); a.set("out", ids(s.out, 3));
        a.set("dtype", Json::string(dtype_name(s.dtype))); a.set("dtype2", Json::string(dtype_name(s.dtype2)));
        a.set("reduce_kind", num(s.reduce_kind)); a.set("scale", num(s.scale)); a.set("eps", num(s.eps));
        a.set("aff_inner", num((double)s.aff_inner)); a.set("aff_period", num((double)s.aff_period));
        a.set("transpose_b", num(s.transpose_b)); a.set("act", num(s.act)); a.set("other", num(s.other));
        a.set("batch", num((double)s.batch)); a.set("flags", num(s.flags));
        for (int k = 0; k < 3; ++k) bs.push(num((double)s.batch_stride[k]));
        a.set("batch_stride", bs);
        if (s.kind == Step::NORM) for (int id : s.idx_buf) res.push(num(id));
        a.set("residual", res);
        if (s.kind == Step::GATHER) {  // one index buffer per data axis, with the axis' extent and stride
          Json idx = Json::array(), dim = Json::array(), stride = Json::array();
          for (size_t k = 0; k < s.idx_buf.size(); ++k) { idx.push(num(s.idx_buf[k])); dim.push(num((double)s.g_dim[k])); stride.push(num((double)s.g_stride[k])); }
          a.set("index", idx); a.set("dim", dim); a.set("stride", stride);
        }
        j.set("args", a);
      }
      steps.push(j);
    }
    d.set("steps", steps);
    Json bufs = Json::array();
    for (auto& b : plan_->buffers) {
      Json j = Json::object();
      j.set("name", Json::string(b.name));
      j.set("arg", Json::number(b.is_arg ? b.arg_index : -1));
      j.set("dtype", Json::string(dtype_name(b.dtype)));
      j.set("bytes", Json::number((double)b.bytes));
      bufs.push(j);
    }
    d.set("buffers", bufs);
    d.set("workspace_bytes", Json::number((double)plan_->workspace_bytes));
    d.set("status_offset", Json::number(plan_->uses_status ? (double)plan_->status_offset : -1.0));
    plan_->description = d;
  }
};

void* buffer_ptr(const ib200_plan& p, int id, void* const* args, void* ws) {
  if (id < 0) return nullptr;
  const Buffer& b = p.buffers[id];
  return b.is_arg ? args[b.arg_index] : static_cast<char*>(ws) + b.ws_offset;
}

int write_out(const std::string& s, char* out, size_t cap) {
  if (!out || cap < s.size() + 1) return fail(IB200_ERR_BUFFER, "output buffer too small: " + std::to_string(s.size() + 1) + " bytes needed");
  std::memcpy(out, s.c_str(), s.size() + 1);
  return IB200_OK;
}

int create(const char* intent_json, const char* bindings_json, std::unique_ptr<ib200_plan>& out) {
  try {
    Json intent = Json::parse(intent_json);
    Json bindings = bindings_json && *bindings_json ? Json::parse(bindings_json) : Json::object();
    Planner pl(intent, bindings);
    out = pl.run();
    return IB200_OK;
  } catch (const Unsupported& e) {
    return fail(IB200_ERR_UNSUPPORTED, e.what());
  } catch (const std::exception& e) {
    return fail(IB200_ERR_INVALID, e.what());
  }
}

}  // namespace
}  // namespace ib200

namespace ib200 {
long plan_status_offset(const ib200_plan* plan) { return plan && plan->uses_status ? (long)plan->status_offset : -1; }
}  // namespace ib200

using namespace ib200;

extern "C" {

int ib200_plan_create(const char* intent_json, const char* bindings_json, ib200_plan_t** plan) {
  if (!plan || !intent_json) return fail(IB200_ERR_INVALID, "plan_create: null argument");
  std::unique_ptr<ib200_plan> p;
  if (int rc = create(intent_json, bindings_json, p)) return rc;
  *plan = p.release();
  return IB200_OK;
}

void ib200_plan_destroy(ib200_plan_t* plan) { delete plan; }

int ib200_plan_describe(const ib200_plan_t* plan, char* out, size_t cap) {
  if (!plan) return fail(IB200_ERR_INVALID, "plan_describe: null plan");
  return write_out(plan->description.dump(), out, cap);
}

int ib200_plan_json(const char* intent_json, const char* bindings_json, char* out, size_t cap) {
  if (!intent_json) return fail(IB200_ERR_INVALID, "plan_json: null intent");
  std::unique_ptr<ib200_plan> p;
  if (int rc = create(intent_json, bindings_json, p)) return rc;
  return write_out(p->description.dump(), out, cap);
}

int ib200_plan_num_args(const ib200_plan_t* plan) { return plan ? (int)plan->arg_names.size() : 0; }
size_t ib200_plan_workspace_bytes(const ib200_plan_t* plan) { return plan ? plan->workspace_bytes : 0; }
int ib200_plan_num_launches(const ib200_plan_t* plan) {
  int n = 0;
  if (plan) for (const Step& st : plan->steps) n += st.kind == Step::GEMM ? (int)st.batch : 1;
  return n;
}

int ib200_plan_check_status(const ib200_plan_t* plan, const void* workspace, void* stream) {
  if (!plan) return fail(IB200_ERR_INVALID, "plan_check_status: null plan");
  if (!plan->uses_status) return IB200_OK;  // no kernel of this plan has a bounded wait
  if (!workspace) return fail(IB200_ERR_INVALID, "plan_check_status: this plan keeps its status word in the workspace; pass it");
  return ib200_check_status(reinterpret_cast<const int32_t*>(static_cast<const char*>(workspace) + plan->status_offset), stream);
}

int ib200_plan_launch(const ib200_plan_t* plan, void* const* args, int n_args, void* workspace, size_t workspace_bytes, void* stream) {
  if (!plan) return fail(IB200_ERR_INVALID, "plan_launch: null plan");
  if (n_args != (int)plan->arg_names.size()) return fail(IB200_ERR_INVALID, "plan_launch: expected " + std::to_string(plan->arg_names.size()) + " arguments");
  if (n_args > 0 && !args) return fail(IB200_ERR_INVALID, "plan_launch: null argument array");
  if (plan->workspace_bytes > 0 && (!workspace || workspace_bytes < plan->workspace_bytes))
    return fail(IB200_ERR_BUFFER, "plan_launch: workspace of " + std::to_string(plan->workspace_bytes) + " bytes needed");
  if (plan->workspace_bytes > 0 && (reinterpret_cast<uintptr_t>(workspace) & 255u)) return fail(IB200_ERR_INVALID, "plan_launch: workspace must be 256-byte aligned");
  for (size_t i = 0; i < plan->arg_names.size(); ++i)
    if (!args[i] && plan->buffers[i].bytes > 0) return fail(IB200_ERR_INVALID, "plan_launch: argument '" + plan->arg_names[i] + "' is null");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int32_t* status = plan->uses_status ? reinterpret_cast<int32_t*>(static_cast<char*>(workspace) + plan->status_offset) : nullptr;
  for (const Step& st : plan->steps) {
    int rc = IB200_OK;
    auto P = [&](int id) { return buffer_ptr(*plan, id, args, workspace); };
    switch (st.kind) {
      case Step::REDUCE:
        rc = launch_reduce(P(st.in[0]), P(st.out[0]), st.dtype, st.dtype2, st.reduce_kind, st.d[0], st.d[1], st.d[2], st.scale, s,
                           st.scratch >= 0 ? P(st.scratch) : nullptr, st.scratch >= 0 ? plan->buffers[st.scratch].bytes : 0);
        break;
      case Step::SOFTMAX: {
        const SoftmaxMask mk{static_cast<const uint8_t*>(st.reduce_kind ? P(st.in[1]) : nullptr), st.aff_inner, (float)st.other, 0};
        rc = launch_softmax(P(st.in[0]), P(st.out[0]), static_cast<float*>(P(st.out[1])), static_cast<float*>(P(st.out[2])), st.dtype,
                            st.d[0], st.d[1], s, st.dtype2, st.reduce_kind ? &mk : nullptr, st.scratch >= 0 ? P(st.scratch) : nullptr,
                            st.scratch >= 0 ? plan->buffers[st.scratch].bytes : 0);
        break;
      }
      case Step::NORM:
        rc = launch_norm_rows(P(st.in[0]), P(st.in[1]), P(st.in[2]), P(st.out[0]), static_cast<float*>(P(st.out[1])),
                              static_cast<float*>(P(st.out[2])), st.dtype, st.dtype2, st.d[0], st.d[1], st.aff_inner, st.aff_period,
                              st.eps, s, status, st.act != 0, st.idx_buf.size() > 0 ? P(st.idx_buf[0]) : nullptr,
                              st.idx_buf.size() > 1 ? P(st.idx_buf[1]) : nullptr, st.scratch >= 0 ? P(st.scratch) : nullptr,
                              st.scratch >= 0 ? plan->buffers[st.scratch].bytes : 0, st.flags);
        break;
      case Step::GEMM:
        for (int64_t bi = 0; bi < st.batch && rc == IB200_OK; ++bi)
          rc = launch_gemm(static_cast<const char*>(P(st.in[0])) + bi * st.batch_stride[0] * dtype_size(st.dtype),
                           static_cast<const char*>(P(st.in[1])) + bi * st.batch_stride[1] * dtype_size(st.dtype), P(st.in[2]),
                           static_cast<char*>(P(st.out[0])) + bi * st.batch_stride[2] * dtype_size(st.dtype2), st.dtype, st.dtype2,
                           st.d[0], st.d[1], st.d[2], st.transpose_b, st.act, status, s, st.flags,
                           st.scratch >= 0 ? P(st.scratch) : nullptr, st.scratch >= 0 ? plan->buffers[st.scratch].bytes : 0);
        break;
      case Step::GATHER: {
        GatherArgs ga{};
        ga.n = st.d[0];
        ga.n_idx = (int)st.idx_buf.size();
        ga.idx_is_64 = st.dtype2 == IB200_I64;
        for (int k = 0; k < ga.n_idx; ++k) { ga.idx[k] = P(st.idx_buf[k]); ga.dim[k] = st.g_dim[k]; ga.stride[k] = st.g_stride[k]; }
        rc = launch_gather(P(st.in[0]), ga, P(st.out[0]), dtype_size(st.dtype), st.other, s);
        break;
      }
      case Step::ROPE:
        rc = launch_rope(static_cast<const float*>(P(st.in[0])), static_cast<const float*>(P(st.in[1])), static_cast<const float*>(P(st.in[2])),
                         static_cast<float*>(P(st.out[0])), st.d[0], st.d[1], st.d[2], s);
        break;
      case Step::DROPOUT:
        rc = launch_dropout(static_cast<const float*>(P(st.in[0])), static_cast<float*>(P(st.out[0])), st.d[0], P(st.in[1]), st.dtype,
                            (float)st.other, P(st.in[2]), st.dtype2, st.seed, (int)st.d[1], s);
        break;
      case Step::CORRELATION:
        rc = launch_correlation(static_cast<const int8_t*>(P(st.in[0])), static_cast<const int8_t*>(P(st.in[1])), static_cast<int8_t*>(P(st.out[0])),
                                st.d[0], st.d[3], st.d[1], st.d[2], P(st.in[2]), st.dtype2, (int)st.seed, s);
        break;
      case Step::RESIZE:
        rc = launch_resize2x(static_cast<const int8_t*>(P(st.in[0])), static_cast<int8_t*>(P(st.out[0])), st.d[0], st.d[1], st.d[2], (int)st.d[3], s);
        break;
      case Step::WARP:
        rc = launch_warp(static_cast<const int8_t*>(P(st.in[0])), static_cast<const int16_t*>(P(st.in[1])), static_cast<int8_t*>(P(st.out[0])),
                         st.d[0], st.d[1], st.d[2], s);
        break;
      case Step::TRANSPOSE:
        rc = launch_transpose2d(P(st.in[0]), P(st.out[0]), dtype_size(st.dtype), st.d[0], st.d[1], s);
        break;
      case Step::ELEMENTWISE: {
        EwProgram prog = st.ew;
        bool vec = prog.dim[prog.rank - 1] % 4 == 0;
        for (int k = 0; k < prog.n_inputs; ++k) {
          EwInput& in = prog.in[k];
          if (in.kind == EW_IN_TENSOR) {
            in.ptr = static_cast<const char*>(P(st.ew_in_buf[k])) + st.ew_in_off[k] * dtype_size(in.dtype);
            bool ok = in.stride[prog.rank - 1] == 1 && aligned16(in.ptr);
            for (int d = 0; d + 1 < prog.rank; ++d) ok &= in.stride[d] % 4 == 0;
            in.vec_ok = ok;
          }
        }
        for (int o = 0; o < prog.n_outputs; ++o) {
          prog.out[o].ptr = P(st.ew_out_buf[o]);
          vec &= aligned16(prog.out[o].ptr);
        }
        prog.vec = vec;
        rc = st.wide ? launch_elementwise_wide(prog, st.ew_imm.data(), s) : launch_elementwise(prog, s);
        break;
      }
      case Step::ROWFUSE: {
        RowProgram prog = st.row;
        for (int k = 0; k < prog.n_inputs; ++k) {
          RowInput& in = prog.in[k];
          if (in.kind != EW_IN_TENSOR) continue;
          in.ptr = static_cast<const char*>(P(st.row_in_buf[k])) + st.row_in_off[k] * dtype_size(in.dtype);
          in.vec_ok = in.col_stride == 1 && aligned16(in.ptr) && in.row_stride % 4 == 0;
        }
        for (int k = 0; k < prog.n_loads; ++k)
          prog.load[k].ptr = static_cast<const char*>(P(st.row_load_buf[k])) + st.row_load_off[k] * dtype_size(prog.load[k].dtype);
        for (int k = 0; k < prog.n_outputs; ++k) {
          RowOutput& o = prog.out[k];
          o.ptr = st.row_out_buf[k] >= 0 ? P(st.row_out_buf[k]) : nullptr;
          o.vec_ok = o.ptr && aligned16(o.ptr) && o.row_stride % 4 == 0;
        }
        rc = launch_row_program(prog, s);
        break;
      }
    }
    if (rc != IB200_OK) return rc;
  }
  return IB200_OK;
}

}  // extern "C"
