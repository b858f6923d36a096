#include "passes.h"

#include <cmath>
#include <cstring>
#include <fstream>
#include <iomanip>
#include <sstream>

namespace b200c {

// ---------------------------------------------------------------------------- helpers
static std::vector<long long> ints(const Json& a) {
  std::vector<long long> out;
  for (size_t i = 0; i < a.size(); ++i) out.push_back(a.at(i).as_int());
  return out;
}
static Json int_array(const std::vector<long long>& v) {
  Json a = Json::make_array();
  for (auto x : v) a.arr.push_back(Json::make_int(x));
  return a;
}
static std::string b64_encode(const std::vector<uint8_t>& in) {
  static const char* tbl = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/";
  std::string out;
  size_t i = 0;
  for (; i + 2 < in.size(); i += 3) {
    uint32_t v = (in[i] << 16) | (in[i + 1] << 8) | in[i + 2];
    out += tbl[(v >> 18) & 63]; out += tbl[(v >> 12) & 63]; out += tbl[(v >> 6) & 63]; out += tbl[v & 63];
  }
  if (i + 1 == in.size()) {
    uint32_t v = in[i] << 16;
    out += tbl[(v >> 18) & 63]; out += tbl[(v >> 12) & 63]; out += "==";
  } else if (i + 2 == in.size()) {
    uint32_t v = (in[i] << 16) | (in[i + 1] << 8);
    out += tbl[(v >> 18) & 63]; out += tbl[(v >> 12) & 63]; out += tbl[(v >> 6) & 63]; out += '=';
  }
  return out;
}

static bool constant_bytes(const Node* n, std::vector<uint8_t>& bytes) {
  if (!n || n->opcode != "constant" || !n->attrs.has("value")) return false;
  const Json& v = n->attrs.at("value");
  if (!v.has("data")) return false;
  bytes = spike::base64_decode(v.at("data").as_string());
  return true;
}

// value is a splat of one scalar: constant (any shape, all elements equal) possibly broadcast / reshaped
static bool splat_f64(const Value* v, double& out) {
  const Node* n = v->producer;
  while (n && (n->opcode == "broadcast" || n->opcode == "reshape")) n = n->inputs[0]->producer;
  std::vector<uint8_t> b;
  if (!constant_bytes(n, b)) return false;
  const std::string dt = n->outputs[0]->dtype;
  const size_t w = dtype_bytes(dt);
  if (b.empty() || b.size() % w) return false;
  for (size_t i = w; i < b.size(); ++i)
    if (b[i] != b[i % w]) return false;
  if (dt == "f32") { float f; std::memcpy(&f, b.data(), 4); out = f; return true; }
  if (dt == "f64") { std::memcpy(&out, b.data(), 8); return true; }
  if (dt == "i32") { int32_t x; std::memcpy(&x, b.data(), 4); out = x; return true; }
  if (dt == "bf16") { uint32_t u = (uint32_t(b[1]) << 24) | (uint32_t(b[0]) << 16); float f; std::memcpy(&f, &u, 4); out = f; return true; }
  bool zero = true;
  for (uint8_t x : b) zero = zero && x == 0;
  if (zero) { out = 0; return true; }
  return false;
}

static Value* make_f32_splat(Graph& g, Node* before, float value, const std::vector<long long>& shape,
                             const std::string& loc) {
  std::vector<uint8_t> raw(4);
  std::memcpy(raw.data(), &value, 4);
  Json t = Json::make_object();
  t.set("__tensor__", Json::make_str("f32"));
  t.set("shape", Json::make_array());
  t.set("data", Json::make_str(b64_encode(raw)));
  Json attrs = Json::make_object();
  attrs.set("value", t);
  Node* c = g.insert_node(before, "constant", {}, attrs, {{"f32", {}}}, loc);
  if (shape.empty()) return c->outputs[0];
  Json battrs = Json::make_object();
  battrs.set("shape", int_array(shape));
  battrs.set("dims", Json::make_array());
  Node* b = g.insert_node(before, "broadcast", {c->outputs[0]}, battrs, {{"f32", shape}}, loc);
  return b->outputs[0];
}

static void dce(Graph& g) {
  bool changed = true;
  while (changed) {
    changed = false;
    auto uses = g.use_counts();
    for (auto it = g.nodes.rbegin(); it != g.nodes.rend(); ++it) {
      Node* n = *it;
      if (n->dead) continue;
      bool used = false;
      for (Value* o : n->outputs) used = used || uses[o] > 0;
      if (!used) {
        n->dead = true;
        changed = true;
      }
    }
    g.sweep();
  }
}

static void forward(Graph& g, Node* n, Value* replacement) {
  g.replace_all_uses(n->outputs[0], replacement);
  n->dead = true;
}

// ---------------------------------------------------------------------------- canonicalize group
static void remove_redundant_zero_fill(Graph& g, const PassOptions&) {
  for (Node* n : g.nodes) {
    if (n->dead || n->opcode != "add") continue;
    double c;
    if (splat_f64(n->inputs[1], c) && c == 0.0) forward(g, n, n->inputs[0]);
    else if (splat_f64(n->inputs[0], c) && c == 0.0) forward(g, n, n->inputs[1]);
  }
  g.sweep();
  dce(g);
}

static void prepare_arithmetic(Graph& g, const PassOptions& o) {
  std::vector<Node*> snapshot = g.nodes;
  for (Node* n : snapshot) {
    if (n->dead) continue;
    double c;
    if (n->opcode == "pow" && splat_f64(n->inputs[1], c) && c == 2.0) {
      n->opcode = "mul";
      n->inputs[1] = n->inputs[0];
    } else if (o.fast_math && n->opcode == "div" && n->outputs[0]->dtype == "f32" && splat_f64(n->inputs[1], c) &&
               c != 0.0 && std::isfinite(c)) {
      Value* r = make_f32_splat(g, n, float(1.0 / c), n->outputs[0]->shape, n->loc);
      n->opcode = "mul";
      n->inputs[1] = r;
    }
  }
  dce(g);
}

static void decompose_batch_matmul(Graph& g, const PassOptions&) {
  for (Node* n : g.nodes) {
    if (n->opcode != "dot") continue;
    const size_t nb = n->attrs.at("lhs_batch").size();
    if (nb == 0) continue;
    long long count = 1;
    for (auto d : ints(n->attrs.at("lhs_batch"))) count *= n->inputs[0]->shape[size_t(d)];
    n->attrs.set("_batch", Json::make_str("grid.z"));
    n->attrs.set("_batch_count", Json::make_int(count));
  }
}

static bool swaps_last_two(const std::vector<long long>& perm) {
  const size_t r = perm.size();
  if (r < 2) return false;
  for (size_t i = 0; i + 2 < r; ++i)
    if (perm[i] != (long long)i) return false;
  return perm[r - 2] == (long long)(r - 1) && perm[r - 1] == (long long)(r - 2);
}

static void canonicalize_partition_dim(Graph& g, const PassOptions&) {
  auto uses = g.use_counts();
  for (Node* n : g.nodes) {
    if (n->dead || n->opcode != "dot") continue;
    for (int side = 0; side < 2; ++side) {
      Value* op = n->inputs[size_t(side)];
      Node* t = op->producer;
      const char* ckey = side == 0 ? "lhs_contract" : "rhs_contract";
      const char* bkey = side == 0 ? "lhs_batch" : "rhs_batch";
      auto contract = ints(n->attrs.at(ckey));
      const long long rank = (long long)op->shape.size();
      const bool batch_leading = [&] {
        auto b = ints(n->attrs.at(bkey));
        for (size_t i = 0; i < b.size(); ++i)
          if (b[i] != (long long)i) return false;
        return (long long)b.size() == rank - 2;
      }();
      std::string major = "K";
      // the operand is K-major when its contracting dimension is the contiguous (last) one
      if (contract.size() == 1 && rank >= 2) major = contract[0] == rank - 1 ? "K" : "MN";
      if (t && t->opcode == "transpose" && uses[op] == 1 && contract.size() == 1 && batch_leading &&
          swaps_last_two(ints(t->attrs.at("perm")))) {
        // dot(transpose(x)) == dot(x) contracting the other of the last two dims
        n->inputs[size_t(side)] = t->inputs[0];
        const long long other = contract[0] == rank - 1 ? rank - 2 : rank - 1;
        n->attrs.set(ckey, int_array({other}));
        major = other == rank - 1 ? "K" : "MN";
      }
      n->attrs.set(side == 0 ? "_a_major" : "_b_major", Json::make_str(major));
    }
  }
  dce(g);
}

static void canonicalize_reshape(Graph& g, const PassOptions&) {
  for (Node* n : g.nodes) {
    if (n->dead || n->opcode != "reshape") continue;
    Node* p = n->inputs[0]->producer;
    if (p && p->opcode == "reshape") n->inputs[0] = p->inputs[0];
    if (n->inputs[0]->shape == n->outputs[0]->shape) forward(g, n, n->inputs[0]);
  }
  g.sweep();
  dce(g);
}

// ---- simplify-linalg: compositions of data-movement operations become one operation, and data movement that moves
// nothing becomes a reshape (a view).  Patterns return true when they rewrote `n`.
static bool compose_transposes(Graph& g, Node* n) {
  if (n->opcode != "transpose") return false;
  auto perm = ints(n->attrs.at("perm"));
  bool changed = false;
  Node* p = n->inputs[0]->producer;
  if (p && p->opcode == "transpose") {
    auto inner = ints(p->attrs.at("perm"));
    std::vector<long long> composed(perm.size());
    for (size_t i = 0; i < perm.size(); ++i) composed[i] = inner[size_t(perm[i])];
    perm = composed;
    n->inputs[0] = p->inputs[0];
    n->attrs.set("perm", int_array(perm));
    changed = true;
  }
  bool identity = true;
  for (size_t i = 0; i < perm.size(); ++i) identity = identity && perm[i] == (long long)i;
  if (identity) return forward(g, n, n->inputs[0]), true;
  return changed;
}

// a transpose that keeps the order of all dimensions larger than one moves no element
static bool transpose_of_unit_dims(Graph&, Node* n) {
  if (n->opcode != "transpose") return false;
  auto perm = ints(n->attrs.at("perm"));
  const auto& in = n->inputs[0]->shape;
  long long last = -1;
  for (long long d : perm) {
    if (in[size_t(d)] == 1) continue;
    if (d < last) return false;
    last = d;
  }
  n->opcode = "reshape";
  Json attrs = Json::make_object();
  attrs.set("shape", int_array(n->outputs[0]->shape));
  for (const auto& kv : n->attrs.obj)
    if (!kv.first.empty() && kv.first[0] == '_') attrs.set(kv.first, kv.second);
  n->attrs = attrs;
  return true;
}

// sum / max / min / prod over dimensions of extent one is a reshape
static bool reduce_of_unit_dims(Graph&, Node* n) {
  if (n->opcode != "reduce") return false;
  const std::string kind = n->attrs.at("kind").as_string();
  if (kind != "sum" && kind != "max" && kind != "min" && kind != "prod") return false;
  if (n->inputs[0]->dtype != n->outputs[0]->dtype) return false;
  for (long long a : ints(n->attrs.at("axes")))
    if (n->inputs[0]->shape[size_t(a)] != 1) return false;
  n->opcode = "reshape";
  Json attrs = Json::make_object();
  attrs.set("shape", int_array(n->outputs[0]->shape));
  n->attrs = attrs;
  return true;
}

static bool compose_slices(Graph&, Node* n) {
  if (n->opcode != "slice") return false;
  Node* p = n->inputs[0]->producer;
  if (!p || p->opcode != "slice") return false;
  auto s1 = ints(p->attrs.at("start")), t1 = ints(p->attrs.at("stride"));
  auto s2 = ints(n->attrs.at("start")), t2 = ints(n->attrs.at("stride"));
  const auto& out = n->outputs[0]->shape;
  std::vector<long long> start(s1.size()), stride(s1.size()), limit(s1.size());
  for (size_t i = 0; i < s1.size(); ++i) {
    start[i] = s1[i] + s2[i] * t1[i];
    stride[i] = t1[i] * t2[i];
    limit[i] = out[i] == 0 ? start[i] : start[i] + (out[i] - 1) * stride[i] + 1;
  }
  n->inputs[0] = p->inputs[0];
  n->attrs.set("start", int_array(start));
  n->attrs.set("stride", int_array(stride));
  n->attrs.set("limit", int_array(limit));
  return true;
}

// a slice that takes everything
static bool full_slice(Graph& g, Node* n) {
  if (n->opcode != "slice" || n->inputs[0]->shape != n->outputs[0]->shape) return false;
  for (long long t : ints(n->attrs.at("stride")))
    if (t != 1) return false;
  return forward(g, n, n->inputs[0]), true;
}

static bool compose_broadcasts(Graph&, Node* n) {
  if (n->opcode != "broadcast") return false;
  Node* p = n->inputs[0]->producer;
  if (!p || p->opcode != "broadcast") return false;
  auto inner = ints(p->attrs.at("dims")), outer = ints(n->attrs.at("dims"));
  std::vector<long long> dims(inner.size());
  for (size_t i = 0; i < inner.size(); ++i) dims[i] = outer[size_t(inner[i])];
  n->inputs[0] = p->inputs[0];
  n->attrs.set("dims", int_array(dims));
  return true;
}

// reshape / transpose / slice of a broadcast scalar is a broadcast of that scalar
static bool view_of_splat(Graph&, Node* n) {
  if (n->opcode != "reshape" && n->opcode != "transpose" && n->opcode != "slice") return false;
  Node* p = n->inputs[0]->producer;
  if (!p || p->opcode != "broadcast" || !p->inputs[0]->shape.empty()) return false;
  n->opcode = "broadcast";
  n->inputs[0] = p->inputs[0];
  Json attrs = Json::make_object();
  attrs.set("dims", Json::make_array());
  attrs.set("shape", int_array(n->outputs[0]->shape));
  n->attrs = attrs;
  return true;
}

// concat(concat(a, b), c) along one axis is concat(a, b, c) when nothing else reads the inner result
static bool flatten_concats(Graph& g, Node* n) {
  if (n->opcode != "concat") return false;
  const long long axis = n->attrs.at("axis").as_int();
  auto uses = g.use_counts();
  std::vector<Value*> flat;
  bool changed = false;
  for (Value* v : n->inputs) {
    Node* p = v->producer;
    if (p && p->opcode == "concat" && p->attrs.at("axis").as_int() == axis && uses[v] == 1 && !g.is_result(v)) {
      flat.insert(flat.end(), p->inputs.begin(), p->inputs.end());
      changed = true;
    } else {
      flat.push_back(v);
    }
  }
  if (changed) n->inputs = flat;
  return changed;
}

static void simplify_linalg(Graph& g, const PassOptions&) {
  using Pattern = bool (*)(Graph&, Node*);
  static const Pattern patterns[] = {compose_transposes, transpose_of_unit_dims, reduce_of_unit_dims, compose_slices,
                                     full_slice,         compose_broadcasts,     view_of_splat,       flatten_concats};
  for (int round = 0; round < 8; ++round) {
    bool changed = false;
    std::vector<Node*> snapshot = g.nodes;
    for (Node* n : snapshot) {
      if (n->dead) continue;
      for (Pattern p : patterns)
        if (p(g, n)) {
          changed = true;
          break;
        }
    }
    g.sweep();
    dce(g);
    if (!changed) break;
  }
}

static void eliminate_uninitialized_copies(Graph& g, const PassOptions&) {
  auto uses = g.use_counts();
  for (Node* n : g.nodes) {
    if (n->dead || n->opcode != "copy") continue;
    Node* p = n->inputs[0]->producer;
    while (p && (p->opcode == "broadcast" || p->opcode == "reshape")) p = p->inputs[0]->producer;
    if (p && (p->opcode == "constant" || p->opcode == "iota") && uses[n->inputs[0]] == 1 &&
        !g.is_result(n->outputs[0]))
      forward(g, n, n->inputs[0]);
  }
  g.sweep();
}

static void eliminate_same_memspace_copy(Graph& g, const PassOptions&) {
  auto uses = g.use_counts();
  for (Node* n : g.nodes) {
    if (n->dead || n->opcode != "copy") continue;
    Value* src = n->inputs[0];
    // a result must keep a buffer of its own when the source is a parameter or another result
    const bool src_owned = src->producer != nullptr && !g.is_result(src);
    if (src_owned && uses[src] == 1) forward(g, n, src);
  }
  g.sweep();
}

static void cse(Graph& g, const PassOptions&) {
  std::map<std::string, Node*> seen;
  for (Node* n : g.nodes) {
    if (n->dead || n->opcode == "custom_call") continue;
    bool collective = n->opcode.rfind("all_", 0) == 0 || n->opcode == "reduce_scatter";
    if (collective) continue;
    std::string key = n->opcode + "(";
    for (Value* v : n->inputs) key += std::to_string(v->id) + ",";
    Json stripped = n->attrs;
    key += ")" + stripped.dump();
    for (Value* o : n->outputs) key += o->type_str();
    auto it = seen.find(key);
    if (it == seen.end()) {
      seen[key] = n;
    } else {
      for (size_t i = 0; i < n->outputs.size(); ++i) g.replace_all_uses(n->outputs[i], it->second->outputs[i]);
      n->dead = true;
    }
  }
  g.sweep();
}

// ---- canonicalize: local rewrites that keep every result value (the one exception, the sign of a zero produced by
// x + 0, is noted at its pattern).  Each pattern returns true when it rewrote `n`.
// A conversion T -> U -> T gives back the input when every T value is exactly representable in U.
static bool widens_losslessly(const std::string& from, const std::string& to) {
  static const std::map<std::string, std::set<std::string>> wider = {
      {"f16", {"f32", "f64"}}, {"bf16", {"f32", "f64"}}, {"f32", {"f64"}},
      {"i8", {"i16", "i32", "i64", "f32", "f64"}}, {"u8", {"i16", "u16", "i32", "u32", "i64", "f16", "f32", "f64"}},
      {"i16", {"i32", "i64", "f32", "f64"}}, {"u16", {"i32", "u32", "i64", "f32", "f64"}}, {"i32", {"i64", "f64"}},
      {"u32", {"i64", "f64"}}, {"pred", {"i8", "u8", "i16", "i32", "i64", "f16", "bf16", "f32", "f64"}}};
  auto it = wider.find(from);
  return it != wider.end() && it->second.count(to) > 0;
}

static bool same_value_operands(const Node* n) { return n->inputs.size() == 2 && n->inputs[0] == n->inputs[1]; }

// x * 1, 1 * x, x + 0, 0 + x, x - 0, x / 1, x ** 1
static bool fold_identity_operand(Graph& g, Node* n) {
  double c;
  const std::string& op = n->opcode;
  if (n->inputs.size() != 2) return false;
  const bool rhs = splat_f64(n->inputs[1], c);
  const double rc = c;
  const bool lhs = splat_f64(n->inputs[0], c);
  const double lc = c;
  // the other operand must already have the result's type and shape: a forward may not change either
  auto fits = [&](Value* v) { return v->dtype == n->outputs[0]->dtype && v->shape == n->outputs[0]->shape; };
  if (op == "mul") {
    if (rhs && rc == 1.0 && fits(n->inputs[0])) return forward(g, n, n->inputs[0]), true;
    if (lhs && lc == 1.0 && fits(n->inputs[1])) return forward(g, n, n->inputs[1]), true;
  } else if (op == "add") {
    // for x = -0 the sum is +0 and the forwarded value -0; every other x is unchanged
    if (rhs && rc == 0.0 && fits(n->inputs[0])) return forward(g, n, n->inputs[0]), true;
    if (lhs && lc == 0.0 && fits(n->inputs[1])) return forward(g, n, n->inputs[1]), true;
  } else if (op == "sub") {
    if (rhs && rc == 0.0 && fits(n->inputs[0])) return forward(g, n, n->inputs[0]), true;
  } else if (op == "div" || op == "pow") {
    if (rhs && rc == 1.0 && fits(n->inputs[0])) return forward(g, n, n->inputs[0]), true;
  }
  return false;
}

// max(x, x), min(x, x), and(x, x), or(x, x), select(c, x, x)
static bool fold_idempotent(Graph& g, Node* n) {
  const std::string& op = n->opcode;
  if ((op == "max" || op == "min" || op == "and" || op == "or") && same_value_operands(n))
    return forward(g, n, n->inputs[0]), true;
  if (op == "select" && n->inputs.size() == 3 && n->inputs[1] == n->inputs[2] &&
      n->inputs[1]->shape == n->outputs[0]->shape)
    return forward(g, n, n->inputs[1]), true;
  return false;
}

// neg(neg(x)), not(not(x)), abs(abs(x)) -> abs(x), abs(neg(x)) -> abs(x)
static bool fold_involution(Graph& g, Node* n) {
  if (n->inputs.size() != 1) return false;
  Node* p = n->inputs[0]->producer;
  if (!p) return false;
  if ((n->opcode == "neg" && p->opcode == "neg") || (n->opcode == "not" && p->opcode == "not"))
    return forward(g, n, p->inputs[0]), true;
  if (n->opcode == "abs" && p->opcode == "abs") return forward(g, n, n->inputs[0]), true;
  if (n->opcode == "abs" && p->opcode == "neg") {
    n->inputs[0] = p->inputs[0];
    return true;
  }
  return false;
}

// convert to the same type; convert(convert(x : T) : U) : T with U holding every T value; convert chains
// T -> U -> V with T -> U lossless collapse to T -> V
static bool fold_convert(Graph& g, Node* n) {
  if (n->opcode != "convert") return false;
  if (n->inputs[0]->dtype == n->outputs[0]->dtype) return forward(g, n, n->inputs[0]), true;
  Node* p = n->inputs[0]->producer;
  if (!p || p->opcode != "convert") return false;
  const std::string& t = p->inputs[0]->dtype;
  const std::string& u = p->outputs[0]->dtype;
  if (!widens_losslessly(t, u)) return false;
  if (t == n->outputs[0]->dtype) return forward(g, n, p->inputs[0]), true;
  n->inputs[0] = p->inputs[0];
  return true;
}

// x / 2^k -> x * 2^-k for f32: both are the correctly rounded value of the same real number
static bool fold_power_of_two_divisor(Graph& g, Node* n) {
  double c;
  if (n->opcode != "div" || n->outputs[0]->dtype != "f32" || !splat_f64(n->inputs[1], c)) return false;
  int e = 0;
  const double m = std::frexp(std::fabs(c), &e);
  if (c == 0.0 || !std::isfinite(c) || m != 0.5 || e < -100 || e > 100) return false;
  Value* r = make_f32_splat(g, n, float(1.0 / c), n->outputs[0]->shape, n->loc);
  n->opcode = "mul";
  n->inputs[1] = r;
  return true;
}

// an elementwise operation whose operands are all splats of f32 scalars is a splat itself
static bool fold_splat_arithmetic(Graph& g, Node* n) {
  if (n->outputs.size() != 1 || n->outputs[0]->dtype != "f32") return false;
  const std::string& op = n->opcode;
  double a, b = 0;
  float r;
  if (n->inputs.size() == 2 && n->inputs[0]->dtype == "f32" && n->inputs[1]->dtype == "f32" &&
      splat_f64(n->inputs[0], a) && splat_f64(n->inputs[1], b)) {
    const float x = float(a), y = float(b);
    if (op == "add") r = x + y;
    else if (op == "sub") r = x - y;
    else if (op == "mul") r = x * y;
    else if (op == "div") r = x / y;
    else if (op == "max") r = std::fmax(x, y);
    else if (op == "min") r = std::fmin(x, y);
    else return false;
    if (std::isnan(x) || std::isnan(y)) return false;          // max / min of NaN differ between libraries
  } else if (n->inputs.size() == 1 && n->inputs[0]->dtype == "f32" && splat_f64(n->inputs[0], a)) {
    const float x = float(a);
    if (op == "neg") r = -x;
    else if (op == "abs") r = std::fabs(x);
    else if (op == "sqrt" && x >= 0) r = std::sqrt(x);          // correctly rounded everywhere
    else return false;
  } else {
    return false;
  }
  Value* v = make_f32_splat(g, n, r, n->outputs[0]->shape, n->loc);
  return forward(g, n, v), true;
}

// broadcast that changes nothing
static bool fold_trivial_broadcast(Graph& g, Node* n) {
  if (n->opcode != "broadcast" || n->inputs[0]->shape != n->outputs[0]->shape) return false;
  return forward(g, n, n->inputs[0]), true;
}

// a constant tensor whose elements are all equal is stored as one scalar and broadcast
static bool fold_splat_storage(Graph& g, Node* n) {
  std::vector<uint8_t> b;
  if (n->opcode != "constant" || n->outputs[0]->shape.empty() || n->outputs[0]->size() < 2 || !constant_bytes(n, b))
    return false;
  const std::string dt = n->outputs[0]->dtype;
  const size_t w = dtype_bytes(dt);
  if (w == 0 || b.size() != size_t(n->outputs[0]->size()) * w) return false;
  for (size_t i = w; i < b.size(); ++i)
    if (b[i] != b[i % w]) return false;
  Json t = Json::make_object();
  t.set("__tensor__", Json::make_str(dt));
  t.set("shape", Json::make_array());
  t.set("data", Json::make_str(b64_encode(std::vector<uint8_t>(b.begin(), b.begin() + long(w)))));
  Json attrs = Json::make_object();
  attrs.set("value", t);
  Node* c = g.insert_node(n, "constant", {}, attrs, {{dt, {}}}, n->loc);
  Json battrs = Json::make_object();
  battrs.set("shape", int_array(n->outputs[0]->shape));
  battrs.set("dims", Json::make_array());
  Node* bc = g.insert_node(n, "broadcast", {c->outputs[0]}, battrs, {{dt, n->outputs[0]->shape}}, n->loc);
  return forward(g, n, bc->outputs[0]), true;
}

static void canonicalize(Graph& g, const PassOptions&) {
  using Pattern = bool (*)(Graph&, Node*);
  static const Pattern patterns[] = {fold_identity_operand, fold_idempotent,           fold_involution,
                                     fold_convert,          fold_power_of_two_divisor, fold_splat_arithmetic,
                                     fold_trivial_broadcast, fold_splat_storage};
  for (int round = 0; round < 8; ++round) {          // rewrites expose one another; graphs settle in two or three
    bool changed = false;
    std::vector<Node*> snapshot = g.nodes;             // patterns insert constants while we walk
    for (Node* n : snapshot) {
      if (n->dead) continue;
      for (Pattern p : patterns)
        if (p(g, n)) {
          changed = true;
          break;
        }
    }
    g.sweep();
    dce(g);
    if (!changed) break;
  }
}

// ---------------------------------------------------------------------------- layout group
struct DotDims { long long b = 1, m = 1, n = 1, k = 1; };
static DotDims dot_dims(const Node* n) {
  DotDims d;
  auto lb = ints(n->attrs.at("lhs_batch")), lc = ints(n->attrs.at("lhs_contract"));
  auto rb = ints(n->attrs.at("rhs_batch")), rc = ints(n->attrs.at("rhs_contract"));
  const auto& a = n->inputs[0]->shape;
  const auto& bshape = n->inputs[1]->shape;
  for (size_t i = 0; i < a.size(); ++i) {
    const bool isb = std::find(lb.begin(), lb.end(), (long long)i) != lb.end();
    const bool isc = std::find(lc.begin(), lc.end(), (long long)i) != lc.end();
    if (isb) d.b *= a[i]; else if (isc) d.k *= a[i]; else d.m *= a[i];
  }
  for (size_t i = 0; i < bshape.size(); ++i) {
    const bool isb = std::find(rb.begin(), rb.end(), (long long)i) != rb.end();
    const bool isc = std::find(rc.begin(), rc.end(), (long long)i) != rc.end();
    if (!isb && !isc) d.n *= bshape[i];
  }
  return d;
}

static long long pick_tn(long long n) {
  for (long long t : {32LL, 64LL, 128LL, 256LL})
    if (n <= t) return t;
  return 256;
}

static void infer_layout(Graph& g, const PassOptions&) {
  auto uses = g.use_counts();
  for (Node* n : g.nodes) {
    // a copy: setting attributes below may move the node's attribute storage
    const Json knob_copy = n->attrs.has("_knob") ? n->attrs.at("_knob") : Json::make_object();
    const Json* knob = n->attrs.has("_knob") ? &knob_copy : nullptr;
    if (n->opcode == "dot") {
      DotDims d = dot_dims(n);
      std::vector<long long> tile = {std::min<long long>(d.m, 128), std::min<long long>(pick_tn(d.n), 256),
                                     std::min<long long>(d.k, 64)};
      if (knob && knob->has("tile_size") && !knob->at("tile_size").is_null()) {
        auto t = ints(knob->at("tile_size"));
        for (size_t i = 0; i < t.size() && i < 2; ++i) tile[i] = t[i];
      }
      if (knob && knob->has("reduction_tile") && !knob->at("reduction_tile").is_null()) {
        auto t = ints(knob->at("reduction_tile"));
        if (!t.empty()) tile[2] = t[0];
      }
      n->attrs.set("_tile", int_array(tile));
      n->attrs.set("_mem", Json::make_str("Tensor"));          // accumulator lives in tensor memory
      n->attrs.set("_operand_mem", Json::make_str("Shared"));
    } else if (is_elementwise(n->opcode)) {
      // elementwise consumers of a dot inherit its output tile (epilogue candidates)
      const Node* src = nullptr;
      for (Value* v : n->inputs)
        if (v->producer && v->producer->attrs.has("_tile") && v->shape == n->outputs[0]->shape) src = v->producer;
      if (src) {
        auto t = ints(src->attrs.at("_tile"));            // [m, n, k] of a dot, or one entry per dimension
        if (t.size() > 2) t.resize(2);
        n->attrs.set("_tile", int_array(t));
        n->attrs.set("_mem", Json::make_str("Register"));
      } else {
        const auto& s = n->outputs[0]->shape;
        std::vector<long long> tile(s.size(), 1);
        if (!s.empty()) tile.back() = std::min<long long>(s.back(), 1024);
        n->attrs.set("_tile", int_array(tile));
        n->attrs.set("_mem", Json::make_str("Global"));
      }
      if (knob && knob->has("mem_space") && !knob->at("mem_space").is_null())
        n->attrs.set("_mem", Json::make_str(knob->at("mem_space").as_string()));
      if (knob && knob->has("tile_size") && !knob->at("tile_size").is_null())
        n->attrs.set("_tile", knob->at("tile_size"));
    } else if (n->opcode == "reduce") {
      auto axes = ints(n->attrs.at("axes"));
      const auto& s = n->inputs[0]->shape;
      std::vector<long long> tile(s.size(), 1);
      for (auto a : axes) tile[size_t(a)] = s[size_t(a)];
      n->attrs.set("_tile", int_array(tile));
      n->attrs.set("_mem", Json::make_str("Global"));
    }
  }
  (void)uses;
}

static bool is_compute(const Node* n) {
  return !is_view_op(n->opcode) && n->opcode != "constant" && n->opcode != "iota";
}

static void assign_linalg_op_ids(Graph& g, const PassOptions&) {
  long long id = 0;
  for (Node* n : g.nodes)
    if (is_compute(n)) n->attrs.set("_op_id", Json::make_int(id++));
}

static void knob_driven_tiling(Graph& g, const PassOptions& o) {
  for (Node* n : g.nodes) {
    if (n->opcode == "dot") {
      DotDims d = dot_dims(n);
      auto tile = n->attrs.has("_tile") ? ints(n->attrs.at("_tile"))
                                        : std::vector<long long>{128, pick_tn(d.n), 64};
      const long long tiles = ((d.m + tile[0] - 1) / tile[0]) * ((d.n + tile[1] - 1) / tile[1]) * d.b;
      long long split = 1;
      if (tiles < o.sm_count * 3 / 4) split = std::max<long long>(1, std::min<long long>({o.sm_count / std::max<long long>(tiles, 1), d.k / 512, 8LL}));
      const long long bytes = (long long)dtype_bytes(n->inputs[0]->dtype);
      const long long stage = (tile[0] + tile[1]) * tile[2] * bytes;
      long long stages = std::max<long long>(2, std::min<long long>(12, (o.smem_capacity - 2048) / std::max<long long>(stage, 1)));
      Json t = Json::make_object();
      t.set("cta_tile", int_array({tile[0], tile[1]}));
      t.set("k_block", Json::make_int(tile[2]));
      t.set("stages", Json::make_int(stages));
      t.set("split_k", Json::make_int(split));
      t.set("grid", Json::make_int(std::min<long long>(tiles * split, o.sm_count)));
      t.set("persistent", Json::make_bool(true));
      n->attrs.set("_tiling", t);
    } else if (is_elementwise(n->opcode) || n->opcode == "reduce") {
      Json t = Json::make_object();
      t.set("block", Json::make_int(256));
      t.set("grid", Json::make_int((n->outputs[0]->size() + 255) / 256));
      n->attrs.set("_tiling", t);
    }
  }
}

static void knob_driven_fusion(Graph& g, const PassOptions&) {
  auto uses = g.use_counts();
  long long group = -1;
  const Node* prev = nullptr;
  for (Node* n : g.nodes) {
    if (is_view_op(n->opcode) || n->opcode == "constant") continue;   // views never break a group
    if (!is_elementwise(n->opcode)) {
      prev = nullptr;
      continue;
    }
    const bool same = prev && prev->outputs[0]->shape == n->outputs[0]->shape;
    if (!same) ++group;
    n->attrs.set("_fuse_group", Json::make_int(group));
    // GEMM epilogue candidate: consumes a dot result that nobody else reads
    for (Value* v : n->inputs)
      if (v->producer && v->producer->opcode == "dot" && uses[v] == 1 && v->producer->attrs.has("_op_id"))
        n->attrs.set("_epilogue_of", v->producer->attrs.at("_op_id"));
    prev = n;
  }
}

static void apply_and_strip_transforms(Graph& g, const PassOptions&) {
  for (Node* n : g.nodes) n->attrs.erase("_knob");
}

static void canonicalize_loop_step(Graph&, const PassOptions&) {}

// ---------------------------------------------------------------------------- memory group
static void annotate_memory_space(Graph& g, const PassOptions&) {
  auto uses = g.use_counts();
  std::map<long long, std::vector<Node*>> groups;
  for (Node* n : g.nodes)
    if (n->attrs.has("_fuse_group")) groups[n->attrs.at("_fuse_group").as_int()].push_back(n);
  for (Node* n : g.nodes) {
    if (n->opcode == "dot") {
      n->attrs.set("_mem", Json::make_str("Tensor"));
      n->attrs.set("_out_mem", Json::make_str("Global"));
      continue;
    }
    if (is_view_op(n->opcode)) {
      n->attrs.set("_mem", Json::make_str("View"));
      continue;
    }
    if (!n->attrs.has("_mem")) n->attrs.set("_mem", Json::make_str("Global"));
  }
  // inside a fusion group only values read outside the group are materialised
  for (auto& kv : groups) {
    std::set<const Node*> members(kv.second.begin(), kv.second.end());
    for (Node* n : kv.second) {
      int inside = 0;
      for (Node* m : kv.second)
        for (Value* v : m->inputs)
          if (v == n->outputs[0]) ++inside;
      const bool escapes = uses[n->outputs[0]] > inside;
      n->attrs.set("_mem", Json::make_str(escapes ? "Global" : "Register"));
    }
  }
}

static void legalize_layout(Graph& g, const PassOptions& o) {
  for (Node* n : g.nodes) {
    if (n->opcode != "dot" || !n->attrs.has("_tile")) continue;
    auto tile = ints(n->attrs.at("_tile"));
    DotDims d = dot_dims(n);
    const long long bytes = (long long)dtype_bytes(n->inputs[0]->dtype);
    // tensor memory: two accumulators of tile_n fp32 columns each
    while (2 * tile[1] > o.tmem_columns && tile[1] > 32) tile[1] /= 2;
    tile[0] = std::min<long long>(tile[0], 128);
    tile[1] = std::min<long long>(tile[1], 256);
    // one 128-byte swizzle row per k-slab
    tile[2] = 128 / bytes;
    const bool tma_ok = (d.k * bytes) % 16 == 0 && (d.n * bytes) % 16 == 0;
    const bool tc = n->inputs[0]->dtype == "bf16" && tma_ok && d.b == 1 && d.k >= 16;
    n->attrs.set("_tile", int_array(tile));
    n->attrs.set("_path", Json::make_str(tc ? "tcgen05" : "simt"));
    if (tc) {
      n->attrs.set("_tma_box_a", int_array({tile[2], tile[0]}));
      n->attrs.set("_tma_box_b", int_array({tile[2], tile[1]}));
      n->attrs.set("_swizzle", Json::make_str("128B"));
    }
  }
}

static void insert_spill_reload(Graph& g, const PassOptions& o) {
  for (Node* n : g.nodes) {
    if (n->opcode != "dot" || !n->attrs.has("_tile")) continue;
    auto tile = ints(n->attrs.at("_tile"));
    const long long bytes = (long long)dtype_bytes(n->inputs[0]->dtype);
    long long stages = n->attrs.has("_tiling") ? n->attrs.at("_tiling").at("stages").as_int() : 4;
    const long long overhead = 2048;
    auto smem = [&] { return stages * (tile[0] + tile[1]) * tile[2] * bytes + overhead; };
    while (smem() > o.smem_capacity && stages > 2) --stages;
    while (smem() > o.smem_capacity && tile[1] > 32) tile[1] /= 2;
    if (smem() > o.smem_capacity)
      throw CompileError("insert-spill-reload: dot tile " + std::to_string(tile[0]) + "x" + std::to_string(tile[1]) +
                         "x" + std::to_string(tile[2]) + " does not fit in " + std::to_string(o.smem_capacity) +
                         " bytes of shared memory even with two stages");
    n->attrs.set("_tile", int_array(tile));
    n->attrs.set("_stages", Json::make_int(stages));
    n->attrs.set("_smem_bytes", Json::make_int(smem()));
    if (n->attrs.has("_tiling")) {
      Json t = n->attrs.at("_tiling");
      t.set("stages", Json::make_int(stages));
      t.set("cta_tile", int_array({tile[0], tile[1]}));
      n->attrs.set("_tiling", t);
    }
  }
}

static void one_shot_bufferize(Graph& g, const PassOptions&) {
  // last use position of every value
  std::map<const Value*, size_t> last;
  for (size_t i = 0; i < g.nodes.size(); ++i)
    for (Value* v : g.nodes[i]->inputs) last[v] = i;
  for (Value* r : g.results) last[r] = g.nodes.size();
  std::map<const Value*, long long> buf;     // value -> buffer id
  std::map<long long, long long> size_of;    // buffer id -> bytes
  std::vector<long long> free_list;
  long long next = 0;
  for (Value* p : g.params) buf[p] = -1;     // caller-owned
  for (size_t i = 0; i < g.nodes.size(); ++i) {
    Node* n = g.nodes[i];
    if (is_view_op(n->opcode)) {
      auto it = buf.find(n->inputs[0]);
      if (it != buf.end()) buf[n->outputs[0]] = it->second;
      n->attrs.set("_buffer", Json::make_int(buf.count(n->outputs[0]) ? buf[n->outputs[0]] : -1));
      continue;
    }
    const bool fused_away = n->attrs.has("_mem") && n->attrs.at("_mem").as_string() == "Register";
    for (Value* o : n->outputs) {
      if (fused_away) {
        buf[o] = -2;   // never materialised
        continue;
      }
      const long long need = o->size() * (long long)dtype_bytes(o->dtype);
      long long chosen = -3;
      // in place: first operand dies here, same byte size, owned by us
      if (is_elementwise(n->opcode) && !n->inputs.empty()) {
        Value* a = n->inputs[0];
        auto it = buf.find(a);
        if (it != buf.end() && it->second >= 0 && last[a] == i && size_of[it->second] == need && !g.is_result(a)) {
          chosen = it->second;
          n->attrs.set("_in_place", Json::make_bool(true));
        }
      }
      if (chosen < 0 && !g.is_result(o)) {
        for (size_t k = 0; k < free_list.size(); ++k)
          if (size_of[free_list[k]] == need) {
            chosen = free_list[k];
            free_list.erase(free_list.begin() + long(k));
            break;
          }
      }
      if (chosen < 0) {
        chosen = next++;
        size_of[chosen] = need;
      }
      buf[o] = chosen;
    }
    n->attrs.set("_buffer", Json::make_int(buf[n->outputs[0]]));
    // release buffers whose every alias died at this node
    std::set<long long> candidates;
    for (Value* v : n->inputs) {
      auto it = buf.find(v);
      if (it != buf.end() && it->second >= 0 && last[v] == i) candidates.insert(it->second);
    }
    for (long long b : candidates) {
      bool alive = false;
      for (auto& kv : buf)
        if (kv.second == b && last.count(kv.first) && last[kv.first] > i) alive = true;
      for (Value* o : n->outputs)
        if (buf[o] == b) alive = true;
      if (!alive && std::find(free_list.begin(), free_list.end(), b) == free_list.end()) free_list.push_back(b);
    }
  }
}

static void insert_memref_dealloc(Graph& g, const PassOptions&) {
  std::map<const Value*, size_t> last;
  for (size_t i = 0; i < g.nodes.size(); ++i)
    for (Value* v : g.nodes[i]->inputs) last[v] = i;
  for (Value* r : g.results) last.erase(r);
  for (Value* p : g.params) last.erase(p);
  for (size_t i = 0; i < g.nodes.size(); ++i) {
    std::vector<long long> ids;
    for (auto& kv : last)
      if (kv.second == i) ids.push_back(kv.first->id);
    std::sort(ids.begin(), ids.end());
    if (!ids.empty()) g.nodes[i]->attrs.set("_last_use_of", int_array(ids));
  }
}

static void inline_nkipy_reference(Graph& g, const PassOptions&) {
  std::vector<Node*> snapshot = g.nodes;
  for (Node* n : snapshot) {
    if (n->opcode != "custom_call" || !n->attrs.has("reference_ir")) continue;
    auto sub = Graph::parse(n->attrs.at("reference_ir").as_string());
    if (sub->params.size() != n->inputs.size() || sub->results.size() != n->outputs.size())
      throw CompileError("inline-nkipy-reference: reference graph arity does not match the custom call");
    std::map<const Value*, Value*> map;
    for (size_t i = 0; i < sub->params.size(); ++i) map[sub->params[i]] = n->inputs[i];
    for (Node* s : sub->nodes) {
      std::vector<Value*> ins;
      for (Value* v : s->inputs) ins.push_back(map.at(v));
      std::vector<std::pair<std::string, std::vector<long long>>> types;
      for (Value* o : s->outputs) types.emplace_back(o->dtype, o->shape);
      Node* c = g.insert_node(n, s->opcode, ins, s->attrs, types, s->loc);
      for (size_t i = 0; i < s->outputs.size(); ++i) map[s->outputs[i]] = c->outputs[i];
    }
    for (size_t i = 0; i < n->outputs.size(); ++i) g.replace_all_uses(n->outputs[i], map.at(sub->results[i]));
    n->dead = true;
  }
  g.sweep();
}

// ---------------------------------------------------------------------------- registry
const std::vector<PassInfo>& default_pipeline() {
  static const std::vector<PassInfo> p = {
      {"remove-redundant-zero-fill", "canonicalize", "drop additions of zero splats", remove_redundant_zero_fill},
      {"prepare-arithmetic", "canonicalize", "strength-reduce pow / constant division", prepare_arithmetic},
      {"decompose-batch-matmul", "canonicalize", "mark batched dots for grid.z batching", decompose_batch_matmul},
      {"canonicalize-partition-dim", "canonicalize", "fold transposed dot operands, record operand majors", canonicalize_partition_dim},
      {"canonicalize-reshape", "canonicalize", "merge reshape chains", canonicalize_reshape},
      {"simplify-linalg", "canonicalize", "compose / remove transposes", simplify_linalg},
      {"eliminate-uninitialized-copies", "canonicalize", "remove copies of created values", eliminate_uninitialized_copies},
      {"eliminate-same-memspace-copy", "canonicalize", "remove copies with a dead source", eliminate_same_memspace_copy},
      {"cse", "canonicalize", "common subexpression elimination", cse},
      {"canonicalize", "canonicalize", "algebraic identities and dead code", canonicalize},
      {"infer-layout", "layout", "tile shapes and placement from dot seeds", infer_layout},
      {"assign-linalg-op-ids", "layout", "stable ids for compute ops", assign_linalg_op_ids},
      {"knob-driven-tiling", "layout", "CTA tile / stages / split-K / grid per op", knob_driven_tiling},
      {"knob-driven-fusion", "layout", "elementwise fusion groups and GEMM epilogues", knob_driven_fusion},
      {"apply-and-strip-transforms", "layout", "consume user knob annotations", apply_and_strip_transforms},
      {"canonicalize-loop-step", "layout", "no work on this target", canonicalize_loop_step},
      {"annotate-memory-space", "memory", "memory space of every value", annotate_memory_space},
      {"legalize-layout", "memory", "TMA / TMEM legality, tcgen05 vs SIMT path", legalize_layout},
      {"insert-spill-reload", "memory", "shared-memory budget: stages / tile shrink", insert_spill_reload},
      {"one-shot-bufferize", "memory", "buffer assignment with reuse", one_shot_bufferize},
      {"insert-memref-dealloc", "memory", "last-use lists", insert_memref_dealloc},
      {"inline-nkipy-reference", "oracle", "inline reference graphs of custom calls", inline_nkipy_reference},
  };
  return p;
}

const PassInfo* find_pass(const std::string& name) {
  for (const PassInfo& p : default_pipeline())
    if (p.name == name) return &p;
  return nullptr;
}

// A `loop` node carries its body as a nested graph (attribute "body", IR text): every pass also runs on
// the bodies, innermost first, so a loop is optimised like straight-line code without being unrolled.
static void run_on_loop_bodies(Graph& g, const PassInfo& p, const PassOptions& opts) {
  for (Node* n : g.nodes) {
    if (n->opcode != "loop" || !n->attrs.has("body")) continue;
    auto body = Graph::parse(n->attrs.at("body").as_string());
    body->verify();
    run_on_loop_bodies(*body, p, opts);
    p.fn(*body, opts);
    body->verify();
    n->attrs.set("body", Json::make_str(body->print()));
  }
}

static void run_one(Graph& g, const PassInfo& p, const PassOptions& opts) {
  if (p.group != "oracle") run_on_loop_bodies(g, p, opts);
  p.fn(g, opts);
  g.verify();
}

void run_pass(Graph& g, const std::string& name, const PassOptions& opts) {
  const PassInfo* p = find_pass(name);
  if (!p) throw CompileError("unknown pass '" + name + "'");
  run_one(g, *p, opts);
}

std::string apply_passes(const std::string& ir_text, const std::vector<std::string>& passes, const PassOptions& opts) {
  auto g = Graph::parse(ir_text);
  g->verify();
  for (const std::string& p : passes) run_pass(*g, p, opts);
  return g->print();
}

std::string run_pipeline(const std::string& ir_text, const std::string& stop_after, const std::string& dump_dir,
                         const PassOptions& opts, int dump_start) {
  const auto& pipe = default_pipeline();
  // resolve stop_after -> index of the last pass to run (inclusive)
  size_t last = pipe.size();
  while (last > 0 && pipe[last - 1].group == "oracle") --last;   // oracle passes run only on request
  if (!stop_after.empty()) {
    bool numeric = std::all_of(stop_after.begin(), stop_after.end(), ::isdigit);
    if (numeric) {
      size_t idx = std::stoul(stop_after);
      if (idx < 1 || idx > pipe.size()) throw CompileError("stop_after index out of range: " + stop_after);
      last = idx;
    } else {
      std::string name = stop_after;
      size_t occurrence = 1;
      size_t colon = stop_after.find(':');
      if (colon != std::string::npos) {
        name = stop_after.substr(0, colon);
        occurrence = std::stoul(stop_after.substr(colon + 1));
      }
      bool found = false;
      size_t seen = 0;
      for (size_t i = 0; i < pipe.size(); ++i) {
        if (pipe[i].name == name && ++seen == occurrence) {
          last = i + 1;
          found = true;
          break;
        }
      }
      if (!found) {
        for (size_t i = 0; i < pipe.size(); ++i)
          if (pipe[i].group == name) {
            last = i + 1;
            found = true;
          }
      }
      if (!found) throw CompileError("stop_after names no pass or group: " + stop_after);
    }
  }
  auto g = Graph::parse(ir_text);
  g->verify();
  for (size_t i = 0; i < last; ++i) {
    run_one(*g, pipe[i], opts);
    if (!dump_dir.empty()) {
      std::ostringstream name;
      name << dump_dir << "/" << std::setw(2) << std::setfill('0') << (dump_start + int(i)) << "_" << pipe[i].name << ".ir";
      std::ofstream out(name.str());
      if (!out) throw CompileError("cannot write " + name.str());
      out << g->print();
    }
  }
  return g->print();
}

}  // namespace b200c
