#include "ir.h"

#include <regex>
#include <sstream>

namespace b200c {

static const std::set<std::string> kElementwise = {
    "add", "sub", "mul", "div", "pow", "max", "min", "rem", "atan2", "and", "or", "xor", "abs", "neg", "exp", "log",
    "sqrt", "rsqrt", "sin", "cos", "tanh", "ceil", "floor", "sign", "not", "round_even", "is_finite", "erf",
    "compare", "select", "convert"};
static const std::set<std::string> kViews = {"reshape", "transpose", "slice", "broadcast"};

bool is_elementwise(const std::string& op) { return kElementwise.count(op) != 0; }
bool is_view_op(const std::string& op) { return kViews.count(op) != 0; }

size_t dtype_bytes(const std::string& d) {
  static const std::map<std::string, size_t> w = {{"pred", 1}, {"i8", 1}, {"u8", 1}, {"f8e5m2", 1}, {"f8e4m3", 1},
                                                  {"i16", 2},  {"u16", 2}, {"f16", 2}, {"bf16", 2},  {"i32", 4},
                                                  {"u32", 4},  {"f32", 4}, {"i64", 8}, {"u64", 8},   {"f64", 8}};
  auto it = w.find(d);
  if (it == w.end()) throw CompileError("unknown dtype '" + d + "'");
  return it->second;
}

std::string Value::type_str() const {
  std::string s = dtype + "[";
  for (size_t i = 0; i < shape.size(); ++i) s += (i ? "," : "") + std::to_string(shape[i]);
  return s + "]";
}

Value* Graph::new_value(const std::string& dtype, const std::vector<long long>& shape) {
  auto v = std::make_unique<Value>();
  v->id = next_id_++;
  v->dtype = dtype;
  v->shape = shape;
  value_store_.push_back(std::move(v));
  return value_store_.back().get();
}

Node* Graph::insert_node(Node* before, const std::string& opcode, const std::vector<Value*>& inputs, const Json& attrs,
                         const std::vector<std::pair<std::string, std::vector<long long>>>& result_types,
                         const std::string& loc) {
  auto n = std::make_unique<Node>();
  n->opcode = opcode;
  n->inputs = inputs;
  n->attrs = attrs.type == Json::Object ? attrs : Json::make_object();
  n->loc = loc;
  for (size_t i = 0; i < result_types.size(); ++i) {
    Value* v = new_value(result_types[i].first, result_types[i].second);
    v->producer = n.get();
    v->index = static_cast<int>(i);
    n->outputs.push_back(v);
  }
  Node* raw = n.get();
  node_store_.push_back(std::move(n));
  if (before) {
    auto it = std::find(nodes.begin(), nodes.end(), before);
    nodes.insert(it, raw);
  } else {
    nodes.push_back(raw);
  }
  return raw;
}

void Graph::replace_all_uses(Value* from, Value* to) {
  for (Node* n : nodes)
    for (auto& in : n->inputs)
      if (in == from) in = to;
  for (auto& r : results)
    if (r == from) r = to;
}

std::map<const Value*, int> Graph::use_counts() const {
  std::map<const Value*, int> c;
  for (const Node* n : nodes)
    if (!n->dead)
      for (const Value* v : n->inputs) c[v]++;
  for (const Value* v : results) c[v]++;
  return c;
}

bool Graph::is_result(const Value* v) const { return std::find(results.begin(), results.end(), v) != results.end(); }

void Graph::sweep() {
  nodes.erase(std::remove_if(nodes.begin(), nodes.end(), [](Node* n) { return n->dead; }), nodes.end());
}

static std::vector<std::pair<std::string, std::vector<long long>>> parse_types(const std::string& s) {
  std::vector<std::pair<std::string, std::vector<long long>>> out;
  static const std::regex re(R"((\w+)\[([\d,]*)\])");
  for (auto it = std::sregex_iterator(s.begin(), s.end(), re); it != std::sregex_iterator(); ++it) {
    std::vector<long long> shape;
    std::stringstream ss((*it)[2].str());
    std::string tok;
    while (std::getline(ss, tok, ','))
      if (!tok.empty()) shape.push_back(std::stoll(tok));
    out.emplace_back((*it)[1].str(), shape);
  }
  return out;
}

static std::vector<int> parse_ids(const std::string& s) {
  std::vector<int> ids;
  static const std::regex re(R"(%(\d+))");
  for (auto it = std::sregex_iterator(s.begin(), s.end(), re); it != std::sregex_iterator(); ++it)
    ids.push_back(std::stoi((*it)[1].str()));
  return ids;
}

// position of the '}' closing the JSON object that starts at `open` (strings respected)
static size_t match_brace(const std::string& s, size_t open) {
  int depth = 0;
  bool in_str = false;
  for (size_t i = open; i < s.size(); ++i) {
    char c = s[i];
    if (in_str) {
      if (c == '\\') ++i;
      else if (c == '"') in_str = false;
      continue;
    }
    if (c == '"') in_str = true;
    else if (c == '{') ++depth;
    else if (c == '}' && --depth == 0) return i;
  }
  throw CompileError("unbalanced braces in IR line: " + s);
}

std::unique_ptr<Graph> Graph::parse(const std::string& text) {
  auto g = std::make_unique<Graph>();
  std::map<int, Value*> values;
  std::istringstream in(text);
  std::string line;
  bool started = false;
  while (std::getline(in, line)) {
    size_t b = line.find_first_not_of(" \t");
    if (b == std::string::npos) continue;
    std::string t = line.substr(b);
    if (t.rfind("graph", 0) == 0) {
      size_t at = t.find('@');
      size_t sp = t.find_first_of(" {", at);
      g->name = t.substr(at + 1, sp - at - 1);
      started = true;
      continue;
    }
    if (!started) throw CompileError("IR text does not start with 'graph @name {'");
    if (t == "}") continue;
    if (t.rfind("return", 0) == 0) {
      size_t pos = 6;
      while (true) {
        size_t pct = t.find('%', pos);
        if (pct == std::string::npos) break;
        size_t end = pct + 1;
        while (end < t.size() && isdigit(t[end])) ++end;
        int id = std::stoi(t.substr(pct + 1, end - pct - 1));
        size_t open = t.find('{', end);
        size_t close = match_brace(t, open);
        Json meta = Json::parse(t.substr(open, close - open + 1));
        if (!values.count(id)) throw CompileError("return of undefined value %" + std::to_string(id));
        g->results.push_back(values[id]);
        g->result_names.push_back(meta.at("name").as_string());
        pos = close + 1;
      }
      continue;
    }
    if (t.rfind("alias", 0) == 0) {
      std::istringstream ss(t.substr(5));
      Alias a{};
      ss >> a.output_index >> a.param_index >> a.user_returned;
      g->aliases.push_back(a);
      continue;
    }
    size_t eq = t.find('=');
    size_t lp = t.find('(', eq);
    size_t rp = t.find(')', lp);
    if (eq == std::string::npos || lp == std::string::npos || rp == std::string::npos)
      throw CompileError("cannot parse IR line: " + t);
    std::vector<int> out_ids = parse_ids(t.substr(0, eq));
    std::string opcode = t.substr(eq + 1, lp - eq - 1);
    opcode.erase(0, opcode.find_first_not_of(' '));
    opcode.erase(opcode.find_last_not_of(' ') + 1);
    std::vector<int> in_ids = parse_ids(t.substr(lp + 1, rp - lp - 1));
    size_t open = t.find('{', rp);
    size_t close = match_brace(t, open);
    Json attrs = Json::parse(t.substr(open, close - open + 1));
    size_t colon = t.find(':', close);
    std::string rest = t.substr(colon + 1);
    std::string loc;
    size_t cm = rest.find("//");
    if (cm != std::string::npos) {
      loc = rest.substr(cm + 2);
      loc.erase(0, loc.find_first_not_of(' '));
      rest = rest.substr(0, cm);
    }
    auto types = parse_types(rest);
    if (types.size() != out_ids.size()) throw CompileError("result count mismatch in IR line: " + t);
    if (opcode == "param") {
      auto v = std::make_unique<Value>();
      v->id = out_ids[0];
      v->dtype = types[0].first;
      v->shape = types[0].second;
      v->name = attrs.has("name") ? attrs.at("name").as_string() : "";
      g->next_id_ = std::max(g->next_id_, v->id + 1);
      values[v->id] = v.get();
      g->params.push_back(v.get());
      g->value_store_.push_back(std::move(v));
      continue;
    }
    auto n = std::make_unique<Node>();
    n->opcode = opcode;
    n->attrs = attrs;
    n->loc = loc;
    for (int id : in_ids) {
      if (!values.count(id)) throw CompileError("use of undefined value %" + std::to_string(id) + " in: " + t);
      n->inputs.push_back(values[id]);
    }
    for (size_t i = 0; i < out_ids.size(); ++i) {
      auto v = std::make_unique<Value>();
      v->id = out_ids[i];
      v->dtype = types[i].first;
      v->shape = types[i].second;
      v->producer = n.get();
      v->index = static_cast<int>(i);
      g->next_id_ = std::max(g->next_id_, v->id + 1);
      values[v->id] = v.get();
      n->outputs.push_back(v.get());
      g->value_store_.push_back(std::move(v));
    }
    g->nodes.push_back(n.get());
    g->node_store_.push_back(std::move(n));
  }
  if (!started) throw CompileError("empty IR text");
  return g;
}

std::string Graph::print(bool with_locations) const {
  std::ostringstream os;
  os << "graph @" << name << " {\n";
  for (const Value* p : params) {
    Json a = Json::make_object();
    a.set("name", Json::make_str(p->name));
    os << "  %" << p->id << " = param() " << a.dump() << " : " << p->type_str() << "\n";
  }
  for (const Node* n : nodes) {
    if (n->dead) continue;
    os << "  ";
    for (size_t i = 0; i < n->outputs.size(); ++i) os << (i ? ", " : "") << "%" << n->outputs[i]->id;
    os << " = " << n->opcode << "(";
    for (size_t i = 0; i < n->inputs.size(); ++i) os << (i ? ", " : "") << "%" << n->inputs[i]->id;
    os << ") " << n->attrs.dump() << " : ";
    for (size_t i = 0; i < n->outputs.size(); ++i) os << (i ? ", " : "") << n->outputs[i]->type_str();
    if (with_locations && !n->loc.empty()) os << "  // " << n->loc;
    os << "\n";
  }
  os << "  return ";
  for (size_t i = 0; i < results.size(); ++i) {
    Json a = Json::make_object();
    a.set("name", Json::make_str(result_names[i]));
    os << (i ? ", " : "") << "%" << results[i]->id << " " << a.dump();
  }
  os << "\n";
  for (const Alias& a : aliases) os << "  alias " << a.output_index << " " << a.param_index << " " << a.user_returned << "\n";
  os << "}\n";
  return os.str();
}

void Graph::verify() const {
  std::set<const Value*> defined(params.begin(), params.end());
  for (const Node* n : nodes) {
    if (n->dead) continue;
    for (const Value* v : n->inputs)
      if (!defined.count(v)) throw CompileError("verify: %" + std::to_string(v->id) + " used before definition by " + n->opcode);
    if (is_elementwise(n->opcode) && n->opcode != "select" && n->opcode != "convert" && n->inputs.size() == 2 &&
        n->inputs[0]->shape != n->inputs[1]->shape)
      throw CompileError("verify: elementwise '" + n->opcode + "' operands differ in shape");
    for (const Value* v : n->outputs) defined.insert(v);
  }
  for (const Value* v : results)
    if (!defined.count(v)) throw CompileError("verify: result %" + std::to_string(v->id) + " is not defined");
  for (const Alias& a : aliases)
    if (a.output_index < 0 || a.output_index >= int(results.size()) || a.param_index < 0 ||
        a.param_index >= int(params.size()))
      throw CompileError("verify: alias index out of range");
}

}  // namespace b200c
