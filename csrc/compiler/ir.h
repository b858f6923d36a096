// Tensor IR of the native compiler: the same textual form the Python frontend prints
// (nkipy_b200/core/ir.py), parsed into an in-memory SSA graph that passes rewrite.
//
// This library stands where the reference has an MLIR dialect plus passes
// (nkigen/mlir/include/nkipy/Dialect/NkipyOps.td, nkigen/mlir/lib/Transforms/*.cpp): a typed
// tensor IR with annotation attributes (tile, memory space, op id, fusion group), a fixed,
// inspectable pass pipeline, and a text-in / text-out driver — self-contained C++ with no
// LLVM dependency.  Pass-added annotations live in node attributes whose key starts with
// an underscore; the frontend ignores the ones it does not know.
#pragma once
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "../runtime/json.h"

namespace b200c {

using spike::Json;

struct Node;

struct Value {
  int id = -1;
  std::string dtype;             // "f32", "bf16", "pred", ...
  std::vector<long long> shape;
  std::string name;              // parameters only
  Node* producer = nullptr;      // null for parameters
  int index = 0;

  long long size() const {
    long long n = 1;
    for (auto d : shape) n *= d;
    return n;
  }
  std::string type_str() const;
};

struct Node {
  std::string opcode;
  std::vector<Value*> inputs;
  Json attrs = Json::make_object();
  std::vector<Value*> outputs;
  std::string loc;               // "file:line" or empty
  bool dead = false;
};

struct Alias {
  int output_index, param_index, user_returned;
};

class CompileError : public std::runtime_error {
 public:
  explicit CompileError(const std::string& m) : std::runtime_error(m) {}
};

class Graph {
 public:
  std::string name = "kernel";
  std::vector<Value*> params;
  std::vector<Node*> nodes;
  std::vector<Value*> results;
  std::vector<std::string> result_names;
  std::vector<Alias> aliases;

  Graph() = default;
  Graph(const Graph&) = delete;
  Graph& operator=(const Graph&) = delete;

  static std::unique_ptr<Graph> parse(const std::string& text);
  std::string print(bool with_locations = true) const;
  void verify() const;

  Value* new_value(const std::string& dtype, const std::vector<long long>& shape);
  // creates a node with explicitly typed results, inserted before `before` (or appended)
  Node* insert_node(Node* before, const std::string& opcode, const std::vector<Value*>& inputs, const Json& attrs,
                    const std::vector<std::pair<std::string, std::vector<long long>>>& result_types,
                    const std::string& loc = "");
  void replace_all_uses(Value* from, Value* to);
  std::map<const Value*, int> use_counts() const;
  void sweep();                  // drop nodes marked dead
  bool is_result(const Value* v) const;

 private:
  std::vector<std::unique_ptr<Value>> value_store_;
  std::vector<std::unique_ptr<Node>> node_store_;
  int next_id_ = 0;
};

bool is_elementwise(const std::string& opcode);
bool is_view_op(const std::string& opcode);
size_t dtype_bytes(const std::string& dtype);

}  // namespace b200c
