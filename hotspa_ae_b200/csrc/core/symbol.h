// Lazily evaluated integer expressions ("symbolic shapes"): leaves hold a value that can be re-set
// between runs, inner nodes are + - * / % of two symbols, so one traced graph serves every
// (batch, sequence-length) without rebuilding.  Reference counterpart: hetu/core/symbol.h.
#pragma once
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>

namespace hsb {

class IntSymbol {
 public:
  enum Op { LEAF, ADD, SUB, MUL, DIV, REM };
  IntSymbol() : node_(std::make_shared<Node>()) {}
  explicit IntSymbol(int64_t v) : node_(std::make_shared<Node>()) { node_->value = v; node_->has_value = true; }
  static IntSymbol make(Op op, const IntSymbol& a, const IntSymbol& b) {
    IntSymbol s;
    s.node_->op = op;
    s.node_->lhs = a.node_;
    s.node_->rhs = b.node_;
    return s;
  }
  bool is_leaf() const { return node_->op == LEAF; }
  bool is_instantiated() const { return node_->op != LEAF || node_->has_value; }
  void set(int64_t v) {
    if (!is_leaf()) throw std::runtime_error("IntSymbol: only leaf symbols can be assigned");
    node_->value = v;
    node_->has_value = true;
  }
  int64_t get() const { return eval(node_.get()); }
  bool same(const IntSymbol& o) const { return node_ == o.node_; }
  std::string repr() const { return repr(node_.get()); }

 private:
  struct Node {
    Op op = LEAF;
    int64_t value = 0;
    bool has_value = false;
    std::shared_ptr<Node> lhs, rhs;
  };
  static int64_t eval(const Node* n) {
    if (n->op == LEAF) {
      if (!n->has_value) throw std::runtime_error("IntSymbol: leaf symbol has no value yet");
      return n->value;
    }
    const int64_t a = eval(n->lhs.get()), b = eval(n->rhs.get());
    switch (n->op) {
      case ADD: return a + b;
      case SUB: return a - b;
      case MUL: return a * b;
      case DIV: if (b == 0) throw std::runtime_error("IntSymbol: division by zero"); return a / b;
      case REM: if (b == 0) throw std::runtime_error("IntSymbol: modulo by zero"); return a % b;
      default: return 0;
    }
  }
  static std::string repr(const Node* n) {
    if (n->op == LEAF) return n->has_value ? std::to_string(n->value) : std::string("?");
    static const char* names[] = {"", "+", "-", "*", "/", "%"};
    return "(" + repr(n->lhs.get()) + names[n->op] + repr(n->rhs.get()) + ")";
  }
  std::shared_ptr<Node> node_;
};

}  // namespace hsb
