// Graphviz dump and scalar-op labels (reference: src/Utils.cpp).  Only element 0
// of each tensor's data and gradient is fetched from the device.
#include "micrograd/Utils.h"

#include <iomanip>
#include <sstream>
#include <unordered_set>
#include <utility>
#include <vector>

std::string to_dot(const std::shared_ptr<Tensor> &tensor) {
  std::ostringstream out;
  out << "digraph {\n";
  out << "  rankdir=LR;\n";

  // Same text, line for line, as the reference's recursive walk: a node, its op
  // box, then per child the edge followed by that child's subtree.  Done with
  // an explicit stack of (node, next child) frames.
  std::unordered_set<Tensor *> seen;
  auto emit_node = [&](Tensor *node) {
    out << "  \"" << node << "\" [label=\"data: " << node->data_.peek(0);
    if (node->size() > 1) {
      out << "...";
    }
    out << " | grad: " << node->grad_.peek(0);
    if (node->size() > 1) {
      out << "...";
    }
    out << "\", shape=record];\n";
    if (!node->op_.empty()) {
      out << "  \"" << node << "_op\" [label=\"" << node->op_ << "\"];\n";
      out << "  \"" << node << "_op\" -> \"" << node << "\";\n";
    }
  };
  std::vector<std::pair<Tensor *, size_t>> stack;
  seen.insert(tensor.get());
  emit_node(tensor.get());
  stack.emplace_back(tensor.get(), 0);
  while (!stack.empty()) {
    Tensor *node = stack.back().first;
    size_t &next = stack.back().second;
    if (node->op_.empty() || next >= node->children_.size()) {
      stack.pop_back();
      continue;
    }
    Tensor *child = node->children_[next].get();
    next++;
    out << "  \"" << child << "\" -> \"" << node << "_op\";\n";
    if (seen.insert(child).second) {
      emit_node(child);
      stack.emplace_back(child, 0);
    }
  }
  out << "}\n";
  return out.str();
}

std::string format_scalar(const std::string &op, double scalar) {
  std::ostringstream label;
  label << op << ' ' << std::fixed << std::setprecision(2) << scalar;
  return label.str();
}
