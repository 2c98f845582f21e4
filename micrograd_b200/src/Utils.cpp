// Graphviz dump and scalar-op labels (reference: src/Utils.cpp).  Only element 0
// of each tensor's data and gradient is fetched from the device.
#include "micrograd/Utils.h"

#include <iomanip>
#include <sstream>
#include <unordered_set>
#include <vector>

std::string to_dot(const std::shared_ptr<Tensor> &tensor) {
  std::ostringstream out;
  out << "digraph {\n  rankdir=LR;\n";

  std::unordered_set<Tensor *> seen;
  std::vector<Tensor *> work{tensor.get()};
  // Depth-first, children in order, like the reference's recursive walk.
  while (!work.empty()) {
    Tensor *node = work.back();
    work.pop_back();
    if (!seen.insert(node).second) {
      continue;
    }
    out << "  \"" << node << "\" [label=\"data: " << node->data_.peek(0);
    if (node->size() > 1) {
      out << "...";
    }
    out << " | grad: " << node->grad_.peek(0);
    if (node->size() > 1) {
      out << "...";
    }
    out << "\", shape=record];\n";
    if (node->op_.empty()) {
      continue;
    }
    out << "  \"" << node << "_op\" [label=\"" << node->op_ << "\"];\n";
    out << "  \"" << node << "_op\" -> \"" << node << "\";\n";
    for (auto &child : node->children_) {
      out << "  \"" << child.get() << "\" -> \"" << node << "_op\";\n";
    }
    for (auto it = node->children_.rbegin(); it != node->children_.rend(); ++it) {
      work.push_back(it->get());
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
