// Reverse-mode sweep.  Same traversal as the reference (src/core/Autograd.cpp:6-31):
// depth-first post-order over children_, root gradient set to 1.0 everywhere,
// closures run in reverse order — so gradients reaching a shared node are
// accumulated in the same sequence.  The walk uses an explicit stack instead of
// recursion, and leaves with a grad_ready_hook_ are notified as soon as their
// last consumer has run (this is where the data-parallel all-reduce starts).
#include "micrograd/Tensor.h"

#include <unordered_map>
#include <unordered_set>
#include <utility>

namespace micrograd::detail {
namespace {
unsigned long long g_backward_sweep = 0;
}
// Number of backward() calls started so far in this process; a grad-ready hook
// reads it to tell one sweep from the next.
unsigned long long backward_sweep() { return g_backward_sweep; }
}  // namespace micrograd::detail

void Tensor::backward() {
  micrograd::detail::g_backward_sweep++;
  std::vector<Tensor *> ordered;
  std::unordered_set<Tensor *> visited;
  std::vector<std::pair<Tensor *, size_t>> stack;

  visited.insert(this);
  stack.emplace_back(this, 0);
  while (!stack.empty()) {
    auto &[node, next_child] = stack.back();
    if (next_child < node->children_.size()) {
      Tensor *child = node->children_[next_child].get();
      next_child++;
      if (visited.insert(child).second) {
        stack.emplace_back(child, 0);
      }
    } else {
      ordered.push_back(node);
      stack.pop_back();
    }
  }

  // How many closures still have to run before a hooked leaf's gradient is final.
  std::unordered_map<Tensor *, int> pending;
  for (Tensor *node : ordered) {
    if (!node->backward_fn_) {
      continue;
    }
    std::unordered_set<Tensor *> seen;
    for (auto &child : node->children_) {
      if (child->grad_ready_hook_ && seen.insert(child.get()).second) {
        pending[child.get()]++;
      }
    }
  }

  grad_.fill(1.0);

  for (auto it = ordered.rbegin(); it != ordered.rend(); ++it) {
    Tensor *node = *it;
    if (!node->backward_fn_) {
      continue;
    }
    if (node->requires_grad_) {
      node->backward_fn_(*node);
    }
    if (pending.empty()) {
      continue;
    }
    std::unordered_set<Tensor *> seen;
    for (auto &child : node->children_) {
      auto found = pending.find(child.get());
      if (found != pending.end() && seen.insert(child.get()).second) {
        if (--found->second == 0) {
          child->grad_ready_hook_(*child);
        }
      }
    }
  }
}
