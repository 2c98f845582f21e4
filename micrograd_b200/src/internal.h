#pragma once
// Private to the library: the one friend of Tensor outside the class, through
// which nn.cpp and mnist.cpp reach storage and graph fields.
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "micrograd/Tensor.h"

namespace micrograd::detail {
unsigned long long backward_sweep();  // Autograd.cpp: backward() calls started so far

struct TensorAccess {
  static Storage &data(Tensor &t) { return t.data_; }
  static Storage &grad(Tensor &t) { return t.grad_; }
  static std::vector<std::shared_ptr<Tensor>> &children(Tensor &t) { return t.children_; }
  static std::function<void(Tensor &)> &backward_fn(Tensor &t) { return t.backward_fn_; }
  static std::function<void(Tensor &)> &hook(Tensor &t) { return t.grad_ready_hook_; }
  static bool requires_grad(const Tensor &t) { return t.requires_grad_; }
  static void mark_relu_output(Tensor &t) { t.relu_output_ = true; }
  static bool is_relu_output(const Tensor &t) { return t.relu_output_; }
  // True if the gradient buffer holds only values that already carry the ReLU
  // mask (or nothing at all).
  static bool grad_fully_masked(Tensor &t) {
    return t.grad_.is_zero() || (t.grad_premasked_ && t.grad_.device_current() &&
                                 t.grad_.write_stamp() == t.grad_premasked_stamp_);
  }
  static void commit_premask(Tensor &t, bool fully_masked) {
    t.grad_premasked_ = fully_masked;
    t.grad_premasked_stamp_ = t.grad_.write_stamp();
  }
  static std::shared_ptr<Tensor> make_result(Tensor &owner, std::vector<size_t> shape,
                                             std::string label,
                                             std::vector<std::shared_ptr<Tensor>> children) {
    return owner.make_result(std::move(shape), std::move(label), std::move(children));
  }
};
}  // namespace micrograd::detail

