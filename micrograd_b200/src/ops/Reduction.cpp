// sum() over all elements (reference: src/ops/Reduction.cpp) and, as an
// addition, the sum over the last axis of a matrix.
#include <stdexcept>

#include "mg_cuda.h"
#include "micrograd/Tensor.h"

using micrograd::detail::check;

std::shared_ptr<Tensor> Tensor::sum() {
  auto result = make_result({1}, "sum", {shared_from_this()});
  check(mg_sum_all_fwd(data_.device_read(), result->data_.device_overwrite(), size()), "sum");
  result->data_.mirror_async();

  // The upstream scalar is read on the device; it never visits the host.
  result->backward_fn_ = [](Tensor &self) {
    Tensor &x = *self.children_[0];
    if (self.grad_.is_zero() || !x.requires_grad_) {
      return;
    }
    const double *g = self.grad_.device_read();
    bool store = false;
    double *gx = x.grad_.device_accumulate(&store);
    check(mg_sum_all_bwd(g, gx, x.size(), store ? MG_ACC_STORE_A : 0), "sum backward");
  };
  return result;
}

std::shared_ptr<Tensor> Tensor::sum(int axis) {
  if (shape_.size() != 2) {
    throw std::invalid_argument("sum(axis) needs a 2D tensor");
  }
  if (axis != 0 && axis != 1 && axis != -1) {
    throw std::invalid_argument("sum(axis): axis must be 0, 1 or -1 for a 2D tensor");
  }
  const size_t rows = shape_[0], cols = shape_[1];
  if (axis == 0) {
    // Column sums [M,N] -> [N]: the same two-stage reduction as a bias gradient.
    auto result = make_result({cols}, "sum axis=0", {shared_from_this()});
    check(mg_add_row_bwd(data_.device_read(), nullptr, result->data_.device_overwrite(), rows, cols,
                         MG_ACC_STORE_B),
          "sum(axis=0)");
    result->backward_fn_ = [rows, cols](Tensor &self) {
      Tensor &x = *self.children_[0];
      if (self.grad_.is_zero() || !x.requires_grad_) {
        return;
      }
      const double *g = self.grad_.device_read();
      double *gx = x.grad_.device_update();  // logical zeros become real zeros first
      check(mg_add_row_fwd(gx, g, gx, rows, cols), "sum(axis=0) backward");  // gx[i,j] += g[j]
    };
    return result;
  }
  auto result = make_result({rows}, "sum axis=-1", {shared_from_this()});
  check(mg_sum_lastaxis_fwd(data_.device_read(), result->data_.device_overwrite(), rows, cols),
        "sum(axis)");
  result->backward_fn_ = [rows, cols](Tensor &self) {
    Tensor &x = *self.children_[0];
    if (self.grad_.is_zero() || !x.requires_grad_) {
      return;
    }
    const double *g = self.grad_.device_read();
    bool store = false;
    double *gx = x.grad_.device_accumulate(&store);
    check(mg_sum_lastaxis_bwd(g, gx, rows, cols, store ? MG_ACC_STORE_A : 0),
          "sum(axis) backward");
  };
  return result;
}
