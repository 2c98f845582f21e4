// 2-D matrix product and its two gradient products (reference:
// src/ops/Matmul.cpp).  Forward C = A.B; backward dA += G.B^T, then dB += A^T.G,
// in that order, each one GEMM on the FP64 tensor cores.
#include <stdexcept>

#include "mg_cuda.h"
#include "micrograd/Tensor.h"

using micrograd::detail::check;

std::shared_ptr<Tensor> Tensor::matmul(const std::shared_ptr<Tensor> &b) {
  if (shape_.size() != 2 || b->shape_.size() != 2) {
    throw std::invalid_argument("Tensors must be 2D for matmul");
  }
  if (shape_[1] != b->shape_[0]) {
    throw std::invalid_argument("Inner dimensions must match for matmul");
  }
  const size_t m = shape_[0], k = shape_[1], n = b->shape_[1];

  auto result = make_result({m, n}, "@", {shared_from_this(), b});
  check(mg_gemm_nn(data_.device_read(), b->data_.device_read(), result->data_.device_overwrite(), m,
                   n, k, 0, MG_EPI_NONE, nullptr),
        "matmul");

  result->backward_fn_ = [m, k, n](Tensor &self) {
    if (self.grad_.is_zero()) {
      return;
    }
    Tensor &lhs = *self.children_[0];
    Tensor &rhs = *self.children_[1];
    const double *g = self.grad_.device_read();
    bool store = false;
    if (lhs.requires_grad_) {
      const double *bv = rhs.data_.device_read();
      double *ga = lhs.grad_.device_accumulate(&store);
      check(mg_gemm_nt(g, bv, ga, m, n, k, store ? 0 : 1, MG_EPI_NONE, nullptr), "matmul dA");
    }
    if (rhs.requires_grad_) {
      const double *av = lhs.data_.device_read();
      double *gb = rhs.grad_.device_accumulate(&store);
      check(mg_gemm_tn(av, g, gb, m, n, k, store ? 0 : 1), "matmul dB");
    }
  };
  return result;
}
