// Elementwise arithmetic: tensor (x) tensor, tensor (x) scalar and pow.
// Counterpart of the reference's src/ops/Arithmetic.cpp.  Each op checks shapes
// with the reference's exception texts, enqueues one forward kernel, and records
// a closure that enqueues one fused accumulate kernel per backward call.
#include <stdexcept>

#include "mg_cuda.h"
#include "micrograd/Tensor.h"
#include "micrograd/Utils.h"

using micrograd::detail::check;

std::shared_ptr<Tensor> Tensor::binary_op(int op, const char *label,
                                          const std::shared_ptr<Tensor> &b) {
  if (shape_ != b->shape_) {
    throw std::invalid_argument("Tensor shapes do not match");
  }
  auto result = make_result(shape_, label, {shared_from_this(), b});
  check(mg_binary_fwd(op, data_.device_read(), b->data_.device_read(),
                      result->data_.device_overwrite(), size()),
        label);
  result->data_.mirror_async();  // one-element results only

  result->backward_fn_ = [op](Tensor &self) {
    if (self.grad_.is_zero()) {
      return;  // an all-zero upstream gradient contributes nothing
    }
    Tensor &lhs = *self.children_[0];
    Tensor &rhs = *self.children_[1];
    const bool needs_values = (op == MG_MUL || op == MG_DIV);
    const double *g = self.grad_.device_read();
    const double *a = needs_values ? lhs.data_.device_read() : nullptr;
    const double *bv = needs_values ? rhs.data_.device_read() : nullptr;
    double *ga = nullptr, *gb = nullptr;
    int flags = 0;
    bool store = false;
    if (lhs.requires_grad_) {
      ga = lhs.grad_.device_accumulate(&store);
      if (store) flags |= MG_ACC_STORE_A;
    }
    if (rhs.requires_grad_) {
      if (&rhs == &lhs) {
        gb = ga;  // x (op) x: both updates land in one buffer, in order
      } else {
        gb = rhs.grad_.device_accumulate(&store);
        if (store) flags |= MG_ACC_STORE_B;
      }
    }
    check(mg_binary_bwd(op, a, bv, g, ga, gb, self.size(), flags), "binary backward");
  };
  return result;
}

std::shared_ptr<Tensor> Tensor::add(const std::shared_ptr<Tensor> &b) {
  // Addition: a row vector on the right broadcasts over the rows of a matrix.
  if (shape_ != b->shape_ && shape_.size() == 2 && shape_[0] > 1 &&
      ((b->shape_.size() == 2 && b->shape_[0] == 1 && b->shape_[1] == shape_[1]) ||
       (b->shape_.size() == 1 && b->shape_[0] == shape_[1]))) {
    return add_row(b);
  }
  return binary_op(MG_ADD, "+", b);
}

std::shared_ptr<Tensor> Tensor::sub(const std::shared_ptr<Tensor> &b) {
  return binary_op(MG_SUB, "-", b);
}

std::shared_ptr<Tensor> Tensor::mul(const std::shared_ptr<Tensor> &b) {
  return binary_op(MG_MUL, "*", b);
}

std::shared_ptr<Tensor> Tensor::div(const std::shared_ptr<Tensor> &b) {
  return binary_op(MG_DIV, "/", b);
}

std::shared_ptr<Tensor> Tensor::add_row(const std::shared_ptr<Tensor> &row) {
  const size_t rows = shape_[0], cols = shape_[1];
  auto result = make_result(shape_, "+row", {shared_from_this(), row});
  check(mg_add_row_fwd(data_.device_read(), row->data_.device_read(),
                       result->data_.device_overwrite(), rows, cols),
        "row broadcast add");
  result->backward_fn_ = [rows, cols](Tensor &self) {
    if (self.grad_.is_zero()) {
      return;
    }
    Tensor &x = *self.children_[0];
    Tensor &r = *self.children_[1];
    const double *g = self.grad_.device_read();
    double *gx = nullptr, *gr = nullptr;
    int flags = 0;
    bool store = false;
    if (x.requires_grad_) {
      gx = x.grad_.device_accumulate(&store);
      if (store) flags |= MG_ACC_STORE_A;
    }
    if (r.requires_grad_) {
      gr = r.grad_.device_accumulate(&store);
      if (store) flags |= MG_ACC_STORE_B;
    }
    check(mg_add_row_bwd(g, gx, gr, rows, cols, flags), "row broadcast add backward");
  };
  return result;
}

// One input, optional scalar: scalar add/sub/mul/div, pow, and the activations.
std::shared_ptr<Tensor> Tensor::unary_op(int op, std::string label, double scalar) {
  auto result = make_result(shape_, std::move(label), {shared_from_this()});
  check(mg_unary_fwd(op, data_.device_read(), scalar, result->data_.device_overwrite(), size()),
        "unary forward");
  result->data_.mirror_async();  // one-element results only (e.g. the mean of mse_loss)
  result->backward_fn_ = [op, scalar](Tensor &self) {
    Tensor &x = *self.children_[0];
    if (self.grad_.is_zero() || !x.requires_grad_) {
      return;
    }
    const bool needs_input = (op == MG_POW || op == MG_RELU);
    const bool needs_output = (op == MG_SIGMOID || op == MG_TANH || op == MG_EXP);
    const double *g = self.grad_.device_read();
    const double *a = needs_input ? x.data_.device_read() : nullptr;
    const double *y = needs_output ? self.data_.device_read() : nullptr;
    bool store = false;
    double *gx = x.grad_.device_accumulate(&store);
    check(mg_unary_bwd(op, a, y, scalar, g, gx, self.size(), store ? MG_ACC_STORE_A : 0),
          "unary backward");
  };
  return result;
}

std::shared_ptr<Tensor> Tensor::add(double scalar) {
  return unary_op(MG_SADD, format_scalar("+", scalar), scalar);
}

std::shared_ptr<Tensor> Tensor::sub(double scalar) {
  return unary_op(MG_SSUB, format_scalar("-", scalar), scalar);
}

std::shared_ptr<Tensor> Tensor::mul(double scalar) {
  return unary_op(MG_SMUL, format_scalar("*", scalar), scalar);
}

std::shared_ptr<Tensor> Tensor::div(double scalar) {
  return unary_op(MG_SDIV, format_scalar("/", scalar), scalar);
}

std::shared_ptr<Tensor> Tensor::pow(double exponent) {
  return unary_op(MG_POW, format_scalar("^", exponent), exponent);
}
