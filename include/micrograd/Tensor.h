#pragma once
// class Tensor — micrograd's public tensor/autograd interface, backed by B200
// device memory.
//
// The public section reproduces the reference's interface
// (include/micrograd/Tensor.h:15-50) signature for signature, so code written
// against the reference — including its test suite — compiles and runs
// unchanged.  Everything below `private:` is different: values and gradients
// are fp64 buffers in GPU memory (detail::Storage), ops enqueue CUDA kernels
// through the C ABI of include/mg_cuda.h and return immediately, and the host
// only waits inside data()/grad()/at()/grad_at().
//
// Additions that the reference does not have are grouped at the end of the
// public section.

#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "micrograd/Backend.h"
#include "micrograd/detail/Storage.h"

namespace micrograd::detail {
struct TensorAccess;
}

class Tensor : public std::enable_shared_from_this<Tensor> {
  friend std::string to_dot(const std::shared_ptr<Tensor> &tensor);
  friend struct micrograd::detail::TensorAccess;

public:
  // ---- reference interface ------------------------------------------------
  Tensor(std::vector<size_t> shape);
  Tensor(std::vector<size_t> shape, std::vector<double> data);
  ~Tensor() = default;

  std::shared_ptr<Tensor> add(const std::shared_ptr<Tensor> &b);
  std::shared_ptr<Tensor> sub(const std::shared_ptr<Tensor> &b);
  std::shared_ptr<Tensor> mul(const std::shared_ptr<Tensor> &b);
  std::shared_ptr<Tensor> div(const std::shared_ptr<Tensor> &b);

  std::shared_ptr<Tensor> add(double scalar);
  std::shared_ptr<Tensor> sub(double scalar);
  std::shared_ptr<Tensor> mul(double scalar);
  std::shared_ptr<Tensor> div(double scalar);
  std::shared_ptr<Tensor> pow(double exponent);

  std::shared_ptr<Tensor> sum();
  std::shared_ptr<Tensor> matmul(const std::shared_ptr<Tensor> &b);

  std::shared_ptr<Tensor> relu();
  std::shared_ptr<Tensor> sigmoid();
  std::shared_ptr<Tensor> tanh();

  void backward();
  void zero_grad();

  const std::vector<size_t> &shape() const;
  size_t size() const;
  double &at(const std::vector<size_t> &indices);
  double at(const std::vector<size_t> &indices) const;
  double &grad_at(const std::vector<size_t> &indices);
  double grad_at(const std::vector<size_t> &indices) const;
  std::vector<double> &data();
  std::vector<double> &grad();
  void to(micrograd::Backend backend);
  micrograd::Backend backend() const;

  // ---- additions of the B200 backend --------------------------------------
  // add(b) also accepts a row vector b of shape [1,N] or [N] against [M,N]
  // (M > 1), broadcasting it over the rows; the reference throws for that case.
  std::shared_ptr<Tensor> exp();
  // Sum over one axis (0, 1 or -1) of a 2-D tensor.
  std::shared_ptr<Tensor> sum(int axis);
  // A tensor that does not require a gradient is skipped by backward(): no
  // gradient buffer is allocated for it and the product that would fill it is
  // not computed.  Defaults to true, the reference's behaviour.
  void set_requires_grad(bool flag);
  bool requires_grad() const;
  // Uploads straight from caller memory (pinned or pageable) without the
  // intermediate std::vector the reference constructor takes by value.
  static std::shared_ptr<Tensor> from_host(std::vector<size_t> shape, const double *values);
  // Overwrites the values with size() doubles from caller memory, keeping the
  // device buffer (and its address) the tensor already has: how the input of a
  // recorded step is refreshed.
  void copy_from_host(const double *values);
  // The same, but the copy runs on the library's copy stream: it starts when the
  // kernels enqueued so far have finished (they may still read the old values),
  // overlaps whatever is enqueued afterwards, and the next operation that uses
  // this tensor waits for it.  With two input tensors refreshed in turn, the batch
  // of step i+1 uploads while step i computes and nothing is allocated per step.
  // `values` must stay unchanged until that next use has completed (pinned memory
  // for a copy that really overlaps).  Not for the input of a recorded step.
  void prefetch_from_host(const double *values);
  // Read-only host views.  Unlike the mutable data()/grad() of the reference
  // interface they do not hand out a writable reference, so the device copy stays
  // current and no re-upload follows the read.
  const std::vector<double> &data() const;
  const std::vector<double> &grad() const;

private:
  // Shared bodies of the public ops (op codes are those of mg_cuda.h).
  std::shared_ptr<Tensor> binary_op(int op, const char *label, const std::shared_ptr<Tensor> &b);
  std::shared_ptr<Tensor> unary_op(int op, std::string label, double scalar);
  std::shared_ptr<Tensor> add_row(const std::shared_ptr<Tensor> &row);
  std::shared_ptr<Tensor> make_result(std::vector<size_t> shape, std::string label,
                                      std::vector<std::shared_ptr<Tensor>> children);
  void compute_strides();
  size_t flat_index(const std::vector<size_t> &indices) const;
  static size_t element_count(const std::vector<size_t> &shape);

  mutable micrograd::detail::Storage data_;
  mutable micrograd::detail::Storage grad_;
  std::vector<size_t> shape_;
  std::vector<size_t> strides_;

  // Graph.  A node's closure receives the node itself and reaches its operands
  // through children_, so it owns nothing and the graph has no reference cycle.
  std::vector<std::shared_ptr<Tensor>> children_;
  std::function<void(Tensor &)> backward_fn_;
  // Called by backward() on a leaf once its gradient is final for this sweep.
  std::function<void(Tensor &)> grad_ready_hook_;

  std::string op_;
  micrograd::Backend backend_ = micrograd::Backend::CPU;
  bool requires_grad_ = true;

  // Set on the output of a fused linear+ReLU node.  A consumer that writes this
  // node's gradient with a GEMM applies the ReLU mask in that GEMM's epilogue
  // and records the gradient's write stamp; if nothing else has written the
  // gradient since, the node's own backward skips its mask pass.
  bool relu_output_ = false;
  bool grad_premasked_ = false;
  unsigned long long grad_premasked_stamp_ = 0;
};
