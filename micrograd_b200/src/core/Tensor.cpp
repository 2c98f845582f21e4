// Tensor construction, shape bookkeeping and the host-view accessors.
// Counterpart of the reference's src/core/Tensor.cpp; storage is on the device.
#include "micrograd/Tensor.h"

#include <stdexcept>

size_t Tensor::element_count(const std::vector<size_t> &shape) {
  size_t total = 1;
  for (size_t dim : shape) {
    total *= dim;
  }
  return total;
}

// Reference: zero-filled data and grad (Tensor.cpp:7-15).  Here both start as
// "logical zeros": no device memory is touched until a kernel needs it.
Tensor::Tensor(std::vector<size_t> shape) : shape_(std::move(shape)) {
  const size_t total = element_count(shape_);
  data_.init_zero(total);
  grad_.init_zero(total);
  compute_strides();
}

// Reference: copies `data`, rejects a size mismatch (Tensor.cpp:17-28).
Tensor::Tensor(std::vector<size_t> shape, std::vector<double> data) : shape_(std::move(shape)) {
  const size_t total = element_count(shape_);
  if (data.size() != total) {
    throw std::invalid_argument("Tensor and data size mismatch");
  }
  data_.init_from_host(std::move(data));
  grad_.init_zero(total);
  compute_strides();
}

std::shared_ptr<Tensor> Tensor::from_host(std::vector<size_t> shape, const double *values) {
  auto t = std::make_shared<Tensor>(std::move(shape));
  t->data_.init_from_pointer(values, t->data_.size());
  return t;
}

void Tensor::compute_strides() {
  strides_.assign(shape_.size(), 1);
  size_t running = 1;
  for (size_t axis = shape_.size(); axis-- > 0;) {
    strides_[axis] = running;
    running *= shape_[axis];
  }
}

size_t Tensor::flat_index(const std::vector<size_t> &indices) const {
  size_t flat = 0;
  for (size_t axis = 0; axis < indices.size(); axis++) {
    flat += indices[axis] * strides_[axis];
  }
  return flat;
}

const std::vector<size_t> &Tensor::shape() const { return shape_; }

size_t Tensor::size() const { return data_.size(); }

// The mutable accessors lend the host mirror (downloading it first if the device
// copy is newer); the const ones only read it.
double &Tensor::at(const std::vector<size_t> &indices) {
  return data_.host_mutable()[flat_index(indices)];
}

double Tensor::at(const std::vector<size_t> &indices) const {
  return data_.host_const()[flat_index(indices)];
}

double &Tensor::grad_at(const std::vector<size_t> &indices) {
  return grad_.host_mutable()[flat_index(indices)];
}

double Tensor::grad_at(const std::vector<size_t> &indices) const {
  return grad_.host_const()[flat_index(indices)];
}

std::vector<double> &Tensor::data() { return data_.host_mutable(); }

std::vector<double> &Tensor::grad() { return grad_.host_mutable(); }

void Tensor::copy_from_host(const double *values) { data_.upload_in_place(values); }

void Tensor::prefetch_from_host(const double *values) { data_.prefetch_in_place(values); }

const std::vector<double> &Tensor::data() const { return data_.host_const(); }

const std::vector<double> &Tensor::grad() const { return grad_.host_const(); }

// Reference: loop writing 0.0 (Tensor.cpp:73-77).  Here the gradient returns to
// the logical-zero state, so the next accumulation is a plain store.
void Tensor::zero_grad() { grad_.set_zero(); }

// Storage is always in device memory; the tag is recorded so that backend()
// reports what the caller asked for (the reference's to() is a no-op off Apple
// hardware, Tensor.cpp:124-126).
void Tensor::to(micrograd::Backend b) { backend_ = b; }

micrograd::Backend Tensor::backend() const { return backend_; }

void Tensor::set_requires_grad(bool flag) { requires_grad_ = flag; }

bool Tensor::requires_grad() const { return requires_grad_; }

std::shared_ptr<Tensor> Tensor::make_result(std::vector<size_t> shape, std::string label,
                                            std::vector<std::shared_ptr<Tensor>> children) {
  auto result = std::make_shared<Tensor>(std::move(shape));
  result->op_ = std::move(label);
  bool needs = false;
  for (const auto &c : children) {
    needs = needs || c->requires_grad_;
  }
  result->requires_grad_ = needs;
  result->children_ = std::move(children);
  return result;
}
