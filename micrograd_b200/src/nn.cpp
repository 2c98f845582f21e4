// Layers, losses and the optimiser (reference: src/nn.cpp), built on the device
// ops.  Linear::forward is a single GEMM with the bias (and optionally ReLU)
// fused into its epilogue, for any batch size; SGD::step is one kernel; the
// additions are softmax cross-entropy, row argmax and the data-parallel
// gradient all-reduce.
#include "micrograd/nn.h"

#include <fstream>
#include <random>
#include <stdexcept>
#include <string>

#include "internal.h"
#include "mg_cuda.h"

using micrograd::detail::check;
using micrograd::detail::DeviceInts;

using micrograd::detail::Storage;

using Access = micrograd::detail::TensorAccess;

// mean((prediction - target)^2), composed from the generic ops exactly as the
// reference composes it (nn.cpp:6-15).
std::shared_ptr<Tensor> mse_loss(const std::shared_ptr<Tensor> &prediction,
                                 const std::shared_ptr<Tensor> &target) {
  auto squared = prediction->sub(target)->pow(2.0);
  return squared->sum()->div(static_cast<double>(prediction->size()));
}

// 28x28 -> 14x14 mean pooling of image row vectors, on the device; like the
// reference (nn.cpp:17-35) it returns a fresh leaf, i.e. it is not
// differentiable.  The reference handles one [1,784] image; any [B,784] batch is
// accepted here (the reference reads row 0 only, which is what B = 1 gives).
std::shared_ptr<Tensor> avg_pool_2x2(const std::shared_ptr<Tensor> &input) {
  const auto &shape = input->shape();
  size_t batch = 1;
  if (shape.size() == 2 && shape[1] == 784) {
    batch = shape[0];
  } else if (input->size() < 784) {
    throw std::invalid_argument("avg_pool_2x2 needs 784 values per image");
  }
  auto pooled = std::make_shared<Tensor>(std::vector<size_t>{batch, 196});
  check(mg_avg_pool_28(Access::data(*input).device_read(), Access::data(*pooled).device_overwrite(),
                       batch),
        "avg_pool_2x2");
  return pooled;
}

// Weights [in, out] ~ U(-0.1, 0.1) from a non-deterministic seed, bias [1, out]
// zero — the reference's initialisation (nn.cpp:37-53).
Linear::Linear(size_t in_features, size_t out_features) {
  std::random_device entropy;
  std::mt19937 engine(entropy());
  std::uniform_real_distribution<> uniform(-0.1, 0.1);
  std::vector<double> w(in_features * out_features);
  for (double &v : w) {
    v = uniform(engine);
  }
  weights_ = std::make_shared<Tensor>(std::vector<size_t>{in_features, out_features}, std::move(w));
  bias_ = std::make_shared<Tensor>(std::vector<size_t>{1, out_features},
                                   std::vector<double>(out_features, 0.0));
}

std::shared_ptr<Tensor> Linear::weights() { return weights_; }
std::shared_ptr<Tensor> Linear::bias() { return bias_; }

// input.matmul(W).add(b) of the reference (nn.cpp:55-57) as one node.
std::shared_ptr<Tensor> Linear::forward(const std::shared_ptr<Tensor> &input) {
  return fused_forward(input, false);
}

std::shared_ptr<Tensor> Linear::forward_relu(const std::shared_ptr<Tensor> &input) {
  return fused_forward(input, true);
}

std::shared_ptr<Tensor> Linear::fused_forward(const std::shared_ptr<Tensor> &input, bool relu) {
  const auto &xs = input->shape();
  const auto &ws = weights_->shape();
  if (xs.size() != 2) {
    throw std::invalid_argument("Tensors must be 2D for matmul");
  }
  if (xs[1] != ws[0]) {
    throw std::invalid_argument("Inner dimensions must match for matmul");
  }
  const size_t batch = xs[0], in = ws[0], out = ws[1];
  auto result = Access::make_result(*input, {batch, out}, relu ? "linear+relu" : "linear",
                                    {input, weights_, bias_});
  check(mg_gemm_nn(Access::data(*input).device_read(), Access::data(*weights_).device_read(),
                   Access::data(*result).device_overwrite(), batch, out, in, 0,
                   relu ? MG_EPI_BIAS_RELU : MG_EPI_BIAS, Access::data(*bias_).device_read()),
        "linear forward");

  if (relu) {
    Access::mark_relu_output(*result);
  }

  Access::backward_fn(*result) = [batch, in, out, relu](Tensor &self) {
    if (Access::grad(self).is_zero()) {
      return;
    }
    auto &kids = Access::children(self);
    Tensor &x = *kids[0];
    Tensor &w = *kids[1];
    Tensor &b = *kids[2];
    // An upstream GEMM may already have applied this node's ReLU mask while
    // writing the gradient (see the dX product below).
    const bool premasked = relu && !Access::grad(self).is_zero() && Access::grad_fully_masked(self);
    const double *g = Access::grad(self).device_read();
    double *masked = nullptr;
    if (relu && !premasked) {
      // dZ = dOut * (out > 0); out > 0 exactly where the pre-activation was.
      check(mg_alloc(batch * out, &masked), "device allocation");
      check(mg_unary_bwd(MG_RELU, Access::data(self).device_read(), nullptr, 0.0, g, masked,
                         batch * out, MG_ACC_STORE_A),
            "relu mask");
      g = masked;
    }
    bool store = false;
    if (Access::requires_grad(w)) {
      double *gw = Access::grad(w).device_accumulate(&store);
      check(mg_gemm_tn(Access::data(x).device_read(), g, gw, batch, out, in, store ? 0 : 1),
            "linear dW");
    }
    if (Access::requires_grad(b)) {
      double *gb = Access::grad(b).device_accumulate(&store);
      check(mg_add_row_bwd(g, nullptr, gb, batch, out, store ? MG_ACC_STORE_B : 0), "linear db");
    }
    if (Access::requires_grad(x)) {
      // If the input is itself the output of a linear+ReLU node, its backward
      // would multiply this gradient by (x > 0) in a separate pass over the
      // whole activation; the GEMM epilogue does it for free.
      const bool mask_input = Access::is_relu_output(x);
      const bool stays_masked = mask_input && Access::grad_fully_masked(x);
      double *gx = Access::grad(x).device_accumulate(&store);
      check(mg_gemm_nt(g, Access::data(w).device_read(), gx, batch, out, in, store ? 0 : 1,
                       mask_input ? MG_EPI_RELU_MASK : MG_EPI_NONE,
                       mask_input ? Access::data(x).device_read() : nullptr),
            "linear dX");
      if (mask_input) {
        Access::commit_premask(x, stays_masked);
      }
    }
    if (masked) {
      check(mg_free(masked), "free");
    }
  };
  return result;
}

// ---------------------------------------------------------------------------
// SGD
// ---------------------------------------------------------------------------
SGD::SGD(std::vector<std::shared_ptr<Tensor>> parameters, double learning_rate)
    : parameters_(std::move(parameters)), learning_rate_(learning_rate) {}

SGD::~SGD() {
  for (auto &p : parameters_) {
    Access::hook(*p) = nullptr;
  }
}

void SGD::zero_grad() {
  if (allreduce_ && buckets_.any_reduced()) {
    // An exchange may still be writing the gradient buffer: order the next
    // writer (the first accumulation of the coming sweep) behind it.
    check(mg_comm_join(), "comm join");
  }
  for (auto &p : parameters_) {
    Access::grad(*p).set_exchange_pending(false);
    p->zero_grad();
  }
  buckets_.end_step();
}

// p -= lr * g elementwise (nn.cpp:71-77), on the device.  A parameter whose
// gradient is still logically zero is left alone (p - lr*0 == p).
void SGD::step() {
  if (allreduce_) {
    // A bounded wait that ran out in an earlier exchange (a rank that never
    // joined) leaves a fault code; the copy read here was made behind the
    // previous step's exchange, so no device synchronisation is needed.  Applying
    // unreduced gradients would let the ranks drift apart silently.
    int fault = 0;
    check(mg_kernel_status_peek(&fault), "kernel status");
    if (fault != 0) {
      mg_check_kernel_status();  // synchronises, clears the word, records the message
      throw std::runtime_error(std::string("SGD::step: gradient exchange failed: ") + mg_last_error());
    }
    // Buckets the backward sweep did not complete (a parameter outside the graph,
    // or halves finished in different sweeps) are exchanged now: every rank takes
    // the same decision, and no rank applies a local-only gradient.
    for (size_t b : buckets_.unreduced()) {
      reduce_bucket(b);
    }
    check(mg_comm_join(), "comm join");
    check(mg_kernel_status_mirror(), "kernel status");
    for (auto &p : parameters_) {
      Access::grad(*p).set_exchange_pending(false);
    }
  }
  bool flat = flat_data_ != nullptr;
  if (flat) {
    for (auto &p : parameters_) {
      flat = flat && Access::grad(*p).device_current() && Access::data(*p).device_current();
    }
  }
  if (flat) {
    // Every parameter and gradient is current in the flat buffers: one launch.
    for (auto &p : parameters_) {
      Access::data(*p).device_update();
    }
    check(mg_sgd_step(flat_data_, flat_grad_, learning_rate_, flat_elems_), "sgd step");
  } else {
    // One launch per eight parameter tensors.
    std::vector<double *> params;
    std::vector<const double *> grads;
    std::vector<size_t> sizes;
    for (auto &p : parameters_) {
      if (Access::grad(*p).is_zero()) {
        continue;
      }
      params.push_back(Access::data(*p).device_update());
      grads.push_back(Access::grad(*p).device_read());
      sizes.push_back(p->size());
    }
    check(mg_sgd_step_multi(params.data(), grads.data(), sizes.data(), static_cast<int>(params.size()),
                            learning_rate_),
          "sgd step");
  }
  buckets_.end_step();
}

namespace {
struct FlatBuffers {
  double *data = nullptr;
  double *grad = nullptr;
  bool grad_shared = false;  // grad came from mg_comm_alloc_shared
  ~FlatBuffers() {
    mg_free(data);
    if (grad_shared) {
      mg_comm_free_shared(grad);
    } else {
      mg_free(grad);
    }
  }
};
}  // namespace

void SGD::enable_allreduce() {
  if (flat_data_) {
    return;
  }
  // Slices start on 256-byte boundaries so every kernel takes its vector path.
  constexpr size_t kAlign = 32;
  offsets_.clear();
  size_t total = 0;
  for (auto &p : parameters_) {
    offsets_.push_back(total);
    total += (p->size() + kAlign - 1) / kAlign * kAlign;
  }
  flat_elems_ = total;
  auto flat = std::make_shared<FlatBuffers>();
  check(mg_alloc(total, &flat->data), "device allocation");
  check(mg_fill(flat->data, 0.0, total), "fill");
  if (micrograd::comm_world() > 1) {
    // Gradients of a multi-rank job live in a buffer every rank maps, so the
    // exchange can run over peer memory (all ranks reach this call together).
    check(mg_comm_alloc_shared(total, &flat->grad), "shared gradient buffer");
    flat->grad_shared = true;
  } else {
    check(mg_alloc(total, &flat->grad), "device allocation");
    check(mg_fill(flat->grad, 0.0, total), "fill");
  }
  flat_data_ = flat->data;
  flat_grad_ = flat->grad;
  for (size_t i = 0; i < parameters_.size(); i++) {
    Tensor &p = *parameters_[i];
    Access::data(p).rehome(flat_data_ + offsets_[i], flat);
    Access::grad(p).rehome(flat_grad_ + offsets_[i], flat);
    Access::hook(p) = [this, i](Tensor &) { on_grad_ready(i); };
  }
  std::vector<std::vector<size_t>> shapes;
  for (auto &p : parameters_) {
    shapes.push_back(p->shape());
  }
  buckets_.plan(shapes, offsets_, requires_flags(), flat_elems_);
  allreduce_ = micrograd::comm_world() > 1;
}

std::vector<char> SGD::requires_flags() const {
  std::vector<char> flags;
  for (auto &p : parameters_) {
    flags.push_back(p->requires_grad() ? 1 : 0);
  }
  return flags;
}

// Called from backward() when parameter `index` has received its last
// contribution of the sweep.  A bucket is exchanged on the communication stream
// as soon as all its members that require a gradient are final.
void SGD::on_grad_ready(size_t index) {
  if (!allreduce_) {
    return;
  }
  const unsigned long long sweep = micrograd::detail::backward_sweep();
  if (buckets_.is_new_sweep(sweep)) {
    buckets_.begin_sweep(sweep, requires_flags());
  }
  const long bucket = buckets_.on_ready(index);
  if (bucket >= 0) {
    reduce_bucket(static_cast<size_t>(bucket));
  }
}

void SGD::reduce_bucket(size_t bucket) {
  const auto &b = buckets_.buckets()[bucket];
  for (size_t i = b.first; i <= b.last; i++) {
    Storage &g = Access::grad(*parameters_[i]);
    g.device_update();  // logical zeros become real zeros
    g.set_exchange_pending(true);
  }
  // The bucket that completes the set has nothing left to hide behind: step() is
  // about to wait for it, so it may use most of the GPU.
  const bool last_one = buckets_.unreduced().size() == 1;
  check(mg_allreduce_sum_async_hint(flat_grad_ + b.begin, b.end - b.begin, last_one ? 1 : 0),
        "gradient all-reduce");
  buckets_.mark_reduced(bucket);
}

// ---------------------------------------------------------------------------
// Model files: raw fp64 W1, b1, W2, b2, no header (nn.cpp:79-125).
// ---------------------------------------------------------------------------
void save_model(const std::string &path, Linear &l1, Linear &l2) {
  std::ofstream file(path, std::ios::binary);
  if (!file.is_open()) {
    throw std::runtime_error("Could not open file for saving: " + path);
  }
  for (auto t : {l1.weights(), l1.bias(), l2.weights(), l2.bias()}) {
    const auto &values = t->data();
    file.write(reinterpret_cast<const char *>(values.data()),
               static_cast<std::streamsize>(values.size() * sizeof(double)));
  }
}

void load_model(const std::string &path, Linear &l1, Linear &l2) {
  std::ifstream file(path, std::ios::binary);
  if (!file.is_open()) {
    throw std::runtime_error("Could not open file for loading: " + path);
  }
  for (auto t : {l1.weights(), l1.bias(), l2.weights(), l2.bias()}) {
    auto &values = t->data();
    file.read(reinterpret_cast<char *>(values.data()),
              static_cast<std::streamsize>(values.size() * sizeof(double)));
  }
}

// ---------------------------------------------------------------------------
// Additions: softmax cross-entropy and argmax
// ---------------------------------------------------------------------------
static std::shared_ptr<Tensor> xent_node(const std::shared_ptr<Tensor> &logits,
                                         std::shared_ptr<DeviceInts> ids, double denom) {
  const auto &shape = logits->shape();
  const size_t rows = shape[0], classes = shape[1];
  if (denom <= 0.0) {
    denom = static_cast<double>(rows);
  }
  auto result = Access::make_result(*logits, {1}, "softmax_xent", {logits});
  check(mg_softmax_xent_fwd(Access::data(*logits).device_read(), ids->get(),
                            Access::data(*result).device_overwrite(), rows, classes, denom),
        "softmax cross-entropy");
  Access::data(*result).mirror_async();
  Access::backward_fn(*result) = [ids, rows, classes, denom](Tensor &self) {
    Tensor &z = *Access::children(self)[0];
    if (Access::grad(self).is_zero() || !Access::requires_grad(z)) {
      return;
    }
    bool store = false;
    const double *gl = Access::grad(self).device_read();
    double *gz = Access::grad(z).device_accumulate(&store);
    check(mg_softmax_xent_bwd(Access::data(z).device_read(), ids->get(), gl, gz, rows, classes,
                              denom, store ? MG_ACC_STORE_A : 0),
          "softmax cross-entropy backward");
  };
  return result;
}

static void check_logits(const std::shared_ptr<Tensor> &logits, size_t label_count) {
  if (logits->shape().size() != 2) {
    throw std::invalid_argument("softmax_cross_entropy needs 2D logits");
  }
  if (label_count != logits->shape()[0]) {
    throw std::invalid_argument("softmax_cross_entropy: one label per row expected");
  }
}

std::shared_ptr<Tensor> softmax_cross_entropy(const std::shared_ptr<Tensor> &logits,
                                              const std::shared_ptr<Tensor> &labels, double denom) {
  check_logits(logits, labels->size());
  auto ids = std::make_shared<DeviceInts>(labels->size());
  check(mg_f64_to_i32(Access::data(*labels).device_read(), ids->get(), labels->size()),
        "label conversion");
  return xent_node(logits, std::move(ids), denom);
}

std::shared_ptr<Tensor> softmax_cross_entropy(const std::shared_ptr<Tensor> &logits,
                                              const std::vector<int> &labels, double denom) {
  check_logits(logits, labels.size());
  auto ids = std::make_shared<DeviceInts>(labels.data(), labels.size());
  return xent_node(logits, std::move(ids), denom);
}

std::vector<int> argmax_rows(const std::shared_ptr<Tensor> &x) {
  if (x->shape().size() != 2) {
    throw std::invalid_argument("argmax_rows needs a 2D tensor");
  }
  const size_t rows = x->shape()[0], cols = x->shape()[1];
  std::vector<int> out(rows);
  if (rows == 0) {
    return out;
  }
  if (cols == 0) {
    throw std::invalid_argument("argmax_rows: rows are empty");
  }
  DeviceInts ids(rows);
  check(mg_argmax_rows(Access::data(*x).device_read(), ids.get(), rows, cols), "argmax");
  check(mg_download_i32(out.data(), ids.get(), rows), "download");
  return out;
}
