#pragma once
// Layers, loss and optimiser on top of Tensor.  The first part mirrors the
// reference's include/micrograd/nn.h:6-34; the marked additions are what batched
// softmax-cross-entropy training and inference on the GPU need.

#include <memory>
#include <string>
#include <vector>

#include "Tensor.h"
#include "detail/GradBuckets.h"

std::shared_ptr<Tensor> mse_loss(const std::shared_ptr<Tensor> &prediction,
                                 const std::shared_ptr<Tensor> &target);
std::shared_ptr<Tensor> avg_pool_2x2(const std::shared_ptr<Tensor> &input);

class Linear {
public:
  Linear(size_t in_features, size_t out_features);
  // input [B, in] -> [B, out] for any batch size B: one GEMM with the bias add
  // fused into its epilogue.
  std::shared_ptr<Tensor> forward(const std::shared_ptr<Tensor> &input);
  std::shared_ptr<Tensor> weights();
  std::shared_ptr<Tensor> bias();

  // addition: relu(forward(input)) as a single node (bias + ReLU epilogue).
  // When the node feeding gradient into it is another Linear, that layer's dX
  // GEMM applies this node's ReLU mask in its epilogue; grad() of the returned
  // tensor then holds the gradient with respect to the pre-activation.
  std::shared_ptr<Tensor> forward_relu(const std::shared_ptr<Tensor> &input);

private:
  std::shared_ptr<Tensor> fused_forward(const std::shared_ptr<Tensor> &input, bool relu);
  std::shared_ptr<Tensor> weights_;
  std::shared_ptr<Tensor> bias_;
};

class SGD {
public:
  SGD(std::vector<std::shared_ptr<Tensor>> parameters, double learning_rate);
  ~SGD();

  void step();
  void zero_grad();

  // addition: moves all parameters and their gradients into two flat device
  // buffers and, when a communicator is up (micrograd::comm_init), sums each
  // parameter's gradient across ranks as soon as backward() has finished it.
  // step() then waits for those sums on the device, not on the host.
  // Parameters travel in one message per layer: a weight directly followed by
  // its bias forms a pair, anything else goes alone.  A parameter that the
  // backward sweep never reaches is reduced by step() itself, and a second
  // backward() before step() throws std::logic_error once sums have been
  // exchanged (they cannot be accumulated into).
  void enable_allreduce();

private:
  void on_grad_ready(size_t index);
  std::vector<std::shared_ptr<Tensor>> parameters_;
  double learning_rate_;
  // flat storage (after enable_allreduce)
  double *flat_data_ = nullptr;
  double *flat_grad_ = nullptr;
  std::vector<size_t> offsets_;
  micrograd::detail::GradBuckets buckets_;
  void reduce_bucket(size_t bucket);
  std::vector<char> requires_flags() const;
  size_t flat_elems_ = 0;
  bool allreduce_ = false;
};

void save_model(const std::string &path, Linear &l1, Linear &l2);
void load_model(const std::string &path, Linear &l1, Linear &l2);

// ---- additions ------------------------------------------------------------
// Mean softmax cross-entropy of logits [B, C] against class ids.  `labels` is a
// tensor of B class ids stored as doubles (shape [B] or [B,1]) or a host vector.
// `denom` overrides the divisor of the mean (0 = B); a rank holding a shard of a
// global batch passes the global batch size.
std::shared_ptr<Tensor> softmax_cross_entropy(const std::shared_ptr<Tensor> &logits,
                                              const std::shared_ptr<Tensor> &labels,
                                              double denom = 0.0);
std::shared_ptr<Tensor> softmax_cross_entropy(const std::shared_ptr<Tensor> &logits,
                                              const std::vector<int> &labels, double denom = 0.0);
// Index of the first strict maximum of each row of a 2-D tensor.
std::vector<int> argmax_rows(const std::shared_ptr<Tensor> &x);
