#pragma once
// MNIST IDX reader.  load_mnist() has the reference's signature and result type
// (include/micrograd/mnist.h:9-15): one [1,784] image tensor (pixels / 255) and
// one one-hot [1,10] label tensor per sample.  Here the whole data set is
// uploaded to the GPU in two copies and the per-sample tensors are views into
// those buffers.

#include <memory>
#include <string>
#include <vector>

#include "Tensor.h"

struct MNISTData {
  std::vector<std::shared_ptr<Tensor>> images;
  std::vector<std::shared_ptr<Tensor>> labels;
};

MNISTData load_mnist(const std::string &images_path, const std::string &labels_path,
                     int sample_count);

// addition: the same files as two batched tensors, images [N,784] and class ids
// [N] (stored as doubles), the form Linear::forward and softmax_cross_entropy take.
struct MNISTBatch {
  std::shared_ptr<Tensor> images;
  std::shared_ptr<Tensor> labels;
};

MNISTBatch load_mnist_batched(const std::string &images_path, const std::string &labels_path,
                              int sample_count);
