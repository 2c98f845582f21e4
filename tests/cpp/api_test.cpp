// C++-level tests of the drop-in Tensor API on the B200 backend, in the style of
// the reference's test/tensor_test.cpp (which itself is compiled unchanged
// against this backend as a separate binary).  Needs a GPU.
#include <gtest/gtest.h>

#include <cmath>
#include <cstdio>
#include <fstream>
#include <memory>
#include <stdexcept>
#include <utility>
#include <vector>

#include "mg_cuda.h"
#include "micrograd/Tensor.h"
#include "micrograd/Utils.h"
#include "micrograd/mnist.h"
#include "micrograd/nn.h"

using TensorPtr = std::shared_ptr<Tensor>;

static TensorPtr make(std::vector<size_t> shape, std::vector<double> values) {
  return std::make_shared<Tensor>(std::move(shape), std::move(values));
}

// README example of the reference (README.md:27-53).
TEST(ApiTest, ReadmeExample) {
  auto a = make({2, 2}, {1, 2, 3, 4});
  auto b = make({2, 2}, {5, 6, 7, 8});
  auto c = a->matmul(b);
  auto loss = c->sum();
  loss->backward();
  const std::vector<double> want_c{19, 22, 43, 50}, want_a{11, 15, 11, 15}, want_b{4, 4, 6, 6};
  for (size_t i = 0; i < 4; i++) {
    EXPECT_NEAR(c->data()[i], want_c[i], 1e-12);
    EXPECT_NEAR(a->grad()[i], want_a[i], 1e-12);
    EXPECT_NEAR(b->grad()[i], want_b[i], 1e-12);
  }
}

TEST(ApiTest, ExceptionsMatchReference) {
  auto a = std::make_shared<Tensor>(std::vector<size_t>{2, 3});
  auto b = std::make_shared<Tensor>(std::vector<size_t>{3, 2});
  EXPECT_THROW(a->add(b), std::invalid_argument);
  EXPECT_THROW(a->matmul(a), std::invalid_argument);
  EXPECT_THROW(std::make_shared<Tensor>(std::vector<size_t>{3}, std::vector<double>{1.0}),
               std::invalid_argument);
  try {
    a->sub(b);
  } catch (const std::invalid_argument &e) {
    EXPECT_EQ(std::string(e.what()), std::string("Tensor shapes do not match"));
  }
}

// data()/grad() hand out mutable references; writes through them are seen by
// the next kernel, as with the reference's host vectors.
TEST(ApiTest, MutableHostViews) {
  auto x = make({3}, {1, 2, 3});
  x->data()[1] = 10.0;
  auto y = x->mul(2.0);
  EXPECT_NEAR(y->data()[1], 20.0, 0.0);
  x->at({2}) = -1.0;
  EXPECT_NEAR(x->sum()->data()[0], 10.0, 0.0);
  x->grad()[0] = 5.0;  // pre-seeded gradient is accumulated into
  x->sum()->backward();
  EXPECT_NEAR(x->grad()[0], 6.0, 0.0);
  EXPECT_NEAR(x->grad_at({1}), 1.0, 0.0);
  EXPECT_EQ(x->size(), static_cast<size_t>(3));
}

// Linear::forward for a batch (the reference's forward only works for batch 1),
// softmax cross-entropy, SGD: loss decreases and a step equals p - lr*g.
TEST(ApiTest, BatchedLinearTrainingStep) {
  const size_t batch = 64, in = 32, hidden = 16, classes = 10;
  std::vector<double> xs(batch * in);
  std::vector<int> labels(batch);
  for (size_t i = 0; i < xs.size(); i++) xs[i] = std::fmod(static_cast<double>(i) * 0.37, 1.0);
  for (size_t i = 0; i < batch; i++) labels[i] = static_cast<int>(i % classes);
  Linear l1(in, hidden), l2(hidden, classes);
  SGD opt({l1.weights(), l1.bias(), l2.weights(), l2.bias()}, 0.5);
  auto x = make({batch, in}, xs);
  x->set_requires_grad(false);
  double first = 0.0, last = 0.0;
  for (int step = 0; step < 20; step++) {
    auto loss = softmax_cross_entropy(l2.forward(l1.forward_relu(x)), labels);
    opt.zero_grad();
    loss->backward();
    if (step == 0) {
      first = loss->data()[0];
      std::vector<double> before = l2.bias()->data();
      std::vector<double> g = l2.bias()->grad();
      opt.step();
      for (size_t j = 0; j < classes; j++) {
        EXPECT_NEAR(l2.bias()->data()[j], before[j] - 0.5 * g[j], 1e-15);
      }
    } else {
      opt.step();
    }
    last = loss->data()[0];
  }
  EXPECT_NEAR(first, std::log(10.0), 0.5);
  EXPECT_LT(last, first);
  EXPECT_EQ(argmax_rows(l2.forward(l1.forward_relu(x))).size(), batch);
}

// Graph nodes do not own themselves: dropping the root frees every intermediate
// buffer, so repeated steps do not grow device memory.
TEST(ApiTest, IntermediatesAreFreed) {
  auto x = std::make_shared<Tensor>(std::vector<size_t>{1 << 20});
  auto run = [&] {
    auto y = x->add(1.0)->mul(2.0)->relu()->tanh()->sum();
    y->backward();
    return y->data()[0];
  };
  run();
  micrograd::synchronize();
  size_t free_before = 0, free_after = 0, total = 0;
  ASSERT_EQ(mg_mem_info(&free_before, &total), 0);
  for (int i = 0; i < 50; i++) run();
  micrograd::synchronize();
  ASSERT_EQ(mg_mem_info(&free_after, &total), 0);
  // 50 iterations x 4 intermediates x (8 + 8) MiB would be 3.2 GB if leaked.
  EXPECT_LT(free_before - std::min(free_before, free_after), static_cast<size_t>(256) << 20);
}

// Two inputs refreshed in turn on the copy stream: each result belongs to the
// batch that was current when its step was built, and a host read sees the new values.
TEST(ApiTest, PrefetchFromHostRefreshesInPlace) {
  micrograd::reserve_device_memory(static_cast<size_t>(64) << 20);
  const size_t n = 1 << 16;
  std::vector<std::vector<double>> batches(4, std::vector<double>(n));
  for (size_t b = 0; b < batches.size(); b++) {
    for (size_t i = 0; i < n; i++) batches[b][i] = static_cast<double>((i % 7) + b);
  }
  std::shared_ptr<Tensor> x[2] = {Tensor::from_host({n}, batches[0].data()),
                                  Tensor::from_host({n}, batches[1].data())};
  std::vector<std::shared_ptr<Tensor>> sums;
  for (size_t b = 0; b < batches.size(); b++) {
    if (b >= 2) x[b % 2]->prefetch_from_host(batches[b].data());
    sums.push_back(x[b % 2]->mul(2.0)->sum());
  }
  for (size_t b = 0; b < batches.size(); b++) {
    double want = 0.0;
    for (double v : batches[b]) want += 2.0 * v;
    EXPECT_DOUBLE_EQ(std::as_const(*sums[b]).data()[0], want);  // small integers: exact in any order
  }
  EXPECT_EQ(std::as_const(*x[1]).data()[5], batches[3][5]);
  EXPECT_EQ(std::as_const(*x[0]).data()[n - 1], batches[2][n - 1]);
}

TEST(ApiTest, ToDotMentionsOps) {
  auto x = make({1}, {2.0});
  auto y = x->mul(3.0)->add(x);
  y->backward();
  const std::string dot = to_dot(y);
  EXPECT_TRUE(dot.find("digraph {") == 0);
  EXPECT_TRUE(dot.find("* 3.00") != std::string::npos);
  EXPECT_EQ(format_scalar("/", 4.0), std::string("/ 4.00"));
}

// IDX reader: same per-sample tensors as the reference's load_mnist (one [1,784]
// image scaled by 1/255 and a one-hot [1,10] label), plus the batched form.
TEST(ApiTest, LoadMnistFromIdxFiles) {
  const char *img_path = "/tmp/mg_b200_test-images-idx3-ubyte";
  const char *lbl_path = "/tmp/mg_b200_test-labels-idx1-ubyte";
  const int count = 5;
  {
    std::ofstream img(img_path, std::ios::binary), lbl(lbl_path, std::ios::binary);
    std::vector<char> header(16, 0);
    img.write(header.data(), 16);
    lbl.write(header.data(), 8);
    for (int i = 0; i < count; i++) {
      for (int j = 0; j < 784; j++) {
        unsigned char px = static_cast<unsigned char>((i * 37 + j * 11) % 256);
        img.write(reinterpret_cast<char *>(&px), 1);
      }
      unsigned char label = static_cast<unsigned char>((i * 3) % 10);
      lbl.write(reinterpret_cast<char *>(&label), 1);
    }
  }
  MNISTData data = load_mnist(img_path, lbl_path, count);
  ASSERT_EQ(data.images.size(), static_cast<size_t>(count));
  ASSERT_EQ(data.labels.size(), static_cast<size_t>(count));
  for (int i = 0; i < count; i++) {
    EXPECT_EQ(data.images[i]->shape().size(), static_cast<size_t>(2));
    EXPECT_EQ(data.images[i]->size(), static_cast<size_t>(784));
    EXPECT_EQ(data.images[i]->at({0, 5}), ((i * 37 + 5 * 11) % 256) / 255.0);
    EXPECT_EQ(data.labels[i]->at({0, static_cast<size_t>((i * 3) % 10)}), 1.0);
    EXPECT_EQ(data.labels[i]->sum()->data()[0], 1.0);
  }
  // the per-sample views feed the ops like any other tensor
  auto pooled = avg_pool_2x2(data.images[2]);
  EXPECT_EQ(pooled->size(), static_cast<size_t>(196));
  MNISTBatch batch = load_mnist_batched(img_path, lbl_path, count);
  EXPECT_EQ(batch.images->shape()[0], static_cast<size_t>(count));
  EXPECT_EQ(batch.labels->at({4}), 2.0);
  EXPECT_EQ(batch.images->at({3, 7}), data.images[3]->at({0, 7}));
  std::remove(img_path);
  std::remove(lbl_path);
}
