// The reference trainer's per-sample loop (src/main.cpp:16-51) on synthetic
// images, written against the public API only, so the same file builds against
// the reference's sources (CPU) and against the B200 backend.  Prints the
// samples/s of the loop and the final average loss.
//   usage: trainer_loop [samples] [epochs] [recorded]
// With MG_TRAINER_RECORDED defined (B200 build only) a third argument "recorded"
// runs the same loop body as one recorded step (micrograd::RecordedStep): the
// first sample runs normally, the second is recorded, every later sample is one
// replay after its image and label have been copied into the step's input tensors.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <string>
#include <vector>

#include "micrograd/nn.h"

int main(int argc, char **argv) {
  const size_t samples = argc > 1 ? static_cast<size_t>(std::atol(argv[1])) : 512;
  const int epochs = argc > 2 ? std::atoi(argv[2]) : 2;
  const bool recorded = argc > 3 && std::string(argv[3]) == "recorded";

  // synthetic "images" and one-hot labels from a small LCG (no data files needed)
  unsigned long long state = 12345;
  auto next = [&]() {
    state = state * 6364136223846793005ULL + 1442695040888963407ULL;
    return static_cast<double>((state >> 33) & 0xFFFFFF) / static_cast<double>(0x1000000);
  };
  std::vector<std::shared_ptr<Tensor>> images, labels;
  std::vector<std::vector<double>> host_images, host_labels;
  for (size_t i = 0; i < samples; i++) {
    std::vector<double> px(784);
    for (double &v : px) v = next();
    std::vector<double> one_hot(10, 0.0);
    one_hot[static_cast<size_t>(next() * 10.0) % 10] = 1.0;
    if (recorded) {
      host_images.push_back(px);
      host_labels.push_back(one_hot);
    } else {
      images.push_back(std::make_shared<Tensor>(std::vector<size_t>{1, 784}, px));
      labels.push_back(std::make_shared<Tensor>(std::vector<size_t>{1, 10}, one_hot));
    }
  }

  Linear l1(196, 100);
  Linear l2(100, 10);
  SGD optimizer({l1.weights(), l1.bias(), l2.weights(), l2.bias()}, 0.01);

  double last_avg = 0.0;
  int correct = 0;
  const auto t0 = std::chrono::steady_clock::now();
#ifdef MG_TRAINER_RECORDED
  if (recorded) {
    auto image = std::make_shared<Tensor>(std::vector<size_t>{1, 784}, host_images[0]);
    auto label = std::make_shared<Tensor>(std::vector<size_t>{1, 10}, host_labels[0]);
    std::shared_ptr<Tensor> out, loss;
    auto body = [&]() {
      auto pooled = avg_pool_2x2(image);
      auto x = l1.forward(pooled)->relu();
      out = l2.forward(x);
      loss = mse_loss(out, label);
      optimizer.zero_grad();
      loss->backward();
      optimizer.step();
    };
    micrograd::RecordedStep step;
    size_t seen = 0;
    for (int epoch = 0; epoch < epochs; epoch++) {
      double total_loss = 0.0;
      correct = 0;
      for (size_t i = 0; i < host_images.size(); i++, seen++) {
        image->copy_from_host(host_images[i].data());
        label->copy_from_host(host_labels[i].data());
        if (seen == 0) {
          body();  // normal run: also creates what cannot be created while recording
        } else {
          if (seen == 1) {
            out.reset();  // nothing made before begin() may be released while recording
            loss.reset();
            step.begin();
            body();
            step.end();
          }
          step.replay();
        }
        const Tensor &logits = *out;
        size_t pred = 0, actual = 0;
        for (size_t j = 0; j < 10; j++) {
          if (logits.at({0, j}) > logits.at({0, pred})) pred = j;
          if (host_labels[i][j] > 0.5) actual = j;
        }
        if (pred == actual) correct++;
        total_loss += static_cast<const Tensor &>(*loss).at({0});
      }
      last_avg = total_loss / static_cast<double>(host_images.size());
    }
  } else
#endif
  for (int epoch = 0; epoch < epochs; epoch++) {
    double total_loss = 0.0;
    correct = 0;
    for (size_t i = 0; i < images.size(); i++) {
      auto pooled = avg_pool_2x2(images[i]);
      auto x = l1.forward(pooled)->relu();
      auto out = l2.forward(x);
      auto loss = mse_loss(out, labels[i]);
      size_t pred = 0, actual = 0;
      for (size_t j = 0; j < 10; j++) {
        if (out->at({0, j}) > out->at({0, pred})) pred = j;
        if (labels[i]->at({0, j}) > 0.5) actual = j;
      }
      if (pred == actual) correct++;
      optimizer.zero_grad();
      loss->backward();
      optimizer.step();
      total_loss += loss->at({0});
    }
    last_avg = total_loss / static_cast<double>(images.size());
  }
  const double seconds =
      std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  std::printf("{\"samples\": %zu, \"epochs\": %d, \"samples_per_s\": %.1f, \"avg_loss\": %.6f, "
              "\"correct\": %d}\n",
              samples, epochs, static_cast<double>(samples) * epochs / seconds, last_avg, correct);
  return 0;
}
