#pragma once
// Bookkeeping of the data-parallel gradient exchange: which parameters travel
// together in one all-reduce message ("bucket"), and which buckets have been
// reduced since the last optimiser step.  Pure host logic with no device calls,
// so it is unit-tested on a machine without a GPU.
//
// The sums being exchanged are the weight and bias gradients, which the
// reference accumulates over all rows of the batch in one loop
// (src/ops/Matmul.cpp:52-58); with the batch sharded over ranks each rank holds
// a partial sum and one all-reduce per bucket completes it.

#include <algorithm>
#include <cstddef>
#include <stdexcept>
#include <vector>

namespace micrograd::detail {

class GradBuckets {
public:
  struct Bucket {
    size_t first = 0, last = 0;  // parameter indices [first, last]
    size_t begin = 0, end = 0;   // element range in the flat gradient buffer
    bool wanted = false;         // at least one member requires a gradient
  };

  // Groups the parameter list into buckets.  A 2-D weight [in, out] directly
  // followed by its bias ([1, out] or [out]) forms one bucket — one message per
  // layer; every other parameter is a bucket of its own.  The grouping is
  // recorded here once and never derived from index parity, so lists such as
  // "all weights, then all biases" or layers without a bias are handled.
  // `offsets[i]` is where parameter i starts in the flat buffer (ascending) and
  // `flat_elems` its total length.
  void plan(const std::vector<std::vector<size_t>> &shapes, const std::vector<size_t> &offsets,
            const std::vector<char> &requires_grad, size_t flat_elems) {
    const size_t count = shapes.size();
    buckets_.clear();
    bucket_of_.assign(count, 0);
    ready_.assign(count, 0);
    needs_.assign(requires_grad.begin(), requires_grad.end());
    needs_.resize(count, 1);
    size_t i = 0;
    while (i < count) {
      Bucket b;
      b.first = b.last = i;
      if (i + 1 < count && is_bias_of(shapes[i], shapes[i + 1])) {
        b.last = i + 1;
      }
      b.begin = offsets[b.first];
      b.end = (b.last + 1 < count) ? offsets[b.last + 1] : flat_elems;
      for (size_t k = b.first; k <= b.last; k++) {
        bucket_of_[k] = buckets_.size();
        b.wanted = b.wanted || needs_[k];
      }
      buckets_.push_back(b);
      i = b.last + 1;
    }
    reduced_.assign(buckets_.size(), 0);
    any_reduced_ = false;
    sweep_ = 0;
  }

  const std::vector<Bucket> &buckets() const { return buckets_; }
  size_t bucket_of(size_t param) const { return bucket_of_[param]; }

  // A backward sweep is identified by `sweep`, a counter that grows with every
  // backward() call.  The first hook of a sweep calls begin_sweep(): flags left
  // by an earlier sweep are dropped, so a stale "ready" can never fire a bucket
  // early, and the requires-gradient flags are refreshed.  A new sweep after a
  // bucket has already been reduced in this step is refused: the buffer then
  // holds sums over all ranks, and reducing local additions on top of them
  // would count the first sweep's gradients once per rank.
  bool is_new_sweep(unsigned long long sweep) const { return sweep != sweep_; }

  void begin_sweep(unsigned long long sweep, const std::vector<char> &requires_grad) {
    if (any_reduced_) {
      throw std::logic_error(
          "SGD with gradient all-reduce: backward() ran again before step(); the gradients of "
          "the first sweep are already summed across ranks. Call step() (or zero_grad()) between "
          "backward sweeps.");
    }
    std::fill(ready_.begin(), ready_.end(), 0);
    for (size_t k = 0; k < needs_.size() && k < requires_grad.size(); k++) {
      needs_[k] = requires_grad[k];
    }
    for (auto &b : buckets_) {
      b.wanted = false;
      for (size_t k = b.first; k <= b.last; k++) {
        b.wanted = b.wanted || needs_[k];
      }
    }
    sweep_ = sweep;
  }

  // The current sweep has finished parameter `param`.  Returns the index of the
  // bucket that is now complete and must be reduced, or -1.
  long on_ready(size_t param) {
    ready_[param] = 1;
    const size_t b = bucket_of_[param];
    if (reduced_[b]) {
      return -1;
    }
    for (size_t k = buckets_[b].first; k <= buckets_[b].last; k++) {
      if (needs_[k] && !ready_[k]) {
        return -1;
      }
    }
    return static_cast<long>(b);
  }

  bool any_reduced() const { return any_reduced_; }

  void mark_reduced(size_t bucket) {
    reduced_[bucket] = 1;
    any_reduced_ = true;
  }

  // Buckets that want a gradient and were not reduced since the last
  // end_step(): a member never received its hook (it is not part of the graph,
  // or its partner finished in another sweep).  step() reduces them before the
  // update, so no rank ever applies an unreduced gradient.
  std::vector<size_t> unreduced() const {
    std::vector<size_t> out;
    for (size_t b = 0; b < buckets_.size(); b++) {
      if (buckets_[b].wanted && !reduced_[b]) {
        out.push_back(b);
      }
    }
    return out;
  }

  // step() or zero_grad(): the next sweep starts a new exchange round.
  void end_step() {
    std::fill(ready_.begin(), ready_.end(), 0);
    std::fill(reduced_.begin(), reduced_.end(), 0);
    any_reduced_ = false;
  }

private:
  static bool is_bias_of(const std::vector<size_t> &weight, const std::vector<size_t> &bias) {
    if (weight.size() != 2) {
      return false;
    }
    const size_t out = weight[1];
    return (bias.size() == 1 && bias[0] == out) ||
           (bias.size() == 2 && bias[0] == 1 && bias[1] == out && weight[0] != 1);
  }

  std::vector<Bucket> buckets_;
  std::vector<size_t> bucket_of_;
  std::vector<char> ready_, reduced_, needs_;
  bool any_reduced_ = false;
  unsigned long long sweep_ = 0;
};

}  // namespace micrograd::detail
