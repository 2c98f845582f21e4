// CPU-only unit tests of the data-parallel bookkeeping (no device, no CUDA link):
// how an optimiser's parameter list is grouped into all-reduce messages, and the
// rules that keep every rank from applying a gradient that was not reduced.
#include <gtest/gtest.h>

#include <stdexcept>
#include <vector>

#include "micrograd/detail/GradBuckets.h"

using micrograd::detail::GradBuckets;
using Shapes = std::vector<std::vector<size_t>>;

namespace {
// Flat layout as SGD::enable_allreduce() makes it: slices on 32-element boundaries.
std::vector<size_t> offsets_of(const Shapes &shapes, size_t *total) {
  std::vector<size_t> offsets;
  size_t at = 0;
  for (const auto &s : shapes) {
    size_t n = 1;
    for (size_t d : s) n *= d;
    offsets.push_back(at);
    at += (n + 31) / 32 * 32;
  }
  *total = at;
  return offsets;
}

GradBuckets planned(const Shapes &shapes, std::vector<char> needs = {}) {
  size_t total = 0;
  auto offsets = offsets_of(shapes, &total);
  if (needs.empty()) needs.assign(shapes.size(), 1);
  GradBuckets b;
  b.plan(shapes, offsets, needs, total);
  return b;
}
}  // namespace

TEST(GradBuckets, WeightBiasPairsFormOneMessagePerLayer) {
  auto b = planned({{784, 1024}, {1, 1024}, {1024, 1024}, {1, 1024}, {1024, 10}, {1, 10}});
  ASSERT_EQ(b.buckets().size(), 3u);
  EXPECT_EQ(b.buckets()[0].first, 0u);
  EXPECT_EQ(b.buckets()[0].last, 1u);
  EXPECT_EQ(b.buckets()[0].begin, 0u);
  EXPECT_EQ(b.buckets()[0].end, 784u * 1024u + 1024u);
  EXPECT_EQ(b.buckets()[2].first, 4u);
  EXPECT_EQ(b.buckets()[2].end - b.buckets()[2].begin, 10240u + 32u);
  EXPECT_EQ(b.bucket_of(3), 1u);
}

TEST(GradBuckets, WeightsThenBiasesAreNotPairedByPosition) {
  // W1, W2, b1, b2: index parity would have paired (W1, W2) and (b1, b2)
  auto b = planned({{8, 16}, {16, 4}, {1, 16}, {1, 4}});
  ASSERT_EQ(b.buckets().size(), 4u);
  for (size_t i = 0; i < 4; i++) {
    EXPECT_EQ(b.buckets()[i].first, i);
    EXPECT_EQ(b.buckets()[i].last, i);
  }
  b.begin_sweep(1, {1, 1, 1, 1});
  EXPECT_EQ(b.on_ready(2), 2);  // every parameter completes its own bucket
  EXPECT_EQ(b.on_ready(0), 0);
}

TEST(GradBuckets, LayerWithoutBiasAndOddCount) {
  // W1 (no bias), W2 + b2, W3 (no bias): three buckets, the middle one a pair
  auto b = planned({{8, 16}, {16, 4}, {4}, {4, 2}});
  ASSERT_EQ(b.buckets().size(), 3u);
  EXPECT_EQ(b.buckets()[1].first, 1u);
  EXPECT_EQ(b.buckets()[1].last, 2u);
  EXPECT_EQ(b.buckets()[2].first, 3u);
}

TEST(GradBuckets, PairFiresOnlyWhenBothHalvesAreFinal) {
  auto b = planned({{8, 16}, {1, 16}, {16, 4}, {1, 4}});
  b.begin_sweep(1, {1, 1, 1, 1});
  EXPECT_EQ(b.on_ready(3), -1);
  EXPECT_EQ(b.on_ready(2), 1);
  b.mark_reduced(1);
  EXPECT_EQ(b.on_ready(1), -1);
  EXPECT_EQ(b.on_ready(0), 0);
  b.mark_reduced(0);
  EXPECT_TRUE(b.unreduced().empty());
}

TEST(GradBuckets, UnusedParameterLeavesItsBucketForStep) {
  auto b = planned({{8, 16}, {1, 16}, {16, 4}, {1, 4}});
  b.begin_sweep(1, {1, 1, 1, 1});
  EXPECT_EQ(b.on_ready(3), -1);
  EXPECT_EQ(b.on_ready(2), 1);
  b.mark_reduced(1);
  EXPECT_EQ(b.on_ready(0), -1);  // bias 1 never shows up in this sweep
  auto left = b.unreduced();
  ASSERT_EQ(left.size(), 1u);
  EXPECT_EQ(left[0], 0u);  // step() must reduce the first layer's bucket itself
  b.mark_reduced(0);
  b.end_step();
  EXPECT_EQ(b.unreduced().size(), 2u);  // a new step starts with nothing reduced
}

TEST(GradBuckets, FrozenHalfDoesNotBlockItsPartner) {
  auto b = planned({{8, 16}, {1, 16}}, {1, 0});
  b.begin_sweep(1, {1, 0});
  EXPECT_EQ(b.on_ready(0), 0);  // the bias takes no gradient: the weight alone completes
  // a bucket nobody wants is never exchanged
  auto frozen = planned({{8, 16}, {1, 16}}, {0, 0});
  EXPECT_TRUE(frozen.unreduced().empty());
}

TEST(GradBuckets, StaleFlagsOfAnEarlierSweepDoNotFireEarly) {
  auto b = planned({{8, 16}, {1, 16}});
  b.begin_sweep(1, {1, 1});
  EXPECT_EQ(b.on_ready(0), -1);  // sweep 1 reaches the weight only
  EXPECT_TRUE(b.is_new_sweep(2));
  b.begin_sweep(2, {1, 1});
  EXPECT_EQ(b.on_ready(1), -1);  // the weight's flag from sweep 1 is gone
  EXPECT_EQ(b.on_ready(0), 0);
}

TEST(GradBuckets, SecondSweepAfterAnExchangeIsRefused) {
  auto b = planned({{8, 16}, {1, 16}});
  b.begin_sweep(1, {1, 1});
  b.on_ready(0);
  EXPECT_EQ(b.on_ready(1), 0);
  b.mark_reduced(0);
  bool threw = false;
  try {
    b.begin_sweep(2, {1, 1});
  } catch (const std::logic_error &) {
    threw = true;
  }
  EXPECT_TRUE(threw);
  b.end_step();  // step() or zero_grad()
  b.begin_sweep(3, {1, 1});
  b.on_ready(1);
  EXPECT_EQ(b.on_ready(0), 0);
}
