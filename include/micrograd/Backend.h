#pragma once
// Placement tags and process-wide runtime controls.
//
// The reference declares `enum class Backend { CPU, Metal }`
// (include/micrograd/Backend.h:4) and uses it only as the argument of
// Tensor::to().  Both enumerators are kept so existing code compiles; in this
// implementation every tensor lives in B200 device memory whatever tag it
// carries, and to() only records the tag.

#include <cstddef>

namespace micrograd {

enum class Backend { CPU, Metal, CUDA };

// ---- additions of the B200 backend (no counterpart in the reference) ----

// Blocks until all device work enqueued so far has finished.
void synchronize();

// Makes sure the device memory pool behind every tensor holds `bytes` that no
// tensor is using.  Tensors are allocated and freed every step; when the pool has
// to grow while kernels are running the calling thread stalls (tens to hundreds
// of milliseconds in a multi-GPU job).  Call once before a loop that must not
// stall, with the loop's peak footprint plus slack.
void reserve_device_memory(std::size_t bytes);

// A launch-bound step — the reference trainer's per-sample loop
// (src/main.cpp:20-46) enqueues about twenty dependent micro-kernels per sample —
// recorded once and replayed with a single launch (a CUDA graph):
//
//   x->copy_from_host(first_batch);  step();          // run it once normally
//   RecordedStep rec;  rec.begin();  loss = step();  rec.end();
//   for (...) { x->copy_from_host(next_batch);  rec.replay();  loss->at({0}); }
//
// step() is ordinary code on the Tensor API (forward, loss, zero_grad, backward,
// SGD::step).  Rules while recording: no host reads (data(), grad(), at(),
// argmax_rows) and no tensors built from host values; labels are passed as a
// Tensor; every tensor that exists before begin() must outlive end().  Inputs are
// tensors created before begin() and refreshed with copy_from_host(); tensors
// created while recording that are still referenced afterwards (the loss) keep
// their device address, and reading them after replay() returns that replay's
// values.  Parameters are updated in place by every replay.
class RecordedStep {
public:
  RecordedStep() = default;
  ~RecordedStep();
  RecordedStep(const RecordedStep &) = delete;
  RecordedStep &operator=(const RecordedStep &) = delete;
  void begin();
  void end();
  void replay();
  bool recorded() const { return id_ >= 0; }
  int kernels() const;  // kernel launches one replay stands for

private:
  int id_ = -1;
  bool recording_ = false;
};

// Data-parallel training, one process per GPU.  Rank 0 obtains an id with
// comm_unique_id(), ships the 128 bytes to the other ranks by any host channel,
// and every rank calls comm_init().  After SGD::enable_allreduce(), backward()
// sums parameter gradients across ranks over NVLink while it is still running.
void comm_unique_id(char *out128);
void comm_init(const char *id128, int rank, int world);
void comm_shutdown();
int comm_rank();
int comm_world();

}  // namespace micrograd
