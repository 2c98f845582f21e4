// Process-wide runtime controls declared in micrograd/Backend.h.
#include "mg_cuda.h"
#include "micrograd/Backend.h"
#include "micrograd/detail/Storage.h"

namespace micrograd {

using detail::check;

void synchronize() { check(mg_sync(), "synchronize"); }

void reserve_device_memory(std::size_t bytes) { check(mg_pool_reserve(bytes), "reserve_device_memory"); }

RecordedStep::~RecordedStep() {
  if (recording_) {
    // Abandoned between begin() and end(): close the recording so that later work
    // executes again, and drop what was recorded.
    int discarded = -1;
    if (mg_graph_end(&discarded) == MG_OK && discarded >= 0) {
      mg_graph_destroy(discarded);
    }
  }
  if (id_ >= 0) {
    mg_graph_destroy(id_);
  }
}

void RecordedStep::begin() {
  if (id_ >= 0) {
    check(mg_graph_destroy(id_), "recorded step");
    id_ = -1;
  }
  check(mg_graph_begin(), "begin recording");
  recording_ = true;
}

void RecordedStep::end() {
  recording_ = false;
  check(mg_graph_end(&id_), "end recording");
}

void RecordedStep::replay() {
  check(mg_graph_launch(id_), "replay");
  // Whatever the step wrote on the device is newer than any host copy.
  detail::advance_device_epoch();
}

int RecordedStep::kernels() const { return mg_graph_kernels(id_); }

void comm_unique_id(char *out128) { check(mg_comm_unique_id(out128), "comm_unique_id"); }

void comm_init(const char *id128, int rank, int world) {
  check(mg_comm_init(id128, rank, world), "comm_init");
}

void comm_shutdown() { check(mg_comm_destroy(), "comm_shutdown"); }

int comm_rank() { return mg_comm_rank(); }

int comm_world() { return mg_comm_world(); }

}  // namespace micrograd
