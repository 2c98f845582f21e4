// Process-wide runtime controls declared in micrograd/Backend.h.
#include "mg_cuda.h"
#include "micrograd/Backend.h"
#include "micrograd/detail/Storage.h"

namespace micrograd {

using detail::check;

void synchronize() { check(mg_sync(), "synchronize"); }

void comm_unique_id(char *out128) { check(mg_comm_unique_id(out128), "comm_unique_id"); }

void comm_init(const char *id128, int rank, int world) {
  check(mg_comm_init(id128, rank, world), "comm_init");
}

void comm_shutdown() { check(mg_comm_destroy(), "comm_shutdown"); }

int comm_rank() { return mg_comm_rank(); }

int comm_world() { return mg_comm_world(); }

}  // namespace micrograd
