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
