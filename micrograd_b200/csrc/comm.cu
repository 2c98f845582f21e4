// Data-parallel gradient exchange: NCCL all-reduce over NVLink on a dedicated
// stream, event-chained to the compute stream so it overlaps the rest of the
// backward pass.
//
// NCCL is bound at run time (dlopen) rather than at link time: the library
// loads on machines without NCCL, and inside a process that has already loaded
// a newer NCCL (e.g. the one bundled with PyTorch) the same instance is reused.
#include "common.cuh"

#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <thread>

namespace mg {
namespace {

struct NcclApi {
  void *handle = nullptr;
  decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
  decltype(&ncclCommInitRank) CommInitRank = nullptr;
  decltype(&ncclCommInitRankConfig) CommInitRankConfig = nullptr;  // optional
  decltype(&ncclCommDestroy) CommDestroy = nullptr;
  decltype(&ncclCommAbort) CommAbort = nullptr;
  decltype(&ncclAllReduce) AllReduce = nullptr;
  decltype(&ncclGetErrorString) GetErrorString = nullptr;
  decltype(&ncclCommGetAsyncError) CommGetAsyncError = nullptr;
};

NcclApi g_nccl;
ncclComm_t g_comm = nullptr;
int g_rank = 0, g_world = 1;

int load_nccl() {
  if (g_nccl.handle) return MG_OK;
  const char *names[] = {"libnccl.so.2", "libnccl.so"};
  void *h = nullptr;
  for (const char *n : names) {
    h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (h) break;
  }
  if (!h) return fail(MG_ERR_NCCL, "cannot load NCCL: %s", dlerror());
#define MG_NCCL_SYM(field, sym)                                                                    \
  g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(h, #sym));                          \
  if (!g_nccl.field) return fail(MG_ERR_NCCL, "NCCL symbol %s not found", #sym);
  MG_NCCL_SYM(GetUniqueId, ncclGetUniqueId)
  MG_NCCL_SYM(CommInitRank, ncclCommInitRank)
  MG_NCCL_SYM(CommDestroy, ncclCommDestroy)
  MG_NCCL_SYM(CommAbort, ncclCommAbort)
  MG_NCCL_SYM(AllReduce, ncclAllReduce)
  MG_NCCL_SYM(GetErrorString, ncclGetErrorString)
  MG_NCCL_SYM(CommGetAsyncError, ncclCommGetAsyncError)
#undef MG_NCCL_SYM
  g_nccl.CommInitRankConfig =
      reinterpret_cast<decltype(g_nccl.CommInitRankConfig)>(dlsym(h, "ncclCommInitRankConfig"));
  g_nccl.handle = h;
  return MG_OK;
}

int nccl_fail(ncclResult_t r, const char *what) {
  return fail(MG_ERR_NCCL, "NCCL error %d (%s) in %s", (int)r,
              g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "?", what);
}

}  // namespace
}  // namespace mg

using namespace mg;

static_assert(sizeof(ncclUniqueId) == 128, "the C ABI passes the NCCL id as 128 bytes");

extern "C" {

int mg_comm_unique_id(char *out128_host) {
  if (!out128_host) return fail(MG_ERR_INVALID, "mg_comm_unique_id: null pointer");
  int rc = load_nccl();
  if (rc != MG_OK) return rc;
  ncclUniqueId id;
  ncclResult_t r = g_nccl.GetUniqueId(&id);
  if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
  std::memcpy(out128_host, &id, sizeof(id));
  return MG_OK;
}

int mg_comm_init(const char *id128_host, int rank, int world) {
  MG_ENSURE_INIT();
  if (!id128_host || world < 1 || rank < 0 || rank >= world)
    return fail(MG_ERR_INVALID, "mg_comm_init: bad rank/world (%d/%d)", rank, world);
  if (g_comm) return fail(MG_ERR_INVALID, "mg_comm_init: communicator already initialised");
  int rc = load_nccl();
  if (rc != MG_OK) return rc;
  ncclUniqueId id;
  std::memcpy(&id, id128_host, sizeof(id));
  // The gradient messages are a few MB: a handful of CTAs moves them at NVLink
  // speed, and every CTA NCCL takes is an SM the overlapped GEMMs lose.
  int max_ctas = 8;
  if (const char *v = std::getenv("MG_NCCL_MAX_CTAS")) {
    if (*v) max_ctas = std::atoi(v);
  }
  ncclResult_t r;
  if (g_nccl.CommInitRankConfig && max_ctas > 0) {
    ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
    config.blocking = 1;
    config.maxCTAs = max_ctas;
    config.minCTAs = 1;
    r = g_nccl.CommInitRankConfig(&g_comm, world, id, rank, &config);
  } else {
    r = g_nccl.CommInitRank(&g_comm, world, id, rank);
  }
  if (r != ncclSuccess) {
    g_comm = nullptr;
    return nccl_fail(r, "ncclCommInitRank");
  }
  g_rank = rank;
  g_world = world;
  return MG_OK;
}

int mg_comm_destroy(void) {
  if (!g_comm) return MG_OK;
  if (ctx().ready) cudaStreamSynchronize(ctx().comm_stream);
  ncclResult_t r = g_nccl.CommDestroy(g_comm);
  g_comm = nullptr;
  g_rank = 0;
  g_world = 1;
  if (r != ncclSuccess) return nccl_fail(r, "ncclCommDestroy");
  return MG_OK;
}

int mg_comm_rank(void) { return g_rank; }
int mg_comm_world(void) { return g_world; }

int mg_allreduce_sum_async(double *buf, size_t n) {
  MG_ENSURE_INIT();
  if (n == 0) return MG_OK;
  if (!buf) return fail(MG_ERR_INVALID, "mg_allreduce_sum_async: null buffer");
  if (!g_comm) {
    if (g_world == 1) return MG_OK;  // single process: the sum over ranks is the buffer itself
    return fail(MG_ERR_NCCL, "mg_allreduce_sum_async: communicator not initialised");
  }
  Context &c = ctx();
  // comm stream picks up after everything enqueued on the compute stream so far
  MG_CUDA_TRY(cudaEventRecord(c.fork_event, c.stream));
  MG_CUDA_TRY(cudaStreamWaitEvent(c.comm_stream, c.fork_event, 0));
  ncclResult_t r = g_nccl.AllReduce(buf, buf, n, ncclDouble, ncclSum, g_comm, c.comm_stream);
  if (r != ncclSuccess) return nccl_fail(r, "ncclAllReduce");
  return MG_OK;
}

int mg_comm_join(void) {
  MG_ENSURE_INIT();
  Context &c = ctx();
  MG_CUDA_TRY(cudaEventRecord(c.join_event, c.comm_stream));
  MG_CUDA_TRY(cudaStreamWaitEvent(c.stream, c.join_event, 0));
  return MG_OK;
}

int mg_comm_wait_bounded(double timeout_s) {
  MG_ENSURE_INIT();
  Context &c = ctx();
  auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(timeout_s);
  for (;;) {
    if (g_comm) {
      ncclResult_t async = ncclSuccess;
      ncclResult_t r = g_nccl.CommGetAsyncError(g_comm, &async);
      if (r != ncclSuccess || (async != ncclSuccess && async != ncclInProgress)) {
        g_nccl.CommAbort(g_comm);
        g_comm = nullptr;
        return nccl_fail(r != ncclSuccess ? r : async, "asynchronous NCCL failure");
      }
    }
    cudaError_t e = cudaStreamQuery(c.comm_stream);
    if (e == cudaSuccess) return MG_OK;
    if (e != cudaErrorNotReady) return cuda_fail(e, "cudaStreamQuery(comm)");
    if (std::chrono::steady_clock::now() >= deadline) {
      if (g_comm) {
        g_nccl.CommAbort(g_comm);
        g_comm = nullptr;
      }
      return fail(MG_ERR_TIMEOUT, "collective not complete after %.3f s; communicator aborted",
                  timeout_s);
    }
    std::this_thread::sleep_for(std::chrono::microseconds(100));
  }
}

}  // extern "C"
