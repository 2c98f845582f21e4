// Lifecycle, storage, events: the parts of the C ABI that hold no arithmetic.
#include "common.cuh"

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace mg {

namespace {
thread_local std::string t_last_error;
std::mutex g_init_mutex;
Context g_ctx;
std::vector<cudaEvent_t> g_events;
struct RecordedStep {
  cudaGraphExec_t exec = nullptr;
  unsigned long long kernels = 0;  // kernel nodes, for the launch counter
};
std::vector<RecordedStep> g_steps;
// Scratch buffers that were outgrown while a recorded step existed: the step's
// kernels carry the old address, so the memory stays allocated until shutdown.
std::vector<void *> g_retired_scratch;

bool any_recorded_step() {
  for (const auto &step : g_steps)
    if (step.exec) return true;
  return false;
}

// Gives up an outgrown scratch buffer (stream-ordered free, or parked, see above).
cudaError_t retire_scratch(void *buf, cudaStream_t stream) {
  if (!buf) return cudaSuccess;
  if (any_recorded_step()) {
    g_retired_scratch.push_back(buf);
    return cudaSuccess;
  }
  return cudaFreeAsync(buf, stream);
}
}  // namespace

Context &ctx() { return g_ctx; }

int fail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  t_last_error = buf;
  return code;
}

int cuda_fail(cudaError_t e, const char *what) {
  int code = (e == cudaErrorMemoryAllocation) ? MG_ERR_OOM : MG_ERR_CUDA;
  return fail(code, "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
}

static int pick_device() {
  const char *names[] = {"MG_DEVICE", "LOCAL_RANK"};
  for (const char *n : names) {
    const char *v = std::getenv(n);
    if (v && *v) return std::atoi(v);
  }
  return 0;
}

static int init_locked(int device) {
  Context &c = g_ctx;
  if (c.ready) {
    if (device >= 0 && device != c.device)
      return fail(MG_ERR_INVALID, "mg_init: already bound to device %d (one device per process)",
                  c.device);
    return MG_OK;
  }
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    return fail(MG_ERR_CUDA,
                "no usable CUDA device (%s); this backend has no CPU fallback",
                e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
  }
  if (device < 0) device = pick_device();
  if (device >= count)
    return fail(MG_ERR_INVALID, "device %d requested but only %d visible", device, count);
  MG_CUDA_TRY(cudaSetDevice(device));
  cudaDeviceProp prop;
  MG_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
  c.device = device;
  c.sm_count = prop.multiProcessorCount;
  MG_CUDA_TRY(cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking));
  // The communication stream gets the highest priority: an all-reduce kernel is
  // placed on the first SMs that free up instead of queueing behind every CTA of
  // the GEMM in flight, so neither rank spins long waiting for its peer.
  int prio_least = 0, prio_greatest = 0;
  MG_CUDA_TRY(cudaDeviceGetStreamPriorityRange(&prio_least, &prio_greatest));
  MG_CUDA_TRY(cudaStreamCreateWithPriority(&c.comm_stream, cudaStreamNonBlocking, prio_greatest));
  MG_CUDA_TRY(cudaStreamCreateWithFlags(&c.copy_stream, cudaStreamNonBlocking));
  MG_CUDA_TRY(cudaEventCreateWithFlags(&c.copy_fork_event, cudaEventDisableTiming));
  MG_CUDA_TRY(cudaEventCreateWithFlags(&c.fork_event, cudaEventDisableTiming));
  MG_CUDA_TRY(cudaEventCreateWithFlags(&c.join_event, cudaEventDisableTiming));
  // Keep freed blocks in the stream-ordered pool instead of returning them to
  // the driver: op results are allocated and freed every step.
  cudaMemPool_t pool;
  MG_CUDA_TRY(cudaDeviceGetDefaultMemPool(&pool, device));
  uint64_t threshold = UINT64_MAX;
  MG_CUDA_TRY(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold));
  MG_CUDA_TRY(cudaMalloc(&c.reduce_partials, sizeof(double) * 2 * kReducePartials));
  MG_CUDA_TRY(cudaMalloc(&c.reduce_ticket, sizeof(unsigned int) * 4));
  MG_CUDA_TRY(cudaMemset(c.reduce_ticket, 0, sizeof(unsigned int) * 4));
  MG_CUDA_TRY(cudaMalloc(&c.kernel_status, sizeof(int)));
  MG_CUDA_TRY(cudaMemset(c.kernel_status, 0, sizeof(int)));
  MG_CUDA_TRY(cudaDeviceSynchronize());
  c.ready = true;
  return MG_OK;
}

int ensure_init() {
  if (g_ctx.ready) return MG_OK;
  std::lock_guard<std::mutex> lock(g_init_mutex);
  return init_locked(-1);
}

int ensure_scratch(double **buf, size_t *have, size_t elems) {
  if (*have >= elems) return MG_OK;
  Context &c = ctx();
  if (c.capturing)
    return fail(MG_ERR_INVALID,
                "a scratch buffer would have to grow while a step is being recorded; run the step "
                "once before mg_graph_begin()");
  MG_CUDA_TRY(retire_scratch(*buf, c.stream));
  *buf = nullptr;
  *have = 0;
  MG_CUDA_TRY(cudaMallocAsync(buf, elems * sizeof(double), c.stream));
  *have = elems;
  return MG_OK;
}

}  // namespace mg

using namespace mg;

// Registers a new event under the smallest free id.
static int create_event(unsigned flags, int *out_id) {
  cudaEvent_t ev;
  MG_CUDA_TRY(cudaEventCreateWithFlags(&ev, flags));
  for (size_t i = 0; i < g_events.size(); i++) {
    if (!g_events[i]) {
      g_events[i] = ev;
      *out_id = (int)i;
      return MG_OK;
    }
  }
  g_events.push_back(ev);
  *out_id = (int)g_events.size() - 1;
  return MG_OK;
}

extern "C" {

const char *mg_last_error(void) { return t_last_error.c_str(); }

int mg_init(int device) {
  std::lock_guard<std::mutex> lock(g_init_mutex);
  return init_locked(device);
}

static void release_mirror_ring_at_shutdown();

int mg_shutdown(void) {
  std::lock_guard<std::mutex> lock(g_init_mutex);
  Context &c = g_ctx;
  if (!c.ready) return MG_OK;
  cudaDeviceSynchronize();
  for (cudaEvent_t ev : g_events)
    if (ev) cudaEventDestroy(ev);
  g_events.clear();
  for (auto &step : g_steps)
    if (step.exec) cudaGraphExecDestroy(step.exec);
  g_steps.clear();
  release_mirror_ring_at_shutdown();
  for (void *buf : g_retired_scratch) cudaFreeAsync(buf, c.stream);
  g_retired_scratch.clear();
  if (c.colsum_scratch) cudaFreeAsync(c.colsum_scratch, c.stream);
  if (c.splitk_scratch) cudaFreeAsync(c.splitk_scratch, c.stream);
  cudaStreamSynchronize(c.stream);
  gemm_release_tables();
  cudaFree(c.reduce_partials);
  cudaFree(c.reduce_ticket);
  cudaFree(c.kernel_status);
  if (c.status_host) cudaFreeHost(c.status_host);
  if (c.flush_buf) cudaFree(c.flush_buf);
  cudaEventDestroy(c.copy_fork_event);
  cudaStreamDestroy(c.copy_stream);
  cudaEventDestroy(c.fork_event);
  cudaEventDestroy(c.join_event);
  cudaStreamDestroy(c.stream);
  cudaStreamDestroy(c.comm_stream);
  unsigned long long launches = c.launches;
  c = Context();
  c.launches = launches;
  return MG_OK;
}

int mg_device(void) { return g_ctx.ready ? g_ctx.device : -1; }

int mg_sm_count(void) {
  if (ensure_init() != MG_OK) return 0;
  return g_ctx.sm_count;
}

static cudaStream_t g_mirror_stream_for_sync();

int mg_sync(void) {
  MG_ENSURE_INIT();
  MG_NOT_WHILE_RECORDING("mg_sync");
  MG_CUDA_TRY(cudaStreamSynchronize(g_ctx.stream));
  MG_CUDA_TRY(cudaStreamSynchronize(g_ctx.comm_stream));
  MG_CUDA_TRY(cudaStreamSynchronize(g_ctx.copy_stream));
  if (g_mirror_stream_for_sync()) MG_CUDA_TRY(cudaStreamSynchronize(g_mirror_stream_for_sync()));
  return MG_OK;
}

int mg_check_kernel_status(void) {
  MG_ENSURE_INIT();
  MG_NOT_WHILE_RECORDING("mg_check_kernel_status");
  int status = 0;
  MG_CUDA_TRY(cudaMemcpyAsync(&status, g_ctx.kernel_status, sizeof(int), cudaMemcpyDeviceToHost,
                              g_ctx.stream));
  MG_CUDA_TRY(cudaStreamSynchronize(g_ctx.stream));
  if (status != 0) {
    cudaMemsetAsync(g_ctx.kernel_status, 0, sizeof(int), g_ctx.stream);
    if (g_ctx.status_host) *g_ctx.status_host = 0;
    gemm_reset_tickets();
    return fail(MG_ERR_KERNEL, "a kernel raised fault code %d (bounded wait expired or bad geometry)",
                status);
  }
  return MG_OK;
}

int mg_kernel_status_mirror(void) {
  MG_ENSURE_INIT();
  MG_NOT_WHILE_RECORDING("mg_kernel_status_mirror");
  Context &c = g_ctx;
  if (!c.status_host) {
    MG_CUDA_TRY(cudaMallocHost(&c.status_host, sizeof(int)));
    *c.status_host = 0;
  }
  MG_CUDA_TRY(cudaMemcpyAsync(c.status_host, c.kernel_status, sizeof(int), cudaMemcpyDeviceToHost,
                              c.stream));
  return MG_OK;
}

int mg_kernel_status_peek(int *out_status) {
  if (!out_status) return fail(MG_ERR_INVALID, "mg_kernel_status_peek: null pointer");
  const volatile int *host = g_ctx.status_host;
  *out_status = host ? *host : 0;
  return MG_OK;
}

int mg_mem_info(size_t *free_bytes, size_t *total_bytes) {
  MG_ENSURE_INIT();
  MG_CUDA_TRY(cudaMemGetInfo(free_bytes, total_bytes));
  return MG_OK;
}

/* ---- storage ---- */

static int alloc_bytes(size_t bytes, void **out) {
  MG_ENSURE_INIT();
  if (!out) return fail(MG_ERR_INVALID, "mg_alloc: null out pointer");
  if (bytes == 0) bytes = 16;
  void *p = nullptr;
  cudaError_t e = cudaMallocAsync(&p, bytes, g_ctx.stream);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(e == cudaErrorMemoryAllocation ? MG_ERR_OOM : MG_ERR_CUDA,
                "device allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
  }
  *out = p;
  return MG_OK;
}

int mg_alloc(size_t n, double **out) { return alloc_bytes(n * sizeof(double), (void **)out); }
int mg_alloc_i32(size_t n, int **out) { return alloc_bytes(n * sizeof(int), (void **)out); }

int mg_free(double *p) {
  if (!p) return MG_OK;
  if (!g_ctx.ready) return MG_OK;  // after shutdown the pool is gone with the context
  cudaError_t e = cudaFreeAsync(p, g_ctx.stream);
  if (e != cudaSuccess) {
    // (e.g. a buffer of a recorded step that was never replayed: its address was only
    // ever reserved.)  Clear the runtime's error slot so the next launch check does
    // not report this failure as its own.
    cudaGetLastError();
    return cuda_fail(e, "cudaFreeAsync");
  }
  return MG_OK;
}

int mg_free_i32(int *p) { return mg_free(reinterpret_cast<double *>(p)); }

int mg_pool_reserve(size_t bytes) {
  MG_ENSURE_INIT();
  MG_NOT_WHILE_RECORDING("mg_pool_reserve");
  if (bytes == 0) return MG_OK;
  // One block of the whole size: if the pool already has such a hole this costs
  // nothing, otherwise the pool grows now rather than in the caller's loop.
  void *block = nullptr;
  int rc = alloc_bytes(bytes, &block);
  if (rc != MG_OK) return rc;
  return mg_free(static_cast<double *>(block));
}

int mg_upload(double *dst, const double *src_host, size_t n) {
  MG_ENSURE_INIT();
  MG_NOT_WHILE_RECORDING("mg_upload (the host address would be baked into the graph)");
  if (n == 0) return MG_OK;
  if (!dst || !src_host) return fail(MG_ERR_INVALID, "mg_upload: null pointer");
  MG_CUDA_TRY(cudaMemcpyAsync(dst, src_host, n * sizeof(double), cudaMemcpyHostToDevice,
                              g_ctx.stream));
  return MG_OK;
}

int mg_upload_async(double *dst, const double *src_host, size_t n, int *out_event_id) {
  MG_ENSURE_INIT();
  MG_NOT_WHILE_RECORDING("mg_upload_async");
  if (!out_event_id) return fail(MG_ERR_INVALID, "mg_upload_async: null event pointer");
  if (n && (!dst || !src_host)) return fail(MG_ERR_INVALID, "mg_upload_async: null pointer");
  Context &c = g_ctx;
  // dst comes from the stream-ordered pool on the compute stream: the copy may
  // touch it only once the compute stream has passed the point of allocation.
  MG_CUDA_TRY(cudaEventRecord(c.copy_fork_event, c.stream));
  MG_CUDA_TRY(cudaStreamWaitEvent(c.copy_stream, c.copy_fork_event, 0));
  if (n)
    MG_CUDA_TRY(cudaMemcpyAsync(dst, src_host, n * sizeof(double), cudaMemcpyHostToDevice,
                                c.copy_stream));
  // Ordering only: an event without timing is cheaper to record and to wait on.
  int id = -1;
  int rc = create_event(cudaEventDisableTiming, &id);
  if (rc != MG_OK) return rc;
  MG_CUDA_TRY(cudaEventRecord(g_events[id], c.copy_stream));
  *out_event_id = id;
  return MG_OK;
}

int mg_compute_wait_event(int id) {
  MG_ENSURE_INIT();
  if (id < 0 || (size_t)id >= g_events.size() || !g_events[id])
    return fail(MG_ERR_INVALID, "unknown event id %d", id);
  MG_CUDA_TRY(cudaStreamWaitEvent(g_ctx.stream, g_events[id], 0));
  return MG_OK;
}

int mg_download(double *dst_host, const double *src, size_t n) {
  MG_ENSURE_INIT();
  MG_NOT_WHILE_RECORDING("mg_download");
  if (n == 0) return MG_OK;
  if (!dst_host || !src) return fail(MG_ERR_INVALID, "mg_download: null pointer");
  MG_CUDA_TRY(cudaMemcpyAsync(dst_host, src, n * sizeof(double), cudaMemcpyDeviceToHost,
                              g_ctx.stream));
  MG_CUDA_TRY(cudaStreamSynchronize(g_ctx.stream));
  return MG_OK;
}

int mg_upload_i32(int *dst, const int *src_host, size_t n) {
  MG_ENSURE_INIT();
  MG_NOT_WHILE_RECORDING("mg_upload_i32 (the host address would be baked into the graph)");
  if (n == 0) return MG_OK;
  if (!dst || !src_host) return fail(MG_ERR_INVALID, "mg_upload_i32: null pointer");
  MG_CUDA_TRY(cudaMemcpyAsync(dst, src_host, n * sizeof(int), cudaMemcpyHostToDevice,
                              g_ctx.stream));
  return MG_OK;
}

int mg_download_i32(int *dst_host, const int *src, size_t n) {
  MG_ENSURE_INIT();
  MG_NOT_WHILE_RECORDING("mg_download_i32");
  if (n == 0) return MG_OK;
  if (!dst_host || !src) return fail(MG_ERR_INVALID, "mg_download_i32: null pointer");
  MG_CUDA_TRY(cudaMemcpyAsync(dst_host, src, n * sizeof(int), cudaMemcpyDeviceToHost,
                              g_ctx.stream));
  MG_CUDA_TRY(cudaStreamSynchronize(g_ctx.stream));
  return MG_OK;
}

int mg_copy(double *dst, const double *src, size_t n) {
  MG_ENSURE_INIT();
  if (n == 0) return MG_OK;
  if (!dst || !src) return fail(MG_ERR_INVALID, "mg_copy: null pointer");
  MG_CUDA_TRY(cudaMemcpyAsync(dst, src, n * sizeof(double), cudaMemcpyDeviceToDevice,
                              g_ctx.stream));
  return MG_OK;
}

/* ---- scalar mirrors ---- */
// A one-element result (a loss, a sum) is usually read by the host a little later,
// when more work has been enqueued behind it; a plain download would then wait for
// all of that work.  mg_scalar_mirror copies the value to a pinned slot on a
// stream of its own right after its producer, and mg_scalar_fetch waits for that
// copy only.  256 slots, reused in turn; a ticket names slot and generation.
namespace {
constexpr int kMirrorSlots = 256;
struct MirrorRing {
  double *pinned = nullptr;
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr;
  cudaEvent_t done[kMirrorSlots] = {};
  unsigned long long generation[kMirrorSlots] = {};
  unsigned long long issued = 0;
};
MirrorRing g_mirror;

int mirror_ring_init() {
  if (g_mirror.pinned) return MG_OK;
  MG_CUDA_TRY(cudaMallocHost(&g_mirror.pinned, kMirrorSlots * sizeof(double)));
  MG_CUDA_TRY(cudaStreamCreateWithFlags(&g_mirror.stream, cudaStreamNonBlocking));
  MG_CUDA_TRY(cudaEventCreateWithFlags(&g_mirror.fork, cudaEventDisableTiming));
  for (auto &ev : g_mirror.done) MG_CUDA_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  return MG_OK;
}

void mirror_ring_release() {
  if (!g_mirror.pinned) return;
  cudaStreamSynchronize(g_mirror.stream);
  for (auto &ev : g_mirror.done) cudaEventDestroy(ev);
  cudaEventDestroy(g_mirror.fork);
  cudaStreamDestroy(g_mirror.stream);
  cudaFreeHost(g_mirror.pinned);
  g_mirror = MirrorRing();
}
}  // namespace

static void release_mirror_ring_at_shutdown() { mirror_ring_release(); }
static cudaStream_t g_mirror_stream_for_sync() { return g_mirror.stream; }

int mg_scalar_mirror(const double *src, unsigned long long *out_ticket) {
  MG_ENSURE_INIT();
  if (!src || !out_ticket) return fail(MG_ERR_INVALID, "mg_scalar_mirror: null pointer");
  if (g_ctx.capturing) {
    // A mirror runs on a stream of its own; a recorded step stays on one stream.
    // Ticket 0 is never valid, so a later fetch falls back to an ordinary download.
    *out_ticket = 0;
    return MG_OK;
  }
  int rc = mirror_ring_init();
  if (rc != MG_OK) return rc;
  MirrorRing &m = g_mirror;
  const unsigned long long ticket = ++m.issued;
  const int slot = (int)(ticket % kMirrorSlots);
  m.generation[slot] = ticket;
  MG_CUDA_TRY(cudaEventRecord(m.fork, g_ctx.stream));
  MG_CUDA_TRY(cudaStreamWaitEvent(m.stream, m.fork, 0));
  MG_CUDA_TRY(cudaMemcpyAsync(m.pinned + slot, src, sizeof(double), cudaMemcpyDeviceToHost, m.stream));
  MG_CUDA_TRY(cudaEventRecord(m.done[slot], m.stream));
  *out_ticket = ticket;
  return MG_OK;
}

int mg_scalar_fetch(unsigned long long ticket, double *out, int *expired) {
  MG_ENSURE_INIT();
  if (!out || !expired) return fail(MG_ERR_INVALID, "mg_scalar_fetch: null pointer");
  MirrorRing &m = g_mirror;
  const int slot = (int)(ticket % kMirrorSlots);
  if (!m.pinned || ticket == 0 || m.generation[slot] != ticket) {
    *expired = 1;  // the slot has been reused since: read the value the ordinary way
    return MG_OK;
  }
  MG_CUDA_TRY(cudaEventSynchronize(m.done[slot]));
  *out = m.pinned[slot];
  *expired = 0;
  return MG_OK;
}

int mg_host_alloc(size_t bytes, void **out_host) {
  MG_ENSURE_INIT();
  if (!out_host) return fail(MG_ERR_INVALID, "mg_host_alloc: null out pointer");
  MG_CUDA_TRY(cudaMallocHost(out_host, bytes ? bytes : 16));
  return MG_OK;
}

int mg_host_free(void *host) {
  if (!host) return MG_OK;
  MG_CUDA_TRY(cudaFreeHost(host));
  return MG_OK;
}

/* ---- recorded steps (CUDA graphs) ---- */
// A launch-bound step (a batch-1 or batch-32 training step is ~20 dependent
// micro-kernels) costs mostly launch overhead.  Between mg_graph_begin() and
// mg_graph_end() everything the library enqueues on its compute stream —
// kernels, fills, device copies, pool allocations and frees — is recorded instead
// of executed; mg_graph_launch() then replays the whole step with one launch.
// Buffers allocated while recording keep their addresses across replays (the
// graph owns them and re-creates them at every launch), so a tensor produced by
// the recorded step can be read after each replay.
int mg_graph_begin(void) {
  MG_ENSURE_INIT();
  Context &c = g_ctx;
  if (c.capturing) return fail(MG_ERR_INVALID, "mg_graph_begin: a step is already being recorded");
  MG_CUDA_TRY(cudaStreamSynchronize(c.stream));
  MG_CUDA_TRY(cudaStreamBeginCapture(c.stream, cudaStreamCaptureModeRelaxed));
  c.capturing = true;
  return MG_OK;
}

int mg_graph_end(int *out_id) {
  MG_ENSURE_INIT();
  Context &c = g_ctx;
  if (!c.capturing) return fail(MG_ERR_INVALID, "mg_graph_end: no step is being recorded");
  c.capturing = false;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(c.stream, &graph);
  if (e != cudaSuccess || !graph) {
    cudaGetLastError();
    return fail(MG_ERR_CUDA, "recording the step failed: %s", cudaGetErrorString(e));
  }
  if (!out_id) {
    cudaGraphDestroy(graph);
    return fail(MG_ERR_INVALID, "mg_graph_end: null out pointer");
  }
  RecordedStep step;
  size_t count = 0;
  if (cudaGraphGetNodes(graph, nullptr, &count) == cudaSuccess && count > 0) {
    std::vector<cudaGraphNode_t> nodes(count);
    if (cudaGraphGetNodes(graph, nodes.data(), &count) == cudaSuccess) {
      for (size_t i = 0; i < count; i++) {
        cudaGraphNodeType type;
        if (cudaGraphNodeGetType(nodes[i], &type) == cudaSuccess && type == cudaGraphNodeTypeKernel)
          step.kernels++;
      }
    }
  }
  // Allocations made while recording and still live are released and re-made by
  // every launch, at the same addresses.
  e = cudaGraphInstantiateWithFlags(&step.exec, graph, cudaGraphInstantiateFlagAutoFreeOnLaunch);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate");
  for (size_t i = 0; i < g_steps.size(); i++) {
    if (!g_steps[i].exec) {
      g_steps[i] = step;
      *out_id = (int)i;
      return MG_OK;
    }
  }
  g_steps.push_back(step);
  *out_id = (int)g_steps.size() - 1;
  return MG_OK;
}

int mg_graph_launch(int id) {
  MG_ENSURE_INIT();
  MG_NOT_WHILE_RECORDING("mg_graph_launch");
  if (id < 0 || (size_t)id >= g_steps.size() || !g_steps[id].exec)
    return fail(MG_ERR_INVALID, "unknown recorded step %d", id);
  MG_CUDA_TRY(cudaGraphLaunch(g_steps[id].exec, g_ctx.stream));
  g_ctx.launches += g_steps[id].kernels;
  return MG_OK;
}

int mg_graph_kernels(int id) {
  if (id < 0 || (size_t)id >= g_steps.size() || !g_steps[id].exec) return 0;
  return (int)g_steps[id].kernels;
}

int mg_graph_destroy(int id) {
  if (id < 0 || (size_t)id >= g_steps.size() || !g_steps[id].exec)
    return fail(MG_ERR_INVALID, "unknown recorded step %d", id);
  if (g_ctx.ready) cudaStreamSynchronize(g_ctx.stream);
  cudaGraphExecDestroy(g_steps[id].exec);
  g_steps[id] = RecordedStep();
  return MG_OK;
}

/* ---- events ---- */

int mg_event_create(int *out_id) {
  MG_ENSURE_INIT();
  if (!out_id) return fail(MG_ERR_INVALID, "mg_event_create: null out pointer");
  return create_event(cudaEventDefault, out_id);
}

static int event_at(int id, cudaEvent_t *ev) {
  if (id < 0 || (size_t)id >= g_events.size() || !g_events[id])
    return fail(MG_ERR_INVALID, "unknown event id %d", id);
  *ev = g_events[id];
  return MG_OK;
}

int mg_event_record(int id) {
  MG_ENSURE_INIT();
  cudaEvent_t ev;
  int rc = event_at(id, &ev);
  if (rc != MG_OK) return rc;
  MG_CUDA_TRY(cudaEventRecord(ev, g_ctx.stream));
  return MG_OK;
}

int mg_event_elapsed_ms(int start_id, int stop_id, float *ms) {
  MG_ENSURE_INIT();
  cudaEvent_t a, b;
  int rc = event_at(start_id, &a);
  if (rc != MG_OK) return rc;
  rc = event_at(stop_id, &b);
  if (rc != MG_OK) return rc;
  MG_CUDA_TRY(cudaEventSynchronize(b));
  MG_CUDA_TRY(cudaEventElapsedTime(ms, a, b));
  return MG_OK;
}

int mg_event_destroy(int id) {
  cudaEvent_t ev;
  int rc = event_at(id, &ev);
  if (rc != MG_OK) return rc;
  cudaEventDestroy(ev);
  g_events[id] = nullptr;
  return MG_OK;
}

int mg_event_wait_bounded(int id, double timeout_s) {
  MG_ENSURE_INIT();
  cudaEvent_t ev;
  int rc = event_at(id, &ev);
  if (rc != MG_OK) return rc;
  auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(timeout_s);
  for (;;) {
    cudaError_t e = cudaEventQuery(ev);
    if (e == cudaSuccess) return MG_OK;
    if (e != cudaErrorNotReady) return cuda_fail(e, "cudaEventQuery");
    if (std::chrono::steady_clock::now() >= deadline)
      return fail(MG_ERR_TIMEOUT, "event %d not complete after %.3f s", id, timeout_s);
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

unsigned long long mg_launch_count(void) { return g_ctx.launches; }

int mg_flush_l2(void) {
  MG_ENSURE_INIT();
  Context &c = g_ctx;
  if (!c.flush_buf) {
    c.flush_bytes = (size_t)256 << 20;  // 256 MiB, twice the 126 MB L2
    MG_CUDA_TRY(cudaMalloc(&c.flush_buf, c.flush_bytes));
  }
  MG_CUDA_TRY(cudaMemsetAsync(c.flush_buf, 0, c.flush_bytes, c.stream));
  return MG_OK;
}

}  // extern "C"
