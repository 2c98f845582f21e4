// Data-parallel gradient exchange on a dedicated high-priority stream,
// event-chained to the compute stream so it overlaps the rest of the backward
// pass.  Two paths:
//
//  * Buffers obtained from mg_comm_alloc_shared() are mapped into every rank's
//    address space (CUDA IPC over NVLink peer access).  Their all-reduce is one
//    kernel of this file: rank r pulls slice r of the message from every peer
//    with plain loads, adds the W copies in rank order (so every rank ends up
//    with bit-identical sums, whatever the arrival order) and stores the result
//    into all W buffers.  Two flag rounds (inputs ready / results delivered)
//    bracket the data movement; every wait is bounded and reports through the
//    kernel fault word.  No multicast loads are used.
//  * Any other buffer, or a job whose ranks could not map each other's memory,
//    goes through ncclAllReduce.
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
#include <utility>
#include <vector>

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
  decltype(&ncclAllGather) AllGather = nullptr;
  decltype(&ncclGetErrorString) GetErrorString = nullptr;
  decltype(&ncclCommGetAsyncError) CommGetAsyncError = nullptr;
};

// Longest a peer kernel waits for another rank, in SM clock cycles: about ten
// seconds (ranks of one job can be that far apart while they start up), or
// MG_PEER_WAIT_MS from the environment.
long long peer_wait_cycles() {
  static const long long v = [] {
    const char *e = std::getenv("MG_PEER_WAIT_MS");
    const long long ms = e && *e ? std::atoll(e) : 10000;
    // clock64() ticks at the SM clock; take the device's maximum (in kHz = cycles
    // per millisecond), so the limit is at least the requested time.
    int khz = 0;
    if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx().device) != cudaSuccess || khz <= 0)
      khz = 2000000;
    return (ms < 1 ? 1 : ms) * (long long)khz;
  }();
  return v;
}

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
  MG_NCCL_SYM(AllGather, ncclAllGather)
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


// ---------------------------------------------------------------------------
// Peer-memory all-reduce
// ---------------------------------------------------------------------------
constexpr int kMaxPeers = 8;
constexpr int kPeerThreads = 512;
constexpr size_t kFlagBytes = 256;  // ready[8] + done[8] (u32) + CTA ticket, padded

struct SharedBuffer {
  double *base = nullptr;   // this rank's allocation: n doubles followed by the flag block
  size_t elems = 0;
  bool peers_mapped = false;
  double *peer[kMaxPeers] = {};  // peer[q]: rank q's allocation as seen from this process
  unsigned seq = 0;              // all-reduce calls issued on this buffer so far
};

std::vector<SharedBuffer> g_shared;

// Optional timing of the exchange (mg_comm_trace): event pairs around every
// all-reduce on the communication stream, and around every point where the
// compute stream waits for that stream (the part of the exchange that is NOT
// hidden behind compute).  Off by default; nothing is recorded then.
struct CommTrace {
  bool on = false;
  std::vector<cudaEvent_t> pool;  // events handed out in order, reused after a summary
  size_t next = 0;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> exchanges, waits;
};
CommTrace g_trace;

cudaEvent_t trace_event() {
  if (g_trace.next == g_trace.pool.size()) {
    cudaEvent_t ev = nullptr;
    if (cudaEventCreate(&ev) != cudaSuccess) return nullptr;
    g_trace.pool.push_back(ev);
  }
  return g_trace.pool[g_trace.next++];
}

struct PeerArgs {
  double *data[kMaxPeers];     // every rank's buffer, indexed by rank
  unsigned *flags[kMaxPeers];  // every rank's flag block
  int rank;
  unsigned seq;
  size_t offset, n;            // message = elements [offset, offset + n) of each buffer; both even
  long long wait_cycles;
  int *status;
};

__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ double2 ld_peer(const double2 *p) {
  double2 v;
  asm volatile("ld.relaxed.sys.global.v2.f64 {%0, %1}, [%2];" : "=d"(v.x), "=d"(v.y) : "l"(p) : "memory");
  return v;
}

// Waits until *flag has reached `seq` (flags only ever grow).  Gives up after
// `limit` clock cycles; the caller then raises the fault word and carries on
// without touching peer data, so a missing rank cannot hang this GPU.
__device__ __forceinline__ bool wait_flag(const unsigned *flag, unsigned seq, long long limit) {
  const long long start = clock64();
  for (;;) {
    if ((int)(ld_acquire_sys(flag) - seq) >= 0) return true;
    if (clock64() - start > limit) return false;
    __nanosleep(64);
  }
}

// Flag block layout (u32): [0, 8) ready[src rank], [8, 16) done[src rank], [16] CTA ticket.
template <int W>
__global__ void __launch_bounds__(kPeerThreads) peer_allreduce_kernel(PeerArgs a) {
  __shared__ int ok_s, last_s;
  const int tid = threadIdx.x;
  if (tid == 0) {
    ok_s = 1;
    last_s = 0;
  }
  __syncthreads();
  unsigned *mine = a.flags[a.rank];

  // Flag phase 1: tell every rank that this rank's inputs are final (they were written
  // by kernels that completed before this one started), then wait for theirs.
  if (blockIdx.x == 0 && tid < W) {
    __threadfence_system();
    st_release_sys(a.flags[tid] + a.rank, a.seq);
  }
  if (tid < W && !wait_flag(mine + tid, a.seq, a.wait_cycles)) {
    ok_s = 0;
    atomicExch(a.status, 301);
  }
  __syncthreads();

  if (ok_s) {
    // Slice of the message this rank reduces: W nearly equal parts of whole 16-byte words.
    const size_t words = a.n >> 1;
    const size_t per = (words + W - 1) / W;
    const size_t lo = min(words, per * (size_t)a.rank), hi = min(words, lo + per);
    const size_t first = (a.offset >> 1) + lo, count = hi - lo;
    const size_t stride = (size_t)gridDim.x * kPeerThreads;
    size_t i = (size_t)blockIdx.x * kPeerThreads + tid;
    // Two words per thread and iteration: 2 W loads in flight before the first add.
    for (; i + stride < count; i += 2 * stride) {
      double2 v0[W], v1[W];
#pragma unroll
      for (int q = 0; q < W; q++) {
        const double2 *src = reinterpret_cast<const double2 *>(a.data[q]) + first;
        v0[q] = ld_peer(src + i);
        v1[q] = ld_peer(src + i + stride);
      }
      double2 s0 = v0[0], s1 = v1[0];
#pragma unroll
      for (int q = 1; q < W; q++) {
        s0.x += v0[q].x; s0.y += v0[q].y;
        s1.x += v1[q].x; s1.y += v1[q].y;
      }
#pragma unroll
      for (int q = 0; q < W; q++) {
        double2 *dst = reinterpret_cast<double2 *>(a.data[q]) + first;
        dst[i] = s0;
        dst[i + stride] = s1;
      }
    }
    for (; i < count; i += stride) {
      double2 v[W];
#pragma unroll
      for (int q = 0; q < W; q++)
        v[q] = ld_peer(reinterpret_cast<const double2 *>(a.data[q]) + first + i);
      double2 s = v[0];
#pragma unroll
      for (int q = 1; q < W; q++) { s.x += v[q].x; s.y += v[q].y; }
#pragma unroll
      for (int q = 0; q < W; q++) (reinterpret_cast<double2 *>(a.data[q]) + first)[i] = s;
    }
  }

  // Flag phase 2: once every CTA of this rank has pushed its results, tell every rank,
  // and have the last CTA stay until all ranks have said the same — when this
  // kernel completes, the whole reduced message is in this rank's buffer.
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    const unsigned prev = atomicAdd(mine + 16, 1u);
    if (prev == gridDim.x - 1) {
      mine[16] = 0;  // next call on this buffer starts from zero (calls are stream-ordered)
      last_s = 1;
    }
    __threadfence_system();
  }
  __syncthreads();
  if (last_s && tid < W) {
    st_release_sys(a.flags[tid] + 8 + a.rank, a.seq);
    if (!wait_flag(mine + 8 + tid, a.seq, a.wait_cycles)) atomicExch(a.status, 302);
  }
}

// CTAs of an exchange that overlaps GEMMs.  A 512-thread CTA cannot share an SM
// with a GEMM CTA, so every CTA here is an SM the GEMMs lose for as long as the
// exchange is in flight (mostly waiting for the slowest peer).  Measured at 4 GPUs,
// whole training step: 16 CTAs 4.99 ms (median 5.03), 8 CTAs 4.95, 4 CTAs 4.92
// (median 4.92), 2 CTAs 4.92.  The one exchange nothing overlaps asks for a wide
// grid instead (the `exposed` hint).
int peer_ctas() {
  static const int v = [] {
    const char *e = std::getenv("MG_PEER_CTAS");
    int n = e && *e ? std::atoi(e) : 4;
    const int sms = ctx().sm_count > 0 ? ctx().sm_count : 1;
    return n < 1 ? 1 : (n > sms ? sms : n);
  }();
  return v;
}

bool peer_path_disabled() {
  static const bool v = [] {
    const char *e = std::getenv("MG_ALLREDUCE");
    return e && std::strcmp(e, "nccl") == 0;
  }();
  return v;
}

SharedBuffer *find_shared(const double *buf, size_t n) {
  for (auto &b : g_shared)
    if (buf >= b.base && buf + n <= b.base + b.elems) return &b;
  return nullptr;
}

// `exposed`: nothing else will be running beside this exchange (the caller is
// about to wait for it), so it may spread over most of the GPU instead of the few
// SMs an exchange that hides behind GEMMs should take from them.
template <int W>
int launch_peer_allreduce(SharedBuffer &b, size_t offset, size_t n, bool exposed) {
  Context &c = ctx();
  PeerArgs a;
  for (int q = 0; q < kMaxPeers; q++) {
    a.data[q] = q < W ? b.peer[q] : nullptr;
    a.flags[q] = q < W ? reinterpret_cast<unsigned *>(b.peer[q] + b.elems) : nullptr;
  }
  a.rank = g_rank;
  a.seq = ++b.seq;
  a.offset = offset;
  a.n = n;
  a.wait_cycles = peer_wait_cycles();
  a.status = c.kernel_status;
  const size_t words_per_rank = (n / 2 + W - 1) / W;
  size_t ctas = (words_per_rank + 2 * kPeerThreads - 1) / (2 * kPeerThreads);
  if (ctas < 1) ctas = 1;
  size_t cap = (size_t)peer_ctas();
  if (exposed) {
    const size_t wide = (size_t)(c.sm_count > 20 ? c.sm_count - 20 : c.sm_count);
    if (wide > cap) cap = wide;
  }
  if (ctas > cap) ctas = cap;
  peer_allreduce_kernel<W><<<(unsigned)ctas, kPeerThreads, 0, c.comm_stream>>>(a);
  MG_LAUNCH_CHECK("peer_allreduce");
  return MG_OK;
}

void unmap_peers(SharedBuffer &b) {
  if (!b.peers_mapped) return;
  for (int q = 0; q < g_world && q < kMaxPeers; q++)
    if (q != g_rank && b.peer[q]) cudaIpcCloseMemHandle(b.peer[q]);
  b.peers_mapped = false;
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
  // Peer mappings end with the communicator; the local allocations stay until
  // mg_comm_free_shared() and fall back to plain local buffers.
  for (auto &b : g_shared) unmap_peers(b);
  ncclResult_t r = g_nccl.CommDestroy(g_comm);
  g_comm = nullptr;
  g_rank = 0;
  g_world = 1;
  if (r != ncclSuccess) return nccl_fail(r, "ncclCommDestroy");
  return MG_OK;
}

int mg_comm_rank(void) { return g_rank; }
int mg_comm_world(void) { return g_world; }

int mg_allreduce_sum_async(double *buf, size_t n) { return mg_allreduce_sum_async_hint(buf, n, 0); }

int mg_allreduce_sum_async_hint(double *buf, size_t n, int exposed) {
  MG_ENSURE_INIT();
  MG_NOT_WHILE_RECORDING("mg_allreduce_sum_async");
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
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  if (g_trace.on && (t0 = trace_event()) && (t1 = trace_event()))
    MG_CUDA_TRY(cudaEventRecord(t0, c.comm_stream));
  int rc = MG_OK;
  bool launched = false;
  // The choice below depends only on values that are equal on every rank.
  SharedBuffer *shared = find_shared(buf, n);
  if (shared && shared->peers_mapped && !peer_path_disabled()) {
    const size_t offset = (size_t)(buf - shared->base);
    if (((offset | n) & 1) == 0) {
      launched = true;
      switch (g_world) {
        case 2: rc = launch_peer_allreduce<2>(*shared, offset, n, exposed != 0); break;
        case 4: rc = launch_peer_allreduce<4>(*shared, offset, n, exposed != 0); break;
        case 8: rc = launch_peer_allreduce<8>(*shared, offset, n, exposed != 0); break;
        default: launched = false; break;
      }
    }
  }
  if (!launched) {
    ncclResult_t r = g_nccl.AllReduce(buf, buf, n, ncclDouble, ncclSum, g_comm, c.comm_stream);
    if (r != ncclSuccess) return nccl_fail(r, "ncclAllReduce");
  }
  if (rc == MG_OK && t0 && t1) {
    MG_CUDA_TRY(cudaEventRecord(t1, c.comm_stream));
    g_trace.exchanges.emplace_back(t0, t1);
  }
  return rc;
}

int mg_comm_alloc_shared(size_t n, double **out) {
  MG_ENSURE_INIT();
  if (!out) return fail(MG_ERR_INVALID, "mg_comm_alloc_shared: null out pointer");
  *out = nullptr;
  Context &c = ctx();
  SharedBuffer b;
  b.elems = (n + 1) & ~(size_t)1;  // flag block stays 16-byte aligned
  void *p = nullptr;
  cudaError_t e = cudaMalloc(&p, b.elems * sizeof(double) + kFlagBytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(e == cudaErrorMemoryAllocation ? MG_ERR_OOM : MG_ERR_CUDA,
                "shared allocation of %zu doubles failed: %s", n, cudaGetErrorString(e));
  }
  b.base = static_cast<double *>(p);
  MG_CUDA_TRY(cudaMemsetAsync(p, 0, b.elems * sizeof(double) + kFlagBytes, c.comm_stream));
  MG_CUDA_TRY(cudaStreamSynchronize(c.comm_stream));

  // Map every peer's allocation.  The handles travel through an NCCL all-gather
  // and a final all-reduce(min) makes the outcome unanimous: either every rank
  // sees every buffer, or all of them use NCCL for this buffer.
  const bool want_peers = g_comm && (g_world == 2 || g_world == 4 || g_world == 8);
  if (want_peers) {
    struct Record {
      cudaIpcMemHandle_t handle;
      int ok;
      int pad[15];
    };
    static_assert(sizeof(Record) == 128, "handle record size");
    Record mine_rec;
    std::memset(&mine_rec, 0, sizeof(mine_rec));
    mine_rec.ok = cudaIpcGetMemHandle(&mine_rec.handle, p) == cudaSuccess ? 1 : 0;
    cudaGetLastError();
    Record *dev = nullptr;
    std::vector<Record> all((size_t)g_world);
    MG_CUDA_TRY(cudaMalloc(&dev, sizeof(Record) * (size_t)(g_world + 1)));
    MG_CUDA_TRY(cudaMemcpyAsync(dev + g_world, &mine_rec, sizeof(Record), cudaMemcpyHostToDevice,
                                c.comm_stream));
    ncclResult_t r = g_nccl.AllGather(dev + g_world, dev, sizeof(Record), ncclChar, g_comm,
                                      c.comm_stream);
    if (r != ncclSuccess) {
      cudaFree(dev);
      cudaFree(p);
      return nccl_fail(r, "ncclAllGather(handles)");
    }
    MG_CUDA_TRY(cudaMemcpyAsync(all.data(), dev, sizeof(Record) * (size_t)g_world,
                                cudaMemcpyDeviceToHost, c.comm_stream));
    MG_CUDA_TRY(cudaStreamSynchronize(c.comm_stream));
    double ok = 1.0;
    for (int q = 0; q < g_world; q++) {
      if (q == g_rank) {
        b.peer[q] = b.base;
        continue;
      }
      void *mapped = nullptr;
      if (!all[(size_t)q].ok ||
          cudaIpcOpenMemHandle(&mapped, all[(size_t)q].handle, cudaIpcMemLazyEnablePeerAccess) !=
              cudaSuccess) {
        cudaGetLastError();
        ok = 0.0;
        continue;
      }
      b.peer[q] = static_cast<double *>(mapped);
    }
    if (!mine_rec.ok) ok = 0.0;
    double *vote = reinterpret_cast<double *>(dev);
    MG_CUDA_TRY(cudaMemcpyAsync(vote, &ok, sizeof(double), cudaMemcpyHostToDevice, c.comm_stream));
    r = g_nccl.AllReduce(vote, vote, 1, ncclDouble, ncclMin, g_comm, c.comm_stream);
    if (r != ncclSuccess) {
      cudaFree(dev);
      cudaFree(p);
      return nccl_fail(r, "ncclAllReduce(vote)");
    }
    MG_CUDA_TRY(cudaMemcpyAsync(&ok, vote, sizeof(double), cudaMemcpyDeviceToHost, c.comm_stream));
    MG_CUDA_TRY(cudaStreamSynchronize(c.comm_stream));
    cudaFree(dev);
    b.peers_mapped = true;  // so that unmap_peers() closes what was opened
    if (ok < 1.0) unmap_peers(b);
  }
  g_shared.push_back(b);
  *out = b.base;
  return MG_OK;
}

int mg_comm_free_shared(double *ptr) {
  if (!ptr) return MG_OK;
  for (size_t i = 0; i < g_shared.size(); i++) {
    if (g_shared[i].base != ptr) continue;
    if (ctx().ready) {
      cudaStreamSynchronize(ctx().comm_stream);
      cudaStreamSynchronize(ctx().stream);
    }
    unmap_peers(g_shared[i]);
    cudaFree(g_shared[i].base);
    g_shared.erase(g_shared.begin() + (long)i);
    return MG_OK;
  }
  return fail(MG_ERR_INVALID, "mg_comm_free_shared: pointer was not returned by mg_comm_alloc_shared");
}

int mg_comm_peer_path(const double *ptr) {
  if (peer_path_disabled()) return 0;
  if (ptr) {
    SharedBuffer *b = find_shared(ptr, 0);
    return (b && b->peers_mapped) ? 1 : 0;
  }
  for (auto &b : g_shared)
    if (b.peers_mapped) return 1;
  return 0;
}

int mg_comm_join(void) {
  MG_ENSURE_INIT();
  MG_NOT_WHILE_RECORDING("mg_comm_join");
  Context &c = ctx();
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  if (g_trace.on && (t0 = trace_event()) && (t1 = trace_event()))
    MG_CUDA_TRY(cudaEventRecord(t0, c.stream));
  MG_CUDA_TRY(cudaEventRecord(c.join_event, c.comm_stream));
  MG_CUDA_TRY(cudaStreamWaitEvent(c.stream, c.join_event, 0));
  if (t0 && t1) {
    MG_CUDA_TRY(cudaEventRecord(t1, c.stream));
    g_trace.waits.emplace_back(t0, t1);
  }
  return MG_OK;
}

int mg_comm_trace(int enable) {
  MG_ENSURE_INIT();
  g_trace.on = enable != 0;
  return MG_OK;
}

int mg_comm_trace_summary(double *exchange_ms, int *exchanges, double *exposed_ms, int *joins) {
  MG_ENSURE_INIT();
  if (!exchange_ms || !exchanges || !exposed_ms || !joins)
    return fail(MG_ERR_INVALID, "mg_comm_trace_summary: null pointer");
  Context &c = ctx();
  MG_CUDA_TRY(cudaStreamSynchronize(c.stream));
  MG_CUDA_TRY(cudaStreamSynchronize(c.comm_stream));
  double ex = 0.0, wt = 0.0;
  for (auto &p : g_trace.exchanges) {
    float ms = 0.f;
    MG_CUDA_TRY(cudaEventElapsedTime(&ms, p.first, p.second));
    ex += ms;
  }
  for (auto &p : g_trace.waits) {
    float ms = 0.f;
    MG_CUDA_TRY(cudaEventElapsedTime(&ms, p.first, p.second));
    wt += ms;
  }
  *exchange_ms = ex;
  *exchanges = (int)g_trace.exchanges.size();
  *exposed_ms = wt;
  *joins = (int)g_trace.waits.size();
  g_trace.exchanges.clear();
  g_trace.waits.clear();
  g_trace.next = 0;
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
