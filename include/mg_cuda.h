/*
 * mg_cuda.h — C ABI of the B200 (sm_100a) device backend for micrograd's fp64
 * tensor-op path.
 *
 * The reference project has no FFI for this path: its ops are loops inside the
 * C++ `Tensor` methods (src/ops/*.cpp, src/core/*.cpp).  This header is the
 * boundary those method bodies are replaced by.  Each entry point names the
 * reference loop it stands in for.  All pointers named `d_*`, and every
 * `double *` / `int *` argument unless marked "host", are DEVICE pointers
 * obtained from mg_alloc(); tensors are dense, row-major, fp64.
 *
 * Conventions
 *   - Every function returns MG_OK (0) or a negative MG_ERR_* code and never
 *     throws; mg_last_error() returns a thread-local description.
 *   - Work is enqueued on one ordered compute stream per process and returns
 *     without waiting; only mg_download*, mg_sync, mg_event_elapsed_ms and the
 *     bounded waits block the host.
 *   - One device per process (one process per GPU), and calls are expected from
 *     threads that have that device current (the thread that ran mg_init does;
 *     any other thread calls cudaSetDevice(mg_device()) first).  mg_init() is implicit: the
 *     first call that needs the device initialises it from MG_DEVICE, else
 *     LOCAL_RANK, else device 0.  There is no CPU fallback: without a usable
 *     CUDA device every call fails with MG_ERR_CUDA.
 *   - One context per process, as the reference keeps one MetalContext
 *     (src/metal/MetalContext.cpp:9-12).  Initialisation and shutdown are
 *     guarded by a lock; everything else (the launch counter, the scratch
 *     buffers, the cache of GEMM segment tables, the recording state) is not,
 *     so calls from several host threads must not overlap: the reference's
 *     Tensor code is single-threaded and so is the layer above this header.
 *     Several GPUs are driven by several processes, never by threads.
 *   - Backward entry points ACCUMULATE (`+=`), like the reference's closures.
 *     `flags` bit MG_ACC_STORE_A / _B says the destination gradient is known to
 *     be all zero, so the kernel may store instead of read-modify-write; the
 *     result is the same value.
 */
#ifndef MG_CUDA_H
#define MG_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MG_OK 0
#define MG_ERR_INVALID (-1) /* bad argument                                */
#define MG_ERR_OOM (-2)     /* device allocation failed                    */
#define MG_ERR_CUDA (-3)    /* CUDA runtime / driver error, or no device   */
#define MG_ERR_NCCL (-4)    /* NCCL error                                  */
#define MG_ERR_TIMEOUT (-5) /* a bounded wait expired                      */
#define MG_ERR_KERNEL (-6)  /* a kernel reported an internal fault flag    */

#define MG_ACC_STORE_A 1 /* first gradient destination is known zero  */
#define MG_ACC_STORE_B 2 /* second gradient destination is known zero */

/* ---- lifecycle -------------------------------------------------------- */
/* Role of the reference's MetalContext singleton
 * (src/metal/MetalContext.cpp:9-63): device, queue, buffers. */
const char *mg_last_error(void);
int mg_init(int device); /* device < 0: MG_DEVICE, LOCAL_RANK, then 0 */
int mg_shutdown(void);
int mg_device(void); /* current device ordinal, -1 before init */
int mg_sm_count(void);
int mg_sync(void);                 /* wait for the compute and comm streams */
int mg_check_kernel_status(void);  /* MG_ERR_KERNEL if a kernel raised its fault flag (syncs) */
/* The same fault word without a device synchronisation: mg_kernel_status_mirror()
 * enqueues, behind everything on the compute stream so far, a copy of the word to
 * pinned host memory; mg_kernel_status_peek() returns the value the most recent
 * completed copy delivered (0 before the first).  A training loop mirrors once per
 * step behind its gradient exchange and peeks at the start of the next step, so a
 * timed-out exchange is seen one step later without ever stalling the device. */
int mg_kernel_status_mirror(void);
int mg_kernel_status_peek(int *out_status);
int mg_mem_info(size_t *free_bytes, size_t *total_bytes);

/* ---- storage ----------------------------------------------------------- */
/* Replaces std::vector<double> data_/grad_ (include/micrograd/Tensor.h:55-56,
 * src/core/Tensor.cpp:7-28).  Stream-ordered: memory freed here may be handed
 * to a later mg_alloc and is safe for work enqueued after that call. */
int mg_alloc(size_t n, double **out);
int mg_free(double *p);
/* Makes sure the pool behind mg_alloc holds at least `bytes` of device memory
 * that no allocation is using (it takes one block of that size and hands it
 * straight back; freed memory stays with the pool until mg_shutdown).  No
 * counterpart in the reference.  Why it exists: when a request cannot be met
 * from memory already in the pool, the pool grows, and growing it while kernels
 * are running stalls the calling thread — measured in a two-process data-parallel
 * loop that reads a loss every step: single stalls of 16 to 740 ms in the first
 * ten steps of a new allocation pattern, none after a reserve.  Call it once,
 * before a loop that must not stall, with the loop's peak footprint plus slack. */
int mg_pool_reserve(size_t bytes);
int mg_alloc_i32(size_t n, int **out);
int mg_free_i32(int *p);
int mg_upload(double *dst, const double *src_host, size_t n);   /* pageable or pinned host */
int mg_download(double *dst_host, const double *src, size_t n); /* blocks until done */
/* Prefetch: copies on a separate copy stream, so the transfer of the next batch
 * overlaps kernels already enqueued on the compute stream.  The copy starts once
 * the compute stream has reached the point of this call (dst is then safe to
 * write) and *out_event_id completes when the data has landed.  Before the first
 * kernel that reads dst, call mg_compute_wait_event(id), then mg_event_destroy(id).
 * src_host must stay unchanged until the event completes (pinned memory makes the
 * copy asynchronous to the host). */
int mg_upload_async(double *dst, const double *src_host, size_t n, int *out_event_id);
int mg_compute_wait_event(int id); /* compute stream waits for the event, not the host */
int mg_upload_i32(int *dst, const int *src_host, size_t n);
int mg_download_i32(int *dst_host, const int *src, size_t n);
/* Byte data (image pixels) from host memory: dst[i] = (double)src_host[i] / divisor,
 * the division done on the device after an upload of n bytes instead of 8n — the
 * `pixel / 255.0` of src/mnist.cpp:21, exactly rounded like the host's.  src_host
 * may be released once the call returns only if it is pageable memory. */
int mg_upload_u8_scaled(double *dst, const unsigned char *src_host, size_t n, double divisor);
int mg_fill(double *dst, double value, size_t n); /* Tensor.cpp:12-13, 73-77; Autograd.cpp:23-25 */
int mg_copy(double *dst, const double *src, size_t n);
/* Pinned host staging memory for callers that stream batches in. */
/* One-element results (no counterpart in the reference: its values are host
 * memory already).  mg_scalar_mirror enqueues, behind everything on the compute
 * stream so far, a copy of *src to a pinned slot on a stream of its own and returns
 * a ticket; mg_scalar_fetch waits for that copy only — not for work enqueued
 * later — and returns the value.  *expired = 1 (value untouched) when the slot has
 * been reused by 256 later mirrors: read the value with mg_download then. */
int mg_scalar_mirror(const double *src, unsigned long long *out_ticket);
int mg_scalar_fetch(unsigned long long ticket, double *out, int *expired);
int mg_host_alloc(size_t bytes, void **out_host);
int mg_host_free(void *host);

/* ---- elementwise, tensor (x) tensor: src/ops/Arithmetic.cpp:9-135 ------ */
enum { MG_ADD = 0, MG_SUB = 1, MG_MUL = 2, MG_DIV = 3 };
int mg_binary_fwd(int op, const double *a, const double *b, double *out, size_t n);
/* ga/gb may be NULL (skipped) and may alias each other (x op x). */
int mg_binary_bwd(int op, const double *a, const double *b, const double *g, double *ga,
                  double *gb, size_t n, int flags);

/* ---- elementwise, tensor (x) scalar and unary -------------------------- */
/* Arithmetic.cpp:137-266 (scalar add/sub/mul/div, pow) and
 * src/ops/Activations.cpp:8-88 (relu, sigmoid, tanh).  MG_EXP has no
 * counterpart in the reference (forward exp(x), backward g*out). */
enum {
  MG_SADD = 0, MG_SSUB = 1, MG_SMUL = 2, MG_SDIV = 3, MG_POW = 4,
  MG_RELU = 5, MG_SIGMOID = 6, MG_TANH = 7, MG_EXP = 8
};
int mg_unary_fwd(int op, const double *a, double s, double *out, size_t n);
/* `a` = forward input, `out` = forward output (used by sigmoid/tanh/exp). */
int mg_unary_bwd(int op, const double *a, const double *out, double s, const double *g,
                 double *ga, size_t n, int flags);

/* ---- row broadcast (no counterpart in the reference; the batched form of
 * Linear::forward's bias add, src/nn.cpp:55-57) --------------------------- */
int mg_add_row_fwd(const double *x, const double *row, double *out, size_t M, size_t N);
/* gx[M,N] += g ; grow[N] += column sums of g.  Either may be NULL. */
int mg_add_row_bwd(const double *g, double *gx, double *grow, size_t M, size_t N, int flags);

/* Column sums of g[M,N] into out_row[N] (out_row += if accumulate != 0) — the bias
 * gradient — for callers that must not allocate device memory when they need it:
 * a latency-critical loop where an allocation would stall the device, a process
 * whose memory belongs in full to another component's pool, a host framework that
 * forbids allocation between its own synchronisation points.  This entry point has
 * no counterpart in the reference.  It calls no cudaMalloc/cudaFree and no
 * allocating library routine; the partial sums of the two-stage reduction live in
 * a fixed 1 MiB array inside the library's device image (each GPU that loads the
 * library holds it until the process exits).
 *   - mg_init() must have run earlier, at set-up time (it allocates); this entry
 *     point never initialises implicitly and fails with MG_ERR_INVALID otherwise.
 *   - The first call looks up the array's address on the device the library is
 *     bound to; make that first call before starting any stream capture.  The
 *     calling thread must have that device current (a new host thread starts on
 *     device 0): otherwise the call fails with MG_ERR_INVALID instead of creating
 *     a context on another GPU.
 *   - Limit: N <= 131072 columns (any M); more is rejected with MG_ERR_INVALID and
 *     a message naming the pooled alternative, mg_add_row_bwd(g, NULL, out_row, ..).
 *   - All calls share the one array.  Each call overwrites every partial it later
 *     reads, so stale contents never matter, but two calls that overlap on the GPU
 *     (other streams, other threads) race on it: keep calls on the library's
 *     ordered compute stream, one at a time. */
int mg_colsum_noalloc(const double *g, double *out_row, size_t M, size_t N, int accumulate);

/* ---- reductions --------------------------------------------------------- */
/* Full sum: src/ops/Reduction.cpp:17-21 (forward), :26-30 (backward, the
 * scalar g[0] is read on the device).  Fixed-shape two-level tree, so the
 * result does not depend on the run. */
int mg_sum_all_fwd(const double *x, double *out1, size_t n);
int mg_sum_all_bwd(const double *g1, double *gx, size_t n, int flags);
/* Last-axis sum [M,N] -> [M] (no counterpart in the reference). */
int mg_sum_lastaxis_fwd(const double *x, double *out, size_t M, size_t N);
int mg_sum_lastaxis_bwd(const double *g, double *gx, size_t M, size_t N, int flags);

/* ---- matmul: src/ops/Matmul.cpp ----------------------------------------- */
enum { MG_EPI_NONE = 0, MG_EPI_BIAS = 1, MG_EPI_BIAS_RELU = 2, MG_EPI_RELU_MASK = 3 };
/* Forward, Matmul.cpp:30-38: C[M,N] (+)= A[M,K] . B[K,N].
 * epilogue MG_EPI_BIAS adds bias[N] to every row, MG_EPI_BIAS_RELU also applies
 * max(.,0) (fused Linear::forward + relu). */
int mg_gemm_nn(const double *A, const double *B, double *C, size_t M, size_t N, size_t K,
               int accumulate, int epilogue, const double *bias);
/* dA, Matmul.cpp:44-50: dA[M,K] (+)= G[M,N] . B[K,N]^T.
 * epilogue MG_EPI_RELU_MASK multiplies element (i,j) by (mask_src[i,j] > 0)
 * before it is accumulated (the relu backward of Activations.cpp:25-30 fused). */
int mg_gemm_nt(const double *G, const double *B, double *dA, size_t M, size_t N, size_t K,
               int accumulate, int epilogue, const double *mask_src);
/* dB, Matmul.cpp:52-58: dB[K,N] (+)= A[M,K]^T . G[M,N]. */
int mg_gemm_tn(const double *A, const double *G, double *dB, size_t M, size_t N, size_t K,
               int accumulate);

/* Host-only view of the dispatcher's decision for an M x N output with a
 * contraction of K on a device with sm_count SMs (no device is touched; no
 * counterpart in the reference).  plan5 = {tile rows, tile columns, spans (0 =
 * whole tiles), work items, packed partial tiles}.  With spans > 0 and segments
 * != NULL, segments receives 5 ints per work item in issue order: first row,
 * first column, first k-tile (16 deep), k-tile count, partial-tile slot (-1 = the
 * segment covers its tile's whole contraction and runs the final epilogue). */
int mg_gemm_plan_describe(size_t M, size_t N, size_t K, int sm_count, int *plan5, int *segments,
                          int max_segments);
/* Diagnostic knob for tests and benchmarks.  path: 0 automatic choice, 1 plain
 * tiled kernel only, 2 tensor-core kernel whenever the operands allow it.
 * dmma_shape: -1 default, else the mma.sync f64 shape as in
 * mg_probe_dmma_tflops(). */
int mg_gemm_config(int path, int dmma_shape);

/* ---- fused loss / prediction (no counterpart in the reference) ---------- */
/* Softmax cross-entropy over rows of logits[M,C] with class ids labels[M]
 * (int).  loss1[0] = sum_i loss_i / denom; denom is the global batch size so a
 * row shard produces its share of the global mean. */
int mg_softmax_xent_fwd(const double *logits, const int *labels, double *loss1, size_t M,
                        size_t C, double denom);
/* glogits[M,C] += gloss1[0] * (softmax - onehot) / denom. */
int mg_softmax_xent_bwd(const double *logits, const int *labels, const double *gloss1,
                        double *glogits, size_t M, size_t C, double denom, int flags);
/* First index of the strict row maximum (the `>` loop of src/main.cpp:29-32). */
int mg_argmax_rows(const double *x, int *out, size_t M, size_t N);
/* labels stored as doubles -> int class ids. */
int mg_f64_to_i32(const double *src, int *dst, size_t n);

/* avg_pool_2x2, src/nn.cpp:17-35, for a batch: x[batch,784] (28x28 images) ->
 * out[batch,196]; each cell is ((a+b)+c)+d over its 2x2 window, divided by 4.0. */
int mg_avg_pool_28(const double *x, double *out, size_t batch);

/* ---- optimiser: src/nn.cpp:65-77 ----------------------------------------- */
int mg_sgd_step(double *param, const double *grad, double lr, size_t n); /* p -= (lr*g) */
/* The same update for `count` tensors (host arrays of device pointers and sizes)
 * in one launch per eight tensors; for optimisers over many small parameters. */
int mg_sgd_step_multi(double *const *params, const double *const *grads, const size_t *sizes, int count,
                      double lr);

/* ---- recorded steps (no counterpart in the reference) -------------------- */
/* A launch-bound step — the reference trainer's batch-1 loop (src/main.cpp:20-46)
 * is ~20 dependent micro-kernels per sample — can be recorded once and replayed
 * with a single launch (a CUDA graph).  Between mg_graph_begin() and
 * mg_graph_end() every kernel, fill, device copy, mg_alloc and mg_free on the
 * compute stream is recorded instead of executed.  Entry points that wait for the
 * device, use another stream or read host memory (mg_upload*, mg_download*,
 * mg_sync, mg_check_kernel_status, the mg_comm_* exchange) fail with
 * MG_ERR_INVALID while recording.  Run the step once normally first: GEMM segment
 * tables and scratch buffers are created on first use and cannot be created while
 * recording.  Buffers allocated while recording keep their addresses across
 * replays, so results can be read (mg_download) after every mg_graph_launch(). */
int mg_graph_begin(void);
int mg_graph_end(int *out_id);
int mg_graph_launch(int id);  /* enqueues the whole recorded step on the compute stream */
int mg_graph_kernels(int id); /* kernel launches the recorded step contains (0 if unknown id) */
int mg_graph_destroy(int id);

/* ---- events / timing on the compute stream ------------------------------ */
int mg_event_create(int *out_id);
int mg_event_record(int id);
int mg_event_elapsed_ms(int start_id, int stop_id, float *ms); /* syncs on stop */
int mg_event_destroy(int id);
/* Host wait with a deadline: MG_ERR_TIMEOUT if the event has not completed. */
int mg_event_wait_bounded(int id, double timeout_s);

/* ---- data-parallel communication (no counterpart in the reference) ------ */
/* One process per GPU over NVLink.  The all-reduce runs on a separate comm
 * stream, ordered after everything enqueued on the compute stream so far; the
 * compute stream does not wait for it until mg_comm_join().
 *
 * mg_allreduce_sum_async() on a range of a buffer from mg_comm_alloc_shared()
 * (even element offset and count, 2/4/8 ranks) runs this library's own kernel
 * over peer memory: rank r pulls slice r of the range from every rank, adds the
 * copies in rank order and stores the sums into every rank's buffer, so all
 * ranks hold bit-identical results.  Its waits on other ranks are bounded (about
 * ten seconds, or MG_PEER_WAIT_MS); an expired wait raises the kernel fault word (codes 301/302,
 * reported by mg_check_kernel_status()).  Any other buffer goes through
 * ncclAllReduce; MG_ALLREDUCE=nccl in the environment forces that everywhere.
 * All ranks must issue the same sequence of calls. */
int mg_comm_unique_id(char *out128_host);
int mg_comm_init(const char *id128_host, int rank, int world);
int mg_comm_destroy(void);
int mg_comm_rank(void);
int mg_comm_world(void);
int mg_allreduce_sum_async(double *buf, size_t n);
/* The same with a hint.  exposed != 0: the caller will wait for this exchange with
 * nothing left to overlap it (the last gradient message of a backward pass), so
 * the peer-memory kernel may spread over most of the SMs; exposed == 0 keeps it on
 * a few SMs so the GEMMs it overlaps lose little.  All ranks pass the same hint. */
int mg_allreduce_sum_async_hint(double *buf, size_t n, int exposed);
/* Collective over the communicator (every rank calls it, in the same order, with
 * the same n): a zero-filled device buffer of n doubles that every rank maps
 * through CUDA IPC.  If any rank cannot map any peer, every rank keeps a plain
 * local buffer and its all-reduces use NCCL.  Without a communicator the call
 * returns a plain local buffer.  Free with mg_comm_free_shared() (not mg_free). */
int mg_comm_alloc_shared(size_t n, double **out);
int mg_comm_free_shared(double *ptr);
/* 1 if all-reduces on the shared buffer containing ptr use the peer-memory
 * kernel; with ptr == NULL, 1 if any live shared buffer does. */
int mg_comm_peer_path(const double *ptr);
int mg_comm_join(void); /* compute stream waits for all all-reduces enqueued so far */
/* Timing of the exchange, off by default.  While enabled, every all-reduce is
 * bracketed by an event pair on the communication stream and every mg_comm_join()
 * by a pair on the compute stream.  mg_comm_trace_summary() waits for both
 * streams, returns the summed duration of the all-reduces and the summed time the
 * compute stream spent waiting in joins (the part of the exchange that compute
 * did not hide), with their counts, and starts a new collection. */
int mg_comm_trace(int enable);
int mg_comm_trace_summary(double *exchange_ms, int *exchanges, double *exposed_ms, int *joins);
/* Polls NCCL's async error state and the comm stream up to timeout_s; aborts
 * the communicator and returns MG_ERR_TIMEOUT / MG_ERR_NCCL on failure. */
int mg_comm_wait_bounded(double timeout_s);

/* ---- measurement helpers -------------------------------------------------- */
/* Issue-rate probe of the FP64 tensor-core instruction (mma.sync ... f64) with
 * register operands only; writes achieved TFLOP/s.  shape: 0 m8n8k4, 1 m16n8k4,
 * 2 m16n8k8, 3 m16n8k16. */
int mg_probe_dmma_tflops(int shape, int iters, double *tflops_host);
/* Synthetic uniform [0,1) inputs made on the device (no counterpart in the
 * reference, which reads its inputs from MNIST files): dst[i] is a pure function
 * of seed and first_index + i (splitmix64, top 53 bits), so a row shard of a large
 * input is generated on the GPU that uses it and the same values can be recomputed
 * on the host for checking. */
int mg_fill_uniform01(double *dst, size_t n, unsigned long long seed, unsigned long long first_index);
/* Overwrites a buffer larger than L2 so the next timed launch starts cold. */
int mg_flush_l2(void);
/* Count of kernel launches issued by this library since process start. */
unsigned long long mg_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* MG_CUDA_H */
