// Measurement helper: issue rate of the FP64 tensor-core instruction with
// register operands only (no memory traffic), i.e. the ceiling any fp64 GEMM on
// this part can reach.  Used by the benchmark as the roofline denominator
// measured on the device it runs on.
#include "common.cuh"
#include "tma.cuh"

namespace mg {

constexpr int kProbeChains = 8;  // independent accumulator sets per warp

template <int SHAPE>
__global__ void __launch_bounds__(256)
dmma_probe_kernel(int iters, double *sink) {
  double c[kProbeChains][4];
#pragma unroll
  for (int i = 0; i < kProbeChains; i++)
#pragma unroll
    for (int r = 0; r < 4; r++) c[i][r] = 0.0;
  // Operands that depend on the thread so nothing is folded away; values stay
  // tiny so the accumulators never overflow.
  const double a = 1e-30 * (double)(threadIdx.x + 1), b = 1e-30 * (double)(blockIdx.x + 1);
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < kProbeChains; i++) {
      if (SHAPE == 0) {
        dmma_m8n8k4(c[i][0], c[i][1], a, b);
        dmma_m8n8k4(c[i][2], c[i][3], b, a);
      } else if (SHAPE == 1) {
        dmma_m16n8k4(c[i], a, b, a);
      } else if (SHAPE == 2) {
        dmma_m16n8k8(c[i], a, b, a, b, b, a);
      } else {
        dmma_m16n8k16(c[i], a, b, a, b, a, b, a, b, b, a, b, a);
      }
    }
  }
  double s = 0.0;
#pragma unroll
  for (int i = 0; i < kProbeChains; i++)
#pragma unroll
    for (int r = 0; r < 4; r++) s += c[i][r];
  if (s == 12345.678) sink[0] = s;  // never true; keeps the loop alive
}

// Synthetic inputs generated where they are used: element i of a virtual
// stream is a pure function of (seed, i), so any shard of a large input can be
// produced on its own GPU and reproduced on the host for checking.
//   z = seed + (i + 1) * 0x9E3779B97F4A7C15      (splitmix64)
//   z = (z ^ z >> 30) * 0xBF58476D1CE4E5B9 ; z = (z ^ z >> 27) * 0x94D049BB133111EB ; z ^= z >> 31
//   value = (z >> 11) * 2^-53                    in [0, 1)
__global__ void uniform01_kernel(double *__restrict__ dst, size_t n, unsigned long long seed,
                                 unsigned long long first) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    unsigned long long z = seed + (first + i + 1ull) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    dst[i] = (double)(z >> 11) * 0x1.0p-53;
  }
}

}  // namespace mg

using namespace mg;

extern "C" int mg_probe_dmma_tflops(int shape, int iters, double *tflops_host) {
  MG_ENSURE_INIT();
  if (shape < 0 || shape > 3 || iters <= 0 || !tflops_host)
    return fail(MG_ERR_INVALID, "mg_probe_dmma_tflops: bad argument");
  Context &c = ctx();
  double *sink = nullptr;
  MG_CUDA_TRY(cudaMallocAsync(&sink, sizeof(double), c.stream));
  const int ctas = c.sm_count * 4, threads = 256;
  // flop per warp-level instruction group issued per chain per iteration
  const double flop_per_chain[4] = {2.0 * 2 * 8 * 8 * 4, 2.0 * 16 * 8 * 4, 2.0 * 16 * 8 * 8,
                                    2.0 * 16 * 8 * 16};
  cudaEvent_t e0, e1;
  MG_CUDA_TRY(cudaEventCreate(&e0));
  MG_CUDA_TRY(cudaEventCreate(&e1));
  float best_ms = 1e30f;
  for (int rep = 0; rep < 4; rep++) {  // first repetition is the warm-up
    MG_CUDA_TRY(cudaEventRecord(e0, c.stream));
    switch (shape) {
      case 0: dmma_probe_kernel<0><<<ctas, threads, 0, c.stream>>>(iters, sink); break;
      case 1: dmma_probe_kernel<1><<<ctas, threads, 0, c.stream>>>(iters, sink); break;
      case 2: dmma_probe_kernel<2><<<ctas, threads, 0, c.stream>>>(iters, sink); break;
      default: dmma_probe_kernel<3><<<ctas, threads, 0, c.stream>>>(iters, sink); break;
    }
    MG_LAUNCH_CHECK("dmma_probe");
    MG_CUDA_TRY(cudaEventRecord(e1, c.stream));
    MG_CUDA_TRY(cudaEventSynchronize(e1));
    float ms = 0.f;
    MG_CUDA_TRY(cudaEventElapsedTime(&ms, e0, e1));
    if (rep > 0 && ms < best_ms) best_ms = ms;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  MG_CUDA_TRY(cudaFreeAsync(sink, c.stream));
  const double warps = (double)ctas * (threads / 32);
  const double flop = warps * (double)iters * kProbeChains * flop_per_chain[shape];
  *tflops_host = flop / ((double)best_ms * 1e-3) / 1e12;
  return MG_OK;
}

extern "C" int mg_fill_uniform01(double *dst, size_t n, unsigned long long seed,
                                 unsigned long long first_index) {
  MG_ENSURE_INIT();
  if (n == 0) return MG_OK;
  if (!dst) return mg::fail(MG_ERR_INVALID, "mg_fill_uniform01: null pointer");
  mg::uniform01_kernel<<<mg::grid_for(n, 256, 8), 256, 0, mg::ctx().stream>>>(dst, n, seed, first_index);
  MG_LAUNCH_CHECK("uniform01");
  return MG_OK;
}
