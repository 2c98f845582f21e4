// fp64 matrix multiply: forward C = A.B (src/ops/Matmul.cpp:30-38) and the two
// gradient products dA += G.B^T (:44-50) and dB += A^T.G (:52-58).
//
// Main kernel: FP64 tensor-core (DMMA, mma.sync ... f64) tiles fed by TMA.
//   - Eight consumer warps and one producer warp group per CTA (registers re-split
//     with setmaxnreg); a ring of stages filled by cp.async.bulk.tensor and handed
//     over through full/empty mbarriers.  Tile configurations (TileCfg): 128 x 128
//     (2 x 4 warps of 64 x 32) for the compute-bound shapes, 128 x 64 when that
//     fills the last wave of CTAs better or the contraction is a single k-tile,
//     128 x 32 and 128 x 16 for outputs at most that many columns wide, 112 x 128
//     for row counts that are multiples of 112 but not of 128.
//   - Operands land in shared memory in the 128-byte swizzle.  With the k index
//     of a 16-deep slab permuted (the same permutation for A and B, so the sum is
//     unchanged) every fragment load is free of bank conflicts: a thread reads
//     16-byte chunk c = {0,3,5,6}[t] (first half of the slab) or c^1 (second
//     half), i.e. k = 2c and 2c+1, for all three operand layouts:
//        k-contiguous tile  [row][16 k]      : one 16-byte load per fragment pair
//        mn-contiguous tile [16-col group][k][16 cols] : 8-byte loads
//   - The accumulators stay in registers (FP64 MMA has no TMEM form); the
//     epilogue adds the bias, applies ReLU or the ReLU mask, and stores or
//     accumulates 16 bytes per thread per row, all loads before the stores.  The
//     mask source tile of the input-gradient product follows the operands
//     through the TMA ring, so its copy overlaps the tile's last MMAs.
//   - When the output has too few tiles to fill 148 SMs (weight gradients: the
//     contraction runs over the batch), the (tile, k-tile) iteration space is cut
//     into one equal span per SM; a span that crosses a tile boundary becomes two
//     segments.  Every segment is one CTA; segments are issued longest first, so
//     the hardware scheduler pairs each SM's long piece with the complementary
//     short one and all SMs finish together.  A tile covered by several segments
//     is written as packed partial tiles; the segment that finishes last (a
//     ticket per tile) adds them up in k order, whatever the arrival order, and
//     runs the epilogue, so the result is reproducible and no second kernel runs.
//   - Short work items run as a persistent grid (one CTA per SM looping over
//     items, the producer prefetching across items); long ones as one item per
//     CTA under the hardware scheduler.
// Fallback kernel: a plain shared-memory tiled FMA kernel with full bounds
// checks for shapes the TMA path cannot take (odd row lengths, unaligned
// bases) and for tiny problems.
#include "common.cuh"
#include "tma.cuh"

#include <algorithm>
#include <cstdlib>
#include <type_traits>
#include <vector>

namespace mg {

constexpr int BK = 16;  // contraction depth of one stage (one 128-byte swizzle row of doubles)
constexpr int kConsumerWarps = 8;
constexpr int kProducerWarps = 4;  // one warp group; only its first lane issues copies
constexpr int kGemmThreads = (kConsumerWarps + kProducerWarps) * 32;  // 384
// Register split between the warp groups (setmaxnreg): 8*32*232 + 4*32*40 <= 64 K.
constexpr int kConsumerRegs = 232, kProducerRegs = 40;

// CTA tile = (8 / WARPS_N) x WARPS_N consumer warps, each owning MT x NT
// sub-tiles of 16 x 8 outputs.
template <int WARPS_N_, int MT_, int NT_, int STAGES_>
struct TileCfg {
  static constexpr int WARPS_N = WARPS_N_, WARPS_M = kConsumerWarps / WARPS_N_;
  static constexpr int MT = MT_, NT = NT_, STAGES = STAGES_;
  static constexpr int BM = WARPS_M * MT * 16, BN = WARPS_N * NT * 8;
  static constexpr int A_BYTES = BM * BK * 8, B_BYTES = BN * BK * 8;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // full + empty barrier per stage, plus the consumers' meeting point around the tile ticket
  static constexpr int kBarriers = 2 * STAGES + 1;
  static constexpr int SMEM_BYTES =
      STAGES * STAGE_BYTES + 1024 /* alignment slack */ + kBarriers * 8;
  // The ReLU-mask source tile of an output tile, staged through the same ring
  // after the last k-tile: BN/16 boxes of BM rows x 16 columns (128-byte rows).
  static constexpr int MASK_BOXES = BN / 16, MASK_BOX_BYTES = BM * 128;
  static constexpr int MASK_BOXES_PER_STAGE = STAGE_BYTES / MASK_BOX_BYTES;
  static constexpr int MASK_STAGES = (MASK_BOXES + MASK_BOXES_PER_STAGE - 1) / MASK_BOXES_PER_STAGE;
  static_assert(MASK_BOXES_PER_STAGE >= 1 && MASK_STAGES <= STAGES, "mask tile must fit the ring");
  static_assert(MASK_BOX_BYTES % 1024 == 0, "swizzled boxes need 1 KB alignment");
  static_assert(A_BYTES % 1024 == 0 && B_BYTES % 1024 == 0, "swizzled tiles need 1 KB alignment");
  static_assert(BM % 16 == 0 && BN % 16 == 0, "tiles are built from 16-wide TMA boxes");
};
// 128 x 128, six 32 KB stages: compute-bound shapes.
using MainCfg = TileCfg<4, 4, 4, 6>;
// 128 x 32, eight 20 KB stages: outputs at most 32 columns wide (the 10 logits).
// All eight warps split the rows, so the MMAs spread over the four SM
// sub-partitions instead of landing on the one that owns a single warp column.
using SkinnyCfg = TileCfg<1, 1, 4, 8>;
// 128 x 16, eight 18 KB stages: outputs at most 16 columns wide.  Such a problem
// streams its tall operand once and is bound by HBM only if the MMAs on padding
// columns stay below the copy time: at 32 columns the 10-logit layer spent 0.52 us
// of tensor-pipe time per k-tile against 0.37 us of copy time, at 16 it is 0.26.
using Skinny16Cfg = TileCfg<1, 1, 2, 8>;
// 128 x 64, eight 24 KB stages: used when 128 x 128 tiles would leave the last
// wave of CTAs mostly empty (e.g. 512 tiles on 148 SMs).
using HalfCfg = TileCfg<2, 2, 4, 8>;
// 112 x 128, six 30 KB stages: eight warps side by side, each 112 rows x 16
// columns.  For outputs whose row count is a multiple of 112 but not of 128
// (784 = 7 x 112, the MNIST-sized input layer's weight gradient), where 128-row
// tiles would spend an eighth of the machine on padding.
using Rows112Cfg = TileCfg<8, 7, 2, 6>;
// 128 x 112, seven 30 KB stages: the same for column counts (the gradient with
// respect to a 784-wide input): 4 x 2 warps of 32 x 56.
using Cols112Cfg = TileCfg<2, 2, 7, 7>;

struct GemmEpilogue {
  double *D;            // output [M][N]
  const double *aux;    // bias[N] or mask source [M][N]
  double *partial;      // packed partial tiles [slot][BM][BN] of split tiles, or null
  int mode;             // MG_EPI_*
  int accumulate;       // D += instead of D =
};

// Fragment pair (k = 2c, 2c+1) of the A operand for the MT row sub-tiles of a
// warp: lo = rows g, hi = rows g + 8 of each 16-row sub-tile.
template <bool KCONTIG, int MT>
__device__ __forceinline__ void load_a_frags(const uint8_t *As, int c, int g, int wm,
                                             double2 (&lo)[MT], double2 (&hi)[MT]) {
  if (KCONTIG) {
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
      const int off = (wm + mt * 16 + g) * 128 + ((c ^ g) << 4);
      lo[mt] = *reinterpret_cast<const double2 *>(As + off);
      hi[mt] = *reinterpret_cast<const double2 *>(As + off + 8 * 128);
    }
  } else {
    const int ka = 2 * c, kb = 2 * c + 1;
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
      const int base = ((wm >> 4) + mt) * 2048;
      const int mlo = g, mhi = g + 8;
      lo[mt].x = *reinterpret_cast<const double *>(
          As + base + ka * 128 + ((((mlo >> 1) ^ (ka & 7))) << 4) + (mlo & 1) * 8);
      lo[mt].y = *reinterpret_cast<const double *>(
          As + base + kb * 128 + ((((mlo >> 1) ^ (kb & 7))) << 4) + (mlo & 1) * 8);
      hi[mt].x = *reinterpret_cast<const double *>(
          As + base + ka * 128 + ((((mhi >> 1) ^ (ka & 7))) << 4) + (mhi & 1) * 8);
      hi[mt].y = *reinterpret_cast<const double *>(
          As + base + kb * 128 + ((((mhi >> 1) ^ (kb & 7))) << 4) + (mhi & 1) * 8);
    }
  }
}

// Fragment pair of the B operand for the NT column sub-tiles of a warp (column g).
template <bool KCONTIG, int NT>
__device__ __forceinline__ void load_b_frags(const uint8_t *Bs, int c, int g, int wn,
                                             double2 (&b)[NT]) {
  if (KCONTIG) {
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      const int off = (wn + nt * 8 + g) * 128 + ((c ^ g) << 4);
      b[nt] = *reinterpret_cast<const double2 *>(Bs + off);
    }
  } else {
    const int ka = 2 * c, kb = 2 * c + 1;
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      const int nl = wn + nt * 8 + g;
      const int base = (nl >> 4) * 2048, nn = nl & 15;
      b[nt].x = *reinterpret_cast<const double *>(
          Bs + base + ka * 128 + ((((nn >> 1) ^ (ka & 7))) << 4) + (nn & 1) * 8);
      b[nt].y = *reinterpret_cast<const double *>(
          Bs + base + kb * 128 + ((((nn >> 1) ^ (kb & 7))) << 4) + (nn & 1) * 8);
    }
  }
}

// One 16-deep stage of MMAs for a warp.
template <bool A_KCONTIG, bool B_KCONTIG, int SHAPE, int MT, int NT>
__device__ __forceinline__ void compute_stage(double (&acc)[MT][NT][4], const uint8_t *As,
                                              const uint8_t *Bs, int c0, int g, int wm, int wn) {
  if (SHAPE == 3) {
    double2 lo0[MT], hi0[MT], b0[NT], lo1[MT], hi1[MT], b1[NT];
    load_a_frags<A_KCONTIG, MT>(As, c0, g, wm, lo0, hi0);
    load_b_frags<B_KCONTIG, NT>(Bs, c0, g, wn, b0);
    load_a_frags<A_KCONTIG, MT>(As, c0 ^ 1, g, wm, lo1, hi1);
    load_b_frags<B_KCONTIG, NT>(Bs, c0 ^ 1, g, wn, b1);
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        dmma_m16n8k16(acc[mt][nt], lo0[mt].x, hi0[mt].x, lo0[mt].y, hi0[mt].y, lo1[mt].x, hi1[mt].x,
                      lo1[mt].y, hi1[mt].y, b0[nt].x, b0[nt].y, b1[nt].x, b1[nt].y);
      }
  } else {
#pragma unroll
    for (int slab = 0; slab < 2; slab++) {
      double2 lo[MT], hi[MT], b[NT];
      load_a_frags<A_KCONTIG, MT>(As, c0 ^ slab, g, wm, lo, hi);
      load_b_frags<B_KCONTIG, NT>(Bs, c0 ^ slab, g, wn, b);
#pragma unroll
      for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            if (SHAPE == 2) {
            dmma_m16n8k8(acc[mt][nt], lo[mt].x, hi[mt].x, lo[mt].y, hi[mt].y, b[nt].x, b[nt].y);
          } else if (SHAPE == 1) {
            dmma_m16n8k4(acc[mt][nt], lo[mt].x, hi[mt].x, b[nt].x);
            dmma_m16n8k4(acc[mt][nt], lo[mt].y, hi[mt].y, b[nt].y);
          } else {
            dmma_m8n8k4(acc[mt][nt][0], acc[mt][nt][1], lo[mt].x, b[nt].x);
            dmma_m8n8k4(acc[mt][nt][2], acc[mt][nt][3], hi[mt].x, b[nt].x);
            dmma_m8n8k4(acc[mt][nt][0], acc[mt][nt][1], lo[mt].y, b[nt].y);
            dmma_m8n8k4(acc[mt][nt][2], acc[mt][nt][3], hi[mt].y, b[nt].y);
          }
        }
    }
  }
}

// Consumer side of the stage ring: wait for a stage, run its MMAs, hand the
// stage back.  `active` is false for a warp whose whole sub-block lies outside
// the matrix (ragged border tiles): it skips the arithmetic but keeps the
// barrier protocol.  Returns false if a bounded wait gave up.
template <bool A_KCONTIG, bool B_KCONTIG, int SHAPE, class Cfg>
__device__ __forceinline__ bool consumer_loop(double (&acc)[Cfg::MT][Cfg::NT][4], const uint8_t *smem,
                                              uint64_t *full_bar, uint64_t *empty_bar, int nkt,
                                              unsigned &ring, volatile int *abort_flag, int c0, int g,
                                              int wm, int wn, int lane, bool active) {
  // `ring` counts stages consumed by this CTA since it started; it runs on across
  // the tiles a persistent CTA processes, so stage index and barrier phase follow.
  for (int it = 0; it < nkt; ++it, ++ring) {
    const unsigned s = ring % Cfg::STAGES;
    if (!mbar_wait_bounded(smem_u32(full_bar + s), (ring / Cfg::STAGES) & 1, abort_flag)) return false;
    const uint8_t *As = smem + s * Cfg::STAGE_BYTES;
    const uint8_t *Bs = As + Cfg::A_BYTES;
    if (active)
      compute_stage<A_KCONTIG, B_KCONTIG, SHAPE, Cfg::MT, Cfg::NT>(acc, As, Bs, c0, g, wm, wn);
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(empty_bar + s));
  }
  return true;
}

// SHAPE: 0 m8n8k4, 1 m16n8k4, 2 m16n8k8, 3 m16n8k16.
// EDGE: the problem has ragged tiles (M or N not a multiple of the tile); only
// then is the per-warp skipping compiled in.
// One unit of work of a launch: an output tile and a range of k-tiles.
struct WorkItem {
  int m0, n0, kt_begin, nkt;
  int slot;  // >= 0: write a packed partial tile into this slot; < 0: final epilogue
  // For a segment of a split tile: the tile's first slot, its segment count and
  // its index (which names the tile's arrival counter).
  int first_slot, count, tile;
};

// One segment of a split contraction, as laid out by the host (32 bytes).
struct SegItem {
  int m0, n0, kt_begin, nkt, slot, first_slot, count, tile;
};

// Work order without a segment table: whole tiles, numbered row-major, so the
// thin bottom border of a ragged problem comes last and its short items fill the
// tail instead of pushing full ones into an extra round.
template <class Cfg>
__device__ __forceinline__ WorkItem decode_work(int id, int tiles_n, int KT,
                                                const SegItem *__restrict__ table) {
  WorkItem w;
  if (table) {
    const int4 a = __ldg(reinterpret_cast<const int4 *>(table + id));
    w.m0 = a.x;
    w.n0 = a.y;
    w.kt_begin = a.z;
    w.nkt = a.w;
    const int4 b = __ldg(reinterpret_cast<const int4 *>(table + id) + 1);
    w.slot = b.x;
    w.first_slot = b.y;
    w.count = b.z;
    w.tile = b.w;
    return w;
  }
  const int tile_m = id / tiles_n, tile_n = id - tile_m * tiles_n;
  w.m0 = tile_m * Cfg::BM;
  w.n0 = tile_n * Cfg::BN;
  w.kt_begin = 0;
  w.nkt = KT;
  w.slot = -1;
  w.first_slot = 0;
  w.count = 0;
  w.tile = id;
  return w;
}

// PERSISTENT: the grid has at most one CTA per SM and CTA b processes work items
// b, b + gridDim.x, ...; the producer runs ahead into the next item while the
// consumers are still in the epilogue of the current one, so the pipeline fill
// of an item is hidden behind the previous item's stores.  Used for short items
// (skinny or shallow problems).  Otherwise every CTA processes exactly one item
// and the hardware scheduler balances the load; the loop below then compiles to
// straight-line code, which keeps the consumer's register budget free of spills.
// MASKED: the epilogue is the ReLU mask and its source tile is staged through the
// ring by the producer (a separate instantiation, so that the other epilogues'
// register allocation is untouched).
// FOLD: launches of a split contraction.  Every segment of a split tile stores its
// packed partial tile and then takes a ticket from the tile's arrival counter;
// the segment that arrives last adds up the tile's partial tiles in slot order
// (= k order, whatever the arrival order: the sum is reproducible) and runs the
// final epilogue itself, so no second kernel is needed and the fold of one tile
// overlaps the other CTAs' MMAs.
template <bool A_KCONTIG, bool B_KCONTIG, int SHAPE, bool EDGE, class Cfg, bool PERSISTENT, bool MASKED,
          bool FOLD>
__global__ void __launch_bounds__(kGemmThreads, 1)
dmma_gemm_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                 const __grid_constant__ CUtensorMap mapMask, GemmEpilogue ep, int M, int N, int K,
                 int tiles_n, const SegItem *__restrict__ table, int grouped_ab, int total_items,
                 unsigned int *tile_tickets, int *status) {
  constexpr int BM = Cfg::BM, BN = Cfg::BN, MT = Cfg::MT, NT = Cfg::NT;
  constexpr int kStages = Cfg::STAGES, kStageBytes = Cfg::STAGE_BYTES, kTileBytes = Cfg::A_BYTES;
  extern __shared__ uint8_t smem_raw[];
  __shared__ int abort_flag_s;
  __shared__ int fold_last_s;
  volatile int *abort_flag = &abort_flag_s;

  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                              ~static_cast<uintptr_t>(1023));
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + kStages * kStageBytes);
  uint64_t *empty_bar = full_bar + kStages;
  uint64_t *fold_bar = full_bar + 2 * kStages;  // consumer warps meet here around the tile ticket
  static_assert(2 * kStages + 1 == Cfg::kBarriers, "barrier area and its users out of step");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KT = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    abort_flag_s = 0;
    for (int s = 0; s < kStages; s++) {
      mbar_init(smem_u32(full_bar + s), 1);
      mbar_init(smem_u32(empty_bar + s), kConsumerWarps);
    }
    mbar_init(smem_u32(fold_bar), kConsumerWarps);
    mbar_fence_init();
  }
  __syncthreads();

  if (warp >= kConsumerWarps) {
    // ---------------- producer warp group: one lane drives the TMA ring ----------------
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kProducerRegs));
    if (warp == kConsumerWarps && lane == 0) {
      prefetch_tensormap(&mapA);
      prefetch_tensormap(&mapB);
      if (MASKED) prefetch_tensormap(&mapMask);
      unsigned ring = 0;  // stages issued by this CTA so far
      bool alive = true;
      int id = blockIdx.x;
      do {
        const WorkItem w = decode_work<Cfg>(id, tiles_n, KT, table);
        for (int it = 0; it < w.nkt; ++it, ++ring) {
          const unsigned s = ring % kStages;
          if (ring >= (unsigned)kStages) {
            if (!mbar_wait_bounded(smem_u32(empty_bar + s), ((ring / kStages) - 1) & 1, abort_flag)) {
              alive = false;
              break;
            }
          }
          const uint32_t bar = smem_u32(full_bar + s);
          mbar_arrive_expect_tx(bar, kStageBytes);
          const int k0 = (w.kt_begin + it) * BK;
          const uint32_t a_dst = smem_u32(smem + s * kStageBytes);
          const uint32_t b_dst = a_dst + kTileBytes;
          if (A_KCONTIG) {
            tma_load_2d(a_dst, &mapA, k0, w.m0, bar);
          } else if (grouped_ab & 1) {
            tma_load_3d(a_dst, &mapA, 0, k0, w.m0 >> 4, bar);  // all 16-column groups in one copy
          } else {
            for (int b = 0; b < BM / 16; b++)
              tma_load_2d(a_dst + b * 2048, &mapA, w.m0 + 16 * b, k0, bar);
          }
          if (B_KCONTIG) {
            tma_load_2d(b_dst, &mapB, k0, w.n0, bar);
          } else if (grouped_ab & 2) {
            tma_load_3d(b_dst, &mapB, 0, k0, w.n0 >> 4, bar);
          } else {
            for (int b = 0; b < BN / 16; b++)
              tma_load_2d(b_dst + b * 2048, &mapB, w.n0 + 16 * b, k0, bar);
          }
        }
        // The mask source of this tile follows its operands through the ring: the
        // copies overlap the tile's last MMAs and the epilogue reads shared memory.
        if (MASKED && w.slot < 0 && alive) {
          for (int ms = 0; ms < Cfg::MASK_STAGES; ++ms, ++ring) {
            const unsigned s = ring % kStages;
            if (ring >= (unsigned)kStages) {
              if (!mbar_wait_bounded(smem_u32(empty_bar + s), ((ring / kStages) - 1) & 1, abort_flag)) {
                alive = false;
                break;
              }
            }
            const uint32_t bar = smem_u32(full_bar + s);
            const int first = ms * Cfg::MASK_BOXES_PER_STAGE;
            const int boxes = min(Cfg::MASK_BOXES_PER_STAGE, Cfg::MASK_BOXES - first);
            mbar_arrive_expect_tx(bar, (uint32_t)(boxes * Cfg::MASK_BOX_BYTES));
            const uint32_t dst = smem_u32(smem + s * kStageBytes);
            for (int b = 0; b < boxes; b++)
              tma_load_2d(dst + b * Cfg::MASK_BOX_BYTES, &mapMask, w.n0 + 16 * (first + b), w.m0, bar);
          }
        }
        if (!PERSISTENT) break;
        id += gridDim.x;
      } while (alive && id < total_items);
    }
  } else {
    // ---------------- consumer warp groups ----------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kConsumerRegs));
    const int g = lane >> 2, t = lane & 3;
    const int wm = (warp / Cfg::WARPS_N) * (MT * 16), wn = (warp % Cfg::WARPS_N) * (NT * 8);
    // 16-byte chunk owned by this thread in the first half-slab; the second
    // half-slab uses chunk ^ 1.
    const int c0 = (t << 1) | (__popc(t) & 1);
    unsigned ring = 0;  // stages consumed by this CTA so far
    unsigned fold_phase = 0;  // uses of fold_bar so far

    int id = blockIdx.x;
    do {
      const WorkItem w = decode_work<Cfg>(id, tiles_n, KT, table);
      const int m0 = w.m0, n0 = w.n0;

      double acc[MT][NT][4];
#pragma unroll
      for (int i = 0; i < MT; i++)
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
          for (int r = 0; r < 4; r++) acc[i][j][r] = 0.0;

      // Ragged border tiles: a warp whose whole sub-block lies outside the matrix
      // does no arithmetic.  (Skipping at the granularity of single MMAs was
      // measured to be slower than issuing them: the guards break up the
      // instruction stream.)  Out-of-range rows and columns of a live warp read
      // zeros from the TMA fill and are dropped in the epilogue.
      const bool active = !EDGE || (M > m0 + wm && N > n0 + wn);
      const bool ok = consumer_loop<A_KCONTIG, B_KCONTIG, SHAPE, Cfg>(
          acc, smem, full_bar, empty_bar, w.nkt, ring, abort_flag, c0, g, wm, wn, lane, active);
      if (!ok) break;
      // Mask source staged by the producer: wait for all of its stages (every warp,
      // also an inactive one, keeps the ring's barrier protocol).
      const bool mask_smem = MASKED && w.slot < 0;
      const unsigned mask_ring = ring;
      bool mask_ok = true;
      if (mask_smem) {
        for (int ms = 0; ms < Cfg::MASK_STAGES && mask_ok; ms++) {
          const unsigned r2 = mask_ring + ms;
          mask_ok = mbar_wait_bounded(smem_u32(full_bar + r2 % kStages), (r2 / kStages) & 1, abort_flag);
        }
        if (!mask_ok) break;
      }
      // ---------------- epilogue ----------------
      // A segment of a split tile stores its whole BM x BN accumulator, packed,
      // into its slot of the scratch buffer (rows and columns beyond the matrix
      // hold zeros or are never read).
      bool finalize = w.slot < 0;
      if (w.slot >= 0) {
        if (active) {
          double *slot = ep.partial + (size_t)w.slot * (size_t)(BM * BN);
#pragma unroll
          for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
              for (int nt = 0; nt < NT; nt++)
                *reinterpret_cast<double2 *>(slot + (wm + mt * 16 + g + 8 * h) * BN + wn + nt * 8 + 2 * t) =
                    make_double2(acc[mt][nt][2 * h], acc[mt][nt][2 * h + 1]);
        }
        if (FOLD) {
          // All consumer warps' stores are fenced before one thread takes the
          // tile's ticket; the meeting point is an mbarrier with a bounded wait, so
          // a warp that gave up earlier cannot strand the others.
          __threadfence();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(fold_bar));
          if (!mbar_wait_bounded(smem_u32(fold_bar), fold_phase++ & 1, abort_flag)) break;
          if (warp == 0 && lane == 0) {
            const unsigned prev = atomicAdd(tile_tickets + w.tile, 1u);
            const bool last = prev == (unsigned)w.count - 1u;
            if (last) tile_tickets[w.tile] = 0u;  // ready for the next launch (stream-ordered)
            fold_last_s = last ? 1 : 0;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(fold_bar));
          if (!mbar_wait_bounded(smem_u32(fold_bar), fold_phase++ & 1, abort_flag)) break;
          if (fold_last_s) {
            __threadfence();
            if (active) {
#pragma unroll
              for (int i = 0; i < MT; i++)
#pragma unroll
                for (int j = 0; j < NT; j++)
#pragma unroll
                  for (int r = 0; r < 4; r++) acc[i][j][r] = 0.0;
              for (int k = 0; k < w.count; k++) {
                const double *part = ep.partial + (size_t)(w.first_slot + k) * (size_t)(BM * BN);
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
#pragma unroll
                  for (int h = 0; h < 2; h++)
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                      const double2 v = __ldcg(reinterpret_cast<const double2 *>(
                          part + (wm + mt * 16 + g + 8 * h) * BN + wn + nt * 8 + 2 * t));
                      acc[mt][nt][2 * h] += v.x;
                      acc[mt][nt][2 * h + 1] += v.y;
                    }
              }
            }
            finalize = true;
          }
        }
      }
      // Final epilogue.  Per 16-row sub-tile: first every global load the epilogue
      // needs (ReLU mask source, old values for accumulation) is issued, then the
      // arithmetic, then the stores.  Interleaving load/store pairs would serialise
      // them (a store may alias the next load as far as the compiler can tell) and
      // turn the epilogue into a chain of exposed memory latencies.
      if (active && finalize) {
      {
      double *dst = ep.D;
      const bool use_mask = ep.mode == MG_EPI_RELU_MASK;
      const bool use_bias = !MASKED && (ep.mode == MG_EPI_BIAS || ep.mode == MG_EPI_BIAS_RELU);
      const bool use_old = ep.accumulate != 0;
      double2 bias[NT];
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        const int col = n0 + wn + nt * 8 + 2 * t;
        bias[nt] = make_double2(0.0, 0.0);
        if (use_bias && col < N) bias[nt] = make_double2(__ldg(ep.aux + col), __ldg(ep.aux + col + 1));
      }
      // Small accumulators (128 x 64 tiles and narrower) leave room to fetch the
      // mask / old values of the whole tile at once: twice the loads in flight,
      // which is what a one-k-tile problem (the gradient through the 10 logits)
      // lives on.  Larger ones go 16 rows at a time.
      constexpr int EG = (MT * NT <= 8) ? MT : 1;
#pragma unroll
      for (int mt0 = 0; mt0 < MT; mt0 += EG) {
        double2 mask[EG][2][NT], old[EG][2][NT];
        if (use_mask || use_old) {
#pragma unroll
          for (int e = 0; e < EG; e++) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
              const int row = m0 + wm + (mt0 + e) * 16 + g + 8 * h;
#pragma unroll
              for (int nt = 0; nt < NT; nt++) {
                const int col = n0 + wn + nt * 8 + 2 * t;
                const bool in = row < M && col < N;
                const size_t at = (size_t)row * (size_t)N + (size_t)col;
                if (mask_smem) {
                  // box = 16-column group of the tile, 128-byte rows, 16-byte chunks
                  // XOR-swizzled with the row; out-of-range elements were zero-filled.
                  const int r = row - m0, cc = col - n0, box = cc >> 4, chunk = (cc & 15) >> 1;
                  const unsigned st = (mask_ring + box / Cfg::MASK_BOXES_PER_STAGE) % kStages;
                  mask[e][h][nt] = *reinterpret_cast<const double2 *>(
                      smem + st * kStageBytes + (box % Cfg::MASK_BOXES_PER_STAGE) * Cfg::MASK_BOX_BYTES +
                      r * 128 + ((chunk ^ (r & 7)) << 4));
                } else {
                  mask[e][h][nt] = (use_mask && in)
                                       ? __ldcs(reinterpret_cast<const double2 *>(ep.aux + at))
                                       : make_double2(0.0, 0.0);
                }
                old[e][h][nt] = (use_old && in) ? __ldcs(reinterpret_cast<const double2 *>(ep.D + at))
                                                : make_double2(0.0, 0.0);
              }
            }
          }
        }
#pragma unroll
        for (int e = 0; e < EG; e++) {
          const int mt = mt0 + e;
#pragma unroll
          for (int h = 0; h < 2; h++) {
            const int row = m0 + wm + mt * 16 + g + 8 * h;
            if (row >= M) continue;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
              const int col = n0 + wn + nt * 8 + 2 * t;
              if (col >= N) continue;
              const size_t at = (size_t)row * (size_t)N + (size_t)col;
              double2 v = make_double2(acc[mt][nt][2 * h], acc[mt][nt][2 * h + 1]);
              if (use_bias) {
                v.x += bias[nt].x;
                v.y += bias[nt].y;
                if (ep.mode == MG_EPI_BIAS_RELU) {
                  v.x = v.x > 0 ? v.x : 0.0;
                  v.y = v.y > 0 ? v.y : 0.0;
                }
              }
              if (use_mask) {
                v.x = v.x * (mask[e][h][nt].x > 0 ? 1.0 : 0.0);
                v.y = v.y * (mask[e][h][nt].y > 0 ? 1.0 : 0.0);
              }
              if (use_old) {
                v.x = old[e][h][nt].x + v.x;
                v.y = old[e][h][nt].y + v.y;
              }
              *reinterpret_cast<double2 *>(dst + at) = v;
            }
          }
        }
      }
      }  // final epilogue
      }  // active
      if (mask_smem) {
        __syncwarp();
        if (lane == 0)
          for (int ms = 0; ms < Cfg::MASK_STAGES; ms++)
            mbar_arrive(smem_u32(empty_bar + (mask_ring + ms) % kStages));
        ring += Cfg::MASK_STAGES;
      }
      if (!PERSISTENT) break;
      id += gridDim.x;
    } while (id < total_items);
  }

  // A bounded wait gave up somewhere in this CTA: raise the fault word, give the
  // copies still in flight time to land in this CTA's shared memory, then leave.
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(status, 201);
    const long long start = clock64();
    while (clock64() - start < 2000000ll) {
    }
  }
}

// ---------------------------------------------------------------------------
// Fallback: D[m,n] (+)= sum_k A(m,k) B(k,n) with arbitrary element strides.
// 64 x 64 x 16 tiles, 256 threads, 4 x 4 outputs per thread, full bounds checks.
// ---------------------------------------------------------------------------
struct StridedOperands {
  const double *A;
  const double *B;
  long long sAm, sAk, sBk, sBn;
};

__global__ void __launch_bounds__(256)
gemm_fallback_kernel(StridedOperands op, GemmEpilogue ep, int M, int N, int K) {
  constexpr int TM = 64, TN = 64, TK = 16;
  __shared__ double As[TK][TM + 1];
  __shared__ double Bs[TK][TN + 1];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int ty = tid / 16, tx = tid % 16;  // thread owns rows ty*4.., cols tx*4..
  double acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.0;

  const bool a_k_fast = (op.sAk == 1);
  const bool b_n_fast = (op.sBn == 1);
  for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const int idx = tid + e * 256;  // 0..1023
      int m, k;
      if (a_k_fast) { m = idx / TK; k = idx % TK; } else { m = idx % TM; k = idx / TM; }
      const int gm = m0 + m, gk = k0 + k;
      As[k][m] = (gm < M && gk < K) ? op.A[(long long)gm * op.sAm + (long long)gk * op.sAk] : 0.0;
      int n, kk;
      if (b_n_fast) { n = idx % TN; kk = idx / TN; } else { n = idx / TK; kk = idx % TK; }
      const int gn = n0 + n, gk2 = k0 + kk;
      Bs[kk][n] = (gn < N && gk2 < K) ? op.B[(long long)gk2 * op.sBk + (long long)gn * op.sBn] : 0.0;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; k++) {
      double a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fma(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int row = m0 + ty * 4 + i;
    if (row >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int col = n0 + tx * 4 + j;
      if (col >= N) continue;
      const size_t at = (size_t)row * (size_t)N + (size_t)col;
      double v = acc[i][j];
      if (ep.mode == MG_EPI_BIAS || ep.mode == MG_EPI_BIAS_RELU) {
        v += ep.aux[col];
        if (ep.mode == MG_EPI_BIAS_RELU) v = v > 0 ? v : 0.0;
      } else if (ep.mode == MG_EPI_RELU_MASK) {
        v = v * (ep.aux[at] > 0 ? 1.0 : 0.0);
      }
      if (ep.accumulate) v = ep.D[at] + v;
      ep.D[at] = v;
    }
  }
}

// ---------------------------------------------------------------------------
// Host dispatch
// ---------------------------------------------------------------------------
struct GemmDesc {
  const double *A;  // a_kcontig ? [M][K] : [K][M]
  const double *B;  // b_kcontig ? [N][K] : [K][N]
  double *D;        // [M][N]
  size_t M, N, K;
  bool a_kcontig, b_kcontig;
  int accumulate, mode;
  const double *aux;
};

static int g_gemm_path = 0;    // 0 auto, 1 fallback only, 2 tensor-core whenever eligible
static int g_dmma_shape = -1;  // -1: default

static int default_dmma_shape() {
  const char *v = std::getenv("MG_DMMA_SHAPE");
  if (v && *v) {
    int s = std::atoi(v);
    if (s >= 0 && s <= 3) return s;
  }
  return 2;
}

struct DmmaLaunch {
  CUtensorMap ma, mb, mmask;
  int mask_tma;  // mmask describes the ReLU-mask source; the producer stages it
  GemmEpilogue ep;
  int M, N, K, tiles_m, tiles_n;
  const SegItem *table;  // segments of a split contraction (device), or null: whole tiles
  unsigned int *tickets;  // arrival counters of the split tiles: fold in the kernel; null: no fold
  int items;             // CTAs' worth of work: segments, or tiles
  int min_nkt;           // shortest item, in k-tiles
  int grouped_ab;  // bit 0 / bit 1: operand A / B uses the grouped 3-D tensor map
};


template <bool AK, bool BK_, int SHAPE, bool EDGE, class Cfg, bool PERSISTENT, bool MASKED, bool FOLD>
static int launch_dmma_masked(const DmmaLaunch &L) {
  static bool configured = false;
  auto kernel = dmma_gemm_kernel<AK, BK_, SHAPE, EDGE, Cfg, PERSISTENT, MASKED, FOLD>;
  if (!configured) {
    MG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     Cfg::SMEM_BYTES));
    configured = true;
  }
  Context &c = ctx();
  // Long items (many k-tiles) are left to the hardware scheduler, one item per
  // CTA: it balances them dynamically.  Short items (skinny or shallow problems)
  // run as a persistent grid, where the cross-item prefetch hides the pipeline
  // fill that would otherwise dominate them.
  dim3 grid((unsigned)((PERSISTENT && L.items > c.sm_count) ? c.sm_count : L.items), 1, 1);
  kernel<<<grid, kGemmThreads, Cfg::SMEM_BYTES, c.stream>>>(L.ma, L.mb, L.mmask, L.ep, L.M, L.N, L.K,
                                                             L.tiles_n, L.table, L.grouped_ab,
                                                             L.items, L.tickets, c.kernel_status);
  MG_LAUNCH_CHECK("dmma_gemm");
  return MG_OK;
}

// The staged-mask instantiation exists for the default mma shape and the layout
// of the input-gradient product (both operands k-contiguous), its only user.
template <bool AK, bool BK_, int SHAPE, bool EDGE, class Cfg, bool PERSISTENT>
static int launch_dmma_variant(const DmmaLaunch &L) {
  if constexpr (AK && BK_ && SHAPE == 2) {
    if (L.mask_tma) return launch_dmma_masked<AK, BK_, SHAPE, EDGE, Cfg, PERSISTENT, true, false>(L);
  }
  // The folding instantiation serves split contractions only: they never run
  // persistently and read their mask (if any) with plain loads.
  if constexpr (!PERSISTENT) {
    if (L.tickets) return launch_dmma_masked<AK, BK_, SHAPE, EDGE, Cfg, false, false, true>(L);
  }
  return launch_dmma_masked<AK, BK_, SHAPE, EDGE, Cfg, PERSISTENT, false, false>(L);
}

template <bool AK, bool BK_, int SHAPE, bool EDGE, class Cfg>
static int launch_dmma_kernel(const DmmaLaunch &L) {
  static const int persist_mode = [] {
    const char *v = std::getenv("MG_GEMM_PERSIST");  // diagnostic: 0 never, 1 always
    return v && *v ? std::atoi(v) : -1;
  }();
  // Segments of a split contraction have unequal lengths and rely on the
  // hardware scheduler's longest-first pairing, so they never run persistently.
  bool persistent = !L.table && (L.min_nkt < 32 || Cfg::BN <= 32) && L.items > ctx().sm_count;
  if (persist_mode == 0) persistent = false;
  if (persist_mode == 1 && !L.table && L.items > ctx().sm_count) persistent = true;
  if (persistent) return launch_dmma_variant<AK, BK_, SHAPE, EDGE, Cfg, true>(L);
  return launch_dmma_variant<AK, BK_, SHAPE, EDGE, Cfg, false>(L);
}

// One launch over all tiles; problems with a ragged border use the instantiation
// that can skip out-of-range sub-tiles.
template <bool AK, bool BK_, int SHAPE, class Cfg>
static int launch_tiles(const DmmaLaunch &L) {
  if ((L.M % Cfg::BM) != 0 || (L.N % Cfg::BN) != 0)
    return launch_dmma_kernel<AK, BK_, SHAPE, true, Cfg>(L);
  return launch_dmma_kernel<AK, BK_, SHAPE, false, Cfg>(L);
}

enum TileChoice {
  kTileMain = 0, kTileSkinny = 1, kTileHalf = 2, kTileRows112 = 3, kTileSkinny16 = 4, kTileCols112 = 5
};

template <bool AK, bool BK_>
static int launch_layout(int shape, int tile, const DmmaLaunch &L) {
  // The narrow and half-width configurations exist for the default mma shape only.
  if (tile == kTileSkinny)
    return launch_dmma_kernel<AK, BK_, 2, true, SkinnyCfg>(L);
  if (tile == kTileSkinny16)
    return launch_dmma_kernel<AK, BK_, 2, true, Skinny16Cfg>(L);
  if (tile == kTileHalf) return launch_tiles<AK, BK_, 2, HalfCfg>(L);
  if (tile == kTileRows112) return launch_tiles<AK, BK_, 2, Rows112Cfg>(L);
  if (tile == kTileCols112) return launch_tiles<AK, BK_, 2, Cols112Cfg>(L);
  switch (shape) {
    case 0: return launch_tiles<AK, BK_, 0, MainCfg>(L);
    case 1: return launch_tiles<AK, BK_, 1, MainCfg>(L);
    case 3: return launch_tiles<AK, BK_, 3, MainCfg>(L);
    default: return launch_tiles<AK, BK_, 2, MainCfg>(L);
  }
}

// Number of equal spans the (tile, k-tile) iteration space of a problem is cut
// into, or 0 to run whole tiles.  Whole tiles are kept when they already fill
// at least 95% of their last wave of CTAs, or when the contraction is too short
// to share; otherwise one span per SM, at least 16 k-tiles long.
static int choose_spans(int tiles, int KT, int sms) {
  if (tiles >= 4 * sms || KT < 32) return 0;
  const int waves = (tiles + sms - 1) / sms;
  if ((double)tiles / ((double)waves * sms) >= 0.95) return 0;
  long long spans = (long long)tiles * KT / 16;
  if (spans > sms) spans = sms;
  return spans > 1 ? (int)spans : 0;
}

// Tile configuration and contraction split for a problem.  Candidates are
// costed as (rounds of CTAs) x (work per CTA), with a small handicap for the
// half-width tile (more operand traffic per flop) and for a split contraction
// (its partial tiles are written and folded: ~22.8 (p+1)/K of the GEMM's time
// when p partial tiles are written per output tile).
struct GemmPlan {
  int tile, bm, bn, spans;
};

static GemmPlan choose_plan(int M, int N, int K, int sms, int shape) {
  const int KT = (K + BK - 1) / BK;
  auto tiles_of = [&](int bm, int bn) { return ((M + bm - 1) / bm) * ((N + bn - 1) / bn); };
  if (N <= Skinny16Cfg::BN) {
    return {kTileSkinny16, Skinny16Cfg::BM, Skinny16Cfg::BN,
            choose_spans(tiles_of(Skinny16Cfg::BM, Skinny16Cfg::BN), KT, sms)};
  }
  if (N <= SkinnyCfg::BN) {
    return {kTileSkinny, SkinnyCfg::BM, SkinnyCfg::BN,
            choose_spans(tiles_of(SkinnyCfg::BM, SkinnyCfg::BN), KT, sms)};
  }
  GemmPlan main_plan{kTileMain, MainCfg::BM, MainCfg::BN,
                     choose_spans(tiles_of(MainCfg::BM, MainCfg::BN), KT, sms)};
  static const int forced = [] {
    const char *v = std::getenv("MG_GEMM_TILE");  // diagnostic: "main" or "half"
    if (!v) return -1;
    return v[0] == 'h' ? (int)kTileHalf : (v[0] == 'm' ? (int)kTileMain : -1);
  }();
  if (shape != 2 || forced == kTileMain) return main_plan;
  GemmPlan half_plan{kTileHalf, HalfCfg::BM, HalfCfg::BN,
                     choose_spans(tiles_of(HalfCfg::BM, HalfCfg::BN), KT, sms)};
  if (forced == kTileHalf) return half_plan;
  // One k-tile: the problem is all epilogue (a rank-16 update streamed through
  // HBM); the half-width tile keeps the whole tile's epilogue loads in flight.
  if (KT == 1) return half_plan;
  // Every CTA also pays about 3.3 us of launch, pipeline fill and epilogue that
  // nothing overlaps: 25 800 in the cost's units (bm x bn x k-tiles).
  constexpr double kPerCta = 25800.0;
  auto cost = [&](const GemmPlan &p, double handicap) {
    const int tiles = tiles_of(p.bm, p.bn);
    if (p.spans == 0) {
      const int waves = (tiles + sms - 1) / sms;
      return (double)waves * ((double)p.bm * p.bn * KT * handicap + kPerCta);
    }
    const double per_cta = (double)tiles * KT / p.spans;
    const double segments = (double)tiles / p.spans + 1.0;
    const double partials = std::min(2.0 * p.spans, (double)p.spans + tiles) / tiles;
    double c = (per_cta * p.bm * p.bn * handicap + segments * kPerCta) *
               (1.0 + 22.8 * (partials + 1.0) / (double)K);
    // With more tiles than SMs most segments are whole tiles and the cut ones
    // lose the L2 sharing of a wave that walks k in step: measured 2 % behind
    // the half-width tile where the model calls it even.
    if (tiles >= sms) c *= 1.04;
    return c;
  };
  GemmPlan best = cost(half_plan, 1.04) < cost(main_plan, 1.0) ? half_plan : main_plan;
  double best_cost = best.tile == kTileHalf ? cost(half_plan, 1.04) : cost(main_plan, 1.0);
  if (M % MainCfg::BM != 0 && M % Rows112Cfg::BM == 0) {
    GemmPlan p112{kTileRows112, Rows112Cfg::BM, Rows112Cfg::BN,
                  choose_spans(tiles_of(Rows112Cfg::BM, Rows112Cfg::BN), KT, sms)};
    if (cost(p112, 1.02) < best_cost) {
      best = p112;
      best_cost = cost(p112, 1.02);
    }
  }
  if (N % MainCfg::BN != 0 && N % Cols112Cfg::BN == 0) {
    GemmPlan c112{kTileCols112, Cols112Cfg::BM, Cols112Cfg::BN,
                  choose_spans(tiles_of(Cols112Cfg::BM, Cols112Cfg::BN), KT, sms)};
    if (cost(c112, 1.02) < best_cost) best = c112;
  }
  return best;
}

// ---------------------------------------------------------------------------
// Segment tables of split contractions.  A table depends only on the tile grid,
// the k-tile count and the span count, so it is built once per shape and kept
// on the device until shutdown.
// ---------------------------------------------------------------------------
struct SegTable {
  int tiles_m, tiles_n, KT, bm, bn, spans;  // key
  int items, slots, min_nkt;
  SegItem *dev_items;  // [items], longest first
  unsigned int *dev_tickets;  // [tiles]: arrival counters of the in-kernel fold, zero between launches
};

static std::vector<SegTable> g_seg_tables;

void gemm_release_tables() {
  for (auto &t : g_seg_tables) {
    cudaFree(t.dev_items);
    cudaFree(t.dev_tickets);
  }
  g_seg_tables.clear();
}

// After a kernel fault (a bounded wait gave up) a split tile may be left with a
// partly counted ticket; clear them all so later launches start clean.
void gemm_reset_tickets() {
  for (auto &t : g_seg_tables)
    cudaMemsetAsync(t.dev_tickets, 0, sizeof(unsigned int) * (size_t)(t.tiles_m * t.tiles_n), ctx().stream);
}

// Host-only construction of a segment table: `segs` in issue order (longest
// first), `tile_info[t]` = (first slot, segment count) of every tile covered by
// more than one segment, (0, 0) otherwise.  Slots number the segments of split
// tiles in (tile, k) order, so a tile's partial tiles are consecutive and in k order.
static void build_segments(int tiles_m, int tiles_n, int KT, int bm, int bn, int spans,
                           std::vector<SegItem> &segs, std::vector<int2> &tile_info, int &slots,
                           int &min_nkt) {
  const int tiles = tiles_m * tiles_n;
  const long long units = (long long)tiles * KT;
  segs.clear();
  std::vector<int> per_tile((size_t)tiles, 0);
  for (int j = 0; j < spans; j++) {
    long long u = units * j / spans;
    const long long end = units * (j + 1) / spans;
    while (u < end) {
      const int tile = (int)(u / KT);
      const int kt = (int)(u - (long long)tile * KT);
      const int n = (int)std::min<long long>(end - u, KT - kt);
      SegItem it{};
      it.m0 = (tile / tiles_n) * bm;
      it.n0 = (tile % tiles_n) * bn;
      it.kt_begin = kt;
      it.nkt = n;
      it.slot = tile;  // provisional: the tile index
      segs.push_back(it);
      per_tile[(size_t)tile]++;
      u += n;
    }
  }
  tile_info.assign((size_t)tiles, make_int2(0, 0));
  slots = 0;
  min_nkt = KT;
  for (auto &it : segs) {
    const int tile = it.slot;
    it.tile = tile;
    if (per_tile[(size_t)tile] > 1) {
      if (tile_info[(size_t)tile].y == 0) tile_info[(size_t)tile].x = slots;
      tile_info[(size_t)tile].y++;
      it.slot = slots++;
    } else {
      it.slot = -1;
    }
    min_nkt = std::min(min_nkt, it.nkt);
  }
  for (auto &it : segs) {
    it.first_slot = tile_info[(size_t)it.tile].x;
    it.count = tile_info[(size_t)it.tile].y;
  }
  std::stable_sort(segs.begin(), segs.end(),
                   [](const SegItem &a, const SegItem &b) { return a.nkt > b.nkt; });
}

static int seg_table_for(int tiles_m, int tiles_n, int KT, int bm, int bn, int spans,
                         const SegTable **out) {
  for (const auto &t : g_seg_tables) {
    if (t.tiles_m == tiles_m && t.tiles_n == tiles_n && t.KT == KT && t.bm == bm && t.bn == bn &&
        t.spans == spans) {
      *out = &t;
      return MG_OK;
    }
  }
  if (ctx().capturing)
    return fail(MG_ERR_INVALID,
                "a GEMM of a new shape needs its segment table built while a step is being recorded; "
                "run the step once before mg_graph_begin()");
  // A job with ever-changing shapes (e.g. a varying batch) would grow the cache
  // without bound: start over beyond 256 tables (cudaFree waits for the kernels
  // that still read them).
  if (g_seg_tables.size() >= 256) gemm_release_tables();
  std::vector<SegItem> segs;
  std::vector<int2> tile_info;
  int slots = 0, min_nkt = KT;
  build_segments(tiles_m, tiles_n, KT, bm, bn, spans, segs, tile_info, slots, min_nkt);
  SegTable t{};
  t.tiles_m = tiles_m; t.tiles_n = tiles_n; t.KT = KT; t.bm = bm; t.bn = bn; t.spans = spans;
  t.items = (int)segs.size();
  t.slots = slots;
  t.min_nkt = min_nkt;
  MG_CUDA_TRY(cudaMalloc(&t.dev_items, segs.size() * sizeof(SegItem)));
  MG_CUDA_TRY(cudaMalloc(&t.dev_tickets, tile_info.size() * sizeof(unsigned int)));
  MG_CUDA_TRY(cudaMemset(t.dev_tickets, 0, tile_info.size() * sizeof(unsigned int)));
  MG_CUDA_TRY(cudaMemcpy(t.dev_items, segs.data(), segs.size() * sizeof(SegItem),
                         cudaMemcpyHostToDevice));
  g_seg_tables.push_back(t);
  *out = &g_seg_tables.back();
  return MG_OK;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static bool dmma_eligible(const GemmDesc &d) {
  const size_t a_row = d.a_kcontig ? d.K : d.M;
  const size_t b_row = d.b_kcontig ? d.K : d.N;
  if ((a_row | b_row | d.N) & 1) return false;
  if (!aligned16(d.A) || !aligned16(d.B) || !aligned16(d.D)) return false;
  if (d.mode == MG_EPI_RELU_MASK && !aligned16(d.aux)) return false;
  const size_t lim = (size_t)1 << 30;
  if (d.M >= lim || d.N >= lim || d.K >= lim) return false;
  return true;
}

static int run_gemm(const GemmDesc &d) {
  if (d.M == 0 || d.N == 0) return MG_OK;
  Context &c = ctx();
  GemmEpilogue ep;
  ep.D = d.D;
  ep.aux = d.aux;
  ep.partial = nullptr;
  ep.mode = d.mode;
  ep.accumulate = d.accumulate;
  if ((d.mode == MG_EPI_BIAS || d.mode == MG_EPI_BIAS_RELU || d.mode == MG_EPI_RELU_MASK) && !d.aux)
    return fail(MG_ERR_INVALID, "gemm: epilogue %d needs its auxiliary operand", d.mode);
  if (d.K == 0) {
    // Empty contraction: the product is all zeros; only the epilogue remains.
    if (d.accumulate && d.mode == MG_EPI_NONE) return MG_OK;
    if (d.accumulate && d.mode == MG_EPI_RELU_MASK) return MG_OK;
  }

  bool use_dmma = dmma_eligible(d) && d.K > 0;
  if (g_gemm_path == 1) use_dmma = false;
  // Below M.N.K = 512 the plain kernel is used.  The bar used to be 64^3; measured on
  // the launch-bound steps (batch-32 training step: 112.6 -> 97.3 us, recorded 83.9 ->
  // 69.6 us; the per-sample trainer loop: 5.6 k -> 7.6 k samples/s), one CTA of the
  // tensor-core kernel finishes a tiny product in less time than the plain
  // kernel's chain of dependent 16-deep global loads.
  static const size_t min_dmma_volume = [] {
    const char *v = std::getenv("MG_GEMM_MIN_VOLUME");  // diagnostic
    return v && *v ? (size_t)std::atoll(v) : (size_t)512;
  }();
  if (g_gemm_path == 0 && use_dmma && d.M * d.N * d.K < min_dmma_volume) use_dmma = false;

  const int M = (int)d.M, N = (int)d.N, K = (int)d.K;
  if (!use_dmma) {
    if (d.M >= ((size_t)1 << 31) || d.N >= ((size_t)1 << 31) || d.K >= ((size_t)1 << 31))
      return fail(MG_ERR_INVALID, "gemm: dimension too large");
    StridedOperands op;
    op.A = d.A;
    op.B = d.B;
    if (d.a_kcontig) { op.sAm = (long long)d.K; op.sAk = 1; } else { op.sAm = 1; op.sAk = (long long)d.M; }
    if (d.b_kcontig) { op.sBk = 1; op.sBn = (long long)d.K; } else { op.sBk = (long long)d.N; op.sBn = 1; }
    dim3 grid((unsigned)((N + 63) / 64), (unsigned)((M + 63) / 64));
    if (grid.y > 65535) return fail(MG_ERR_INVALID, "gemm fallback: too many row tiles (%u)", grid.y);
    gemm_fallback_kernel<<<grid, 256, 0, c.stream>>>(op, ep, M, N, K);
    MG_LAUNCH_CHECK("gemm_fallback");
    return MG_OK;
  }

  const int shape = g_dmma_shape >= 0 ? g_dmma_shape : default_dmma_shape();
  const GemmPlan plan = choose_plan(M, N, K, c.sm_count, shape);
  const int bm = plan.bm, bn = plan.bn;
  DmmaLaunch L;
  // Operands whose contiguous axis is m or n arrive as 16-column groups.  When the
  // row length is a multiple of 16 one 3-D copy per stage brings all groups of the
  // tile; otherwise each group is its own 2-D copy.
  L.grouped_ab = 0;
  bool ok_a, ok_b;
  if (d.a_kcontig) {
    ok_a = make_tensor_map_f64(&L.ma, d.A, d.M, d.K, BK, bm);
  } else if (d.M % 16 == 0 && make_tensor_map_f64_grouped(&L.ma, d.A, d.K, d.M, BK, bm / 16)) {
    ok_a = true;
    L.grouped_ab |= 1;
  } else {
    ok_a = make_tensor_map_f64(&L.ma, d.A, d.K, d.M, 16, BK);
  }
  if (d.b_kcontig) {
    ok_b = make_tensor_map_f64(&L.mb, d.B, d.N, d.K, BK, bn);
  } else if (d.N % 16 == 0 && make_tensor_map_f64_grouped(&L.mb, d.B, d.K, d.N, BK, bn / 16)) {
    ok_b = true;
    L.grouped_ab |= 2;
  } else {
    ok_b = make_tensor_map_f64(&L.mb, d.B, d.K, d.N, 16, BK);
  }
  if (!ok_a || !ok_b) return fail(MG_ERR_CUDA, "gemm: cuTensorMapEncodeTiled failed");
  // ReLU-mask source [M][N]: boxes of bm rows x 16 columns.  If the map cannot be
  // built the epilogue reads the mask with plain loads instead.
  L.mmask = L.ma;
  L.mask_tma = (d.mode == MG_EPI_RELU_MASK && d.a_kcontig && d.b_kcontig && shape == 2 &&
                make_tensor_map_f64(&L.mmask, d.aux, d.M, d.N, 16, bm))
                   ? 1 : 0;

  const int tiles_m = (M + bm - 1) / bm, tiles_n = (N + bn - 1) / bn;
  const int KT = (K + BK - 1) / BK;
  const SegTable *table = nullptr;
  if (plan.spans > 0) {
    int rc = seg_table_for(tiles_m, tiles_n, KT, bm, bn, plan.spans, &table);
    if (rc != MG_OK) return rc;
    if (table->slots > 0) {
      rc = ensure_scratch(&c.splitk_scratch, &c.splitk_scratch_elems,
                          (size_t)table->slots * (size_t)bm * (size_t)bn);
      if (rc != MG_OK) return rc;
      ep.partial = c.splitk_scratch;
    }
  }
  L.ep = ep;
  L.M = M; L.N = N; L.K = K;
  L.tiles_m = tiles_m; L.tiles_n = tiles_n;
  L.table = table ? table->dev_items : nullptr;
  // Split tiles are folded inside the kernel by their last-arriving segment.
  const bool fold = table && table->slots > 0;
  L.tickets = fold ? table->dev_tickets : nullptr;
  if (fold) L.mask_tma = 0;
  L.items = table ? table->items : tiles_m * tiles_n;
  L.min_nkt = table ? table->min_nkt : KT;
  int rc;
  if (d.a_kcontig && !d.b_kcontig)
    rc = launch_layout<true, false>(shape, plan.tile, L);
  else if (d.a_kcontig && d.b_kcontig)
    rc = launch_layout<true, true>(shape, plan.tile, L);
  else if (!d.a_kcontig && !d.b_kcontig)
    rc = launch_layout<false, false>(shape, plan.tile, L);
  else
    return fail(MG_ERR_INVALID, "gemm: unsupported operand layout");
  if (rc != MG_OK) return rc;
  return MG_OK;
}

}  // namespace mg

using namespace mg;

extern "C" {

int mg_gemm_plan_describe(size_t M, size_t N, size_t K, int sm_count, int *plan5, int *segments,
                          int max_segments) {
  if (!plan5 || M == 0 || N == 0 || K == 0 || sm_count < 1 || M >= ((size_t)1 << 30) ||
      N >= ((size_t)1 << 30) || K >= ((size_t)1 << 30))
    return fail(MG_ERR_INVALID, "mg_gemm_plan_describe: bad arguments");
  const GemmPlan plan = choose_plan((int)M, (int)N, (int)K, sm_count, 2);
  const int tiles_m = ((int)M + plan.bm - 1) / plan.bm, tiles_n = ((int)N + plan.bn - 1) / plan.bn;
  const int KT = ((int)K + BK - 1) / BK;
  plan5[0] = plan.bm;
  plan5[1] = plan.bn;
  plan5[2] = plan.spans;
  plan5[3] = tiles_m * tiles_n;
  plan5[4] = 0;
  if (plan.spans == 0) return MG_OK;
  std::vector<SegItem> segs;
  std::vector<int2> tile_info;
  int slots = 0, min_nkt = 0;
  build_segments(tiles_m, tiles_n, KT, plan.bm, plan.bn, plan.spans, segs, tile_info, slots, min_nkt);
  plan5[3] = (int)segs.size();
  plan5[4] = slots;
  if (segments) {
    if ((int)segs.size() > max_segments)
      return fail(MG_ERR_INVALID, "mg_gemm_plan_describe: %zu segments, room for %d", segs.size(),
                  max_segments);
    for (size_t i = 0; i < segs.size(); i++) {
      segments[5 * i + 0] = segs[i].m0;
      segments[5 * i + 1] = segs[i].n0;
      segments[5 * i + 2] = segs[i].kt_begin;
      segments[5 * i + 3] = segs[i].nkt;
      segments[5 * i + 4] = segs[i].slot;
    }
  }
  return MG_OK;
}

int mg_gemm_config(int path, int dmma_shape) {
  if (path < 0 || path > 2) return fail(MG_ERR_INVALID, "mg_gemm_config: path must be 0, 1 or 2");
  if (dmma_shape < -1 || dmma_shape > 3)
    return fail(MG_ERR_INVALID, "mg_gemm_config: shape must be -1..3");
  g_gemm_path = path;
  g_dmma_shape = dmma_shape;
  return MG_OK;
}

int mg_gemm_nn(const double *A, const double *B, double *C, size_t M, size_t N, size_t K,
               int accumulate, int epilogue, const double *bias) {
  MG_ENSURE_INIT();
  if (M && N && (!C || (K && (!A || !B)))) return fail(MG_ERR_INVALID, "mg_gemm_nn: null pointer");
  if (epilogue != MG_EPI_NONE && epilogue != MG_EPI_BIAS && epilogue != MG_EPI_BIAS_RELU)
    return fail(MG_ERR_INVALID, "mg_gemm_nn: epilogue %d not valid here", epilogue);
  GemmDesc d{A, B, C, M, N, K, true, false, accumulate, epilogue, bias};
  return run_gemm(d);
}

int mg_gemm_nt(const double *G, const double *B, double *dA, size_t M, size_t N, size_t K,
               int accumulate, int epilogue, const double *mask_src) {
  MG_ENSURE_INIT();
  if (M && K && (!dA || (N && (!G || !B)))) return fail(MG_ERR_INVALID, "mg_gemm_nt: null pointer");
  if (epilogue != MG_EPI_NONE && epilogue != MG_EPI_RELU_MASK)
    return fail(MG_ERR_INVALID, "mg_gemm_nt: epilogue %d not valid here", epilogue);
  // Output [M][K]; contraction over N; G is [M][N] (k-contiguous), B is [K][N]
  // (output-column major, k-contiguous).
  GemmDesc d{G, B, dA, M, K, N, true, true, accumulate, epilogue, mask_src};
  return run_gemm(d);
}

int mg_gemm_tn(const double *A, const double *G, double *dB, size_t M, size_t N, size_t K,
               int accumulate) {
  MG_ENSURE_INIT();
  if (K && N && (!dB || (M && (!A || !G)))) return fail(MG_ERR_INVALID, "mg_gemm_tn: null pointer");
  // Output [K][N]; contraction over M; A is [M][K] (output-row contiguous),
  // G is [M][N] (output-column contiguous).
  GemmDesc d{A, G, dB, K, N, M, false, false, accumulate, MG_EPI_NONE, nullptr};
  return run_gemm(d);
}

}  // extern "C"
