"""CPU: the GEMM dispatcher's host logic — tile choice and the segment tables of
split contractions — checked through mg_gemm_plan_describe, which touches no
device.  148 SMs as on B200."""
import ctypes as C

import numpy as np
import pytest

import micrograd_b200

SMS = 148
BK = 16


def describe(M, N, K, sms=SMS, want_segments=True):
    abi = micrograd_b200.load_abi()
    plan = (C.c_int * 5)()
    cap = 4096
    segs = (C.c_int * (5 * cap))()
    abi.mg_gemm_plan_describe(M, N, K, sms, plan, segs if want_segments else None, cap)
    bm, bn, spans, items, slots = list(plan)
    table = np.array(segs[: 5 * items], dtype=np.int64).reshape(items, 5) if spans else None
    return bm, bn, spans, items, slots, table


# (M, N, K) -> expected (tile rows, tile cols, split?) for the config-4 layer shapes
# at 65536 rows per GPU (one GPU) and 8192 rows per GPU (eight GPUs).
@pytest.mark.parametrize("shape,expect", [
    ((65536, 1024, 784), (128, 128, False)),    # layer-1 forward
    ((65536, 1024, 1024), (128, 128, False)),   # layer-2 forward / input gradient
    ((65536, 10, 1024), (128, 16, True)),       # logits forward: 512 tiles, 3.46 waves -> spans
    ((65536, 1024, 10), (128, 64, False)),      # gradient through the logits: one k-tile
    ((1024, 1024, 65536), (128, 128, True)),    # dW2: 64 tiles, contraction over the batch
    ((784, 1024, 65536), (112, 128, True)),     # dW1: 784 = 7 x 112
    ((1024, 10, 65536), (128, 16, True)),       # dW3
    ((8192, 1024, 1024), (128, 64, False)),     # 512 full tiles would leave the 4th wave half empty
    ((1024, 1024, 8192), (128, 128, True)),
    ((4096, 4096, 4096), (128, 128, False)),
    ((65536, 784, 1024), (128, 112, False)),    # gradient w.r.t. a 784-wide input: 784 = 7 x 112
])
def test_tile_choice_for_benchmark_shapes(shape, expect):
    bm, bn, spans, items, slots, _ = describe(*shape)
    assert (bm, bn, spans > 0) == expect
    if not expect[2]:
        assert items == -(-shape[0] // bm) * -(-shape[1] // bn) and slots == 0


@pytest.mark.parametrize("M,N,K", [(1024, 1024, 65536), (784, 1024, 8192), (1024, 10, 65536),
                                   (200, 136, 6000), (1024, 1024, 1024), (3000, 258, 4096),
                                   (130, 72, 100000)])
def test_segments_cover_every_k_tile_once_and_issue_longest_first(M, N, K):
    bm, bn, spans, items, slots, table = describe(M, N, K)
    assert spans > 0, "shape was chosen to need a split contraction"
    tiles_m, tiles_n, KT = -(-M // bm), -(-N // bn), -(-K // BK)
    assert 1 < spans <= SMS
    covered = np.zeros((tiles_m * tiles_n, KT), dtype=np.int32)
    for m0, n0, kt0, nkt, slot in table:
        assert m0 % bm == 0 and n0 % bn == 0 and nkt >= 1 and kt0 >= 0 and kt0 + nkt <= KT
        covered[(m0 // bm) * tiles_n + n0 // bn, kt0:kt0 + nkt] += 1
    assert np.array_equal(covered, np.ones_like(covered))
    # issue order: longest first (the hardware scheduler then pairs complements)
    assert np.all(np.diff(table[:, 3]) <= 0)
    # balance: no SM's share exceeds the ideal by more than one segment's rounding
    per_span = tiles_m * tiles_n * KT / spans
    assert table[:, 3].max() <= np.ceil(per_span)
    # slots: a tile covered by several segments owns consecutive slots in k order;
    # a tile covered by one segment has none
    by_tile = {}
    for m0, n0, kt0, nkt, slot in table:
        by_tile.setdefault((m0, n0), []).append((kt0, slot))
    used = []
    for segs in by_tile.values():
        segs.sort()
        if len(segs) == 1:
            assert segs[0][1] == -1
        else:
            ids = [s for _, s in segs]
            assert ids == list(range(ids[0], ids[0] + len(ids)))
            used += ids
    assert sorted(used) == list(range(slots))


def test_short_contractions_and_full_waves_are_not_split():
    assert describe(128 * 148, 128, 4096)[2] == 0        # 148 tiles: one full wave
    assert describe(1024, 1024, 256)[2] == 0             # 16 k-tiles: too short to share
    assert describe(128 * 600, 128, 4096)[2] == 0        # more than four waves of tiles


def test_plan_scales_with_the_sm_count():
    few = describe(1024, 1024, 65536, sms=16)
    assert few[2] == 0                                    # 64 tiles on 16 SMs: four full waves
    many = describe(1024, 1024, 65536, sms=148)
    assert many[2] == 148 and many[3] <= 148 + 64


def test_bad_arguments_are_rejected():
    abi = micrograd_b200.load_abi()
    plan = (C.c_int * 5)()
    from micrograd_b200.cabi import MgError
    with pytest.raises(MgError):
        abi.mg_gemm_plan_describe(0, 8, 8, SMS, plan, None, 0)
    with pytest.raises(MgError):
        abi.mg_gemm_plan_describe(8, 8, 8, 0, plan, None, 0)
    segs = (C.c_int * 5)()
    with pytest.raises(MgError):
        abi.mg_gemm_plan_describe(1024, 1024, 65536, SMS, plan, segs, 1)   # table does not fit
