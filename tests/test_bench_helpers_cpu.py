"""CPU: host-side helpers of bench.py — the one global batch that every world
size shards, the host twin of the on-device input generator, and the class-id
checksum that must come out the same at every number of GPUs."""
import numpy as np

import bench
from micrograd_b200.dist import shard_rows


def test_every_world_size_sees_the_same_global_batch():
    total = 3 * bench.BATCH_BLOCK + 100                   # ragged last block
    X, y = bench.global_batch_rows(0, total)
    assert X.shape == (total, 784) and y.shape == (total,)
    assert X.min() >= 0.0 and X.max() < 1.0 and y.min() >= 0 and y.max() <= 9
    for world in (2, 4, 8, 3):
        xs, ys = [], []
        for rank in range(world):
            b, e = shard_rows(total, rank, world)
            Xr, yr = bench.global_batch_rows(b, e)
            xs.append(Xr)
            ys.append(yr)
        assert np.array_equal(np.concatenate(xs), X)
        assert np.array_equal(np.concatenate(ys), y)
    empty_X, empty_y = bench.global_batch_rows(5, 5)
    assert empty_X.shape == (0, 784) and empty_y.size == 0


def test_uniform_generator_twin_is_splitmix64():
    # first outputs of splitmix64 seeded with 0 (state advances by the golden-ratio
    # increment before each output): a published test vector of the generator
    got = bench.uniform01_host(0, 0, 3)
    want = [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]
    assert [int(v * 2.0 ** 53) for v in got] == [w >> 11 for w in want]
    # a shard generated on its own equals the same range of the whole stream
    whole = bench.uniform01_host(123, 0, 5000)
    assert np.array_equal(bench.uniform01_host(123, 1234, 100), whole[1234:1334])
    assert whole.min() >= 0.0 and whole.max() < 1.0


def test_class_id_checksum_adds_over_shards():
    rng = np.random.default_rng(0)
    ids = rng.integers(0, 10, 1 << 16).astype(np.int32)
    whole = bench.ids_checksum(ids, 0)
    for world in (2, 4, 8):
        parts = 0
        for rank in range(world):
            b, e = shard_rows(ids.size, rank, world)
            parts += bench.ids_checksum(ids[b:e], b)
        assert parts == whole
    flipped = ids.copy()
    flipped[777] = (flipped[777] + 1) % 10
    assert bench.ids_checksum(flipped, 0) != whole
