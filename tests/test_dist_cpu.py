"""CPU, two gloo ranks: the host side of the minibatch-sharded path.

Each rank takes its row shard of a global batch, computes its gradients with the
CPU oracle using the GLOBAL batch size as the loss divisor (what each GPU rank
does), the shards' gradients are summed with a gloo all-reduce (standing in for
the library's NCCL all-reduce), and the result must equal the single-process
full-batch gradients.  Also covers the byte broadcast that ships the NCCL id, and the row-sharded
inference pass (no exchange; class ids and their checksum equal the
single-process ones).
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from micrograd_b200.dist import broadcast_bytes, max_over_ranks, shard_rows


def test_shard_rows_partitions_exactly():
    for total in (0, 1, 7, 65536, 1048576, 10):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_rows(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    assert shard_rows(65536, 3, 8) == (24576, 32768)
    with pytest.raises(ValueError):
        shard_rows(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    fast = oracle.fast
    fast.set_num_threads(1)
    rng = np.random.default_rng(123)                       # same data on every rank
    sizes, batch = [12, 16, 10], 22
    params = [(rng.standard_normal((i, o)) / np.sqrt(i), np.zeros(o)) for i, o in zip(sizes[:-1], sizes[1:])]
    X, y = rng.random((batch, 12)), rng.integers(0, 10, batch)
    b, e = shard_rows(batch, rank, world)
    local = [(W.copy(), bb.copy()) for W, bb in params]
    loss, grads, _ = fast.mlp_train_step(local, X[b:e], y[b:e], 0.1, denom=batch, apply=False)
    flat = np.concatenate([np.concatenate([gW.reshape(-1), gb]) for gW, gb in grads])
    t = torch.from_numpy(flat)
    dist.all_reduce(t)                                      # sum of shard gradients
    lt = torch.tensor([loss], dtype=torch.float64)
    dist.all_reduce(lt)
    uid = bytes(range(128)) if rank == 0 else None
    got_uid = broadcast_bytes(uid, 128)
    slowest = max_over_ranks(float(rank + 1))
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), flat=t.numpy(), loss=lt.numpy(),
             uid=np.frombuffer(got_uid, dtype=np.uint8), slowest=slowest)
    dist.destroy_process_group()


def test_two_rank_sharded_gradients_equal_full_batch(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    import oracle
    fast = oracle.fast
    rng = np.random.default_rng(123)
    sizes, batch = [12, 16, 10], 22
    params = [(rng.standard_normal((i, o)) / np.sqrt(i), np.zeros(o)) for i, o in zip(sizes[:-1], sizes[1:])]
    X, y = rng.random((batch, 12)), rng.integers(0, 10, batch)
    loss, grads, _ = fast.mlp_train_step(params, X, y, 0.1, apply=False)
    full = np.concatenate([np.concatenate([gW.reshape(-1), gb]) for gW, gb in grads])
    for r in range(world):
        got = np.load(tmp_path / f"rank{r}.npz")
        np.testing.assert_allclose(got["flat"], full, rtol=1e-12, atol=1e-15)
        assert abs(got["loss"][0] - loss) <= 1e-13 * abs(loss)
        assert bytes(got["uid"]) == bytes(range(128))
        assert float(got["slowest"]) == float(world)


def _inference_worker(rank, world, port, out_dir, rows):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    import oracle
    fast = oracle.fast
    fast.set_num_threads(1)
    params = _inference_params()
    b, e = shard_rows(rows, rank, world)
    # every rank generates only its own rows of the one global input stream
    X = bench.uniform01_host(77, b * 20, (e - b) * 20).reshape(e - b, 20)
    logits, _ = fast.mlp_forward(params, X)
    ids = fast.argmax_rows(logits)
    part = torch.tensor([bench.ids_checksum(ids, b)], dtype=torch.int64)
    dist.all_reduce(part)                                   # the only cross-rank step: a checksum
    np.savez(os.path.join(out_dir, f"inf{rank}.npz"), ids=ids, checksum=part.numpy(), span=[b, e])
    dist.destroy_process_group()


def _inference_params():
    rng = np.random.default_rng(5)
    sizes = [20, 16, 12, 10]
    return [(rng.standard_normal((i, o)) / np.sqrt(i), 0.1 * rng.standard_normal(o))
            for i, o in zip(sizes[:-1], sizes[1:])]


def test_two_rank_sharded_inference_gives_the_same_class_ids(tmp_path):
    """Inference shards rows with no exchange: the ranks' class ids, put side by
    side, are the single-process ids, and the summed checksums agree."""
    import bench
    import oracle
    world, rows = 2, 1001                                   # odd: the shards differ in length
    mp.spawn(_inference_worker, args=(world, _free_port(), str(tmp_path), rows), nprocs=world, join=True)
    X = bench.uniform01_host(77, 0, rows * 20).reshape(rows, 20)
    logits, _ = oracle.fast.mlp_forward(_inference_params(), X)
    want = oracle.fast.argmax_rows(logits)
    got = [np.load(tmp_path / f"inf{r}.npz") for r in range(world)]
    assert [tuple(g["span"]) for g in got] == [(0, 501), (501, 1001)]
    assert np.array_equal(np.concatenate([g["ids"] for g in got]), want)
    assert len(set(want.tolist())) > 1                      # not a degenerate classifier
    for g in got:
        assert int(g["checksum"][0]) == bench.ids_checksum(want, 0)
