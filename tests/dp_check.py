"""Data-parallel parity check, run as one process per GPU:

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P tests/dp_check.py

Every rank trains the same MLP for a few SGD steps on its row shard of a global
batch through the public Tensor API, with parameter gradients summed across
ranks by the library's all-reduce (started from backward(); the peer-memory
kernel where ranks can map each other's buffers, NCCL otherwise).  Before that
the all-reduce itself is checked on a shared buffer: sub-ranges at even offsets
must equal the rank-ordered sum bit for bit on every rank, and agree with the
NCCL path on a plain buffer.  Rank 0
compares losses and final parameters with the CPU oracle's full-batch training
(normwise <= 1e-9) and prints DP_PARITY_OK.  Also checks that sharded inference
yields the oracle's argmax ids on every rank's rows.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import micrograd_b200  # noqa: E402
from micrograd_b200.dist import env_rank_world, init_comm, shard_rows  # noqa: E402


def check_allreduce(abi, rank, world):
    """Peer-memory all-reduce against the rank-ordered sum computed on the host."""
    import ctypes as C
    n = 200_000
    per_rank = [np.random.default_rng(1000 + q).standard_normal(n) for q in range(world)]
    shared = C.c_void_p()
    abi.mg_comm_alloc_shared(n, C.byref(shared))
    peer = abi.mg_comm_peer_path(shared.value)
    plain = abi.array(per_rank[rank])
    abi.mg_upload(shared.value, per_rank[rank].ctypes.data, n)
    ranges = [(0, 4096), (4096, 150_000), (154_096, 2), (160_000, 39_998)]   # (offset, count), even
    for _ in range(3):                       # repeated calls reuse the flags
        for off, cnt in ranges:
            abi.mg_allreduce_sum_async(shared.value + 8 * off, cnt)
    for off, cnt in ranges:                  # a fourth round with the wide ("exposed") grid
        abi.mg_allreduce_sum_async_hint(shared.value + 8 * off, cnt, 1)
    for off, cnt in ranges:
        abi.mg_allreduce_sum_async(plain.ptr + 8 * off, cnt)   # not a shared buffer: NCCL
    abi.mg_comm_join()
    abi.mg_sync()
    abi.mg_check_kernel_status()
    got = np.empty(n)
    abi.mg_download(got.ctypes.data, shared.value, n)
    nccl = plain.numpy()
    ok = True
    for off, cnt in ranges:
        once = per_rank[0][off:off + cnt].copy()
        for q in range(1, world):
            once = once + per_rank[q][off:off + cnt]          # rank order, like the kernel
        twice = once.copy()
        for _ in range(world - 1):
            twice = twice + once                               # second call sums W equal copies
        thrice = twice.copy()
        for _ in range(world - 1):
            thrice = thrice + twice
        fourth = thrice.copy()
        for _ in range(world - 1):
            fourth = fourth + thrice
        # NCCL adds the ranks' values in its own order: equal up to rounding of O(1) sums
        checks = [("nccl", np.allclose(nccl[off:off + cnt], once, rtol=0, atol=1e-13))]
        if peer:
            checks.append(("peer (bit-exact)", np.array_equal(got[off:off + cnt], fourth)))
        else:
            checks.append(("fallback", np.allclose(got[off:off + cnt], fourth, rtol=0, atol=1e-10)))
        for what, passed in checks:
            if not passed:
                ok = False
                ref_v = once if what == "nccl" else fourth
                got_v = nccl[off:off + cnt] if what == "nccl" else got[off:off + cnt]
                print(f"rank {rank}: {what} mismatch on range ({off}, {cnt}): "
                      f"max abs diff {np.abs(got_v - ref_v).max():.3e}", flush=True)
    untouched = np.ones(n, dtype=bool)
    for off, cnt in ranges:
        untouched[off:off + cnt] = False
    if not np.array_equal(got[untouched], per_rank[rank][untouched]):
        ok = False
        print(f"rank {rank}: elements outside the reduced ranges changed", flush=True)
    abi.mg_comm_free_shared(shared.value)
    print(f"rank {rank}: allreduce check {'ok' if ok else 'FAILED'} peer_path={peer}", flush=True)
    return ok, peer


def main():
    rank, world, local_rank = env_rank_world()
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    abi = micrograd_b200.load_abi()
    abi.mg_init(local_rank)
    api = micrograd_b200.load_api()
    init_comm(api)
    assert api.comm_world() == world and api.comm_rank() == rank
    allreduce_ok, peer = check_allreduce(abi, rank, world)

    rng = np.random.default_rng(77)                      # identical on all ranks
    sizes, batch, steps, lr = [784, 256, 128, 10], 1024, 4, 0.05
    params = [(rng.standard_normal((i, o)) / np.sqrt(i), np.zeros(o)) for i, o in zip(sizes[:-1], sizes[1:])]
    X, y = rng.random((batch, sizes[0])), rng.integers(0, 10, batch).astype(np.int32)
    b, e = shard_rows(batch, rank, world)

    layers = []
    for W, bias in params:
        lin = api.Linear(W.shape[0], W.shape[1])
        lin.weights().set_data(W)
        lin.bias().set_data(bias)
        layers.append(lin)
    # A layer the graph never uses rides along in the optimiser: its bucket is never
    # completed by a backward sweep, so step() has to exchange it itself (all ranks
    # alike) instead of hanging or applying a rank-local gradient.
    spare = api.Linear(16, 8)
    spare_w = rng.standard_normal((16, 8))
    spare.weights().set_data(spare_w)
    opt = api.SGD([t for lin in layers for t in (lin.weights(), lin.bias())] +
                  [spare.weights(), spare.bias()], lr)
    opt.enable_allreduce()
    x = api.Tensor([e - b, sizes[0]], X[b:e])
    x.set_requires_grad(False)

    def logits_of(inp):
        return layers[2].forward(layers[1].forward_relu(layers[0].forward_relu(inp)))

    losses = []
    for _ in range(steps):
        loss = api.softmax_cross_entropy(logits_of(x), y[b:e], batch)   # divisor = global batch
        opt.zero_grad()
        loss.backward()
        opt.step()
        # each rank's loss is its share of the global mean; sum the shares
        t = torch.tensor([loss.data()[0]], dtype=torch.float64, device="cuda")
        dist.all_reduce(t)
        losses.append(float(t.item()))
    ids = api.argmax_rows(logits_of(x))
    abi.mg_check_kernel_status()
    ok_extra = np.array_equal(spare.weights().data(), spare_w.reshape(-1)) and not spare.bias().data().any()
    if not ok_extra:
        print(f"rank {rank}: the unused layer's parameters changed")
    # A second backward() before step(): the first sweep's gradients are already summed
    # over the ranks, so the library refuses instead of reducing them a second time.
    final = [(lin.weights().data().copy(), lin.bias().data().copy()) for lin in layers]
    loss = api.softmax_cross_entropy(logits_of(x), y[b:e], batch)
    opt.zero_grad()
    loss.backward()
    try:
        loss.backward()
        refused = False
    except RuntimeError as exc:
        refused = "before step()" in str(exc)
    if not refused:
        ok_extra = False
        print(f"rank {rank}: a second backward() before step() was not refused")
    opt.zero_grad()                                       # drops the sweep; parameters untouched
    abi.mg_sync()
    for lin, (w0, b0) in zip(layers, final):
        if not (np.array_equal(lin.weights().data(), w0) and np.array_equal(lin.bias().data(), b0)):
            ok_extra = False
            print(f"rank {rank}: parameters changed by the refused sweep")

    import oracle
    fast = oracle.fast
    ref = [(W.copy(), bias.copy()) for W, bias in params]
    ok = allreduce_ok and ok_extra
    for s in range(steps):
        ref_loss, _, _ = fast.mlp_train_step(ref, X, y, lr)
        if abs(losses[s] - ref_loss) > 1e-10 * abs(ref_loss):
            ok = False
            print(f"rank {rank}: loss mismatch at step {s}: {losses[s]} vs {ref_loss}")
    for lin, (W, bias) in zip(layers, ref):
        err_w = np.abs(lin.weights().data() - W.reshape(-1)).max() / np.abs(W).max()
        err_b = np.abs(lin.bias().data() - bias).max() / max(np.abs(bias).max(), 1e-300)
        if err_w > 1e-9 or err_b > 1e-9:
            ok = False
            print(f"rank {rank}: parameter mismatch {err_w} {err_b}")
    ref_logits, _ = fast.mlp_forward(ref, X[b:e])
    # the device ids must match ids computed from the device's own parameters' oracle twin
    flips = int((ids != fast.argmax_rows(ref_logits)).sum())
    if flips:
        ok = False
        print(f"rank {rank}: {flips} argmax flips")
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    api.comm_shutdown()
    dist.destroy_process_group()
    if rank == 0:
        print("DP_PARITY_OK" if int(flag.item()) == 1 else "DP_PARITY_FAILED",
              f"world={world} peer_path={peer} losses={losses}")
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
