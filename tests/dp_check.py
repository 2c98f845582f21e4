"""Data-parallel parity check, run as one process per GPU:

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P tests/dp_check.py

Every rank trains the same MLP for a few SGD steps on its row shard of a global
batch through the public Tensor API, with parameter gradients summed across
ranks by the library's NCCL all-reduce (started from backward()).  Rank 0
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


def main():
    rank, world, local_rank = env_rank_world()
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    abi = micrograd_b200.load_abi()
    abi.mg_init(local_rank)
    api = micrograd_b200.load_api()
    init_comm(api)
    assert api.comm_world() == world and api.comm_rank() == rank

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
    opt = api.SGD([t for lin in layers for t in (lin.weights(), lin.bias())], lr)
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

    import oracle
    fast = oracle.fast
    ref = [(W.copy(), bias.copy()) for W, bias in params]
    ok = True
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
        print("DP_PARITY_OK" if int(flag.item()) == 1 else "DP_PARITY_FAILED", f"world={world} losses={losses}")
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
