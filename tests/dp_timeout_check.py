"""Bounded-wait check of the peer-memory all-reduce, run as two processes on two GPUs:

    MG_PEER_WAIT_MS=300 python -m torch.distributed.run --nproc-per-node 2 \
        --master-addr 127.0.0.1 --master-port P tests/dp_timeout_check.py

Rank 0 starts an all-reduce that rank 1 never joins (the failure is made on the
host: a rank that does not show up).  Rank 0's kernel must give up after the
configured limit and report through the kernel fault word; an optimiser in
all-reduce mode must then refuse its next step() instead of applying unreduced
gradients; and the context and the communicator must stay usable: afterwards
both ranks run a normal all-reduce on a fresh shared buffer and check its
result.  Nothing faults or hangs the GPU.
"""
import ctypes as C
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import micrograd_b200  # noqa: E402
from micrograd_b200 import cabi as K  # noqa: E402
from micrograd_b200.dist import env_rank_world, init_comm  # noqa: E402


def main():
    rank, world, local_rank = env_rank_world()
    assert world == 2, "this check is written for two ranks"
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    abi = micrograd_b200.load_abi()
    abi.mg_init(local_rank)
    api = micrograd_b200.load_api()
    init_comm(api)

    n = 4096
    lonely = C.c_void_p()
    abi.mg_comm_alloc_shared(n, C.byref(lonely))
    peer = abi.mg_comm_peer_path(lonely.value)
    dist.barrier()
    ok = True
    if peer:
        if rank == 0:
            t0 = time.perf_counter()
            abi.mg_allreduce_sum_async(lonely.value, n)      # rank 1 never issues its half
            abi.mg_comm_join()
            abi.mg_sync()
            waited = time.perf_counter() - t0
            ok = ok and waited < 5.0
        else:
            time.sleep(1.5)
    dist.barrier()

    # An optimiser in all-reduce mode notices the fault by itself, without a device
    # synchronisation: step() mirrors the fault word to pinned memory behind its
    # exchange and looks at the copy at the start of the next step.  On rank 0 the
    # word still holds the code of the unanswered exchange: its first step() mirrors
    # it, its second step() throws (and clears the word); a retry then goes through.
    # Rank 1 saw no fault and steps normally.  Both ranks issue two exchanges.
    lin = api.Linear(8, 4)
    lin.weights().set_data(np.full((8, 4), 1.0 + rank))
    opt = api.SGD([lin.weights(), lin.bias()], 0.1)
    opt.enable_allreduce()
    opt.step()
    abi.mg_sync()
    if peer and rank == 0:
        try:
            opt.step()
            ok = False
            print("rank 0: step() applied gradients after a timed-out exchange", flush=True)
        except RuntimeError as e:
            ok = ok and "gradient exchange failed" in str(e) and "fault code 30" in str(e)
            print(f"rank 0: step() refused to go on: {e}", flush=True)
        st = C.c_int(-1)
        abi.mg_kernel_status_peek(C.byref(st))
        ok = ok and st.value == 0                             # cleared by the refusal
    opt.step()
    abi.mg_sync()
    abi.mg_check_kernel_status()
    ok = ok and bool(np.all(lin.weights().data() == 1.0 + rank))   # zero gradients: nothing moved
    del opt, lin
    dist.barrier()
    abi.mg_comm_free_shared(lonely.value)

    # the context and the communicator still work
    fresh = C.c_void_p()
    abi.mg_comm_alloc_shared(n, C.byref(fresh))
    mine = np.full(n, float(rank + 1))
    abi.mg_upload(fresh.value, mine.ctypes.data, n)
    abi.mg_allreduce_sum_async(fresh.value, n)
    abi.mg_comm_join()
    abi.mg_sync()
    abi.mg_check_kernel_status()
    got = np.empty(n)
    abi.mg_download(got.ctypes.data, fresh.value, n)
    ok = ok and bool(np.all(got == 3.0))
    abi.mg_comm_free_shared(fresh.value)

    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    api.comm_shutdown()
    dist.destroy_process_group()
    if rank == 0:
        print("DP_TIMEOUT_OK" if int(flag.item()) == 1 else "DP_TIMEOUT_FAILED", f"peer_path={peer}")
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
