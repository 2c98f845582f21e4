"""Bounded-wait check of the peer-memory all-reduce, run as two processes on two GPUs:

    MG_PEER_WAIT_MS=300 python -m torch.distributed.run --nproc-per-node 2 \
        --master-addr 127.0.0.1 --master-port P tests/dp_timeout_check.py

Rank 0 starts an all-reduce that rank 1 never joins (the failure is made on the
host: a rank that does not show up).  Rank 0's kernel must give up after the
configured limit, report through the kernel fault word, and leave the context
and the communicator usable: afterwards both ranks run a normal all-reduce on a
fresh shared buffer and check its result.  Nothing faults or hangs the GPU.
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
            try:
                abi.mg_check_kernel_status()
                ok = False
                print("rank 0: the unanswered all-reduce reported no fault", flush=True)
            except K.MgError as e:
                ok = e.code == K.ERR_KERNEL and "fault code 30" in str(e)
                print(f"rank 0: gave up after {waited:.2f} s: {e}", flush=True)
            ok = ok and waited < 5.0
            abi.mg_check_kernel_status()                      # the fault word was cleared
        else:
            time.sleep(1.5)
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
