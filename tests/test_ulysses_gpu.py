"""Two-GPU check of the Ulysses path over NCCL: the sequence-parallel output equals the single-GPU output
bit for bit (every head is computed by exactly one rank from identical inputs).  Skipped on a single GPU."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    from oracle import sage3_oracle as O
    from sageattention_b200 import sageattn3
    from sageattention_b200.ulysses import ulysses_attention
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        q, k, v = O.make_inputs(2, 8, 4, 1000, 1000, 64, seed=31, k_outlier_channels=4)   # ragged N, GQA
        n = 1000 // world
        cut = lambda x: x[:, :, rank * n:(rank + 1) * n].contiguous().to(dev)
        out = ulysses_attention(cut(q), cut(k), cut(v), is_causal=False)
        full = sageattn3(q.to(dev), k.to(dev), v.to(dev))
        torch.cuda.synchronize()
        ret[rank] = bool(torch.equal(out, full[:, :, rank * n:(rank + 1) * n]))
    finally:
        dist.destroy_process_group()


def test_ulysses_two_gpus_bit_identical(cuda_device):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}
