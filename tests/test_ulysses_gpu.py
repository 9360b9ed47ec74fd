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


def test_regrouping_on_one_gpu_matches_torch(cuda_device):
    """pack / unpack around the two all-to-alls go through the library's slab copy on the GPU: the result must equal the
    plain tensor expressions (which the gloo tests check against a simulated exchange)."""
    from sageattention_b200 import ulysses as U
    g = torch.Generator(device=cuda_device).manual_seed(3)
    P, B, Hq, Hkv, n, D = 4, 2, 8, 4, 100, 64
    q = torch.randn(B, Hq, n, D, device=cuda_device, dtype=torch.bfloat16, generator=g)
    k = torch.randn(B, Hkv, n, D, device=cuda_device, dtype=torch.bfloat16, generator=g)
    v = torch.randn(B, Hkv, n, D, device=cuda_device, dtype=torch.bfloat16, generator=g)
    send = U.pack_heads_for_exchange(q, k, v, P)
    ref = torch.cat([q.reshape(B, P, Hq // P, n, D), k.reshape(B, P, Hkv // P, n, D), v.reshape(B, P, Hkv // P, n, D)],
                    dim=2).permute(1, 0, 2, 3, 4).contiguous()
    assert torch.equal(send, ref)
    ql, kl, vl = U.unpack_heads_after_exchange(send, Hq // P, Hkv // P)       # (as if every rank had sent this buffer)
    full = send.permute(1, 2, 0, 3, 4).reshape(B, -1, P * n, D)
    for got, want in zip((ql, kl, vl), torch.split(full, [Hq // P, Hkv // P, Hkv // P], dim=1)):
        assert got.is_contiguous() and torch.equal(got, want)
    o = torch.randn(B, Hq // P, P * n, D, device=cuda_device, dtype=torch.bfloat16, generator=g)
    so = U.pack_tokens_for_exchange(o, P)
    assert torch.equal(so, o.reshape(B, Hq // P, P, n, D).permute(2, 0, 1, 3, 4).contiguous())
    # NHD inputs (slabs not contiguous) take the generic copy
    send2 = U.pack_heads_for_exchange(q.transpose(1, 2).contiguous().transpose(1, 2), k, v, P)
    assert torch.equal(send2, ref)
