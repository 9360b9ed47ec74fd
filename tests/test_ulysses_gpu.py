"""Multi-GPU checks of the sequence-parallel paths: the output equals the single-GPU output bit for bit (every head is
computed by exactly one rank from identical inputs).  The Ulysses tests use the largest of 2, 4, 8 ranks the machine has
GPUs for; skipped on a single GPU."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _world():
    return max([w for w in (2, 4, 8) if w <= torch.cuda.device_count()], default=0)


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
        q, k, v = O.make_inputs(2, 16, 8, 1000, 1000, 64, seed=31, k_outlier_channels=4)   # ragged N, GQA
        n = 1000 // world
        cut = lambda x: x[:, :, rank * n:(rank + 1) * n].contiguous().to(dev)
        out = ulysses_attention(cut(q), cut(k), cut(v), is_causal=False)
        full = sageattn3(q.to(dev), k.to(dev), v.to(dev))
        torch.cuda.synchronize()
        ret[rank] = bool(torch.equal(out, full[:, :, rank * n:(rank + 1) * n]))
    finally:
        dist.destroy_process_group()


def test_ulysses_two_gpus_bit_identical(cuda_device):
    world = _world()
    if world < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        assert dict(ret) == {r: True for r in range(world)}


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


def test_merge_kernel_matches_host_formula(cuda_device):
    from sageattention_b200 import ulysses as U
    g = torch.Generator().manual_seed(9)
    for dt, D in ((torch.bfloat16, 128), (torch.float16, 64)):
        parts = [(torch.randn(2, 3, 50, D, generator=g).to(dt), torch.randn(2, 3, 50, generator=g) * 3) for _ in range(3)]
        parts[1][1][0, 0, :5] = -float("inf")                   # rows without keys in one partial result
        for p_ in parts:
            p_[1][1, 2, 7] = -float("inf")                      # ... and in all of them
        acc = lse = out = acc_d = lse_d = out_d = None
        for i, (o, l) in enumerate(parts):
            acc, lse, out = U.merge_partial(acc, lse, o, l, want_out=(i == 2))
            acc_d, lse_d, out_d = U.merge_partial(acc_d, lse_d, o.to(cuda_device), l.to(cuda_device), want_out=(i == 2))
        torch.cuda.synchronize()
        assert torch.allclose(lse_d.cpu(), lse, atol=1e-5, rtol=1e-5)
        assert torch.allclose(acc_d.cpu(), acc, atol=1e-5, rtol=1e-4)
        assert torch.allclose(out_d.cpu().float(), out.float(), atol=1e-2, rtol=1e-2)
        assert out_d[1, 2, 7].abs().max() == 0 and torch.isinf(lse_d[1, 2, 7])


def _worker_ring(rank, world, port, ret):
    import torch.distributed as dist
    from oracle import sage3_oracle as O
    from sageattention_b200 import sageattn3
    from sageattention_b200.ulysses import ring_attention
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        q, k, v = O.make_inputs(1, 3, 3, 2048, 2048, 128, seed=33, k_offset_std=1.0)     # 3 heads on 2 GPUs
        n = 2048 // world
        cut = lambda x: x[:, :, rank * n:(rank + 1) * n].contiguous().to(dev)
        out = ring_attention(cut(q), cut(k), cut(v))
        one = sageattn3(q.to(dev), k.to(dev), v.to(dev))[:, :, rank * n:(rank + 1) * n]
        torch.cuda.synchronize()
        full = O.fp32_attention(q, k, v)[:, :, rank * n:(rank + 1) * n]
        ret[rank] = (O.cosine(out.cpu(), one.cpu()), O.cosine(out.cpu(), full), O.cosine(one.cpu(), full))
    finally:
        dist.destroy_process_group()


def test_ring_attention_two_gpus(cuda_device):
    """Per-shard smoothing and quantization: not bit-identical to the single-GPU call, but as close to fp32 attention."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker_ring, args=(2, _free_port(), ret), nprocs=2, join=True)
        for r in range(2):
            c_one, c_full, c_ref = ret[r]
            print(f"rank {r}: ring vs single GPU cos {c_one:.4f} | ring vs fp32 {c_full:.4f} | single GPU vs fp32 {c_ref:.4f}")
            assert c_one > 0.97 and c_full > c_ref - 0.01


def _worker_peer(rank, world, port, ret):
    import torch.distributed as dist
    from oracle import sage3_oracle as O
    from sageattention_b200 import sageattn3
    from sageattention_b200.ulysses import PeerUlysses
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        B, Hq, Hkv, N, D = 2, 16, 8, 1000, 64                                          # ragged N, GQA
        n = N // world
        pu = PeerUlysses(B, Hq, Hkv, n, D, torch.bfloat16, device=dev)
        ok = True
        for it in range(3):                                                          # three calls: both buffer sets, and reuse
            q, k, v = O.make_inputs(B, Hq, Hkv, N, N, D, seed=31 + it, k_outlier_channels=4)
            cut = lambda x: x[:, :, rank * n:(rank + 1) * n].contiguous().to(dev)
            if it == 1:                                                              # the caller writes into the staging views
                sq, sk, sv = pu.stage()
                sq.copy_(cut(q)); sk.copy_(cut(k)); sv.copy_(cut(v))
                out = pu(sq, sk, sv)
            else:
                out = pu(cut(q), cut(k), cut(v))
            full = sageattn3(q.to(dev), k.to(dev), v.to(dev))
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(out, full[:, :, rank * n:(rank + 1) * n]))
        ret[rank] = ok
        pu.close()
    finally:
        dist.destroy_process_group()


def test_peer_ulysses_two_gpus_bit_identical(cuda_device):
    """Peer-to-peer sequence parallelism (token shards read and written in place over NVLink, no all-to-all): same bits
    as the single-GPU call, over several calls."""
    world = _world()
    if world < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker_peer, args=(world, _free_port(), ret), nprocs=world, join=True)
        assert dict(ret) == {r: True for r in range(world)}


def _worker_cp(rank, world, port, ret):
    import torch.distributed as dist
    from oracle import sage3_oracle as O
    from sageattention_b200 import sageattn3
    from sageattention_b200.ulysses import context_parallel_attention
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        res = []
        for causal, (Hq, Hkv, n, D) in ((False, (3, 3, 1024, 128)), (True, (4, 2, 512, 64)), (True, (3, 1, 1024, 128))):
            N = n * world
            q, k, v = O.make_inputs(1, Hq, Hkv, N, N, D, seed=35 + n + Hq, k_offset_std=1.0)
            cut = lambda x: x[:, :, rank * n:(rank + 1) * n].contiguous().to(dev)
            out, lse = context_parallel_attention(cut(q), cut(k), cut(v), is_causal=causal, return_lse=True)
            one, lse1 = sageattn3(q.to(dev), k.to(dev), v.to(dev), is_causal=causal, return_lse=True)
            torch.cuda.synchronize()
            res.append(bool(torch.equal(out, one[:, :, rank * n:(rank + 1) * n])) and
                       bool(torch.equal(lse, lse1[:, :, rank * n:(rank + 1) * n])))
        ret[rank] = res
    finally:
        dist.destroy_process_group()


def test_context_parallel_two_gpus_bit_identical(cuda_device):
    """Key shards walked in the single call's order with the accumulator state carried along, K smoothed with the mean of
    the whole sequence: the same bits as sageattn3 on the gathered tensors, causal masks and odd head counts included."""
    world = _world()
    if world < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker_cp, args=(world, _free_port(), ret), nprocs=world, join=True)
        assert dict(ret) == {r: [True, True, True] for r in range(world)}
