"""CPU tests of the multi-GPU partitioning logic: index math against a single-process simulation of P ranks,
and a real two-rank run over gloo."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import sage3_oracle as O
from sageattention_b200 import ulysses as U


def test_shard_units_cover_everything_once():
    for B, H, P in [(4, 32, 8), (8, 8, 8), (1, 24, 8), (2, 3, 4), (1, 1, 2)]:
        seen = []
        sizes = []
        for r in range(P):
            u = U.shard_units(B, H, r, P)
            seen += u
            sizes.append(len(u))
        assert sorted(seen) == [(b, h) for b in range(B) for h in range(H)]
        assert max(sizes) - min(sizes) <= 1


@pytest.mark.parametrize("P,Hq,Hkv", [(2, 4, 4), (4, 8, 4), (8, 48, 48), (8, 24, 8)])
def test_exchange_layouts_by_simulation(P, Hq, Hkv):
    """Simulate the two all-to-alls with plain indexing: rank r receives slice r of every rank's send buffer."""
    B, n, D = 2, 3, 8
    N = P * n
    g = torch.Generator().manual_seed(P)
    q = torch.randn(B, Hq, N, D, generator=g)
    k = torch.randn(B, Hkv, N, D, generator=g)
    v = torch.randn(B, Hkv, N, D, generator=g)
    shard = lambda x, r: x[:, :, r * n:(r + 1) * n]
    sends = [U.pack_heads_for_exchange(shard(q, r), shard(k, r), shard(v, r), P) for r in range(P)]
    outs = []
    for r in range(P):
        recv = torch.stack([sends[src][r] for src in range(P)])
        ql, kl, vl = U.unpack_heads_after_exchange(recv, Hq // P, Hkv // P)
        assert torch.equal(ql, q[:, r * Hq // P:(r + 1) * Hq // P])
        assert torch.equal(kl, k[:, r * Hkv // P:(r + 1) * Hkv // P])
        assert torch.equal(vl, v[:, r * Hkv // P:(r + 1) * Hkv // P])
        outs.append(ql * 2.0)          # stands in for the local attention output [B, Hq/P, N, D]
    sends_o = [U.pack_tokens_for_exchange(o, P) for o in outs]
    for r in range(P):
        recv_o = torch.stack([sends_o[src][r] for src in range(P)])
        assert torch.equal(U.unpack_tokens_after_exchange(recv_o), shard(q, r) * 2.0)


def test_head_count_must_divide():
    x = torch.zeros(1, 3, 4, 8)
    with pytest.raises(ValueError):
        U.pack_heads_for_exchange(x, x, x, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, layout, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v = O.make_inputs(1, 4, 2, 256, 256, 64, seed=77, k_offset_std=1.0)
        n = 256 // world
        cut = lambda x: x[:, :, rank * n:(rank + 1) * n]
        args = [cut(t) for t in (q, k, v)]
        if layout == "NHD":
            args = [t.transpose(1, 2).contiguous() for t in args]
        out = U.ulysses_attention(*args, tensor_layout=layout, is_causal=True, attn_fn=O.sageattn3_oracle)
        if layout == "NHD":
            out = out.transpose(1, 2)
        full = O.sageattn3_oracle(q, k, v, is_causal=True)
        ret[rank] = bool(torch.equal(out, cut(full)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("layout", ["HND", "NHD"])
def test_two_ranks_over_gloo_match_single_process(layout):
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), layout, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def _worker_slices(rank, world, port, groups, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v = O.make_inputs(1, 12, 6, 128, 128, 64, seed=78, k_offset_std=1.0)
        n = 128 // world
        cut = lambda x: x[:, :, rank * n:(rank + 1) * n]
        out = U.ulysses_attention(cut(q), cut(k), cut(v), attn_fn=O.sageattn3_oracle, overlap_groups=groups)
        full = O.sageattn3_oracle(q, k, v)
        ret[rank] = bool(torch.equal(out, cut(full)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("groups", [3, 2, 7])
def test_head_slices_overlap_gives_the_same_result(groups):
    """Three kv heads (six q heads) per rank, processed in 3, 2 (uneven) and 3 (clamped) slices."""
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker_slices, args=(world, _free_port(), groups, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def _worker_ring(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v = O.make_inputs(1, 3, 3, 384, 384, 64, seed=79, k_offset_std=1.0)     # 3 heads: Ulysses could not split them
        n = 384 // world
        cut = lambda x: x[:, :, rank * n:(rank + 1) * n]
        out = U.ring_attention(cut(q), cut(k), cut(v), attn_fn=O.sageattn3_oracle)
        # the same composition in one process: this rank's queries against every key shard, merged in ring order
        acc = lse = exp = None
        for step in range(world):
            j = (rank - step) % world
            o_j, l_j = O.sageattn3_oracle(cut(q), k[:, :, j * n:(j + 1) * n], v[:, :, j * n:(j + 1) * n], return_lse=True)
            acc, lse, exp = U.merge_partial(acc, lse, o_j, l_j, want_out=(step + 1 == world))
        full = O.fp32_attention(q, k, v)
        ret[rank] = (bool(torch.equal(out, exp)), O.cosine(out, cut(full)), O.rel_l1(out, cut(full)))
    finally:
        dist.destroy_process_group()


def test_ring_attention_over_gloo():
    """Three heads on two ranks (not divisible: the case ring attention exists for).  The distributed result equals the
    single-process composition bit for bit, and sits at the method's usual distance from fp32 attention."""
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker_ring, args=(world, _free_port(), ret), nprocs=world, join=True)
        for r in range(world):
            same, cos, l1 = ret[r]
            assert same and cos > 0.97 and l1 < 0.3, (r, same, cos, l1)


def test_merge_partial_is_softmax_composition():
    """Merging attention over two disjoint key sets through their LSE equals attention over the union (fp32 check)."""
    g = torch.Generator().manual_seed(4)
    q = torch.randn(1, 2, 16, 32, generator=g)
    k = torch.randn(1, 2, 48, 32, generator=g)
    v = torch.randn(1, 2, 48, 32, generator=g)
    def part(ks):
        s = torch.matmul(q, k[:, :, ks].transpose(-1, -2)) * 32 ** -0.5
        return torch.matmul(torch.softmax(s, -1), v[:, :, ks]).to(torch.bfloat16), torch.logsumexp(s, -1)
    acc = lse = out = None
    for ks in (slice(0, 16), slice(16, 48)):
        o, l = part(ks)
        acc, lse, out = U.merge_partial(acc, lse, o, l, want_out=True)
    ref, ref_lse = part(slice(0, 48))
    assert torch.allclose(out.float(), ref.float(), atol=2e-2) and torch.allclose(lse, ref_lse, atol=1e-5)


def test_ring_attention_is_non_causal_only():
    with pytest.raises(NotImplementedError):
        U.ring_attention(torch.zeros(1, 1, 8, 16), torch.zeros(1, 1, 8, 16), torch.zeros(1, 1, 8, 16), is_causal=True)
