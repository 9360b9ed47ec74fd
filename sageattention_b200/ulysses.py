"""Multi-GPU partitioning of the attention path on one NVSwitch box (one process per GPU, NCCL).

Two schemes, as the reference's parallel example uses them through xfuser
(reference: example/parallel_sageattn_cogvideo.py:8-14, 89-95; no collective exists in the reference itself):

* independent units: (batch, kv-head) pairs are split across ranks, every rank runs the whole path on its
  shard, nothing is exchanged (`shard_units`);
* Ulysses sequence parallelism for long sequences: every rank holds a token shard of all heads; one
  all-to-all turns that into all tokens of H/P heads, attention runs locally (smoothing means and NVFP4
  quantization need the whole sequence of a head, so they run after the exchange), a second all-to-all
  returns the output to token shards (`ulysses_attention`).

For head counts smaller than (or not divisible by) the number of GPUs there is context parallelism on the same token
shards: `context_parallel_attention` walks the key shards in the single call's block order with the accumulator state
carried from shard to shard, which reproduces the single-GPU result exactly (causal masks included);
`ring_attention` is the classical form (K / V shards travel around the ring, partial results merged through their
log-sum-exp, the use `return_lse` exists for, sageattention/core.py:120-122), which for FP4 attention is a slightly
different function.

With `ulysses_attention` and `ring_attention` the exchanged tensors land in this GPU's own memory (NCCL) before any
kernel reads them.  `PeerUlysses` is the peer-to-peer form of the same exchange on one NVSwitch node: the token shards
stay where they are, in buffers that every rank maps (CUDA IPC); the pre-pass of the rank that owns a head reads the
shards over NVLink with plain loads, and the attention epilogue stores every output row straight into the shard of the
rank that owns the token.  No all-to-all, no regrouping pass: two small barriers per call.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def shard_units(B: int, Hkv: int, rank: int, world: int) -> list[tuple[int, int]]:
    """(batch, kv-head) units of `rank`: contiguous, sizes differing by at most one.  All query heads of a
    kv head stay with it, so K, V and the K mean are loaded once."""
    units = [(b, h) for b in range(B) for h in range(Hkv)]
    base, extra = divmod(len(units), world)
    start = rank * base + min(rank, extra)
    return units[start: start + base + (1 if rank < extra else 0)]


# ------------------------------------------------------------------------------------------------------
# layout helpers (pure tensor reshuffles; tested on CPU by simulating the exchange)
# ------------------------------------------------------------------------------------------------------
def _to_hnd(x: torch.Tensor, tensor_layout: str) -> torch.Tensor:
    if tensor_layout == "HND":
        return x
    if tensor_layout == "NHD":
        return x.transpose(1, 2)
    raise ValueError(f"tensor_layout must be 'HND' or 'NHD', got {tensor_layout!r}")


def _regroup(dst: torch.Tensor, src: torch.Tensor) -> None:
    """dst[i0, i1, i2] <- src[i0, i1, i2] for 5-D views whose [n, D] slabs are contiguous: one launch of the
    library's slab copy on the GPU (torch's strided copy reaches about a quarter of the HBM copy rate here)."""
    ok = (dst.is_cuda and dst.dim() == 5 and dst.shape == src.shape and dst.dtype == src.dtype
          and all(t.stride(-1) == 1 and t.stride(-2) == t.shape[-1] for t in (dst, src))
          and dst.shape[0] * dst.shape[1] * dst.shape[2] <= 65535)
    es = dst.element_size()
    slab = dst.shape[-2] * dst.shape[-1] * es
    if ok:
        ok = (slab % 16 == 0 and dst.data_ptr() % 16 == 0 and src.data_ptr() % 16 == 0
              and all((t.stride(i) * es) % 16 == 0 for t in (dst, src) for i in range(3)))
    if not ok:
        dst.copy_(src)          # host tensors (the gloo tests) and layouts the slab copy does not cover
        return
    import ctypes as C
    from . import _cabi
    ds = (C.c_int64 * 3)(*(dst.stride(i) * es for i in range(3)))
    ss = (C.c_int64 * 3)(*(src.stride(i) * es for i in range(3)))
    with torch.cuda.device(dst.device):
        _cabi.check(_cabi.lib().sage3_slab_copy(dst.data_ptr(), src.data_ptr(), dst.shape[0], dst.shape[1], dst.shape[2],
                                                C.byref(ds), C.byref(ss), slab,
                                                torch.cuda.current_stream(dst.device).cuda_stream), "sage3_slab_copy")


def pack_heads_for_exchange(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, world: int) -> torch.Tensor:
    """q [B,Hq,n,D], k/v [B,Hkv,n,D] (token shard, all heads) -> send buffer [P, B, (Hq+2Hkv)/P, n, D]:
    slice p holds the heads destined to rank p (its query heads, then its k heads, then its v heads)."""
    B, Hq, n, D = q.shape
    Hkv = k.shape[1]
    if Hq % world or Hkv % world:
        raise ValueError(f"Ulysses needs the head counts ({Hq}, {Hkv}) to be multiples of the world size {world}")
    hq, hk = Hq // world, Hkv // world
    send = torch.empty(world, B, hq + 2 * hk, n, D, dtype=q.dtype, device=q.device)
    # one pass over the data: every (batch, head) slab [n, D] moves as one contiguous run
    _regroup(send[:, :, :hq], q.reshape(B, world, hq, n, D).permute(1, 0, 2, 3, 4))
    _regroup(send[:, :, hq:hq + hk], k.reshape(B, world, hk, n, D).permute(1, 0, 2, 3, 4))
    _regroup(send[:, :, hq + hk:], v.reshape(B, world, hk, n, D).permute(1, 0, 2, 3, 4))
    return send


def unpack_heads_after_exchange(recv: torch.Tensor, Hq_local: int, Hkv_local: int):
    """recv [P (source rank = token shard), B, Hq_l+2Hkv_l, n, D] -> q [B,Hq_l,P*n,D], k, v [B,Hkv_l,P*n,D]."""
    P, B, _, n, D = recv.shape
    outs, h0 = [], 0
    for h in (Hq_local, Hkv_local, Hkv_local):          # one pass over the data, contiguous results
        x = torch.empty(B, h, P, n, D, dtype=recv.dtype, device=recv.device)
        _regroup(x, recv[:, :, h0:h0 + h].permute(1, 2, 0, 3, 4))
        outs.append(x.view(B, h, P * n, D))
        h0 += h
    return tuple(outs)


def pack_tokens_for_exchange(o: torch.Tensor, world: int) -> torch.Tensor:
    """o [B,Hq_l,N,D] (all tokens, local heads) -> send buffer [P, B, Hq_l, N/P, D]: slice p = token shard p."""
    B, H, N, D = o.shape
    send = torch.empty(world, B, H, N // world, D, dtype=o.dtype, device=o.device)
    _regroup(send, o.reshape(B, H, world, N // world, D).permute(2, 0, 1, 3, 4))
    return send


def unpack_tokens_after_exchange(recv: torch.Tensor) -> torch.Tensor:
    """recv [P (source rank = head group), B, Hq_l, n, D] -> o [B, P*Hq_l, n, D]."""
    P, B, H, n, D = recv.shape
    return recv.permute(1, 0, 2, 3, 4).reshape(B, P * H, n, D)


# ------------------------------------------------------------------------------------------------------
def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND",
                      is_causal: bool = False, group: dist.ProcessGroup | None = None,
                      attn_fn: Callable | None = None, overlap_groups: int | None = None,
                      profile: list | None = None, **kwargs) -> torch.Tensor:
    """Sequence-parallel attention.  Every rank passes its contiguous token shard
    [rank * N/P, (rank + 1) * N/P) of all heads and gets the output for the same shard.

    q: [B, Hq, N/P, D] ("HND") or [B, N/P, Hq, D] ("NHD"); k, v likewise with Hkv.  Hq and Hkv must be
    multiples of the group size.  `attn_fn(q, k, v, tensor_layout="HND", is_causal=..., **kwargs)` defaults to
    sageattn3; the result equals attn_fn on the gathered tensors, bit for bit, because every head is
    computed by exactly one rank from exactly the same inputs.

    With `overlap_groups` = G > 1 the rank's heads are processed in G slices (whole kv heads each): the
    all-to-all of slice g + 1 and the return all-to-all of slice g - 1 run on NCCL's stream while slice g is
    in the pre-pass and attention kernels.  The default is one slice: on NVSwitch the exchange is a few per cent
    of a step, and at two GPUs three slices measured 3 % slower than one (more, smaller launches).

    `profile`: a list that receives (name, CUDA event) pairs recorded on the current stream at the phase boundaries of
    a one-slice call ("start", "exchanged_in", "attended", "exchanged_out"), for a time split; None in normal use.
    """
    def mark(name):
        if profile is not None and q.is_cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream(q.device))
            profile.append((name, ev))

    if attn_fn is None:
        from .api import sageattn3 as attn_fn
    world = dist.get_world_size(group)
    qh, kh, vh = (_to_hnd(t, tensor_layout) for t in (q, k, v))
    if world == 1:
        o = attn_fn(qh.contiguous(), kh.contiguous(), vh.contiguous(), tensor_layout="HND", is_causal=is_causal, **kwargs)
        return o if tensor_layout == "HND" else o.transpose(1, 2)
    B, Hq, n, D = qh.shape
    Hkv = kh.shape[1]
    if Hq % world or Hkv % world:
        raise ValueError(f"Ulysses needs the head counts ({Hq}, {Hkv}) to be multiples of the world size {world}")
    hq_l, hkv_l = Hq // world, Hkv // world          # heads this rank computes
    rep = hq_l // hkv_l
    G = overlap_groups if overlap_groups is not None else 1
    G = max(1, min(G, hkv_l))
    bounds = [(g * hkv_l) // G for g in range(G + 1)]      # slices of the local kv heads
    q5, k5, v5 = (t.reshape(B, world, -1, n, D) for t in (qh, kh, vh))   # [B, dest rank, its heads, n, D]
    mark("start")
    works_in, recvs = [], []
    for g in range(G):
        a, b_ = bounds[g], bounds[g + 1]
        send = pack_heads_for_exchange(q5[:, :, a * rep:b_ * rep].reshape(B, -1, n, D), k5[:, :, a:b_].reshape(B, -1, n, D),
                                       v5[:, :, a:b_].reshape(B, -1, n, D), world)
        recv = torch.empty_like(send)
        works_in.append(dist.all_to_all_single(recv, send, group=group, async_op=True))
        recvs.append((recv, send))
    out5 = torch.empty(B, world, hq_l, n, D, dtype=qh.dtype, device=qh.device)
    works_out = []
    for g in range(G):
        a, b_ = bounds[g], bounds[g + 1]
        works_in[g].wait()
        ql, kl, vl = unpack_heads_after_exchange(recvs[g][0], (b_ - a) * rep, b_ - a)
        mark("exchanged_in")
        ol = attn_fn(ql.contiguous(), kl.contiguous(), vl.contiguous(), tensor_layout="HND", is_causal=is_causal, **kwargs)
        mark("attended")
        send_o = pack_tokens_for_exchange(ol, world)
        recv_o = torch.empty_like(send_o)
        works_out.append((dist.all_to_all_single(recv_o, send_o, group=group, async_op=True), recv_o, send_o, a, b_))
    for work, recv_o, _send_o, a, b_ in works_out:
        work.wait()
        _regroup(out5[:, :, a * rep:b_ * rep], recv_o.permute(1, 0, 2, 3, 4))     # [B, source rank, its slice of heads, n, D]
    mark("exchanged_out")
    o = out5.reshape(B, Hq, n, D)
    return o if tensor_layout == "HND" else o.transpose(1, 2)


# ------------------------------------------------------------------------------------------------------
# ring attention (context parallel): merges partial results over disjoint key shards through their LSE
# ------------------------------------------------------------------------------------------------------
def merge_partial(acc: torch.Tensor | None, lse_acc: torch.Tensor | None, o_part: torch.Tensor, lse_part: torch.Tensor,
                  want_out: bool):
    """Folds (o_part [.., n, D] in 16-bit, lse_part [.., n] fp32) into the running (acc fp32, lse_acc).  Returns
    (acc, lse_acc, out) where out is the merged result in o_part's dtype when `want_out`, else None.
    On the GPU this is one launch of the library's merge kernel; host tensors (the gloo tests) use tensor
    expressions of the same formula."""
    first = acc is None
    D = o_part.shape[-1]
    if o_part.is_cuda:
        import ctypes as C
        from . import _cabi
        o_part = o_part.contiguous()
        lse_part = lse_part.contiguous()
        if first:
            acc = torch.empty(o_part.shape, dtype=torch.float32, device=o_part.device)
            lse_acc = torch.empty(lse_part.shape, dtype=torch.float32, device=o_part.device)
        out = torch.empty_like(o_part) if want_out else None
        dt = {torch.float16: _cabi.SAGE3_FP16, torch.bfloat16: _cabi.SAGE3_BF16}[o_part.dtype]
        with torch.cuda.device(o_part.device):
            _cabi.check(_cabi.lib().sage3_merge_partial(
                acc.data_ptr(), lse_acc.data_ptr(), o_part.data_ptr(), lse_part.data_ptr(),
                None if out is None else out.data_ptr(), o_part.numel() // D, D, dt, int(first),
                torch.cuda.current_stream(o_part.device).cuda_stream), "sage3_merge_partial")
        return acc, lse_acc, out
    la = torch.full_like(lse_part, -float("inf")) if first else lse_acc
    mx = torch.maximum(la, lse_part)
    dead = torch.isinf(mx) & (mx < 0)
    mz = torch.where(dead, torch.zeros_like(mx), mx)
    ln = torch.where(dead, mx, mz + torch.log(torch.exp(la - mz) + torch.exp(lse_part - mz)))
    wa = torch.where(dead, torch.zeros_like(mx), torch.exp(la - torch.where(dead, torch.zeros_like(ln), ln)))
    wp = torch.where(dead, torch.zeros_like(mx), torch.exp(lse_part - torch.where(dead, torch.zeros_like(ln), ln)))
    base = torch.zeros(o_part.shape, dtype=torch.float32) if first else acc
    acc = base * wa.unsqueeze(-1) + o_part.to(torch.float32) * wp.unsqueeze(-1)
    return acc, ln, (acc.to(o_part.dtype) if want_out else None)


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND",
                   group: dist.ProcessGroup | None = None, attn_fn: Callable | None = None, **kwargs):
    """Context-parallel attention without a head-count condition.  Every rank passes its contiguous token shard
    of all heads (q [B,Hq,N/P,D], k, v [B,Hkv,N/P,D] for "HND") and gets the output for the same shard.

    P steps: the rank attends its queries to the K / V shard it currently holds
    (`attn_fn(q, k, v, tensor_layout="HND", return_lse=True, **kwargs)` -> (o, lse), default sageattn3) while that
    shard is sent on to the next rank and the next one arrives from the previous rank; the P partial results are
    merged through their log-sum-exp.  Smoothing and quantization are per shard (every partial call is a complete
    attention over its own keys), so the result agrees with the single-GPU call to within the FP4 noise of the
    method, not bit for bit.  Non-causal only."""
    if kwargs.get("is_causal"):
        raise NotImplementedError("ring_attention is non-causal (the shards would need per-step masks)")
    if attn_fn is None:
        from .api import sageattn3 as attn_fn
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    qh, kh, vh = (_to_hnd(t, tensor_layout).contiguous() for t in (q, k, v))
    kv = torch.stack((kh, vh))                      # one buffer per hop
    nxt = dist.get_global_rank(group, (rank + 1) % world) if group is not None else (rank + 1) % world
    prv = dist.get_global_rank(group, (rank - 1) % world) if group is not None else (rank - 1) % world
    acc = lse_acc = out = None
    for step in range(world):
        reqs, kv_next = [], None
        if step + 1 < world:
            kv_next = torch.empty_like(kv)
            reqs = dist.batch_isend_irecv([dist.P2POp(dist.isend, kv, nxt, group), dist.P2POp(dist.irecv, kv_next, prv, group)])
        o, lse = attn_fn(qh, kv[0], kv[1], tensor_layout="HND", return_lse=True, **kwargs)
        acc, lse_acc, out = merge_partial(acc, lse_acc, o, lse, want_out=(step + 1 == world))
        for r in reqs:
            r.wait()
        if kv_next is not None:
            kv = kv_next
    return out if tensor_layout == "HND" else out.transpose(1, 2)


def context_parallel_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND",
                               is_causal: bool = False, sm_scale=None, per_block_mean: bool = True,
                               group: dist.ProcessGroup | None = None, return_lse: bool = False):
    """Context-parallel attention that equals the single-GPU call: every rank passes its contiguous token shard of all
    heads (q [B,Hq,n,D], k, v [B,Hkv,n,D] for "HND"; rank r owns tokens [r n, (r + 1) n)) and gets the output for its
    queries.  No head-count condition; causal masks supported.

    How it differs from `ring_attention`: the key shards are walked in the order in which a single call walks its key
    blocks -- from the LAST shard to the FIRST -- with the accumulator state (unnormalized O, running maximum, row sum)
    carried from shard to shard (`sage3_attn_fwd_carry`), and every shard is smoothed with the K mean of the whole
    sequence (`sage3_prepass_kmean`; the mean is formed from the ranks' partial column sums in the single call's
    summation order).  The blocks, their order and the arithmetic are then the single call's: for shard lengths
    that are multiples of 512 tokens the result is bit-identical to `sageattn3` on the gathered tensors (multiples of
    128: identical up to the last bit of the K mean).  Each step's shard is broadcast by its owner (NCCL) while the
    previous shard is being attended; under a causal mask a rank skips the shards that lie entirely in its future.
    """
    import ctypes as C
    from . import _cabi
    from .api import Sage3Problem
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    qh, kh, vh = (_to_hnd(t, tensor_layout).contiguous() for t in (q, k, v))
    B, Hq, n, D = qh.shape
    Hkv, dev, dt = kh.shape[1], qh.device, qh.dtype
    if kh.shape[2] != n:
        raise ValueError("context_parallel_attention shards queries and keys alike (self-attention)")
    lib = _cabi.lib()
    stream = torch.cuda.current_stream(dev).cuda_stream
    out = torch.empty_like(qh)
    lse = torch.empty(B, Hq, n, dtype=torch.float32, device=dev) if return_lse else None
    prob = Sage3Problem(qh, kh, vh, "HND", is_causal, sm_scale, per_block_mean, out=out)

    # K mean of the whole sequence, in the single call's order: per-rank partial column sums (512-row chunks, written by
    # the pre-pass into its workspace), gathered, added chunk by chunk in fp32, scaled by 1 / N, rounded once
    prob.prepass()
    lay = prob.ws.layout
    chunks = lay.kchunks
    kpart = prob.ws.buf[lay.kpart: lay.kpart + B * Hkv * chunks * D * 4].view(torch.float32).view(B * Hkv, chunks, D)
    allpart = torch.empty(world, B * Hkv, chunks, D, dtype=torch.float32, device=dev)
    dist.all_gather_into_tensor(allpart, kpart.contiguous(), group=group)
    ordered = allpart.permute(1, 0, 2, 3).contiguous()         # [B*Hkv][shard][chunk][D]: the single call's chunk order
    km = torch.empty(B, Hkv, D, dtype=dt, device=dev)
    with torch.cuda.device(dev):
        _cabi.check(lib.sage3_mean_from_partial_sums(ordered.data_ptr(), B * Hkv, world * chunks, D, prob.desc.dtype, world * n,
                                                     km.data_ptr(), stream), "sage3_mean_from_partial_sums")

    o_acc = torch.empty(B, Hq, n, D, dtype=torch.float32, device=dev)
    m_acc = torch.empty(B, Hq, n, dtype=torch.float32, device=dev)
    l_acc = torch.empty(B, Hq, n, 2, dtype=torch.float32, device=dev)
    mine = torch.stack((kh, vh))
    order = list(range(world - 1, -1, -1))                     # last shard first
    grank = (lambda r_: dist.get_global_rank(group, r_)) if group is not None else (lambda r_: r_)

    def fetch(s_):
        buf = mine if s_ == rank else torch.empty_like(mine)
        return buf, dist.broadcast(buf, src=grank(s_), group=group, async_op=True)

    nxt = fetch(order[0])
    started = False
    for i, s_ in enumerate(order):
        buf, work = nxt
        if i + 1 < world:
            nxt = fetch(order[i + 1])                          # travels while this shard is attended
        work.wait()
        if is_causal and s_ > rank:
            continue                                           # entirely in the future of this rank's queries
        last = (s_ == 0)
        c = _cabi.Sage3Carry()
        if started:
            c.o_in, c.m_in, c.l_in = o_acc.data_ptr(), m_acc.data_ptr(), l_acc.data_ptr()
        if not last:
            c.o_out, c.m_out, c.l_out = o_acc.data_ptr(), m_acc.data_ptr(), l_acc.data_ptr()
        if is_causal:
            c.use_causal_shift, c.causal_shift = 1, (rank - s_) * n
        with torch.cuda.device(dev):
            _cabi.check(lib.sage3_prepass_kmean(C.byref(prob.desc), qh.data_ptr(), buf[0].data_ptr(), buf[1].data_ptr(),
                                                km.data_ptr(), prob.ws.buf.data_ptr(), stream), "sage3_prepass_kmean")
            _cabi.check(lib.sage3_attn_fwd_carry(C.byref(prob.desc), prob.ws.buf.data_ptr(), C.byref(c),
                                                 out.data_ptr() if last else None,
                                                 lse.data_ptr() if (last and lse is not None) else None, stream),
                        "sage3_attn_fwd_carry")
        started = True
    o = out if tensor_layout == "HND" else out.transpose(1, 2)
    return (o, lse) if return_lse else o


# ------------------------------------------------------------------------------------------------------
# peer-to-peer sequence parallelism (one NVSwitch node)
# ------------------------------------------------------------------------------------------------------
class _DeviceBytes:
    """Lets torch wrap device memory that the library allocated (CUDA array interface, no copy)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = dict(shape=(nbytes,), typestr="|u1", data=(ptr, False), version=3)


class PeerUlysses:
    """Sequence-parallel attention without all-to-alls, for ranks that are GPUs of one node.

    Every rank owns the token shard [rank * n, (rank + 1) * n) of all heads and computes attention for the heads
    [rank * H / P, (rank + 1) * H / P) over all tokens, exactly as `ulysses_attention` does; the result for a rank's
    tokens equals `ulysses_attention`'s and the single-GPU call's bit for bit.  The difference is the transport:

      * q, k, v shards are copied once into buffers that all ranks have mapped (or written there by the caller in the
        first place: `stage()` returns the views) -- barrier --
      * the pre-pass kernels read the rows they need directly from the owners' buffers (plain loads over NVLink),
      * the attention kernel's epilogue writes each output row directly into the output buffer of the rank that owns the
        token (plain stores over NVLink) -- barrier --
      * the rank returns a view of its own output buffer, [B, Hq, n, D].

    Buffers come in two sets used alternately, so a call may start while a slower rank still reads the previous
    call's buffers; the view returned by call i is overwritten by call i + 2.  Shapes are fixed at construction.
    The barriers are one-element NCCL all-reduces on the caller's stream (the host is not blocked).
    """

    def __init__(self, B: int, Hq: int, Hkv: int, tokens_per_rank: int, D: int, dtype: torch.dtype = torch.bfloat16,
                 group: dist.ProcessGroup | None = None, device: torch.device | None = None):
        import ctypes as C
        from . import _cabi
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > _cabi.MAX_PARTS:
            raise ValueError(f"PeerUlysses supports up to {_cabi.MAX_PARTS} ranks (one node)")
        if Hq % self.world or Hkv % self.world or Hq % Hkv:
            raise ValueError(f"head counts ({Hq}, {Hkv}) must be multiples of the group size {self.world}")
        self.B, self.Hq, self.Hkv, self.n, self.D, self.dtype = B, Hq, Hkv, tokens_per_rank, D, dtype
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        es = torch.empty(0, dtype=dtype).element_size()
        self._es = es
        q_bytes, kv_bytes = B * Hq * self.n * D * es, B * Hkv * self.n * D * es
        # one allocation per set: [q | k | v | out]
        self._offs = (0, q_bytes, q_bytes + kv_bytes, q_bytes + 2 * kv_bytes)
        self._set_bytes = 2 * q_bytes + 2 * kv_bytes
        lib = _cabi.lib()
        self._own, handles = [], []
        with torch.cuda.device(self.device):
            for _ in range(2):
                ptr, h = C.c_void_p(), C.create_string_buffer(64)
                _cabi.check(lib.sage3_shared_alloc(self._set_bytes, C.byref(ptr), h), "sage3_shared_alloc")
                self._own.append(ptr.value)
                handles.append(h.raw)
        gathered = [None] * self.world
        dist.all_gather_object(gathered, handles, group=group)
        self._peer = []                                    # [set][rank] -> device pointer valid in this process
        with torch.cuda.device(self.device):
            for s_ in range(2):
                row = []
                for r in range(self.world):
                    if r == self.rank:
                        row.append(self._own[s_])
                    else:
                        ptr = C.c_void_p()
                        _cabi.check(lib.sage3_shared_open(gathered[r][s_], C.byref(ptr)), "sage3_shared_open")
                        row.append(ptr.value)
                self._peer.append(row)
        self._views = []
        for s_ in range(2):
            raw = torch.as_tensor(_DeviceBytes(self._own[s_], self._set_bytes), device=self.device)
            o = self._offs
            q_v = raw[o[0]:o[1]].view(dtype).view(B, Hq, self.n, D)
            k_v = raw[o[1]:o[2]].view(dtype).view(B, Hkv, self.n, D)
            v_v = raw[o[2]:o[3]].view(dtype).view(B, Hkv, self.n, D)
            out_v = raw[o[3]:].view(dtype).view(B, Hq, self.n, D)
            self._views.append((q_v, k_v, v_v, out_v))
        self._flag = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._calls = 0
        self._prob = None
        dist.all_reduce(self._flag, group=group)            # every rank has mapped every buffer before anyone touches one
        torch.cuda.synchronize(self.device)

    def stage(self):
        """(q, k, v) views of the buffers the NEXT call reads: [B, Hq, n, D], [B, Hkv, n, D] x 2.  A caller that writes
        its projections there directly and then passes these very views to the call saves the staging copy."""
        return self._views[self._calls % 2][:3]

    def _parts(self, set_idx: int, which: int, head0: int, heads_total: int):
        from . import _cabi
        p = _cabi.Sage3Parts()
        p.parts, p.rows_per_part = self.world, self.n
        off = self._offs[which] + head0 * self.n * self.D * self._es
        for r in range(self.world):
            p.base[r] = self._peer[set_idx][r] + off
        return p

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool = False, sm_scale=None,
                 per_block_mean: bool = True) -> torch.Tensor:
        import ctypes as C
        from . import _cabi
        from .api import Sage3Problem
        set_idx = self._calls % 2
        self._calls += 1
        q_v, k_v, v_v, out_v = self._views[set_idx]
        for dst, src in ((q_v, q), (k_v, k), (v_v, v)):
            if src.data_ptr() != dst.data_ptr():
                dst.copy_(src)
        dist.all_reduce(self._flag, group=self.group)       # all shards staged (and every rank is done with this set's last use)
        P, hq_l, hkv_l, N = self.world, self.Hq // self.world, self.Hkv // self.world, self.world * self.n
        if self._prob is None:
            # descriptor and workspace of the local problem: hq_l heads over all N tokens, addressed inside every rank's
            # buffer with that buffer's strides ([B, H, n, D])
            self._prob = Sage3Problem.for_shape(self.B, hq_l, hkv_l, N, N, self.D, self.dtype, self.device, is_causal=is_causal,
                                                sm_scale=sm_scale, per_block_mean=per_block_mean,
                                                q_stride=(self.Hq * self.n * self.D, self.n * self.D, self.D),
                                                k_stride=(self.Hkv * self.n * self.D, self.n * self.D, self.D),
                                                o_stride=(self.Hq * self.n * self.D, self.n * self.D, self.D))
        prob = self._prob
        prob.desc.is_causal = int(bool(is_causal))
        lib = _cabi.lib()
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            qp = self._parts(set_idx, 0, self.rank * hq_l, self.Hq)
            kp = self._parts(set_idx, 1, self.rank * hkv_l, self.Hkv)
            vp = self._parts(set_idx, 2, self.rank * hkv_l, self.Hkv)
            op = self._parts(set_idx, 3, self.rank * hq_l, self.Hq)
            _cabi.check(lib.sage3_prepass_parts(C.byref(prob.desc), C.byref(qp), C.byref(kp), C.byref(vp),
                                                prob.ws.buf.data_ptr(), stream), "sage3_prepass_parts")
            _cabi.check(lib.sage3_attn_fwd_parts(C.byref(prob.desc), prob.ws.buf.data_ptr(), C.byref(op), None, stream),
                        "sage3_attn_fwd_parts")
        dist.all_reduce(self._flag, group=self.group)       # every rank's rows have arrived in every output buffer
        return out_v

    def close(self) -> None:
        """Unmaps the peers' buffers and frees this rank's (collective: every rank must call it)."""
        from . import _cabi
        if self._peer is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        lib = _cabi.lib()
        with torch.cuda.device(self.device):
            for s_ in range(2):
                for r in range(self.world):
                    if r != self.rank:
                        lib.sage3_shared_close(self._peer[s_][r])
            dist.barrier(group=self.group)
            self._views = None
            for ptr in self._own:
                lib.sage3_shared_free(ptr)
        self._peer = None
