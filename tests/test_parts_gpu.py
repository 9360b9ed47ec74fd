"""Token-split tensors (Sage3Parts) and the caller-supplied K mean, through the C ABI on one GPU: the pieces are separate
allocations here; in the sequence-parallel use they are buffers of other GPUs mapped into the process."""
import ctypes as C

import pytest
import torch

from oracle import sage3_oracle as O
from sageattention_b200 import Sage3Problem, _cabi, sageattn3

pytestmark = pytest.mark.gpu


def _parts(tensors, rows):
    p = _cabi.Sage3Parts()
    p.parts, p.rows_per_part = len(tensors), rows
    for i, t in enumerate(tensors):
        p.base[i] = t.data_ptr()
    return p


@pytest.mark.parametrize("B,Hq,Hkv,n,P,D,causal", [(2, 4, 2, 100, 3, 64, False), (1, 2, 2, 256, 2, 128, True), (1, 2, 1, 37, 8, 128, False)])
def test_split_tensors_equal_the_contiguous_call(cuda_device, B, Hq, Hkv, n, P, D, causal):
    N = n * P
    q, k, v = (t.to(cuda_device) for t in O.make_inputs(B, Hq, Hkv, N, N, D, seed=60 + n, k_offset_std=1.0))
    ref = sageattn3(q, k, v, is_causal=causal)
    # every piece [B, H, n, D] is its own allocation; 8 more heads of padding in front show that base pointers may be offset
    cut = lambda x: [x[:, :, i * n:(i + 1) * n].contiguous() for i in range(P)]
    qs, ks, vs = cut(q), cut(k), cut(v)
    outs = [torch.full((B, Hq, n, D), float("nan"), dtype=q.dtype, device=cuda_device) for _ in range(P)]
    prob = Sage3Problem.for_shape(B, Hq, Hkv, N, N, D, q.dtype, cuda_device, is_causal=causal,
                                  q_stride=(Hq * n * D, n * D, D), k_stride=(Hkv * n * D, n * D, D))
    lib, st = _cabi.lib(), torch.cuda.current_stream(cuda_device).cuda_stream
    qp, kp, vp, op = _parts(qs, n), _parts(ks, n), _parts(vs, n), _parts(outs, n)
    assert lib.sage3_prepass_parts(C.byref(prob.desc), C.byref(qp), C.byref(kp), C.byref(vp), prob.ws.buf.data_ptr(), st) == 0
    assert lib.sage3_attn_fwd_parts(C.byref(prob.desc), prob.ws.buf.data_ptr(), C.byref(op), None, st) == 0
    assert prob.check_status() == 0
    got = torch.cat(outs, dim=2)
    assert torch.equal(got, ref)


def test_parts_argument_checks(cuda_device):
    prob = Sage3Problem.for_shape(1, 2, 2, 256, 256, 64, torch.bfloat16, cuda_device)
    lib = _cabi.lib()
    x = torch.zeros(1, 2, 128, 64, dtype=torch.bfloat16, device=cuda_device)
    good = _parts([x, x], 128)
    short = _parts([x], 128)                               # one piece of 128 rows cannot hold 256 tokens
    assert lib.sage3_prepass_parts(C.byref(prob.desc), C.byref(short), C.byref(good), C.byref(good), prob.ws.buf.data_ptr(), None) == -2
    bad = _parts([x, x], 128)
    bad.parts = 9
    assert lib.sage3_attn_fwd_parts(C.byref(prob.desc), prob.ws.buf.data_ptr(), C.byref(bad), None, None) == -2
    assert lib.sage3_prepass_parts(C.byref(prob.desc), None, C.byref(good), C.byref(good), prob.ws.buf.data_ptr(), None) == -1


def test_prepass_with_supplied_k_mean(cuda_device):
    """The K mean of a longer sequence, supplied by the caller: a shard smoothed with it quantizes exactly as the same
    rows do inside the whole sequence."""
    from tests._util import read_workspace
    B, H, N, D = 1, 2, 1024, 128
    q, k, v = (t.to(cuda_device) for t in O.make_inputs(B, H, H, N, N, D, seed=77, k_offset_std=2.0))
    whole = Sage3Problem(q, k, v)
    whole.prepass()
    torch.cuda.synchronize()
    w = read_workspace(whole)
    km = w["km"].to(cuda_device)
    half = slice(512, 1024)
    kh, vh = k[:, :, half].contiguous(), v[:, :, half].contiguous()
    shard = Sage3Problem(q, kh, vh)
    st = torch.cuda.current_stream(cuda_device).cuda_stream
    rc = _cabi.lib().sage3_prepass_kmean(C.byref(shard.desc), q.data_ptr(), kh.data_ptr(), vh.data_ptr(), km.data_ptr(),
                                         shard.ws.buf.data_ptr(), st)
    assert rc == 0
    torch.cuda.synchronize()
    s = read_workspace(shard)
    assert torch.equal(s["km"], w["km"])
    assert torch.equal(s["k_codes"], w["k_codes"][:, :, half]) and torch.equal(s["k_sf"], w["k_sf"][:, :, half])
    assert torch.equal(s["delta"], w["delta"][..., half])
    assert torch.equal(s["vt_codes"], w["vt_codes"][..., half])


def _carry(o_in=None, m_in=None, l_in=None, o_out=None, m_out=None, l_out=None, shift=None):
    c = _cabi.Sage3Carry()
    for name, t in (("o_in", o_in), ("m_in", m_in), ("l_in", l_in), ("o_out", o_out), ("m_out", m_out), ("l_out", l_out)):
        setattr(c, name, None if t is None else t.data_ptr())
    if shift is not None:
        c.use_causal_shift, c.causal_shift = 1, shift
    return c


@pytest.mark.parametrize("B,Hq,Hkv,Nq,cuts,D,causal", [
    (1, 2, 2, 384, [0, 256, 640, 1000], 128, False),       # three key ranges, the last one ragged
    (2, 4, 2, 300, [0, 128, 300], 64, True),               # causal, GQA, Nq == Nk
    (1, 2, 1, 200, [0, 384, 768], 128, True),              # causal, Nk > Nq (bottom-right aligned)
])
def test_key_ranges_with_carried_state_equal_one_call(cuda_device, B, Hq, Hkv, Nq, cuts, D, causal):
    """One attention computed as several calls over consecutive key ranges, walked from the last range to the first
    with the accumulator state carried along: the same bits as the single call (same blocks, same order)."""
    from tests._util import read_workspace
    Nk = cuts[-1]
    q, k, v = (t.to(cuda_device) for t in O.make_inputs(B, Hq, Hkv, Nq, Nk, D, seed=90 + Nq, k_offset_std=1.5))
    whole = Sage3Problem(q, k, v, is_causal=causal, return_lse=True)
    ref = whole.run().clone()
    ref_lse = whole.lse.clone()
    torch.cuda.synchronize()
    km = read_workspace(whole)["km"].to(cuda_device)

    lib, st = _cabi.lib(), torch.cuda.current_stream(cuda_device).cuda_stream
    o_acc = torch.empty(B, Hq, Nq, D, dtype=torch.float32, device=cuda_device)
    m_acc = torch.empty(B, Hq, Nq, dtype=torch.float32, device=cuda_device)
    l_acc = torch.empty(B, Hq, Nq, 2, dtype=torch.float32, device=cuda_device)
    out = torch.full_like(q, float("nan"))
    lse = torch.empty(B, Hq, Nq, dtype=torch.float32, device=cuda_device)
    ranges = list(zip(cuts[:-1], cuts[1:]))[::-1]                      # last range first
    for idx, (k0, k1) in enumerate(ranges):
        ks, vs = k[:, :, k0:k1].contiguous(), v[:, :, k0:k1].contiguous()
        prob = Sage3Problem(q, ks, vs, is_causal=causal, out=out)
        assert lib.sage3_prepass_kmean(C.byref(prob.desc), q.data_ptr(), ks.data_ptr(), vs.data_ptr(), km.data_ptr(),
                                       prob.ws.buf.data_ptr(), st) == 0
        first, last = idx == 0, idx == len(ranges) - 1
        carry = _carry(*((None, None, None) if first else (o_acc, m_acc, l_acc)),
                       *((None, None, None) if last else (o_acc, m_acc, l_acc)),
                       shift=(Nk - Nq - k0) if causal else None)
        rc = lib.sage3_attn_fwd_carry(C.byref(prob.desc), prob.ws.buf.data_ptr(), C.byref(carry),
                                      out.data_ptr() if last else None, lse.data_ptr() if last else None, st)
        assert rc == 0
        assert prob.check_status() == 0
    assert torch.equal(out, ref)
    assert torch.equal(lse, ref_lse)
