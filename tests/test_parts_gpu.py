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
