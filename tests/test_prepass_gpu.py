"""GPU parity of the pre-pass, through the C ABI: the Q block means bit for bit (a 16-bit sum in the reference's order),
the fp32-accumulated means (K, and Q when per_block_mean is off) within one ulp of the oracle's, and everything
downstream of the means (smoothed values -> codes, scale bytes, delta_s) bit for bit / within one ulp."""
import pytest
import torch

from oracle import sage3_oracle as O
from sageattention_b200 import Sage3Problem
from tests._util import canon, read_workspace

pytestmark = pytest.mark.gpu

CASES = [
    # B, Hq, Hkv, Nq, Nk, D, dtype, per_block_mean, layout
    (1, 2, 2, 1024, 1024, 128, torch.bfloat16, True, "HND"),      # BASELINE config 1 shape
    (2, 4, 2, 200, 333, 64, torch.bfloat16, True, "HND"),         # ragged, GQA, D = 64
    (1, 2, 1, 130, 144, 128, torch.float16, True, "NHD"),         # fp16, NHD, Nk % 128 == 16
    (1, 3, 3, 272, 1200, 64, torch.bfloat16, False, "HND"),       # one mean per head, several K chunks
    (1, 8, 2, 640, 640, 128, torch.bfloat16, True, "NHD"),        # GQA group of 4
]


def _ulp_close(a, b, ulps=1):
    a32, b32 = a.float(), b.float()
    eps = torch.finfo(a.dtype).eps
    tol = ulps * eps * torch.maximum(a32.abs(), b32.abs()).clamp_min(torch.finfo(a.dtype).tiny)
    return bool(((a32 - b32).abs() <= tol).all())


@pytest.mark.parametrize("B,Hq,Hkv,Nq,Nk,D,dt,pbm,layout", CASES)
def test_prepass_matches_oracle(cuda_device, B, Hq, Hkv, Nq, Nk, D, dt, pbm, layout):
    q, k, v = O.make_inputs(B, Hq, Hkv, Nq, Nk, D, seed=7 + Nq, dtype=dt, k_offset_std=2.0)
    to_dev = (lambda t: t.transpose(1, 2).contiguous().to(cuda_device)) if layout == "NHD" else (lambda t: t.to(cuda_device))
    qd, kd, vd = to_dev(q), to_dev(k), to_dev(v)
    k_before = kd.clone()
    prob = Sage3Problem(qd, kd, vd, tensor_layout=layout, per_block_mean=pbm)
    prob.prepass()
    torch.cuda.synchronize()
    assert torch.equal(kd, k_before), "inputs must not be modified"
    ws = read_workspace(prob)

    ref0 = O.prepass(q, k, v, per_block_mean=pbm)
    assert _ulp_close(ws["km"], ref0.km), "K mean"
    if pbm:
        # the block mean is a 16-bit sum in the reference's (Triton) order: identical, not just close
        assert torch.equal(ws["qm"], ref0.qm), "Q block mean"
    else:
        assert _ulp_close(ws["qm"], ref0.qm), "Q mean"
    # everything after the means, with the device's means substituted: must be identical
    ref = O.prepass(q, k, v, per_block_mean=pbm, km_override=ws["km"], qm_override=ws["qm"])
    assert torch.equal(ws["q_sf"], ref.q_sf), "Q scale bytes"
    assert torch.equal(ws["k_sf"], ref.k_sf), "K scale bytes"
    assert torch.equal(ws["vt_sf"], ref.vt_sf), "V scale bytes"
    assert ws["vt_sf_pad"].numel() == 0 or ws["vt_sf_pad"].abs().max() == 0   # rows >= D of a 128-row atom
    assert torch.equal(canon(ws["q_codes"]), canon(ref.q_codes)), "Q codes"
    assert torch.equal(canon(ws["k_codes"]), canon(ref.k_codes)), "K codes"
    assert torch.equal(canon(ws["vt_codes"]), canon(ref.vt_codes)), "V codes"
    # delta_s: fp32 accumulation order differs -> at most one ulp of the 16-bit result (plus an absolute floor
    # where the sum cancels)
    d_ref = ref.delta
    d_dev = ws["delta"].float()
    eps = torch.finfo(dt).eps
    scale = (ws["qm"].float().abs().unsqueeze(-2) * 1.0).amax()      # crude magnitude of the products
    tol = eps * d_ref.abs() + 1e-3 * eps * scale * D
    bad = (d_dev - d_ref).abs() > tol + eps * d_ref.abs()
    assert bad.float().mean() < 1e-3, f"delta_s mismatch fraction {bad.float().mean():.2e}"
    assert (d_dev - d_ref).abs().max() <= 4 * eps * d_ref.abs().max() + 1e-6


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("pbm", [True, False])
def test_packed_16bit_arithmetic_equals_fp32_then_round(cuda_device, dt, pbm):
    """The kernels subtract the means, add the chain sums of the block mean and take the microblock maxima on packed
    16-bit pairs (one rounding to the input type per operation); the oracle computes in fp32 and rounds.  The two must
    agree bit for bit also where operands differ by many binades: channels scaled from 2^-12 to 2^6, means far larger or
    far smaller than the values they are subtracted from, exact cancellations."""
    B, H, N, D = 1, 2, 512, 128
    g = torch.Generator().manual_seed(77)
    scale = torch.pow(2.0, torch.randint(-12, 7, (1, H, 1, D), generator=g).float())
    q = (torch.randn(B, H, N, D, generator=g) * scale + torch.randn(1, H, 1, D, generator=g) * scale.flip(-1)).to(dt)
    k = (torch.randn(B, H, N, D, generator=g) * scale.flip(-1) + 3 * torch.randn(1, H, 1, D, generator=g) * scale).to(dt)
    k[:, :, :, 5] = k[:, :, :1, 5]                       # a constant channel: k - mean cancels exactly
    q[:, :, 128:256, 9] = q[:, :, 128:129, 9]            # a constant channel inside one 128-row block
    v = (torch.randn(B, H, N, D, generator=g) * scale).to(dt)
    prob = Sage3Problem(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), per_block_mean=pbm)
    prob.prepass()
    torch.cuda.synchronize()
    assert prob.check_status() == 0
    ws = read_workspace(prob)
    ref0 = O.prepass(q, k, v, per_block_mean=pbm)
    if pbm:
        assert torch.equal(ws["qm"], ref0.qm), "Q block mean (16-bit chain sums)"
    ref = O.prepass(q, k, v, per_block_mean=pbm, km_override=ws["km"], qm_override=ws["qm"])
    for name in ("q_sf", "k_sf", "vt_sf"):
        assert torch.equal(ws[name], getattr(ref, name)), name
    for name in ("q_codes", "k_codes", "vt_codes"):
        assert torch.equal(canon(ws[name]), canon(getattr(ref, name))), name
