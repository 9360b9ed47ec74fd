"""The CPU oracle's smoothing + quantization stage against what the reference itself produces.

tests/golden/ref_prepass.pt holds outputs of the reference's own code -- its unmodified `preprocess_qkv` (K smoothing
in place, padding, the Triton block-mean kernel or the global mean, delta_s) and its unmodified fp4_quantization_4d.cu
kernels compiled for sm_100a -- recorded on a B200 by tests/golden/make_ref_prepass_golden.py.  The reference stores K
with its rows permuted inside groups of 32 and all scale bytes in 64-row atoms (artefacts of its sm_120 register
layout); tests/_refmap.py maps both back to natural order.

Bars: means, smoothed tensors, E2M1 codes and E4M3 scale bytes bit for bit; delta_s (a bf16 GEMM with fp32
accumulation in cuBLAS's order) within one unit in the last place of the 16-bit result.
"""
import pathlib

import pytest
import torch

from oracle import sage3_oracle as O
from tests._refmap import deatomize_sf64, k_row_of_stored_row, unpermute_k_rows

FIX = pathlib.Path(__file__).resolve().parent / "golden" / "ref_prepass.pt"
CASES = torch.load(FIX)["cases"]


def _canon(codes):
    return torch.where(codes == 8, torch.zeros_like(codes), codes)      # -0 and +0 are the same number


def test_index_maps():
    src = k_row_of_stored_row(64)
    # the order the reference's source states for one group of 32 (fp4_quantization_4d.cu:162)
    assert src[:32].tolist() == [0, 1, 8, 9, 16, 17, 24, 25, 2, 3, 10, 11, 18, 19, 26, 27,
                                 4, 5, 12, 13, 20, 21, 28, 29, 6, 7, 14, 15, 22, 23, 30, 31]
    assert src[32:].tolist() == [x + 32 for x in src[:32].tolist()]
    x = torch.arange(64 * 3).reshape(64, 3)
    assert torch.equal(unpermute_k_rows(x[src]), x)
    # scale atoms: byte (c // 4) * 256 + (r % 16) * 16 + (r // 16) * 4 + c % 4 inside a 64-row group
    rows, cols = 128, 8
    flat = torch.zeros(rows * cols, dtype=torch.int64)
    for r in range(rows):
        for c in range(cols):
            off = (r // 64) * 64 * cols + (c // 4) * 256 + (r % 16) * 16 + ((r % 64) // 16) * 4 + c % 4
            flat[off] = r * cols + c
    assert torch.equal(deatomize_sf64(flat.reshape(rows, cols)), torch.arange(rows * cols).reshape(rows, cols))


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_prepass_equals_reference_output(case):
    dt = getattr(torch, case["dtype"])
    pp = O.prepass(case["q"], case["k"], case["v"], per_block_mean=case["per_block_mean"])
    # means (api.py:84, 87-89): bit for bit, from the raw inputs
    assert torch.equal(pp.km, case["km"].squeeze(-2)), "K mean"
    assert torch.equal(pp.qm, case["qm"]), "Q mean"
    # smoothed, padded tensors (api.py:84-90)
    assert torch.equal(pp.k_s, case["k_s"]), "smoothed K"
    assert torch.equal(pp.q_s, case["q_s"]), "smoothed Q"
    # delta_s (api.py:91): one unit in the last place of the 16-bit result, and nearly always identical
    d_ref, d_or = case["delta"].float(), pp.delta
    eps = torch.finfo(dt).eps
    assert ((d_ref - d_or).abs() <= eps * torch.maximum(d_ref.abs(), d_or.abs())).all(), "delta_s beyond one ulp"
    assert (d_ref != d_or).float().mean() < 0.01
    # codes and scale bytes (fp4_quantization_4d.cu:133-386), mapped to natural order
    q_codes = O.unpack_nibbles(case["q_codes"])
    k_codes = unpermute_k_rows(O.unpack_nibbles(case["k_codes"]))
    v_codes = O.unpack_nibbles(case["v_codes"])
    q_sf, k_sf, v_sf = deatomize_sf64(case["q_sf"]), unpermute_k_rows(deatomize_sf64(case["k_sf"])), deatomize_sf64(case["v_sf"])
    assert torch.equal(q_sf, pp.q_sf) and torch.equal(k_sf, pp.k_sf) and torch.equal(v_sf, pp.vt_sf), "scale bytes"
    assert torch.equal(_canon(q_codes), _canon(pp.q_codes)), "Q codes"
    assert torch.equal(_canon(k_codes), _canon(pp.k_codes)), "K codes"
    assert torch.equal(_canon(v_codes), _canon(pp.vt_codes)), "V codes"


def test_fp32_block_mean_is_not_what_the_reference_computes():
    """The more accurate alternative (fp32 sum, one rounding) differs from the reference's 16-bit sum in most entries:
    the reason the oracle and the CUDA pre-pass follow the Triton kernel's order."""
    case = CASES[0]
    pp = O.prepass(case["q"], case["k"], case["v"], block_mean="fp32")
    frac = (pp.qm != case["qm"]).float().mean().item()
    assert 0.3 < frac < 0.95
