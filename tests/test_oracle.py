"""CPU tests of the oracle: codecs against NVIDIA's host converters, hand-checkable cases, golden fixtures."""
import math
import pathlib

import numpy as np
import pytest
import torch

from oracle import sage3_oracle as O

GOLD = pathlib.Path(__file__).resolve().parent / "golden"


def test_codecs_match_nvidia_host_converters():
    d = np.load(GOLD / "codec_pin.npz")
    x = torch.from_numpy(d["x_bits"].view(np.float32).copy())
    assert torch.equal(O.e2m1_rn_satfinite(x), torch.from_numpy(d["e2m1"]))
    assert torch.equal(O.e4m3_rn_satfinite(x.abs())[0], torch.from_numpy(d["e4m3"]))


def test_e2m1_table_and_ties():
    vals = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    assert torch.equal(O.e2m1_rn_satfinite(vals), torch.arange(8, dtype=torch.uint8))
    assert torch.equal(O.e2m1_rn_satfinite(-vals[1:]), torch.arange(9, 16, dtype=torch.uint8))
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, 1e9])
    assert O.e2m1_decode(O.e2m1_rn_satfinite(ties)).tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, 6.0]
    assert torch.equal(O.e2m1_decode(torch.arange(16, dtype=torch.uint8))[:8], vals)


def test_e4m3_all_bytes_roundtrip_and_saturation():
    b = torch.arange(0, 0x7F, dtype=torch.uint8)                 # 0x7f is NaN in e4m3fn
    v = b.view(torch.float8_e4m3fn).to(torch.float32)
    rb, rv = O.e4m3_rn_satfinite(v)
    assert torch.equal(rb, b) and torch.equal(rv, v)
    assert O.e4m3_rn_satfinite(torch.tensor([449.0, 1e6]))[1].tolist() == [448.0, 448.0]


def test_nibble_packing_order():
    codes = torch.tensor([[1, 2, 3, 4]], dtype=torch.uint8)
    packed = O.pack_nibbles(codes)
    assert packed.tolist() == [[0x21, 0x43]]
    assert torch.equal(O.unpack_nibbles(packed), codes)


def test_microblock_quant_by_hand():
    x = torch.zeros(1, 16, dtype=torch.bfloat16)
    x[0, 0], x[0, 1], x[0, 2], x[0, 3] = 12.0, -6.0, 1.0, 0.4
    codes, sf, deq = O.quant_microblocks(x)
    assert sf.view(torch.float8_e4m3fn).float().item() == 2.0     # amax / 6
    # 12/2 = 6 -> code 7; -6/2 = -3 -> code 8|5; 1/2 = 0.5 -> 1; 0.4/2 = 0.2 -> 0
    assert codes[0, :4].tolist() == [7, 13, 1, 0]
    assert deq[0, :4].tolist() == [12.0, -6.0, 1.0, 0.0]


def test_single_block_attention_by_hand():
    """One query row, one KV block: every number can be followed by hand."""
    D = 64
    q = torch.zeros(1, 1, 1, D, dtype=torch.bfloat16)
    k = torch.zeros(1, 1, 2, D, dtype=torch.bfloat16)
    v = torch.zeros(1, 1, 2, D, dtype=torch.bfloat16)
    q[0, 0, 0, 0] = 8.0            # q block mean over the 128 padded rows = 8/128 = 1/16
    k[0, 0, 0, 0], k[0, 0, 1, 0] = 4.0, -4.0     # km = 0 -> k' = k
    v[0, 0, 0, :], v[0, 0, 1, :] = 1.0, 3.0
    pp = O.prepass(q, k, v)
    assert pp.km.float().abs().max() == 0
    assert pp.qm[0, 0, 0, 0].item() == 0.0625
    assert pp.delta[0, 0, 0, :2].tolist() == [0.25, -0.25]
    out = O.attention_from_prepass(pp)
    # S = q'.k' + delta = (8 - 1/16) * (+-4) + (+-1/4) = +-32 exactly; scale = 1/8 -> logits +-4
    w = math.exp(-8.0)
    expect = (1.0 + 3.0 * w) / (1.0 + w)
    assert abs(out[0, 0, 0, 0].item() - expect) < 2e-2            # FP4 P: weight e^-8 rounds to 0 or the first step
    ref = O.fp32_attention(q, k, v)
    assert abs(ref[0, 0, 0, 0].item() - expect) < 1e-4


@pytest.mark.parametrize("causal", [False, True])
def test_oracle_close_to_fp32_attention(causal):
    q, k, v = O.make_inputs(1, 2, 2, 256, 384, 64, seed=3, k_offset_std=1.0)
    out = O.sageattn3_oracle(q, k, v, is_causal=causal)
    ref = O.fp32_attention(q, k, v, is_causal=causal)
    assert O.cosine(out, ref) > 0.97 and O.rel_l1(out, ref) < 0.25   # FP4 noise level, not a parity gate


def test_smoothing_helps_with_channel_offset():
    q, k, v = O.make_inputs(1, 1, 1, 256, 256, 128, seed=9, k_offset_std=3.0)
    ref = O.fp32_attention(q, k, v)
    good = O.rel_l1(O.sageattn3_oracle(q, k, v), ref)
    pp = O.prepass(q, k, v, km_override=torch.zeros(1, 1, 128))
    bad = O.rel_l1(O.attention_from_prepass(pp), ref)
    assert good < bad


def test_row_sampling_is_exact():
    q, k, v = O.make_inputs(1, 2, 1, 300, 300, 64, seed=11, k_offset_std=1.0)
    pp = O.prepass(q, k, v)
    full = O.attention_from_prepass(pp, is_causal=True)
    part = O.attention_from_prepass(pp, is_causal=True, q_rows=slice(128, 256))
    assert torch.equal(full[:, :, 128:256], part)


def test_layouts_gqa_and_ragged_rows():
    q, k, v = O.make_inputs(2, 4, 2, 200, 333, 64, seed=5)
    a = O.sageattn3_oracle(q, k, v)
    b = O.sageattn3_oracle(q.transpose(1, 2).contiguous(), k.transpose(1, 2).contiguous(),
                           v.transpose(1, 2).contiguous(), tensor_layout="NHD")
    assert a.shape == (2, 4, 200, 64) and torch.equal(a, b.transpose(1, 2))
    # causal with more queries than keys: the first Nq - Nk rows see nothing and must be exactly zero
    q2, k2, v2 = O.make_inputs(1, 1, 1, 200, 72, 64, seed=6)
    c = O.sageattn3_oracle(q2, k2, v2, is_causal=True)
    assert c[0, 0, :128].abs().max() == 0 and c[0, 0, 128:].abs().max() > 0
    assert not torch.isnan(c.float()).any()


def test_golden_fixtures():
    """Outputs of this oracle on seeded inputs, stored by tests/golden/make_golden.py: guards against drift."""
    g = torch.load(GOLD / "sage3_small.pt")
    for case in g["cases"]:
        q, k, v = O.make_inputs(**case["inputs"])
        out = O.sageattn3_oracle(q, k, v, is_causal=case["is_causal"], per_block_mean=case["per_block_mean"])
        assert torch.equal(out, case["out"]), case["name"]
        pp = O.prepass(q, k, v, per_block_mean=case["per_block_mean"])
        assert torch.equal(O.pack_nibbles(pp.q_codes)[0, 0, :8], case["q_codes_head"])
        assert torch.equal(pp.k_sf[0, 0, :8], case["k_sf_head"])


def test_lse_close_to_fp32():
    """The oracle's log-sum-exp (quantized scores + sm_scale * q.km) tracks the fp32 value of the unquantized inputs."""
    q, k, v = O.make_inputs(1, 4, 2, 300, 300, 64, seed=5, k_offset_std=1.0)
    _, lse = O.sageattn3_oracle(q, k, v, is_causal=True, return_lse=True)
    ref = O.fp32_lse(q, k, is_causal=True)
    assert lse.shape == (1, 4, 300)
    assert (lse - ref).abs().max() < 0.5 and (lse - ref).abs().mean() < 0.05
