"""Writes tests/golden/sage3_small.pt: outputs of the CPU oracle on small seeded cases.

The reference ships no golden vectors and its kernels cannot run here or on the test machine, so these
fixtures come from the oracle itself; they pin its behaviour against accidental change.
Usage:  python tests/golden/make_golden.py
"""
import pathlib
import sys

import torch

ROOT = pathlib.Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import sage3_oracle as O  # noqa: E402

CASES = [
    dict(name="c1_like", inputs=dict(B=1, Hq=2, Hkv=2, Nq=256, Nk=256, D=128, seed=1000, k_offset_std=3.0),
         is_causal=False, per_block_mean=True),
    dict(name="ragged_gqa_causal", inputs=dict(B=1, Hq=4, Hkv=2, Nq=200, Nk=333, D=64, seed=1001, k_offset_std=1.0),
         is_causal=True, per_block_mean=True),
    dict(name="global_mean", inputs=dict(B=2, Hq=1, Hkv=1, Nq=130, Nk=144, D=64, seed=1002, k_outlier_channels=4),
         is_causal=False, per_block_mean=False),
]


def main():
    out_cases = []
    for c in CASES:
        q, k, v = O.make_inputs(**c["inputs"])
        pp = O.prepass(q, k, v, per_block_mean=c["per_block_mean"])
        out = O.attention_from_prepass(pp, is_causal=c["is_causal"])
        out_cases.append(dict(c, out=out, q_codes_head=O.pack_nibbles(pp.q_codes)[0, 0, :8].clone(),
                              k_sf_head=pp.k_sf[0, 0, :8].clone()))
    torch.save(dict(cases=out_cases), ROOT / "tests" / "golden" / "sage3_small.pt")
    print("wrote", len(out_cases), "cases")


if __name__ == "__main__":
    main()
