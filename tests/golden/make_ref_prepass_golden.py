"""Records what the reference's own smoothing + NVFP4 quantization stage produces on a B200.

TEST INFRASTRUCTURE ONLY.  Needs a CUDA device of compute capability 10.0 and oracle/_ref/ filled by
oracle/build_ref_quant.py (the reference's unmodified fp4_quantization_4d.cu compiled for sm_100a, and its unmodified
sageattn3/api.py).  The reference's attention extension only runs on sm_120, so a stub module stands in for it; it is
never called.  For every case below the script feeds seeded inputs through the reference's
    preprocess_qkv            (api.py:75-92: K smoothing in place, padding, Triton block mean or global mean, delta_s)
    scale_and_quant_fp4 / _permute / _transpose   (api.py:94-116 -> fp4quant_cuda kernels)
and stores inputs and outputs, raw, in tests/golden/ref_prepass.pt.  tests/test_ref_pin.py then holds the CPU oracle
against these tensors.

Usage (on the GPU machine):  python tests/golden/make_ref_prepass_golden.py [--out PATH]
"""
from __future__ import annotations

import argparse
import importlib.util
import pathlib
import sys
import types

import torch

ROOT = pathlib.Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import sage3_oracle as O  # noqa: E402  (seeded input generator only)

REF = ROOT / "oracle" / "_ref"

CASES = [
    # BASELINE config 1: B=1, H=2, N=1024, D=128, bf16, K with a per-channel offset of std 3
    dict(name="config1", inputs=dict(B=1, Hq=2, Hkv=2, Nq=1024, Nk=1024, D=128, seed=1000, k_offset_std=3.0),
         dtype="bfloat16", per_block_mean=True),
    # ragged lengths (240 = 112 mod 128, 496 = 112 mod 128), D = 64, outlier channels as in config 3
    dict(name="ragged_d64", inputs=dict(B=1, Hq=2, Hkv=2, Nq=240, Nk=496, D=64, seed=1003, k_outlier_channels=4),
         dtype="bfloat16", per_block_mean=True),
    # one mean per head (per_block_mean=False), fp16, lengths = 16 mod 128
    dict(name="global_mean_fp16", inputs=dict(B=1, Hq=1, Hkv=1, Nq=272, Nk=400, D=128, seed=1004, k_offset_std=2.0),
         dtype="float16", per_block_mean=False),
    # fp16 with the Triton block mean, D = 64
    dict(name="block_mean_fp16_d64", inputs=dict(B=1, Hq=1, Hkv=1, Nq=384, Nk=256, D=64, seed=1005, k_offset_std=1.0),
         dtype="float16", per_block_mean=True),
]


def load_reference():
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    spec = importlib.util.spec_from_file_location("fp4quant_cuda", REF / "fp4quant_cuda.so")
    quant = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(quant)
    sys.modules["fp4quant_cuda"] = quant
    sys.modules["fp4attn_cuda"] = types.ModuleType("fp4attn_cuda")     # sm_120-only; imported by api.py, never called
    spec = importlib.util.spec_from_file_location("ref_sageattn3_api", REF / "ref_sageattn3_api.py")
    api = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(api)
    return api


def pad_128(x):
    pad = (-x.size(2)) % 128
    return x.contiguous() if pad == 0 else torch.nn.functional.pad(x, (0, 0, 0, pad), value=0).contiguous()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(ROOT / "tests" / "golden" / "ref_prepass.pt"))
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    assert torch.cuda.get_device_capability(dev) == (10, 0), "record the fixtures on a B200"
    api = load_reference()
    import triton
    out_cases = []
    for c in CASES:
        dt = getattr(torch, c["dtype"])
        q, k, v = O.make_inputs(dtype=dt, **c["inputs"])
        qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
        pbm = c["per_block_mean"]
        # the two means the reference forms on its way (same expressions, evaluated on their own so they can be stored)
        km = kd.mean(dim=-2, keepdim=True)                                   # api.py:84
        if pbm:
            _, qm = api.triton_group_mean(pad_128(qd))                       # api.py:87
        else:
            qm = pad_128(qd).mean(dim=-2, keepdim=True)                      # api.py:89
        q_s, k_s, v_p, delta = api.preprocess_qkv(qd.clone(), kd.clone(), vd.clone(), pbm)
        assert torch.equal(delta.to(dt).float(), delta), "delta_s is not exactly representable in the input type"
        q_codes, q_sf = api.scale_and_quant_fp4(q_s)
        k_codes, k_sf = api.scale_and_quant_fp4_permute(k_s)
        v_codes, v_sf = api.scale_and_quant_fp4_transpose(v_p)
        torch.cuda.synchronize()
        keep = lambda x: x.detach().cpu().contiguous().clone()
        rec = dict(name=c["name"], inputs=c["inputs"], dtype=c["dtype"], per_block_mean=pbm,
                   q=q, k=k, v=v, km=keep(km), qm=keep(qm), q_s=keep(q_s), k_s=keep(k_s), delta=keep(delta.to(dt)),
                   q_codes=keep(q_codes), q_sf=keep(q_sf.view(torch.uint8)), k_codes=keep(k_codes),
                   k_sf=keep(k_sf.view(torch.uint8)), v_codes=keep(v_codes), v_sf=keep(v_sf.view(torch.uint8)))
        out_cases.append(rec)
        fm = pad_128(qd).float().unflatten(2, (-1, 128)).mean(dim=3) if pbm else pad_128(qd).float().mean(dim=2, keepdim=True)
        d = (qm.float() - fm.to(dt).float()).abs()
        print(f"{c['name']}: recorded; qm differs from round(fp32 mean) in {(d > 0).float().mean().item():.3f} of the entries, "
              f"max |diff| {d.max().item():.3e} (|mean| max {fm.abs().max().item():.3e})")
    meta = dict(torch=str(torch.__version__), triton=str(triton.__version__), device=torch.cuda.get_device_name(dev),
                note="outputs of the reference's preprocess_qkv + fp4quant_cuda kernels, unmodified sources, built for sm_100a")
    torch.save(dict(meta=meta, cases=out_cases), args.out)
    print("wrote", args.out, meta)


if __name__ == "__main__":
    main()
