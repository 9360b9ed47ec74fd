"""Builds oracle/codec_pin.cu (host-only program around NVIDIA's cuda_fp4.h / cuda_fp8.h converters),
runs it and stores its known answers in tests/golden/codec_pin.npz.

TEST INFRASTRUCTURE ONLY.  Usage:  python oracle/make_codec_pin.py
"""
import pathlib
import subprocess

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parent.parent


def main() -> None:
    out_dir = ROOT / "oracle" / "_ref"
    out_dir.mkdir(parents=True, exist_ok=True)
    exe = out_dir / "codec_pin"
    subprocess.check_call(["nvcc", "-O1", "-o", str(exe), str(ROOT / "oracle" / "codec_pin.cu")])
    txt = subprocess.check_output([str(exe)], text=True)
    rows = np.array([[int(t) for t in line.split()] for line in txt.splitlines()], dtype=np.uint32)
    np.savez_compressed(ROOT / "tests" / "golden" / "codec_pin.npz",
                        x_bits=rows[:, 0], e2m1=rows[:, 1].astype(np.uint8), e4m3=rows[:, 2].astype(np.uint8))
    print(f"wrote {rows.shape[0]} known answers")


if __name__ == "__main__":
    main()
