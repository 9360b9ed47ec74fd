"""Builds the reference's own NVFP4 quantization extension for sm_100a, from its sources where they lie.

TEST INFRASTRUCTURE ONLY.  The reference's `fp4quant_cuda` extension
(sageattention3_blackwell/sageattn3/quantization/fp4_quantization_4d.cu in the reference project) needs only
PyTorch and cuda_fp8.h: no CUTLASS, no architecture gate.  This recipe compiles that one file, unmodified, with the
flags of the reference's setup.py (sageattention3_blackwell/setup.py:88-110: -O3, --use_fast_math, the -U__CUDA_NO_*
switches, -DNDEBUG) for compute_100a, and stages the reference's unmodified Python front end
(sageattention3_blackwell/sageattn3/api.py) beside it, so that a machine with a B200 can run the reference's
smoothing + quantization stage and record what it produces (tests/golden/make_ref_prepass_golden.py).

Everything lands in oracle/_ref/ (kept out of version control): fp4quant_cuda*.so and ref_sageattn3_api.py.
Nothing of the product imports either.  The attention extension (`fp4attn_cuda`) is not built: it needs a CUTLASS
checkout and only executes on sm_120 (blackwell/api.cu:219-222).

Usage:  python oracle/build_ref_quant.py --reference-root <checkout of the reference project>
"""
from __future__ import annotations

import argparse
import os
import pathlib
import shutil
import sys

ROOT = pathlib.Path(__file__).resolve().parent.parent
OUT = ROOT / "oracle" / "_ref"

NVCC_FLAGS = [
    "-O3", "-std=c++17",
    "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT16_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT162_OPERATORS__", "-U__CUDA_NO_BFLOAT162_CONVERSIONS__",
    "--expt-relaxed-constexpr", "--expt-extended-lambda", "--use_fast_math", "-lineinfo",
    "-DNDEBUG", "-DQBLKSIZE=128", "-DKBLKSIZE=128", "-DCTA256", "-DDQINRMEM", "-DEXECMODE=0",
    "-gencode", "arch=compute_100a,code=sm_100a",
]


def build(reference_root: pathlib.Path, verbose: bool = False) -> pathlib.Path:
    pkg = reference_root / "sageattention3_blackwell" / "sageattn3"
    src = pkg / "quantization" / "fp4_quantization_4d.cu"
    api = pkg / "api.py"
    if not src.exists() or not api.exists():
        raise FileNotFoundError(f"{src} / {api}: not a checkout of the reference project")
    OUT.mkdir(parents=True, exist_ok=True)
    build_dir = OUT / "build_fp4quant"
    build_dir.mkdir(exist_ok=True)
    # torch adds its own -gencode from this list; an empty arch list would make it probe for a GPU
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load
    mod = load(name="fp4quant_cuda", sources=[str(src)], extra_cflags=["-O3", "-std=c++17"],
               extra_cuda_cflags=NVCC_FLAGS, extra_include_paths=[str(pkg)], build_directory=str(build_dir),
               verbose=verbose, is_python_module=False)
    del mod
    so = build_dir / "fp4quant_cuda.so"
    shutil.copy2(so, OUT / "fp4quant_cuda.so")
    shutil.copy2(api, OUT / "ref_sageattn3_api.py")       # unmodified; imported with a stub for fp4attn_cuda
    shutil.rmtree(build_dir)
    return OUT / "fp4quant_cuda.so"


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-root", required=True)
    ap.add_argument("-v", action="store_true")
    a = ap.parse_args()
    print(build(pathlib.Path(a.reference_root), a.v))
    sys.exit(0)
