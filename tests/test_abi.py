"""CPU tests of the C-ABI boundary: the library loads, exports what the header declares, validates arguments."""
import ctypes as C
import pathlib
import re

import pytest

from sageattention_b200 import _cabi

ROOT = pathlib.Path(__file__).resolve().parent.parent


def _desc(**kw):
    d = _cabi.Sage3Desc()
    base = dict(B=1, Hq=2, Hkv=2, Nq=1024, Nk=1024, D=128, dtype=_cabi.SAGE3_BF16, is_causal=0, per_block_mean=1)
    base.update(kw)
    for k_, v_ in base.items():
        setattr(d, k_, v_)
    n = max(base["Nq"], base["Nk"])
    for name in ("q_stride", "k_stride", "v_stride", "o_stride"):
        setattr(d, name, (C.c_int64 * 3)(base["Hq"] * n * base["D"], n * base["D"], base["D"]))
    return d


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "sage3_b200.h").read_text()
    declared = re.findall(r"SAGE3_API\s+[\w\s\*]+?\b(sage3_\w+)\s*\(", header)
    assert sorted(declared) == sorted(_cabi.EXPORTED)
    lib = _cabi.lib()
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.sage3_version() == _cabi.ABI_VERSION == 4


def test_strerror_is_total():
    lib = _cabi.lib()
    for code in range(-12, 2):
        assert len(lib.sage3_strerror(code)) > 0


def test_workspace_layout_config1():
    lib = _cabi.lib()
    d = _desc()
    w = _cabi.Sage3Workspace()
    assert lib.sage3_workspace_layout(C.byref(d), C.byref(w)) == 0
    assert (w.nq_pad, w.nk_pad, w.nqm, w.kchunks) == (1024, 1024, 8, 2)
    offs = [w.status, w.kpart, w.km, w.qm, w.delta, w.q_codes, w.q_sf, w.k_codes, w.k_sf, w.v_codes, w.v_sf, w.qkm, w.total_bytes]
    assert offs == sorted(offs) and all(o % 1024 == 0 for o in offs)
    assert w.q_sf - w.q_codes == 2 * 1024 * 64               # packed codes: D/2 bytes per row
    assert w.k_codes - w.q_sf == 2 * 8 * 2 * 512             # 2 heads x 8 tiles x 2 atoms x 512 bytes
    assert w.qkm - w.v_sf == 2 * 8 * 1024
    assert w.total_bytes - w.qkm == 2 * 1024 * 4                  # one fp32 per (head, padded query row)
    assert lib.sage3_workspace_bytes(C.byref(d)) == w.total_bytes


def test_ragged_and_global_mean_layout():
    lib = _cabi.lib()
    d = _desc(Nq=17776, Nk=17776, D=64, Hq=48, Hkv=48, B=2, per_block_mean=0)
    w = _cabi.Sage3Workspace()
    assert lib.sage3_workspace_layout(C.byref(d), C.byref(w)) == 0
    assert (w.nq_pad, w.nk_pad, w.nqm, w.kchunks) == (17792, 17792, 1, 35)


@pytest.mark.parametrize("kw,code", [
    (dict(D=96), -2), (dict(D=256), -2), (dict(Hq=3, Hkv=2), -2), (dict(Nq=0), -2), (dict(B=-1), -2),
    (dict(dtype=7), -3), (dict(Nk=1 << 25), -8),
    (dict(B=2048, Hq=64, Hkv=64, Nq=128, Nk=128), -8),          # B * Hq beyond the 65535 (batch, head) slabs of a launch
])
def test_validation_codes(kw, code):
    lib = _cabi.lib()
    d = _desc(**kw)
    w = _cabi.Sage3Workspace()
    assert lib.sage3_workspace_layout(C.byref(d), C.byref(w)) == code
    assert lib.sage3_workspace_bytes(C.byref(d)) == 0


def test_bad_stride_and_null():
    lib = _cabi.lib()
    d = _desc()
    d.q_stride[2] = 132                                     # not a multiple of 8 elements
    w = _cabi.Sage3Workspace()
    assert lib.sage3_workspace_layout(C.byref(d), C.byref(w)) == -4
    assert lib.sage3_workspace_layout(None, C.byref(w)) == -1
    assert lib.sage3_prepass(C.byref(_desc()), None, None, None, None, None) == -1
    assert lib.sage3_check_status(None, None, None) == -1


def test_python_surface_rejects_cpu_tensors():
    import torch
    from sageattention_b200 import sageattn3
    q = torch.zeros(1, 1, 128, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        sageattn3(q, q, q)
    with pytest.raises(NotImplementedError):
        sageattn3(q, q, q, attn_mask=torch.ones(1))
    with pytest.raises(RuntimeError):
        sageattn3(q, q, q, return_lse=True)


def test_varlen_entry_validates_before_touching_the_device():
    """sage3_fwd_varlen: null and misaligned arguments are refused with codes; the Python wrapper refuses host tensors
    and badly shaped cu_seqlens."""
    import torch
    from sageattention_b200 import sageattn_varlen
    lib = _cabi.lib()
    d = _desc(B=3)
    assert lib.sage3_fwd_varlen(C.byref(d), None, None, None, None, None, None, None, None, None) == -1
    assert lib.sage3_fwd_varlen(C.byref(d), 4, 4, 16, 16, 16, 16, None, None, None) == -1             # no workspace
    assert lib.sage3_fwd_varlen(C.byref(d), 2, 4, 16, 16, 16, 16, None, 256, None) == -5   # SAGE3_E_ALIGN: cu_seqlens_q not 4-byte aligned
    assert lib.sage3_fwd_varlen(C.byref(d), 4, 4, 8, 16, 16, 16, None, 256, None) == -5    # SAGE3_E_ALIGN: q not 16-byte aligned
    q = torch.zeros(10, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        sageattn_varlen(q, q, q, [0, 10], [0, 10])
    with pytest.raises(ValueError):
        sageattn_varlen(q.unsqueeze(0), q, q, [0, 10], [0, 10])
