"""GPU test of sage3_kmean_noalloc, the entry point for callers that may not allocate device memory (a serving
engine whose pool owns all of it, a loop that cannot afford cudaMalloc's synchronization): its scratch is a
fixed array inside the library.  Called through the C ABI twice in a row, with different inputs, and compared
with what the regular pre-pass leaves in its workspace -- same kernels, same summation order, so the bits
must agree.  The file name makes pytest collect it last."""
import ctypes as C

import pytest
import torch

from oracle import sage3_oracle as O
from sageattention_b200 import Sage3Problem, _cabi
from tests._util import read_workspace

pytestmark = pytest.mark.gpu


def _km_both_ways(device, B, H, Hkv, N, D, dtype, seed):
    q, k, v = O.make_inputs(B, H, Hkv, 128, N, D, seed=seed, dtype=dtype, k_offset_std=2.0)
    qd, kd, vd = q.to(device), k.to(device), v.to(device)
    prob = Sage3Problem(qd, kd, vd)
    prob.prepass()                                            # existing entry point: km lands in the workspace
    torch.cuda.synchronize()
    km_ref = read_workspace(prob)["km"]
    km_new = torch.full((B, Hkv, D), float("nan"), dtype=dtype, device=device)
    rc = _cabi.lib().sage3_kmean_noalloc(C.byref(prob.desc), kd.data_ptr(), km_new.data_ptr(),
                                         torch.cuda.current_stream(device).cuda_stream)
    assert rc == 0, _cabi.lib().sage3_strerror(rc)
    torch.cuda.synchronize()
    return km_new.cpu(), km_ref, k


def test_no_alloc_kmean_matches_prepass_twice(cuda_device):
    # first call: several chunks per head; second call: other data, other shape, fewer chunks -- what the first
    # call left in the shared scratch must not show through
    for (B, H, Hkv, N, D, dt, seed) in [(2, 4, 2, 1500, 128, torch.bfloat16, 11), (1, 3, 3, 200, 64, torch.float16, 12)]:
        km_new, km_ref, k = _km_both_ways(cuda_device, B, H, Hkv, N, D, dt, seed)
        assert torch.equal(km_new, km_ref)                   # bit for bit against the existing entry point
        oracle = k.float().mean(dim=-2)
        assert (km_new.float() - oracle).abs().max() <= 2 * torch.finfo(dt).eps * oracle.abs().max() + 1e-6


def test_no_alloc_kmean_rejects_oversize(cuda_device):
    d = _cabi.Sage3Desc()
    d.B, d.Hq, d.Hkv, d.Nq, d.Nk, d.D = 64, 64, 64, 128, 1 << 20, 128      # 64 * 64 * 2048 chunks * 128 floats
    d.dtype = _cabi.SAGE3_BF16
    d.k_stride = (C.c_int64 * 3)(64 * (1 << 20) * 128, (1 << 20) * 128, 128)
    dummy = torch.zeros(64, dtype=torch.bfloat16, device=cuda_device)
    rc = _cabi.lib().sage3_kmean_noalloc(C.byref(d), dummy.data_ptr(), dummy.data_ptr(), None)
    assert rc == -8
    assert b"limit" in _cabi.lib().sage3_strerror(rc)
