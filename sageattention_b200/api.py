"""Host-side mirror of the reference's Python call surface, in front of the sm_100a C-ABI library.

Keeps the keyword surface of
  sageattn3_blackwell(q, k, v, attn_mask=None, is_causal=False, per_block_mean=True, **kwargs)
      (reference: sageattention3_blackwell/sageattn3/api.py:131-152)
  sageattn(q, k, v, tensor_layout="HND", is_causal=False, sm_scale=None, return_lse=False, **kwargs)
  sageattn_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, is_causal=False, sm_scale=None, **kwargs)
      (reference: sageattention/core.py:79-157)
so the function can be patched over F.scaled_dot_product_attention or called from an attention
processor exactly like the reference's.  Differences, all deliberate:
  * inputs are never modified (the reference smooths k in place, api.py:84);
  * no fallback: an unsupported head dim, device or a missing library raises (the reference falls back to
    torch SDPA for D >= 256, api.py:132-134, and the v2 dispatcher raises on sm_100, core.py:156-157);
  * attn_mask other than None raises (the reference ignores it silently);
  * GQA (Hq a multiple of Hkv), Nq != Nk, "NHD" layout and a per-head sm_scale tensor are accepted;
  * the causal mask is bottom-right aligned on the real lengths (key j visible to query i iff j <= i + Nk - Nq); the
    reference aligns on the lengths padded to 128, which is the same whenever both are multiples of 128.
PyTorch is used for device memory and the current stream only.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _cabi

_DTYPES = {torch.float16: _cabi.SAGE3_FP16, torch.bfloat16: _cabi.SAGE3_BF16}


def _bhn_strides(x: torch.Tensor, tensor_layout: str) -> tuple[int, int, int]:
    s = x.stride()
    return (s[0], s[1], s[2]) if tensor_layout == "HND" else (s[0], s[2], s[1])


def _usable(x: torch.Tensor) -> bool:
    return x.stride(-1) == 1 and all(st % 8 == 0 for st in x.stride()[:-1]) and x.data_ptr() % 16 == 0


@dataclass
class Workspace:
    """Caller-owned scratch + quantized operands of one problem shape (see Sage3Workspace in the C header)."""
    buf: torch.Tensor            # uint8
    layout: _cabi.Sage3Workspace

    def region(self, name: str, nbytes: int | None = None) -> torch.Tensor:
        off = getattr(self.layout, name)
        return self.buf[off: off + nbytes] if nbytes is not None else self.buf[off:]


CACHED_WORKSPACE = object()      # `workspace=` value: take the per-(device, stream) buffer the functional entry points share


class Sage3Problem:
    """Shapes, strides and workspace of one call; reusable while shapes, strides and dtype stay the same."""

    def __init__(self, q, k, v, tensor_layout="HND", is_causal=False, sm_scale=None, per_block_mean=True,
                 out: torch.Tensor | None = None, workspace: torch.Tensor | None = None, return_lse: bool = False):
        if tensor_layout not in ("HND", "NHD"):
            raise ValueError(f"tensor_layout must be 'HND' or 'NHD', got {tensor_layout!r}")
        for name, t in (("q", q), ("k", k), ("v", v)):
            if t.dim() != 4:
                raise ValueError(f"{name} must have 4 dimensions, got {t.dim()}")
            if not t.is_cuda:
                raise RuntimeError(f"{name} must be a CUDA tensor: sageattention_b200 has no CPU path")
        if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
            raise TypeError("q, k, v must share dtype torch.float16 or torch.bfloat16")
        if not (q.device == k.device == v.device):
            raise RuntimeError("q, k, v must be on the same device")
        if torch.cuda.get_device_capability(q.device) != (10, 0):
            raise RuntimeError("sageattention_b200 runs on compute capability 10.0 (B200) only")
        hd, nd = (1, 2) if tensor_layout == "HND" else (2, 1)
        B, Hq, Nq, D = q.shape[0], q.shape[hd], q.shape[nd], q.shape[3]
        Hkv, Nk = k.shape[hd], k.shape[nd]
        if k.shape[0] != B or v.shape != k.shape or k.shape[3] != D:
            raise ValueError("k and v must have the shape of q except for the head and sequence dimensions")
        if D not in (64, 128):
            raise ValueError(f"head dim must be 64 or 128, got {D}")
        if Hq % Hkv != 0:
            raise ValueError(f"number of query heads ({Hq}) must be a multiple of kv heads ({Hkv})")
        self.q = q if _usable(q) else q.contiguous()
        self.k = k if _usable(k) else k.contiguous()
        self.v = v if _usable(v) else v.contiguous()
        if out is None:
            out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        elif out.shape != q.shape or out.dtype != q.dtype or not _usable(out):
            raise ValueError("out must match q in shape and dtype, with 16-byte aligned rows")
        self.out = out
        # natural-log log-sum-exp of the scaled scores per query row, [B, Hq, Nq] fp32 (sageattention/core.py:327)
        self.lse = torch.empty(B, Hq, Nq, dtype=torch.float32, device=q.device) if return_lse else None
        self.tensor_layout = tensor_layout
        self.device = q.device

        d = _cabi.Sage3Desc()
        d.B, d.Hq, d.Hkv, d.Nq, d.Nk, d.D = B, Hq, Hkv, Nq, Nk, D
        d.dtype = _DTYPES[q.dtype]
        d.is_causal = int(bool(is_causal))
        d.per_block_mean = int(bool(per_block_mean))
        d.q_stride = (C.c_int64 * 3)(*_bhn_strides(self.q, tensor_layout))
        d.k_stride = (C.c_int64 * 3)(*_bhn_strides(self.k, tensor_layout))
        d.v_stride = (C.c_int64 * 3)(*_bhn_strides(self.v, tensor_layout))
        d.o_stride = (C.c_int64 * 3)(*_bhn_strides(self.out, tensor_layout))
        self._scale_tensor = None
        if sm_scale is None:
            d.sm_scale = 0.0
        elif isinstance(sm_scale, torch.Tensor) and sm_scale.numel() > 1:
            if sm_scale.numel() != Hq:
                raise ValueError(f"a per-head sm_scale must have {Hq} elements")
            self._scale_tensor = sm_scale.detach().to(device=q.device, dtype=torch.float32).contiguous()
            d.sm_scale_per_head = self._scale_tensor.data_ptr()
        else:
            d.sm_scale = float(sm_scale)
            if not d.sm_scale > 0:
                raise ValueError("sm_scale must be positive")
        self.desc = d

        lay = _cabi.Sage3Workspace()
        _cabi.check(_cabi.lib().sage3_workspace_layout(C.byref(d), C.byref(lay)), "sage3_workspace_layout")
        if workspace is CACHED_WORKSPACE:
            workspace = _shared_buffer(q.device, lay.total_bytes + 256)
        elif workspace is None:
            workspace = torch.empty(lay.total_bytes + 256, dtype=torch.uint8, device=q.device)
        elif workspace.numel() < lay.total_bytes + 256 or workspace.dtype != torch.uint8 or workspace.device != q.device:
            raise ValueError(f"workspace must be a uint8 CUDA tensor of at least {lay.total_bytes + 256} bytes")
        shift = (-workspace.data_ptr()) % 256
        self.ws = Workspace(workspace[shift: shift + lay.total_bytes], lay)

    @classmethod
    def for_shape(cls, B: int, Hq: int, Hkv: int, Nq: int, Nk: int, D: int, dtype: torch.dtype, device: torch.device,
                  is_causal: bool = False, sm_scale=None, per_block_mean: bool = True, q_stride=None, k_stride=None,
                  v_stride=None, o_stride=None) -> "Sage3Problem":
        """A problem described by its shape alone (descriptor + workspace, no tensors): for callers that hand the
        buffers to the library themselves, e.g. token-split buffers (`sage3_prepass_parts`).  Strides are element
        strides for (batch, head, token); default: contiguous [B, H, N, D]."""
        if dtype not in _DTYPES:
            raise TypeError("dtype must be torch.float16 or torch.bfloat16")
        if torch.cuda.get_device_capability(device) != (10, 0):
            raise RuntimeError("sageattention_b200 runs on compute capability 10.0 (B200) only")
        self = cls.__new__(cls)
        self.q = self.k = self.v = self.out = self.lse = None
        self.tensor_layout, self.device, self._scale_tensor = "HND", device, None
        d = _cabi.Sage3Desc()
        d.B, d.Hq, d.Hkv, d.Nq, d.Nk, d.D = B, Hq, Hkv, Nq, Nk, D
        d.dtype = _DTYPES[dtype]
        d.is_causal, d.per_block_mean = int(bool(is_causal)), int(bool(per_block_mean))
        d.q_stride = (C.c_int64 * 3)(*(q_stride or (Hq * Nq * D, Nq * D, D)))
        d.k_stride = (C.c_int64 * 3)(*(k_stride or (Hkv * Nk * D, Nk * D, D)))
        d.v_stride = (C.c_int64 * 3)(*(v_stride or k_stride or (Hkv * Nk * D, Nk * D, D)))
        d.o_stride = (C.c_int64 * 3)(*(o_stride or q_stride or (Hq * Nq * D, Nq * D, D)))
        d.sm_scale = 0.0 if sm_scale is None else float(sm_scale)
        self.desc = d
        lay = _cabi.Sage3Workspace()
        _cabi.check(_cabi.lib().sage3_workspace_layout(C.byref(d), C.byref(lay)), "sage3_workspace_layout")
        workspace = torch.empty(lay.total_bytes + 256, dtype=torch.uint8, device=device)
        shift = (-workspace.data_ptr()) % 256
        self.ws = Workspace(workspace[shift: shift + lay.total_bytes], lay)
        return self

    # -- launches -------------------------------------------------------------------------------------
    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def prepass(self) -> None:
        with torch.cuda.device(self.device):
            _cabi.check(_cabi.lib().sage3_prepass(C.byref(self.desc), self.q.data_ptr(), self.k.data_ptr(),
                                                  self.v.data_ptr(), self.ws.buf.data_ptr(), self._stream()),
                        "sage3_prepass")

    def _lse_ptr(self):
        return None if self.lse is None else self.lse.data_ptr()

    def attention(self) -> torch.Tensor:
        with torch.cuda.device(self.device):
            _cabi.check(_cabi.lib().sage3_attn_fwd(C.byref(self.desc), self.ws.buf.data_ptr(), self.out.data_ptr(),
                                                   self._lse_ptr(), self._stream()), "sage3_attn_fwd")
        return self.out

    def run(self) -> torch.Tensor:
        with torch.cuda.device(self.device):
            _cabi.check(_cabi.lib().sage3_fwd(C.byref(self.desc), self.q.data_ptr(), self.k.data_ptr(),
                                              self.v.data_ptr(), self.ws.buf.data_ptr(), self.out.data_ptr(),
                                              self._lse_ptr(), self._stream()), "sage3_fwd")
        return self.out

    def check_status(self) -> int:
        """Synchronizes and returns the device status word (0 = fine); raises if a bounded wait gave up."""
        word = C.c_int32(0)
        with torch.cuda.device(self.device):
            rc = _cabi.lib().sage3_check_status(self.ws.buf.data_ptr(), C.byref(word), self._stream())
        if rc == _cabi.SAGE3_E_DEVICE_WAIT:
            raise _cabi.Sage3Error(rc, f"device status word {word.value}")
        _cabi.check(rc, "sage3_check_status")
        return word.value


def sageattn3(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND", is_causal: bool = False,
              sm_scale=None, per_block_mean: bool = True, return_lse: bool = False, attn_mask=None,
              workspace: torch.Tensor | None = None, **kwargs) -> torch.Tensor:
    """SageAttention3 (NVFP4 attention) on B200.

    q: [B, Hq, Nq, D] ("HND") or [B, Nq, Hq, D] ("NHD"); k, v likewise with Hkv, Nk.  fp16 or bf16 CUDA
    tensors, D in {64, 128}.  Returns a tensor shaped and typed like q.  `sm_scale` defaults to D**-0.5 and
    may be a float or a tensor with one scale per query head.  Extra keyword arguments (dropout_p, scale, ...)
    are accepted and ignored, as the reference does, so the function can replace
    F.scaled_dot_product_attention in place.

    With `return_lse=True` the result is `(out, lse)`, lse = ln sum_k exp(sm_scale * q.k) per query row as fp32
    [B, Hq, Nq] (the keyword and meaning of sageattention/core.py:86, 327): taken from the quantized scores plus
    sm_scale * q.mean(k), the part of the scores that K smoothing removes.
    """
    if attn_mask is not None:
        raise NotImplementedError("attn_mask is not supported by the FP4 attention path")
    if sm_scale is None and kwargs.get("scale") is not None:
        sm_scale = kwargs["scale"]          # F.scaled_dot_product_attention's name for the same thing
    if torch.compiler.is_compiling():
        # under torch.compile the call is one opaque operator (registered below) instead of a graph break
        scale_f = None if isinstance(sm_scale, torch.Tensor) or sm_scale is None else float(sm_scale)
        scale_t = sm_scale if isinstance(sm_scale, torch.Tensor) else None
        if return_lse:
            return torch.ops.sageattention_b200.fwd_lse(q, k, v, tensor_layout, bool(is_causal), scale_f, scale_t, bool(per_block_mean))
        return torch.ops.sageattention_b200.fwd(q, k, v, tensor_layout, bool(is_causal), scale_f, scale_t, bool(per_block_mean))
    # Repeated calls with one signature (the common case: every layer of a model) reuse the validated descriptor: what is
    # left per call is two allocations and one call into the library.
    plan_key = None
    if workspace is None and not isinstance(sm_scale, torch.Tensor) and q.is_cuda:
        plan_key = (q.device.index, q.dtype, k.dtype, v.dtype, tuple(q.shape), tuple(k.shape), tuple(v.shape), q.stride(), k.stride(),
                    v.stride(), tensor_layout, bool(is_causal), sm_scale, bool(per_block_mean))
        plan = _PLANS.get(plan_key)
        if plan is not None:
            desc, total_bytes, lse_shape = plan
            dev = q.device
            out = torch.empty(q.shape, dtype=q.dtype, device=dev)
            lse = torch.empty(lse_shape, dtype=torch.float32, device=dev) if return_lse else None
            buf = _shared_buffer(dev, total_bytes + 256)
            ws_ptr = buf.data_ptr()
            ws_ptr += (-ws_ptr) % 256
            args = (C.byref(desc), q.data_ptr(), k.data_ptr(), v.data_ptr(), ws_ptr, out.data_ptr(),
                    None if lse is None else lse.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
            if torch.cuda.current_device() == dev.index:
                rc = _cabi.lib().sage3_fwd(*args)
            else:
                with torch.cuda.device(dev):
                    rc = _cabi.lib().sage3_fwd(*args)
            _cabi.check(rc, "sage3_fwd")
            return (out, lse) if return_lse else out
    prob = Sage3Problem(q, k, v, tensor_layout, is_causal, sm_scale, per_block_mean,
                        workspace=CACHED_WORKSPACE if workspace is None else workspace, return_lse=return_lse)
    out = prob.run()
    if plan_key is not None and prob.q is q and prob.k is k and prob.v is v:      # no copies were needed: the signature is reusable
        if len(_PLANS) >= 256:
            _PLANS.clear()
        hd, nd = (1, 2) if tensor_layout == "HND" else (2, 1)
        _PLANS[plan_key] = (prob.desc, prob.ws.layout.total_bytes, (q.shape[0], q.shape[hd], q.shape[nd]))
    return (out, prob.lse) if return_lse else out


# ------------------------------------------------------------------------------------------------------
# workspace cache of the functional entry points
# ------------------------------------------------------------------------------------------------------
# One workspace per (device, stream), grown on demand and reused by later calls: kernels of successive calls on one
# stream run in order, so they may share it; calls on different streams get different buffers.  (Allocating 3.4 GB anew
# on every call of the benchmark shape costs more than the pre-pass.)  Sage3Problem users manage their own.
_WORKSPACES: dict = {}
_PLANS: dict = {}            # signature of a sageattn3 call -> (validated descriptor, workspace bytes, LSE shape)


def _shared_buffer(device: torch.device, nbytes: int) -> torch.Tensor:
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _WORKSPACES.get(key)
    if buf is None or buf.numel() < nbytes:
        _WORKSPACES.pop(key, None)
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = buf
    return buf


def release_workspaces() -> None:
    """Drops the workspaces (and call signatures) that sageattn3 / sageattn / sageattn_varlen keep between calls."""
    _WORKSPACES.clear()
    _PLANS.clear()


# ------------------------------------------------------------------------------------------------------
# torch.library registration: lets torch.compile trace through the call (the reference registers its v2 kernels the
# same way: sageattention/sm89_compile.py:5-23, 69-101 -- a custom op plus a fake implementation that only
# describes the output)
# ------------------------------------------------------------------------------------------------------
def _op_impl(q, k, v, tensor_layout, is_causal, sm_scale, sm_scale_per_head, per_block_mean, return_lse):
    scale = sm_scale_per_head if sm_scale_per_head is not None else sm_scale
    prob = Sage3Problem(q, k, v, tensor_layout, is_causal, scale, per_block_mean, workspace=CACHED_WORKSPACE, return_lse=return_lse)
    out = prob.run()
    return (out, prob.lse) if return_lse else out


@torch.library.custom_op("sageattention_b200::fwd", mutates_args=(), device_types="cuda")
def _fwd_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str, is_causal: bool,
            sm_scale: float | None, sm_scale_per_head: torch.Tensor | None, per_block_mean: bool) -> torch.Tensor:
    return _op_impl(q, k, v, tensor_layout, is_causal, sm_scale, sm_scale_per_head, per_block_mean, False)


@_fwd_op.register_fake
def _(q, k, v, tensor_layout, is_causal, sm_scale, sm_scale_per_head, per_block_mean):
    return torch.empty(q.shape, dtype=q.dtype, device=q.device)


@torch.library.custom_op("sageattention_b200::fwd_lse", mutates_args=(), device_types="cuda")
def _fwd_lse_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str, is_causal: bool,
                sm_scale: float | None, sm_scale_per_head: torch.Tensor | None,
                per_block_mean: bool) -> tuple[torch.Tensor, torch.Tensor]:
    return _op_impl(q, k, v, tensor_layout, is_causal, sm_scale, sm_scale_per_head, per_block_mean, True)


@_fwd_lse_op.register_fake
def _(q, k, v, tensor_layout, is_causal, sm_scale, sm_scale_per_head, per_block_mean):
    hd, nd = (1, 2) if tensor_layout == "HND" else (2, 1)
    return (torch.empty(q.shape, dtype=q.dtype, device=q.device),
            torch.empty(q.shape[0], q.shape[hd], q.shape[nd], dtype=torch.float32, device=q.device))


def sageattn3_blackwell(q, k, v, attn_mask=None, is_causal=False, per_block_mean=True, **kwargs):
    """Signature of the reference's v3 entry (api.py:131): HND layout, D**-0.5 scale."""
    return sageattn3(q, k, v, tensor_layout="HND", is_causal=is_causal, per_block_mean=per_block_mean,
                     attn_mask=attn_mask, **kwargs)


def sageattn(q, k, v, tensor_layout="HND", is_causal=False, sm_scale=None, return_lse=False, **kwargs):
    """Signature of the reference's v2 dispatcher (core.py:79-88); on B200 it always runs the FP4 path."""
    return sageattn3(q, k, v, tensor_layout=tensor_layout, is_causal=is_causal, sm_scale=sm_scale,
                     return_lse=return_lse, **kwargs)


def sageattn_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q, cu_seqlens_k,
                    max_seqlen_q: int | None = None, max_seqlen_k: int | None = None, is_causal: bool = False,
                    sm_scale=None, per_block_mean: bool = True, return_lse: bool = False, **kwargs):
    """Signature of the reference's packed variable-length entry (sageattention/core.py:334-345): q
    [total_q, Hq, D], k, v [total_k, Hkv, D]; sequence i owns rows cu_seqlens[i]:cu_seqlens[i+1].  Returns
    [total_q, Hq, D].

    The whole batch is ONE launch of every kernel (`sage3_fwd_varlen`): the kernels read cu_seqlens on the device, every
    sequence is smoothed, quantized and attended exactly as a call on it alone would be, and a sequence without keys
    gets zeros.  With `max_seqlen_q` / `max_seqlen_k` given and cu_seqlens already int32 CUDA tensors the call does not
    synchronize with the device; without them the maxima are read from cu_seqlens (one device-to-host copy).  Scratch is
    sized for `number of sequences x maximum lengths`.  `smooth_k` is accepted for compatibility; a scalar `sm_scale`
    only.  With `return_lse=True` the result is `(out, lse)`, lse fp32 [number of sequences, Hq, max_seqlen_q]: row i of
    sequence b at [b, :, i], -inf beyond a sequence's length (natural log, as `sageattn3(..., return_lse=True)`)."""
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
        raise ValueError("q, k, v must be packed as [tokens, heads, head_dim]")
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor: sageattention_b200 has no CPU path")
    if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("q, k, v must share dtype torch.float16 or torch.bfloat16")
    if k.shape != v.shape or k.shape[2] != q.shape[2]:
        raise ValueError("k and v must have one shape and the head dim of q")
    if isinstance(sm_scale, torch.Tensor):
        raise ValueError("sageattn_varlen takes a scalar sm_scale")
    kwargs.pop("smooth_k", None)
    dev = q.device
    Hq, Hkv, D = q.shape[1], k.shape[1], q.shape[2]
    if D not in (64, 128):
        raise ValueError(f"head dim must be 64 or 128, got {D}")
    if Hq % Hkv != 0:
        raise ValueError(f"number of query heads ({Hq}) must be a multiple of kv heads ({Hkv})")

    def as_cu(x):
        t = x if isinstance(x, torch.Tensor) else torch.tensor(list(x), dtype=torch.int32)
        return t.to(device=dev, dtype=torch.int32).contiguous()
    cq, ck = as_cu(cu_seqlens_q), as_cu(cu_seqlens_k)
    if cq.dim() != 1 or cq.shape != ck.shape or cq.numel() < 2:
        raise ValueError("cu_seqlens_q / cu_seqlens_k must be 1-D, of equal length >= 2")
    if torch.compiler.is_compiling():
        # one opaque operator under torch.compile (the maxima must be given: reading them back would break the graph)
        if max_seqlen_q is None or max_seqlen_k is None:
            raise ValueError("under torch.compile sageattn_varlen needs max_seqlen_q and max_seqlen_k")
        if return_lse:
            raise NotImplementedError("return_lse of sageattn_varlen is not registered for torch.compile")
        return torch.ops.sageattention_b200.fwd_varlen(q, k, v, cq, ck, int(max_seqlen_q), int(max_seqlen_k), bool(is_causal),
                                                       None if sm_scale is None else float(sm_scale), bool(per_block_mean))
    return _varlen_impl(q, k, v, cq, ck, max_seqlen_q, max_seqlen_k, is_causal, sm_scale, per_block_mean, return_lse)


def _varlen_impl(q, k, v, cq, ck, max_seqlen_q, max_seqlen_k, is_causal, sm_scale, per_block_mean, return_lse=False):
    dev = q.device
    Hq, Hkv, D = q.shape[1], k.shape[1], q.shape[2]
    nseq = cq.numel() - 1
    if max_seqlen_q is None or max_seqlen_k is None:
        # the one place that looks at the lengths on the host (and checks them while it is at it)
        hq, hk = cq.tolist(), ck.tolist()
        if hq[0] != 0 or hk[0] != 0 or hq[-1] != q.shape[0] or hk[-1] != k.shape[0] or \
                any(b < a for a, b in zip(hq, hq[1:])) or any(b < a for a, b in zip(hk, hk[1:])):
            raise ValueError("cu_seqlens_q / cu_seqlens_k must start at 0, be non-decreasing and end at the token counts")
        max_seqlen_q = max(b - a for a, b in zip(hq, hq[1:]))
        max_seqlen_k = max(b - a for a, b in zip(hk, hk[1:]))
    qc, kc, vc = (t if _usable(t) else t.contiguous() for t in (q, k, v))
    out = torch.empty_like(qc)
    max_seqlen_q, max_seqlen_k = max(int(max_seqlen_q), 1), max(int(max_seqlen_k), 1)
    lse = torch.full((nseq, Hq, max_seqlen_q), float("-inf"), dtype=torch.float32, device=dev) if return_lse else None
    if q.shape[0] == 0:
        return (out, lse) if return_lse else out
    d = _cabi.Sage3Desc()
    d.B, d.Hq, d.Hkv, d.Nq, d.Nk, d.D = nseq, Hq, Hkv, max_seqlen_q, max_seqlen_k, D
    d.dtype = _DTYPES[q.dtype]
    d.is_causal = int(bool(is_causal))
    d.per_block_mean = int(bool(per_block_mean))
    d.q_stride = (C.c_int64 * 3)(0, qc.stride(1), qc.stride(0))
    d.k_stride = (C.c_int64 * 3)(0, kc.stride(1), kc.stride(0))
    d.v_stride = (C.c_int64 * 3)(0, vc.stride(1), vc.stride(0))
    d.o_stride = (C.c_int64 * 3)(0, out.stride(1), out.stride(0))
    if sm_scale is not None:
        d.sm_scale = float(sm_scale)
        if not d.sm_scale > 0:
            raise ValueError("sm_scale must be positive")
    need = _cabi.lib().sage3_workspace_bytes(C.byref(d))
    if need == 0:
        raise ValueError("sageattn_varlen: shape not supported (see sage3_workspace_layout)")
    buf = _shared_buffer(dev, need + 256)
    shift = (-buf.data_ptr()) % 256
    with torch.cuda.device(dev):
        _cabi.check(_cabi.lib().sage3_fwd_varlen(C.byref(d), cq.data_ptr(), ck.data_ptr(), qc.data_ptr(), kc.data_ptr(),
                                                 vc.data_ptr(), out.data_ptr(), lse.data_ptr() if lse is not None else None,
                                                 buf.data_ptr() + shift, torch.cuda.current_stream(dev).cuda_stream),
                    "sage3_fwd_varlen")
    return (out, lse) if return_lse else out


@torch.library.custom_op("sageattention_b200::fwd_varlen", mutates_args=(), device_types="cuda")
def _fwd_varlen_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor,
                   max_seqlen_q: int, max_seqlen_k: int, is_causal: bool, sm_scale: float | None,
                   per_block_mean: bool) -> torch.Tensor:
    return _varlen_impl(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, is_causal, sm_scale, per_block_mean)


@_fwd_varlen_op.register_fake
def _(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, is_causal, sm_scale, per_block_mean):
    return torch.empty(q.shape, dtype=q.dtype, device=q.device)


_OFFLOAD_STATE: dict = {}
_OFFLOAD_SLOTS = 2          # chunk buffers in flight (the pipeline is bound by the host link; more slots measured no gain)


def _retire_offload_state(st) -> None:
    """Work that may still use the buffers has been enqueued on the state's streams: wait for it before the
    allocator may hand the memory to someone else."""
    if st is not None:
        for s_ in st["streams"]:
            s_.synchronize()


def sageattn3_offload_release() -> None:
    """Drops the device buffers and streams that sageattn3_offload keeps between calls."""
    _retire_offload_state(_OFFLOAD_STATE.pop("state", None))


def sageattn3_offload(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor | None = None,
                      tensor_layout: str = "HND", is_causal: bool = False, sm_scale=None, per_block_mean: bool = True,
                      device: torch.device | str | None = None, kv_heads_per_chunk: int | None = None,
                      non_blocking: bool = False) -> torch.Tensor:
    """sageattn3 for operands that live in host memory (use pinned tensors): q, k, v are CPU tensors, the result
    is a CPU tensor (pinned when allocated here).

    (Batch, kv-head) groups are independent, so the call is pipelined over chunks of them on three streams:
    while one chunk is being computed, the next one is copied in and the previous result is copied out.  Device
    memory holds two chunks at a time, so the host tensors may be larger than the GPU; the chunk buffers and
    streams are kept for the next call of the same shape (`sageattn3_offload_release()` drops them).  The caller's current
    stream orders the call as a whole (it is waited for at entry and waits for the last copy at exit).  A scalar or None
    `sm_scale` only.

    HOST SYNCHRONIZATION.  The copies run on side streams.  By default the function returns only after the last
    device-to-host copy has completed, so `out` can be read and q, k, v reused at once.  With `non_blocking=True`
    it returns as soon as everything is enqueued: then neither `out` may be read nor q, k, v modified on the host
    until the caller's current stream (which waits for the last copy) has been synchronized.
    """
    if any(t.is_cuda for t in (q, k, v)):
        raise ValueError("sageattn3_offload takes host tensors; call sageattn3 for CUDA tensors")
    if tensor_layout not in ("HND", "NHD"):
        raise ValueError(f"tensor_layout must be 'HND' or 'NHD', got {tensor_layout!r}")
    if isinstance(sm_scale, torch.Tensor):
        raise ValueError("sageattn3_offload takes a scalar sm_scale")
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    hd = 1 if tensor_layout == "HND" else 2
    B, Hq, Hkv = q.shape[0], q.shape[hd], k.shape[hd]
    if Hq % Hkv != 0:
        raise ValueError(f"number of query heads ({Hq}) must be a multiple of kv heads ({Hkv})")
    group = Hq // Hkv
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    elif out.shape != q.shape or out.dtype != q.dtype or out.is_cuda:
        raise ValueError("out must be a host tensor shaped and typed like q")
    if kv_heads_per_chunk is None:
        # about 64 chunks in total, whole kv heads per chunk, equal chunks (a divisor of Hkv)
        target = max(1, (B * Hkv + 63) // 64)
        kv_heads_per_chunk = max(d_ for d_ in range(1, Hkv + 1) if Hkv % d_ == 0 and d_ <= max(target, 1))
    kv_heads_per_chunk = min(kv_heads_per_chunk, Hkv)
    chunks = [(b, h0, min(h0 + kv_heads_per_chunk, Hkv)) for b in range(B) for h0 in range(0, Hkv, kv_heads_per_chunk)]

    def cut(t, b, h0, h1, g=1):
        return t[b:b + 1, h0 * g:h1 * g] if tensor_layout == "HND" else t[b:b + 1, :, h0 * g:h1 * g]

    cur = torch.cuda.current_stream(dev)
    # Streams, device buffers and their events survive the call (one set per process, replaced when the shapes or
    # options change): allocating two chunks' worth of operands and workspace anew on every call costs more than
    # a chunk's copy.  `sageattn3_offload_release()` gives the memory back.
    state_key = (dev.index, tuple(q.shape), tuple(k.shape), q.dtype, tensor_layout, bool(is_causal), sm_scale,
                 bool(per_block_mean), kv_heads_per_chunk, _OFFLOAD_SLOTS)
    st = _OFFLOAD_STATE.get("state")
    if st is None or st["key"] != state_key:
        _retire_offload_state(st)
        st = dict(key=state_key, streams=tuple(torch.cuda.Stream(dev) for _ in range(3)), bufs=[{} for _ in range(_OFFLOAD_SLOTS)],
                  comp_done=[None] * _OFFLOAD_SLOTS, out_done=[None] * _OFFLOAD_SLOTS)
        _OFFLOAD_STATE["state"] = st
    s_in, s_comp, s_out = st["streams"]
    start = torch.cuda.Event()
    start.record(cur)
    for s_ in (s_in, s_comp, s_out):
        s_.wait_event(start)
    bufs, comp_done, out_done = st["bufs"], st["comp_done"], st["out_done"]     # per slot; carried over between calls
    for i, (b, h0, h1) in enumerate(chunks):
        slot = i % len(bufs)
        qh, kh, vh = cut(q, b, h0, h1, group), cut(k, b, h0, h1), cut(v, b, h0, h1)
        key = (tuple(qh.shape), tuple(kh.shape))
        with torch.cuda.stream(s_in):
            if comp_done[slot] is not None:
                s_in.wait_event(comp_done[slot])            # the chunk that used these buffers has been computed
            if key not in bufs[slot]:                       # one set per chunk shape (a ragged last chunk has its own)
                qd = torch.empty(qh.shape, dtype=q.dtype, device=dev)
                kd = torch.empty(kh.shape, dtype=q.dtype, device=dev)
                vd = torch.empty(vh.shape, dtype=q.dtype, device=dev)
                prob = Sage3Problem(qd, kd, vd, tensor_layout, is_causal, sm_scale, per_block_mean)
                bufs[slot][key] = (qd, kd, vd, prob)        # kept alive by the state, ordered by the events below
            qd, kd, vd, prob = bufs[slot][key]
            qd.copy_(qh, non_blocking=True)
            kd.copy_(kh, non_blocking=True)
            vd.copy_(vh, non_blocking=True)
            in_done = torch.cuda.Event()
            in_done.record(s_in)
        with torch.cuda.stream(s_comp):
            s_comp.wait_event(in_done)
            if out_done[slot] is not None:
                s_comp.wait_event(out_done[slot])           # the previous result in this slot has left the device
            prob.run()
            comp_done[slot] = torch.cuda.Event()
            comp_done[slot].record(s_comp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(comp_done[slot])
            cut(out, b, h0, h1, group).copy_(prob.out, non_blocking=True)
            out_done[slot] = torch.cuda.Event()
            out_done[slot].record(s_out)
    for ev in out_done:
        if ev is not None:
            cur.wait_event(ev)
    if not non_blocking:
        for ev in out_done:
            if ev is not None:
                ev.synchronize()
    return out
