"""Caller-side integration: how diffusion and language models reach the kernel.

The reference's users do not call the operator directly.  They either replace `F.scaled_dot_product_attention`
(reference: example/cogvideox_infer.py:34-35) or install an attention processor on every transformer block
(reference: example/modify_model/modify_wan.py:8-107, the same pattern in modify_hunyuan.py, modify_ltx.py,
modify_mochi.py), and the SageAttention3 README prescribes a per-timestep hybrid for models that FP4 attention does not
serve losslessly: a higher-precision kernel at the first and last denoising steps, FP4 for all others
(reference: sageattention3_blackwell/README.md:16-22).

This module provides the three pieces without importing diffusers (the processor is duck-typed, as diffusers'
processor protocol is):
  * `HybridAttention`  -- a callable with the signature of F.scaled_dot_product_attention that routes every call
                          to the FP4 kernel or to a caller-supplied higher-precision function, as a policy decides
                          from (step, layer);
  * `SageAttnProcessor` / `set_sage_attn` -- a processor for attention modules of the Wan / CogVideoX kind
                          (to_q / to_k / to_v projections, optional q/k norms, rotary embedding, optional image
                          context of image-to-video models); tensors go to the kernel in "NHD" layout, so the two
                          transposes of the reference's processor disappear;
  * `patched_sdpa`     -- context manager that swaps F.scaled_dot_product_attention in and out.
"""
from __future__ import annotations

import contextlib
from typing import Callable, Iterable, Optional

import torch
import torch.nn.functional as F

from .api import sageattn3


def first_and_last_steps(total_steps: int, n_first: int = 1, n_last: int = 1) -> Callable[[int, int], bool]:
    """The policy the reference's README recommends: `True` (FP4) for every step except the first `n_first`
    and the last `n_last` of `total_steps` denoising steps.  The layer index is ignored."""
    def policy(step: int, layer: int) -> bool:
        return n_first <= step < total_steps - n_last
    return policy


class HybridAttention:
    """Drop-in for F.scaled_dot_product_attention(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None).

    `policy(step, layer) -> bool` says whether a call runs in FP4 (`fp4_fn`, default sageattn3) or in higher
    precision (`hp_fn`, default torch's scaled_dot_product_attention; pass an FP8 / INT8 kernel here where one is
    available).  The step is advanced by the sampling loop (`set_step`, or `step_callback` as a diffusers
    `callback_on_step_end`); the layer index comes from the processor that calls (`for_layer`).  Calls that FP4
    attention cannot serve (an attention mask, dropout, a head dim other than 64 / 128) always go to `hp_fn`.
    """

    def __init__(self, policy: Callable[[int, int], bool] | None = None, fp4_fn: Callable = sageattn3,
                 hp_fn: Callable | None = None, tensor_layout: str = "HND"):
        self.policy = policy if policy is not None else (lambda step, layer: True)
        self.fp4_fn = fp4_fn
        self.hp_fn = hp_fn if hp_fn is not None else F.scaled_dot_product_attention
        self.tensor_layout = tensor_layout
        self.step = 0
        self.calls = {"fp4": 0, "hp": 0}

    def set_step(self, step: int) -> None:
        self.step = int(step)

    def step_callback(self, pipe, step: int, timestep, callback_kwargs: dict) -> dict:
        """Signature of diffusers' `callback_on_step_end`: the next attention calls belong to step + 1."""
        self.step = int(step) + 1
        return callback_kwargs

    def for_layer(self, layer: int) -> Callable:
        def attn(q, k, v, **kw):
            return self(q, k, v, _layer=layer, **kw)
        return attn

    def __call__(self, q, k, v, attn_mask=None, dropout_p: float = 0.0, is_causal: bool = False, scale=None,
                 _layer: int = 0, **kwargs):
        fp4_ok = attn_mask is None and not dropout_p and q.shape[-1] in (64, 128) and q.dtype in (torch.float16, torch.bfloat16)
        if fp4_ok and self.policy(self.step, _layer):
            self.calls["fp4"] += 1
            return self.fp4_fn(q, k, v, tensor_layout=self.tensor_layout, is_causal=is_causal, sm_scale=scale, **kwargs)
        self.calls["hp"] += 1
        if self.tensor_layout == "NHD":                      # torch's SDPA wants [B, H, N, D]
            o = self.hp_fn(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=attn_mask,
                           dropout_p=dropout_p, is_causal=is_causal, scale=scale)
            return o.transpose(1, 2)
        return self.hp_fn(q, k, v, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal, scale=scale)


def _rotate_interleaved(x: torch.Tensor, freqs_cos: torch.Tensor, freqs_sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding on interleaved pairs (x[..., 0::2], x[..., 1::2]) with Wan-style frequency tensors
    (cos taken at even, sin at odd positions of the last dim); broadcast over the leading dims."""
    x1, x2 = x[..., 0::2], x[..., 1::2]
    cos, sin = freqs_cos[..., 0::2], freqs_sin[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = x1 * cos - x2 * sin
    out[..., 1::2] = x1 * sin + x2 * cos
    return out.type_as(x)


class SageAttnProcessor:
    """Attention processor (diffusers protocol: `processor(attn, hidden_states, encoder_hidden_states=None,
    attention_mask=None, rotary_emb=None)`) for modules that carry `to_q`, `to_k`, `to_v`, `to_out`, `heads` and,
    optionally, `norm_q`, `norm_k`, and the image-context projections `add_k_proj`, `add_v_proj`, `norm_added_k` of
    image-to-video models.  `attn_fn(q, k, v, attn_mask=..., dropout_p=0.0, is_causal=False)` receives tensors
    [B, N, H, D] when `tensor_layout == "NHD"` (default; no transposes) or [B, H, N, D] for "HND".

    `text_context_len`: number of trailing text tokens in `encoder_hidden_states` when an image context precedes them
    (512 for Wan).
    """

    def __init__(self, attn_fn: Callable | None = None, tensor_layout: str = "NHD", text_context_len: int = 512):
        if attn_fn is None:
            attn_fn = lambda q, k, v, **kw: sageattn3(q, k, v, tensor_layout=tensor_layout, **kw)   # noqa: E731
        self.attn_fn = attn_fn
        self.tensor_layout = tensor_layout
        self.text_context_len = text_context_len

    def _heads(self, x: torch.Tensor, heads: int) -> torch.Tensor:
        x = x.unflatten(2, (heads, -1))                     # [B, N, H, D]
        return x if self.tensor_layout == "NHD" else x.transpose(1, 2)

    def _merge(self, o: torch.Tensor) -> torch.Tensor:
        if self.tensor_layout == "HND":
            o = o.transpose(1, 2)
        return o.flatten(2, 3)

    def __call__(self, attn, hidden_states: torch.Tensor, encoder_hidden_states: Optional[torch.Tensor] = None,
                 attention_mask: Optional[torch.Tensor] = None, rotary_emb=None, **kwargs) -> torch.Tensor:
        img_context = None
        if getattr(attn, "add_k_proj", None) is not None and encoder_hidden_states is not None:
            n_img = encoder_hidden_states.shape[1] - self.text_context_len
            img_context, encoder_hidden_states = encoder_hidden_states[:, :n_img], encoder_hidden_states[:, n_img:]
        kv_src = hidden_states if encoder_hidden_states is None else encoder_hidden_states
        q, k, v = attn.to_q(hidden_states), attn.to_k(kv_src), attn.to_v(kv_src)
        if getattr(attn, "norm_q", None) is not None:
            q = attn.norm_q(q)
        if getattr(attn, "norm_k", None) is not None:
            k = attn.norm_k(k)
        q, k, v = (x.unflatten(2, (attn.heads, -1)) for x in (q, k, v))          # [B, N, H, D]
        if rotary_emb is not None:
            q = _rotate_interleaved(q, *rotary_emb)
            k = _rotate_interleaved(k, *rotary_emb)
        if self.tensor_layout == "HND":
            q, k, v = (x.transpose(1, 2) for x in (q, k, v))
        out = self.attn_fn(q, k, v, attn_mask=attention_mask, dropout_p=0.0, is_causal=False)
        out = self._merge(out).type_as(hidden_states)
        if img_context is not None:
            k_img = attn.add_k_proj(img_context)
            if getattr(attn, "norm_added_k", None) is not None:
                k_img = attn.norm_added_k(k_img)
            v_img = attn.add_v_proj(img_context)
            o_img = self.attn_fn(q, self._heads(k_img, attn.heads), self._heads(v_img, attn.heads), attn_mask=None,
                                 dropout_p=0.0, is_causal=False)
            out = out + self._merge(o_img).type_as(hidden_states)
        out = attn.to_out[0](out)
        return attn.to_out[1](out) if len(attn.to_out) > 1 else out


def set_sage_attn(model, attn_fn: Callable | HybridAttention | None = None, blocks_attr: str = "blocks",
                  attn_attrs: Iterable[str] = ("attn1",), tensor_layout: str = "NHD") -> int:
    """Installs a SageAttnProcessor on `getattr(block, a)` for every block of `getattr(model, blocks_attr)` and every
    name a in `attn_attrs` (the reference patches the self-attention `attn1` of every Wan block,
    modify_wan.py:100-107).  A HybridAttention gets its layer index from the block position and its `tensor_layout`
    set to the processors'.  Returns the number of processors installed."""
    n = 0
    if isinstance(attn_fn, HybridAttention):
        attn_fn.tensor_layout = tensor_layout
    for idx, block in enumerate(getattr(model, blocks_attr)):
        fn = attn_fn.for_layer(idx) if isinstance(attn_fn, HybridAttention) else attn_fn
        for a in attn_attrs:
            mod = getattr(block, a, None)
            if mod is None:
                continue
            proc = SageAttnProcessor(fn, tensor_layout=tensor_layout)
            if hasattr(mod, "set_processor"):
                mod.set_processor(proc)
            else:
                mod.processor = proc
            n += 1
    return n


@contextlib.contextmanager
def patched_sdpa(attn_fn: Callable | None = None):
    """Replaces F.scaled_dot_product_attention by `attn_fn` (default: the FP4 kernel behind SDPA's signature) inside
    the `with` block, the way the reference's inference scripts do for models that call SDPA directly."""
    fn = attn_fn if attn_fn is not None else HybridAttention()
    saved = F.scaled_dot_product_attention
    F.scaled_dot_product_attention = fn
    try:
        yield fn
    finally:
        F.scaled_dot_product_attention = saved
