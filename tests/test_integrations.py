"""Caller-side integration (attention processor, hybrid FP4 / higher-precision schedule, SDPA patch, torch.compile
registration).  CPU tests use a fake attention module and a plain-torch attention function; the GPU tests put the FP4
kernel behind the same objects."""
import math

import pytest
import torch
import torch.nn.functional as F

from sageattention_b200.integrations import (HybridAttention, SageAttnProcessor, first_and_last_steps, patched_sdpa,
                                             set_sage_attn)


class FakeAttn(torch.nn.Module):
    """The attributes a diffusers Wan / CogVideoX attention module exposes to its processor."""

    def __init__(self, dim=128, heads=2, image_context=False, dtype=torch.float32):
        super().__init__()
        self.heads = heads
        self.to_q, self.to_k, self.to_v = (torch.nn.Linear(dim, dim, dtype=dtype) for _ in range(3))
        self.norm_q, self.norm_k = torch.nn.LayerNorm(dim, dtype=dtype), torch.nn.LayerNorm(dim, dtype=dtype)
        self.to_out = torch.nn.ModuleList([torch.nn.Linear(dim, dim, dtype=dtype), torch.nn.Dropout(0.0)])
        self.add_k_proj = torch.nn.Linear(dim, dim, dtype=dtype) if image_context else None
        self.add_v_proj = torch.nn.Linear(dim, dim, dtype=dtype) if image_context else None
        self.norm_added_k = torch.nn.LayerNorm(dim, dtype=dtype) if image_context else None
        self.processor = None

    def forward(self, x, **kw):
        return self.processor(self, x, **kw)


def sdpa_nhd(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, **kw):
    return F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=is_causal).transpose(1, 2)


def manual(attn, x, enc=None, rotary=None, n_text=None):
    """Straightforward restatement of what the processor must compute, in [B, H, N, D]."""
    img = None
    if attn.add_k_proj is not None and enc is not None:
        img, enc = enc[:, :enc.shape[1] - n_text], enc[:, enc.shape[1] - n_text:]
    src = x if enc is None else enc
    q, k, v = attn.norm_q(attn.to_q(x)), attn.norm_k(attn.to_k(src)), attn.to_v(src)
    split = lambda t: t.unflatten(2, (attn.heads, -1))
    q, k, v = split(q), split(k), split(v)
    if rotary is not None:
        def rot(t):
            c, s = rotary[0][..., 0::2], rotary[1][..., 1::2]
            a, b = t[..., 0::2], t[..., 1::2]
            return torch.stack([a * c - b * s, a * s + b * c], dim=-1).flatten(-2)
        q, k = rot(q), rot(k)
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).flatten(2, 3)
    if img is not None:
        ki, vi = split(attn.norm_added_k(attn.add_k_proj(img))), split(attn.add_v_proj(img))
        o = o + F.scaled_dot_product_attention(q.transpose(1, 2), ki.transpose(1, 2), vi.transpose(1, 2)).transpose(1, 2).flatten(2, 3)
    return attn.to_out[1](attn.to_out[0](o))


@pytest.mark.parametrize("layout", ["NHD", "HND"])
def test_processor_matches_manual_computation(layout):
    torch.manual_seed(0)
    attn = FakeAttn()
    x = torch.randn(2, 50, 128)
    ang = torch.rand(1, 50, 1, 64) * 6.28
    rotary = (ang.cos(), ang.sin())
    fn = sdpa_nhd if layout == "NHD" else (lambda q, k, v, **kw: F.scaled_dot_product_attention(q, k, v))
    proc = SageAttnProcessor(fn, tensor_layout=layout)
    assert torch.allclose(proc(attn, x, rotary_emb=rotary), manual(attn, x, rotary=rotary), atol=1e-5)
    enc = torch.randn(2, 20, 128)                                      # cross attention
    assert torch.allclose(proc(attn, x, encoder_hidden_states=enc), manual(attn, x, enc=enc), atol=1e-5)


def test_processor_image_context_branch():
    torch.manual_seed(1)
    attn = FakeAttn(image_context=True)
    x, enc = torch.randn(1, 30, 128), torch.randn(1, 7 + 16, 128)       # 7 image tokens + 16 text tokens
    proc = SageAttnProcessor(sdpa_nhd, text_context_len=16)
    assert torch.allclose(proc(attn, x, encoder_hidden_states=enc), manual(attn, x, enc=enc, n_text=16), atol=1e-5)


def test_hybrid_schedule_routes_by_step_and_layer():
    seen = []
    fp4 = lambda q, k, v, **kw: (seen.append(("fp4", kw["tensor_layout"])), q)[1]
    hp = lambda q, k, v, **kw: (seen.append(("hp", None)), q)[1]
    h = HybridAttention(first_and_last_steps(total_steps=5), fp4_fn=fp4, hp_fn=hp)
    q = torch.zeros(1, 2, 8, 64, dtype=torch.bfloat16)
    kinds = []
    for step in range(5):
        h.set_step(step)
        h(q, q, q)
        kinds.append(seen[-1][0])
    assert kinds == ["hp", "fp4", "fp4", "fp4", "hp"]                  # first and last step in higher precision
    assert h.calls == {"fp4": 3, "hp": 2}
    h.set_step(2)
    h(q, q, q, attn_mask=torch.ones(8, 8, dtype=torch.bool))            # masks never go to the FP4 kernel
    h(q.float(), q.float(), q.float())                                   # nor fp32 tensors
    assert [s[0] for s in seen[-2:]] == ["hp", "hp"]
    # a policy that keeps one layer in higher precision; step_callback follows diffusers' callback protocol
    h2 = HybridAttention(lambda step, layer: layer != 0, fp4_fn=fp4, hp_fn=hp)
    assert h2.step_callback(None, 3, None, {"latents": 1}) == {"latents": 1} and h2.step == 4
    h2.for_layer(0)(q, q, q)
    h2.for_layer(3)(q, q, q)
    assert [s[0] for s in seen[-2:]] == ["hp", "fp4"]


def test_set_sage_attn_installs_processors_and_patched_sdpa_restores():
    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.attn1, self.attn2 = FakeAttn(), FakeAttn()

    class Model(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.blocks = torch.nn.ModuleList([Block() for _ in range(3)])

    m = Model()
    layers = []
    h = HybridAttention(lambda step, layer: (layers.append(layer), False)[1], hp_fn=lambda q, k, v, **kw: F.scaled_dot_product_attention(q, k, v))
    h.policy_dtype = None
    assert set_sage_attn(m, h) == 3
    assert all(isinstance(b.attn1.processor, SageAttnProcessor) and b.attn2.processor is None for b in m.blocks)
    x = torch.randn(1, 10, 128).to(torch.bfloat16)
    for b in m.blocks:
        b.attn1.to(torch.bfloat16)(x)
    assert layers == [0, 1, 2]
    orig = F.scaled_dot_product_attention
    with patched_sdpa(lambda *a, **k: "patched") as fn:
        assert F.scaled_dot_product_attention is fn and F.scaled_dot_product_attention() == "patched"
    assert F.scaled_dot_product_attention is orig


def test_custom_op_traces_with_fake_tensors():
    """The registered fake implementation describes the outputs, so the call can be traced without running it."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    import sageattention_b200  # noqa: F401  (registers the ops)
    with FakeTensorMode():
        q = torch.empty(2, 8, 300, 64, dtype=torch.bfloat16, device="cuda")
        k = torch.empty(2, 4, 500, 64, dtype=torch.bfloat16, device="cuda")
        o = torch.ops.sageattention_b200.fwd(q, k, k, "HND", False, None, None, True)
        assert o.shape == q.shape and o.dtype == q.dtype
        o, lse = torch.ops.sageattention_b200.fwd_lse(q.transpose(1, 2), k.transpose(1, 2), k.transpose(1, 2), "NHD", True, 0.1, None, True)
        assert o.shape == (2, 300, 8, 64) and lse.shape == (2, 8, 300) and lse.dtype == torch.float32
        qp = torch.empty(100, 4, 64, dtype=torch.bfloat16, device="cuda")
        kp = torch.empty(120, 2, 64, dtype=torch.bfloat16, device="cuda")
        cu = torch.empty(3, dtype=torch.int32, device="cuda")
        o = torch.ops.sageattention_b200.fwd_varlen(qp, kp, kp, cu, cu, 60, 70, True, None, True)
        assert o.shape == qp.shape and o.dtype == qp.dtype


# ------------------------------------------------------------------------------------------------------ GPU
@pytest.mark.gpu
def test_processor_with_fp4_kernel_matches_oracle(cuda_device):
    from oracle import sage3_oracle as O
    torch.manual_seed(2)
    attn = FakeAttn(dim=256, heads=2, dtype=torch.bfloat16).to(cuda_device)
    x = torch.randn(1, 300, 256, device=cuda_device, dtype=torch.bfloat16)
    captured = {}

    def oracle_fn(q, k, v, **kw):                                       # same processor, CPU oracle as the attention
        captured["q"] = q
        return O.sageattn3_oracle(q.cpu(), k.cpu(), v.cpu(), tensor_layout="NHD").to(cuda_device)

    with torch.no_grad():
        out = SageAttnProcessor()(attn, x)                               # default: sageattn3 in NHD layout
        ref = SageAttnProcessor(oracle_fn)(attn, x)
    torch.cuda.synchronize()
    assert captured["q"].shape == (1, 300, 2, 128)
    assert O.cosine(out.cpu(), ref.cpu()) >= 0.999 and O.rel_l1(out.cpu(), ref.cpu()) <= 0.01


@pytest.mark.gpu
def test_torch_compile_fullgraph(cuda_device):
    """sageattn3 inside a compiled block: one opaque operator, no graph break (fullgraph=True would raise)."""
    from sageattention_b200 import sageattn3

    class Blk(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.qkv = torch.nn.Linear(128, 3 * 128, dtype=torch.bfloat16)

        def forward(self, x):
            q, k, v = self.qkv(x).unflatten(2, (3, 2, 64)).unbind(2)     # [B, N, H, D]
            o, lse = sageattn3(q, k, v, tensor_layout="NHD", is_causal=True, return_lse=True)
            return o.flatten(2) + x, lse

    blk = Blk().to(cuda_device)
    x = torch.randn(2, 200, 128, device=cuda_device, dtype=torch.bfloat16)
    with torch.no_grad():                                                 # an inference operator: no autograd formula
        eager, lse_e = blk(x)
        comp, lse_c = torch.compile(blk, fullgraph=True, backend="aot_eager")(x)
    torch.cuda.synchronize()
    assert torch.allclose(eager.float(), comp.float(), atol=2e-2, rtol=2e-2)
    assert torch.allclose(lse_e, lse_c, atol=1e-3)


@pytest.mark.gpu
def test_torch_compile_varlen_fullgraph(cuda_device):
    """sageattn_varlen inside a compiled function: one opaque operator (cu_seqlens on the device, maxima given)."""
    from sageattention_b200 import sageattn_varlen
    g = torch.Generator().manual_seed(8)
    lens = [70, 200, 33]
    cu = torch.tensor([0, 70, 270, 303], dtype=torch.int32, device=cuda_device)
    q = torch.randn(303, 4, 64, generator=g).to(torch.bfloat16).to(cuda_device)
    k = (torch.randn(303, 2, 64, generator=g) + 1).to(torch.bfloat16).to(cuda_device)
    v = torch.randn(303, 2, 64, generator=g).to(torch.bfloat16).to(cuda_device)

    def fn(q, k, v, cu):
        return sageattn_varlen(q * 1.0, k, v, cu, cu, max(lens), max(lens), is_causal=True) + 0.0

    with torch.no_grad():
        eager = fn(q, k, v, cu)
        comp = torch.compile(fn, fullgraph=True, backend="aot_eager")(q, k, v, cu)
    torch.cuda.synchronize()
    assert torch.equal(eager, comp)
