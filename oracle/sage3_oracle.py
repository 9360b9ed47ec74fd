"""CPU oracle for the SageAttention3 hot path (smooth -> NVFP4 quantize -> block-scaled FP4 attention).

TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA path and the timed CPU baseline of
the benchmark; the product never imports it.  It restates, in torch fp32 on the CPU, the arithmetic of
the reference's SageAttention3 pipeline, with every rounding point made explicit.

PINNING.  The reference ships no tests, golden vectors or fixtures for this path.  What pins this restatement:
  * the smoothing + quantization stage (`prepass` below) against the reference itself: its unmodified
    fp4_quantization_4d.cu (compiled for sm_100a by oracle/build_ref_quant.py) and its unmodified sageattn3/api.py
    (preprocess_qkv with the Triton block-mean kernel) were run on a B200 on seeded inputs and their outputs stored
    in tests/golden/ref_prepass.pt (tests/golden/make_ref_prepass_golden.py); tests/test_ref_pin.py holds `prepass`
    against them: means, smoothed tensors, codes and scale bytes bit for bit, delta_s within one unit in the last place;
  * the E2M1 and E4M3 codecs against NVIDIA's host-side converters in cuda_fp4.h / cuda_fp8.h
    (oracle/codec_pin.cu -> tests/golden/codec_pin.npz).
ATTENTION KERNEL: PARITY UNPINNED.  The reference's attention extension executes on sm_120 hardware only
(blackwell/api.cu:219-222), so nothing it produced exists to pin `attention_from_prepass` against; it follows the
cited source lines.

Reference locations (paths inside the reference project):
  sageattention3_blackwell/sageattn3/api.py:75-92      smoothing, padding to 128, delta_s
  sageattention3_blackwell/sageattn3/api.py:26-72      per-128-row Q block mean
  .../quantization/fp4_quantization_4d.cu:185-225      1x16 microblock quantization of Q and K
  .../quantization/fp4_quantization_4d.cu:300-349      V quantized along tokens (V transposed)
  .../blackwell/softmax_fused.h:39-170                 online softmax with FP4 re-quantization of P
  .../blackwell/mainloop_tma_ws.h:691-797, 864-901     delta_s add, masks, KV walk last -> first
  .../blackwell/api.cu:142, api.py:127                 softmax scale (D**-0.5 * log2 e)

Deliberate differences from the reference source (documented, not accidental):
  * masks are applied on the real token index (the reference masks the permuted MMA column index), and the causal
    mask is aligned on the real lengths (the reference: on the lengths padded to 128);
  * every accumulator starts from zero / -inf;
  * inputs are never modified in place;
  * divisions are IEEE fp32 (the reference compiles with --use_fast_math).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

BLOCK = 128          # Q tile rows and KV block length (launch.h:105)
MICRO = 16           # NVFP4 microblock
LOG2E = 1.4426950408889634
# softmax_fused.h:32-34
P_SCALE_LOG2 = -11.392317422778762     # log2(1 / (448 * 6))
FP4_SCALE_LOG2 = -2.584962500721156    # log2(1 / 6)

E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=torch.float32)


# --------------------------------------------------------------------------------------------------
# codecs
# --------------------------------------------------------------------------------------------------
def e4m3_rn_satfinite(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 (>= 0) -> (E4M3 byte, decoded fp32).  Round to nearest even, saturate at 448.

    Mirrors `__nv_fp8_e4m3(float)` (fp4_quantization_4d.cu:199-202) and
    `cvt.rn.satfinite.e4m3x2.f32` (blackwell/utils.h:199-213).  torch's own conversion yields NaN
    above 448, hence the clamp.
    """
    b = x.to(torch.float32).clamp(max=448.0).to(torch.float8_e4m3fn)
    return b.view(torch.uint8), b.to(torch.float32)


def e2m1_rn_satfinite(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit E2M1 code (uint8 in 0..15), round to nearest, ties to the even code, |x|>6 -> 6.

    Mirrors `cvt.rn.satfinite.e2m1x2.f32` (fp4_quantization_4d.cu:86-89, blackwell/utils.h:228-231).
    Bit 3 is the sign and is kept for values that round to zero.
    """
    x = x.to(torch.float32)
    a = x.abs()
    # thresholds between successive magnitudes; '>' where the tie goes down, '>=' where it goes up
    code = (a > 0.25).to(torch.uint8)            # 0    | 0.5   tie 0.25 -> 0
    code += (a >= 0.75).to(torch.uint8)          # 0.5  | 1.0   tie 0.75 -> 1.0
    code += (a > 1.25).to(torch.uint8)           # 1.0  | 1.5   tie 1.25 -> 1.0
    code += (a >= 1.75).to(torch.uint8)          # 1.5  | 2.0   tie 1.75 -> 2.0
    code += (a > 2.5).to(torch.uint8)            # 2.0  | 3.0   tie 2.5  -> 2.0
    code += (a >= 3.5).to(torch.uint8)           # 3.0  | 4.0   tie 3.5  -> 4.0
    code += (a > 5.0).to(torch.uint8)            # 4.0  | 6.0   tie 5.0  -> 4.0
    sign = torch.signbit(x).to(torch.uint8) << 3
    return code | sign


def e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    mag = E2M1_VALUES[(code & 7).long()]
    return torch.where((code & 8) != 0, -mag, mag)


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """[..., 2n] codes -> [..., n] bytes: element 2i in bits 0-3, 2i+1 in bits 4-7
    (fp4_quantization_4d.cu:86, 235-239)."""
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).contiguous()


def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    lo = packed & 0xF
    hi = packed >> 4
    return torch.stack([lo, hi], dim=-1).flatten(-2)


# --------------------------------------------------------------------------------------------------
# quantization
# --------------------------------------------------------------------------------------------------
def quant_microblocks(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """NVFP4-quantize along the last dim in groups of 16 (fp4_quantization_4d.cu:185-225).

    x: [..., n] (n % 16 == 0), values already in the input dtype's grid (bf16 / fp16).
    Returns (codes uint8 [..., n], sf_bytes uint8 [..., n/16], dequantized fp32 [..., n]).
    """
    xf = x.to(torch.float32)
    g = xf.unflatten(-1, (-1, MICRO))
    amax = g.abs().amax(dim=-1, keepdim=True)
    sf_b, sf = e4m3_rn_satfinite(amax / 6.0)
    inv = torch.where(sf == 0, torch.zeros_like(sf), 1.0 / sf)
    codes = e2m1_rn_satfinite(g * inv)
    deq = e2m1_decode(codes) * sf
    return codes.flatten(-2), sf_b.squeeze(-1), deq.flatten(-2)


def block_mean_16bit_tree(q_blocks: torch.Tensor) -> torch.Tensor:
    """Mean over the 128 rows of every query block exactly as the reference's Triton kernel forms it
    (api.py:45-48: `tl.sum(q_group, axis=0) / GROUP_SIZE` on 16-bit data).  Triton does not widen a 16-bit sum, so
    every addition rounds to the input type and the order matters.  The order below is the one Triton 3.6 generates for
    this kernel (4 warps, blocked layout, 8 elements per thread along D); it reproduces the reference's means bit for
    bit on the recorded fixtures (bf16 and fp16, D = 64 and 128):
      * a thread owns row  rep * R + warp * L + lane_row  of every repetition rep, with L = 32 / (D / 8) rows per
        warp and R = 4 L rows per repetition; it adds its rows in order of rep;
      * inside a warp the L partial sums are combined by a butterfly over the lane rows (distance L/2, then L/4, ...);
      * the four warp sums are combined as (w0 + w2) + (w1 + w3).
    q_blocks: [..., 128, D] (bf16 / fp16) -> [..., D] in the same type."""
    dt = q_blocks.dtype
    D = q_blocks.shape[-1]
    warps, lane_rows = 4, 32 // (D // 8)
    reps = BLOCK // (warps * lane_rows)

    def add(a, b):
        return (a.to(torch.float32) + b.to(torch.float32)).to(dt)

    x = q_blocks.reshape(*q_blocks.shape[:-2], reps, warps, lane_rows, D)
    acc = x[..., 0, :, :, :]
    for r in range(1, reps):
        acc = add(acc, x[..., r, :, :, :])                       # [..., warps, lane_rows, D]
    vals = [acc[..., i, :] for i in range(lane_rows)]
    n = lane_rows // 2
    while n > 0:
        vals = [add(vals[i], vals[i ^ n]) for i in range(lane_rows)]
        n //= 2
    w = [vals[0][..., i, :] for i in range(warps)]
    n = warps // 2
    while n > 0:
        w = [add(w[i], w[i ^ n]) for i in range(warps)]
        n //= 2
    return (w[0].to(torch.float32) / BLOCK).to(dt)


def pad_rows(x: torch.Tensor, mult: int = BLOCK) -> torch.Tensor:
    """zero-pad dim -2 to a multiple of `mult` (api.py:77-85)."""
    n = x.shape[-2]
    pad = (-n) % mult
    if pad == 0:
        return x
    return torch.nn.functional.pad(x, (0, 0, 0, pad))


@dataclass
class Prepass:
    """Everything the pre-pass produces, for one call.  Shapes use HND: [B, H, N, D]."""
    km: torch.Tensor          # [B, Hkv, D]  input dtype
    qm: torch.Tensor          # [B, Hq, nqm, D] input dtype (nqm = Nq_p/128, or 1)
    q_s: torch.Tensor         # smoothed, padded Q  [B,Hq,Nq_p,D] input dtype
    k_s: torch.Tensor         # smoothed, padded K
    v_p: torch.Tensor         # padded V
    delta: torch.Tensor       # [B, Hq, nqm, Nk_p] fp32 (values on the input dtype's grid)
    q_codes: torch.Tensor     # [B,Hq,Nq_p,D] u8 codes
    q_sf: torch.Tensor        # [B,Hq,Nq_p,D/16] e4m3 bytes
    q_deq: torch.Tensor       # fp32
    k_codes: torch.Tensor
    k_sf: torch.Tensor
    k_deq: torch.Tensor
    vt_codes: torch.Tensor    # [B,Hkv,D,Nk_p] codes (microblocks along tokens)
    vt_sf: torch.Tensor       # [B,Hkv,D,Nk_p/16]
    vt_deq: torch.Tensor      # [B,Hkv,D,Nk_p] fp32
    nq: int
    nk: int


def prepass(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, per_block_mean: bool = True,
            km_override: torch.Tensor | None = None, qm_override: torch.Tensor | None = None,
            block_mean: str = "reference") -> Prepass:
    """Smoothing + quantization (api.py:75-116).  q: [B,Hq,Nq,D]; k, v: [B,Hkv,Nk,D]; bf16 or fp16.

    `block_mean`: "reference" forms the per-block Q mean as the reference's Triton kernel does (16-bit additions in
    its order, see block_mean_16bit_tree); "fp32" sums in fp32 and rounds once (more accurate, but not what the
    reference computes: about 70 % of the means then differ from the reference's in the last bits).

    `km_override` / `qm_override` let a test substitute means computed elsewhere (a different fp32
    summation order can flip the rounding of a mean by one ulp), so that everything downstream of the
    means can be compared bit for bit.
    """
    dt = q.dtype
    assert dt in (torch.bfloat16, torch.float16) and k.dtype == dt and v.dtype == dt
    B, Hq, Nq, D = q.shape
    _, Hkv, Nk, _ = k.shape
    assert Hq % Hkv == 0 and D % MICRO == 0
    group = Hq // Hkv

    # api.py:84 -- K smoothing: mean over the unpadded tokens, fp32 accumulate, rounded to dt;
    # subtraction rounded to dt.
    km = k.to(torch.float32).mean(dim=-2).to(dt) if km_override is None else km_override.to(dt)
    k_s = (k.to(torch.float32) - km.to(torch.float32).unsqueeze(-2)).to(dt)
    # api.py:85 -- pad after smoothing: pad rows are exactly zero
    q_p, k_s, v_p = pad_rows(q), pad_rows(k_s), pad_rows(v)
    Nq_p, Nk_p = q_p.shape[-2], k_s.shape[-2]

    # api.py:86-90 -- Q smoothing.  Pad rows take part in the mean (padding happens first).  The block mean is a
    # 16-bit sum in the Triton kernel's order; the subtraction uses the stored (rounded) mean, api.py:50.
    if qm_override is not None:
        qm = qm_override.to(dt)
    elif per_block_mean and block_mean == "reference":
        qm = block_mean_16bit_tree(q_p.unflatten(-2, (-1, BLOCK)))                   # [B,Hq,nb,D]
    elif per_block_mean:
        qm = q_p.to(torch.float32).unflatten(-2, (-1, BLOCK)).mean(dim=-2).to(dt)
    else:
        qm = q_p.to(torch.float32).mean(dim=-2, keepdim=True).to(dt)                 # [B,Hq,1,D]
    if per_block_mean:
        qm_rows = qm.repeat_interleave(BLOCK, dim=-2)
    else:
        qm_rows = qm.expand(B, Hq, Nq_p, D)
    q_s = (q_p.to(torch.float32) - qm_rows.to(torch.float32)).to(dt)

    # api.py:91 -- delta_s = (qm @ k_s^T) rounded to dt, widened to fp32
    k_s_q = k_s.repeat_interleave(group, dim=1) if group > 1 else k_s
    delta = torch.matmul(qm.to(torch.float32), k_s_q.to(torch.float32).transpose(-1, -2)).to(dt).to(torch.float32)

    q_codes, q_sf, q_deq = quant_microblocks(q_s)
    k_codes, k_sf, k_deq = quant_microblocks(k_s)
    # fp4_quantization_4d.cu:300-349 -- V: microblocks of 16 consecutive tokens of one channel
    vt_codes, vt_sf, vt_deq = quant_microblocks(v_p.transpose(-1, -2).contiguous())
    return Prepass(km, qm, q_s, k_s, v_p, delta, q_codes, q_sf, q_deq, k_codes, k_sf, k_deq,
                   vt_codes, vt_sf, vt_deq, Nq, Nk)


# --------------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------------
def _scale_log2(sm_scale, Hq: int, D: int) -> torch.Tensor:
    if sm_scale is None:
        sm_scale = D ** -0.5
    s = torch.as_tensor(sm_scale, dtype=torch.float32).reshape(-1)
    if s.numel() == 1:
        s = s.expand(Hq)
    assert s.numel() == Hq
    return (s.to(torch.float64) * LOG2E).to(torch.float32)


def attention_from_prepass(pp: Prepass, is_causal: bool = False, sm_scale=None,
                           out_dtype: torch.dtype | None = None, q_rows: slice | None = None,
                           return_lse_parts: bool = False):
    """Block-scaled FP4 attention with online softmax (softmax_fused.h:39-170; mainloop_tma_ws.h:864-901).

    KV blocks of 128 keys are walked from the LAST to the FIRST; the running row max is updated once
    per block; P~ = 2^(S*s - m*s) * 2688; the row sum is over the unquantized P~; each 16-key microblock
    of P~ is divided by the *unrounded* fp32 scale max(P~)/6 before E2M1 rounding while the product
    uses the E4M3-rounded scale; O = O*alpha + P^ V^ in fp32; out = O / l.

    q_rows: optional slice of (padded) query rows to evaluate -- rows are independent given the
    pre-pass, so a sampled evaluation is exact for the sampled rows.
    """
    B, Hq, Nq_p, D = pp.q_deq.shape
    Hkv, Nk_p = pp.k_deq.shape[1], pp.k_deq.shape[2]
    group = Hq // Hkv
    nkb = Nk_p // BLOCK
    s2 = _scale_log2(sm_scale, Hq, D).view(1, Hq, 1, 1)
    rs = q_rows if q_rows is not None else slice(0, Nq_p)
    rows = torch.arange(Nq_p)[rs]
    R = rows.numel()
    qd = pp.q_deq[:, :, rs]
    per_block = pp.qm.shape[2] > 1
    drow = (rows // BLOCK) if per_block else torch.zeros_like(rows)

    m = torch.full((B, Hq, R, 1), -math.inf)
    l = torch.zeros(B, Hq, R, 1)
    O = torch.zeros(B, Hq, R, D)
    # causal mask, bottom-right aligned on the real lengths (the reference, mainloop_tma_ws.h:286-289, 732-734,
    # aligns on the lengths padded to 128: the same whenever Nq and Nk are multiples of 128): key j visible to
    # query i iff j <= i + Nk - Nq
    lim = rows.view(1, 1, R, 1) + (pp.nk - pp.nq)

    for j in range(nkb - 1, -1, -1):
        ks = slice(j * BLOCK, (j + 1) * BLOCK)
        kd = pp.k_deq[:, :, ks]
        vd = pp.vt_deq[:, :, :, ks]                      # [B,Hkv,D,128]
        if group > 1:
            kd = kd.repeat_interleave(group, dim=1)
            vd = vd.repeat_interleave(group, dim=1)
        S = torch.matmul(qd, kd.transpose(-1, -2)) + pp.delta[:, :, drow][:, :, :, ks]
        keys = torch.arange(j * BLOCK, (j + 1) * BLOCK).view(1, 1, 1, BLOCK)
        dead = keys >= pp.nk
        if is_causal:
            dead = dead | (keys > lim)
        S = S.masked_fill(dead, -math.inf)

        bmax = S.unflatten(-1, (-1, MICRO)).amax(dim=-1)                  # [B,H,R,8]
        m_new = torch.maximum(m, bmax.amax(dim=-1, keepdim=True))
        finite = torch.isfinite(m_new)
        m_cur = torch.where(finite, m_new, torch.zeros_like(m_new))       # InfCheck (softmax_fused.h:70-72)
        alpha = torch.exp2((m - m_cur) * s2)                              # m = -inf  ->  0
        max_scaled = torch.where(finite, m_new * s2 + P_SCALE_LOG2, torch.zeros_like(m_new))
        Pt = torch.exp2(S * s2 - max_scaled)                              # in [0, 2688]
        l = l * alpha + Pt.sum(dim=-1, keepdim=True)
        sf = torch.exp2(bmax * s2 - max_scaled + FP4_SCALE_LOG2)          # = blockmax(P~)/6, fp32
        sf = torch.where(torch.isfinite(bmax), sf, torch.zeros_like(sf))
        inv = torch.where(sf == 0, torch.zeros_like(sf), 1.0 / sf)
        codes = e2m1_rn_satfinite(Pt.unflatten(-1, (-1, MICRO)) * inv.unsqueeze(-1))
        _, sf_r = e4m3_rn_satfinite(sf)
        Pq = (e2m1_decode(codes) * sf_r.unsqueeze(-1)).flatten(-2)        # [B,H,R,128]
        O = O * alpha + torch.matmul(Pq, vd.transpose(-1, -2))
        m = m_new

    inv_l = torch.where((l == 0) | torch.isnan(l), torch.zeros_like(l), 1.0 / l)   # softmax_fused.h:147-148
    out = O * inv_l
    keep = rows < pp.nq
    out = out[:, :, keep]
    dt = out_dtype if out_dtype is not None else pp.q_s.dtype
    if return_lse_parts:
        return out.to(dt), m[:, :, keep], l[:, :, keep]
    return out.to(dt)


def _to_hnd(x: torch.Tensor, tensor_layout: str) -> torch.Tensor:
    if tensor_layout == "HND":
        return x
    if tensor_layout == "NHD":
        return x.transpose(1, 2)
    raise ValueError(f"unknown tensor_layout {tensor_layout!r}")


def lse_from_parts(pp: Prepass, q: torch.Tensor, m: torch.Tensor, l: torch.Tensor, sm_scale=None) -> torch.Tensor:
    """ln sum_k exp(sm_scale * q.k) per query row, [B,Hq,Nq] fp32, from the running maximum m and row sum l of the
    quantized, smoothed scores plus sm_scale * q.km, the part K smoothing took out of every score of the row
    (sageattention/core.py:289-293, 327: `lse / 1.44269504 + lse_correction * sm_scale`).  q: [B,Hq,Nq,D]."""
    B, Hq, Nq, D = q.shape
    s2 = _scale_log2(sm_scale, Hq, D).view(1, Hq, 1)
    group = Hq // pp.km.shape[1]
    km = pp.km.to(torch.float32).repeat_interleave(group, dim=1) if group > 1 else pp.km.to(torch.float32)
    qkm = torch.einsum("bhnd,bhd->bhn", q.to(torch.float32), km)
    m, l = m.squeeze(-1), l.squeeze(-1)
    m_cur = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    lse2 = m_cur * s2 + torch.log2(l) + P_SCALE_LOG2            # l = 2688 * sum_k 2^((S_k - m) s)
    lse = lse2 / LOG2E + (s2 / LOG2E) * qkm
    return torch.where(l == 0, torch.full_like(lse, -math.inf), lse)


def sageattn3_oracle(q, k, v, tensor_layout: str = "HND", is_causal: bool = False, sm_scale=None,
                     per_block_mean: bool = True, return_lse: bool = False):
    """Whole pipeline (api.py:131-152) on CPU tensors; returns the output in the caller's layout
    (and the [B,Hq,Nq] log-sum-exp when `return_lse`)."""
    qh, kh, vh = (_to_hnd(t, tensor_layout) for t in (q, k, v))
    pp = prepass(qh, kh, vh, per_block_mean)
    if return_lse:
        o, m, l = attention_from_prepass(pp, is_causal, sm_scale, return_lse_parts=True)
        lse = lse_from_parts(pp, qh, m, l, sm_scale)
        return (o if tensor_layout == "HND" else o.transpose(1, 2)), lse
    o = attention_from_prepass(pp, is_causal, sm_scale)
    return o if tensor_layout == "HND" else o.transpose(1, 2)


def fp32_lse(q, k, tensor_layout: str = "HND", is_causal: bool = False, sm_scale=None) -> torch.Tensor:
    """ln sum_k exp(sm_scale * q.k) in fp32 from the unquantized inputs, [B,Hq,Nq]."""
    qh, kh = (_to_hnd(t, tensor_layout).to(torch.float32) for t in (q, k))
    B, Hq, Nq, D = qh.shape
    Hkv, Nk = kh.shape[1], kh.shape[2]
    if Hq != Hkv:
        kh = kh.repeat_interleave(Hq // Hkv, dim=1)
    s = _scale_log2(sm_scale, Hq, D).view(1, Hq, 1, 1) / LOG2E
    S = torch.matmul(qh, kh.transpose(-1, -2)) * s
    if is_causal:
        i = torch.arange(Nq).view(-1, 1)
        j = torch.arange(Nk).view(1, -1)
        S = S.masked_fill(j > i + (Nk - Nq), -math.inf)
    return torch.logsumexp(S, dim=-1)


def fp32_attention(q, k, v, tensor_layout: str = "HND", is_causal: bool = False, sm_scale=None) -> torch.Tensor:
    """Full-precision softmax(QK^T * scale)V in fp32, for the 'reported, not gated' comparison."""
    qh, kh, vh = (_to_hnd(t, tensor_layout).to(torch.float32) for t in (q, k, v))
    B, Hq, Nq, D = qh.shape
    Hkv, Nk = kh.shape[1], kh.shape[2]
    if Hq != Hkv:
        kh = kh.repeat_interleave(Hq // Hkv, dim=1)
        vh = vh.repeat_interleave(Hq // Hkv, dim=1)
    s = _scale_log2(sm_scale, Hq, D).view(1, Hq, 1, 1) / LOG2E
    S = torch.matmul(qh, kh.transpose(-1, -2)) * s
    if is_causal:
        i = torch.arange(Nq).view(-1, 1)
        j = torch.arange(Nk).view(1, -1)
        S = S.masked_fill(j > i + (Nk - Nq), -math.inf)
    P = torch.softmax(S, dim=-1)
    P = torch.nan_to_num(P, nan=0.0)
    o = torch.matmul(P, vh)
    return o if tensor_layout == "HND" else o.transpose(1, 2)


# --------------------------------------------------------------------------------------------------
# metrics
# --------------------------------------------------------------------------------------------------
def cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.to(torch.float64).flatten()
    b = b.to(torch.float64).flatten()
    return float((a @ b) / (a.norm() * b.norm()).clamp_min(1e-300))


def rel_l1(a: torch.Tensor, ref: torch.Tensor) -> float:
    a = a.to(torch.float64)
    ref = ref.to(torch.float64)
    return float((a - ref).abs().sum() / ref.abs().sum().clamp_min(1e-300))


# --------------------------------------------------------------------------------------------------
# synthetic inputs of the benchmark configurations (seeded; shapes and distributions only)
# --------------------------------------------------------------------------------------------------
def make_inputs(B: int, Hq: int, Hkv: int, Nq: int, Nk: int, D: int, seed: int, dtype=torch.bfloat16,
                k_offset_std: float = 0.0, k_outlier_channels: int = 0, rope_base: float | None = None):
    """Q, V ~ N(0,1); K ~ N(0,1) + per-(b,h) channel offset ~ N(0, k_offset_std^2) shared over tokens;
    optionally K scaled x2 on `k_outlier_channels` random channels; optionally rotate-half RoPE on Q, K."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, Nq, D, generator=g)
    k = torch.randn(B, Hkv, Nk, D, generator=g)
    v = torch.randn(B, Hkv, Nk, D, generator=g)
    if k_offset_std:
        k = k + k_offset_std * torch.randn(B, Hkv, 1, D, generator=g)
    if k_outlier_channels:
        idx = torch.randperm(D, generator=g)[:k_outlier_channels]
        k[..., idx] *= 2.0
    if rope_base is not None:
        def rope(x, n):
            half = D // 2
            inv = rope_base ** (-torch.arange(half, dtype=torch.float32) / half)
            ang = torch.arange(n, dtype=torch.float32).view(-1, 1) * inv.view(1, -1)
            c, s = ang.cos(), ang.sin()
            x1, x2 = x[..., :half], x[..., half:]
            return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
        q, k = rope(q, Nq), rope(k, Nk)
    return q.to(dtype), k.to(dtype), v.to(dtype)
