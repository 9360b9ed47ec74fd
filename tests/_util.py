"""Test helpers: decode the workspace the C-ABI library fills into plain [rows, cols] tensors on the CPU."""
import torch

from oracle import sage3_oracle as O


def deatomize_sf(buf: torch.Tensor, n_heads: int, n_tiles: int, n_atoms: int) -> torch.Tensor:
    """[heads][tiles][atoms][512] bytes in 128-row x 4-scale atoms -> [heads][tiles*128 rows][atoms*4 scales]."""
    x = buf.reshape(n_heads, n_tiles, n_atoms, 32, 4, 4)          # (r % 32, r // 32, c)
    x = x.permute(0, 1, 4, 3, 2, 5)                               # heads, tiles, r // 32, r % 32, atom, c
    return x.reshape(n_heads, n_tiles * 128, n_atoms * 4).contiguous()


def read_workspace(prob) -> dict:
    """All pre-pass products of a Sage3Problem as CPU tensors in the oracle's shapes."""
    d, lay = prob.desc, prob.ws.layout
    B, Hq, Hkv, D = d.B, d.Hq, d.Hkv, d.D
    nqp, nkp, nqm = lay.nq_pad, lay.nk_pad, lay.nqm
    dt = prob.q.dtype
    buf = prob.ws.buf.cpu()

    def reg(name, nbytes):
        off = getattr(lay, name)
        return buf[off: off + nbytes]

    out = {}
    out["km"] = reg("km", B * Hkv * D * 2).view(dt).reshape(B, Hkv, D)
    out["qm"] = reg("qm", B * Hq * nqm * D * 2).view(dt).reshape(B, Hq, nqm, D)
    out["delta"] = reg("delta", B * Hq * nqm * nkp * 2).view(dt).reshape(B, Hq, nqm, nkp)
    out["q_codes"] = O.unpack_nibbles(reg("q_codes", B * Hq * nqp * D // 2).reshape(B, Hq, nqp, D // 2))
    out["k_codes"] = O.unpack_nibbles(reg("k_codes", B * Hkv * nkp * D // 2).reshape(B, Hkv, nkp, D // 2))
    out["vt_codes"] = O.unpack_nibbles(reg("v_codes", B * Hkv * D * nkp // 2).reshape(B, Hkv, D, nkp // 2))
    na = D // 64
    out["q_sf"] = deatomize_sf(reg("q_sf", B * Hq * (nqp // 128) * na * 512), B * Hq, nqp // 128, na).reshape(B, Hq, nqp, D // 16)
    out["k_sf"] = deatomize_sf(reg("k_sf", B * Hkv * (nkp // 128) * na * 512), B * Hkv, nkp // 128, na).reshape(B, Hkv, nkp, D // 16)
    v = reg("v_sf", B * Hkv * (nkp // 128) * 1024).reshape(B * Hkv, nkp // 128, 2, 32, 4, 4)   # tile, atom, r%32, r//32, c
    v = v.permute(0, 4, 3, 1, 2, 5).reshape(B * Hkv, 128, (nkp // 128) * 8)                    # channel rows, token groups
    out["vt_sf"] = v[:, :D].reshape(B, Hkv, D, nkp // 16).contiguous()
    out["vt_sf_pad"] = v[:, D:]
    return out


def canon(codes: torch.Tensor) -> torch.Tensor:
    """-0 and +0 are the same number: fold code 8 onto code 0 before comparing."""
    return torch.where(codes == 8, torch.zeros_like(codes), codes)
