"""Index maps from the reference's quantized-tensor layouts (an sm_120 register-layout artefact) to natural order.

Used only by the tests that hold the CPU oracle against tensors recorded from the reference's own kernels.
Reference locations (paths inside the reference project, sageattention3_blackwell/sageattn3/quantization/):
  fp4_quantization_4d.cu:160-168   K: inside every group of 32 rows, stored row p holds input row
                                   (p // 8) * 2 + ((p % 8) // 2) * 8 + (p % 8) % 2
  fp4_quantization_4d.cu:242-249   scale bytes of Q / K: per (batch, head) slab, groups of 64 rows; inside a group
                                   byte (c // 4) * 256 + (r % 16) * 16 + (r // 16) * 4 + c % 4 for row r, scale column c
  fp4_quantization_4d.cu:367-377   scale bytes of V^T: the same atoms with r = channel, c = token // 16
"""
import torch


def k_row_of_stored_row(n_rows: int) -> torch.Tensor:
    """src[p] = the input row whose data the reference's K kernel stores at row p."""
    p = torch.arange(n_rows)
    base, q = (p // 32) * 32, p % 32
    return base + (q // 8) * 2 + ((q % 8) // 2) * 8 + (q % 8) % 2


def unpermute_k_rows(stored: torch.Tensor) -> torch.Tensor:
    """[..., rows, x] in the reference's stored K row order -> natural row order."""
    src = k_row_of_stored_row(stored.shape[-2])
    nat = torch.empty_like(stored)
    nat[..., src, :] = stored
    return nat


def deatomize_sf64(sf: torch.Tensor) -> torch.Tensor:
    """[..., rows, cols] whose bytes (per leading index) are laid out in the reference's 64-row x 4-column atoms
    -> the same shape in plain row-major meaning.  rows % 64 == 0, cols % 4 == 0."""
    *lead, rows, cols = sf.shape
    x = sf.reshape(*lead, rows // 64, cols // 4, 16, 4, 4)          # group, atom, r % 16, r // 16, c % 4
    n = len(lead)
    x = x.permute(*range(n), n, n + 3, n + 2, n + 1, n + 4)         # group, r // 16, r % 16, atom, c % 4
    return x.reshape(*lead, rows, cols).contiguous()
