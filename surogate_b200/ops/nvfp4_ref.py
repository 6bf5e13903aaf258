"""PyTorch emulation of the NVFP4 format (E2M1 values, UE4M3 scale per 16 elements, fp32 tensor scale).

Used as the oracle of the CUDA quantisers / block-scaled GEMM and as the CPU implementation of the recipe.
Parity: recipes/nvfp4/kernels/quant_nvfp4_cutlass.cu (two-level scaling, encode scale 448*6 = 2688).
"""
from __future__ import annotations

import torch

E2M1_GRID = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
ENCODE = 2688.0  # 448 (max e4m3) * 6 (max e2m1)


def e2m1_round_nearest(s: torch.Tensor) -> torch.Tensor:
    """4-bit codes (sign << 3 | magnitude index); ties go to the even mantissa, as the hardware conversion does."""
    a = s.abs().clamp(max=6.0)
    code = torch.zeros_like(a, dtype=torch.int64)
    for thr, inclusive, c in [(0.25, True, 1), (0.75, False, 2), (1.25, True, 3), (1.75, False, 4), (2.5, True, 5), (3.5, False, 6), (5.0, True, 7)]:
        code = torch.where((a > thr) if inclusive else (a >= thr), torch.full_like(code, c), code)
    return code + 8 * (s < 0).long()


def decode_codes(codes: torch.Tensor) -> torch.Tensor:
    mag = E2M1_GRID.to(codes.device)[codes & 7]
    return torch.where((codes & 8) != 0, -mag, mag)


def quantize(x: torch.Tensor, amax: float | torch.Tensor | None = None, block2d: bool = False):
    """x [rows, K] -> (codes int64 [rows, K], decoded block scales fp32 [rows, K/16], global encode scale)."""
    x = x.float()
    rows, K = x.shape
    at = x.abs().max() if amax is None else torch.as_tensor(amax, dtype=torch.float32, device=x.device)
    # correctly rounded fp32 quotient (GPU tensor division may be off by an ulp, which flips exact rounding ties)
    ge = torch.tensor(float(torch.tensor(ENCODE / float(at), dtype=torch.float32)) if float(at) > 0 else 1.0, device=x.device)
    xb = x.view(rows, K // 16, 16)
    bmax = xb.abs().amax(-1)
    if block2d:
        bmax = bmax.view(rows // 16, 16, K // 16).amax(1, keepdim=True).expand(rows // 16, 16, K // 16).reshape(rows, K // 16)
    sf = (bmax * ge / 6.0).clamp(max=448.0).to(torch.float8_e4m3fn)
    sfd = sf.float()
    mul = torch.where(sfd > 0, ge / sfd, torch.zeros_like(sfd))
    codes = e2m1_round_nearest(xb * mul.unsqueeze(-1)).view(rows, K)
    return codes, sfd, ge


def dequantize(codes: torch.Tensor, sfd: torch.Tensor, ge: torch.Tensor) -> torch.Tensor:
    rows, K = codes.shape
    return (decode_codes(codes).view(rows, K // 16, 16) * (sfd / ge).unsqueeze(-1)).view(rows, K)


def pack_codes(codes: torch.Tensor) -> torch.Tensor:
    """Two codes per byte, even element in the low nibble."""
    c = codes.to(torch.uint8)
    return (c[:, 0::2] | (c[:, 1::2] << 4)).contiguous()


def unpack_codes(q: torch.Tensor) -> torch.Tensor:
    lo, hi = (q & 15).long(), (q >> 4).long()
    return torch.stack([lo, hi], -1).view(q.shape[0], -1)


def sf_to_atoms(sf_bytes: torch.Tensor) -> torch.Tensor:
    """[rows, K/16] uint8 -> flat atom layout: ((r/128)*atoms_k + kb/4)*512 + (r%32)*16 + ((r%128)/32)*4 + kb%4."""
    rows, kb = sf_bytes.shape
    R, KB = (rows + 127) // 128 * 128, (kb + 3) // 4 * 4
    p = torch.zeros(R, KB, dtype=torch.uint8, device=sf_bytes.device)
    p[:rows, :kb] = sf_bytes
    # (rm, m1, m0, ak, k1) -> (rm, ak, m0, m1, k1)
    return p.view(R // 128, 4, 32, KB // 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(-1)


def atoms_to_sf(flat: torch.Tensor, rows: int, kb: int) -> torch.Tensor:
    R, KB = (rows + 127) // 128 * 128, (kb + 3) // 4 * 4
    p = flat[: R * KB].view(R // 128, KB // 4, 32, 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(R, KB)
    return p[:rows, :kb]


def hadamard16(x: torch.Tensor, sign_mask: int) -> torch.Tensor:
    """Orthonormal 16-point Hadamard (Sylvester order) with random signs, applied to the last dimension in blocks of 16."""
    H = torch.ones(1, 1)
    for _ in range(4):
        H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
    signs = torch.tensor([-1.0 if (sign_mask >> i) & 1 else 1.0 for i in range(16)])
    M = (H * 0.25) @ torch.diag(signs)
    shp = x.shape
    return (x.float().reshape(-1, 16) @ M.t().to(x.device)).reshape(shp)
