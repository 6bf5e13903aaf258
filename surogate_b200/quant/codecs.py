"""Block-quantised storage formats for frozen base weights.

Every codec works on a flat tensor whose length is a multiple of its block size and returns a dict of tensors (the
"state") from which ``dequantize`` rebuilds bf16 values:

* ``BnbNF4``     — 4-bit NormalFloat, blocks of 64, fp32 abs-max per block; optional double quantisation of the abs-max
                   values (uint8 codes in blocks of 256 with an fp32 scale per block after subtracting their mean).
* ``BlockFP8``   — E4M3 values with one fp32 scale per block of 64 / 128 / 256 (also the layout of pre-quantised
                   "fp8 block" checkpoints, where blocks are 128 x 128 tiles: see ``dequantize_2d``).
* ``NVFP4Storage`` — E2M1 values, UE4M3 scale per 16 elements, one fp32 tensor scale.
* ``MXFP4``      — E2M1 values with an E8M0 (power of two) scale per 32 elements: read-only, for pre-quantised checkpoints.

Parity: csrc/src/kernels/bnb_quant.cu, block_quant.cu, mxfp4_dequant.cu, csrc/src/runtime/qlora/ (generic_weight_manager.cpp).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

NF4_LEVELS = [-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635, -0.18477343022823334,
              -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
              0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0]
E2M1_LEVELS = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def _cuda_ext(t: torch.Tensor):
    """The kernel extension when ``t`` lives on a GPU (QLoRA rebuilds every frozen layer twice per step: that runs on the CUDA
    dequantisers of csrc/qlora_kernels.cu); None on CPU, where the PyTorch statements below are used."""
    if not t.is_cuda:
        return None
    from ..ops import ext

    return ext()


def _pack4(codes: torch.Tensor) -> torch.Tensor:
    c = codes.reshape(-1, 2).to(torch.uint8)
    return (c[:, 0] | (c[:, 1] << 4)).contiguous()


def _unpack4(packed: torch.Tensor) -> torch.Tensor:
    return torch.stack([packed & 0xF, packed >> 4], dim=1).reshape(-1)


def _nearest(x: torch.Tensor, levels: torch.Tensor) -> torch.Tensor:
    """Index of the nearest level (levels sorted ascending): searchsorted on the midpoints."""
    mids = (levels[1:] + levels[:-1]) / 2
    return torch.searchsorted(mids, x.contiguous())


class BnbNF4:
    name = "bnb_nf4"

    def __init__(self, block: int = 64, double_quant: bool = True):
        self.block, self.double = block, double_quant

    def quantize(self, x: torch.Tensor) -> Dict[str, torch.Tensor]:
        n = x.numel()
        assert n % self.block == 0, f"NF4: {n} elements are not a multiple of the block size {self.block}"
        xb = x.reshape(-1, self.block).float()
        absmax = xb.abs().amax(1).clamp_min(1e-12)
        lv = torch.tensor(NF4_LEVELS, device=x.device)
        codes = _nearest((xb / absmax[:, None]).reshape(-1), lv)
        st = {"codes": _pack4(codes)}
        if self.double:
            nb = absmax.numel()
            pad = (-nb) % 256
            a = torch.nn.functional.pad(absmax, (0, pad))
            offset = absmax.mean()
            a2 = (a - offset).reshape(-1, 256)
            s2 = a2.abs().amax(1).clamp_min(1e-12) / 127.0
            st.update(absmax_q=torch.round(a2 / s2[:, None]).clamp(-127, 127).to(torch.int8).reshape(-1)[:nb + pad], absmax_scale=s2,
                      absmax_offset=offset.reshape(1), n_blocks=torch.tensor([nb]))
        else:
            st["absmax"] = absmax
        return st

    def _absmax(self, st) -> torch.Tensor:
        if "absmax" in st:
            return st["absmax"]
        nb = int(st["n_blocks"])
        a = st["absmax_q"].float().reshape(-1, 256) * st["absmax_scale"][:, None]
        return (a.reshape(-1)[:nb] + st["absmax_offset"])

    def dequantize(self, st, dtype=torch.bfloat16) -> torch.Tensor:
        e = _cuda_ext(st["codes"])
        n = st["codes"].numel() * 2
        if e is not None and n % 8 == 0 and self.block % 8 == 0:
            if "absmax" in st:
                out = e.dequant_blockwise("bnb_nf4", st["codes"], st["absmax"].float().contiguous(), None, None, n, self.block)
            else:
                out = e.dequant_blockwise("bnb_nf4", st["codes"], st["absmax_q"].contiguous(), st["absmax_scale"].float().contiguous(),
                                          st["absmax_offset"].float().contiguous(), n, self.block)
            return out if dtype == torch.bfloat16 else out.to(dtype)
        return self.dequantize_reference(st, dtype)

    def dequantize_reference(self, st, dtype=torch.bfloat16) -> torch.Tensor:
        lv = torch.tensor(NF4_LEVELS, device=st["codes"].device)
        v = lv[_unpack4(st["codes"]).long()].reshape(-1, self.block) * self._absmax(st)[:, None]
        return v.reshape(-1).to(dtype)

    def bits_per_element(self) -> float:
        return 4 + (8 / self.block + 32 / (self.block * 256) if self.double else 32 / self.block)


class BlockFP8:
    name = "fp8_block"

    def __init__(self, block: int = 128):
        assert block in (64, 128, 256)
        self.block = block

    def quantize(self, x: torch.Tensor) -> Dict[str, torch.Tensor]:
        assert x.numel() % self.block == 0
        xb = x.reshape(-1, self.block).float()
        scale = xb.abs().amax(1).clamp_min(1e-12) / 448.0
        return {"q": (xb / scale[:, None]).to(torch.float8_e4m3fn).reshape(-1), "scale": scale}

    def dequantize(self, st, dtype=torch.bfloat16) -> torch.Tensor:
        e = _cuda_ext(st["q"])
        if e is not None and st["q"].numel() % 8 == 0:
            out = e.dequant_blockwise("fp8_block", st["q"].contiguous(), st["scale"].float().contiguous(), None, None, st["q"].numel(), self.block)
            return out if dtype == torch.bfloat16 else out.to(dtype)
        return self.dequantize_reference(st, dtype)

    def dequantize_reference(self, st, dtype=torch.bfloat16) -> torch.Tensor:
        return (st["q"].float().reshape(-1, self.block) * st["scale"][:, None]).reshape(-1).to(dtype)

    @staticmethod
    def dequantize_2d(q: torch.Tensor, scale_inv: torch.Tensor, block=(128, 128), dtype=torch.bfloat16) -> torch.Tensor:
        """Pre-quantised checkpoints: ``weight`` [N, K] E4M3 with ``weight_scale_inv`` [ceil(N/128), ceil(K/128)]."""
        N, K = q.shape
        s = scale_inv.float().repeat_interleave(block[0], 0)[:N].repeat_interleave(block[1], 1)[:, :K]
        return (q.float() * s).to(dtype)

    def bits_per_element(self) -> float:
        return 8 + 32 / self.block


class NVFP4Storage:
    name = "nvfp4"

    def __init__(self, four_over_six: bool = True):
        self.four_over_six = four_over_six

    def _quant_blocks(self, xb: torch.Tensor, ge: torch.Tensor, vmax: float):
        lv = torch.tensor(E2M1_LEVELS, device=xb.device)
        amax = xb.abs().amax(1)
        sf = (amax * ge / vmax).to(torch.float8_e4m3fn).float().clamp_min(2 ** -9)
        y = xb * ge / sf[:, None]
        idx = _nearest(y.abs().reshape(-1), lv).reshape(y.shape)
        deq = lv[idx] * torch.sign(y) * sf[:, None] / ge
        return idx, sf, deq

    def quantize(self, x: torch.Tensor) -> Dict[str, torch.Tensor]:
        assert x.numel() % 16 == 0
        xb = x.reshape(-1, 16).float()
        g = xb.abs().max().clamp_min(1e-12)
        # tensor encode factor: 2688 = 448 * 6 for plain NVFP4; 1536 = 256 * 6 = 384 * 4 with four-over-six, so that the block scale of
        # either mapping stays inside the UE4M3 range (arXiv 2512.02010)
        ge = (1536.0 if self.four_over_six else 448.0 * 6.0) / g
        idx, sf, deq = self._quant_blocks(xb, ge, 6.0)
        if self.four_over_six:  # per block, keep whichever of max=6 / max=4 mapping reconstructs better
            idx4, sf4, deq4 = self._quant_blocks(xb, ge, 4.0)
            better = ((deq4 - xb) ** 2).sum(1) < ((deq - xb) ** 2).sum(1)
            idx = torch.where(better[:, None], idx4, idx)
            sf = torch.where(better, sf4, sf)
        sign = (xb < 0).to(torch.uint8) << 3
        return {"codes": _pack4((idx.to(torch.uint8) | sign).reshape(-1)), "sf": sf.to(torch.float8_e4m3fn), "ge_inv": (1.0 / ge).reshape(1)}

    def dequantize(self, st, dtype=torch.bfloat16) -> torch.Tensor:
        e = _cuda_ext(st["codes"])
        n = st["codes"].numel() * 2
        if e is not None and n % 16 == 0:
            out = e.dequant_blockwise("nvfp4", st["codes"], st["sf"].contiguous().view(torch.uint8), st["ge_inv"].float().contiguous(), None, n, 16)
            return out if dtype == torch.bfloat16 else out.to(dtype)
        return self.dequantize_reference(st, dtype)

    def dequantize_reference(self, st, dtype=torch.bfloat16) -> torch.Tensor:
        lv = torch.tensor(E2M1_LEVELS, device=st["codes"].device)
        c = _unpack4(st["codes"])
        v = lv[(c & 7).long()] * torch.where((c & 8) > 0, -1.0, 1.0)
        return (v.reshape(-1, 16) * st["sf"].float()[:, None] * st["ge_inv"]).reshape(-1).to(dtype)

    def bits_per_element(self) -> float:
        return 4.5


class MXFP4:
    """E2M1 codes (two per byte, low nibble first) + E8M0 scales per 32 elements, as stored by pre-quantised checkpoints."""
    name = "mxfp4"

    def dequantize(self, st, dtype=torch.bfloat16) -> torch.Tensor:
        e = _cuda_ext(st["blocks"])
        n = st["blocks"].numel() * 2
        if e is not None and n % 32 == 0:
            out = e.dequant_blockwise("mxfp4", st["blocks"].reshape(-1).contiguous(), st["scales"].reshape(-1).contiguous(), None, None, n, 32)
            return out if dtype == torch.bfloat16 else out.to(dtype)
        return self.dequantize_reference(st, dtype)

    def dequantize_reference(self, st, dtype=torch.bfloat16) -> torch.Tensor:
        lv = torch.tensor(E2M1_LEVELS, device=st["blocks"].device)
        c = _unpack4(st["blocks"].reshape(-1))
        v = lv[(c & 7).long()] * torch.where((c & 8) > 0, -1.0, 1.0)
        scale = torch.exp2(st["scales"].reshape(-1).float() - 127.0)
        return (v.reshape(-1, 32) * scale[:, None]).reshape(-1).to(dtype)

    def quantize(self, x: torch.Tensor) -> Dict[str, torch.Tensor]:
        xb = x.reshape(-1, 32).float()
        e = torch.ceil(torch.log2(xb.abs().amax(1).clamp_min(2.0 ** -126) / 6.0)).clamp(-127, 127)
        lv = torch.tensor(E2M1_LEVELS, device=x.device)
        y = xb / torch.exp2(e)[:, None]
        idx = _nearest(y.abs().reshape(-1), lv).reshape(y.shape).to(torch.uint8) | ((y < 0).to(torch.uint8) << 3)
        return {"blocks": _pack4(idx.reshape(-1)), "scales": (e + 127).to(torch.uint8)}

    def bits_per_element(self) -> float:
        return 4.25


CODECS = {"bnb_nf4": BnbNF4, "fp8_block": BlockFP8, "nvfp4": NVFP4Storage, "mxfp4": MXFP4}


def make_codec(kind: Optional[str], **kw):
    if not kind:
        return None
    if kind not in CODECS:
        raise ValueError(f"unknown QLoRA storage '{kind}' (known: {sorted(CODECS)})")
    return CODECS[kind](**kw)
