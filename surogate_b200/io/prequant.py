"""Reading pre-quantised HuggingFace checkpoints: a view over a checkpoint that hands out full-precision tensors.

Formats (detected per tensor from the companion tensors that stand next to it, so mixed checkpoints work):

* block FP8 (DeepSeek / Qwen3 ``-FP8`` releases): ``X.weight`` float8_e4m3fn ``[N, K]`` + ``X.weight_scale_inv`` fp32
  ``[ceil(N/bn), ceil(K/bk)]`` (block from ``quantization_config.weight_block_size``, default 128 x 128); per-tensor variants
  carry a scalar ``X.weight_scale``.
* NVFP4 (ModelOpt): ``X.weight`` uint8 ``[N, K/2]`` (two E2M1 codes per byte, low nibble first), ``X.weight_scale`` float8_e4m3fn
  ``[N, K/16]``, ``X.weight_scale_2`` fp32 scalar; value = code x block scale x tensor scale.
* MXFP4 (gpt-oss): ``X_blocks`` uint8 ``[..., R, K/32, 16]`` + ``X_scales`` uint8 E8M0 ``[..., R, K/32]`` (bias 127); the stored
  matrix is the transpose of the bf16 layout, as in transformers' gpt-oss integration, so the result is transposed back.
* bitsandbytes NF4: ``X.weight`` uint8 ``[numel/2, 1]`` (high nibble first), ``X.weight.absmax`` (fp32, or uint8 with
  ``nested_absmax`` / ``nested_quant_map`` and an offset: double quantisation), ``X.weight.quant_map`` and the JSON blob
  ``X.weight.quant_state.bitsandbytes__nf4`` (shape, block sizes, offset).

The parameter store then re-quantises frozen weights into its own storage codec (``ParamStore.quantize_frozen``): the flat bucket
layout with 1-D blocks differs from every checkpoint layout above, so the bytes are not adopted as they are.

Parity: csrc/src/runtime/qlora/{fp8,nvfp4,mxfp4,bnb}_weight_provider.*, surogate/utils/hf.py (quantization_config detection).
"""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional, Tuple

import torch

E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])
SUFFIXES = ("_scale_inv", "_scale", "_scale_2", "_blocks", "_scales", ".absmax", ".quant_map", ".nested_absmax", ".nested_quant_map")


def dequant_fp8_block(q: torch.Tensor, scale_inv: torch.Tensor, block: Tuple[int, int] = (128, 128), dtype=torch.bfloat16) -> torch.Tensor:
    w = q.to(torch.float32)
    if scale_inv.numel() == 1:
        return (w * scale_inv.float().reshape(())).to(dtype)
    bn, bk = block
    s = scale_inv.float().repeat_interleave(bn, 0)[: w.shape[0]].repeat_interleave(bk, 1)[:, : w.shape[1]]
    return (w * s).to(dtype)


def dequant_nvfp4(packed: torch.Tensor, block_scale: torch.Tensor, tensor_scale: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    lut = E2M1.to(packed.device)
    lo, hi = lut[(packed & 0x0F).long()], lut[(packed >> 4).long()]
    w = torch.stack([lo, hi], -1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
    s = block_scale.to(torch.float32).repeat_interleave(16, -1)[..., : w.shape[-1]]
    return (w * s * tensor_scale.float().reshape(())).to(dtype)


def dequant_mxfp4(blocks: torch.Tensor, scales: torch.Tensor, dtype=torch.bfloat16, transpose: bool = True) -> torch.Tensor:
    lut = E2M1.to(blocks.device)
    lo, hi = lut[(blocks & 0x0F).long()], lut[(blocks >> 4).long()]
    w = torch.stack([lo, hi], -1).reshape(*blocks.shape[:-1], 32)                    # [..., R, K/32, 32]
    w = torch.ldexp(w, (scales.to(torch.int32) - 127).unsqueeze(-1))
    w = w.reshape(*blocks.shape[:-2], blocks.shape[-2] * 32)                          # [..., R, K]
    if transpose and w.dim() >= 2:
        w = w.transpose(-1, -2)
    return w.contiguous().to(dtype)


def dequant_bnb_nf4(packed: torch.Tensor, absmax: torch.Tensor, quant_map: torch.Tensor, state: Dict[str, Any], nested_absmax: Optional[torch.Tensor] = None,
                    nested_quant_map: Optional[torch.Tensor] = None, dtype=torch.bfloat16) -> torch.Tensor:
    shape = [int(x) for x in state["shape"]]
    numel = 1
    for d in shape:
        numel *= d
    block = int(state.get("blocksize", 64))
    if nested_absmax is not None:     # double quantisation: absmax itself is 8-bit with its own blocks and an offset
        nb = int(state.get("nested_blocksize", 256))
        a = nested_quant_map.float()[absmax.long()]
        a = a * nested_absmax.float().repeat_interleave(nb)[: a.numel()] + float(state.get("nested_offset", 0.0))
    else:
        a = absmax.float()
    p = packed.reshape(-1)
    codes = torch.stack([p >> 4, p & 0x0F], -1).reshape(-1)[:numel]
    w = quant_map.float()[codes.long()] * a.repeat_interleave(block)[:numel]
    return w.reshape(shape).to(dtype)


class DequantizingCheckpoint:
    """Same interface as ``LazyCheckpoint`` (``in``, ``get``, ``names``); quantised tensors come back dequantised and their
    companion tensors are hidden from ``names``."""

    def __init__(self, ckpt, hf_config: Optional[Dict[str, Any]] = None, dtype=torch.bfloat16):
        self.ckpt, self.dtype = ckpt, dtype
        q = (hf_config or {}).get("quantization_config") or {}
        wb = q.get("weight_block_size") or [128, 128]
        self.fp8_block = (int(wb[0]), int(wb[1]))
        self.stats = {"fp8": 0, "nvfp4": 0, "mxfp4": 0, "bnb_nf4": 0, "plain": 0}

    def _has(self, n: str) -> bool:
        return n in self.ckpt

    def __contains__(self, name: str) -> bool:
        return self._has(name) or self._has(name + "_blocks")

    def names(self) -> List[str]:
        out = []
        for n in self.ckpt.names():
            if n.endswith("_blocks"):
                out.append(n[: -len("_blocks")])
            elif not (any(n.endswith(s) for s in SUFFIXES) or ".quant_state." in n):
                out.append(n)
        return out

    def get(self, name: str) -> torch.Tensor:
        g = self.ckpt.get
        if not self._has(name) and self._has(name + "_blocks"):
            self.stats["mxfp4"] += 1
            return dequant_mxfp4(g(name + "_blocks"), g(name + "_scales"), self.dtype)
        t = g(name)
        if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            self.stats["fp8"] += 1
            if self._has(name + "_scale_inv"):
                return dequant_fp8_block(t, g(name + "_scale_inv"), self.fp8_block, self.dtype)
            if self._has(name + "_scale"):
                return dequant_fp8_block(t, g(name + "_scale"), self.fp8_block, self.dtype)
            return t.to(self.dtype)
        if t.dtype == torch.uint8 and self._has(name + "_scale_2"):
            self.stats["nvfp4"] += 1
            return dequant_nvfp4(t, g(name + "_scale"), g(name + "_scale_2"), self.dtype)
        if t.dtype == torch.uint8 and self._has(name + ".absmax"):
            self.stats["bnb_nf4"] += 1
            key = next((n for n in self.ckpt.names() if n.startswith(name + ".quant_state.")), None)
            if key is None:
                raise KeyError(f"'{name}' is bitsandbytes-packed but its quant_state blob is missing")
            state = json.loads(bytes(g(key).to(torch.uint8).tolist()).decode())
            nested = g(name + ".nested_absmax") if self._has(name + ".nested_absmax") else None
            nmap = g(name + ".nested_quant_map") if nested is not None else None
            return dequant_bnb_nf4(t, g(name + ".absmax"), g(name + ".quant_map"), state, nested, nmap, self.dtype)
        self.stats["plain"] += 1
        return t


def wrap_if_quantized(ckpt, hf_config: Optional[Dict[str, Any]]):
    """The dequantising view when the config declares a quantisation or the checkpoint carries companion tensors, else ``ckpt``."""
    declared = bool((hf_config or {}).get("quantization_config"))
    if not declared:
        probe = ckpt.names()
        declared = any(n.endswith(("_scale_inv", "_blocks", "_scale_2", ".absmax")) for n in probe)
    return DequantizingCheckpoint(ckpt, hf_config) if declared else ckpt
