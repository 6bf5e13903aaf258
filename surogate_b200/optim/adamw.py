"""AdamW with fp32 state and with 8-bit state, stepping directly on flat bucket shards.

Hyper-parameters reach the kernels through an 8-float device vector
``[lr, beta1, beta2, eps, weight_decay, 1-beta1^t, 1-beta2^t, grad_scale]`` so that the
clip scale (computed on the device from the gradient norm) never visits the host and
a captured step can be replayed with new values.

8-bit state (the reference's production optimizer): momentum as int8 through a softsign
transform of the group-normalised value, variance as uint8 of sqrt(v), groups of 32 elements
with fp16 scales (csrc/src/runtime/optimizers/flash_adamw_8bit.h:1-27).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch


@dataclass
class OptimizerConfig:
    name: str = "adamw_8bit"
    learning_rate: float = 2e-4
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0
    max_grad_norm: float = 1.0
    normuon_momentum: float = 0.95
    normuon_beta2: float = 0.95
    normuon_cautious_wd: bool = True
    normuon_lr_scale: float = 1.0
    normuon_momentum_8bit: bool = False   # momentum as int8 codes with an fp16 scale per 128 values instead of bf16


def _softsign_quant_reference(mi, vi):
    """Pure-PyTorch twin of the 8-bit state encoding (used on CPU and as the kernel's oracle)."""
    n = mi.numel()
    pad = (-n) % 32
    mp = torch.nn.functional.pad(mi, (0, pad)).view(-1, 32)
    sp = torch.nn.functional.pad(vi.sqrt(), (0, pad)).view(-1, 32)
    am = mp.abs().amax(1).clamp_min(6e-8).half().float().clamp_min(6e-8)
    av = sp.amax(1).clamp_min(6e-8).half().float().clamp_min(6e-8)
    # scales are rounded up in the kernel; emulate by nudging when half rounding went below the true max
    am = torch.where(am < mp.abs().amax(1), torch.nextafter(am.half(), torch.tensor(float("inf"), dtype=torch.half, device=am.device)).float(), am)
    av = torch.where(av < sp.amax(1), torch.nextafter(av.half(), torch.tensor(float("inf"), dtype=torch.half, device=av.device)).float(), av)
    xn = mp / am[:, None]
    m8 = torch.round(2 * xn / (1 + xn.abs()) * 127).clamp(-127, 127).to(torch.int8)
    v8 = torch.round(sp / av[:, None] * 255).clamp(0, 255).to(torch.uint8)
    return m8.view(-1)[:n], v8.view(-1)[:n], am.half(), av.half()


def _softsign_dequant_reference(m8, v8, ms, vs):
    n = m8.numel()
    pad = (-n) % 32
    y = torch.nn.functional.pad(m8.float(), (0, pad)).view(-1, 32) / 127.0
    m = y / (2 - y.abs()) * ms.float()[:, None]
    s = torch.nn.functional.pad(v8.float(), (0, pad)).view(-1, 32) / 255.0 * vs.float()[:, None]
    return m.view(-1)[:n], (s * s).view(-1)[:n]


class AdamW:
    """fp32 first/second moments (4 + 4 bytes per parameter)."""
    state_bytes_per_param = 8

    def __init__(self, cfg: OptimizerConfig, store):
        self.cfg = cfg
        self.store = store
        self.state: Dict[str, Dict[str, torch.Tensor]] = {}
        self.offload_state = False  # moments in pinned host memory (streamed through the GPU by StreamedOptimizerStep)
        self.use_kernels = store.device.type == "cuda"
        if self.use_kernels:
            from ..ops import ext

            self.ext = ext()

    def _zeros(self, n: int, dtype) -> torch.Tensor:
        if self.offload_state and self.store.device.type == "cuda":
            return torch.zeros(n, dtype=dtype, pin_memory=True)
        return torch.zeros(n, dtype=dtype, device=self.store.device)

    def _state(self, b):
        st = self.state.get(b.name)
        if st is None:
            n = b.master.numel()
            st = self.state[b.name] = {"m": self._zeros(n, torch.float32), "v": self._zeros(n, torch.float32)}
        return st

    def step_bucket(self, b, grad: torch.Tensor, hp: torch.Tensor, hp_host) -> None:
        st = self._state(b)
        mask = self.store.decay_mask(b)
        if self.use_kernels:
            self.ext.adamw_step(b.master, grad.contiguous(), st["m"], st["v"], mask, hp)
            return
        lr, b1, b2, eps, wd, bc1, bc2 = hp_host
        if float(hp[7]) == 0.0:  # skipped update (non-finite gradient norm), as in the kernels
            return
        g = grad.float() * hp[7]
        st["m"].mul_(b1).add_(g, alpha=1 - b1)
        st["v"].mul_(b2).addcmul_(g, g, value=1 - b2)
        p = b.master.float()
        p = p * (1 - lr * wd * mask.float()) - lr * (st["m"] / bc1) / ((st["v"] / bc2).sqrt() + eps)
        b.master.copy_(p.to(b.master.dtype))

    def state_tensors(self, b):
        return self._state(b)


class AdamW8bit(AdamW):
    """int8 softsign momentum + uint8 sqrt variance, group 32, fp16 scales (≈2.13 bytes per parameter)."""
    state_bytes_per_param = 2.125

    def _state(self, b):
        st = self.state.get(b.name)
        if st is None:
            n = b.master.numel()
            ng = (n + 31) // 32
            st = self.state[b.name] = {"m": self._zeros(n, torch.int8), "v": self._zeros(n, torch.uint8),
                                       "m.scales": self._zeros(ng, torch.float16), "v.scales": self._zeros(ng, torch.float16)}
        return st

    def step_bucket(self, b, grad, hp, hp_host) -> None:
        st = self._state(b)
        if self.use_kernels:
            self.ext.adamw8_step(b.master, grad.contiguous(), st["m"], st["v"], st["m.scales"], st["v.scales"], self.store.decay_mask_blocks(b), hp)
            return
        mask = self.store.decay_mask(b)
        lr, b1, b2, eps, wd, bc1, bc2 = hp_host
        if float(hp[7]) == 0.0:
            return
        m, v = _softsign_dequant_reference(st["m"], st["v"], st["m.scales"], st["v.scales"])
        g = grad.float() * hp[7]
        m = b1 * m + (1 - b1) * g
        v = b2 * v + (1 - b2) * g * g
        p = b.master.float()
        p = p * (1 - lr * wd * mask.float()) - lr * (m / bc1) / ((v / bc2).sqrt() + eps)
        b.master.copy_(p.to(b.master.dtype))
        m8, v8, ms, vs = _softsign_quant_reference(m, v)
        st["m"].copy_(m8), st["v"].copy_(v8), st["m.scales"].copy_(ms), st["v.scales"].copy_(vs)


def make_optimizer(cfg: OptimizerConfig, store):
    name = cfg.name.lower()
    if name in ("adamw_8bit", "adamw8bit"):
        return AdamW8bit(cfg, store)
    if name == "adamw":
        return AdamW(cfg, store)
    if name == "normuon":
        from .normuon import NorMuon

        return NorMuon(cfg, store)
    raise ValueError(f"unknown optimizer '{cfg.name}' (adamw_8bit | adamw | normuon)")
