"""NorMuon: momentum -> Newton-Schulz ("Polar Express") orthogonalisation -> neuron-wise second-moment
normalisation -> cautious weight decay, for 2-D hidden matrices; AdamW (8-bit state) for everything else
(embeddings, LM head, norms, biases, routers).

Orthogonalisation needs whole matrices, so with sharded state each 2-D parameter is updated by the rank
that owns the start of its slice range after gathering the momentum update for that matrix (the bucket
layout keeps every matrix contiguous); the small-batch GEMMs of the iteration run through the tcgen05
GEMM on a GPU.

Parity: csrc/src/runtime/optimizers/normuon.cu, polar_express.cu:96-400; docs/guides/optimizers.md.
"""
from __future__ import annotations

from typing import Dict

import torch

from .adamw import AdamW8bit, OptimizerConfig

# (a, b, c) coefficients of the quintic iteration X <- aX + (bA + cA^2)X with A = X X^T, per step
POLAR_EXPRESS_COEFFS = [
    (8.28721201814563, -23.595886519098837, 17.300387312530933),
    (4.107059111542203, -2.9478499167379106, 0.5448431082926601),
    (3.9486908534822946, -2.908902115962949, 0.5518191394370137),
    (3.3184196573706015, -2.488488024314874, 0.51004894012372),
    (2.300652019954817, -1.6689039845747493, 0.4188073119525673),
]


def polar_express(G: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Approximate the orthogonal polar factor of G (fp32 in, fp32 out; bf16 matmuls on a GPU)."""
    X = G.float()
    transposed = X.shape[0] > X.shape[1]
    if transposed:
        X = X.t()
    X = X / (X.norm() * 1.01 + 1e-7)
    work = torch.bfloat16 if X.is_cuda else torch.float32
    X = X.to(work)
    for a, b, c in POLAR_EXPRESS_COEFFS[:steps]:
        A = X @ X.t()
        B = b * A + c * (A @ A)
        X = a * X + B @ X
    X = X.float()
    return X.t() if transposed else X


class NorMuon(AdamW8bit):
    def __init__(self, cfg: OptimizerConfig, store):
        super().__init__(cfg, store)
        self.mom: Dict[str, torch.Tensor] = {}
        self.second: Dict[str, torch.Tensor] = {}

    @staticmethod
    def is_matrix_param(slot) -> bool:
        return len(slot.shape) == 2 and slot.entry.layer is not None and slot.entry.local not in ("router_weight",)

    def step_bucket(self, b, grad, hp, hp_host) -> None:
        """AdamW-8bit on the whole shard first (cheap), then overwrite matrix parameters with the NorMuon update."""
        store = self.store
        lo, hi = store.shard_range(b)
        matrices = [s for s in b.slots if s.trainable and self.is_matrix_param(s)]
        if not matrices:
            return super().step_bucket(b, grad, hp, hp_host)
        before = b.master.clone()
        super().step_bucket(b, grad, hp, hp_host)
        lr, _, _, eps, wd, _, _ = hp_host
        mu, beta2 = self.cfg.normuon_momentum, self.cfg.normuon_beta2
        gs = hp[7]
        for s in matrices:
            a, z = s.offset, s.offset + s.numel
            if store.sharded and not (a >= lo and z <= hi):
                # matrix straddles a shard boundary: gather its gradient slice from the owners
                g_full = store.grad_of(s.name).reshape(s.shape).float()
                own = a >= lo and a < hi
            else:
                g_full = grad[a - lo:z - lo].reshape(s.shape).float()
                own = True
            g_full = g_full * gs
            m = self.mom.get(s.name)
            if m is None:
                m = self.mom[s.name] = torch.zeros(s.shape, dtype=torch.float32, device=store.device)
            m.mul_(mu).add_(g_full, alpha=1 - mu)
            upd = polar_express(g_full.lerp(m, mu))
            # neuron-wise (row) second moment of the orthogonalised update, then renormalise to keep its norm
            v = self.second.get(s.name)
            row_ms = upd.pow(2).mean(1, keepdim=True)
            if v is None:
                v = self.second[s.name] = torch.zeros_like(row_ms)
            v.mul_(beta2).add_(row_ms, alpha=1 - beta2)
            scaled = upd / (v.sqrt() + eps)
            scaled = scaled * (upd.norm() / (scaled.norm() + 1e-12))
            scale = 0.2 * max(s.shape[0], s.shape[1]) ** 0.5 * self.cfg.normuon_lr_scale
            w_old = before if not store.sharded else None
            pa, pz = max(a, lo), min(z, hi)
            if pa >= pz:
                continue
            seg = slice(pa - lo, pz - lo)
            w = before[seg].float()
            u = scaled.reshape(-1)[pa - a:pz - a]
            if self.cfg.normuon_cautious_wd:
                decay = wd * lr * w * ((u * w) > 0).float()
            else:
                decay = wd * lr * w
            b.master[seg] = (w - decay - lr * scale * u).to(b.master.dtype)
