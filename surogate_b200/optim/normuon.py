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


def polar_express_device(X: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """The same iteration on the tcgen05 GEMM, for a bf16 matrix already scaled to spectral norm < 1; returns a bf16 matrix of the
    same shape.  No transposed copies: a tall matrix [R, C] (R > C) iterates with A = X^T X ([C, C], both operands read MN-major)
    and X <- a X + X (bA + cA^2) (A is symmetric); a wide one with A = X X^T and X <- a X + (bA + cA^2) X."""
    from ..runtime.ops_cuda import gemm

    tall = X.shape[0] > X.shape[1]
    for a, b, c in POLAR_EXPRESS_COEFFS[:steps]:
        A = gemm(X, X, a_mn=True, b_mn=True) if tall else gemm(X, X)          # [m, m], m = min(R, C)
        B = A * b
        gemm(A, A, B, accumulate=True, alpha=c)                               # b A + c A A^T  (A = A^T)
        Xn = X * a
        if tall:
            gemm(X, B, Xn, accumulate=True)                                   # X B^T = X B
        else:
            gemm(B, X, Xn, b_mn=True, accumulate=True)                        # B X
        X = Xn
    return X


class NorMuon(AdamW8bit):
    def __init__(self, cfg: OptimizerConfig, store):
        super().__init__(cfg, store)
        self.mom: Dict[str, torch.Tensor] = {}
        self.mom_scales: Dict[str, torch.Tensor] = {}
        self.second: Dict[str, torch.Tensor] = {}
        self.momentum_8bit = bool(getattr(cfg, "normuon_momentum_8bit", False))

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
        if self.use_kernels and grad.dtype in (torch.bfloat16, torch.float32) and b.master.dtype in (torch.bfloat16, torch.float32):
            return self._step_matrices_device(b, grad, hp, before, matrices, lo, hi)
        lr, _, _, eps, wd, _, _ = hp_host
        mu, beta2 = self.cfg.normuon_momentum, self.cfg.normuon_beta2
        gs = hp[7]
        if float(gs) == 0.0:   # skipped update (non-finite gradient norm)
            b.master.copy_(before)
            return
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

    # ------------------------------------------------------------------ device path
    def _step_matrices_device(self, b, grad, hp, before, matrices, lo, hi) -> None:
        """Matrix parameters on the GPU: momentum / Nesterov blend / Frobenius norm (one kernel), normalisation (one kernel), five
        Polar-Express iterations on the tcgen05 GEMM, row statistics (one kernel) and the update with cautious weight decay (one kernel).
        Momentum is kept in bf16 (or, with ``normuon_momentum_8bit``, as int8 codes with an fp16 scale per 128 values), the row second moments in fp32; hyper-parameters and the clip scale are read from the device vector, so
        nothing here synchronises with the host.  A matrix that straddles a shard boundary is orthogonalised by every rank that owns a
        part of it (from the gathered gradient) and each rank applies its own slice."""
        store, ext = self.store, self.ext
        mu, beta2 = float(self.cfg.normuon_momentum), float(self.cfg.normuon_beta2)
        for s in matrices:
            a, z = s.offset, s.offset + s.numel
            pa, pz = max(a, lo), min(z, hi)
            if store.sharded and not (a >= lo and z <= hi):
                g_full = store.grad_of(s.name).reshape(-1).contiguous()       # collective: every rank takes part
            else:
                g_full = grad[a - lo:z - lo].contiguous()
            if pa >= pz:
                continue
            if g_full.dtype not in (torch.bfloat16, torch.float32):
                g_full = g_full.float()
            if self.momentum_8bit and s.numel % 128 == 0:     # int8 codes + one fp16 scale per 128 values (1.02 bytes per parameter)
                m = self.mom.get(s.name)
                if m is None or m.dtype != torch.int8:
                    m = self.mom[s.name] = torch.zeros(s.numel, dtype=torch.int8, device=store.device)
                    self.mom_scales[s.name] = torch.zeros(s.numel // 128, dtype=torch.float16, device=store.device)
                u, sumsq = ext.normuon_momentum8(g_full, m, self.mom_scales[s.name], hp, mu)
            else:
                m = self.mom.get(s.name)
                if m is None or m.dtype != torch.bfloat16:
                    m = self.mom[s.name] = torch.zeros(s.numel, dtype=torch.bfloat16, device=store.device)
                u, sumsq = ext.normuon_momentum(g_full, m.view(-1), hp, mu)
            ext.normuon_normalise(u, sumsq)
            X = polar_express_device(u.view(s.shape))
            v = self.second.get(s.name)
            if v is None or v.numel() != s.shape[0]:
                v = self.second[s.name] = torch.zeros(s.shape[0], dtype=torch.float32, device=store.device)
            sums = ext.normuon_row_stats(X.contiguous(), v.view(-1), hp, beta2)
            seg = slice(pa - lo, pz - lo)
            w = before[seg].clone()          # the AdamW pass above also touched these elements: start again from the old values
            scale = 0.2 * max(s.shape[0], s.shape[1]) ** 0.5 * self.cfg.normuon_lr_scale
            ext.normuon_apply(w, X.contiguous(), v.view(-1), sums, hp, float(scale), bool(self.cfg.normuon_cautious_wd), pa - a)
            b.master[seg] = w

