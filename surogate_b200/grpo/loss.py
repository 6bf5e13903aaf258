"""GRPO / PPO-clip token objective, its torch reference, and its gradient as per-token weights for the fused loss kernel.

Per completion token t with advantage A_t, behaviour log-prob l_old (from the rollout engine), current log-prob l and
reference log-prob l_ref:

    r = exp(l - l_old)
    policy term   J_t = min(r A, clip(r, 1 - eps_lo, 1 + eps_hi) A)            (maximised)
    KL term       k3_t = exp(l_ref - l) - (l_ref - l) - 1                       (minimised, weight kl_coef)
    loss          L = sum_t m_t (-J_t + kl_coef k3_t) / Z

with m_t the completion mask (tokens whose ratio exceeds ``ratio_cap`` are masked out as too off-policy) and Z either the
number of masked tokens (token normalisation) or per-sequence lengths averaged over sequences.

dL/dl = m_t / Z * ( -A r [unclipped] + kl_coef (1 - exp(l_ref - l)) ), and since l_t = -CE_t the kernel weight on the CE
gradient of token t is -dL/dl.

Parity: surogate/grpo/loss.py (numpy reference), csrc/src/kernels/fused_classifier.cu (grpo_custom_dloss_kernel).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch


def _normaliser(mask: torch.Tensor, seq_ids: Optional[torch.Tensor], mode: str) -> torch.Tensor:
    """Per-token 1/Z.  ``seq_ids`` ([rows, T] int, -1 outside sequences) identifies packed sequences for sequence mode."""
    m = mask.float()
    if mode == "token" or seq_ids is None:
        return m / m.sum().clamp_min(1.0)
    flat = seq_ids.reshape(-1).long()
    valid = (flat >= 0) & (mask.reshape(-1) > 0)
    n_seq = int(flat.max().item()) + 1 if valid.any() else 1
    counts = torch.zeros(n_seq, dtype=torch.float32, device=mask.device).index_add_(0, flat[valid], torch.ones_like(flat[valid], dtype=torch.float32))
    present = (counts > 0).float().sum().clamp_min(1.0)
    per_tok = torch.zeros_like(m).reshape(-1)
    per_tok[valid] = 1.0 / (counts[flat[valid]] * present)
    return per_tok.reshape(mask.shape)


def grpo_loss_reference(logp: torch.Tensor, old_logp: torch.Tensor, advantages: torch.Tensor, mask: torch.Tensor, ref_logp: Optional[torch.Tensor] = None,
                        clip_eps_low: float = 0.2, clip_eps_high: float = 0.2, kl_coef: float = 0.0, ratio_cap: float = 10.0,
                        normalization: str = "token", seq_ids: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    """Differentiable torch version (the oracle for ``grpo_token_weights``)."""
    ratio = torch.exp(logp - old_logp)
    m = mask.float() * (ratio.detach() <= ratio_cap).float()
    clipped = torch.clamp(ratio, 1 - clip_eps_low, 1 + clip_eps_high)
    j = torch.minimum(ratio * advantages, clipped * advantages)
    per_tok = -j
    kl = torch.zeros_like(logp)
    if ref_logp is not None and kl_coef:
        d = ref_logp - logp
        kl = torch.exp(d) - d - 1
        per_tok = per_tok + kl_coef * kl
    z = _normaliser(m, seq_ids, normalization)
    loss = (per_tok * z).sum()
    with torch.no_grad():
        msum = m.sum().clamp_min(1.0)
        metrics = {"ratio_mean": (ratio * m).sum() / msum, "clip_frac": (((ratio * advantages) > (clipped * advantages)).float() * m).sum() / msum,
                   "kl": (kl * m).sum() / msum, "masked_by_cap": (mask.float() - m).sum()}
    return loss, metrics


@torch.no_grad()
def grpo_token_weights(logp: torch.Tensor, old_logp: torch.Tensor, advantages: torch.Tensor, mask: torch.Tensor, ref_logp: Optional[torch.Tensor] = None,
                       clip_eps_low: float = 0.2, clip_eps_high: float = 0.2, kl_coef: float = 0.0, ratio_cap: float = 10.0,
                       normalization: str = "token", seq_ids: Optional[torch.Tensor] = None):
    """(loss, per-token CE weights, metrics) — the weights multiply each token's log-likelihood (= -CE) gradient."""
    ratio = torch.exp(logp - old_logp)
    m = mask.float() * (ratio <= ratio_cap).float()
    ra, ca = ratio * advantages, torch.clamp(ratio, 1 - clip_eps_low, 1 + clip_eps_high) * advantages
    unclipped = (ra <= ca).float()  # min picks the ratio branch: gradient flows
    dl = -advantages * ratio * unclipped
    per_tok = -torch.minimum(ra, ca)
    kl = torch.zeros_like(logp)
    if ref_logp is not None and kl_coef:
        d = ref_logp - logp
        kl = torch.exp(d) - d - 1
        per_tok = per_tok + kl_coef * kl
        dl = dl + kl_coef * (1 - torch.exp(d))
    z = _normaliser(m, seq_ids, normalization)
    loss = (per_tok * z).sum()
    weights = -(dl * z)  # l = -CE  =>  dL/dCE = -dL/dl ; the kernel scales dCE by this
    msum = m.sum().clamp_min(1.0)
    metrics = {"ratio_mean": (ratio * m).sum() / msum, "clip_frac": ((1 - unclipped) * m).sum() / msum, "kl": (kl * m).sum() / msum,
               "masked_by_cap": (mask.float() - m).sum()}
    return loss, weights, metrics


def group_advantages(rewards: torch.Tensor, group_size: int, std_eps: float = 1e-6, clip: float = 0.0) -> torch.Tensor:
    """rewards [prompts * group_size] -> advantages: reward minus the group mean, divided by the group std."""
    r = rewards.reshape(-1, group_size).float()
    adv = (r - r.mean(1, keepdim=True)) / (r.std(1, keepdim=True, unbiased=False) + std_eps)
    if clip:
        adv = adv.clamp(-clip, clip)
    return adv.reshape(-1)
