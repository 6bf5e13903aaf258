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

A second objective, ``type: ipo`` (probability-difference masking with a squared log-ratio penalty):

    keep_t   = m_t and not (p - p_old > mask_high or p - p_old < -mask_low)      with p = exp(l), p_old = exp(l_old)
    A'_t     = adv_tau A_t + teacher_tau (l_teacher - l)                           (the teacher term is detached)
    loss     L = sum_t ( -keep_t A'_t r_t + kl_tau m_t (l - l_old)^2 ) / Z,       Z = number of completion tokens
    dL/dl    = ( -keep_t A'_t min(r_t, ratio_clip) + 2 kl_tau m_t (l - l_old) ) / Z

i.e. a token whose probability moved further than the mask thresholds since the rollout stops contributing to the policy term
(but still feels the penalty that pulls it back), and the ratio that multiplies the gradient is capped at ``ratio_clip``.

Parity: surogate/grpo/loss.py (numpy reference; its objective is the ``ipo`` one), csrc/src/kernels/fused_classifier.cu
(grpo_custom_dloss_kernel).
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


def ipo_loss_reference(logp: torch.Tensor, old_logp: torch.Tensor, advantages: torch.Tensor, mask: torch.Tensor, teacher_logp: Optional[torch.Tensor] = None,
                       ipo_mask_low: float = 0.2, ipo_mask_high: float = 0.2, adv_tau: float = 1.0, teacher_tau: float = 0.0, kl_tau: float = 1e-3,
                       ratio_clip: float = 7.389056, normalization: str = "token", seq_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Differentiable surrogate whose gradient with respect to ``logp`` is the ``ipo`` gradient (the oracle of ``ipo_token_weights``):
    mask, advantage, teacher term and the capped ratio are detached, as they are in the objective's definition."""
    with torch.no_grad():
        ratio = torch.exp(logp - old_logp)
        pdiff = torch.exp(logp) - torch.exp(old_logp)
        keep = mask.bool() & ~((pdiff > ipo_mask_high) | (pdiff < -ipo_mask_low))
        adv = adv_tau * advantages + (teacher_tau * (teacher_logp - logp) if teacher_logp is not None else 0.0)
        coef = keep.float() * adv * ratio.clamp(max=ratio_clip)
        z = _normaliser(mask.float(), seq_ids, normalization)
    return ((-coef * logp + kl_tau * mask.float() * (logp - old_logp) ** 2) * z).sum()


@torch.no_grad()
def ipo_token_weights(logp: torch.Tensor, old_logp: torch.Tensor, advantages: torch.Tensor, mask: torch.Tensor, teacher_logp: Optional[torch.Tensor] = None,
                      ipo_mask_low: float = 0.2, ipo_mask_high: float = 0.2, adv_tau: float = 1.0, teacher_tau: float = 0.0, kl_tau: float = 1e-3,
                      ratio_clip: float = 7.389056, normalization: str = "token", seq_ids: Optional[torch.Tensor] = None):
    """(loss, per-token CE weights, metrics) of the ``ipo`` objective; same contract as ``grpo_token_weights``."""
    m = mask.float()
    log_ratio = logp - old_logp
    ratio = torch.exp(log_ratio)
    pdiff = torch.exp(logp) - torch.exp(old_logp)
    high, low = pdiff > ipo_mask_high, pdiff < -ipo_mask_low
    masked = high | low
    keep = m * (~masked).float()
    adv = adv_tau * advantages
    if teacher_logp is not None:
        adv = adv + teacher_tau * (teacher_logp - logp)
    z = _normaliser(m, seq_ids, normalization)
    per_tok = -keep * adv * ratio + kl_tau * m * log_ratio ** 2
    dl = -keep * adv * ratio.clamp(max=ratio_clip) + 2.0 * kl_tau * m * log_ratio
    loss = (per_tok * z).sum()
    weights = -(dl * z)
    msum, ksum = m.sum().clamp_min(1.0), keep.sum().clamp_min(1.0)
    mismatch = ratio - log_ratio - 1.0
    metrics = {"ratio_mean": (ratio * m).sum() / msum, "mismatch_kl": (mismatch * m).sum() / msum, "unmasked_mismatch_kl": (mismatch * keep).sum() / ksum,
               "is_masked": (masked.float() * m).sum() / msum, "is_masked_low": (low.float() * m).sum() / msum, "is_masked_high": (high.float() * m).sum() / msum,
               "keep_tokens": keep.sum(), "ratio_clipped": ((ratio > ratio_clip).float() * keep).sum() / ksum, "kl": (log_ratio ** 2 * m).sum() / msum}
    if teacher_logp is not None:
        metrics["teacher_kl"] = ((teacher_logp - logp) * m).sum() / msum
    return loss, weights, metrics


def group_advantages(rewards: torch.Tensor, group_size: int, std_eps: float = 1e-6, clip: float = 0.0) -> torch.Tensor:
    """rewards [prompts * group_size] -> advantages: reward minus the group mean, divided by the group std."""
    r = rewards.reshape(-1, group_size).float()
    adv = (r - r.mean(1, keepdim=True)) / (r.std(1, keepdim=True, unbiased=False) + std_eps)
    if clip:
        adv = adv.clamp(-clip, clip)
    return adv.reshape(-1)
