"""DPO objective on sequence log-probabilities, and its gradient expressed as per-sequence weights.

With ``pi = logp_policy(chosen) - logp_policy(rejected)`` and ``ref`` the same difference under the reference policy,
``h = beta * (pi - ref)``:

* sigmoid:  L = -(1-eps) log sigmoid(h) - eps log sigmoid(-h)      dL/dh = -(1-eps) sigmoid(-h) + eps sigmoid(h)
* ipo:      L = (pi - ref - 1/(2 beta))^2                           dL/d(pi) = 2 (pi - ref - 1/(2 beta))
* hinge:    L = relu(1 - h)                                         dL/dh = -1[h < 1]

Since logp(sequence) = -sum_t CE_t, the gradient of L is the ordinary cross-entropy gradient of every chosen token scaled
by ``-dL/d logp_chosen`` and of every rejected token by ``-dL/d logp_rejected`` — which is what the fused LM-head loss
kernel's per-token weights implement.

Parity: csrc/src/kernels/fused_classifier.cu (dpo_custom_dloss_kernel), surogate/dpo/trainer.py.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.nn.functional as F


def dpo_loss_and_weights(pol_c: torch.Tensor, pol_r: torch.Tensor, ref_c: torch.Tensor, ref_r: torch.Tensor, beta: float,
                         label_smoothing: float = 0.0, loss_type: str = "sigmoid") -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, Dict[str, torch.Tensor]]:
    """All inputs are [pairs] sequence log-probabilities.  Returns (mean loss, CE weight for chosen sequences, CE weight for
    rejected sequences, metrics).  The weights already include the 1/pairs of the mean."""
    n = pol_c.numel()
    pi, ref = pol_c - pol_r, ref_c - ref_r
    h = beta * (pi - ref)
    if loss_type == "sigmoid":
        loss = -(1 - label_smoothing) * F.logsigmoid(h) - label_smoothing * F.logsigmoid(-h)
        dh = -(1 - label_smoothing) * torch.sigmoid(-h) + label_smoothing * torch.sigmoid(h)
        dpi = dh * beta
    elif loss_type == "ipo":
        d = pi - ref - 1.0 / (2 * beta)
        loss = d * d
        dpi = 2 * d
    elif loss_type == "hinge":
        loss = torch.relu(1 - h)
        dpi = -(h < 1).float() * beta
    else:
        raise ValueError(loss_type)
    # dL/dlogp_chosen = dpi, dL/dlogp_rejected = -dpi; logp = -sum CE  =>  weight on the CE gradient = -dL/dlogp
    w_c = -dpi / n
    w_r = dpi / n
    metrics = {"rewards/chosen": (beta * (pol_c - ref_c)).mean(), "rewards/rejected": (beta * (pol_r - ref_r)).mean(),
               "rewards/accuracy": (h > 0).float().mean(), "rewards/margin": h.mean(), "logps/chosen": pol_c.mean(), "logps/rejected": pol_r.mean()}
    return loss.mean(), w_c, w_r, metrics
