"""Health check of a mixture-of-experts checkpoint: have the experts diverged from each other, does the router have opinions?

    python -m surogate_b200.utils.expert_divergence --model moe_dir [--layer 17] [--tokens 512]

1. Expert weights: mean pairwise cosine similarity of the experts' projections in one layer.  Freshly upcycled experts are clones
   (similarity 1.0000); below 0.9990 they have started to diverge and the router has something to learn from; below 0.990 they
   specialise.
2. Router: rows of the router matrix compared with each other, and (with ``--tokens``) the router run on embedded random tokens:
   mean top-1 probability against the 1/E of random routing, and the share of experts that win a token.

The checkpoint is read tensor by tensor from its safetensors files (HuggingFace names ``...mlp.experts.<e>.<proj>.weight`` and
``...mlp.gate.weight``); no model is built.

Parity: scripts/check_expert_divergence.py.
"""
from __future__ import annotations

import argparse
import json
import re
from typing import Any, Dict, List, Optional

import torch

from ..io.hf_checkpoint import LazyCheckpoint

EXPERT_RE = re.compile(r"(.*\.layers\.(\d+)\.mlp)\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")


def _pairwise_cosine(rows: torch.Tensor) -> Dict[str, float]:
    x = torch.nn.functional.normalize(rows.float().flatten(1), dim=1)
    sim = x @ x.t()
    n = sim.shape[0]
    off = sim[~torch.eye(n, dtype=torch.bool)]
    return {"mean": float(off.mean()) if n > 1 else 1.0, "min": float(off.min()) if n > 1 else 1.0, "max": float(off.max()) if n > 1 else 1.0}


def verdict(similarity: float) -> str:
    if similarity > 0.9999:
        return "clones: the router has no signal yet"
    if similarity > 0.9990:
        return "barely diverged"
    if similarity > 0.990:
        return "diverging: the router can start to learn"
    return "specialised"


def expert_divergence(model_dir: str, layer: Optional[int] = None, tokens: int = 0, seed: int = 0) -> Dict[str, Any]:
    ck = LazyCheckpoint(model_dir)
    layers: Dict[int, Dict[str, Dict[int, str]]] = {}
    prefix: Dict[int, str] = {}
    for name in ck.names():
        m = EXPERT_RE.match(name)
        if m:
            L = int(m.group(2))
            layers.setdefault(L, {}).setdefault(m.group(4), {})[int(m.group(3))] = name
            prefix[L] = m.group(1)
    if not layers:
        raise ValueError(f"{model_dir} has no `mlp.experts.<e>.<proj>.weight` tensors: not a mixture-of-experts checkpoint in the HuggingFace layout")
    L = sorted(layers)[len(layers) // 2] if layer is None else layer
    if L not in layers:
        raise ValueError(f"layer {L} has no experts (layers with experts: {sorted(layers)[:4]} ... {sorted(layers)[-1]})")
    out: Dict[str, Any] = {"layer": L, "num_experts": len(next(iter(layers[L].values()))), "projections": {}}
    sims: List[float] = []
    for proj, by_e in sorted(layers[L].items()):
        stack = torch.stack([ck.get(by_e[e]) for e in sorted(by_e)])
        s = _pairwise_cosine(stack)
        out["projections"][proj] = s
        sims.append(s["mean"])
    out["expert_similarity"] = sum(sims) / len(sims)
    out["experts"] = verdict(out["expert_similarity"])
    gate_name = prefix[L] + ".gate.weight"
    if gate_name in ck:
        W = ck.get(gate_name).float()                     # [E, d]
        out["router_row_similarity"] = _pairwise_cosine(W)["mean"]
        if tokens > 0:
            embed = next((n for n in ("model.embed_tokens.weight", "model.language_model.embed_tokens.weight") if n in ck), None)
            g = torch.Generator().manual_seed(seed)
            if embed is not None:
                E = ck.get(embed)
                x = E[torch.randint(0, E.shape[0], (tokens,), generator=g)].float()
            else:
                x = torch.randn(tokens, W.shape[1], generator=g)
            x = x / x.pow(2).mean(-1, keepdim=True).add(1e-6).sqrt()       # what the pre-MLP norm hands the router, up to its gain
            p = torch.softmax(x @ W.t(), -1)
            top = p.max(-1)
            n_e = W.shape[0]
            out["router"] = {"mean_top1_probability": float(top.values.mean()), "random_level": 1.0 / n_e,
                             "experts_winning_a_token": float(top.indices.unique().numel()) / n_e,
                             "confidence": "strong" if top.values.mean() > 0.30 else "emerging" if top.values.mean() > max(0.15, 1.5 / n_e) else "close to random"}
    return out


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m surogate_b200.utils.expert_divergence")
    p.add_argument("--model", required=True)
    p.add_argument("--layer", type=int, default=None, help="default: the middle layer that has experts")
    p.add_argument("--tokens", type=int, default=512, help="random tokens to run through the router (0 = skip)")
    a = p.parse_args(argv)
    print(json.dumps(expert_divergence(a.model, a.layer, a.tokens), indent=1))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
