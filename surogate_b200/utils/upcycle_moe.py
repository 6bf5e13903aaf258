"""Dense -> mixture-of-experts "upcycling" of a HuggingFace checkpoint (Qwen3 -> Qwen3-MoE layout).

Every expert of every layer starts as a copy of that layer's dense MLP (optionally a contiguous slice of its intermediate
dimension when ``expert_d_ff`` is smaller, plus small noise so experts can diverge); routers start near zero so routing is
uniform.  ``python -m surogate_b200.utils.upcycle_moe --src dense_dir --dst moe_dir --experts 8 --top-k 2``.

Parity: scripts/upcycle_moe.py.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
from typing import Dict, Optional

import torch
from safetensors import safe_open
from safetensors.torch import save_file


def upcycle(src: str, dst: str, num_experts: int, top_k: int, expert_d_ff: Optional[int] = None, noise: float = 0.0, router_std: float = 0.02, seed: int = 0) -> Dict:
    with open(os.path.join(src, "config.json")) as f:
        cfg = json.load(f)
    d_ff = cfg["intermediate_size"]
    m = expert_d_ff or d_ff
    if m > d_ff:
        raise ValueError("expert_d_ff cannot exceed the dense intermediate_size")
    gen = torch.Generator().manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    files = [f for f in sorted(os.listdir(src)) if f.endswith(".safetensors")]
    for fn in files:
        with safe_open(os.path.join(src, fn), framework="pt") as f:
            for k in f.keys():
                t = f.get_tensor(k)
                if ".mlp." not in k:
                    out[k] = t
                    continue
                layer_prefix, leaf = k.split(".mlp.")
                proj = leaf.split(".")[0]  # gate_proj | up_proj | down_proj
                for e in range(num_experts):
                    lo = (e * m) % max(1, d_ff - m + 1) if m < d_ff else 0
                    w = t[lo:lo + m] if proj in ("gate_proj", "up_proj") else t[:, lo:lo + m]
                    if noise:
                        w = w + noise * w.float().std() * torch.randn(w.shape, generator=gen).to(w.dtype)
                    out[f"{layer_prefix}.mlp.experts.{e}.{proj}.weight"] = w.contiguous().clone()
                gate = f"{layer_prefix}.mlp.gate.weight"
                if gate not in out:
                    out[gate] = (torch.randn(num_experts, cfg["hidden_size"], generator=gen) * router_std).to(t.dtype)
    os.makedirs(dst, exist_ok=True)
    save_file(out, os.path.join(dst, "model.safetensors"), metadata={"format": "pt"})
    moe_cfg = dict(cfg, architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe", num_experts=num_experts, num_experts_per_tok=top_k,
                   moe_intermediate_size=m, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[], router_aux_loss_coef=1e-3)
    with open(os.path.join(dst, "config.json"), "w") as f:
        json.dump(moe_cfg, f, indent=1)
    for fn in os.listdir(src):
        if fn.startswith("tokenizer") or fn in ("generation_config.json", "chat_template.jinja", "vocab.json", "merges.txt", "special_tokens_map.json"):
            shutil.copy2(os.path.join(src, fn), os.path.join(dst, fn))
    return {"tensors": len(out), "experts": num_experts, "expert_d_ff": m}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m surogate_b200.utils.upcycle_moe")
    p.add_argument("--src", required=True)
    p.add_argument("--dst", required=True)
    p.add_argument("--experts", type=int, required=True)
    p.add_argument("--top-k", type=int, default=2)
    p.add_argument("--expert-d-ff", type=int, default=None)
    p.add_argument("--noise", type=float, default=0.0)
    a = p.parse_args(argv)
    print(json.dumps(upcycle(a.src, a.dst, a.experts, a.top_k, a.expert_d_ff, a.noise)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
