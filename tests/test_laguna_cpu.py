"""Laguna has no transformers implementation to compare with here, so the oracle is a plain PyTorch restatement of the
architecture over checkpoint-named tensors: softplus-gated attention (full / sliding, per-kind rotary setup and head count),
dense or sigmoid-routed sparse feed-forward with a selection-only bias, routed scaling and an ungated shared expert."""
import json
import math
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F
from safetensors.torch import load_file, save_file

from surogate_b200.config.rope import rope_inv_freq
from surogate_b200.dsl.compiler import load_hf_config
from surogate_b200.runtime.trainer import Trainer, TrainerConfig

CFG = dict(architectures=["LagunaForCausalLM"], model_type="laguna", vocab_size=320, hidden_size=64, num_hidden_layers=4, num_attention_heads=4,
           num_key_value_heads=2, head_dim=16, intermediate_size=96, moe_intermediate_size=32, shared_expert_intermediate_size=48, num_experts=4,
           num_experts_per_tok=2, moe_routed_scaling_factor=2.5, gating=True, sliding_window=8, max_position_embeddings=256, rms_norm_eps=1e-6,
           layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"], mlp_layer_types=["dense", "sparse", "sparse", "sparse"],
           num_attention_heads_per_layer=[8, 4, 8, 4], tie_word_embeddings=False,
           rope_parameters={"full_attention": {"rope_type": "yarn", "rope_theta": 500000.0, "partial_rotary_factor": 0.5, "factor": 4.0,
                                               "original_max_position_embeddings": 64, "beta_fast": 32.0, "beta_slow": 1.0},
                            "sliding_attention": {"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 1.0}})


def random_state(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    C, D, Hkv, E = cfg["hidden_size"], cfg["head_dim"], cfg["num_key_value_heads"], cfg["num_experts"]

    def w(*shape, std=0.05):
        return torch.randn(*shape, generator=g) * std

    sd = {"model.embed_tokens.weight": w(cfg["vocab_size"], C, std=0.5), "model.norm.weight": 1 + w(C, std=0.1), "lm_head.weight": w(cfg["vocab_size"], C, std=0.1)}
    for L in range(cfg["num_hidden_layers"]):
        p, Hq = f"model.layers.{L}", cfg["num_attention_heads_per_layer"][L]
        sd.update({f"{p}.input_layernorm.weight": 1 + w(C, std=0.1), f"{p}.post_attention_layernorm.weight": 1 + w(C, std=0.1),
                   f"{p}.self_attn.q_proj.weight": w(Hq * D, C), f"{p}.self_attn.k_proj.weight": w(Hkv * D, C), f"{p}.self_attn.v_proj.weight": w(Hkv * D, C),
                   f"{p}.self_attn.g_proj.weight": w(Hq, C, std=0.3), f"{p}.self_attn.o_proj.weight": w(C, Hq * D),
                   f"{p}.self_attn.q_norm.weight": 1 + w(D, std=0.1), f"{p}.self_attn.k_norm.weight": 1 + w(D, std=0.1)})
        if cfg["mlp_layer_types"][L] == "dense":
            M = cfg["intermediate_size"]
            sd.update({f"{p}.mlp.gate_proj.weight": w(M, C), f"{p}.mlp.up_proj.weight": w(M, C), f"{p}.mlp.down_proj.weight": w(C, M)})
        else:
            M, S = cfg["moe_intermediate_size"], cfg["shared_expert_intermediate_size"]
            sd[f"{p}.mlp.gate.weight"] = w(E, C, std=0.3)
            sd[f"{p}.mlp.experts.e_score_correction_bias"] = w(E, std=0.2)
            for e in range(E):
                sd.update({f"{p}.mlp.experts.{e}.gate_proj.weight": w(M, C), f"{p}.mlp.experts.{e}.up_proj.weight": w(M, C), f"{p}.mlp.experts.{e}.down_proj.weight": w(C, M)})
            sd.update({f"{p}.mlp.shared_expert.gate_proj.weight": w(S, C), f"{p}.mlp.shared_expert.up_proj.weight": w(S, C), f"{p}.mlp.shared_expert.down_proj.weight": w(C, S)})
    return sd


def rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def oracle_logits(sd, cfg, tokens):
    B, T = tokens.shape
    C, D, Hkv, eps = cfg["hidden_size"], cfg["head_dim"], cfg["num_key_value_heads"], cfg["rms_norm_eps"]
    h = sd["model.embed_tokens.weight"][tokens]
    pos = torch.arange(T, dtype=torch.float32)
    i = torch.arange(T)
    for L in range(cfg["num_hidden_layers"]):
        p, Hq, kind = f"model.layers.{L}", cfg["num_attention_heads_per_layer"][L], cfg["layer_types"][L]
        rp = cfg["rope_parameters"][kind]
        R = int(D * rp["partial_rotary_factor"])
        inv, att_scale = rope_inv_freq(R, rp["rope_theta"], rp if rp["rope_type"] != "default" else None, cfg["max_position_embeddings"])
        ang = pos[:, None] * inv
        cos, sin = (ang.cos() * att_scale)[None, :, None], (ang.sin() * att_scale)[None, :, None]

        def rope(t):
            a, b, rest = t[..., :R // 2], t[..., R // 2:R], t[..., R:]
            return torch.cat([a * cos - b * sin, b * cos + a * sin, rest], -1)

        x = rms(h, sd[f"{p}.input_layernorm.weight"], eps)
        q = rope(rms(F.linear(x, sd[f"{p}.self_attn.q_proj.weight"]).view(B, T, Hq, D), sd[f"{p}.self_attn.q_norm.weight"], eps))
        k = rope(rms(F.linear(x, sd[f"{p}.self_attn.k_proj.weight"]).view(B, T, Hkv, D), sd[f"{p}.self_attn.k_norm.weight"], eps))
        v = F.linear(x, sd[f"{p}.self_attn.v_proj.weight"]).view(B, T, Hkv, D)
        G = Hq // Hkv
        s = q.permute(0, 2, 1, 3) @ k.permute(0, 2, 1, 3).repeat_interleave(G, 1).transpose(-1, -2) / math.sqrt(D)
        ok = i[:, None] >= i[None, :]
        if kind == "sliding_attention":
            ok = ok & ((i[:, None] - i[None, :]) < cfg["sliding_window"])
        o = (torch.softmax(s.masked_fill(~ok, float("-inf")), -1) @ v.permute(0, 2, 1, 3).repeat_interleave(G, 1)).permute(0, 2, 1, 3)
        gate = F.softplus(F.linear(x, sd[f"{p}.self_attn.g_proj.weight"]))  # one gate per head
        h = h + F.linear((o * gate[..., None]).reshape(B, T, Hq * D), sd[f"{p}.self_attn.o_proj.weight"])
        x = rms(h, sd[f"{p}.post_attention_layernorm.weight"], eps)

        def swiglu_mlp(t, pre):
            return F.linear(F.silu(F.linear(t, sd[f"{pre}.gate_proj.weight"])) * F.linear(t, sd[f"{pre}.up_proj.weight"]), sd[f"{pre}.down_proj.weight"])

        if cfg["mlp_layer_types"][L] == "dense":
            h = h + swiglu_mlp(x, f"{p}.mlp")
        else:
            x2 = x.reshape(-1, C)
            scores = torch.sigmoid(F.linear(x2, sd[f"{p}.mlp.gate.weight"]))
            idx = torch.topk(scores + sd[f"{p}.mlp.experts.e_score_correction_bias"], cfg["num_experts_per_tok"], -1).indices
            wts = scores.gather(1, idx)
            wts = wts / wts.sum(-1, keepdim=True) * cfg["moe_routed_scaling_factor"]
            y = torch.zeros_like(x2)
            for e in range(cfg["num_experts"]):
                tok, slot = torch.where(idx == e)
                if tok.numel():
                    y = y.index_add(0, tok, swiglu_mlp(x2[tok], f"{p}.mlp.experts.{e}") * wts[tok, slot, None])
            h = h + (y + swiglu_mlp(x2, f"{p}.mlp.shared_expert")).reshape(B, T, C)
    return F.linear(rms(h, sd["model.norm.weight"], eps), sd["lm_head.weight"])


def test_laguna_matches_plain_pytorch_oracle_and_round_trips(tmp_path):
    sd = random_state(CFG)
    src = os.path.join(tmp_path, "laguna")
    os.makedirs(src)
    save_file({k: v.contiguous() for k, v in sd.items()}, os.path.join(src, "model.safetensors"), metadata={"format": "pt"})
    with open(os.path.join(src, "config.json"), "w") as f:
        json.dump(CFG, f)
    tok = np.random.default_rng(0).integers(0, 320, (2, 24)).astype(np.int32)
    tr = Trainer(TrainerConfig(model=load_hf_config(src), batch_size=2, seq_len=24, zero_level=0), device=torch.device("cpu"))
    tr.import_weights(src)
    leaves = {k: v.clone().requires_grad_(True) for k, v in sd.items()}
    want = oracle_logits(leaves, CFG, torch.from_numpy(tok).long())
    got = tr.logits(tok)
    assert torch.allclose(got, want.detach(), atol=3e-4, rtol=1e-3), float((got - want).abs().max())
    tgt = np.roll(tok, -1, axis=1).astype(np.int32)
    tgt[:, -1] = -100
    r = tr.forward_backward(tok, tgt)
    loss = F.cross_entropy(want.reshape(-1, 320), torch.from_numpy(tgt).long().reshape(-1), ignore_index=-100)
    loss.backward()
    assert abs(float(r["loss_sum"] / r["n_valid"]) - float(loss)) < 1e-4
    want_norm = torch.sqrt(sum((v.grad ** 2).sum() for v in leaves.values() if v.grad is not None))
    assert abs(float(tr.grad_norm()) - float(want_norm)) < 2e-3 * float(want_norm)
    tr.store.release_grads()
    out = os.path.join(tmp_path, "export")
    tr.export_model(out, load_hf_config(src))
    back = load_file(os.path.join(out, "model.safetensors"))
    assert set(back) == set(sd)
    for k, v in sd.items():
        assert torch.allclose(back[k].float(), v, atol=1e-2, rtol=1e-2), k


def test_laguna_layer_structure_is_validated():
    from surogate_b200.dsl.models.laguna import layer_structure

    kinds, heads = layer_structure(3, ["full_attention", "sliding_attention", "full_attention"], None, [4, 8, 4], 4)
    assert kinds == ["full_dense", "sliding_sparse", "full_sparse"] and heads == {"full": 4, "sliding": 8}
    with pytest.raises(ValueError):
        layer_structure(3, ["full_attention"] * 3, None, [4, 8, 4], 4)  # head count differs within one attention kind
    with pytest.raises(ValueError):
        layer_structure(2, ["full_attention"], None, None, 4)
