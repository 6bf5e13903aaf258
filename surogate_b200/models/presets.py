"""Architecture presets: the ``config.json`` of well-known models by name, for runs that need the shape but not the weights
(pre-training from scratch, benchmarks, memory planning) on machines without hub access.

``model: preset:qwen3-8b`` in a config, ``PretrainedConfig.from_name("qwen3-8b")`` in the Python API, ``surogate info preset:...``.
Names are matched case-insensitively, with or without the organisation prefix (``Qwen/Qwen3-8B``).  Values are the published
configurations of the models.

Parity: csrc/src/config/pretrained_config.cpp (``from_name`` presets).
"""
from __future__ import annotations

from typing import Any, Dict, List


def _qwen3(hidden: int, layers: int, heads: int, kv: int, ffn: int, tie: bool, max_pos: int = 40960) -> Dict[str, Any]:
    return dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
                num_key_value_heads=kv, head_dim=128, intermediate_size=ffn, rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=max_pos,
                tie_word_embeddings=tie, attention_bias=False, hidden_act="silu", bos_token_id=151643, eos_token_id=151645, torch_dtype="bfloat16")


def _qwen25(hidden: int, layers: int, heads: int, kv: int, ffn: int, tie: bool, vocab: int = 152064) -> Dict[str, Any]:
    return dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=vocab, hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
                num_key_value_heads=kv, intermediate_size=ffn, rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=32768, tie_word_embeddings=tie,
                hidden_act="silu", bos_token_id=151643, eos_token_id=151645, torch_dtype="bfloat16")


def _llama3(hidden: int, layers: int, heads: int, kv: int, ffn: int, tie: bool = False, scaling: bool = True) -> Dict[str, Any]:
    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=128256, hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
               num_key_value_heads=kv, intermediate_size=ffn, rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=131072 if scaling else 8192,
               tie_word_embeddings=tie, attention_bias=False, hidden_act="silu", bos_token_id=128000, eos_token_id=128001, torch_dtype="bfloat16")
    if scaling:
        cfg["rope_scaling"] = dict(rope_type="llama3", factor=32.0 if tie else 8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192)
    return cfg


PRESETS: Dict[str, Dict[str, Any]] = {
    "qwen3-0.6b": _qwen3(1024, 28, 16, 8, 3072, True),
    "qwen3-1.7b": _qwen3(2048, 28, 16, 8, 6144, True),
    "qwen3-4b": _qwen3(2560, 36, 32, 8, 9728, True),
    "qwen3-8b": _qwen3(4096, 36, 32, 8, 12288, False),
    "qwen3-14b": _qwen3(5120, 40, 40, 8, 17408, False),
    "qwen3-32b": _qwen3(5120, 64, 64, 8, 25600, False),
    "qwen3-30b-a3b": dict(_qwen3(2048, 48, 32, 4, 6144, False), architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe", moe_intermediate_size=768, num_experts=128,
                          num_experts_per_tok=8, norm_topk_prob=True, router_aux_loss_coef=0.001, decoder_sparse_step=1, mlp_only_layers=[]),
    "qwen3-235b-a22b": dict(_qwen3(4096, 94, 64, 4, 12288, False), architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe", moe_intermediate_size=1536, num_experts=128,
                            num_experts_per_tok=8, norm_topk_prob=True, router_aux_loss_coef=0.001, decoder_sparse_step=1, mlp_only_layers=[]),
    "qwen2.5-0.5b": _qwen25(896, 24, 14, 2, 4864, True, 151936),
    "qwen2.5-1.5b": _qwen25(1536, 28, 12, 2, 8960, True, 151936),
    "qwen2.5-3b": _qwen25(2048, 36, 16, 2, 11008, True, 151936),
    "qwen2.5-7b": _qwen25(3584, 28, 28, 4, 18944, False),
    "qwen2.5-14b": _qwen25(5120, 48, 40, 8, 13824, False),
    "qwen2.5-32b": _qwen25(5120, 64, 40, 8, 27648, False),
    "qwen2.5-72b": _qwen25(8192, 80, 64, 8, 29568, False),
    "llama-3.2-1b": _llama3(2048, 16, 32, 8, 8192, tie=True),
    "llama-3.2-3b": _llama3(3072, 28, 24, 8, 8192, tie=True),
    "llama-3.1-8b": _llama3(4096, 32, 32, 8, 14336),
    "llama-3.1-70b": _llama3(8192, 80, 64, 8, 28672),
    "llama-3-8b": _llama3(4096, 32, 32, 8, 14336, scaling=False),
    "mistral-7b-v0.3": dict(architectures=["MistralForCausalLM"], model_type="mistral", vocab_size=32768, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32,
                            num_key_value_heads=8, intermediate_size=14336, rms_norm_eps=1e-5, rope_theta=1000000.0, max_position_embeddings=32768, sliding_window=None,
                            tie_word_embeddings=False, hidden_act="silu", bos_token_id=1, eos_token_id=2, torch_dtype="bfloat16"),
}
for _k in ("llama-3.2-1b", "llama-3.2-3b"):
    PRESETS[_k]["head_dim"] = PRESETS[_k]["hidden_size"] // PRESETS[_k]["num_attention_heads"] if _k != "llama-3.2-3b" else 128
PRESETS["llama-3.2-1b"]["head_dim"] = 64

PREFIX = "preset:"


def normalise(name: str) -> str:
    n = name[len(PREFIX):] if name.lower().startswith(PREFIX) else name
    n = n.rsplit("/", 1)[-1].lower().replace("_", "-")
    for suffix in ("-instruct", "-base", "-chat", "-it"):
        if n.endswith(suffix):
            n = n[:-len(suffix)]
    if n.startswith("meta-llama-"):
        n = n[len("meta-"):]
    return n


def list_presets() -> List[str]:
    return sorted(PRESETS)


def is_preset(name: Any) -> bool:
    return isinstance(name, str) and name.lower().startswith(PREFIX)


def preset_config(name: str) -> Dict[str, Any]:
    """A copy of the preset's ``config.json`` dictionary; raises ``KeyError`` listing the known names."""
    key = normalise(name)
    if key not in PRESETS:
        raise KeyError(f"no architecture preset '{name}' (known: {', '.join(list_presets())})")
    import copy

    return copy.deepcopy(PRESETS[key])
