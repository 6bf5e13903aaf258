"""Speed-of-light model: transformer FLOPs per token and the fraction of the GPU's peak a run achieves.

Peak table: nominal dense tensor throughput per device (B200: bf16 2250, fp8 4500, fp4 9000 TFLOP/s) —
a measured peak (e.g. a cuBLAS bf16 burst) can be passed instead so fractions read "of measured".

Parity: csrc/src/utilities/sol.{h,cpp} (get_transformer_ops, estimate_speed_of_light; table :436-449).
"""
from __future__ import annotations

from typing import Dict, Optional

PEAK_TFLOPS = {
    "B200": {"bf16": 2250.0, "fp8": 4500.0, "fp4": 9000.0, "tf32": 1125.0},
    "B300": {"bf16": 2500.0, "fp8": 5000.0, "fp4": 15000.0, "tf32": 1250.0},
    "H100": {"bf16": 989.0, "fp8": 1979.0, "fp4": 1979.0, "tf32": 494.0},
    "H200": {"bf16": 989.0, "fp8": 1979.0, "fp4": 1979.0, "tf32": 494.0},
    "A100": {"bf16": 312.0, "fp8": 312.0, "fp4": 312.0, "tf32": 156.0},
    "RTX 5090": {"bf16": 209.5, "fp8": 419.0, "fp4": 838.0, "tf32": 104.8},
}


def transformer_flops_per_token(*, d_model: int, n_layers: int, n_q_heads: int, n_kv_heads: int, head_dim: int, d_ff: int, vocab: int,
                                seq_len: int, num_experts_per_tok: int = 0, moe_d_ff: int = 0, num_experts: int = 0,
                                lora_rank: int = 0, causal: bool = True, backward: bool = True, recompute: bool = False) -> Dict[str, float]:
    """Returns FLOPs per token split into matmul (by precision class) and attention."""
    qkv = 2 * d_model * (n_q_heads + 2 * n_kv_heads) * head_dim
    out = 2 * n_q_heads * head_dim * d_model
    if num_experts_per_tok:
        mlp = num_experts_per_tok * (2 * d_model * 2 * moe_d_ff + 2 * moe_d_ff * d_model) + 2 * d_model * num_experts
    else:
        mlp = 2 * d_model * 2 * d_ff + 2 * d_ff * d_model
    block = (qkv + out + mlp) * n_layers
    head = 2 * d_model * vocab
    attn = 4 * seq_len * n_q_heads * head_dim * n_layers * (0.5 if causal else 1.0)
    mult = (3.0 if backward else 1.0) + (1.0 if (recompute and backward) else 0.0)
    attn_mult = (3.5 if backward else 1.0) + (1.0 if (recompute and backward) else 0.0)
    if lora_rank and backward:  # frozen base weights: no wgrad for the base GEMMs
        mult -= 1.0
    return {"block_matmul": block * mult, "lm_head": head * (3.0 if backward else 1.0), "attention": attn * attn_mult,
            "total": block * mult + head * (3.0 if backward else 1.0) + attn * attn_mult}


def device_peak(name: str, precision: str) -> Optional[float]:
    for key, table in PEAK_TFLOPS.items():
        if key.lower() in name.lower():
            return table.get(precision)
    return None


def speed_of_light_fraction(flops: Dict[str, float], tokens_per_s: float, device_name: str, recipe: str, n_gpus: int = 1,
                            measured_bf16_tflops: Optional[float] = None) -> Optional[float]:
    """Achieved / ideal, where ideal runs block matmuls at the recipe's precision peak and the rest at bf16 peak."""
    prec = {"bf16": "bf16", "fp8_hybrid": "fp8", "nvfp4": "fp4"}.get(recipe.replace("-", "_"), "bf16")
    bf = measured_bf16_tflops or device_peak(device_name, "bf16")
    if not bf:
        return None
    nominal_bf = device_peak(device_name, "bf16") or bf
    pk = (device_peak(device_name, prec) or bf) * (bf / nominal_bf)
    ideal_s_per_token = flops["block_matmul"] / (pk * 1e12) + (flops["lm_head"] + flops["attention"]) / (bf * 1e12)
    return (tokens_per_s / n_gpus) * ideal_s_per_token
