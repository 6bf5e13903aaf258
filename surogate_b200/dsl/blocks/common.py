"""Canonical parameter / activation names shared by every architecture.

Module-qualified names produced while tracing (``self_attn.qkv_weight``) are
rewritten to the flat canonical names used by checkpoints, debug dumps and
tests (``qkv_weight``, ``ln1``, ``res_att`` ...).

Parity: surogate/dsl/blocks/common.py:12-111.
"""

DENSE_BLOCK_NAME_REMAP = {
    "attn_norm.weight": "ln1_weight",
    "attn_norm.ln": "ln1",
    "attn_norm.ln_rstd": "ln1_rstd",
    "attn_norm.res": "res_ffn",
    "mlp_norm.weight": "ln2_weight",
    "mlp_norm.ln": "ln2",
    "mlp_norm.ln_rstd": "ln2_rstd",
    "mlp_norm.res": "res_att",
    "self_attn.*": "",
    "mlp.up_weight": "mlp_up_weight",
    "mlp.down_weight": "mlp_down_weight",
    "mlp.*": "",
}

MOE_BLOCK_NAME_REMAP = {
    **{k: v for k, v in DENSE_BLOCK_NAME_REMAP.items() if not k.startswith("mlp.")},
    "mlp.*": "",
    "shared_expert.up_weight": "shared_expert_up_weight",
    "shared_expert.down_weight": "shared_expert_down_weight",
    "shared_expert.*": "",
}

STANDARD_MODEL_NAME_REMAP = {
    "embedding.weight": "embedding",
    "embedding.x0": "x0",
    "final_norm.weight": "final_norm",
    "final_norm.ln": "xF",
    "final_norm.ln_rstd": "ln_final_rstd",
    "final_norm.res": "residual_final",
    "lm_head.weight": "lm_head",
    "lm_head.loss": "loss",
    "blocks.*": "",
}
