"""Qwen3-VL (``Qwen3VLForConditionalGeneration``): the text decoder is trained; the vision tower runs frozen outside the graph
and its outputs enter as per-batch side inputs (``visual_pos_masks``, ``visual_embeds``, ``deepstack_visual_embeds``,
``mrope_position_ids``) set with ``Trainer.set_visual_inputs``.  Text-only batches need none of them.

Parity: surogate/dsl/models/qwen3_vl.py.
"""
from __future__ import annotations

from .. import functional as F
from .. import nn
from ..blocks import STANDARD_MODEL_NAME_REMAP
from ..blocks.qwen3_vl import Qwen3VLBlock
from ..modules import Embedding, LMHead, RMSNorm


@nn.hf_config(architecture="Qwen3VLForConditionalGeneration", model_type="qwen3_vl", d_model="text_config.hidden_size", n_layers="text_config.num_hidden_layers",
              num_query_heads="text_config.num_attention_heads", num_kv_heads="text_config.num_key_value_heads", d_ff="text_config.intermediate_size",
              vocab_size="text_config.vocab_size", max_seq="text_config.max_position_embeddings", head_size="text_config.head_dim",
              eps="text_config.rms_norm_eps", use_qkv_bias="text_config.attention_bias", rope_parameters="text_config.rope_parameters",
              rope_scaling="text_config.rope_scaling", rope_theta="text_config.rope_theta", deepstack_visual_indexes="vision_config.deepstack_visual_indexes",
              tie_word_embeddings="tie_word_embeddings", text_tie="text_config.tie_word_embeddings")
class Qwen3VLModel(nn.Model):
    _name_remap_ = STANDARD_MODEL_NAME_REMAP

    def __init__(self, vocab_size: int = 151936, d_model: int = 4096, n_layers: int = 36, num_query_heads: int = 32, num_kv_heads: int = 8, d_ff: int = 12288,
                 max_seq: int = 262144, head_size: int = 128, eps: float = 1e-6, use_qkv_bias: bool = False, rope_parameters=None, rope_scaling=None,
                 rope_theta: float = 5e6, deepstack_visual_indexes=None, tie_word_embeddings: bool = False, text_tie: bool = False):
        super().__init__()
        self.vocab_size, self.d_model, self.n_layers = vocab_size, d_model, n_layers
        rp = rope_parameters if isinstance(rope_parameters, dict) else (rope_scaling if isinstance(rope_scaling, dict) else {})
        section = list(rp.get("mrope_section") or (24, 20, 20))
        self.mrope_section_t, self.mrope_section_h, self.mrope_section_w = (int(v) for v in section)
        self.deepstack_layers = len(deepstack_visual_indexes) if isinstance(deepstack_visual_indexes, (list, tuple)) else 3
        self.embedding = Embedding(vocab_size, d_model, hf_name="model.language_model.embed_tokens.weight")
        self.blocks = nn.BlockStack(n_layers, Qwen3VLBlock, d_model=d_model, num_query_heads=num_query_heads, num_kv_heads=num_kv_heads,
                                    head_size=head_size or d_model // num_query_heads, d_ff=d_ff, max_seq=max_seq, eps=eps, use_qkv_bias=bool(use_qkv_bias),
                                    rope_theta=float(rp.get("rope_theta", rope_theta)), mrope_section=section)
        self.final_norm = RMSNorm(d_model, eps=eps, hf_name="model.language_model.norm.weight")
        self.lm_head = LMHead(vocab_size, d_model, tie_to="embedding" if (tie_word_embeddings or text_tie) else None)

    def forward(self, token_ids, position_ids, targets):
        x = self.embedding(token_ids)
        x = F.torch_fn("visual_scatter", [x], [("x0_visual", x.shape, "act")], side_inputs=["visual_pos_masks", "visual_embeds"])
        residual = F.zeros(("B", "T", self.d_model), name="residual0")
        x, residual = self.blocks(x, residual, position_ids)
        residual, x = self.final_norm(residual, x)
        return self.lm_head(x, targets)
