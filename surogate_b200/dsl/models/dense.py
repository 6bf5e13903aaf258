"""Dense decoder-only models (Qwen3, Qwen2/2.5, Llama, Mistral).

Parity: surogate/dsl/models/qwen3.py:28, models/llama.py.
"""
from __future__ import annotations

from .. import functional as F
from .. import nn
from ..blocks import LlamaBlock, Qwen2Block, Qwen3Block, STANDARD_MODEL_NAME_REMAP
from ..modules import Embedding, LMHead, RMSNorm

_COMMON = dict(d_model="hidden_size", n_layers="num_hidden_layers", num_query_heads="num_attention_heads",
               num_kv_heads="num_key_value_heads", d_ff="intermediate_size", vocab_size="vocab_size",
               max_seq="max_position_embeddings", head_size="head_dim", eps="rms_norm_eps", rope_theta="rope_theta",
               tie_word_embeddings="tie_word_embeddings")


class DenseModel(nn.Model):
    _name_remap_ = STANDARD_MODEL_NAME_REMAP
    block_cls = LlamaBlock
    block_extra: dict = {}

    def __init__(self, vocab_size: int = 151936, d_model: int = 1024, n_layers: int = 28, num_query_heads: int = 16,
                 num_kv_heads: int = 8, d_ff: int = 3072, max_seq: int = 40960, head_size: int = 0, eps: float = 1e-6,
                 rope_theta: float = 1e6, tie_word_embeddings: bool = False, **block_overrides):
        super().__init__()
        self.vocab_size, self.d_model, self.n_layers = vocab_size, d_model, n_layers
        self.num_query_heads, self.num_kv_heads, self.d_ff, self.max_seq = num_query_heads, num_kv_heads, d_ff, max_seq
        self.head_size = head_size if head_size and head_size > 0 else d_model // num_query_heads
        self.eps, self.rope_theta, self.tie_word_embeddings = eps, float(rope_theta), bool(tie_word_embeddings)
        self.embedding = Embedding(vocab_size, d_model)
        self.blocks = nn.BlockStack(
            n_layers, self.block_cls, d_model=d_model, num_query_heads=num_query_heads, num_kv_heads=num_kv_heads,
            head_size=self.head_size, d_ff=d_ff, max_seq=max_seq, eps=eps, rope_theta=self.rope_theta,
            **{**self.block_extra, **block_overrides})
        self.final_norm = RMSNorm(d_model, eps=eps, hf_name="model.norm.weight")
        self.lm_head = LMHead(vocab_size, d_model, tie_to="embedding" if self.tie_word_embeddings else None)

    def forward(self, token_ids, position_ids, targets):
        x = self.embedding(token_ids)
        residual = F.zeros(("B", "T", self.d_model), name="residual0")
        x, residual = self.blocks(x, residual, position_ids)
        residual, x = self.final_norm(residual, x)
        return self.lm_head(x, targets)


@nn.hf_config(architecture="Qwen3ForCausalLM", model_type="qwen3", **_COMMON)
class Qwen3Model(DenseModel):
    block_cls = Qwen3Block


@nn.hf_config(architecture="Qwen2ForCausalLM", model_type="qwen2", **_COMMON)
class Qwen2Model(DenseModel):
    block_cls = Qwen2Block


@nn.hf_config(architecture="LlamaForCausalLM", model_type="llama", **_COMMON)
class LlamaModel(DenseModel):
    block_cls = LlamaBlock

    def __init__(self, **kw):
        kw.setdefault("rope_theta", 10000.0)
        super().__init__(**kw)


@nn.hf_config(architecture="MistralForCausalLM", model_type="mistral", **_COMMON)
class MistralModel(LlamaModel):
    pass
