"""Model definitions.  Parity: surogate/dsl/models/*.py."""
from .dense import Qwen3Model, Qwen2Model, LlamaModel, MistralModel
from .moe import Qwen3MoEModel

__all__ = ["Qwen3Model", "Qwen2Model", "LlamaModel", "MistralModel", "Qwen3MoEModel"]
