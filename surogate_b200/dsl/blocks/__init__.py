"""Per-architecture transformer blocks.  Parity: surogate/dsl/blocks/*.py."""
from .common import DENSE_BLOCK_NAME_REMAP, MOE_BLOCK_NAME_REMAP, STANDARD_MODEL_NAME_REMAP
from .dense import DenseBlock, Qwen3Block, LlamaBlock, Qwen2Block
from .moe import Qwen3MoEBlock

__all__ = ["DenseBlock", "Qwen3Block", "LlamaBlock", "Qwen2Block", "Qwen3MoEBlock", "DENSE_BLOCK_NAME_REMAP",
           "MOE_BLOCK_NAME_REMAP", "STANDARD_MODEL_NAME_REMAP"]
