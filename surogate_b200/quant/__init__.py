"""Weight-storage codecs for QLoRA (NF4, block FP8, NVFP4) and pre-quantised checkpoints (MXFP4, block FP8)."""
from .codecs import CODECS, BnbNF4, BlockFP8, MXFP4, NVFP4Storage, make_codec  # noqa: F401
