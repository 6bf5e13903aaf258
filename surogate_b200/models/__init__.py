"""Model registry: what a ``config.json`` says about a model (family, MoE, multimodal, pre-quantisation)."""
from .registry import describe_config, quant_info, supported_architectures  # noqa: F401
