"""YAML configuration system.  Parity: surogate/core/config/."""
from .loader import load_config, expand_env, DictDefault
from .sft_config import SFTConfig, PTConfig, DistributedConfig, DistillationConfig, DatasetConfig

__all__ = ["load_config", "expand_env", "DictDefault", "SFTConfig", "PTConfig", "DistributedConfig", "DistillationConfig", "DatasetConfig"]
