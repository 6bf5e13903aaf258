"""Model definitions.  Parity: surogate/dsl/models/*.py."""
from .dense import Qwen3Model, Qwen2Model, LlamaModel, MistralModel
from .moe import Qwen3MoEModel
from .gpt_oss import GptOssModel
from .lfm2 import Lfm2Model
from .nemotron_h import NemotronHModel
from .qwen3_5 import Qwen35Model
from .qwen3_5_moe import Qwen35MoEModel
from .qwen3_vl import Qwen3VLModel
from .laguna import LagunaModel
from .gemma4 import Gemma4Model

__all__ = ["Qwen3Model", "Qwen2Model", "LlamaModel", "MistralModel", "Qwen3MoEModel", "GptOssModel", "Lfm2Model", "NemotronHModel", "Qwen35Model", "Qwen35MoEModel", "Qwen3VLModel", "LagunaModel", "Gemma4Model"]
