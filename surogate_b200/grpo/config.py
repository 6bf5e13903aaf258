"""GRPO configuration: trainer side (``surogate grpo``), orchestrator side (``grpo-orch``) and inference server (``grpo-infer``).

Parity: surogate/core/config/grpo_orch_config.py, grpo_inference_config.py, surogate/grpo/config.py.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from ..config.sft_config import SFTConfig


@dataclass
class GRPOLossConfig:
    clip_eps_low: float = 0.2
    clip_eps_high: float = 0.2
    kl_coef: float = 0.0                 # weight of the k3 KL estimate against the reference policy
    ratio_cap: float = 10.0              # tokens whose importance ratio exceeds this are dropped (stale rollouts)
    normalization: str = "token"         # token (DAPO style: / total tokens) | sequence (mean per sequence, then mean)
    advantage_clip: float = 0.0


@dataclass
class GRPOConfig(SFTConfig):
    loss: GRPOLossConfig = field(default_factory=GRPOLossConfig)
    transport: str = "filesystem"        # filesystem | zmq
    transport_dir: str = "output/grpo/rollouts"
    zmq_endpoint: str = "tcp://127.0.0.1:5599"
    weight_broadcast: str = "filesystem"  # filesystem | nccl | colocate
    weight_dir: str = "output/grpo/weights"
    broadcast_every: int = 1
    max_async_level: int = 2             # rollouts may lag the trainer by at most this many policy versions
    sample_packing: bool = True
    learning_rate: float = 1e-6

    @classmethod
    def from_dict(cls, d):
        d = dict(d)
        loss = d.pop("loss", None)
        cfg = super().from_dict(d)
        if loss:
            from ..config.loader import coerce_fields

            cfg.loss = GRPOLossConfig(**coerce_fields(GRPOLossConfig, dict(loss)))
        return cfg


@dataclass
class InferenceConfig:
    model: str = ""
    host: str = "127.0.0.1"
    port: int = 8000
    tensor_parallel_size: int = 1
    gpu_memory_utilization: float = 0.85
    max_model_len: Optional[int] = None
    enable_lora: bool = True
    max_lora_rank: int = 64
    weight_dir: str = "output/grpo/weights"
    weight_broadcast: str = "filesystem"   # filesystem | nccl | colocate: which receiver the engine's workers mix in (grpo/vllm_worker.py)
    extra_args: List[str] = field(default_factory=list)


@dataclass
class OrchestratorConfig:
    model: str = ""
    base_url: str = "http://127.0.0.1:8000/v1"
    prompts: str = ""                    # jsonl with {"prompt": str | messages, "answer": optional}
    reward: str = "exact_match"          # name in grpo.rewards.REWARDS or "module:function"
    environment: str = ""                # an environment id (grpo/environments, or a scaffolded one): supplies prompts and the reward
    environment_args: Dict[str, Any] = field(default_factory=dict)
    environments_path: str = "./environments"
    group_size: int = 8                  # rollouts per prompt
    prompts_per_step: int = 8
    max_tokens: int = 512
    temperature: float = 1.0
    top_p: float = 1.0
    seed: int = 0
    sequence_len: int = 2048
    rows_per_step: int = 8               # packed rows handed to the trainer per optimizer step (all ranks together)
    max_async_level: int = 2
    transport: str = "filesystem"
    transport_dir: str = "output/grpo/rollouts"
    zmq_endpoint: str = "tcp://127.0.0.1:5599"
    weight_dir: str = "output/grpo/weights"
    max_steps: int = 100
    filter_zero_advantage: bool = True   # groups whose rewards are all equal carry no signal
    advantage_std_eps: float = 1e-6
    length_penalty: float = 0.0
    request_timeout_s: float = 600.0
    extra_sampling: Dict[str, Any] = field(default_factory=dict)
