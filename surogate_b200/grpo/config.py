"""GRPO configuration: trainer side (``surogate grpo``), orchestrator side (``grpo-orch``) and inference server (``grpo-infer``).

Parity: surogate/core/config/grpo_orch_config.py, grpo_inference_config.py, surogate/grpo/config.py.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from ..config.sft_config import SFTConfig


@dataclass
class GRPOLossConfig:
    """``type: clip`` = PPO-style ratio clipping (``clip_eps_*``, ``kl_coef``, ``ratio_cap``); ``type: ipo`` = probability-difference
    masking with a squared log-ratio penalty (``ipo_mask_*``, ``adv_tau``, ``teacher_tau``, ``kl_tau``, ``ratio_clip``), the objective of
    surogate/grpo/config.py:GRPOLossConfig.  With ``type`` unset, a section that sets any of the ``ipo`` keys selects ``ipo``."""
    type: Optional[str] = None           # clip | ipo
    clip_eps_low: float = 0.2
    clip_eps_high: float = 0.2
    kl_coef: float = 0.0                 # weight of the k3 KL estimate against the reference policy
    ratio_cap: float = 10.0              # tokens whose importance ratio exceeds this are dropped (stale rollouts)
    normalization: str = "token"         # token (DAPO style: / total tokens) | sequence (mean per sequence, then mean)
    advantage_clip: float = 0.0
    ipo_mask_low: Optional[float] = None     # 0.2: a token whose probability fell by more than this since the rollout leaves the policy term
    ipo_mask_high: Optional[float] = None    # 0.2: ... or rose by more than this
    adv_tau: Optional[float] = None          # 1.0: weight of the advantage
    teacher_tau: Optional[float] = None      # 0.0: weight of the (detached) teacher log-ratio added to the advantage
    kl_tau: Optional[float] = None           # 1e-3: weight of the squared log-ratio penalty
    ratio_clip: Optional[float] = None       # e^2: cap of the importance ratio that multiplies the gradient

    IPO_DEFAULTS = {"ipo_mask_low": 0.2, "ipo_mask_high": 0.2, "adv_tau": 1.0, "teacher_tau": 0.0, "kl_tau": 1e-3, "ratio_clip": 7.389056}

    def __post_init__(self):
        given = [k for k in self.IPO_DEFAULTS if getattr(self, k) is not None]
        if self.type is None:
            self.type = "ipo" if given else "clip"
        if self.type not in ("clip", "ipo"):
            raise ValueError(f"loss.type must be clip or ipo, got {self.type!r}")
        for k, v in self.IPO_DEFAULTS.items():
            if getattr(self, k) is None:
                setattr(self, k, v)


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
    noise_scheduler: Optional[Dict[str, Any]] = None   # {enabled, sigma_start, sigma_end, num_stages}: exploration noise on published weights (grpo/noise.py)
    pad_to_multiple_of: int = 1
    single_sample_bins: bool = False     # one sample per packed row (no packing of several samples into a row)
    doc_masking: bool = True             # attention stays inside each packed sample
    turn_diagnostics: bool = False       # per-turn KL / loss shares in the step metrics (grpo/turn_stats.py)

    @classmethod
    def from_dict(cls, d):
        d = dict(d)
        # the other spellings of two keys (surogate/grpo/config.py: GRPOTrainConfig)
        if "transport_type" in d:
            d.setdefault("transport", d.pop("transport_type"))
        if "weight_broadcast_type" in d:
            d.setdefault("weight_broadcast", d.pop("weight_broadcast_type"))
        loss = d.pop("loss", None)
        cfg = super().from_dict(d)
        if loss:
            from ..config.loader import coerce_fields

            cfg.loss = GRPOLossConfig(**coerce_fields(GRPOLossConfig, dict(loss)))
        return cfg


@dataclass
class InferenceConfig:
    """The rollout engine (a vLLM OpenAI server).  ``tp`` / ``dp`` / ``weight_broadcast_type`` are the short spellings of
    ``tensor_parallel_size`` / ``data_parallel_size`` / ``weight_broadcast``; keys left at None keep the engine's own default.
    Parity: surogate/core/config/grpo_inference_config.py."""
    model: str = ""
    host: str = "127.0.0.1"
    port: int = 8000
    tensor_parallel_size: int = 1
    data_parallel_size: int = 1
    tp: Optional[int] = None
    dp: Optional[int] = None
    gpu_memory_utilization: float = 0.85
    dtype: str = "auto"                       # auto | float16 | bfloat16 | float32
    max_model_len: Optional[int] = None
    max_num_seqs: Optional[int] = None
    kv_cache_dtype: Optional[str] = None      # e.g. fp8
    enforce_eager: bool = False
    attention_backend: Optional[str] = None
    trust_remote_code: bool = False
    enable_auto_tool_choice: bool = False
    tool_call_parser: Optional[str] = "hermes"
    reasoning_parser: Optional[str] = None
    rope_scaling: Optional[Any] = None
    enable_lora: bool = True
    max_loras: int = 8
    max_cpu_loras: int = 100
    max_lora_rank: Optional[int] = 64
    enable_prefix_caching: Optional[bool] = None
    api_server_count: int = 1
    seed: int = 0
    enable_expert_parallel: bool = False
    all2all_backend: Optional[str] = None
    enable_eplb: bool = False
    weight_dir: str = "output/grpo/weights"
    weight_broadcast: str = "filesystem"   # filesystem | nccl | colocate: which receiver the engine's workers mix in (grpo/vllm_worker.py)
    weight_broadcast_type: Optional[str] = None
    extra_args: List[str] = field(default_factory=list)

    VALID_LORA_RANKS = (8, 16, 32, 64, 128, 256, 320, 512)

    def __post_init__(self):
        if self.tp is not None:
            self.tensor_parallel_size = int(self.tp)
        if self.dp is not None:
            self.data_parallel_size = int(self.dp)
        if self.weight_broadcast_type:
            self.weight_broadcast = self.weight_broadcast_type
        if self.weight_broadcast not in ("filesystem", "nccl", "colocate"):
            raise ValueError(f"weight_broadcast must be filesystem, nccl or colocate, got {self.weight_broadcast!r}")
        if self.max_lora_rank is not None:  # the engine accepts a fixed set of ranks: round up to the next one
            fit = next((r for r in self.VALID_LORA_RANKS if r >= int(self.max_lora_rank)), None)
            if fit is None:
                raise ValueError(f"max_lora_rank={self.max_lora_rank} exceeds the engine's maximum of {self.VALID_LORA_RANKS[-1]}")
            self.max_lora_rank = fit
        self.api_server_count = max(int(self.api_server_count), int(self.data_parallel_size))
        if self.enable_lora:
            self.api_server_count = 1  # adapter hot-loading needs a single API server


@dataclass
class OrchestratorConfig:
    model: str = ""
    base_url: str = "http://127.0.0.1:8000/v1"
    prompts: str = ""                    # jsonl with {"prompt": str | messages, "answer": optional}
    reward: str = "exact_match"          # name in grpo.rewards.REWARDS or "module:function"
    environment: str = ""                # an environment id (grpo/environments, or a scaffolded one): supplies prompts and the reward
    environment_args: Dict[str, Any] = field(default_factory=dict)
    environments: List[Dict[str, Any]] = field(default_factory=list)   # several environments training together: [{id, name, args, path}]; prompts carry `task` = name
    environments_path: str = "./environments"
    environment_import_path: str = ""    # a directory put in front of sys.path before importing the environment's package (a local checkout)
    group_size: int = 8                  # rollouts per prompt
    prompts_per_step: int = 8
    max_tokens: int = 512
    temperature: float = 1.0
    top_p: float = 1.0
    seed: int = 0
    sequence_len: int = 2048
    rows_per_step: int = 8               # packed rows handed to the trainer per optimizer step (all ranks together); 0 = as many as needed
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
    teacher: Dict[str, Any] = field(default_factory=dict)  # {model, base_url, api_key_var, timeout}: a served teacher that scores every rollout's tokens (loss.teacher_tau)
    ruler: Dict[str, Any] = field(default_factory=dict)   # LLM-judge group reward (grpo/ruler.py): enabled, mode, judge_model, judge {base_url, ...}, rubric, weight ...
