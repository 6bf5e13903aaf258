"""Training configuration for ``surogate sft`` / ``surogate pt``: the public YAML key set, defaults,
validation and the derived runtime settings.

Parity: surogate/core/config/sft_config.py (fields :337-471, validation :664-780,
create_runtime_config :1026-1153), docs/reference/config.md.
"""
from __future__ import annotations

import dataclasses
import json
import os
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

RECIPES = ("bf16", "fp8_hybrid", "nvfp4")
OPTIMIZERS = ("adamw_8bit", "adamw", "normuon")
SCHEDULERS = ("linear", "cosine", "constant", "wsd")
LORA_TARGETS_ALL = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]


@dataclass
class DatasetConfig:
    path: str = ""
    type: str = "auto"  # auto | text | instruction | conversation | preference | alpaca | messages
    split: str = "train"
    subset: Optional[str] = None
    text_field: str = "text"
    samples: Optional[int] = None
    # instruction / alpaca
    system_prompt_type: Optional[str] = None  # field | fixed
    system_prompt_field: Optional[str] = None
    system_prompt: Optional[str] = None
    instruction_field: str = "instruction"
    input_field: Optional[str] = "input"
    output_field: str = "output"
    prompt_format: Optional[str] = None
    prompt_format_no_input: Optional[str] = None
    # conversation / messages
    system_field: Optional[str] = None
    messages_field: str = "messages"
    completion_field: Optional[str] = None
    tools_field: Optional[str] = None
    message_property_mappings: Dict[str, str] = field(default_factory=dict)
    # preference (DPO)
    prompt_field: str = "prompt"
    chosen_field: str = "chosen"
    rejected_field: str = "rejected"
    enable_thinking_field: Optional[str] = None  # preference rows: column with a bool that switches the chat template's thinking prefix (default "enable_thinking" when present)
    fields: Dict[str, str] = field(default_factory=dict)

    @staticmethod
    def from_any(d) -> "DatasetConfig":
        if isinstance(d, str):
            return DatasetConfig(path=d)
        known = {f.name for f in dataclasses.fields(DatasetConfig)}
        return DatasetConfig(**{k: v for k, v in dict(d).items() if k in known})


@dataclass
class DistributedConfig:
    ray_address: Optional[str] = None
    num_nodes: int = 1
    gpus_per_node: int = 0
    worker_output_dir: Optional[str] = None
    master_addr: str = "127.0.0.1"
    master_port: int = 29500


@dataclass
class DistillationConfig:
    """Offline top-K distillation: training mixes ``kd_weight * tau^2 * KL(teacher || student)`` into the loss from ``.kd`` sidecars
    written by ``surogate distill-capture``.  A ``distillation:`` section switches it on unless it says ``enabled: false``.
    ``teacher_model`` / ``kd_dir`` are the other spellings of ``teacher`` / ``sidecar_dir``.  Keys marked capture are read by the
    capture command only.  Parity: surogate/core/config/sft_config.py:48-90."""
    enabled: Optional[bool] = None
    teacher: Optional[str] = None            # capture: model id / directory, or the served model's name with teacher_api_base
    teacher_model: Optional[str] = None
    top_k: int = 32
    temperature: float = 1.0
    kd_weight: float = 0.5
    ce_weight: Optional[float] = None        # default 1 - kd_weight
    teacher_batch_size: int = 4              # capture: rows per teacher forward
    sidecar_dir: Optional[str] = None        # sidecars live here instead of next to the token shards
    kd_dir: Optional[str] = None
    teacher_api_base: Optional[str] = None   # capture: OpenAI-compatible base URL of a served teacher (prompt_logprobs)
    teacher_api_key_var: Optional[str] = "VLLM_API_KEY"
    teacher_api_concurrency: int = 8
    teacher_api_timeout: int = 1200

    def __post_init__(self):
        self.teacher = self.teacher or self.teacher_model
        self.sidecar_dir = self.sidecar_dir or self.kd_dir
        if self.enabled is None:
            self.enabled = True
        if not 1 <= int(self.top_k) <= 1024:
            raise ValueError("[E115] distillation.top_k must be in 1..1024")
        if not float(self.temperature) > 0:
            raise ValueError("[E115] distillation.temperature must be > 0")
        if self.ce_weight is None:
            self.ce_weight = 1.0 - float(self.kd_weight)

    def api_key(self) -> str:
        return (os.environ.get(self.teacher_api_key_var) if self.teacher_api_key_var else None) or "EMPTY"


@dataclass
class SFTConfig:
    # model
    model: str = ""
    tokenizer_path: Optional[str] = None    # tokenizer directory when `model` is an inline config or `preset:<name>` (default: the model's own)
    torch_dtype: str = "bfloat16"
    max_model_len: Optional[int] = None
    rope_scaling: Optional[Dict[str, Any]] = None
    # run
    run_name: Optional[str] = None
    output_dir: str = "output"
    checkpoint_dir: Optional[str] = None
    resume_from_checkpoint: bool = True
    save_steps: int = 50
    save_total_limit: int = 5
    num_epochs: int = 3
    max_steps: int = -1
    eval_steps: int = 100
    logging_steps: int = 1
    log_file: Optional[str] = None
    report_to: List[str] = field(default_factory=list)
    log_gpu_util: int = 100
    wandb_project: Optional[str] = None     # default "Surogate"
    wandb_name: Optional[str] = None        # default run_name
    aim_experiment: Optional[str] = None    # default "Surogate"
    aim_repo: Optional[str] = None          # Aim repository path or URL (default: the working directory's)
    aim_name: Optional[str] = None          # default run_name
    surogate_metrics_path: str = "/tmp/surogate_metrics.jsonl"
    apply_recommended_values: bool = False
    # batch / data
    per_device_train_batch_size: int = 2
    gradient_accumulation_steps: int = 4
    sequence_len: int = 1024
    sample_packing: bool = True
    datasets: List[DatasetConfig] = field(default_factory=list)
    validation_datasets: List[DatasetConfig] = field(default_factory=list)
    validation_split_ratio: float = 0.1
    train_seed: int = 1234
    eval_seed: int = 5678
    dataloader_num_workers: int = 0
    truncation_strategy: str = "right"
    use_chat_template: bool = True
    loss_scale: str = "default"  # default (assistant turns) | last_round (assistant turns after the last user message) | all; a message's own `loss` field (0 / 1) overrides it
    # optimisation
    optimizer: str = "adamw_8bit"
    learning_rate: float = 2e-4
    lr_scheduler_type: str = "linear"
    warmup_ratio: float = 0.0
    warmup_steps: int = 0
    cooldown_steps: int = 0
    wsd_decay_steps_fraction: float = 0.1
    final_lr_fraction: float = 0.0
    max_grad_norm: float = 1.0
    weight_decay: float = 0.0
    adamw_beta1: float = 0.9
    adamw_beta2: float = 0.999
    adamw_epsilon: float = 1e-8
    normuon_momentum: float = 0.95
    normuon_beta2: float = 0.95
    normuon_cautious_wd: bool = True
    normuon_momentum_8bit: bool = False
    auto_lr_reduction: bool = False
    early_stop: bool = False
    epoch_adjustment: bool = False
    # precision
    recipe: str = "bf16"
    fp8_amax_history: int = 16
    fp4_four_over_six: bool = True
    fp4_backend: str = "native"
    skip_quant_first_layers: int = 0
    skip_quant_last_layers: int = 0
    gradient_dtype: Optional[str] = None
    master_dtype: Optional[str] = None
    use_fused_rope: bool = True
    # memory
    recompute: bool = True
    offload_residual: bool = False
    offload_saved_tensors: bool = False
    cpu_training: bool = False
    offload_master: bool = False
    resident_layers: int = -1  # with offload_master: frozen weights of the first N layers stay on the device (-1: SUROGATE_RESIDENT_LAYERS or 0)
    offload_quants: bool = False
    offload_optimizer: bool = False
    offload_grads: bool = False
    persistent_quants: bool = False
    use_zero_copy: bool = False
    use_write_combined: bool = False
    lmhead_chunks: int = 1
    auto_lmhead_chunks: bool = True
    lmhead_drop_ignored_rows: bool = False
    attn_bwd_chunks: int = 1
    long_context: bool = False
    train_vision: bool = False  # vision-language fine-tuning: rows with images, frozen vision tower, decoder trained (train/vision.py)
    sequence_chunks: int = 1
    use_cuda_graphs: bool = True  # replay forward + backward per micro-batch from CUDA graphs where that applies (dense models, replicated weights, bf16 / fp8)
    # parallelism
    gpus: int = 1
    zero_level: int = 1
    shard_weights: bool = False
    shard_gradients: bool = False
    use_all_to_all_reduce: bool = False
    memcpy_all_gather: bool = False
    memcpy_send_recv: bool = False
    ep_size: int = 1
    ep_load_balance_threshold: float = 1.3
    ep_capacity_factor: float = 1.5  # receive-buffer rows per rank relative to a perfectly balanced step; copies beyond it are dropped and counted
    ep_plan_refresh_interval: int = 16
    ep_spill_threshold: float = 0.0
    ep_spill_min_rows: int = 64
    async_optimizer: Optional[str] = None                   # with cpu_training: overlap | inline (host update one step behind, overlapped with compute)
    trainable_param_substrings: Optional[List[str]] = None  # full fine-tuning of a subset: names containing one of these train
    gradient_mask_mode: Optional[str] = None                # allow_substrings | mlp_growth_new_half
    parallelism: str = "ddp"  # ddp | dispatch_pp
    dispatch_pp: Dict[str, Any] = field(default_factory=dict)
    distributed: Optional[DistributedConfig] = None
    collectives: str = "auto"  # auto | nccl | symm  (symm = hand-written peer-memory kernels)
    # init
    from_scratch: bool = False
    init_projections_to_zero: bool = False
    adapter_path: Optional[str] = None
    adapter_init_mode: str = "merge"
    merge_adapter: bool = False
    # LoRA / QLoRA
    lora: bool = True
    lora_rank: int = 16
    lora_alpha: int = 32
    lora_dropout: float = 0.0
    lora_dtype: str = "fp32"
    lora_target_modules: List[str] = field(default_factory=lambda: list(LORA_TARGETS_ALL))
    use_rslora: bool = False
    train_router: bool = False
    router_aux_loss_coef: Optional[float] = None
    router_z_loss_coef: Optional[float] = None
    qlora_fp4: bool = False
    qlora_fp8: bool = False
    qlora_bnb: bool = False
    qlora_block_size: int = 128
    qlora_bnb_block_size: int = 64
    qlora_bnb_double_quant: bool = True
    qlora_four_over_six: bool = True
    qlora_selective_expert_dequant: bool = False
    qlora_offload_experts: bool = False
    # debug
    debug_time_breakdown: bool = False
    debug_memory_breakdown: bool = False
    train_vision: bool = False
    distillation: Optional[DistillationConfig] = None
    # synthetic data (benchmarks / tests without datasets)
    synthetic_data: bool = False

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_dict(cls, d) -> "SFTConfig":
        known = {f.name for f in dataclasses.fields(cls)}
        unknown = [k for k in d if k not in known]
        if unknown:
            raise ValueError(f"[E100] unknown config key(s): {sorted(unknown)}")
        kw = dict(d)
        kw["datasets"] = [DatasetConfig.from_any(x) for x in (kw.get("datasets") or [])]
        kw["validation_datasets"] = [DatasetConfig.from_any(x) for x in (kw.get("validation_datasets") or [])]
        if kw.get("distributed"):
            from .loader import coerce_fields as _cf

            kw["distributed"] = DistributedConfig(**_cf(DistributedConfig, dict(kw["distributed"])))
        if kw.get("distillation"):
            from .loader import coerce_fields as _cf

            kw["distillation"] = DistillationConfig(**_cf(DistillationConfig, dict(kw["distillation"])))
        if isinstance(kw.get("report_to"), str):
            kw["report_to"] = [kw["report_to"]]
        kw = {k: v for k, v in kw.items() if v is not None or k in ("run_name",)}
        from .loader import coerce_fields

        cfg = cls(**coerce_fields(cls, kw))
        cfg.finalize()
        return cfg

    # ------------------------------------------------------------------ validation + derived settings
    def finalize(self) -> None:
        self.recipe = self.recipe.replace("-", "_").lower()
        if self.recipe not in RECIPES:
            raise ValueError(f"[E101] recipe must be one of {RECIPES}, got '{self.recipe}'")
        self.optimizer = self.optimizer.lower()
        if self.optimizer not in OPTIMIZERS:
            raise ValueError(f"[E102] optimizer must be one of {OPTIMIZERS}, got '{self.optimizer}'")
        if self.lr_scheduler_type not in SCHEDULERS:
            raise ValueError(f"[E103] lr_scheduler_type must be one of {SCHEDULERS}")
        if self.zero_level not in (0, 1, 2, 3):
            raise ValueError("[E104] zero_level must be 0..3")
        # zero_level <-> shard flags (either spelling may be used)
        if self.shard_weights:
            self.zero_level = 3
        elif self.shard_gradients:
            self.zero_level = max(self.zero_level, 2)
        self.shard_gradients = self.zero_level >= 2
        self.shard_weights = self.zero_level >= 3
        if self.gpus < 1:
            raise ValueError("[E105] gpus must be >= 1")
        if self.ep_size > 1 and self.gpus % self.ep_size != 0:
            raise ValueError(f"[E106] ep_size={self.ep_size} must divide gpus={self.gpus}")
        if self.sequence_chunks > 1 and self.per_device_train_batch_size != 1:
            raise ValueError("[E107] sequence_chunks > 1 requires per_device_train_batch_size == 1")
        if self.sequence_chunks > 1 and self.sequence_len % self.sequence_chunks != 0:
            raise ValueError("[E108] sequence_len must be divisible by sequence_chunks")
        if sum([self.qlora_fp4, self.qlora_fp8, self.qlora_bnb]) > 1:
            raise ValueError("[E109] choose at most one of qlora_fp4 / qlora_fp8 / qlora_bnb")
        if (self.qlora_fp4 or self.qlora_fp8 or self.qlora_bnb) and not self.lora:
            raise ValueError("[E110] QLoRA requires lora: true")
        if self.cpu_training:
            self.offload_master = self.offload_optimizer = self.offload_grads = True
        if self.parallelism not in ("ddp", "dispatch_pp"):
            raise ValueError("[E111] parallelism must be ddp or dispatch_pp")
        if self.from_scratch and self.lora:
            raise ValueError("[E112] from_scratch (pre-training) trains all weights: set lora: false")
        if self.attn_bwd_chunks < 1 or (self.attn_bwd_chunks > 1 and self.per_device_train_batch_size % self.attn_bwd_chunks != 0):
            raise ValueError("[E113] attn_bwd_chunks must be >= 1 and divide per_device_train_batch_size")
        if self.async_optimizer and not self.cpu_training:
            raise ValueError("[E114] async_optimizer overlaps the host optimizer with device compute: set cpu_training: true")
        if self.checkpoint_dir is None:
            self.checkpoint_dir = self.output_dir
        if self.run_name is None:
            self.run_name = f"run-{time.strftime('%Y%m%d-%H%M%S')}"
        if self.log_file is None:
            self.log_file = os.path.join(self.output_dir, f"log-{self.run_name}.json")
        # CUDA graphs are only kept where every op in the step is capture-safe
        if any([self.qlora_fp4, self.qlora_fp8, self.qlora_bnb, self.offload_master, self.sequence_chunks > 1, self.debug_time_breakdown,
                self.lmhead_drop_ignored_rows, self.distillation is not None and self.distillation.enabled,
                self.parallelism == "dispatch_pp", self.ep_size > 1]):
            self.use_cuda_graphs = False

    def auto_lmhead_rows(self, tokens_per_micro_batch: int, vocab: int) -> int:
        """Rows per LM-head chunk: bound the transient logits buffer to ~2 GiB unless lmhead_chunks is given."""
        if self.lmhead_chunks > 1 or not self.auto_lmhead_chunks:
            return max(1, tokens_per_micro_batch // max(1, self.lmhead_chunks))
        rows = max(256, (2 << 30) // (2 * vocab))
        return min(tokens_per_micro_batch, rows // 128 * 128 or 128)

    def lora_dict(self) -> Optional[Dict[str, Any]]:
        if not self.lora:
            return None
        return dict(rank=self.lora_rank, alpha=self.lora_alpha, dropout=self.lora_dropout, dtype=self.lora_dtype,
                    targets=list(self.lora_target_modules), rslora=self.use_rslora, train_router=self.train_router)

    def to_trainer_config(self, hf_config: Dict[str, Any]):
        from ..runtime.trainer import TrainerConfig

        vocab = hf_config.get("vocab_size", 151936)
        tokens = self.per_device_train_batch_size * self.sequence_len
        return TrainerConfig(
            model=hf_config, batch_size=self.per_device_train_batch_size, seq_len=self.sequence_len, grad_accum=self.gradient_accumulation_steps,
            recipe=self.recipe, optimizer=self.optimizer, learning_rate=self.learning_rate, beta1=self.adamw_beta1, beta2=self.adamw_beta2,
            eps=self.adamw_epsilon, weight_decay=self.weight_decay, max_grad_norm=self.max_grad_norm, zero_level=self.zero_level,
            recompute=self.recompute, grad_dtype={"fp32": "fp32", "float32": "fp32"}.get(self.gradient_dtype or "", "bf16"),
            master_dtype={"fp32": "fp32", "float32": "fp32"}.get(self.master_dtype or "", None),
            lmhead_chunk_rows=self.auto_lmhead_rows(tokens, vocab), ep_size=self.ep_size, ep_load_balance_threshold=self.ep_load_balance_threshold, ep_capacity_factor=self.ep_capacity_factor,
            ep_plan_refresh_interval=self.ep_plan_refresh_interval, ep_spill_threshold=self.ep_spill_threshold, ep_spill_min_rows=self.ep_spill_min_rows,
            lora=self.lora_dict(),
            async_optimizer=self.async_optimizer, trainable_param_substrings=self.trainable_param_substrings, gradient_mask_mode=self.gradient_mask_mode,
            fp8_amax_history=self.fp8_amax_history, skip_quant_first_layers=self.skip_quant_first_layers,
            skip_quant_last_layers=self.skip_quant_last_layers, offload_optimizer=self.offload_optimizer and not self.cpu_training,
            offload_master=self.offload_master and not self.cpu_training, cpu_training=self.cpu_training, long_context=self.long_context, sequence_chunks=self.sequence_chunks, use_cuda_graphs=self.use_cuda_graphs, lmhead_drop_ignored_rows=self.lmhead_drop_ignored_rows, time_breakdown=self.debug_time_breakdown, resident_layers=self.resident_layers,
            offload_saved_tensors=self.offload_saved_tensors or self.offload_residual,
            qlora="bnb_nf4" if self.qlora_bnb else "fp8_block" if self.qlora_fp8 else "nvfp4" if self.qlora_fp4 else None,
            qlora_offload_experts=self.qlora_offload_experts,
            qlora_block_size=self.qlora_bnb_block_size if self.qlora_bnb else self.qlora_block_size, qlora_double_quant=self.qlora_bnb_double_quant,
            qlora_four_over_six=self.qlora_four_over_six, fp4_four_over_six=self.fp4_four_over_six,
            normuon_momentum=self.normuon_momentum, normuon_beta2=self.normuon_beta2, normuon_cautious_wd=self.normuon_cautious_wd, normuon_momentum_8bit=self.normuon_momentum_8bit,
            init_projections_to_zero=self.init_projections_to_zero, seed=self.train_seed, collectives=self.collectives)

    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self), default=str)


@dataclass
class PTConfig(SFTConfig):
    """Pre-training = SFT with every token in the loss, random init allowed and no adapters by default."""
    lora: bool = False
    loss_scale: str = "all"
    use_chat_template: bool = False
