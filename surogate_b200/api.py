"""The trainer-level Python API under the names of the reference's extension module, on top of this package's ``Trainer``.

    from surogate_b200.api import DataLoader, OptimizerConfig, PretrainedConfig, RuntimeOptions, SurogateTrainer

    trainer = SurogateTrainer.from_pretrained(name="/models/Qwen3-8B", ngpu=1, dtype="bf16", options=RuntimeOptions(recipe="fp8-hybrid"),
                                              batch_size=2, seq_len=4096, grad_accum=4)
    loader = DataLoader(["tokens/train-000.bin"], chunk_size=2 * 4096, seed=42)
    for step in range(100):
        for _ in range(4):                       # grad_accum micro-steps
            loader.load_batch(inputs, targets)
            trainer.step(inputs, targets)
        print(trainer.update_with_config(OptimizerConfig.adamw_8bit(lr=1e-5), step + 1))

Differences that come from the execution model: the reference drives ``ngpu`` GPUs from one process, here one process drives one
GPU, so ``ngpu`` must equal the number of ranks the script was started with (``torchrun --nproc-per-node N script.py``; 1 without
a launcher) and every rank passes the same ``[batch_size * ngpu, seq_len]`` arrays, of which it uses its own rows.  A micro-step
is queued by ``step`` / ``step_with_custom_loss`` / ``step_with_kd`` and the whole accumulation window runs inside
``update_with_config`` (the loss normaliser is the number of target tokens of the window, which is only known then).

Parity: surogate/_surogate.pyi (SurogateTrainer, PretrainedConfig, RuntimeOptions, OptimizerConfig, LoRAAdapterConfig, QLoRAConfig,
DataLoader, SystemInfo, GPUInfo), docs/reference/python-api.md.
"""
from __future__ import annotations

import os
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import numpy as np

IGNORE = -100


# ---------------------------------------------------------------------- configuration objects
@dataclass
class OptimizerConfig:
    optimizer: str = "adamw_8bit"
    learning_rate: float = 2e-4
    weight_decay: float = 0.1
    grad_clip: float = 0.0
    adamw_beta1: float = 0.9
    adamw_beta2: float = 0.999
    adamw_epsilon: float = 1e-8
    normuon_momentum: float = 0.95
    normuon_beta2: float = 0.95
    normuon_lr: float = 0.02
    normuon_cautious_wd: bool = True

    @property
    def type(self) -> str:
        return self.optimizer

    @type.setter
    def type(self, v: str) -> None:
        self.optimizer = v

    @staticmethod
    def adamw(lr: float = 2e-4, beta1: float = 0.9, beta2: float = 0.999, epsilon: float = 1e-8, weight_decay: float = 0.1, grad_clip: float = 0.0) -> "OptimizerConfig":
        return OptimizerConfig("adamw", lr, weight_decay, grad_clip, beta1, beta2, epsilon)

    @staticmethod
    def adamw_8bit(lr: float = 2e-4, beta1: float = 0.9, beta2: float = 0.999, epsilon: float = 1e-8, weight_decay: float = 0.1, grad_clip: float = 0.0) -> "OptimizerConfig":
        return OptimizerConfig("adamw_8bit", lr, weight_decay, grad_clip, beta1, beta2, epsilon)

    @staticmethod
    def normuon(lr: float = 0.02, momentum: float = 0.95, beta2: float = 0.95, weight_decay: float = 0.01, grad_clip: float = 0.0, cautious_wd: bool = True) -> "OptimizerConfig":
        return OptimizerConfig("normuon", lr, weight_decay, grad_clip, normuon_momentum=momentum, normuon_beta2=beta2, normuon_lr=lr, normuon_cautious_wd=cautious_wd)


DTYPES = {"bf16": "bf16", "bfloat16": "bf16", "fp16": "fp16", "float16": "fp16", "fp32": "fp32", "float32": "fp32"}


@dataclass
class PretrainedConfig:
    architecture: str = "Qwen3ForCausalLM"
    hidden_size: int = 0
    intermediate_size: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    num_hidden_layers: int = 0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    vocab_size: Optional[int] = None
    max_position_embeddings: Optional[int] = None
    rope_theta: Optional[float] = None
    use_qkv_bias: Optional[bool] = None
    dtype: str = "bf16"
    extra: Dict[str, Any] = field(default_factory=dict)  # every other key of a config.json (head_dim, MoE sizes, rope_scaling ...)

    SHORT_NAMES = {"qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM", "llama": "LlamaForCausalLM", "mistral": "MistralForCausalLM",
                   "qwen3_moe": "Qwen3MoeForCausalLM", "gpt_oss": "GptOssForCausalLM"}

    @property
    def head_size(self) -> int:
        return int(self.extra.get("head_dim") or (self.hidden_size // max(1, self.num_attention_heads)))

    @property
    def qkv_channels(self) -> int:
        return self.head_size * (self.num_attention_heads + 2 * self.num_key_value_heads)

    @property
    def model_name(self) -> str:
        return self.architecture

    @classmethod
    def from_pretrained(cls, name: str, dtype: str = "bf16") -> "PretrainedConfig":
        """From a directory with ``config.json`` (or a hub id resolved through the local cache / the hub)."""
        from .dsl.compiler import load_hf_config
        from .hub import download_model

        path = name if os.path.exists(name) else download_model(name)
        return cls.from_hf_dict(load_hf_config(path), dtype)

    @classmethod
    def from_name(cls, name: str, dtype: str = "bf16") -> "PretrainedConfig":
        """An architecture preset by name (``qwen3-8b``, ``Qwen/Qwen3-8B``, ``llama-3.1-8b`` ...; ``models/presets.py``); names without a
        preset fall back to ``from_pretrained``."""
        from .models.presets import preset_config

        try:
            return cls.from_hf_dict(preset_config(name), dtype)
        except KeyError:
            return cls.from_pretrained(name, dtype)

    @classmethod
    def from_hf_dict(cls, hf: Dict[str, Any], dtype: str = "bf16") -> "PretrainedConfig":
        arch = (hf.get("architectures") or [hf.get("architecture") or "Qwen3ForCausalLM"])[0]
        own = {"hidden_size", "intermediate_size", "num_attention_heads", "num_key_value_heads", "num_hidden_layers", "rms_norm_eps", "tie_word_embeddings",
               "bos_token_id", "eos_token_id", "vocab_size", "max_position_embeddings", "rope_theta"}
        kw = {k: hf[k] for k in own if k in hf}
        if "attention_bias" in hf:
            kw["use_qkv_bias"] = bool(hf["attention_bias"])
        return cls(architecture=arch, dtype=DTYPES.get(dtype, dtype), extra={k: v for k, v in hf.items() if k not in own and k not in ("architectures", "architecture")}, **kw)

    def to_hf_dict(self) -> Dict[str, Any]:
        arch = self.SHORT_NAMES.get(self.architecture.lower(), self.architecture)
        out = dict(self.extra, architectures=[arch], hidden_size=self.hidden_size, intermediate_size=self.intermediate_size,
                   num_attention_heads=self.num_attention_heads, num_key_value_heads=self.num_key_value_heads, num_hidden_layers=self.num_hidden_layers,
                   rms_norm_eps=self.rms_norm_eps, tie_word_embeddings=self.tie_word_embeddings)
        for k in ("bos_token_id", "eos_token_id", "vocab_size", "max_position_embeddings", "rope_theta"):
            if getattr(self, k) is not None:
                out[k] = getattr(self, k)
        if self.use_qkv_bias is not None:
            out["attention_bias"] = self.use_qkv_bias
        return out


@dataclass
class RuntimeOptions:
    recompute_swiglu: bool = False
    recompute_rmsnorm: bool = False
    recompute_ffn: bool = False
    recompute_qkv: bool = False
    recompute_att: bool = False
    recompute_block: bool = False
    offload_residual: bool = False
    use_cuda_graphs: bool = True
    trigger_timing_events: bool = False
    offload_master: bool = False
    offload_quants: bool = False
    offload_optimizer: bool = False
    offload_grads: bool = False
    use_zero_copy: bool = False
    use_write_combined: bool = False
    shard_weights: bool = False
    persistent_quants: bool = False
    shard_gradients: bool = False
    use_all_to_all_reduce: bool = False
    init_projections_to_zero: bool = False
    lmhead_chunks: int = 1
    attn_bwd_chunks: int = 1
    matmul_type: str = ""
    gradient_type: str = ""
    master_dtype: str = ""
    recipe: str = "bf16"
    matmul_backend: str = ""
    use_fused_rope: bool = False
    doc_masking: bool = True
    fp8_amax_history: int = 1024
    fp4_backend: str = "cutlass"
    no_fp4_stochastic_rounding: bool = False
    skip_quant_first_layers: int = 0
    skip_quant_last_layers: int = 0

    def set_recipe(self, recipe_name: str) -> None:
        self.recipe = recipe_name

    @property
    def recipe_name(self) -> str:
        return self.recipe

    @property
    def fp8_enabled(self) -> bool:
        return self.recipe.replace("_", "-") == "fp8-hybrid"

    @property
    def fp4_enabled(self) -> bool:
        return self.recipe.startswith("nvfp4")

    def trainer_kwargs(self) -> Dict[str, Any]:
        """These options as ``TrainerConfig`` fields.  Any ``recompute_*`` switches block recomputation on (this engine recomputes
        whole blocks from their saved inputs); sharding flags map to the ZeRO level; the options that pick a library back end
        (``matmul_backend``, ``fp4_backend``, ``use_fused_rope``, ``use_zero_copy``, ``use_write_combined``,
        ``use_all_to_all_reduce``, ``persistent_quants``) have no counterpart: there is one code path."""
        recompute = any([self.recompute_block, self.recompute_att, self.recompute_ffn, self.recompute_qkv, self.recompute_swiglu, self.recompute_rmsnorm])
        zero = 3 if self.shard_weights else 2 if self.shard_gradients else 1
        kw: Dict[str, Any] = dict(recipe=self.recipe.replace("-", "_").replace("nvfp4_quartet", "nvfp4"), recompute=recompute, zero_level=zero,
                                  offload_saved_tensors=self.offload_residual, offload_master=self.offload_master, offload_optimizer=self.offload_optimizer,
                                  use_cuda_graphs=self.use_cuda_graphs, skip_quant_first_layers=self.skip_quant_first_layers,
                                  skip_quant_last_layers=self.skip_quant_last_layers, fp8_amax_history=self.fp8_amax_history,
                                  time_breakdown=self.trigger_timing_events, init_projections_to_zero=self.init_projections_to_zero)
        # options this engine does not have as switches: reported by the trainer as ``options_without_effect`` when set
        for name, on in (("offload_grads", self.offload_grads), ("offload_quants", self.offload_quants), ("attn_bwd_chunks", self.attn_bwd_chunks > 1),
                         ("no_fp4_stochastic_rounding", self.no_fp4_stochastic_rounding)):
            if on:
                kw[name] = True
        if self.gradient_type:
            kw["grad_dtype"] = DTYPES.get(self.gradient_type, self.gradient_type)
        if self.master_dtype:
            kw["master_dtype"] = DTYPES.get(self.master_dtype, self.master_dtype)
        return kw


@dataclass
class LoRAAdapterConfig:
    rank: int = 8
    alpha: float = 16.0
    dropout: float = 0.0
    target_modules: Sequence[str] = ("q_proj", "k_proj", "v_proj", "o_proj")
    dtype: str = "bf16"
    use_rslora: bool = False

    @property
    def scaling(self) -> float:
        return self.alpha / (self.rank ** 0.5 if self.use_rslora else self.rank)

    def applies_to(self, module_name: str) -> bool:
        return any(module_name.endswith(t) for t in self.target_modules)

    def as_dict(self) -> Dict[str, Any]:
        return dict(rank=self.rank, alpha=self.alpha, dropout=self.dropout, targets=list(self.target_modules), rslora=self.use_rslora)


@dataclass
class QLoRAConfig:
    enabled: bool = False
    strategy: str = "none"        # none | fp8 | nvfp4 | bnb
    block_size: int = 128
    base_dtype: str = ""
    adapter_dtype: str = "bf16"
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0

    STORAGE = {"fp8": "fp8_block", "nvfp4": "nvfp4", "fp4": "nvfp4", "bnb": "bnb_nf4", "nf4": "bnb_nf4"}

    @property
    def is_fp8(self) -> bool:
        return self.strategy == "fp8"

    @property
    def is_fp4(self) -> bool:
        return self.strategy in ("nvfp4", "fp4")

    @property
    def is_quantized(self) -> bool:
        return self.enabled and self.strategy != "none"

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0


# ---------------------------------------------------------------------- system information
@dataclass
class GPUInfo:
    device_id: int = 0
    name: str = ""
    total_memory: int = 0
    compute_capability_major: int = 0
    compute_capability_minor: int = 0


class SystemInfo:
    @staticmethod
    def get_cuda_runtime_version() -> int:
        import torch

        v = (torch.version.cuda or "0.0").split(".")
        return int(v[0]) * 1000 + int(v[1]) * 10

    @staticmethod
    def get_cuda_driver_version() -> int:
        try:
            from cuda.bindings import driver

            err, v = driver.cuDriverGetVersion()
            return int(v) if int(err) == 0 else 0
        except Exception:  # noqa: BLE001 - no driver on this machine
            return 0

    @staticmethod
    def get_nccl_version() -> int:
        import torch

        try:
            a, b, c = torch.cuda.nccl.version()
            return a * 10000 + b * 100 + c
        except Exception:  # noqa: BLE001
            return 0

    @staticmethod
    def get_cudnn_version() -> int:
        import torch

        return int(torch.backends.cudnn.version() or 0)

    @staticmethod
    def get_gpu_info() -> List[GPUInfo]:
        import torch

        out = []
        for i in range(torch.cuda.device_count() if torch.cuda.is_available() else 0):
            p = torch.cuda.get_device_properties(i)
            out.append(GPUInfo(i, p.name, p.total_memory, p.major, p.minor))
        return out


# ---------------------------------------------------------------------- data loader
class DataLoader:
    """Token shards -> ``[rows, seq_len]`` int32 batches written into caller-owned arrays.  ``chunk_size`` is the number of tokens
    per ``load_batch`` call (rows x seq_len); the row length is taken from the arrays passed to ``load_batch``."""

    def __init__(self, file_list: Sequence[str], chunk_size: int, seed: int = 42):
        from .data.tokfile import read_header

        self.files, self.chunk_size, self._seed = list(file_list), int(chunk_size), int(seed)
        self._headers = [read_header(f) for f in self.files]
        self._inner = None
        self._kd_k: Optional[int] = None
        self._kd = None
        self._pending_state = None

    def _ensure(self, rows: int, T: int):
        if self._inner is None:
            from .data.loader import DataLoader as Inner

            self._inner = Inner(self.files, rows, T, seed=self._seed, native=False if self._kd_k else None)
            if self._pending_state is not None:
                self._inner.load_state_dict(self._pending_state)
                self._pending_state = None
            if self._kd_k:
                from .data.loader import DistillationFeed

                self._kd = DistillationFeed(self._inner)
                if self._kd.K != self._kd_k:
                    raise ValueError(f"sidecars hold top-{self._kd.K}, expected top-{self._kd_k}")
        return self._inner

    def load_batch(self, inputs: np.ndarray, targets: np.ndarray, position_ids: Optional[np.ndarray] = None, kd_ids: Optional[np.ndarray] = None,
                   kd_logprobs: Optional[np.ndarray] = None) -> None:
        rows, T = inputs.shape
        if rows * T != self.chunk_size:
            raise ValueError(f"arrays hold {rows * T} tokens, the loader was created for chunks of {self.chunk_size}")
        x, y, p = self._ensure(rows, T).next_batch()
        inputs[...] = x
        targets[...] = y
        if position_ids is not None:
            position_ids[...] = p
        if kd_ids is not None or kd_logprobs is not None:
            if self._kd is None:
                raise RuntimeError("call enable_kd(k) before asking for teacher log-probabilities")
            ki, kl = self._kd.batch()
            if kd_ids is not None:
                kd_ids[...] = ki
            if kd_logprobs is not None:
                kd_logprobs[...] = kl

    def enable_kd(self, expected_k: int) -> None:
        if self._inner is not None:
            raise RuntimeError("enable_kd must be called before the first load_batch")
        self._kd_k = int(expected_k)

    def has_kd(self) -> bool:
        from .distill.sidecar import sidecar_path

        return all(os.path.exists(sidecar_path(f)) for f in self.files)

    def has_next(self, chunks: int = 1) -> bool:
        """The loader wraps around at the end of an epoch (``epoch`` then increases), so another batch is always available."""
        return True

    def advance_epoch(self) -> None:
        """Epochs advance by themselves when the last chunk has been served; kept for scripts that call it."""

    def set_state(self, seed: int, epoch: int, file_index: int, chunk_index: int) -> None:
        state = {"seed": seed, "epoch": epoch, "file_index": file_index, "chunk_index": chunk_index}
        if self._inner is None:
            self._seed, self._pending_state = int(seed), state
        else:
            self._inner.load_state_dict(state)

    @property
    def epoch(self) -> int:
        return 0 if self._inner is None else int(self._inner.epoch)

    @property
    def progress(self) -> float:
        inner = self._inner
        if inner is None:
            return 0.0
        st = inner.state_dict()
        return 100.0 * min(1.0, (st.get("file_index", 0) + 0.0) / max(1, len(self.files)))

    @property
    def num_files(self) -> int:
        return len(self.files)

    @property
    def num_tokens(self) -> int:
        return int(sum(h["n_tokens"] for h in self._headers))

    @property
    def num_chunks(self) -> int:
        return self.num_tokens // max(1, self.chunk_size)

    @property
    def seed(self) -> int:
        return self._seed

    @property
    def vocab_size(self) -> int:
        return int(self._headers[0]["vocab"]) if self._headers else 0

    @property
    def seq_len(self) -> int:
        return 0 if self._inner is None else int(self._inner.T)


# ---------------------------------------------------------------------- trainer
class SurogateTrainer:
    def __init__(self, ngpu: int, config: PretrainedConfig, options: RuntimeOptions, batch_size: int, seq_len: int, grad_accum: int,
                 memcpy_all_gather: bool = True, memcpy_send_recv: bool = True, lora_config: Optional[LoRAAdapterConfig] = None,
                 qlora_config: Optional[QLoRAConfig] = None, device=None, backend: Optional[str] = None, optimizer: str = "adamw_8bit"):
        import torch

        from .parallel.dist import TorchComm, init_distributed
        from .runtime.trainer import Trainer, TrainerConfig

        info = init_distributed() if int(os.environ.get("WORLD_SIZE", "1")) > 1 else None
        world = info.world if info is not None else 1
        if ngpu != world:
            raise ValueError(f"ngpu={ngpu}, but this script runs as {world} process(es): one process drives one GPU here, start it with "
                             f"`torchrun --nproc-per-node {ngpu} <script>`")
        kw = options.trainer_kwargs()
        if backend:
            kw["backend"] = backend
        if lora_config is not None:
            kw["lora"] = lora_config.as_dict()
        if qlora_config is not None and qlora_config.is_quantized:
            kw.update(qlora=QLoRAConfig.STORAGE[qlora_config.strategy], qlora_block_size=qlora_config.block_size)
        known = set(TrainerConfig.__dataclass_fields__)
        dropped = sorted(k for k in kw if k not in known)
        cfg = TrainerConfig(model=config.to_hf_dict(), batch_size=batch_size, seq_len=seq_len, grad_accum=grad_accum, optimizer=optimizer,
                            param_dtype=DTYPES.get(config.dtype, config.dtype), **{k: v for k, v in kw.items() if k in known})
        self.options_without_effect = dropped
        if device is None:
            device = torch.device("cuda", info.local_rank if info is not None else 0) if torch.cuda.is_available() else torch.device("cpu")
        self.trainer = Trainer(cfg, device=device, comm=TorchComm() if world > 1 else None)
        self.config, self.options = config, options
        self._B, self._T, self._GA, self._world, self._rank = batch_size, seq_len, grad_accum, world, (info.rank if info is not None else 0)
        self._queue: List[Dict[str, Any]] = []
        self._kd_loss = 0.0
        self._initialised = False

    @classmethod
    def from_pretrained(cls, name: str, ngpu: int, dtype: str, options: RuntimeOptions, batch_size: int, seq_len: int, grad_accum: int,
                        memcpy_all_gather: bool = True, memcpy_send_recv: bool = True, lora_config: Optional[LoRAAdapterConfig] = None,
                        qlora_config: Optional[QLoRAConfig] = None, **kw) -> "SurogateTrainer":
        from .hub import download_model

        path = name if os.path.exists(name) else download_model(name)
        t = cls(ngpu, PretrainedConfig.from_pretrained(path, dtype), options, batch_size, seq_len, grad_accum, memcpy_all_gather, memcpy_send_recv,
                lora_config, qlora_config, **kw)
        t.import_weights(path)
        return t

    # -- properties
    @property
    def batch_size(self) -> int:
        return self._B

    @property
    def seq_length(self) -> int:
        return self._T

    @property
    def world_size(self) -> int:
        return self._world

    # -- weights and checkpoints
    def init_weights(self) -> None:
        self.trainer.init_weights(0)
        self._initialised = True

    def import_weights(self, path: str) -> None:
        self.trainer.import_weights(path if os.path.isdir(path) else os.path.dirname(path))
        if self.trainer.lora is not None:
            self.trainer.lora.init_weights(0)
        self._initialised = True

    def import_adapter(self, file_name: str) -> None:
        from .train.adapter_init import apply_adapter_init

        apply_adapter_init(self.trainer, file_name if os.path.isdir(file_name) else os.path.dirname(file_name), "resume", "")

    def export_model(self, path: str) -> None:
        self.trainer.export_model(path, self.config.to_hf_dict())

    def export_adapter(self, path: str, base_model_path: str = "") -> None:
        self.trainer.export_adapter(path, base_model=base_model_path)

    def save_checkpoint(self, path: str, step: int) -> None:
        self.trainer.save_checkpoint(path, step)

    def load_checkpoint(self, path: str, step: int) -> None:
        self.trainer.load_checkpoint(path, step)

    # -- micro-steps
    def _mine(self, a: Optional[np.ndarray]) -> Optional[np.ndarray]:
        """This rank's rows of a ``[batch_size * ngpu, ...]`` array (arrays that already hold ``batch_size`` rows pass through)."""
        if a is None:
            return None
        a = np.asarray(a)
        if a.shape[0] == self._B * self._world and self._world > 1:
            return a[self._rank * self._B:(self._rank + 1) * self._B]
        if a.shape[0] != self._B:
            raise ValueError(f"expected {self._B * self._world} (or {self._B}) rows, got {a.shape[0]}")
        return a

    def _push(self, **item) -> None:
        if len(self._queue) >= self._GA:
            raise RuntimeError(f"{self._GA} micro-steps are queued already: call update_with_config() before the next step()")
        self._queue.append({k: (np.array(self._mine(v), copy=True) if isinstance(v, np.ndarray) else v) for k, v in item.items()})

    def step(self, inputs: np.ndarray, targets: np.ndarray, position_ids: Optional[np.ndarray] = None) -> None:
        self._push(inputs=inputs, targets=targets, position_ids=position_ids)

    def step_with_custom_loss(self, input_ids: np.ndarray, targets: np.ndarray, per_token_grads: np.ndarray, position_ids: Optional[np.ndarray] = None,
                              temperatures: Optional[np.ndarray] = None) -> None:
        if temperatures is not None and not np.allclose(temperatures, 1.0):
            raise NotImplementedError("per-token temperatures other than 1 are not supported")
        self._push(inputs=input_ids, targets=targets, position_ids=position_ids, weights=per_token_grads)

    def step_with_kd(self, input_ids: np.ndarray, targets: np.ndarray, kd_ids: np.ndarray, kd_logprobs: np.ndarray, position_ids: Optional[np.ndarray] = None,
                     top_k: int = 32, temperature: float = 1.0, kd_weight: float = 0.5, ce_weight: float = 0.5) -> None:
        self._push(inputs=input_ids, targets=targets, position_ids=position_ids, kd_ids=kd_ids, kd_logprobs=kd_logprobs,
                   kd=dict(weight=kd_weight, ce_weight=ce_weight, temperature=temperature))

    def update_with_config(self, config: OptimizerConfig, step: int) -> Dict[str, float]:
        """Run the queued micro-steps (forward + backward each), reduce, clip and update.  Returns ``{"loss", "norm"}``."""
        if len(self._queue) != self._GA:
            raise RuntimeError(f"{len(self._queue)} micro-steps queued, grad_accum is {self._GA}")
        q, self._queue = self._queue, []
        cat = lambda k: np.concatenate([m[k] for m in q]) if all(m.get(k) is not None for m in q) else None  # noqa: E731
        x, y, pos = cat("inputs"), cat("targets"), cat("position_ids")
        weights = cat("weights") if any("weights" in m for m in q) else None
        kd = None
        if any("kd" in m for m in q):
            kd = dict(q[0]["kd"], idx=cat("kd_ids"), logp=cat("kd_logprobs"))
            kd.pop("temperature", None)
        t = self.trainer
        opt = dict(asdict(config), max_grad_norm=config.grad_clip, beta1=config.adamw_beta1, beta2=config.adamw_beta2, eps=config.adamw_epsilon)
        if weights is not None:  # the caller's multipliers are the whole objective: no division by the token count
            res = t.forward_backward(x, y, pos, row_weights=weights, loss_scale_override=1.0)
        else:
            res = t.forward_backward(x, y, pos, kd=kd)
        out = t.update_with_config(opt, step)
        n = float(res["n_valid"]) if hasattr(res["n_valid"], "item") else float(res["n_valid"])
        out["loss"] = float(res["loss_sum"]) / max(1.0, n) if weights is None else float(res["loss_sum"])
        if kd is not None:
            self._kd_loss = out["loss"]
        return out

    def train_step_graphed(self, inputs: np.ndarray, targets: np.ndarray, config: OptimizerConfig, step: int, position_ids: Optional[np.ndarray] = None) -> Dict[str, float]:
        """All ``grad_accum`` micro-batches (``[grad_accum * batch_size * ngpu, T]`` arrays, micro-batch major) and the update in one call."""
        B, GA, W = self._B, self._GA, self._world
        for i in range(GA):
            sl = slice(i * B * W, (i + 1) * B * W)
            self.step(inputs[sl], targets[sl], None if position_ids is None else position_ids[sl])
        return self.update_with_config(config, step)

    def get_kd_loss(self) -> float:
        v, self._kd_loss = self._kd_loss, 0.0
        return v

    # -- evaluation and inspection
    def validate(self, inputs: np.ndarray, targets: np.ndarray, position_ids: Optional[np.ndarray] = None) -> float:
        return float(self.trainer.validate(self._mine(inputs), self._mine(targets), self._mine(position_ids))["loss"])

    def compute_logprobs(self, input_ids: np.ndarray, targets: np.ndarray, use_lora: bool = True, position_ids: Optional[np.ndarray] = None,
                         temperatures: Optional[np.ndarray] = None) -> np.ndarray:
        if temperatures is not None and not np.allclose(temperatures, 1.0):
            raise NotImplementedError("per-token temperatures other than 1 are not supported")
        return self.trainer.token_logprobs(np.asarray(input_ids), np.asarray(targets), None if position_ids is None else np.asarray(position_ids),
                                           use_adapters=use_lora).float().cpu().numpy()

    def get_gradients(self, gpu_id: int = 0) -> Dict[str, Any]:
        return self.trainer.get_gradients()

    def get_lora_gradients(self, gpu_id: int = 0) -> Dict[str, Any]:
        lora = self.trainer.lora
        return {} if lora is None else {name: g.detach().clone() for name, g in lora.named_grads()}

    def get_allocator_info(self, gpu_id: int = 0) -> Dict[str, int]:
        return dict(self.trainer.memory_breakdown())

    def get_gpu_info(self) -> List[Dict[str, Any]]:
        return [self.trainer.get_gpu_info()]
