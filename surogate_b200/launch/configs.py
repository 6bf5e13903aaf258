"""A training config from a handful of launch fields, and the overlays a launcher appends to a user's own config.

``build_config`` returns the config as YAML text whose keys are the SFT config's own, so what the launcher writes is an ordinary
config file a user can keep and re-run by hand.  Overlays are appended as a second YAML document section of plain ``key: value``
lines: the loader keeps the last value of a repeated key, so the user's file is otherwise run exactly as written.

Parity: jackalope/src/launch.ts (LaunchFields, buildConfigYaml, overlayExistingSft, buildResumeYaml, buildCommand).
"""
from __future__ import annotations

import json
import shlex
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import yaml

RECIPES = ("bf16", "fp8-hybrid", "nvfp4")
OPTIMIZERS = ("adamw_8bit", "adamw", "normuon")
LR_SCHEDULERS = ("linear", "cosine", "constant", "wsd")
DEFAULT_TARGET_MODULES = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


@dataclass
class LaunchFields:
    model: str = ""
    dataset_path: str = ""
    dataset_type: str = "auto"
    recipe: str = "fp8-hybrid"
    max_steps: int = 200
    learning_rate: float = 2e-4
    per_device_batch: int = 2
    grad_accum: int = 4
    sequence_len: int = 2048
    eval_steps: int = 25
    warmup_ratio: float = 0.15
    recompute: bool = True
    optimizer: str = "adamw_8bit"
    lr_scheduler: str = "linear"
    weight_decay: float = 0.0
    max_grad_norm: float = 1.0
    lora: bool = True
    lora_rank: int = 16
    lora_alpha: int = 32
    lora_target_modules: List[str] = field(default_factory=lambda: list(DEFAULT_TARGET_MODULES))
    save_steps: int = 50
    save_total_limit: int = 5
    resume_from_checkpoint: bool = False
    merge_adapter: bool = False
    output_dir: str = "./watch-out"

    def problems(self) -> List[str]:
        out = []
        if not self.model:
            out.append("no model picked")
        if not self.dataset_path:
            out.append("no dataset picked")
        if self.recipe not in RECIPES:
            out.append(f"recipe must be one of {RECIPES}")
        if self.optimizer not in OPTIMIZERS:
            out.append(f"optimizer must be one of {OPTIMIZERS}")
        if self.lr_scheduler not in LR_SCHEDULERS:
            out.append(f"lr_scheduler must be one of {LR_SCHEDULERS}")
        for k in ("max_steps", "per_device_batch", "grad_accum", "sequence_len"):
            if int(getattr(self, k)) < 1:
                out.append(f"{k} must be at least 1")
        return out


def config_dict(f: LaunchFields, n_gpus: int = 1, metrics_path: Optional[str] = None) -> Dict[str, Any]:
    cfg: Dict[str, Any] = {
        "model": f.model, "output_dir": f.output_dir, "gpus": max(1, n_gpus), "recipe": f.recipe,
        "per_device_train_batch_size": f.per_device_batch, "gradient_accumulation_steps": f.grad_accum, "sequence_len": f.sequence_len,
        "sample_packing": True, "max_steps": f.max_steps, "eval_steps": f.eval_steps, "learning_rate": f.learning_rate,
        "warmup_ratio": f.warmup_ratio, "optimizer": f.optimizer, "lr_scheduler_type": f.lr_scheduler, "weight_decay": f.weight_decay,
        "max_grad_norm": f.max_grad_norm, "recompute": f.recompute, "save_steps": f.save_steps, "save_total_limit": f.save_total_limit,
        "resume_from_checkpoint": f.resume_from_checkpoint, "lora": f.lora,
    }
    if f.lora:
        cfg.update(lora_rank=f.lora_rank, lora_alpha=f.lora_alpha, lora_target_modules=list(f.lora_target_modules))
    if f.merge_adapter:
        cfg["merge_adapter"] = True
    cfg.update(logging_steps=1, log_gpu_util=5, report_to=["surogate"])  # live monitoring
    if metrics_path:
        cfg["surogate_metrics_path"] = metrics_path
    cfg["datasets"] = [{"path": f.dataset_path, "type": f.dataset_type}]
    return cfg


def build_config(f: LaunchFields, n_gpus: int = 1, metrics_path: Optional[str] = None) -> str:
    return yaml.safe_dump(config_dict(f, n_gpus, metrics_path), sort_keys=False, default_flow_style=False)


def _overlay(base: str, title: str, values: Dict[str, Any]) -> str:
    lines = [f"# --- {title} (overrides the above) ---"] + [f"{k}: {json.dumps(v)}" for k, v in values.items()]  # JSON scalars are YAML
    return base.rstrip() + "\n" + "\n".join(lines) + "\n"


def monitoring_overlay(base_yaml: str, n_gpus: int, metrics_path: str) -> str:
    """A user's own config with the GPU count and the feed of this run appended."""
    return _overlay(base_yaml, "monitoring overlay", {"gpus": max(1, n_gpus), "report_to": ["surogate"], "surogate_metrics_path": metrics_path})


def resume_overlay(base_yaml: str, metrics_path: str) -> str:
    """A previous run's config set to continue from its newest checkpoint (its ``output_dir`` already points there) with a
    fresh feed."""
    return _overlay(base_yaml, "resume overlay", {"resume_from_checkpoint": True, "report_to": ["surogate"], "surogate_metrics_path": metrics_path})


def load_overlaid(text: str) -> Dict[str, Any]:
    """Parse a config with overlays (the YAML loader keeps the last value of a repeated top-level key)."""
    return yaml.safe_load(text) or {}


def build_command(gpu_ids: Sequence[int], config_path: str, mode: str = "sft", surogate_bin: str = "surogate") -> str:
    """The shell line that starts the run (shown as a preview and sent to remote shells)."""
    prefix = f"CUDA_VISIBLE_DEVICES={','.join(str(g) for g in gpu_ids)} " if gpu_ids else ""
    return f"{prefix}{surogate_bin} {mode} {shlex.quote(config_path)}"
