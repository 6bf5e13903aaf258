"""SFT / pre-training workflow: config -> token shards -> Trainer -> step loop with schedule, logging,
evaluation, checkpoints, monitors and out-of-memory recovery.

Parity: surogate/train/sft.py (SurogateSFT.run :20, train_with_oom_recovery :97-172), train/pt.py:13-21,
train/trainer.py (run_training_loop :1160-1553).
"""
from __future__ import annotations

import contextlib
import glob
import json
import math
import os
import time
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from ..config.sft_config import PTConfig, SFTConfig
from ..data.loader import DataLoader, write_synthetic_tokens
from ..dsl.compiler import load_hf_config
from ..io.checkpoint import clean_old_checkpoints, find_latest_checkpoint
from ..parallel.dist import TorchComm, init_distributed
from ..runtime.trainer import Trainer
from ..utils.sol import speed_of_light_fraction, transformer_flops_per_token
from .logging import TrainingRunLogger, resolve_metrics_path
from .lr_schedule import LRSchedule
from .monitors import EarlyStopping, GradientTracker, LossGuard, MoEMonitor, PhaseDetector, TrainingAdvisor


def resolve_model_config(cfg: SFTConfig) -> Dict[str, Any]:
    """``model`` may be a directory with config.json, a config.json path, or inline JSON (``{"architecture": ...}``)."""
    m = cfg.model
    if isinstance(m, dict):
        return dict(m)
    if m.strip().startswith("{"):
        return json.loads(m)
    from ..models.presets import is_preset, preset_config

    if is_preset(m):   # ``model: preset:qwen3-8b``: the architecture by name, no weights (from_scratch runs, planning)
        return preset_config(m)
    if os.path.exists(m):
        return load_hf_config(m)
    from ..hub import download_model

    return load_hf_config(download_model(m))


def prepare_data(cfg: SFTConfig, hf_cfg: Dict[str, Any], rank: int, comm=None) -> Dict[str, List[str]]:
    """Token shards for training / evaluation (tokenises datasets on first use, cached by content hash)."""
    out = os.path.join(cfg.output_dir, "tokens")
    vocab = hf_cfg.get("vocab_size", 151936)
    if cfg.synthetic_data or not cfg.datasets:
        rows = max(64, cfg.per_device_train_batch_size * cfg.gradient_accumulation_steps * cfg.gpus * 8)
        train = os.path.join(out, "train-000.bin")
        ev = os.path.join(out, "eval.bin")
        if rank == 0 and not os.path.exists(train):
            write_synthetic_tokens(train, rows, cfg.sequence_len, vocab, seed=cfg.train_seed)
            write_synthetic_tokens(ev, max(8, rows // 8), cfg.sequence_len, vocab, seed=cfg.eval_seed)
        return {"train": [train], "eval": [ev]}
    from .tokenize import TokenizeDatasets

    job = TokenizeDatasets(cfg, hf_cfg, out)
    if rank == 0:
        files = job.run(write=True)
    if comm is not None:
        comm.barrier()  # the shards and their manifest are on disk
    if rank != 0:
        files = job.run(write=False)
    return files


class SurogateSFT:
    config_cls = SFTConfig

    def __init__(self, cfg: SFTConfig):
        self.cfg = cfg

    def run(self) -> Dict[str, Any]:
        cfg = self.cfg
        if cfg.distributed is not None and cfg.distributed.num_nodes > 1:
            from .distributed import run_multinode

            return run_multinode(cfg, type(self), command="pt" if isinstance(self, SurogatePT) else "sft", config_path=getattr(cfg, "_config_path", None))
        return train_with_oom_recovery(cfg)


class SurogatePT(SurogateSFT):
    config_cls = PTConfig


def train_with_oom_recovery(cfg: SFTConfig, max_retries: int = 3) -> Dict[str, Any]:
    """On a CUDA out-of-memory error halve the micro-batch and double gradient accumulation (same global batch)."""
    attempt = 0
    while True:
        try:
            return run_training(cfg)
        except torch.cuda.OutOfMemoryError as e:  # pragma: no cover - needs a GPU
            attempt += 1
            if attempt > max_retries or cfg.per_device_train_batch_size <= 1:
                raise
            cfg.per_device_train_batch_size = max(1, cfg.per_device_train_batch_size // 2)
            cfg.gradient_accumulation_steps *= 2
            torch.cuda.empty_cache()
            print(f"[oom] retrying with per_device_train_batch_size={cfg.per_device_train_batch_size}, "
                  f"gradient_accumulation_steps={cfg.gradient_accumulation_steps} ({e})")


def run_training(cfg: SFTConfig) -> Dict[str, Any]:
    info = init_distributed()
    comm = TorchComm() if info.world > 1 else None
    device = torch.device("cuda", info.local_rank) if torch.cuda.is_available() else torch.device("cpu")
    hf_cfg = resolve_model_config(cfg)
    if cfg.router_aux_loss_coef is not None:
        hf_cfg["router_aux_loss_coef"] = cfg.router_aux_loss_coef
    files = prepare_data(cfg, hf_cfg, info.rank, comm) if not cfg.train_vision else {}
    if comm is not None:
        comm.barrier()
    tcfg = cfg.to_trainer_config(hf_cfg)
    pp = cfg.parallelism == "dispatch_pp" and info.world > 1
    if pp:  # pipeline stages: layer ranges per rank, micro-batches in a wavefront, boundaries sent GPU to GPU
        from ..parallel.dispatch_pp import PipelineTrainer

        tcfg.zero_level = 0
        trainer = PipelineTrainer(tcfg, device=device, stage_layers=int(cfg.dispatch_pp.get("stage_layers", cfg.dispatch_pp.get("stage_blocks", 0)) or 0))
    else:
        trainer = Trainer(tcfg, device=device, comm=comm)
    logger = TrainingRunLogger(cfg.log_file, resolve_metrics_path(cfg.surogate_metrics_path) if "surogate" in cfg.report_to else None, is_main=info.is_main)
    logger.log_record("options", config=json.loads(cfg.to_json()))

    B, GA, T = cfg.per_device_train_batch_size, cfg.gradient_accumulation_steps, cfg.sequence_len
    distill = cfg.distillation if (cfg.distillation is not None and cfg.distillation.enabled) else None
    if cfg.train_vision:
        if distill or cfg.sample_packing:
            raise ValueError("train_vision builds batches on the fly: it cannot be combined with distillation sidecars or sample packing")
        loader = _vision_loader(cfg, hf_cfg, trainer, info, device, B * GA, T)
    else:
        # pipeline stages: every rank reads the same rows (world * GA micro-batches of B); only the end stages use them
        loader = DataLoader(files["train"], B * GA * (info.world if pp else 1), T, seed=cfg.train_seed, rank=0 if pp else info.rank,
                            world=1 if pp else info.world, native=False if distill else None)
    kd_feed = None
    if distill:
        from ..data.loader import DistillationFeed

        kd_feed = DistillationFeed(loader, distill.sidecar_dir)  # needs train-NNN.kd for every shard (surogate distill-capture)
    eval_loader = DataLoader(files["eval"], B, T, seed=cfg.eval_seed, rank=0 if pp else info.rank, world=1 if pp else info.world,
                             shuffle=False) if files.get("eval") else None
    steps_per_epoch = max(1, loader.steps_per_epoch())
    max_steps = cfg.max_steps if cfg.max_steps > 0 else steps_per_epoch * cfg.num_epochs
    warmup = cfg.warmup_steps or int(cfg.warmup_ratio * max_steps)
    sched = LRSchedule(cfg.learning_rate, max_steps, warmup, cfg.cooldown_steps, cfg.final_lr_fraction * cfg.learning_rate,
                       cfg.lr_scheduler_type, cfg.wsd_decay_steps_fraction)

    start_step = 0
    model_dir = cfg.model if isinstance(cfg.model, str) and os.path.isdir(cfg.model) else None
    latest = (trainer.latest_checkpoint(cfg.checkpoint_dir) if pp else find_latest_checkpoint(cfg.checkpoint_dir)) if cfg.resume_from_checkpoint else None
    if latest is not None:
        if getattr(trainer, "lora", None) is not None:  # adapter-only checkpoints: the frozen base comes from its source again
            if cfg.from_scratch or model_dir is None or not glob.glob(os.path.join(model_dir, "*.safetensors")):
                trainer.init_weights(cfg.train_seed)
            else:
                trainer.import_weights(model_dir)
        meta = trainer.load_checkpoint(cfg.checkpoint_dir, latest)
        start_step = meta["run"]["step"]
        if meta.get("data-loader"):
            loader.load_state_dict(meta["data-loader"])
        logger.message(f"resumed from {cfg.checkpoint_dir}/step_{latest:08d}")
    elif cfg.from_scratch or model_dir is None or not glob.glob(os.path.join(model_dir, "*.safetensors")):
        trainer.init_weights(cfg.train_seed)
    else:
        trainer.import_weights(model_dir)
        if trainer.lora is not None:
            trainer.lora.init_weights(cfg.train_seed)
    if cfg.adapter_path and trainer.lora is not None and latest is None:
        from .adapter_init import apply_adapter_init

        logger.message(f"adapter {cfg.adapter_path}: {apply_adapter_init(trainer, cfg.adapter_path, cfg.adapter_init_mode, cfg.output_dir)}")
    from .reporter import make_reporters

    reporters = make_reporters([r for r in cfg.report_to if r != "surogate"], cfg.run_name, config=json.loads(cfg.to_json())) if info.is_main else []

    flops = transformer_flops_per_token(
        d_model=hf_cfg.get("hidden_size", hf_cfg.get("d_model", 0)), n_layers=hf_cfg.get("num_hidden_layers", hf_cfg.get("n_layers", 0)),
        n_q_heads=hf_cfg.get("num_attention_heads", hf_cfg.get("num_query_heads", 1)),
        n_kv_heads=hf_cfg.get("num_key_value_heads", hf_cfg.get("num_kv_heads", 1)), head_dim=hf_cfg.get("head_dim", hf_cfg.get("head_size", 128)),
        d_ff=hf_cfg.get("intermediate_size", hf_cfg.get("d_ff", 0)), vocab=hf_cfg.get("vocab_size", 0), seq_len=T,
        num_experts_per_tok=hf_cfg.get("num_experts_per_tok", 0) if hf_cfg.get("num_experts") else 0,
        moe_d_ff=hf_cfg.get("moe_intermediate_size", hf_cfg.get("moe_d_ff", 0)), num_experts=hf_cfg.get("num_experts", 0),
        lora_rank=cfg.lora_rank if cfg.lora else 0, recompute=cfg.recompute)
    dev_name = torch.cuda.get_device_name(device) if device.type == "cuda" else "cpu"
    losses: List[float] = []
    norms: List[float] = []
    from ..parallel.watchdog import RemoteRankFailed, install as install_watchdog

    # failure detection: heartbeats + root-cause notes between ranks; a failed or silent peer ends this rank at its next step
    watchdog = install_watchdog(info.rank, info.world) if info.world > 1 and os.environ.get("SUROGATE_WATCHDOG", "1") != "0" else None
    try:
        last = _run_steps(cfg, trainer, logger, loader, eval_loader, sched, watchdog, info, hf_cfg, device, start_step, max_steps, steps_per_epoch, warmup,
                          flops, dev_name, kd_feed, distill, reporters, losses, norms)
    except BaseException as e:  # noqa: BLE001
        if watchdog is not None and not isinstance(e, RemoteRankFailed):
            watchdog.report_failure(e)  # the other ranks learn why the job ended
        raise
    finally:
        if watchdog is not None:
            watchdog.stop()
    # final artefacts: adapter (LoRA) or full model in HF format (with the tokenizer files of the source model)
    if isinstance(cfg.model, str) and not cfg.model.strip().startswith("{"):
        try:
            from ..hub import download_model

            trainer.tokenizer_source = cfg.model if os.path.isdir(cfg.model) else download_model(cfg.model)
        except Exception:  # noqa: BLE001 - no local copy of the model: the export carries weights and config only
            pass
    if trainer.lora is not None:
        trainer.export_adapter(os.path.join(cfg.output_dir, "adapter"), base_model=cfg.model if isinstance(cfg.model, str) else "")
        if cfg.merge_adapter:
            trainer.lora.merge_into(trainer.store)
            trainer.export_model(os.path.join(cfg.output_dir, "merged"), hf_cfg)
    else:
        trainer.export_model(cfg.output_dir, hf_cfg)
    for rep in reporters:
        rep.finish()
    logger.close()
    return {"final": last, "losses": losses, "norms": norms, "steps": len(losses)}


def _vision_loader(cfg, hf_cfg, trainer, info, device, rows_per_step: int, seq_len: int):
    """Multimodal rows of this rank (``rank::world``) -> on-the-fly batches through the frozen vision tower."""
    from . import vision

    paths = [d.path for d in cfg.datasets]
    rows = vision.load_multimodal_rows(paths)[info.rank::info.world]
    if not rows:
        raise ValueError(f"train_vision: no rows for rank {info.rank} in {paths}")
    _, enc, tower = vision.init_mm_helpers(cfg.model, device)
    batcher = vision.OnTheFlyMultimodalBatcher(rows, enc.encode, tower, rows_per_step, seq_len, image_token_id=hf_cfg["image_token_id"],
                                               video_token_id=hf_cfg.get("video_token_id"), pad_token_id=int(hf_cfg.get("pad_token_id") or 0))
    return vision.VisionTrainLoader(batcher, trainer)


def _run_steps(cfg, trainer, logger, loader, eval_loader, sched, watchdog, info, hf_cfg, device, start_step, max_steps, steps_per_epoch, warmup, flops, dev_name,
               kd_feed, distill, reporters, losses, norms) -> Dict[str, Any]:
    """The optimizer-step loop of a run: data, step, monitors, logging, evaluation, checkpoints.  Returns the last step's result."""
    B, GA, T = cfg.per_device_train_batch_size, cfg.gradient_accumulation_steps, cfg.sequence_len
    guard = LossGuard(enabled=cfg.auto_lr_reduction)
    phase_det, grads, moe_mon, advisor = PhaseDetector(warmup), GradientTracker(), MoEMonitor(), TrainingAdvisor()
    stopper = EarlyStopping(cfg.early_stop)
    step_tokens = B * GA * T * info.world
    last: Dict[str, Any] = {}
    from ..regression.artifact import RunArtifact

    artifact = RunArtifact.from_env() if info.is_main else None  # SUROGATE_REGRESSION_ARTIFACT: curve + timings + plan summary of this run
    for step in range(start_step, max_steps):
        t0 = time.perf_counter()
        if watchdog is not None:
            watchdog.tick(step)
            watchdog.check()  # a failed / silent peer ends the run here, before this step's first collective
        x, y, p = loader.next_batch()
        if cfg.loss_scale == "all":
            pass  # every token is a target (pre-training); masks in the shard are already all ones
        lr = sched.get_lr(step)
        kd = None
        if kd_feed is not None:
            ki, kl = kd_feed.batch()
            kd = {"idx": ki, "logp": kl, "weight": distill.kd_weight, "ce_weight": distill.ce_weight}
        out = trainer.step(x, y, p if (cfg.sample_packing or cfg.train_vision) else None, lr=lr, kd=kd)
        ms = (time.perf_counter() - t0) * 1e3
        if cfg.debug_time_breakdown and getattr(trainer, "last_time_breakdown", None):
            logger.log_record("timing", step=step + 1, **{k: round(v, 3) for k, v in trainer.last_time_breakdown.items()})
        if cfg.debug_memory_breakdown and step == start_step and hasattr(trainer, "memory_breakdown"):
            mem = dict(trainer.memory_breakdown())
            if device.type == "cuda":
                mem.update(cuda_allocated=int(torch.cuda.memory_allocated(device)), cuda_reserved=int(torch.cuda.memory_reserved(device)),
                           cuda_peak=int(torch.cuda.max_memory_allocated(device)))
            logger.log_record("memory", step=step + 1, **mem)
        losses.append(out["loss"])
        norms.append(out["norm"])
        if artifact is not None:
            artifact.add(step + 1, out["loss"], out["norm"], lr, ms, int(torch.cuda.max_memory_allocated(device)) if device.type == "cuda" else None)
        phase = phase_det.update(step, out["loss"])
        gstat = grads.update(out["norm"])
        act = guard.check(out["loss"], out["norm"])
        if act.kind == "override":
            sched.override_lr(lr * act.factor, step, act.grace)
            logger.message(f"[loss-guard] {act.reason}: LR x{act.factor} for {act.grace} steps")
        elif act.kind == "reduce":
            sched.reduce_lr(act.factor)
            logger.message(f"[loss-guard] {act.reason}: LR permanently x{act.factor}")
        elif act.kind == "abort":
            logger.message(f"[loss-guard] {act.reason}: stopping")
            break
        if (step + 1) % cfg.logging_steps == 0:
            tps = 1000.0 * step_tokens / ms
            sol = speed_of_light_fraction(flops, tps, dev_name, cfg.recipe, info.world) if flops["total"] else None
            logger.log_step(step + 1, max_steps, (step + 1) / steps_per_epoch, out["loss"], out["norm"], lr, step_tokens, ms, sol, phase)
            for rep in reporters:
                rep.log(step + 1, {"loss": out["loss"], "norm": out["norm"], "lr": lr, "tps": tps, "ms": ms})
        if trainer.last_moe_stats:
            stats = trainer.get_moe_stats()
            if (step + 1) % max(1, cfg.logging_steps) == 0:
                logger.log_record("moe", step=step + 1, aux_loss=out.get("aux_loss", 0.0), **stats)
            for w in moe_mon.check(stats):
                logger.message(f"[moe] {w}")
        if cfg.log_gpu_util and (step + 1) % cfg.log_gpu_util == 0 and device.type == "cuda":
            logger.log_record("gpu", step=step + 1, **trainer.get_gpu_info())
        for tip in advisor.advise(phase, gstat, []) if (step + 1) % 100 == 0 else []:
            logger.message(f"[advisor] {tip}")
        if eval_loader is not None and cfg.eval_steps > 0 and (step + 1) % cfg.eval_steps == 0:
            ex, ey, _ = eval_loader.next_batch()
            logger.log_eval(step + 1, trainer.validate(ex, ey)["loss"])
        if cfg.save_steps > 0 and (step + 1) % cfg.save_steps == 0 and step + 1 < max_steps:
            try:
                trainer.save_checkpoint(cfg.checkpoint_dir, step + 1, {"data_loader": loader.state_dict(), "past_losses": losses[-32:],
                                                                       "past_norms": norms[-32:]})
                if info.is_main:
                    clean_old_checkpoints(cfg.checkpoint_dir, cfg.save_total_limit)
            except OSError as e:  # a failed save must not kill the run; save_checkpoint raises on every rank together
                logger.message(f"[checkpoint] save failed: {e}")
        last = out
        if stopper.should_stop(out["loss"], phase):
            logger.message("[early-stop] stopping")
            break
    if artifact is not None:
        logger.message(f"[regression] artifact written to {artifact.write(trainer)}")
    return last


def sft_main(config_path: str, **overrides):
    from ..config.loader import load_config

    cfg = load_config(SFTConfig, config_path, **overrides)
    cfg._config_path = config_path
    return SurogateSFT(cfg).run()


def pt_main(config_path: str, **overrides):
    from ..config.loader import load_config

    cfg = load_config(PTConfig, config_path, **overrides)
    cfg._config_path = config_path
    return SurogatePT(cfg).run()
