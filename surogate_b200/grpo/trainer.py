"""GRPO trainer: consumes packed rollout batches, takes one clipped-policy-gradient step per batch, publishes weights.

Step: (1) current-policy token log-probs (no-grad forward); (2) reference log-probs with adapters disabled when a KL
term is configured; (3) per-token weights from ``grpo/loss.py``; (4) forward+backward where the fused LM-head loss kernel
scales each token's log-likelihood gradient by its weight; (5) clip + optimizer; (6) every ``broadcast_every`` steps the
new policy is published and the version counter advances.

Parity: surogate/grpo/trainer.py, surogate/grpo/loss.py.
"""
from __future__ import annotations

import os
import time
from typing import Any, Dict, Optional

import numpy as np
import torch

from ..runtime.trainer import Trainer
from .config import GRPOConfig, GRPOLossConfig
from .loss import grpo_token_weights, ipo_token_weights


class GRPOTrainer:
    def __init__(self, trainer: Trainer, loss: Optional[GRPOLossConfig] = None):
        self.t = trainer
        self.loss = loss or GRPOLossConfig()
        self.policy_version = 0
        self.turn_diagnostics = False

    def _slice(self, a: np.ndarray) -> np.ndarray:
        t = self.t
        rows = t.cfg.batch_size * t.cfg.grad_accum
        if a.shape[0] == rows * t.world and t.world > 1:
            return a[t.rank * rows:(t.rank + 1) * rows]
        assert a.shape[0] == rows, f"batch has {a.shape[0]} rows, expected {rows} per rank"
        return a

    def fit_rows(self, batch: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
        """A batch with any number of rows: padded with empty rows (no targets, zero advantage) to a multiple of
        ``batch_size x ranks``, and the number of micro-batches of this step set from it."""
        t = self.t
        unit = t.cfg.batch_size * t.world
        n = batch["inputs"].shape[0]
        padded = -(-n // unit) * unit
        if padded != n:
            fill = {"targets": -100, "seq_ids": -1}
            batch = {k: (np.concatenate([v, np.full((padded - n,) + v.shape[1:], fill.get(k, 0), v.dtype)]) if isinstance(v, np.ndarray) and v.shape[:1] == (n,) else v)
                     for k, v in batch.items()}
        t.cfg.grad_accum = padded // unit
        return batch

    def step(self, batch: Dict[str, np.ndarray], lr: Optional[float] = None) -> Dict[str, float]:
        t, L = self.t, self.loss
        if batch["inputs"].shape[0] not in (t.cfg.batch_size * t.cfg.grad_accum, t.cfg.batch_size * t.cfg.grad_accum * t.world):
            batch = self.fit_rows(batch)
        x, y, pos = self._slice(batch["inputs"]), self._slice(batch["targets"]), self._slice(batch["position_ids"])
        dev = t.device
        adv = torch.from_numpy(self._slice(batch["advantages"])).to(dev)
        old = torch.from_numpy(self._slice(batch["old_logprobs"])).to(dev)
        seq = torch.from_numpy(self._slice(batch["seq_ids"])).to(dev)
        mask = torch.from_numpy((y != -100)).to(dev)
        if L.advantage_clip:
            adv = adv.clamp(-L.advantage_clip, L.advantage_clip)
        logp = t.token_logprobs(x, y, pos)
        if L.type == "ipo":
            teacher = torch.from_numpy(self._slice(batch["teacher_logprobs"])).to(dev) if (L.teacher_tau and "teacher_logprobs" in batch) else None
            loss, w, metrics = ipo_token_weights(logp, old, adv, mask, teacher, L.ipo_mask_low, L.ipo_mask_high, L.adv_tau, L.teacher_tau, L.kl_tau, L.ratio_clip,
                                                 L.normalization, seq)
        else:
            ref = t.token_logprobs(x, y, pos, use_adapters=False) if (L.kl_coef and t.lora is not None) else None
            loss, w, metrics = grpo_token_weights(logp, old, adv, mask, ref, L.clip_eps_low, L.clip_eps_high, L.kl_coef, L.ratio_cap, L.normalization, seq)
        if t.world > 1:  # the normaliser above is per rank: average the ranks' objectives
            w = w / t.world
        t.forward_backward(x, y, pos, row_weights=w, loss_scale_override=1.0)
        norm = t.optimizer_step(lr)
        keys = sorted(metrics)
        vals = torch.stack([loss, norm] + [metrics[k].float() for k in keys]).float()
        if t.world > 1:
            red = vals.clone()
            t.comm.all_reduce(red, "sum")
            red /= t.world
            red[1] = vals[1]
            vals = red
        host = vals.to("cpu").tolist()
        out = {"loss": host[0], "norm": host[1], **{k: v for k, v in zip(keys, host[2:])}}
        if self.turn_diagnostics:
            out.update(self._turn_summary(logp, old, mask, seq, w))
        return out

    @staticmethod
    def _turn_summary(logp, old, mask, seq, weights) -> Dict[str, float]:
        """Per-turn shares of tokens, |log-ratio| and loss weight over this rank's samples (``grpo/turn_stats.py``): in a packed row a
        sample is one value of ``seq_ids``, a turn one run of supervised tokens inside it."""
        from .turn_stats import TurnStats, turn_ids_from_mask

        lp, lo, m, s, w = (a.detach().float().cpu().numpy() for a in (logp, old, mask.float(), seq.float(), weights))
        stats = TurnStats()
        for r in range(lp.shape[0]):
            for sid in np.unique(s[r][s[r] >= 0]):
                sel = s[r] == sid
                stats.add_sample(turn_ids_from_mask(m[r][sel]), m[r][sel], lp[r][sel], lo[r][sel], w[r][sel])
        return stats.summary()


def start_step_override() -> Optional[int]:
    """``SUROGATE_GRPO_START_STEP``: the step a trainer without a checkpoint starts at (it then waits for that step's batch instead of
    replaying the rollout history from step 0, e.g. beside an orchestrator that was resumed).  Parity: surogate/grpo/runs.py:20-30."""
    raw = os.environ.get("SUROGATE_GRPO_START_STEP")
    if raw is None or raw == "":
        return None
    try:
        step = int(raw)
    except ValueError as e:
        raise ValueError(f"Invalid SUROGATE_GRPO_START_STEP={raw!r}; expected an integer") from e
    if step < 0:
        raise ValueError(f"Invalid SUROGATE_GRPO_START_STEP={raw!r}; expected a non-negative integer")
    return step


def run_grpo(cfg: GRPOConfig) -> Dict[str, Any]:
    from ..io.checkpoint import clean_old_checkpoints, find_latest_checkpoint
    from ..parallel.dist import TorchComm, init_distributed
    from ..train.logging import TrainingRunLogger
    from ..train.lr_schedule import LRSchedule
    from ..train.sft import resolve_model_config
    from .transport import make_transport
    from .weight_broadcast import FilesystemBroadcast

    info = init_distributed()
    comm = TorchComm() if info.world > 1 else None
    device = torch.device("cuda", info.local_rank) if torch.cuda.is_available() else torch.device("cpu")
    hf_cfg = resolve_model_config(cfg)
    trainer = Trainer(cfg.to_trainer_config(hf_cfg), device=device, comm=comm)
    if isinstance(cfg.model, str) and os.path.isdir(cfg.model):
        trainer.import_weights(cfg.model)
        if trainer.lora is not None:
            trainer.lora.init_weights(cfg.train_seed)
    else:
        trainer.init_weights(cfg.train_seed)
    start_step, start_version = 0, 0
    latest = find_latest_checkpoint(cfg.checkpoint_dir) if (cfg.resume_from_checkpoint and cfg.checkpoint_dir) else None
    if latest is not None:  # weights (or the adapter over the base loaded above), optimizer state, step and policy version continue
        meta = trainer.load_checkpoint(cfg.checkpoint_dir, latest)
        start_step = int(meta["run"]["step"])
        start_version = int((meta.get("data-loader") or {}).get("policy_version", start_step // max(1, cfg.broadcast_every)))
    else:
        start_step = start_step_override() or 0
        start_version = start_step // max(1, cfg.broadcast_every)
    transport = make_transport(cfg.transport, directory=cfg.transport_dir, endpoint=cfg.zmq_endpoint, role="consumer")
    max_steps = cfg.max_steps if cfg.max_steps > 0 else 100
    noise = None
    if cfg.noise_scheduler and cfg.noise_scheduler.get("enabled"):
        from .noise import NoiseConfig

        ns = cfg.noise_scheduler
        noise = NoiseConfig(enabled=True, sigma_start=float(ns.get("sigma_start", 5e-2)), sigma_end=float(ns.get("sigma_end", 5e-4)),
                            stages=int(ns.get("num_stages", ns.get("stages", 10))), seed=cfg.train_seed)
    bcast = FilesystemBroadcast(cfg.weight_dir, noise=noise, total_steps=max_steps // max(1, cfg.broadcast_every))
    g = GRPOTrainer(trainer, cfg.loss)
    g.turn_diagnostics = bool(cfg.turn_diagnostics)
    g.policy_version = start_version
    bcast.publish(trainer, start_version, hf_cfg)  # the policy the orchestrator starts from: version 0, or the one a resumed run had reached
    sched = LRSchedule(cfg.learning_rate, max_steps, cfg.warmup_steps, cfg.cooldown_steps, cfg.final_lr_fraction * cfg.learning_rate,
                       cfg.lr_scheduler_type, cfg.wsd_decay_steps_fraction)
    logger = TrainingRunLogger(cfg.log_file, None, is_main=info.is_main)
    if cfg.weight_broadcast != "filesystem":
        # the tensor-level publishers (process group of trainer + engine workers, CUDA IPC handles) exist in grpo/weight_broadcast.py with
        # their receivers in grpo/vllm_worker.py; this loop publishes through the watched directory, which works with every engine set-up
        logger.message(f"[grpo] weight_broadcast: {cfg.weight_broadcast} is not wired into this trainer loop: publishing versions under {cfg.weight_dir} instead")
    if start_step:
        logger.message(f"[grpo] continuing at step {start_step}, policy version {start_version}"
                       + (f" (checkpoint {cfg.checkpoint_dir}/step_{latest:08d})" if latest is not None else " (SUROGATE_GRPO_START_STEP)"))
    history = []
    for step in range(start_step, max_steps):
        t0 = time.perf_counter()
        batch, meta = transport.receive(step)
        wait_ms = (time.perf_counter() - t0) * 1e3
        out = g.step(batch, lr=sched.get_lr(step))
        out.update(wait_ms=wait_ms, ms=(time.perf_counter() - t0) * 1e3, off_policy=g.policy_version - int(meta.get("policy_version", 0)),
                   reward_mean=meta.get("reward_mean"))
        if (step + 1) % cfg.broadcast_every == 0:
            g.policy_version += 1
            bcast.publish(trainer, g.policy_version, hf_cfg)
        if info.is_main:
            transport.ack(step)
        logger.log_record("grpo", step=step + 1, **out)
        history.append(out)
        if cfg.save_steps > 0 and cfg.checkpoint_dir and (step + 1) % cfg.save_steps == 0 and step + 1 < max_steps:
            try:
                trainer.save_checkpoint(cfg.checkpoint_dir, step + 1, {"data_loader": {"policy_version": g.policy_version}})
                if info.is_main:
                    clean_old_checkpoints(cfg.checkpoint_dir, cfg.save_total_limit)
            except OSError as e:  # a failed save must not end the run; save_checkpoint raises on every rank together
                logger.message(f"[checkpoint] save failed: {e}")
    logger.close()
    return {"steps": len(history), "history": history}
