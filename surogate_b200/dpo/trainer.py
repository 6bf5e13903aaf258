"""DPO training loop.

One optimizer step over ``P`` preference pairs (rows ordered chosen, rejected, chosen, ...):

1. reference log-probabilities: a no-grad forward of the frozen base model (LoRA adapters disabled), skipped when
   ``reference_free``;
2. policy log-probabilities: a no-grad forward with adapters;
3. per-sequence weights from the DPO objective (``dpo/loss.py``);
4. one forward+backward whose fused LM-head loss kernel scales every token's log-likelihood gradient by its
   sequence's weight, then the usual gradient norm / clip / optimizer step.

Parity: surogate/dpo/trainer.py (inline frozen-reference forward, then the native DPO step).
"""
from __future__ import annotations

import json
import os
import time
from typing import Any, Dict, Optional

import numpy as np
import torch

from ..config.loader import load_config
from ..data.datasets import load_dataset_rows
from ..parallel.dist import TorchComm, init_distributed
from ..runtime.trainer import Trainer
from ..train.logging import TrainingRunLogger
from ..train.lr_schedule import LRSchedule
from .config import DPOConfig
from .data import PairLoader, build_pairs
from .loss import dpo_loss_and_weights

IGNORE = -100


class DPOTrainer:
    def __init__(self, trainer: Trainer, beta: float = 0.1, label_smoothing: float = 0.0, loss_type: str = "sigmoid", reference_free: bool = False):
        self.t, self.beta, self.ls, self.loss_type, self.reference_free = trainer, beta, label_smoothing, loss_type, reference_free

    def sequence_logps(self, x, y, use_adapters: bool) -> torch.Tensor:
        return self.t.token_logprobs(x, y, use_adapters=use_adapters).sum(dim=1)

    def step(self, x: np.ndarray, y: np.ndarray, lr: Optional[float] = None) -> Dict[str, float]:
        """x, y: [2 * pairs, T] for this rank (chosen row then rejected row of each pair)."""
        t = self.t
        assert x.shape[0] % 2 == 0 and x.shape[0] == t.cfg.batch_size * t.cfg.grad_accum, "rows per step must equal batch_size * grad_accum"
        pol = self.sequence_logps(x, y, True)
        ref = torch.zeros_like(pol) if self.reference_free else self.sequence_logps(x, y, False)
        loss, w_c, w_r, metrics = dpo_loss_and_weights(pol[0::2], pol[1::2], ref[0::2], ref[1::2], self.beta, self.ls, self.loss_type)
        seq_w = torch.stack([w_c, w_r], dim=1).reshape(-1) / t.world  # mean over all ranks' pairs
        row_w = seq_w[:, None].expand(-1, x.shape[1]).contiguous()
        t.forward_backward(x, y, row_weights=row_w, loss_scale_override=1.0)
        norm = t.optimizer_step(lr)
        vals = torch.stack([loss, norm] + [metrics[k] for k in sorted(metrics)]).float()
        if t.world > 1:
            red = vals.clone()
            t.comm.all_reduce(red, "sum")
            red /= t.world
            red[1] = vals[1]
            vals = red
        host = vals.to("cpu").tolist()
        out = {"loss": host[0], "norm": host[1]}
        out.update({k: v for k, v in zip(sorted(metrics), host[2:])})
        return out


def run_dpo(cfg: DPOConfig) -> Dict[str, Any]:
    from ..data.tokenizer import Tokenizer
    from ..train.sft import resolve_model_config

    info = init_distributed()
    comm = TorchComm() if info.world > 1 else None
    device = torch.device("cuda", info.local_rank) if torch.cuda.is_available() else torch.device("cpu")
    hf_cfg = resolve_model_config(cfg)
    tok = Tokenizer.from_pretrained(cfg.model)
    rows = [r for ds in cfg.datasets for r in load_dataset_rows(ds)]
    rows = [r for r in rows if "chosen" in r]
    X, Y = build_pairs(tok, rows, cfg.sequence_len, cfg.max_prompt_length)
    pairs_per_step = cfg.per_device_train_batch_size * cfg.gradient_accumulation_steps // 2
    if pairs_per_step < 1:
        raise ValueError("[E133] per_device_train_batch_size * gradient_accumulation_steps must be an even number >= 2 (chosen + rejected rows)")
    loader = PairLoader(X, Y, pairs_per_step, seed=cfg.train_seed, rank=info.rank, world=info.world)
    tcfg = cfg.to_trainer_config(hf_cfg)
    trainer = Trainer(tcfg, device=device, comm=comm)
    if os.path.isdir(cfg.model):
        trainer.import_weights(cfg.model)
        if trainer.lora is not None:
            trainer.lora.init_weights(cfg.train_seed)
    else:
        trainer.init_weights(cfg.train_seed)
    dpo = DPOTrainer(trainer, cfg.beta, cfg.label_smoothing, cfg.loss_type, cfg.reference_free)
    max_steps = cfg.max_steps if cfg.max_steps > 0 else loader.steps_per_epoch() * cfg.num_epochs
    sched = LRSchedule(cfg.learning_rate, max_steps, cfg.warmup_steps or int(cfg.warmup_ratio * max_steps), cfg.cooldown_steps,
                       cfg.final_lr_fraction * cfg.learning_rate, cfg.lr_scheduler_type, cfg.wsd_decay_steps_fraction)
    logger = TrainingRunLogger(cfg.log_file, None, is_main=info.is_main)
    history = []
    for step in range(max_steps):
        t0 = time.perf_counter()
        x, y = loader.next()
        out = dpo.step(x, y, lr=sched.get_lr(step))
        out["ms"] = (time.perf_counter() - t0) * 1e3
        history.append(out)
        logger.log_record("dpo", step=step + 1, **out)
    if trainer.lora is not None:
        trainer.export_adapter(os.path.join(cfg.output_dir, "adapter"), base_model=cfg.model)
    else:
        trainer.export_model(cfg.output_dir, hf_cfg)
    logger.close()
    return {"steps": len(history), "history": history}


def dpo_main(config_path: str, **overrides):
    return run_dpo(load_config(DPOConfig, config_path, **overrides))
