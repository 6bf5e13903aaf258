"""Pipeline execution of the stage plan in ``train/dispatch_pp.py``: one process per GPU, stage ``s`` on rank ``s % world``.

Each rank holds only the parameters (and optimizer state) of its stages.  ``M = world * grad_accum`` micro-batches move
through the stages in the diagonal wavefront of ``wavefront()``; the boundary tensors (hidden state and residual stream
forward, their gradients backward) go rank to rank with ``torch.distributed`` point-to-point sends, which on NVSwitch machines
are NVLink copies between the two GPUs' memories; nothing is staged through the host.  The first stage also embeds the
tokens, the last one applies the final norm and the fused LM-head loss.  After the backward wave every rank clips with the
global gradient norm and steps its own parameters; a tied embedding / LM-head weight lives on the first and the last rank and
its gradient is summed between the two before the step.

Parity: csrc/src/binding/py_train.cpp:2484-3060 (dispatch-PP step), surogate/train/dispatch_pp.py, docs/guides/dispatch-pp.md.
The reference hands boundaries GPU -> host -> GPU for PCIe boxes and keeps weights on the host; with NVLink peers and 180 GB
per GPU the weights stay resident and the hand-off is a peer copy.
"""
from __future__ import annotations

import os
from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ..runtime.trainer import Trainer, TrainerConfig
from ..train.dispatch_pp import Stage, plan_stages, wavefront


class PipelineTrainer:
    def __init__(self, cfg: TrainerConfig, device: Optional[torch.device] = None, stage_layers: int = 0, group=None):
        if cfg.lora or cfg.ep_size > 1 or cfg.zero_level > 0:
            raise ValueError("pipeline stages hold whole layers: use zero_level 0, no expert parallelism and full fine-tuning")
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        n_layers = int(cfg.model.get("num_hidden_layers", cfg.model.get("n_layers", 0)))
        if n_layers < self.world:
            raise ValueError(f"{n_layers} layers cannot feed {self.world} pipeline ranks")
        self.stages: List[Stage] = plan_stages(n_layers, self.world, stage_layers or -(-n_layers // self.world))
        self.mine = [s for s in self.stages if s.gpu == self.rank]
        self.first_rank, self.last_rank = self.stages[0].gpu, self.stages[-1].gpu
        own_layers = {L for s in self.mine for L in s.layers}
        has_first, has_last = self.rank == self.first_rank, self.rank == self.last_rank

        def owned(e) -> bool:
            if e.layer is not None:
                return e.layer in own_layers
            if e.group == "embedding":
                return has_first or (has_last and self._tied)
            return has_last  # final norm, LM head

        # whether the LM head shares the embedding weight decides who holds the embedding: probe the compiled model once
        from ..dsl.compiler import compile_model
        from ..runtime.trainer import build_model

        probe = compile_model(build_model(cfg.model)).params
        self._tied = any(p.tied_to for p in probe)
        self._emb_name = next((p.tied_to for p in probe if p.tied_to), "")
        self.inner = Trainer(cfg, device=device, comm=None, owned=owned)
        self.cfg, self.device = cfg, self.inner.device
        self.n_micro = self.world * cfg.grad_accum
        self.ticks = wavefront(len(self.stages), self.n_micro)
        self.act_dtype = self.inner.executor.options.act_dtype
        self.d_model = int(self.inner.cm.model.d_model)
        self.step_index = 0
        self.tied_group = None
        if self._tied and self.first_rank != self.last_rank:
            self.tied_group = dist.new_group([self.first_rank, self.last_rank])
        # One communicator per DIRECTED pair of neighbouring ranks.  With interleaved stages two ranks send to each other in
        # the same tick; on one communicator each side's send would sit in front of the receive the other side is waiting
        # for.  Separate communicators (own streams) keep the two directions independent.
        self.link: Dict[Tuple[int, int], Any] = {}
        pairs = []
        for a, b in zip(self.stages, self.stages[1:]):
            for pair in ((a.gpu, b.gpu), (b.gpu, a.gpu)):  # forward boundary, backward gradient
                if pair[0] != pair[1] and pair not in pairs:
                    pairs.append(pair)
        for src, dst in pairs:  # every rank creates every group, in the same order
            self.link[(src, dst)] = dist.new_group([src, dst]) if self.world > 2 or len(pairs) > 1 else group

    # ------------------------------------------------------------------ weights
    def init_weights(self, seed: Optional[int] = None) -> None:
        self.inner.init_weights(seed)  # per-parameter seeds: the same values as an unpartitioned run

    def import_weights(self, path: str) -> None:
        self.inner.import_weights(path)

    def export_model(self, out_dir: str, hf_config: Optional[Dict[str, Any]] = None) -> None:
        """Every rank writes the tensors it holds to its own shard; rank 0 writes the index and config."""
        import json

        from safetensors.torch import save_file

        from ..io.hf_checkpoint import to_hf_config

        os.makedirs(out_dir, exist_ok=True)
        entries = {p.name: p for p in self.inner.cm.params}
        tensors: Dict[str, torch.Tensor] = {}
        for name, full in self.inner.store.named_full_tensors():
            p = entries[name]
            if p.spec.hf is None or (p.group == "embedding" and self.rank != self.first_rank):
                continue
            for hf_name, t in p.spec.hf.export(full.detach().to("cpu"), p.layer).items():
                tensors[hf_name] = t.to(torch.bfloat16).contiguous()
        cfgd = hf_config or self.cfg.model
        fn = f"model-{self.rank + 1:05d}-of-{self.world:05d}.safetensors"
        save_file(tensors, os.path.join(out_dir, fn), metadata={"format": "pt"})
        names: List[Any] = [None] * self.world
        dist.all_gather_object(names, (fn, list(tensors), sum(t.numel() * t.element_size() for t in tensors.values())), group=self.group)
        if self.rank == 0:
            with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
                json.dump({"metadata": {"total_size": sum(n[2] for n in names)}, "weight_map": {k: n[0] for n in names for k in n[1]}}, f, indent=1)
            with open(os.path.join(out_dir, "config.json"), "w") as f:
                json.dump(to_hf_config(self.inner.cm, cfgd), f, indent=1)
        dist.barrier(group=self.group)

    # ------------------------------------------------------------------ point-to-point boundaries
    def _send(self, tensors: Tuple[torch.Tensor, ...], dst: int, pending: list) -> None:
        g = self.link.get((self.rank, dst), self.group)
        for t in tensors:
            t = t.contiguous()
            pending.append((dist.isend(t, dst, group=g), t))  # the tensor stays referenced until the send completes

    def _recv(self, rows: int, T: int, src: int) -> Tuple[torch.Tensor, torch.Tensor]:
        g = self.link.get((src, self.rank), self.group)
        out = []
        for _ in range(2):
            buf = torch.empty(rows, T, self.d_model, dtype=self.act_dtype, device=self.device)
            dist.recv(buf, src, group=g)
            out.append(buf)
        return out[0], out[1]

    # ------------------------------------------------------------------ one optimizer step
    def step(self, inputs: np.ndarray, targets: np.ndarray, position_ids: Optional[np.ndarray] = None, lr: Optional[float] = None, kd=None,
             row_weights=None) -> Dict[str, float]:
        """``inputs`` / ``targets``: [n_micro * batch_size, T], the same arrays on every rank (only the first and the last rank
        read them)."""
        if kd is not None or row_weights is not None:
            raise NotImplementedError("pipeline stages run the plain next-token objective (no distillation term or per-token weights)")
        tr, ex = self.inner, self.inner.executor
        B, M = self.cfg.batch_size, self.n_micro
        assert inputs.shape[0] == B * M, f"expected {B * M} rows ({M} micro-batches of {B}), got {inputs.shape[0]}"
        T = inputs.shape[1]
        has_first, has_last = self.rank == self.first_rank, self.rank == self.last_rank
        inp = tr._stage("inputs", inputs) if has_first else None
        tgt = tr._stage("targets", targets) if has_last else None
        pos_all = tr._stage("position_ids", position_ids) if position_ids is not None else \
            torch.arange(T, dtype=torch.int32, device=self.device)[None].expand(B * M, T).contiguous()
        n_valid = torch.zeros((), dtype=torch.float32, device=self.device)
        if has_last:
            n_valid += (tgt != -100).sum()
        dist.broadcast(n_valid, self.last_rank, group=self.group)
        loss_scale = (1.0 / n_valid.clamp_min(1.0)).reshape(1)
        if self.device.type != "cuda":
            loss_scale = float(loss_scale)
        tr.store.begin_step()
        tr.recipe.begin_step(tr.step_index)
        loss_sum = torch.zeros((), dtype=torch.float32, device=self.device)
        aux_sum = torch.zeros((), dtype=torch.float32, device=self.device)
        states: Dict[Tuple[int, int], Any] = {}
        pending: list = []
        older: list = []
        n_stages = len(self.stages)
        seen_bwd = 0
        for tick in self.ticks:
            for phase, s, m in tick:
                st = self.stages[s]
                if st.gpu != self.rank:
                    continue
                first, last = s == 0, s == n_stages - 1
                rows = slice(m * B, (m + 1) * B)
                layers = (st.first_layer, st.last_layer)
                if phase == "fwd":
                    ctx = ex.new_context(pos_all[rows], True)
                    ctx.loss_scale, ctx.aux_scale, ctx.micro_step = loss_scale, 1.0 / M, m
                    x = res = None
                    if not first:
                        x, res = self._recv(B, T, self.stages[s - 1].gpu)
                    x, res, aux, outs = ex.stage_forward(ctx, layers, first, last, pos_all[rows], token_ids=inp[rows] if first else None,
                                                         targets=tgt[rows] if last else None, x=x, residual=res)
                    for a in aux:
                        if a is not None:
                            aux_sum += a / M
                    if last:
                        loss_sum += outs[0]
                    else:
                        self._send((x, res), self.stages[s + 1].gpu, pending)
                    states[(s, m)] = (ctx, ex.detach_state())
                else:
                    ctx, state = states.pop((s, m))
                    ex.attach_state(state)
                    tr.store.begin_micro_step(seen_bwd, len(self.mine) * M)
                    seen_bwd += 1
                    dx = dres = None
                    if not last:
                        dx, dres = self._recv(B, T, self.stages[s + 1].gpu)
                    dx, dres = ex.stage_backward(ctx, layers, first, last, dx, dres)
                    if not first:
                        self._send((dx, dres if dres is not None else torch.zeros_like(dx)), self.stages[s - 1].gpu, pending)
            # A send completes only once its receiver has posted the matching receive, which happens in the receiver's NEXT
            # tick; with interleaved stages two ranks send to each other in the same tick, so waiting here for this tick's
            # sends would deadlock.  Wait for the previous tick's sends instead: their receives were posted during this tick.
            for work, _ in older:
                work.wait()
            older, pending = pending, []
        for work, _ in older:
            work.wait()
        tr.store.finish_reduce()
        # tied embedding / head: both holders sum their gradient contributions
        if self.tied_group is not None and self.rank in (self.first_rank, self.last_rank):
            g = tr.store.grad_of(self._emb_name)
            if g is not None:
                dist.all_reduce(g, group=self.tied_group)
        sq = tr.grad_norm().float() ** 2
        if self.tied_group is not None and self.rank == self.last_rank:
            g = tr.store.grad_of(self._emb_name)
            if g is not None:
                sq = sq - g.float().pow(2).sum()  # counted on the first rank
        stats = torch.stack([sq, loss_sum if has_last else torch.zeros_like(loss_sum), aux_sum])
        dist.all_reduce(stats, group=self.group)
        norm = stats[0].clamp_min(0).sqrt()
        tr.optimizer_step(lr, norm=norm)
        self.step_index += 1
        out = torch.stack([stats[1] / n_valid.clamp_min(1.0) + stats[2], norm, stats[2]]).to("cpu")
        return {"loss": float(out[0]), "norm": float(out[1]), "aux_loss": float(out[2])}

    # ------------------------------------------------------------------ the rest of the trainer interface used by the SFT loop
    lora = None
    last_moe_stats = None

    @property
    def store(self):
        return self.inner.store

    def get_gpu_info(self):
        return self.inner.get_gpu_info()

    def num_parameters(self) -> int:
        return self.inner.cm.num_parameters()

    @torch.no_grad()
    def validate(self, inputs: np.ndarray, targets: np.ndarray, position_ids=None) -> Dict[str, float]:
        """Forward-only wave over the stages (one micro-batch of all given rows); every rank returns the same loss."""
        tr, ex = self.inner, self.inner.executor
        rows, T = inputs.shape
        has_first, has_last = self.rank == self.first_rank, self.rank == self.last_rank
        inp = tr._stage("v_inputs", inputs) if has_first else None
        tgt = tr._stage("v_targets", targets) if has_last else None
        pos = torch.arange(T, dtype=torch.int32, device=self.device)[None].expand(rows, T).contiguous()
        stats = torch.zeros(2, dtype=torch.float32, device=self.device)
        tr.store.grads_enabled = False
        try:
            x = res = None
            for s, st in enumerate(self.stages):
                first, last = s == 0, s == len(self.stages) - 1
                if st.gpu == self.rank:
                    ctx = ex.new_context(pos, False)
                    if not first and self.stages[s - 1].gpu != self.rank:
                        x, res = self._recv(rows, T, self.stages[s - 1].gpu)
                    x, res, _, outs = ex.stage_forward(ctx, (st.first_layer, st.last_layer), first, last, pos, token_ids=inp if first else None,
                                                       targets=tgt if last else None, x=x, residual=res)
                    ex.detach_state()
                    if last:
                        stats[0], stats[1] = outs[0], (tgt != -100).sum()
                    elif self.stages[s + 1].gpu != self.rank:
                        pend: list = []
                        self._send((x, res), self.stages[s + 1].gpu, pend)
                        for w, _ in pend:
                            w.wait()
        finally:
            tr.store.grads_enabled = True
        dist.all_reduce(stats, group=self.group)
        return {"loss": float(stats[0] / stats[1].clamp_min(1.0))}

    def _ckpt_root(self, root: str) -> str:
        return os.path.join(root, f"stage_rank_{self.rank:03d}")

    def save_checkpoint(self, ckpt_dir: str, step: Optional[int] = None, extra: Optional[Dict[str, Any]] = None) -> str:
        """Each rank checkpoints the parameters and optimizer state it holds under its own sub-directory."""
        out = self.inner.save_checkpoint(self._ckpt_root(ckpt_dir), self.step_index if step is None else step, extra)
        dist.barrier(group=self.group)
        return out

    def load_checkpoint(self, ckpt_dir: str, step: Optional[int] = None) -> Dict[str, Any]:
        meta = self.inner.load_checkpoint(self._ckpt_root(ckpt_dir), step)
        self.step_index = self.inner.step_index
        return meta

    def latest_checkpoint(self, ckpt_dir: str) -> Optional[int]:
        from ..io.checkpoint import find_latest_checkpoint

        mine = find_latest_checkpoint(self._ckpt_root(ckpt_dir))
        t = torch.tensor([-1 if mine is None else mine], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)  # a step counts only if every stage has it
        return None if int(t) < 0 else int(t)
