"""Trainer: owns the compiled model, parameter store, recipe, optimizer and the step loop.

One process drives one GPU.  ``step(inputs, targets)`` takes int32 numpy arrays
``[B * grad_accum, T]`` for this rank (or ``[world * B * grad_accum, T]`` for the whole
job, of which the rank takes its slice), stages them through pinned host memory, runs
forward/backward for every micro-batch, reduces gradients (overlapped with backward),
computes the global gradient norm and clip scale on the device, runs the optimizer on
this rank's shards and returns ``{"loss", "norm"}`` as Python floats — the only
host synchronisation of the step is that final read-back.

Parity: csrc/src/binding/py_train.h:55-501 (MultiGPUPyTrainer: step / update_with_config /
train_step_graphed / validate / import / export / checkpoints), docs/reference/python-api.md.
"""
from __future__ import annotations

import math
import os
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from ..dsl.compiler import CompiledModel, compile_model, model_from_hf_config
from ..dsl.nn import model_class_for
from ..optim import OptimizerConfig, make_optimizer
from ..recipes import make_recipe
from .executor import ExecOptions, Executor
from .params import ParamStore, SingleProcessComm


@dataclass
class TrainerConfig:
    model: Dict[str, Any] = field(default_factory=dict)  # HF config.json dict, or ctor kwargs + "architecture"
    batch_size: int = 2
    seq_len: int = 1024
    grad_accum: int = 1
    recipe: str = "bf16"
    optimizer: str = "adamw_8bit"
    learning_rate: float = 2e-4
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0
    max_grad_norm: float = 1.0
    zero_level: int = 1
    recompute: bool = False
    backend: str = "auto"  # auto | cuda | ref
    attention: str = "auto"
    param_dtype: str = "bf16"
    grad_dtype: str = "bf16"
    master_dtype: Optional[str] = None
    lmhead_chunk_rows: int = 4096
    keep_gathered: bool = True
    collectives: str = "auto"  # auto | nccl | symm
    ep_size: int = 1
    ep_capacity_factor: float = 1.5
    ep_load_balance_threshold: float = 1.3   # re-place experts when a layer's busiest rank exceeds this multiple of the mean load
    ep_spill_threshold: float = 0.0          # > 0 (PyTorch backend): per step, row ranges of overloaded experts go to helper ranks above this imbalance
    ep_spill_min_rows: int = 64              # smallest chunk worth shipping an expert's weights for
    trainable_param_substrings: Optional[List[str]] = None  # partial-update runs: only parameters whose name contains one of these train
    gradient_mask_mode: Optional[str] = None  # allow_substrings | mlp_growth_new_half (None: the SUROGATE_GRADIENT_MASK_MODE variable)
    ep_plan_refresh_interval: int = 16       # steps between placement refreshes (0 = never)
    lora: Optional[Dict[str, Any]] = None
    fp8_amax_history: int = 16
    skip_quant_first_layers: int = 0
    skip_quant_last_layers: int = 0
    offload_optimizer: bool = False
    offload_master: bool = False
    resident_layers: int = -1   # with offload_master: frozen weights of the first N layers stay in device memory (-1: SUROGATE_RESIDENT_LAYERS or 0)
    qlora: Optional[str] = None  # bnb_nf4 | fp8_block | nvfp4: frozen base weights stored block-quantised, rebuilt per layer
    qlora_block_size: int = 64
    qlora_double_quant: bool = True
    qlora_four_over_six: bool = True
    qlora_experts: bool = True            # MoE: frozen expert weights are stored quantised too (they are most of the model)
    qlora_offload_experts: bool = False   # ... and wait in pinned host memory, streamed one MoE layer ahead
    fp4_four_over_six: bool = True   # NVFP4 recipe: per block of 16 keep the better of the abs-max -> 6 and abs-max -> 4 mappings (round-to-nearest operands)
    time_breakdown: bool = False            # per-step milliseconds of forward / LM head / backward / optimizer in Trainer.last_time_breakdown
    lmhead_drop_ignored_rows: bool = False  # only rows with a target go through the LM head
    offload_saved_tensors: bool = False     # saved activations (or, with recompute, the per-layer input checkpoints) wait in pinned host memory
    use_cuda_graphs: bool = False  # capture each micro-batch's forward + backward in a CUDA graph (one GPU, dense models, bf16 / fp8 recipes)
    sequence_chunks: int = 1    # > 1: each sequence is trained in this many pieces against a key/value prefix (attention models only)
    long_context: bool = False  # tiled MLP: tile = min(tokens, hidden size) rows, recomputed per tile in backward (dense models)
    async_optimizer: Optional[str] = None  # with cpu_training: "overlap" runs the host update of step N while step N+1 computes on weights one update old; "inline" = same bookkeeping, no overlap
    cpu_training: bool = False  # fp32 masters + AdamW moments on the host, update on the CPU, bf16 weights streamed per layer
    normuon_momentum: float = 0.95
    normuon_beta2: float = 0.95
    normuon_cautious_wd: bool = True
    normuon_momentum_8bit: bool = False
    init_projections_to_zero: bool = False
    seed: int = 0


_DT = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16, None: None}


def build_model(spec: Dict[str, Any], **overrides):
    spec = dict(spec)
    if "architectures" in spec or "model_type" in spec:
        return model_from_hf_config(spec, **overrides)
    arch = spec.pop("architecture")
    spec.update(overrides)
    return model_class_for(arch)(**spec)


class Trainer:
    def __init__(self, cfg: TrainerConfig, device: Optional[torch.device] = None, comm=None, owned=None):
        """``owned(param entry) -> bool`` restricts the parameters this process holds (pipeline stages)."""
        self.cfg = cfg
        self.device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self.comm = comm or SingleProcessComm()
        self.world, self.rank = self.comm.world, self.comm.rank
        on_gpu = self.device.type == "cuda"
        extra = {"ep_size": cfg.ep_size} if cfg.ep_size > 1 else {}
        if cfg.long_context:
            hidden = cfg.model.get("hidden_size", cfg.model.get("d_model", 4096))
            extra["mlp_tile_rows"] = max(128, min(cfg.batch_size * cfg.seq_len, hidden))
        self.model = build_model(cfg.model, **extra)
        self.cm: CompiledModel = compile_model(self.model)
        pd = _DT[cfg.param_dtype] if on_gpu else torch.float32
        gd = _DT[cfg.grad_dtype] if on_gpu else torch.float32
        md = _DT[cfg.master_dtype] if cfg.master_dtype else pd
        if cfg.cpu_training:
            md = torch.float32
        self.lora = None
        frozen = None
        if cfg.lora:
            from .lora import LoRAManager

            self.lora = LoRAManager(self.cm, cfg.lora, device=self.device, comm=self.comm, dtype=pd)
            frozen = self.lora.freezes
        if cfg.collectives in ("auto", "symm") and on_gpu and self.world > 1 and cfg.zero_level >= 1:
            from ..parallel import symm

            self.comm = symm.try_create(self.comm, self.device, required=cfg.collectives == "symm")
        from .grad_mask import GradientMask

        # expert-parallel x data-parallel mesh: with ep_size < world the expert group is a sub-group (dispatch / combine inside it) and
        # expert gradients are summed over the ranks that hold the same experts
        self.ep_comm = self.expert_dp_comm = None
        if cfg.ep_size > 1 and self.world > cfg.ep_size:
            from ..parallel.mesh import build_ep_mesh

            self.ep_comm, self.expert_dp_comm = build_ep_mesh(getattr(self.comm, "base", self.comm), cfg.ep_size)
        elif cfg.ep_size > self.world:
            raise ValueError(f"ep_size={cfg.ep_size} exceeds the {self.world} ranks of this run")
        self.grad_mask = None if cfg.lora else GradientMask.resolve(cfg.trainable_param_substrings, cfg.gradient_mask_mode)
        self.store = ParamStore(self.cm, device=self.device, grad_mask=self.grad_mask, param_dtype=pd, grad_dtype=gd, master_dtype=md, comm=self.comm,
                                ep_comm=self.ep_comm, expert_dp_comm=self.expert_dp_comm,
                                zero_level=cfg.zero_level, keep_gathered=cfg.keep_gathered, frozen=frozen, expert_parallel=cfg.ep_size,
                                offload_master=cfg.offload_master or cfg.cpu_training,
                                host_work_copy=("double" if cfg.async_optimizer else True) if cfg.cpu_training else False, owned=owned,
                                resident_layers=cfg.resident_layers if cfg.resident_layers >= 0 else int(os.environ.get("SUROGATE_RESIDENT_LAYERS", "0")))
        from .ops_cuda import make_backend

        self.backend = make_backend(self.device, cfg.backend, lmhead_chunk_rows=cfg.lmhead_chunk_rows, attention=cfg.attention)
        rname = cfg.recipe if (on_gpu and self.backend.name == "cuda") else "bf16"
        self.recipe = make_recipe(rname, self.cm, self.device, **self._recipe_kwargs(rname))
        if hasattr(self.recipe, "quantizes") and rname.replace("-", "_") == "fp8_hybrid" and cfg.lora is None:
            self.store.enable_fp8_gather(self.recipe.quantizes)
        self.ep = None
        if cfg.ep_size > 1:
            group_comm = self.ep_comm if self.ep_comm is not None else self.comm
            if on_gpu and self.backend.name == "cuda":
                from ..parallel.ep import ExpertParallel

                if self.ep_comm is not None:   # the expert group's own symmetric arena, barriers and peer pointers
                    from ..parallel import symm

                    group_comm = symm.try_create(self.ep_comm, self.device, required=True)
                self.ep = ExpertParallel(group_comm, cfg.ep_size, self.device, capacity_factor=cfg.ep_capacity_factor)
                if hasattr(self.recipe, "dispatch_fp8"):
                    self.recipe.ep_group_comm = group_comm     # delayed scales of dispatched rows are agreed inside the expert group
                self.ep.replica_comm = self.expert_dp_comm
            else:                              # PyTorch backend (CPU ranks over gloo included): the library all-to-all
                from ..parallel.ep_ref import AllToAllExpertParallel

                self.ep = AllToAllExpertParallel(getattr(group_comm, "base", group_comm), cfg.ep_size, self.device, spill_threshold=cfg.ep_spill_threshold,
                                                 spill_min_rows=cfg.ep_spill_min_rows)
        self.executor = Executor(self.cm, self.store, self.backend, recipe=self.recipe,
                                 options=ExecOptions(recompute=cfg.recompute, act_dtype=pd, lmhead_drop_ignored_rows=cfg.lmhead_drop_ignored_rows,
                                                     offload_saved=cfg.offload_saved_tensors, time_breakdown=cfg.time_breakdown), device=self.device, ep=self.ep, lora=self.lora)
        self.opt_cfg = OptimizerConfig(cfg.optimizer, cfg.learning_rate, cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay, cfg.max_grad_norm,
                                       cfg.normuon_momentum, cfg.normuon_beta2, cfg.normuon_cautious_wd, normuon_momentum_8bit=cfg.normuon_momentum_8bit)
        self.streamed = None
        if cfg.async_optimizer and not cfg.cpu_training:
            raise ValueError("async_optimizer overlaps the HOST update with device compute: it needs cpu_training")
        if cfg.async_optimizer not in (None, "overlap", "inline"):
            raise ValueError(f"async_optimizer: '{cfg.async_optimizer}' (overlap | inline)")
        if cfg.cpu_training:
            from .offload import CpuAdamW

            if cfg.optimizer not in ("adamw", "adamw_8bit"):
                raise ValueError("cpu_training runs AdamW on the host: choose optimizer adamw (adamw_8bit is treated as adamw)")
            self.optimizer = CpuAdamW(self.opt_cfg, self.store, stale=cfg.async_optimizer)
        else:
            self.optimizer = make_optimizer(self.opt_cfg, self.store)
            if cfg.offload_optimizer or cfg.offload_master:
                from .offload import StreamedOptimizerStep

                if cfg.optimizer == "normuon":
                    raise ValueError("offload_optimizer / offload_master are implemented for adamw and adamw_8bit")
                self.optimizer.offload_state = bool(cfg.offload_optimizer)
                self.streamed = StreamedOptimizerStep(self.store, self.optimizer, self.device)
        self.step_index = 0
        self.kernel_launch_estimate = 0
        self._pinned: Dict[str, torch.Tensor] = {}
        self._visual: Optional[Dict[str, Any]] = None  # see set_visual_inputs
        self._hp = torch.zeros(8, dtype=torch.float32, device=self.device)
        self.last_moe_stats = None
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def _recipe_kwargs(self, name: str) -> Dict[str, Any]:
        n = name.replace("-", "_")
        if n == "fp8_hybrid":
            return dict(history=self.cfg.fp8_amax_history, skip_first_layers=self.cfg.skip_quant_first_layers,
                        skip_last_layers=self.cfg.skip_quant_last_layers)
        if n == "nvfp4":
            return dict(skip_first_layers=self.cfg.skip_quant_first_layers, skip_last_layers=self.cfg.skip_quant_last_layers,
                        four_over_six=self.cfg.fp4_four_over_six)
        return {}

    # ------------------------------------------------------------------ weights
    def _apply_qlora(self) -> None:
        c = self.cfg
        if not c.qlora:
            return
        if self.lora is None:
            raise ValueError("qlora needs LoRA adapters (the quantised base is frozen)")
        from ..quant import make_codec

        kw = {"bnb_nf4": dict(block=c.qlora_block_size, double_quant=c.qlora_double_quant), "fp8_block": dict(block=max(64, c.qlora_block_size)),
              "nvfp4": dict(four_over_six=c.qlora_four_over_six)}[c.qlora]
        codec = make_codec(c.qlora, **kw)
        self.qlora_bytes_saved = self.store.quantize_frozen(codec)
        if c.qlora_experts and any(b.expert and not b.trainable for b in self.store.buckets.values()):
            from .expert_offload import ExpertOffloadManager

            self.store.expert_offload = ExpertOffloadManager(self.store, codec, offload=c.qlora_offload_experts)
            self.qlora_bytes_saved += self.store.expert_offload.attach()

    def init_weights(self, seed: Optional[int] = None) -> None:
        self.store.init_weights(seed if seed is not None else self.cfg.seed, zero_projections=self.cfg.init_projections_to_zero)
        self._apply_qlora()
        self.recipe.on_weights_updated(self.store)
        if self.lora is not None:
            self.lora.init_weights(seed if seed is not None else self.cfg.seed)

    def import_weights(self, path: str) -> None:
        self.drain_optimizer()
        from ..io.hf_checkpoint import import_hf_weights

        import_hf_weights(self.cm, self.store, path)
        self._imported_from = path
        self.store.sync_work_from_master()
        self._apply_qlora()
        self.recipe.on_weights_updated(self.store)

    def export_model(self, out_dir: str, hf_config: Optional[Dict[str, Any]] = None) -> None:
        self.drain_optimizer()
        from ..io.hf_checkpoint import export_hf_weights

        export_hf_weights(self.cm, self.store, out_dir, hf_config or self.cfg.model, write=self.rank == 0,
                          passthrough_from=getattr(self, "_imported_from", None))
        if self.rank == 0:
            from ..io.hf_checkpoint import copy_tokenizer_files

            copy_tokenizer_files(getattr(self, "tokenizer_source", None) or getattr(self, "_imported_from", None), out_dir)

    def export_adapter(self, out_dir: str, base_model: str = "") -> None:
        if self.lora is None:
            raise RuntimeError("export_adapter: LoRA is not enabled")
        self.lora.export_peft(out_dir, base_model, write=self.rank == 0)

    def save_checkpoint(self, ckpt_dir: str, step: Optional[int] = None, extra: Optional[Dict[str, Any]] = None) -> str:
        self.drain_optimizer()
        from ..io.checkpoint import save_checkpoint

        return save_checkpoint(self, ckpt_dir, self.step_index if step is None else step, extra or {})

    def load_checkpoint(self, ckpt_dir: str, step: Optional[int] = None) -> Dict[str, Any]:
        self.drain_optimizer()
        from ..io.checkpoint import load_checkpoint

        return load_checkpoint(self, ckpt_dir, step)

    # ------------------------------------------------------------------ data staging
    def _stage(self, name: str, arr, dtype=torch.int32) -> torch.Tensor:
        """numpy / CPU tensor -> pinned host buffer -> device (async).  Counts the bytes moved."""
        t = torch.from_numpy(np.ascontiguousarray(arr)) if isinstance(arr, np.ndarray) else arr
        if t.device.type != "cpu":
            return t.to(self.device, dtype=dtype)
        t = t.to(dtype)
        if self.device.type != "cuda":
            return t
        buf = self._pinned.get(name)
        if buf is None or buf.shape != t.shape:
            buf = self._pinned[name] = torch.empty(t.shape, dtype=dtype, pin_memory=True)
        buf.copy_(t)
        self.h2d_bytes += buf.numel() * buf.element_size()
        return buf.to(self.device, non_blocking=True)

    def _local_slice(self, arr):
        B, GA = self.cfg.batch_size, self.cfg.grad_accum
        if arr.shape[0] == self.world * B * GA and self.world > 1:
            return arr[self.rank * B * GA:(self.rank + 1) * B * GA]
        assert arr.shape[0] == B * GA, f"expected {B * GA} (or {self.world * B * GA}) rows, got {arr.shape[0]}"
        return arr

    # ------------------------------------------------------------------ multimodal side inputs
    def set_visual_inputs(self, visual_pos_masks=None, visual_embeds=None, deepstack_visual_embeds=None, mrope_position_ids=None) -> None:
        """Vision-tower outputs for the NEXT batches of this rank (kept until replaced; call with no arguments to clear).

        ``visual_pos_masks`` [rows, T] marks image / video placeholder tokens; ``visual_embeds`` [n_visual, C] are their
        embeddings in row-major mask order; ``deepstack_visual_embeds`` is a list (one per early layer) of [n_visual, C];
        ``mrope_position_ids`` [3, rows, T] are the temporal / height / width positions.
        Parity: csrc/src/binding/py_train.cpp (set_visual_inputs)."""
        if visual_pos_masks is None and mrope_position_ids is None:
            self._visual = None
            return
        v: Dict[str, Any] = {"mask": None, "embeds": None, "deep": [], "pos3": None, "cum": None}
        if visual_pos_masks is not None:
            m = torch.as_tensor(np.asarray(visual_pos_masks) if not torch.is_tensor(visual_pos_masks) else visual_pos_masks).to(torch.bool)
            v["cum"] = [0] + torch.cumsum(m.reshape(m.shape[0], -1).sum(1).cpu(), 0).tolist()
            v["mask"] = m.to(self.device)
            v["embeds"] = torch.as_tensor(visual_embeds).to(self.device) if visual_embeds is not None else None
            v["deep"] = [torch.as_tensor(d).to(self.device) for d in (deepstack_visual_embeds or [])]
        if mrope_position_ids is not None:
            v["pos3"] = torch.as_tensor(np.asarray(mrope_position_ids) if not torch.is_tensor(mrope_position_ids) else mrope_position_ids).to(self.device, torch.int32)
        self._visual = v

    def _extras(self, rows: slice) -> Optional[Dict[str, Any]]:
        v = getattr(self, "_visual", None)
        if v is None:
            return None
        out: Dict[str, Any] = {}
        if v["mask"] is not None:
            a, b = v["cum"][rows.start], v["cum"][min(rows.stop, len(v["cum"]) - 1)]
            out["visual_pos_masks"] = v["mask"][rows]
            out["visual_embeds"] = v["embeds"][a:b] if v["embeds"] is not None else None
            out["deepstack_visual_embeds"] = [d[a:b] for d in v["deep"]]
        if v["pos3"] is not None:
            out["mrope_position_ids"] = v["pos3"][:, rows]
        return out

    # ------------------------------------------------------------------ the step
    def forward_backward(self, inputs, targets, position_ids=None, row_weights=None, kd=None, loss_scale_override=None) -> Dict[str, torch.Tensor]:
        """All micro-batches of one optimizer step; leaves reduced gradients in the store.  Returns device scalars.

        ``row_weights`` ([rows, T] float) multiplies each token's log-likelihood gradient (sequence-level objectives: DPO,
        GRPO); ``kd`` = {"idx", "logp", "weight", "ce_weight"} adds top-K distillation; ``loss_scale_override`` replaces the
        default 1 / (global number of target tokens) normalisation."""
        cfg = self.cfg
        B, GA, T = cfg.batch_size, cfg.grad_accum, inputs.shape[1]
        inp = self._stage("inputs", self._local_slice(inputs))
        tgt = self._stage("targets", self._local_slice(targets))
        if position_ids is None:
            pos = torch.arange(T, dtype=torch.int32, device=self.device)[None].expand(B * GA, T).contiguous()
            doc_ids = None
        else:
            pos = self._stage("position_ids", self._local_slice(position_ids))
            doc_ids = None
            if bool((position_ids[:, 1:] <= position_ids[:, :-1]).any()) if isinstance(position_ids, np.ndarray) else False:
                doc_ids = torch.cumsum((pos == 0).to(torch.int32), dim=1)  # packed documents: id increments at each reset
        n_valid = (tgt != -100).sum().to(torch.float32)
        if self.world > 1:
            self.comm.all_reduce(n_valid, "sum")
        loss_scale = (1.0 / n_valid.clamp_min(1.0)).reshape(1)
        if loss_scale_override is not None:
            loss_scale = torch.full((1,), float(loss_scale_override), dtype=torch.float32, device=self.device)
        if row_weights is not None:
            row_weights = self._stage("row_weights", self._local_slice(row_weights), dtype=torch.float32)
        if kd is not None:
            kd = dict(kd, idx=self._stage("kd_idx", self._local_slice(kd["idx"])), logp=self._stage("kd_logp", self._local_slice(kd["logp"]), dtype=torch.float32))
        if self.device.type != "cuda":
            loss_scale = float(loss_scale)
        aux_scale = 1.0 / (GA * self.world)
        self.store.begin_step()
        self.recipe.begin_step(self.step_index)
        loss_sum = torch.zeros((), dtype=torch.float32, device=self.device)
        aux_sum = torch.zeros((), dtype=torch.float32, device=self.device)
        stats = []
        for i in range(GA):
            self.store.begin_micro_step(i, GA)
            sl = slice(i * B, (i + 1) * B)
            if self._graphs_allowed(doc_ids, row_weights, kd):
                ctx, outs = self._graphed_forward_backward(inp[sl], pos[sl], tgt[sl], loss_scale, aux_scale, i, GA)
            elif cfg.sequence_chunks > 1:
                if doc_ids is not None or row_weights is not None or kd is not None or self._visual is not None:
                    raise NotImplementedError("sequence_chunks runs the plain next-token objective on unpacked, text-only rows")
                ctx, outs = self._chunked_forward_backward(inp[sl], pos[sl], tgt[sl], loss_scale, aux_scale, i, GA)
            else:
                ctx, outs = self.executor.forward_backward(inp[sl], pos[sl], tgt[sl], loss_scale=loss_scale, aux_scale=aux_scale,
                                                           doc_ids=doc_ids[sl] if doc_ids is not None else None, micro_step=i,
                                                           row_weights=row_weights[sl] if row_weights is not None else None,
                                                           kd=dict(kd, idx=kd["idx"][sl], logp=kd["logp"][sl]) if kd is not None else None,
                                                           extras=self._extras(sl))
            loss_sum += outs[0]
            if len(outs) > 1 and outs[1] is not None:
                aux_sum += outs[1] * aux_scale
            stats.extend(ctx.moe_stats)
        self.last_moe_stats = stats
        if self.lora is not None:
            self.lora.reduce_grads()
        self.store.finish_reduce()
        return {"loss_sum": loss_sum, "n_valid": n_valid, "aux": aux_sum}

    # ------------------------------------------------------------------ CUDA graphs
    def _graphs_allowed(self, doc_ids, row_weights, kd) -> bool:
        """Graph replay needs a step whose launches do not depend on Python state that changes between steps: no collective
        inside the captured region (the peer-memory kernels pass a barrier epoch as a kernel argument; so one GPU, or replicated
        weights with the gradient reductions issued after the replay), dense model, no streamed weights or optimizer
        state, no per-batch side inputs, a recipe without step-dependent seeds, and scaling history already present (the
        first two steps of this process run eagerly, also after a resume: they are the warm-up that graph capture requires)."""
        c = self.cfg
        multi_ok = self.world == 1 or c.zero_level <= 1  # replicated weights: the gradient reductions run after the replay, outside the graph
        if self.executor.op_profile is not None or self.executor.options.dump_tensors is not None or self.executor.options.check_finite:
            return False  # all three read results back op by op, which a captured region cannot do
        return bool(c.use_cuda_graphs and self.device.type == "cuda" and self.backend.name == "cuda" and multi_ok and self.lora is None
                    and self.ep is None and not (c.offload_master or c.offload_optimizer or c.cpu_training or c.qlora or c.offload_saved_tensors or c.lmhead_drop_ignored_rows or c.time_breakdown)
                    and c.sequence_chunks <= 1
                    and doc_ids is None and row_weights is None and kd is None and self._visual is None and not getattr(self.model, "num_experts", 0)
                    and type(self.recipe).__name__ in ("BF16Recipe", "Recipe", "FP8HybridRecipe") and getattr(self, "_steps_here", 0) >= 2)

    def _graphed_forward_backward(self, inp, pos, tgt, loss_scale, aux_scale, index: int, total: int):
        """One micro-batch through a captured graph.  Inputs are copied into static buffers; there is one graph per
        (first micro-batch?, last micro-batch?) combination because the first one overwrites the gradient buffers and the
        later ones accumulate.  All graphs share one memory pool: tensors cached across micro-batches of a step (quantised
        weights) are produced by the first graph and read by the others."""
        g = self.__dict__.setdefault("_graphs", {"pool": None, "static": None, "by_key": {}})
        if g["static"] is None or g["static"]["inp"].shape != inp.shape:
            g["by_key"].clear()
            g["static"] = {"inp": inp.clone(), "pos": pos.clone(), "tgt": tgt.clone(), "scale": loss_scale.clone()}
            g["pool"] = torch.cuda.graph_pool_handle()
        st = g["static"]
        st["inp"].copy_(inp)
        st["pos"].copy_(pos)
        st["tgt"].copy_(tgt)
        st["scale"].copy_(loss_scale)
        key = (index == 0, index == total - 1)
        self.store.begin_micro_step(index, total)
        self.store.defer_reduce = self.world > 1
        entry = g["by_key"].get(key)
        if entry is None:
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            try:
                with torch.cuda.graph(graph, pool=g["pool"], capture_error_mode="thread_local"):  # other threads (data prefetch) may pin memory meanwhile
                    ctx, outs = self.executor.forward_backward(st["inp"], st["pos"], st["tgt"], loss_scale=st["scale"], aux_scale=aux_scale, micro_step=index)
            except Exception as e:  # noqa: BLE001 - an op in this configuration is not capturable: nothing ran, so run the step eagerly from here on
                import warnings

                warnings.warn(f"CUDA graph capture failed ({type(e).__name__}: {e}); continuing without graphs")
                self.cfg.use_cuda_graphs = False
                g["by_key"].clear()
                self.store.defer_reduce = False
                self.store.begin_micro_step(index, total)
                return self.executor.forward_backward(inp, pos, tgt, loss_scale=loss_scale, aux_scale=aux_scale, micro_step=index)
            entry = g["by_key"][key] = (graph, ctx, outs)
        entry[0].replay()  # capture records without executing, so a freshly captured graph is replayed too
        if self.world > 1:
            if index == total - 1:
                self.store.reduce_deferred()
            self.store.defer_reduce = False
        self.graph_replays = getattr(self, "graph_replays", 0) + 1
        return entry[1], entry[2]

    def _chunked_forward_backward(self, inp, pos, tgt, loss_scale, aux_scale, micro_index: int, micro_total: int):
        """One micro-batch of long rows in ``sequence_chunks`` pieces: pass A fills the per-layer key/value prefix left to
        right (block stack only, nothing saved), pass B walks right to left doing forward + backward per piece, so activation
        memory is that of one piece while keys / values (and their fp32 gradient accumulators) cover the whole row."""
        from .executor import ChunkState

        N, T = self.cfg.sequence_chunks, inp.shape[1]
        if T % N:
            raise ValueError(f"sequence length {T} is not divisible by sequence_chunks={N}")
        Tc = T // N
        ex = self.executor
        cs = ChunkState(N, Tc)
        for c in range(N):
            cs.index = c
            cols = slice(c * Tc, (c + 1) * Tc)
            ctx = ex.new_context(inp[:, cols], False)
            ctx.chunk = cs
            ex.stage_forward(ctx, (0, self.cm.n_layers), True, False, pos[:, cols].contiguous(), token_ids=inp[:, cols].contiguous())
            ex.detach_state()
        total = None
        for k, c in enumerate(reversed(range(N))):
            cs.index = c
            cols = slice(c * Tc, (c + 1) * Tc)
            self.store.begin_micro_step(micro_index * N + k, micro_total * N)
            ctx, outs = ex.forward_backward(inp[:, cols].contiguous(), pos[:, cols].contiguous(), tgt[:, cols].contiguous(), loss_scale=loss_scale,
                                            aux_scale=aux_scale / N, micro_step=micro_index * N + k, chunk=cs)
            total = list(outs) if total is None else [a + b if (a is not None and b is not None) else a for a, b in zip(total, outs)]
        if len(total) > 1 and total[1] is not None:
            total[1] = total[1] / N  # the auxiliary loss is a per-piece mean
        return ctx, total

    def grad_norm(self) -> torch.Tensor:
        """Global L2 norm of the (already reduced) gradients, as a device scalar.

        Three kinds of terms, each counted exactly once: dense buckets (replicated after an all-reduce, or one shard per rank under
        ZeRO), expert buckets (one copy per rank of an expert group; with an expert-parallel x data-parallel mesh the same copy exists
        in every replica of the group) and the adapter buffer (already all-reduced, identical everywhere)."""
        on_gpu = self.device.type == "cuda" and self.backend.name == "cuda"

        def sumsq(g):
            return self.backend.ext.sumsq(g) if on_gpu else g.float().pow(2).sum()

        fused = self.store.fused_sumsq is not None and self.store.sumsq_valid and self.lora is None
        parts = torch.zeros(2, dtype=torch.float32, device=self.device)   # [dense, experts]
        for b in self.store.trainable_buckets():
            if b.grad_shard is None:
                continue
            if b.expert:
                parts[1] += sumsq(b.grad_shard)
            elif not fused:
                parts[0] += sumsq(b.grad_shard)
        if fused:  # the reduce-scatter kernels already accumulated this rank's shard norms
            parts[0] += self.store.fused_sumsq.reshape(())
            if os.environ.get("SUROGATE_CHECK_FUSED_NORM") == "1":  # self-check: recompute from the reduced shards
                ref = sum(sumsq(b.grad_shard) for b in self.store.trainable_buckets() if b.grad_shard is not None and not b.expert)
                if abs(float(ref) - float(parts[0])) > 1e-2 * abs(float(ref)):
                    raise RuntimeError(f"fused gradient norm mismatch on rank {self.rank}: fused {float(parts[0])} vs recomputed {float(ref)}")
        if self.world > 1:
            dense_local = parts[0].clone()
            if self.store.sharded or self.store.ep > 1:
                self.comm.all_reduce(parts, "sum")
            if not self.store.sharded:
                parts[0] = dense_local                              # replicated gradients: every rank already holds the whole dense part
            parts[1] = parts[1] / float(self.store.expert_dp)      # each expert's gradient exists once per replica of the expert group
        total = parts[0] + parts[1]
        if self.lora is not None:
            # the adapter gradient is already all-reduced (identical on every rank): it joins after the cross-rank sum
            total = total + self.lora.grad_sumsq()
        return total.sqrt()

    def drain_optimizer(self) -> None:
        """With ``async_optimizer``: wait for the update in flight and make its weights the ones the next step reads."""
        flush = getattr(self.optimizer, "flush", None)
        if flush is not None and getattr(self.optimizer, "_pending", None):
            flush()
            for b in self.store.buckets.values():
                b.work_host_fresh = getattr(b, "work_host", None) is not None and getattr(b, "work_next", None) is not None
            self.store.sync_work_from_master()

    def optimizer_step(self, lr: Optional[float] = None, norm: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``norm``: the global gradient norm when this process holds only part of the model (pipeline stages)."""
        cfg = self.opt_cfg
        self.step_index += 1
        self._steps_here = getattr(self, "_steps_here", 0) + 1
        t = self.step_index
        lr = cfg.learning_rate if lr is None else lr
        norm = self.grad_norm() if norm is None else norm
        clip = torch.clamp(cfg.max_grad_norm / (norm + 1e-6), max=1.0) if cfg.max_grad_norm and cfg.max_grad_norm > 0 else torch.ones_like(norm)
        clip = torch.where(torch.isfinite(norm), clip, torch.zeros_like(clip))  # a non-finite norm skips the update: the optimizer kernels and CPU paths return early on a zero scale
        host = (lr, cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay, 1 - cfg.beta1 ** t, 1 - cfg.beta2 ** t)
        hp_cpu = torch.tensor(list(host) + [1.0], dtype=torch.float32)
        self._hp.copy_(hp_cpu, non_blocking=True)
        self._hp[7] = clip
        fence = getattr(self.comm, "fence", None)
        if fence is not None:
            fence()  # every rank has finished reading master shards / gradient buckets of this step
        if self.cfg.cpu_training:
            self.optimizer.step_all([b for b in self.store.trainable_buckets() if not b.expert], lr, float(clip), t)  # host sync: clip scale
        elif self.streamed is not None:
            self.streamed.run(self.store.trainable_buckets(), self._hp, host)
        else:
            for b in self.store.trainable_buckets():
                if b.grad_shard is None:
                    continue
                self.optimizer.step_bucket(b, b.grad_shard, self._hp, host)
        if self.lora is not None:
            self.lora.optimizer_step(self._hp, host)
        self.store.release_grads()
        self.store.sync_work_from_master()
        # the initial placement is arbitrary, so the first decision comes after two steps of this process; later ones every interval
        refresh_now = self.cfg.ep_plan_refresh_interval > 0 and (self.step_index % self.cfg.ep_plan_refresh_interval == 0 or self._steps_here == 2)
        if self.ep is not None and refresh_now and self.cfg.optimizer in ("adamw", "adamw_8bit") and not self.cfg.cpu_training:
            self.last_rebalance = self.ep.rebalance(self.store, self.optimizer, self.cfg.ep_load_balance_threshold)
        self.recipe.on_weights_updated(self.store)
        self.recipe.end_step()
        return norm

    def step(self, inputs, targets, position_ids=None, lr: Optional[float] = None, kd=None, row_weights=None) -> Dict[str, float]:
        r = self.forward_backward(inputs, targets, position_ids, row_weights=row_weights, kd=kd)
        timer = self.executor.timer
        if timer is not None:
            timer.mark("start")
        norm = self.optimizer_step(lr)
        if timer is not None:
            timer.mark("optimizer")
            self.last_time_breakdown = timer.totals()
        loss = r["loss_sum"].clone()
        if self.world > 1:
            self.comm.all_reduce(loss, "sum")
        out = torch.stack([loss / r["n_valid"].clamp_min(1.0) + r["aux"], norm, r["aux"]]).to("cpu")  # the step's only D2H sync
        self.d2h_bytes += out.numel() * 4
        if self.device.type == "cuda" and self.backend.name == "cuda":
            from ..ops import check_device_errors

            check_device_errors()
        return {"loss": float(out[0]), "norm": float(out[1]), "aux_loss": float(out[2])}

    # ------------------------------------------------------------------ call-compatible spellings of the reference's Python API
    def train_step_graphed(self, inputs, targets, position_ids=None, lr: Optional[float] = None) -> Dict[str, float]:
        """``step`` with CUDA-graph replay of forward + backward switched on (falls back to eager where graphs do not apply).
        Parity: SurogateTrainer.train_step_graphed (csrc/src/binding/py_train.h)."""
        self.cfg.use_cuda_graphs = True
        return self.step(inputs, targets, position_ids, lr=lr)

    def update_with_config(self, opt_config: Any, step: Optional[int] = None) -> Dict[str, float]:
        """Optimizer update after one or more ``forward_backward`` calls, with hyper-parameters taken from ``opt_config`` (a dict
        or an object with learning_rate / weight_decay / beta1 / beta2 / eps / max_grad_norm).  ``step`` is the 1-based number of
        this update (the ``t`` of Adam's bias correction), as callers of the reference API pass it.  Returns {"norm": ...}.
        Parity: SurogateTrainer.update_with_config."""
        get = opt_config.get if isinstance(opt_config, dict) else (lambda k, d=None: getattr(opt_config, k, d))
        for mine, theirs in (("weight_decay", "weight_decay"), ("beta1", "beta1"), ("beta2", "beta2"), ("eps", "eps"), ("max_grad_norm", "max_grad_norm"),
                             ("beta1", "adamw_beta1"), ("beta2", "adamw_beta2"), ("eps", "adamw_epsilon")):
            v = get(theirs, None)
            if v is not None:
                setattr(self.opt_cfg, mine, float(v))
        if step is not None:
            self.step_index = max(0, int(step) - 1)  # optimizer_step counts this update itself
        norm = self.optimizer_step(get("learning_rate", None))
        return {"norm": float(norm)}

    @torch.no_grad()
    def token_logprobs(self, inputs, targets, position_ids=None, use_adapters: bool = True) -> torch.Tensor:
        """log p(target_t | prefix) for every position ([rows, T] float32 on the device, 0 where the target is ignored).
        ``use_adapters=False`` runs the frozen base model of a LoRA run (the DPO / GRPO reference policy)."""
        inp = self._stage("lp_inputs", inputs)
        tgt = self._stage("lp_targets", targets)
        rows, T = inp.shape
        if position_ids is None:
            pos = torch.arange(T, dtype=torch.int32, device=self.device)[None].expand(rows, T).contiguous()
        else:
            pos = self._stage("lp_pos", position_ids)
        out = torch.empty(rows, T, dtype=torch.float32, device=self.device)
        self.store.grads_enabled = False
        saved_lora = self.executor.lora
        if not use_adapters:
            self.executor.lora = None
        try:
            B = max(1, self.cfg.batch_size)
            for s in range(0, rows, B):
                ctx, _ = self.executor.forward(inp[s:s + B], pos[s:s + B], tgt[s:s + B], training=False, want_token_losses=True,
                                               extras=self._extras(slice(s, s + B)))
                out[s:s + B] = -ctx.stash["token_losses"].reshape(-1, T)
        finally:
            self.store.grads_enabled = True
            self.executor.lora = saved_lora
        return out

    @torch.no_grad()
    def logits(self, inputs, position_ids=None) -> torch.Tensor:
        """Full logits [rows, T, V] (fp32) — for teacher capture and debugging, not a training path."""
        self.drain_optimizer()
        inp = self._stage("lg_inputs", inputs)
        rows, T = inp.shape
        pos = torch.arange(T, dtype=torch.int32, device=self.device)[None].expand(rows, T).contiguous() if position_ids is None \
            else self._stage("lg_pos", position_ids)
        tgt = torch.full_like(inp, -100)
        captured = {}
        prev = self.executor.options.dump_tensors
        self.executor.options.dump_tensors = lambda name, layer, val: captured.__setitem__(name, val) if layer is None else None
        self.store.grads_enabled = False
        try:
            self.executor.forward(inp, pos, tgt, training=False, extras=self._extras(slice(0, rows)))
        finally:
            self.executor.options.dump_tensors = prev
            self.store.grads_enabled = True
        fwd = self.cm.fwd
        head = next(op for op in fwd.ops if op.kind == "fused_lm_head_loss")
        x = captured[head.inputs[0]]
        if not torch.is_tensor(x):
            x = x.hp if getattr(x, "hp", None) is not None else x.dequantize()
        w = self.store.get(head.inputs[1])
        out = (x.reshape(-1, x.shape[-1]).float() @ w.float().t()).reshape(rows, T, -1)
        cap = float(head.attrs.get("softcap") or 0.0)
        return cap * torch.tanh(out / cap) if cap else out

    @torch.no_grad()
    def validate(self, inputs, targets, position_ids=None) -> Dict[str, float]:
        self.drain_optimizer()
        inp = self._stage("v_inputs", inputs)
        tgt = self._stage("v_targets", targets)
        T = inp.shape[1]
        pos = torch.arange(T, dtype=torch.int32, device=self.device)[None].expand(inp.shape[0], T).contiguous()
        self.store.grads_enabled = False
        try:
            ctx, outs = self.executor.forward(inp, pos, tgt, training=False, extras=self._extras(slice(0, inp.shape[0])))
        finally:
            self.store.grads_enabled = True
        n = (tgt != -100).sum().clamp_min(1).float()
        loss = outs[0].clone()
        if self.world > 1:
            self.comm.all_reduce(loss, "sum")
            self.comm.all_reduce(n, "sum")
        return {"loss": float(loss / n)}

    # ------------------------------------------------------------------ introspection
    def get_gradients(self) -> Dict[str, torch.Tensor]:
        return {p.name: self.store.grad_of(p.name) for p in self.cm.params if not p.tied_to}

    def get_moe_stats(self):
        from ..utils.moe_stats import summarize

        return summarize(self.last_moe_stats or [])

    def get_gpu_info(self):
        from ..utils.gpu_info import gpu_info

        return gpu_info(self.device)

    def num_parameters(self) -> int:
        return self.cm.num_parameters()

    def activation_plan(self):
        """Static buffer plan of the block graphs for this configuration's micro-batch (``dsl/graph_compiler.py: plan_model``)."""
        from ..dsl.graph_compiler import plan_model

        act = 2 if self.cfg.param_dtype in ("bf16", "fp16") else 4
        return plan_model(self.cm, self.cfg.batch_size, self.cfg.seq_len, self.cfg.recompute, act_bytes=act)

    def memory_breakdown(self) -> Dict[str, int]:
        """Bytes by use (``master`` / ``work`` / ``grad`` / ...), by category and memory kind from the native allocation registry
        (``category.*``, ``kind.*``), the transient stack's high-water mark, and the allocator's totals on a GPU."""
        out = self.store.memory_breakdown()
        try:
            from .memory import registry_for

            reg = registry_for(self)
            out.update({f"category.{k}": int(v) for k, v in reg.by_category().items()})
            out.update({f"kind.{k}": int(v) for k, v in reg.by_kind().items()})
        except Exception:  # noqa: BLE001 - the host runtime is not built: the coarse numbers above remain
            pass
        stack = getattr(self.backend, "stack", None)
        if stack is not None:
            out["stack_high_water"] = stack.high_water
        try:   # the graph compiler's static plan: what one micro-batch's activations will need, known before the first step
            plan = self.activation_plan()
            out["planned.saved_activations"] = int(plan.saved_bytes)
            out["planned.temporaries"] = int(plan.temp_bytes)
        except Exception:  # noqa: BLE001 - a graph with run-time-only dimensions everywhere
            pass
        if self.device.type == "cuda":
            out["allocated"] = torch.cuda.memory_allocated(self.device)
            out["reserved"] = torch.cuda.memory_reserved(self.device)
            out["peak"] = torch.cuda.max_memory_allocated(self.device)
        return out
