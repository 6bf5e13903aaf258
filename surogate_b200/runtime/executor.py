"""Graph executor: runs compiled forward/backward op lists against a parameter store.

One flat interpreter loop per graph: look up the op's implementation on the
backend object, call it, bind outputs, and drop every tensor after its last
reader (liveness is computed once per graph, ahead of time).  The block stack is
unrolled here, which is where per-layer behaviour lives:

* ``store.layer_start / layer_end`` hooks (ZeRO-3 weight gather + prefetch,
  gradient bucket reduce overlapped with the next layer's backward),
* which forward tensors a layer keeps for its backward (the AOT "saved" list) or,
  with ``recompute``, only the block inputs followed by a replay of the layer's
  forward just before its backward.

Parity: csrc/src/runtime/executor/ (GraphExecutor graph_executor.h:185,
CompiledExecutor, handle_layer_start/end compiled_ops.cpp:982-1074,
replay_layer_forward compiled_ops_execute.cpp:85).
"""
from __future__ import annotations

import os

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Set, Tuple

import torch

from ..dsl.autodiff import GRAD_PREFIX
from ..dsl.compiler import CompiledModel
from ..dsl.graph_compiler import bake_program
from ..dsl.ir import Graph, OpNode, eval_shape

_DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16, "int32": torch.int32}


@dataclass
class ExecOptions:
    recompute: bool = False
    act_dtype: torch.dtype = torch.float32
    check_finite: bool = False
    lmhead_drop_ignored_rows: bool = False  # compact away rows with ignored targets before the LM head (one host sync per micro-batch)
    time_breakdown: bool = False             # CUDA-event marks around forward / LM head / backward / optimizer (read with PhaseTimer.totals)
    offload_saved: bool = False              # park each layer's saved tensors (or, with recompute, its input checkpoint) in pinned host memory
    dump_tensors: Optional[Callable[[str, Optional[int], torch.Tensor], None]] = None


class ExecContext:
    """Per-call state handed to every op implementation."""

    def __init__(self, executor: "Executor"):
        ex = executor
        self.ex = ex
        self.device = ex.device
        self.act_dtype = ex.options.act_dtype
        self.recipe = ex.recipe
        self.training = True
        self.dims: Dict[str, int] = {}
        self.layer: Optional[int] = None
        self.graph: Optional[Graph] = None
        self.stash: Dict[str, Any] = {}
        self.loss_scale: Any = 1.0
        self.aux_scale: float = 1.0
        self.doc_ids: Optional[torch.Tensor] = None
        self.ep = ex.ep
        self.micro_step = 0
        self.phase = "fwd"
        self.moe_stats: List[Tuple[int, torch.Tensor, torch.Tensor]] = []
        self.lora = ex.lora
        # objective hooks read by the fused LM-head loss op
        self.row_weights: Optional[torch.Tensor] = None    # [tokens] multiplier on each token's log-likelihood gradient (DPO / GRPO)
        self.kd: Optional[Dict[str, Any]] = None           # {"idx": int32 [tokens, K], "logp": fp32 [tokens, K], "weight": float, "ce_weight": float}
        self.want_token_losses = False                     # leave per-token CE in stash["token_losses"] (and KD in stash["token_kd"])
        # per-batch side inputs that are not graph values (multimodal: visual_pos_masks, visual_embeds, deepstack_visual_embeds,
        # mrope_position_ids); ``torch_fn`` ops name the ones they read in their ``side_inputs`` attribute
        self.extras: Dict[str, Any] = {}
        # chunked-sequence training: the attention op reads / extends the per-layer key-value prefix kept here
        self.chunk: Optional["ChunkState"] = None
        # values that cross layer boundaries outside the block interface, and the gradients flowing back to their producers
        self.shared: Dict[str, torch.Tensor] = {}
        self.shared_grad: Dict[str, torch.Tensor] = {}

    def eval_shape(self, shape) -> Tuple[int, ...]:
        return eval_shape(tuple(shape), self.dims)

    def dtype_of(self, tag: str) -> torch.dtype:
        return self.act_dtype if tag in ("act", "param") else _DTYPES[tag]

    def full_name(self, local: str) -> str:
        return f"blocks.{self.layer}.{local}" if self.layer is not None else local

    def grad_target(self, out_name: Optional[str]):
        """(gradient buffer view, accumulate?) for a ``grad::<param>`` output, or (None, False) if frozen/absent."""
        if out_name is None:
            return None, False
        local = out_name[len(GRAD_PREFIX):] if out_name.startswith(GRAD_PREFIX) else out_name
        return self.ex.store.grad_target(self.full_name(local))

    def local_experts(self, w: torch.Tensor) -> torch.Tensor:
        return w

    def record_moe_stats(self, counts: torch.Tensor, probs: torch.Tensor) -> None:
        if self.phase == "fwd" and self.layer is not None:
            self.moe_stats.append((self.layer, counts.detach(), probs.detach().mean(0)))


class PhaseTimer:
    """Marks on the launching stream; the time between two marks is attributed to the later mark's name.
    Parity: debug_time_breakdown (csrc/src/runtime/training/model.h:323-333, py_train.cpp:577-597)."""

    def __init__(self, device: torch.device):
        self.cuda = device.type == "cuda"
        self.marks: List[Tuple[str, Any]] = []

    def mark(self, name: str) -> None:
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.marks.append((name, e))
        else:
            import time

            self.marks.append((name, time.perf_counter()))

    def totals(self) -> Dict[str, float]:
        """Milliseconds per phase since the last call (synchronises the device once)."""
        out: Dict[str, float] = {}
        if self.cuda and self.marks:
            self.marks[-1][1].synchronize()
        for (_, a), (name, b) in zip(self.marks, self.marks[1:]):
            if name == "start":
                continue
            out[name + "_ms"] = out.get(name + "_ms", 0.0) + (a.elapsed_time(b) if self.cuda else (b - a) * 1e3)
        self.marks = []
        return out


class SavedTensorOffload:
    """Per-layer saved tensors in pinned host memory between a layer's forward and its backward.

    ``push`` starts device -> host copies on a side stream as soon as the layer's forward has produced the tensors and lets the
    caching allocator reuse the device memory once the copies are done; ``prefetch`` starts the copies back one layer ahead of
    the backward sweep; ``fetch`` makes the compute stream wait for them.  With per-layer recompute only the layer's input
    checkpoint is saved, so activation memory on the device stays O(1) in the number of layers.
    Parity: offload_saved_tensors / offload_residual (csrc/src/runtime/executor/compiled_ops.cpp:982-1055, docs/guides/offloading.md)."""

    MIN_BYTES = 1 << 16

    def __init__(self, device: torch.device):
        self.device = device
        self.stream = torch.cuda.Stream(device=device)
        self.free: Dict[Tuple[Tuple[int, ...], torch.dtype], List[torch.Tensor]] = {}
        self.inflight: Dict[int, Tuple[Dict[str, Any], Any]] = {}
        self.bytes_out = 0

    def _pinned(self, t: torch.Tensor) -> torch.Tensor:
        key = (tuple(t.shape), t.dtype)
        pool = self.free.setdefault(key, [])
        return pool.pop() if pool else torch.empty(t.shape, dtype=t.dtype, pin_memory=True)

    def _out(self, v):
        if torch.is_tensor(v) and v.is_cuda and v.numel() * v.element_size() >= self.MIN_BYTES:
            h = self._pinned(v)
            h.copy_(v, non_blocking=True)
            v.record_stream(self.stream)
            self.bytes_out += h.numel() * h.element_size()
            return ("host", h)
        return ("keep", v)

    def push(self, saved: Dict[str, Any]) -> Dict[str, Any]:
        ready = torch.cuda.Event()
        ready.record()
        self.stream.wait_event(ready)
        out: Dict[str, Any] = {}
        seen: Dict[int, str] = {}
        with torch.cuda.stream(self.stream):
            for k, v in saved.items():
                if id(v) in seen:  # the same object saved under two names: move it once
                    out[k] = ("same", seen[id(v)])
                    continue
                seen[id(v)] = k
                if hasattr(v, "scale_inv") and not torch.is_tensor(v):  # quantised activation: move its payload, rebuild the wrapper on the way back
                    out[k] = ("fp8", type(v), v.scale_inv, self._out(v.data), self._out(v.hp) if getattr(v, "hp", None) is not None else None)
                else:
                    out[k] = self._out(v)
        done = torch.cuda.Event()
        done.record(self.stream)
        return {"__offloaded__": out, "__done__": done}

    def _in(self, item, used: List[torch.Tensor]):
        kind, v = item
        if kind == "keep":
            return v
        d = torch.empty(v.shape, dtype=v.dtype, device=self.device)
        d.copy_(v, non_blocking=True)
        used.append(v)
        return d

    def prefetch(self, layer: int, parked: Dict[str, Any]) -> None:
        if layer in self.inflight or "__offloaded__" not in parked:
            return
        self.stream.wait_event(parked["__done__"])
        out: Dict[str, Any] = {}
        used: List[torch.Tensor] = []
        with torch.cuda.stream(self.stream):
            for k, item in parked["__offloaded__"].items():
                if item[0] == "same":
                    continue
                if item[0] == "fp8":
                    _, cls, scale_inv, data, hp = item
                    out[k] = cls(self._in(data, used), scale_inv, self._in(hp, used) if hp is not None else None)
                else:
                    out[k] = self._in(item, used)
            for k, item in parked["__offloaded__"].items():
                if item[0] == "same":
                    out[k] = out[item[1]]
        ev = torch.cuda.Event()
        ev.record(self.stream)
        self.inflight[layer] = (out, (ev, used))

    def fetch(self, layer: int, parked: Dict[str, Any]) -> Dict[str, Any]:
        if "__offloaded__" not in parked:
            return parked
        self.prefetch(layer, parked)
        out, (ev, used) = self.inflight.pop(layer)
        cur = torch.cuda.current_stream(self.device)
        cur.wait_event(ev)
        for v in out.values():
            for t in ((v,) if torch.is_tensor(v) else (getattr(v, "data", None), getattr(v, "hp", None))):
                if torch.is_tensor(t) and t.is_cuda:
                    t.record_stream(cur)
        for h in used:  # pinned buffers return to the pool: their copies back were issued, and later pushes run on the same side stream
            self.free.setdefault((tuple(h.shape), h.dtype), []).append(h)
        return out


class ChunkState:
    """Key / value prefix and its gradient accumulators for training one long sequence in ``n_chunks`` pieces.

    Pass A runs the chunks left to right without saving activations; each attention layer appends its rotated keys and values
    here.  Pass B runs them right to left as ordinary forward + backward steps: a chunk attends to the frozen prefix plus its own
    rows, its backward adds dK / dV for every row it attended to into the fp32 accumulators, and the gradient it takes for its
    own keys and values is the accumulated one, which by then holds the contributions of all later chunks.
    Parity: csrc/src/binding/py_train.cpp:649-714, csrc/src/runtime/attention/backend_kvprefix.cpp."""

    def __init__(self, n_chunks: int, chunk_len: int):
        self.n_chunks, self.chunk_len = int(n_chunks), int(chunk_len)
        self.index = 0
        self.k: Dict[int, torch.Tensor] = {}
        self.v: Dict[int, torch.Tensor] = {}
        self.dk: Dict[int, torch.Tensor] = {}
        self.dv: Dict[int, torch.Tensor] = {}

    def store_kv(self, layer: int, k: torch.Tensor, v: torch.Tensor) -> None:
        B, Tc = k.shape[:2]
        if layer not in self.k:
            shape = (B, self.n_chunks * self.chunk_len) + tuple(k.shape[2:])
            self.k[layer], self.v[layer] = torch.empty(shape, dtype=k.dtype, device=k.device), torch.empty(shape, dtype=v.dtype, device=v.device)
        a = self.index * self.chunk_len
        self.k[layer][:, a:a + Tc].copy_(k)
        self.v[layer][:, a:a + Tc].copy_(v)

    def grad_buffers(self, layer: int):
        if layer not in self.dk:
            self.dk[layer] = torch.zeros(self.k[layer].shape, dtype=torch.float32, device=self.k[layer].device)
            self.dv[layer] = torch.zeros(self.v[layer].shape, dtype=torch.float32, device=self.v[layer].device)
        return self.dk[layer], self.dv[layer]


class Executor:
    def __init__(self, compiled: CompiledModel, store, backend, recipe=None, options: Optional[ExecOptions] = None,
                 device: Optional[torch.device] = None, ep=None, lora=None):
        self.cm = compiled
        self.store = store
        self.backend = backend
        self.recipe = recipe
        self.options = options or ExecOptions()
        if self.options.dump_tensors is None and os.environ.get("SUROGATE_DEBUG_DUMP_TENSORS"):
            from ..debug.dump import env_dump_hook  # file dumps of named tensors, switched on by the environment

            self.options.dump_tensors = env_dump_hook()
        if os.environ.get("SUROGATE_DEBUG_CHECK_NONFINITE", "0") not in ("", "0"):
            self.options.check_finite = True  # every op output is tested; the first NaN / Inf raises with the tensor, layer and op named
        self.device = device or torch.device("cpu")
        self.op_profile = None  # debug.op_profile.OpProfile: time per op kind (SUROGATE_OP_PROFILE=1, or set by the caller)
        if os.environ.get("SUROGATE_OP_PROFILE"):
            from ..debug.op_profile import env_op_profile

            self.op_profile = env_op_profile(self.device)
        self.ep = ep
        self.lora = lora
        self._liveness: Dict[int, Dict[str, int]] = {}
        self._programs: Dict[Any, Any] = {}
        self._saved_sets: Dict[str, Set[str]] = {}
        for bt, bwd in self.cm.block_bwd.items():
            self._saved_sets[bt] = set(bwd.meta["saved"])
        self._top_saved: Set[str] = set(self.cm.bwd.meta["saved"])
        self._layer_saved: List[Optional[Dict[str, Any]]] = [None] * self.cm.n_layers
        self._top_env: Dict[str, Any] = {}
        self.layer_range: Optional[Tuple[int, int]] = None  # pipeline stage: the block stack runs only layers [first, last)
        self.timer = PhaseTimer(self.device) if self.options.time_breakdown else None
        self.offload = SavedTensorOffload(self.device) if (self.options.offload_saved and self.device.type == "cuda") else None

    # ------------------------------------------------------------------ generic graph run
    def _last_use(self, g: Graph) -> Dict[str, int]:
        key = id(g)
        if key not in self._liveness:
            self._liveness[key] = g.last_use()
        return self._liveness[key]

    def run_graph(self, g: Graph, env: Dict[str, Any], ctx: ExecContext, keep: Set[str], ops: Optional[List[OpNode]] = None) -> None:
        """Interpret ``g`` (or only ``ops``, a subsequence of its ops: pipeline stages run the part of the top-level graph
        before, inside or after the block stack)."""
        prev_graph = ctx.graph
        ctx.graph = g
        get_param = self.store.get
        key = (id(g), id(ops) if ops is not None else 0, frozenset(keep))
        program = self._programs.get(key)
        if program is None:   # bound methods, input classes and free lists are resolved once per (graph, op range, keep set)
            program = self._programs[key] = (bake_program(g, self.backend, set(keep), ops), ops)   # holding ``ops`` keeps its id unique
        for baked in program[0]:
            op = baked.op
            if self.timer is not None and op.kind == "fused_lm_head_loss":
                self.timer.mark("forward")
            if op.kind == "block_stack":
                outs = self._block_stack_forward(op, env, ctx)
            elif op.kind == "block_stack_backward":
                outs = self._block_stack_backward(op, env, ctx)
            else:
                ins = [None if c == 0 else (get_param(ctx.full_name(n)) if c == 1 else env.get(n)) for c, n in baked.sources]
                outs = baked.fn(ctx, op, *ins) if self.op_profile is None else self.op_profile.timed(op.kind, baked.fn, ctx, op, *ins)
            if self.timer is not None and op.kind == "fused_lm_head_loss":
                self.timer.mark("lm_head")  # in training mode this includes the head's own backward (fused)
            for name, val in zip(op.outputs, outs):
                if name is None:
                    continue
                if name.startswith(GRAD_PREFIX):
                    if val is not None:
                        self._accumulate_grad(ctx, name, val)
                    continue
                env[name] = val
                if self.options.dump_tensors is not None and torch.is_tensor(val):
                    self.options.dump_tensors(name, ctx.layer, val)
                if self.options.check_finite and torch.is_tensor(val) and val.is_floating_point() and not torch.isfinite(val).all():
                    raise FloatingPointError(f"non-finite values in '{name}' (layer {ctx.layer}, op {op.kind})")
            for n in baked.frees:
                env.pop(n, None)
        ctx.graph = prev_graph

    def _accumulate_grad(self, ctx: ExecContext, out_name: str, val: torch.Tensor) -> None:
        tgt, acc = ctx.grad_target(out_name)
        if tgt is None:
            return
        v = val.reshape(tgt.shape).to(tgt.dtype)
        if acc:
            tgt.add_(v)
        else:
            tgt.copy_(v)

    # ------------------------------------------------------------------ block stack
    def _block_stack_forward(self, op: OpNode, env, ctx: ExecContext):
        x, res, pos = (env[n] for n in op.inputs)
        aux_names: List[str] = op.attrs.get("aux", [])
        aux_tot = [None] * len(aux_names)
        lo, hi = self.layer_range or (0, self.cm.n_layers)
        for L in range(lo, hi):
            bt = self.cm.layer_types[L]
            g = self.cm.block_fwd[bt]
            ctx.layer = L
            self.store.layer_start(L, "fwd")
            benv = {"x": x, "residual": res, "position_ids": pos}
            if ctx.training and self.options.recompute:
                keep: Set[str] = set(g.outputs)
                self._layer_saved[L] = {"x": x, "residual": res, "position_ids": pos, "__recompute__": True}
            else:
                keep = (self._saved_sets[bt] if ctx.training else set()) | set(g.outputs)
            self.run_graph(g, benv, ctx, keep)
            outs = [benv[o] for o in g.outputs]
            x, res = outs[0], outs[1]
            for i, a in enumerate(outs[2:]):
                aux_tot[i] = a if aux_tot[i] is None else aux_tot[i] + a
            if ctx.training and not self.options.recompute:
                self._layer_saved[L] = {k: v for k, v in benv.items() if k in self._saved_sets[bt]}
            if ctx.training and self.offload is not None and self._layer_saved[L] is not None and L < hi - 1:  # the last layer's backward starts right away
                self._layer_saved[L] = self.offload.push(self._layer_saved[L])
            self.store.layer_end(L, "fwd")
        ctx.layer = None
        return [x, res] + aux_tot

    def _block_stack_backward(self, op: OpNode, env, ctx: ExecContext):
        d_x, d_res = env.get(op.inputs[0]), env.get(op.inputs[1])
        d_aux = [env.get(n) if n is not None else None for n in op.inputs[2:]]
        aux_names: List[str] = op.attrs.get("aux", [])
        lo, hi = self.layer_range or (0, self.cm.n_layers)
        for L in reversed(range(lo, hi)):
            bt = self.cm.layer_types[L]
            fg, bg = self.cm.block_fwd[bt], self.cm.block_bwd[bt]
            ctx.layer = L
            self.store.layer_start(L, "bwd")
            saved = self._layer_saved[L]
            self._layer_saved[L] = None
            if self.offload is not None:
                saved = self.offload.fetch(L, saved)
                if L - 1 >= lo and self._layer_saved[L - 1] is not None:
                    self.offload.prefetch(L - 1, self._layer_saved[L - 1])  # copies back overlap this layer's backward
            if saved.get("__recompute__"):
                benv = {k: v for k, v in saved.items() if k != "__recompute__"}
                ctx.phase = "recompute"
                self.run_graph(fg, benv, ctx, self._saved_sets[bt] | set(fg.outputs))
                ctx.phase = "bwd"
                saved = {k: v for k, v in benv.items() if k in self._saved_sets[bt]}
            benv = dict(saved)
            og = bg.meta["out_grads"]
            benv[og[fg.outputs[0]]] = d_x
            benv[og[fg.outputs[1]]] = d_res
            for i, a in enumerate(fg.outputs[2:]):
                benv[og[a]] = d_aux[i] if i < len(d_aux) else None
            if d_res is None:
                # residual stream gradient absent (never happens after a final norm, kept for generality)
                benv[og[fg.outputs[1]]] = torch.zeros_like(d_x)
            self.run_graph(bg, benv, ctx, set(bg.outputs))
            ig = bg.meta["input_grads"]
            d_x, d_res = benv[ig["x"]], benv[ig["residual"]]
            self.store.layer_end(L, "bwd")
        ctx.layer = None
        return [d_x, d_res]

    # ------------------------------------------------------------------ public API
    def new_context(self, token_ids: torch.Tensor, training: bool) -> ExecContext:
        ctx = ExecContext(self)
        ctx.training = training
        ctx.dims = {"B": int(token_ids.shape[0]), "T": int(token_ids.shape[1])}
        return ctx

    def forward(self, token_ids, position_ids, targets, *, training: bool = True, loss_scale: Any = 1.0,
                aux_scale: float = 1.0, doc_ids=None, micro_step: int = 0, row_weights=None, kd=None,
                want_token_losses: bool = False, extras: Optional[Dict[str, Any]] = None, chunk=None) -> Tuple[ExecContext, List[Any]]:
        """Run the forward graph.  In training mode the LM-head op also produces d_x / d_w (fused loss backward)."""
        ctx = self.new_context(token_ids, training)
        ctx.loss_scale, ctx.aux_scale, ctx.doc_ids, ctx.micro_step = loss_scale, aux_scale, doc_ids, micro_step
        ctx.row_weights, ctx.kd, ctx.want_token_losses = row_weights, kd, want_token_losses
        ctx.extras = dict(extras or {})
        ctx.chunk = chunk
        ctx.phase = "fwd"
        if self.timer is not None:
            self.timer.mark("start")
        g = self.cm.fwd
        env = {"token_ids": token_ids, "position_ids": position_ids, "targets": targets}
        self.store.group_start("embedding", "fwd")
        keep = (self._top_saved if training else set()) | set(g.outputs)
        self.run_graph(g, env, ctx, keep)
        self._top_env = env
        if self.timer is not None:
            self.timer.mark("forward")
        return ctx, [env[o] for o in g.outputs]

    def backward(self, ctx: ExecContext) -> None:
        g, bg = self.cm.fwd, self.cm.bwd
        env = {k: v for k, v in self._top_env.items() if k in self._top_saved or k in g.inputs}
        self._top_env = {}
        og = bg.meta["out_grads"]
        env[og[g.outputs[0]]] = 1.0
        for o in g.outputs[1:]:
            env[og[o]] = ctx.aux_scale
        ctx.phase = "bwd"
        self.run_graph(bg, env, ctx, set())
        self.store.group_end("embedding", "bwd")
        if self.timer is not None:
            self.timer.mark("backward")

    def forward_backward(self, token_ids, position_ids, targets, **kw):
        ctx, outs = self.forward(token_ids, position_ids, targets, training=True, **kw)
        self.backward(ctx)
        return ctx, outs

    # ------------------------------------------------------------------ pipeline stages
    # A stage is a contiguous layer range.  The first stage also runs the top-level ops before the block stack (embedding),
    # the last one those after it (final norm, LM head + loss).  Several micro-batches are in flight per stage, so the saved
    # tensors of a forward are detached from the executor and attached again for the matching backward.
    @staticmethod
    def _op_index(g: Graph, kind: str) -> int:
        return next(i for i, op in enumerate(g.ops) if op.kind == kind)

    def stage_forward(self, ctx: ExecContext, layers: Tuple[int, int], is_first: bool, is_last: bool, position_ids, token_ids=None, targets=None,
                      x=None, residual=None):
        """Returns (x, residual, aux losses of this stage's layers) and, on the last stage, also the model outputs."""
        g = self.cm.fwd
        i = self._op_index(g, "block_stack")
        stack = g.ops[i]
        env: Dict[str, Any] = {"position_ids": position_ids, "token_ids": token_ids, "targets": targets}
        ctx.phase = "fwd"
        keep = (self._top_saved if ctx.training else set()) | set(g.outputs) | {n for n in stack.outputs if n} | set(stack.inputs)
        if is_first:
            self.run_graph(g, env, ctx, keep, ops=g.ops[:i])
        else:
            env[stack.inputs[0]], env[stack.inputs[1]] = x, residual
        self.layer_range = tuple(layers)
        try:
            self.run_graph(g, env, ctx, keep, ops=[stack])
        finally:
            self.layer_range = None
        outs = None
        if is_last:
            self.run_graph(g, env, ctx, keep, ops=g.ops[i + 1:])
            outs = [env.get(o) for o in g.outputs]
        self._top_env = env
        return env[stack.outputs[0]], env[stack.outputs[1]], [env[n] for n in stack.outputs[2:]], outs

    def stage_backward(self, ctx: ExecContext, layers: Tuple[int, int], is_first: bool, is_last: bool, d_x=None, d_residual=None):
        """Backward of one stage; returns the gradients of its incoming (x, residual)."""
        g, bg = self.cm.fwd, self.cm.bwd
        j = self._op_index(bg, "block_stack_backward")
        sb = bg.ops[j]
        env = {k: v for k, v in self._top_env.items() if k in self._top_saved or k in g.inputs}
        self._top_env = {}
        og = bg.meta["out_grads"]
        for o in g.outputs[1:]:
            env[og[o]] = ctx.aux_scale
        ctx.phase = "bwd"
        if is_last:
            env[og[g.outputs[0]]] = 1.0
            self.run_graph(bg, env, ctx, set(sb.inputs), ops=bg.ops[:j])
        else:
            env[sb.inputs[0]], env[sb.inputs[1]] = d_x, d_residual
        self.layer_range = tuple(layers)
        try:
            self.run_graph(bg, env, ctx, {n for n in sb.outputs if n}, ops=[sb])
        finally:
            self.layer_range = None
        out = env.get(sb.outputs[0]), env.get(sb.outputs[1])
        if is_first:
            self.run_graph(bg, env, ctx, set(), ops=bg.ops[j + 1:])
        return out

    def detach_state(self):
        state = (self._layer_saved, self._top_env)
        self._layer_saved, self._top_env = [None] * self.cm.n_layers, {}
        return state

    def attach_state(self, state) -> None:
        self._layer_saved, self._top_env = state
