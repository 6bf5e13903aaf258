"""Compile-only tensor introspection: ``surogate debug tensor-arena | tensor-layout | tensor-aliasing | tensor-resolve``.

All four build the model's graphs from its config (no weights, no GPU) and read the graph compiler's buffer plan
(``dsl/graph_compiler.py``):

``tensor-arena``     one record per (block type, graph) with the region sizes (saved / temp), the size without reuse, the number
                     of planned tensors and a hash of the layout (equal hashes = equal plans on every rank), plus a model summary.
``tensor-layout``    one record per planned tensor: graph, name, region, offset, bytes, first write, last use, shape, dtype.
``tensor-aliasing``  static mode: validates every plan (two tensors alive together never share bytes) and lists the legal
                     byte-sharing pairs; runtime mode: runs one forward + backward on the reference backend and reports every op
                     whose output shares storage with one of its own inputs that is read later (an in-place hazard).
``tensor-resolve``   everything known about one tensor name: graphs it appears in, producer op, readers, lifetime, plan entry,
                     whether backward needs it (saved), consumer annotation.

Parity: surogate/debug/tensor_arena.py, tensor_layout.py, tensor_aliasing.py, tensor_resolve.py.
"""
from __future__ import annotations

import hashlib
import json
from typing import Any, Dict, List, Optional

from ..dsl.compiler import compile_model, load_hf_config, model_from_hf_config
from ..dsl.graph_compiler import BufferPlan, plan_model
from .tools import write_jsonl


def _compiled(model_dir_or_cfg):
    cfg = load_hf_config(model_dir_or_cfg)
    return compile_model(model_from_hf_config(cfg))


def _graphs(cm):
    for bt in cm.block_fwd:
        yield bt, "forward", cm.block_fwd[bt]
        yield bt, "backward", cm.block_bwd[bt]


def _layout_hash(plan: BufferPlan) -> str:
    h = hashlib.sha256()
    for t in sorted(plan.tensors.values(), key=lambda t: t.name):
        h.update(f"{t.name}:{t.region}:{t.offset}:{t.nbytes};".encode())
    return h.hexdigest()[:16]


def tensor_arena(model, batch: int = 1, seq_len: int = 2048, recompute: bool = False, out: Optional[str] = None) -> List[Dict[str, Any]]:
    cm = _compiled(model)
    mp = plan_model(cm, batch, seq_len, recompute)
    rows: List[Dict[str, Any]] = []
    for bt, plans in mp.per_block.items():
        for which, plan in (("forward", plans["fwd"]), ("backward", plans["bwd"])):
            g = cm.block_fwd[bt] if which == "forward" else cm.block_bwd[bt]
            named = {o for op in g.ops for o in op.outputs if o is not None and not o.startswith("grad::")}
            rows.append({"tag": "TENSOR_ARENA", "block": bt, "graph": which, "regions": plan.region_bytes, "without_reuse": plan.unpacked_bytes,
                         "tensors": len(plan.tensors), "coverage": len(plan.tensors) / max(1, len(named)), "layout_hash": _layout_hash(plan), "ops": len(g.ops)})
            for region, size in plan.region_bytes.items():
                members = [t for t in plan.tensors.values() if t.region == region]
                rows.append({"tag": "TENSOR_REGION", "block": bt, "graph": which, "region": region, "bytes": size, "tensors": len(members),
                             "sum_bytes": sum(t.nbytes for t in members)})
    rows.append({"tag": "SUMMARY", "dims": mp.dims, "layers": len(mp.layer_types), "recompute": recompute, **mp.summary()})
    return write_jsonl(out, rows)


def tensor_layout(model, batch: int = 1, seq_len: int = 2048, out: Optional[str] = None) -> List[Dict[str, Any]]:
    cm = _compiled(model)
    mp = plan_model(cm, batch, seq_len)
    rows = []
    for bt, plans in mp.per_block.items():
        for which, plan in (("forward", plans["fwd"]), ("backward", plans["bwd"])):
            g = cm.block_fwd[bt] if which == "forward" else cm.block_bwd[bt]
            for t in sorted(plan.tensors.values(), key=lambda t: (t.region, t.offset)):
                spec = g.tensors.get(t.name)
                rows.append({"tag": "TENSOR_LAYOUT", "block": bt, "graph": which, "name": t.name, "region": t.region, "offset": t.offset, "bytes": t.nbytes,
                             "first_write_op": t.first, "last_use_op": t.last, "shape": list(spec.shape) if spec else None, "dtype": spec.dtype if spec else None,
                             "retain_through_forward": t.region == "saved"})
    return write_jsonl(out, rows)


def tensor_aliasing(model, batch: int = 1, seq_len: int = 128, mode: str = "static", out: Optional[str] = None) -> List[Dict[str, Any]]:
    cm = _compiled(model)
    rows: List[Dict[str, Any]] = []
    if mode == "static":
        mp = plan_model(cm, batch, seq_len)
        for bt, plans in mp.per_block.items():
            for which, plan in (("forward", plans["fwd"]), ("backward", plans["bwd"])):
                try:
                    plan.validate()
                    ok, err = True, None
                except AssertionError as e:
                    ok, err = False, str(e)
                shared = plan.aliases()
                rows.append({"tag": "TENSOR_ALIAS_STATIC", "block": bt, "graph": which, "valid": ok, "error": err, "legal_sharing_pairs": len(shared),
                             "examples": shared[:8]})
        return write_jsonl(out, rows)
    # runtime: in-place hazards on the reference backend
    import torch

    from ..runtime.trainer import Trainer, TrainerConfig

    cfg = load_hf_config(model)
    tr = Trainer(TrainerConfig(model=cfg, batch_size=batch, seq_len=seq_len, backend="ref", zero_level=0), device=torch.device("cpu"))
    tr.init_weights(seed=0)
    events: List[Dict[str, Any]] = []
    ex = tr.executor
    orig = ex.run_graph

    def checked(g, env, ctx, keep, ops=None):
        last = g.last_use()
        be = ex.backend
        for op in (g.ops if ops is None else ops):
            if op.kind in ("block_stack", "block_stack_backward"):
                continue
            fn = getattr(be, op.kind, None)
            if fn is None or getattr(fn, "_alias_checked", False):
                continue

            def wrap(fn=fn):
                def inner(ctx2, op2, *ins):
                    outs = fn(ctx2, op2, *ins)
                    for on, ov in zip(op2.outputs, outs):
                        if not torch.is_tensor(ov) or on is None:
                            continue
                        for iname, iv in zip(op2.inputs, ins):
                            if torch.is_tensor(iv) and iv.numel() and ov.numel() and iv.untyped_storage().data_ptr() == ov.untyped_storage().data_ptr() \
                                    and ctx2.graph is not None and ctx2.graph.last_use().get(iname, -1) > op2.idx and op2.kind != "view":
                                events.append({"tag": "TENSOR_ALIAS_RUNTIME", "graph": ctx2.graph.name, "op": op2.kind, "op_idx": op2.idx, "output": on,
                                               "input": iname, "input_last_use": ctx2.graph.last_use().get(iname)})
                    return outs
                inner._alias_checked = True
                return inner
            setattr(be, op.kind, wrap())
        return orig(g, env, ctx, keep, ops)

    ex.run_graph = checked
    ex._programs.clear()
    x = torch.randint(0, int(cfg.get("vocab_size", 256)), (batch, seq_len))
    pos = torch.arange(seq_len).expand(batch, seq_len).contiguous()
    tr.forward_backward(x, x, pos)
    rows = events or [{"tag": "TENSOR_ALIAS_RUNTIME", "events": 0}]
    return write_jsonl(out, rows)


def tensor_resolve(model, name: str, batch: int = 1, seq_len: int = 2048, out: Optional[str] = None) -> List[Dict[str, Any]]:
    cm = _compiled(model)
    mp = plan_model(cm, batch, seq_len)
    rows = []
    graphs = [("model", "forward", cm.fwd, None), ("model", "backward", cm.bwd, None)]
    for bt, plans in mp.per_block.items():
        graphs.append((bt, "forward", cm.block_fwd[bt], plans["fwd"]))
        graphs.append((bt, "backward", cm.block_bwd[bt], plans["bwd"]))
    for bt, which, g, plan in graphs:
        if name not in g.tensors and name not in g.params and name not in g.inputs:
            continue
        prod = g.producers().get(name)
        readers = [{"op": op.kind, "idx": op.idx, "role": op.attrs.get("role")} for op in g.ops if name in op.inputs]
        spec = g.tensors.get(name)
        entry = plan.tensors.get(name) if plan is not None else None
        rows.append({"tag": "TENSOR_RESOLVE", "block": bt, "graph": which, "name": name,
                     "kind": "param" if name in g.params else ("input" if name in g.inputs else (spec.kind if spec else None)),
                     "shape": list(spec.shape) if spec else (list(g.params[name].shape) if name in g.params else None),
                     "dtype": spec.dtype if spec else None, "producer": {"op": prod.kind, "idx": prod.idx} if prod else None, "readers": readers,
                     "saved_for_backward": name in (cm.block_bwd[bt].meta.get("saved", []) if bt in cm.block_bwd else cm.bwd.meta.get("saved", [])),
                     "plan": None if entry is None else {"region": entry.region, "offset": entry.offset, "bytes": entry.nbytes, "live": [entry.first, entry.last]},
                     "consumers": (g.meta.get("consumers") or {}).get(name)})
    if not rows:
        rows = [{"tag": "TENSOR_RESOLVE", "name": name, "error": "no graph of this model defines a tensor of that name"}]
    return write_jsonl(out, rows)


def main_json(rows: List[Dict[str, Any]], limit: int = 40) -> None:
    for r in rows[:limit]:
        print(json.dumps(r, default=str))
    if len(rows) > limit:
        print(json.dumps({"more_rows": len(rows) - limit}))
