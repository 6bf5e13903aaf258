"""Graph compiler passes over the DSL IR: fusion rules, consumer annotations, a static buffer plan, and baked op programs.

The traced graphs are already coarse (modules emit fused ops such as ``fused_residual_rmsnorm`` directly), so the passes here
exist for graphs written from primitives (new model families, hand-written blocks, imported IR), for facts that recipes and
the executor would otherwise re-derive at run time, and for memory planning:

``apply_fusion_rules``     registry of peephole rewrites (residual add + RMSNorm, scale folding, view folding, SiLU x up ->
                           SwiGLU over a concatenated projection, matmul + bias) followed by dead-op elimination.  Runs before
                           autodiff, so the backward graph is derived from the fused forward.
``annotate_consumers``     per tensor: which ops read it and whether all of them are quantised matmuls (``quant_only``) --
                           what lets a norm / activation kernel emit FP8 or FP4 directly instead of a bf16 tensor plus a
                           quantise pass.  Stored in ``graph.meta['consumers']``; recipes read it instead of scanning op lists.
``plan_buffers``           liveness intervals of every activation for bound dimensions (B, T), split into regions -- *saved*
                           (kept from forward to backward, once per layer), *forward temporaries*, *backward temporaries* --
                           and packed into arenas by interval colouring (largest first, lowest non-overlapping offset).
                           Gives offsets, region sizes and the peak, and is checked by ``BufferPlan.validate`` (no two
                           tensors alive at the same time overlap).  The trainer uses it for pre-flight memory estimates and
                           the debug tools print it; tensors themselves still come from the stream-ordered caching allocator,
                           whose steady state reproduces such a packing without baked offsets.
``bake_program``           the interpreter's per-op work done once: backend method bound, inputs classified as parameter /
                           environment slot, tensors to free after each op listed.  ``Executor.run_graph`` walks the baked
                           list instead of re-resolving names on every op of every step.

Parity: csrc/src/runtime/dsl/graph_compiler.cpp (tensor regions, phase arenas, baked offsets),
csrc/src/runtime/dsl/fusion_rule_registrations.cpp:62-76 (rule registry), csrc/src/runtime/dsl/buffer_plan.h.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Set, Tuple

from .ir import Graph, OpNode, eval_shape

DTYPE_BYTES = {"act": 2, "bf16": 2, "fp16": 2, "fp32": 4, "int32": 4, "int64": 8, "param": 2, "fp8": 1, "uint8": 1, "bool": 1}
QUANT_MATMUL_ROLES = {"qkv", "out", "mlp_up", "mlp_down"}

# ---------------------------------------------------------------------------------------------------------------- fusion rules


@dataclass
class FusionRule:
    """``match(graph, i)`` looks at ``graph.ops[i:]`` and returns ``(n_ops_consumed_positions, replacement_ops)`` or None.
    ``positions`` are indices into ``graph.ops`` of the ops the rule replaces (they need not be adjacent)."""
    name: str
    match: Callable[[Graph, int, Dict[str, List[int]]], Optional[Tuple[List[int], List[OpNode]]]]
    doc: str = ""


FUSION_RULES: List[FusionRule] = []


def register_fusion_rule(name: str, doc: str = ""):
    def deco(fn):
        FUSION_RULES.append(FusionRule(name, fn, doc or (fn.__doc__ or "").strip()))
        return fn
    return deco


def _readers(g: Graph) -> Dict[str, List[int]]:
    out: Dict[str, List[int]] = {}
    for k, op in enumerate(g.ops):
        for i in op.inputs:
            if i is not None:
                out.setdefault(i, []).append(k)
    return out


def _sole_reader(name: str, readers: Dict[str, List[int]], g: Graph) -> Optional[int]:
    r = readers.get(name, [])
    if len(r) == 1 and name not in g.outputs:
        return r[0]
    return None


@register_fusion_rule("residual_add_rmsnorm")
def _rule_add_rmsnorm(g: Graph, i: int, readers):
    """add(a, b) -> r ; rmsnorm(r, w) -> (y, rstd)   =>   fused_residual_rmsnorm(a, b, w) -> (r, y, rstd): one pass over the row."""
    op = g.ops[i]
    if op.kind != "add":
        return None
    r = op.outputs[0]
    for j in readers.get(r, []):
        nxt = g.ops[j]
        if nxt.kind == "rmsnorm" and nxt.inputs[0] == r and j > i:
            if any(g.ops[k].kind != "rmsnorm" and k < j for k in readers.get(r, []) if k != j):
                return None    # something reads the sum before the norm: keep the order of evaluation simple
            fused = OpNode("fused_residual_rmsnorm", [op.inputs[0], op.inputs[1], nxt.inputs[1]], [r, nxt.outputs[0], nxt.outputs[1]], dict(nxt.attrs))
            return [i, j], [fused]
    return None


@register_fusion_rule("scale_folding")
def _rule_scale_scale(g: Graph, i: int, readers):
    """scale(scale(x, a), b) => scale(x, a * b) when nothing else reads the inner result."""
    op = g.ops[i]
    if op.kind != "scale":
        return None
    j = _sole_reader(op.outputs[0], readers, g)
    if j is None or g.ops[j].kind != "scale":
        return None
    nxt = g.ops[j]
    return [i, j], [OpNode("scale", [op.inputs[0]], [nxt.outputs[0]], {**nxt.attrs, "factor": float(op.attrs["factor"]) * float(nxt.attrs["factor"])})]


@register_fusion_rule("view_folding")
def _rule_view_view(g: Graph, i: int, readers):
    """view(view(x, s1), s2) => view(x, s2)."""
    op = g.ops[i]
    if op.kind != "view":
        return None
    j = _sole_reader(op.outputs[0], readers, g)
    if j is None or g.ops[j].kind != "view":
        return None
    nxt = g.ops[j]
    return [i, j], [OpNode("view", [op.inputs[0]], [nxt.outputs[0]], dict(nxt.attrs))]


@register_fusion_rule("matmul_bias")
def _rule_matmul_bias(g: Graph, i: int, readers):
    """matmul(x, w, None) -> y ; add(y, bias_param) -> z   =>   matmul(x, w, bias) -> z (bias added in the GEMM epilogue)."""
    op = g.ops[i]
    if op.kind != "matmul" or (len(op.inputs) > 2 and op.inputs[2] is not None):
        return None
    j = _sole_reader(op.outputs[0], readers, g)
    if j is None or g.ops[j].kind != "add":
        return None
    nxt = g.ops[j]
    other = nxt.inputs[1] if nxt.inputs[0] == op.outputs[0] else nxt.inputs[0]
    if other not in g.params or len(g.params[other].shape) != 1:
        return None
    return [i, j], [OpNode("matmul", [op.inputs[0], op.inputs[1], other], [nxt.outputs[0]], dict(op.attrs))]


@register_fusion_rule("silu_mul_swiglu")
def _rule_silu_mul(g: Graph, i: int, readers):
    """silu(gate) * up where gate and up are the two halves (views) of one projection  =>  swiglu(projection)."""
    op = g.ops[i]
    if op.kind != "silu":
        return None
    j = _sole_reader(op.outputs[0], readers, g)
    if j is None or g.ops[j].kind != "mul":
        return None
    nxt = g.ops[j]
    up = nxt.inputs[1] if nxt.inputs[0] == op.outputs[0] else nxt.inputs[0]
    prod = g.producers()
    pg, pu = prod.get(op.inputs[0]), prod.get(up)
    if pg is None or pu is None or pg.kind != "view" or pu.kind != "view" or pg.inputs[0] != pu.inputs[0]:
        return None
    if pg.attrs.get("half") != "gate" or pu.attrs.get("half") != "up":
        return None
    return [i, j], [OpNode("swiglu", [pg.inputs[0]], [nxt.outputs[0]], {})]


def eliminate_dead_ops(g: Graph, keep: Optional[Set[str]] = None) -> int:
    """Drop ops none of whose outputs is read, is a graph output, a gradient, or listed in ``keep`` (saved tensors)."""
    keep = set(keep or ()) | set(g.outputs) | set(g.meta.get("saved", []))
    removed = 0
    while True:
        readers = _readers(g)
        dead = [k for k, op in enumerate(g.ops)
                if op.kind not in ("block_stack", "block_stack_backward") and op.outputs
                and all(o is None or (o not in readers and o not in keep and not o.startswith("grad::")) for o in op.outputs)]
        if not dead:
            break
        for k in reversed(dead):
            for o in g.ops[k].outputs:
                if o is not None:
                    g.tensors.pop(o, None)
            del g.ops[k]
            removed += 1
        for k, op in enumerate(g.ops):
            op.idx = k
    return removed


def apply_fusion_rules(g: Graph, rules: Optional[Sequence[FusionRule]] = None, recurse: bool = True) -> Dict[str, int]:
    """Rewrites ``g`` in place until no rule matches; returns how often each rule fired (``dead_ops`` = ops removed)."""
    rules = list(FUSION_RULES if rules is None else rules)
    fired: Dict[str, int] = {}
    changed = True
    while changed:
        changed = False
        readers = _readers(g)
        for i in range(len(g.ops)):
            for rule in rules:
                m = rule.match(g, i, readers)
                if m is None:
                    continue
                positions, repl = m
                first = min(positions)
                last = max(positions)
                # the replacement goes where the LAST replaced op stood (all of its inputs exist by then) unless an output of the
                # first op is read in between, in which case it goes where the first stood (its inputs must then exist there)
                outs_first = {o for p in positions for o in g.ops[p].outputs if o is not None}
                between = any(any(x in outs_first for x in g.ops[k].inputs if x is not None) for k in range(first + 1, last) if k not in positions)
                at = first if between else last
                if between:
                    known = set(g.inputs) | set(g.params) | {o for k in range(first) for o in g.ops[k].outputs if o is not None}
                    if any(x is not None and x not in known for r in repl for x in r.inputs):
                        continue
                new_ops: List[OpNode] = []
                for k, op in enumerate(g.ops):
                    if k == at:
                        new_ops.extend(repl)
                    if k in positions:
                        continue
                    new_ops.append(op)
                produced = {o for r in repl for o in r.outputs if o is not None}
                for p in positions:
                    for o in g.ops[p].outputs:
                        if o is not None and o not in produced:
                            g.tensors.pop(o, None)
                g.ops = new_ops
                for k, op in enumerate(g.ops):
                    op.idx = k
                fired[rule.name] = fired.get(rule.name, 0) + 1
                changed = True
                break
            if changed:
                break
    dead = eliminate_dead_ops(g)
    if dead:
        fired["dead_ops"] = dead
    g.validate()
    if recurse:
        for sub in g.subgraphs.values():
            for k, v in apply_fusion_rules(sub, rules, recurse=True).items():
                fired[k] = fired.get(k, 0) + v
    return fired


# ------------------------------------------------------------------------------------------------------ consumer annotations


def annotate_consumers(g: Graph) -> Dict[str, Dict[str, Any]]:
    """``graph.meta['consumers'][tensor] = {'readers': [(kind, role)], 'quant_only': bool, 'sole_backward_matmul': role | None}``."""
    info: Dict[str, Dict[str, Any]] = {}
    for op in g.ops:
        for pos, name in enumerate(op.inputs):
            if name is None:
                continue
            e = info.setdefault(name, {"readers": [], "quant_only": True, "sole_backward_matmul": None})
            role = op.attrs.get("role", "")
            e["readers"].append((op.kind, role))
            if not (op.kind == "matmul" and pos == 0 and role in QUANT_MATMUL_ROLES):
                e["quant_only"] = False
    for name, e in info.items():
        e["quant_only"] = bool(e["readers"]) and e["quant_only"] and name not in g.outputs
        if len(e["readers"]) == 1 and e["readers"][0][0] == "matmul_backward":
            reader = next(op for op in g.ops if name in op.inputs)
            if reader.inputs[0] == name and (len(reader.outputs) < 3 or reader.outputs[2] is None):
                e["sole_backward_matmul"] = e["readers"][0][1]
    g.meta["consumers"] = info
    return info


# -------------------------------------------------------------------------------------------------------------- buffer plan


@dataclass
class PlannedTensor:
    name: str
    region: str          # saved | temp
    nbytes: int
    first: int           # op index that writes it (-1: graph input)
    last: int            # last op index that reads it
    offset: int = 0


@dataclass
class BufferPlan:
    graph: str
    dims: Dict[str, int]
    tensors: Dict[str, PlannedTensor] = field(default_factory=dict)
    region_bytes: Dict[str, int] = field(default_factory=dict)
    unpacked_bytes: Dict[str, int] = field(default_factory=dict)   # the same tensors without reuse

    def validate(self) -> None:
        """No two tensors of one region whose lifetimes intersect may overlap in memory."""
        by_region: Dict[str, List[PlannedTensor]] = {}
        for t in self.tensors.values():
            by_region.setdefault(t.region, []).append(t)
        for region, ts in by_region.items():
            for a_i, a in enumerate(ts):
                if a.offset % 256:
                    raise AssertionError(f"{self.graph}: '{a.name}' is not 256-byte aligned")
                if a.offset + a.nbytes > self.region_bytes[region]:
                    raise AssertionError(f"{self.graph}: '{a.name}' ends outside region '{region}'")
                for b in ts[a_i + 1:]:
                    alive_together = a.first <= b.last and b.first <= a.last
                    overlap = a.offset < b.offset + b.nbytes and b.offset < a.offset + a.nbytes
                    if alive_together and overlap and a.nbytes and b.nbytes:
                        raise AssertionError(f"{self.graph}: '{a.name}' [{a.first},{a.last}] and '{b.name}' [{b.first},{b.last}] alias in region '{region}'")

    def aliases(self) -> List[Tuple[str, str]]:
        """Pairs that share bytes (legally: their lifetimes are disjoint)."""
        out = []
        ts = list(self.tensors.values())
        for i, a in enumerate(ts):
            for b in ts[i + 1:]:
                if a.region == b.region and a.nbytes and b.nbytes and a.offset < b.offset + b.nbytes and b.offset < a.offset + a.nbytes:
                    out.append((a.name, b.name))
        return out

    def table(self) -> str:
        rows = [f"graph {self.graph}  dims {self.dims}"]
        for region, size in sorted(self.region_bytes.items()):
            rows.append(f"  region {region:6s} {size / 2**20:10.2f} MiB  (without reuse {self.unpacked_bytes.get(region, 0) / 2**20:.2f} MiB)")
        for t in sorted(self.tensors.values(), key=lambda t: (t.region, t.offset, t.first)):
            rows.append(f"    {t.region:6s} {t.offset:>14d} +{t.nbytes:>12d}  live [{t.first:>3d},{t.last:>3d}]  {t.name}")
        return "\n".join(rows)


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


def _native_planner():
    try:
        from ..ops import host

        h = host()
        return h if hasattr(h, "plan_buffer_offsets") else None
    except Exception:  # noqa: BLE001 -- the host runtime is not built: the Python statement below is used
        return None


def _pack(ts: List[PlannedTensor], use_native: bool = True) -> int:
    """Interval colouring: largest tensors first, each at the lowest offset that is free during its whole lifetime.  Runs in the
    native host runtime (csrc/host/buffer_planner.cpp) when it is built; the Python loop below is the same procedure and its oracle."""
    h = _native_planner() if use_native else None
    if h is not None and ts:
        offsets, total = h.plan_buffer_offsets([int(t.nbytes) for t in ts], [int(t.first) for t in ts], [int(t.last) for t in ts])
        for t, off in zip(ts, offsets):
            t.offset = int(off)
        return int(total)
    placed: List[PlannedTensor] = []
    top = 0
    for t in sorted(ts, key=lambda t: (-t.nbytes, t.first)):
        busy = sorted((p.offset, p.offset + _align(p.nbytes)) for p in placed if p.first <= t.last and t.first <= p.last and p.nbytes)
        off = 0
        for lo, hi in busy:
            if off + _align(t.nbytes) <= lo:
                break
            off = max(off, hi)
        t.offset = off
        placed.append(t)
        top = max(top, off + _align(t.nbytes))
    return top


def plan_buffers(g: Graph, dims: Dict[str, int], saved: Optional[Sequence[str]] = None, act_bytes: int = 2) -> BufferPlan:
    """Static plan for one graph with the symbolic dimensions bound (``{'B': 2, 'T': 4096}``)."""
    saved_set = set(saved if saved is not None else g.meta.get("saved", []))
    last = g.last_use()
    plan = BufferPlan(g.name, dict(dims))
    first: Dict[str, int] = {n: -1 for n in g.inputs}
    for op in g.ops:
        for o in op.outputs:
            if o is not None and not o.startswith("grad::"):
                first.setdefault(o, op.idx)
    temps: List[PlannedTensor] = []
    keeps: List[PlannedTensor] = []
    for name, f in first.items():
        spec = g.tensors.get(name)
        if spec is None:
            continue
        try:
            shape = eval_shape(spec.shape, dims)
        except Exception:  # noqa: BLE001 -- a dimension that is only known at run time (routed rows): not planned
            continue
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * (act_bytes if spec.dtype == "act" else DTYPE_BYTES.get(spec.dtype, 2))
        if name in saved_set and f >= 0:
            keeps.append(PlannedTensor(name, "saved", nbytes, f, len(g.ops)))
        elif f >= 0:
            temps.append(PlannedTensor(name, "temp", nbytes, f, last.get(name, f)))
    plan.region_bytes["temp"] = _pack(temps)
    off = 0
    for t in keeps:      # saved tensors all live until the backward: laid end to end
        t.offset = off
        off += _align(t.nbytes)
    plan.region_bytes["saved"] = off
    plan.unpacked_bytes = {"temp": sum(_align(t.nbytes) for t in temps), "saved": off}
    for t in temps + keeps:
        plan.tensors[t.name] = t
    return plan


@dataclass
class ModelMemoryPlan:
    dims: Dict[str, int]
    per_block: Dict[str, Dict[str, BufferPlan]]     # block type -> {'fwd': plan, 'bwd': plan}
    layer_types: List[str]
    recompute: bool
    act_bytes: int = 2

    @property
    def saved_bytes(self) -> int:
        if self.recompute:     # block inputs (x, residual) survive the forward; one block's saved set is rebuilt at a time in backward
            rebuilt = max((p["fwd"].region_bytes.get("saved", 0) for p in self.per_block.values()), default=0)
            boundary = 2 * self.dims.get("B", 1) * self.dims.get("T", 1) * self.dims.get("C", 0) * self.act_bytes
            return rebuilt + len(self.layer_types) * boundary
        return sum(self.per_block[bt]["fwd"].region_bytes.get("saved", 0) for bt in self.layer_types)

    @property
    def temp_bytes(self) -> int:
        return max((max(p["fwd"].region_bytes.get("temp", 0), p["bwd"].region_bytes.get("temp", 0)) for p in self.per_block.values()), default=0)

    @property
    def activation_bytes(self) -> int:
        return self.saved_bytes + self.temp_bytes

    def summary(self) -> Dict[str, float]:
        return {"saved_gib": self.saved_bytes / 2**30, "temp_gib": self.temp_bytes / 2**30, "activations_gib": self.activation_bytes / 2**30,
                "layers": float(len(self.layer_types))}


def plan_model(cm, batch: int, seq_len: int, recompute: bool = False, act_bytes: int = 2) -> ModelMemoryPlan:
    """Buffer plans of every block type (forward and backward graphs) and the model-level totals for ``batch`` x ``seq_len``."""
    dims = {"B": int(batch), "T": int(seq_len)}
    x = cm.fwd.tensors.get("x0")
    if x is not None and isinstance(x.shape[-1], int):
        dims["C"] = int(x.shape[-1])
    per_block: Dict[str, Dict[str, BufferPlan]] = {}
    for bt, g in cm.block_fwd.items():
        bwd = cm.block_bwd[bt]
        per_block[bt] = {"fwd": plan_buffers(g, dims, saved=bwd.meta.get("saved", []), act_bytes=act_bytes),
                         "bwd": plan_buffers(bwd, dims, saved=[], act_bytes=act_bytes)}
    return ModelMemoryPlan(dims, per_block, list(cm.layer_types), recompute, act_bytes)


# ------------------------------------------------------------------------------------------------------------ baked programs


@dataclass
class BakedOp:
    op: OpNode
    fn: Any                                  # bound backend method, or None for the block-stack ops the executor handles itself
    sources: Tuple[Tuple[int, Any], ...]     # per input: (0, None) missing | (1, local param name) | (2, env name)
    frees: Tuple[str, ...]                   # env entries dead after this op


def bake_program(g: Graph, backend, keep: Set[str], ops: Optional[Sequence[OpNode]] = None) -> List[BakedOp]:
    last = g.last_use()
    params = g.params
    out: List[BakedOp] = []
    ginputs = set(g.inputs)
    for op in (g.ops if ops is None else ops):
        if op.kind in ("block_stack", "block_stack_backward"):
            fn = None
        else:
            fn = getattr(backend, op.kind, None)
            if fn is None:
                raise NotImplementedError(f"[E030] backend '{backend.name}' has no implementation of op '{op.kind}'")
        src = tuple((0, None) if n is None else ((1, n) if n in params else (2, n)) for n in op.inputs)
        frees = tuple(dict.fromkeys(n for n in op.inputs if n is not None and n not in params and last.get(n, -1) == op.idx and n not in keep and n not in ginputs))
        out.append(BakedOp(op, fn, src, frees))
    return out
