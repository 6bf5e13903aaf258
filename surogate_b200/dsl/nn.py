"""torch.nn-style model definition that traces to an explicit forward graph.

A model is written as ordinary Python modules whose ``forward`` calls the
functional ops in :mod:`surogate_b200.dsl.functional`.  Calling
``Model.trace()`` runs ``forward`` once on symbolic :class:`Proxy` values and
records a :class:`~surogate_b200.dsl.ir.Graph`.  A :class:`BlockStack` traces
its block class once per distinct block type; the model graph then holds a
single ``block_stack`` op that the executor unrolls over layers, so layer hooks
(weight gather, gradient reduce, recompute) fall out of the structure.

Backward is never written by the model author; it is derived ahead of time
(:mod:`surogate_b200.dsl.autodiff`).

Parity: surogate/dsl/nn.py (Module :281, Block :507, Model :635, BlockStack :795,
HybridBlockStack :852, Tracer :100).
"""
from __future__ import annotations

import contextlib
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple, Type

from .ir import Graph, ParamSpec, Shape

_TRACE_STACK: List["Tracer"] = []


class Proxy:
    """Symbolic tensor flowing through a trace."""

    __slots__ = ("name", "shape", "dtype", "tracer")

    def __init__(self, name: str, shape: Shape, dtype: str, tracer: "Tracer"):
        self.name, self.shape, self.dtype, self.tracer = name, tuple(shape), dtype, tracer

    def __repr__(self):
        return f"Proxy({self.name}:{self.dtype}{list(self.shape)})"

    def __add__(self, other):
        from . import functional as F

        return F.add(self, other)

    def __mul__(self, other):
        from . import functional as F

        if isinstance(other, (int, float)):
            return F.scale(self, float(other))
        return F.mul(self, other)

    __rmul__ = __mul__


class Tracer:
    """Records ops into a Graph while a module's forward runs."""

    def __init__(self, graph: Graph):
        self.graph = graph
        self.scope: List[str] = []
        self.remap: Dict[str, str] = {}

    def qualify(self, name: str) -> str:
        full = ".".join(self.scope + [name]) if self.scope else name
        if full in self.remap:
            return self.remap[full]
        for key, val in self.remap.items():  # "prefix.*": "newprefix" rewrites a whole scope
            if key.endswith(".*") and full.startswith(key[:-1]):
                return val + full[len(key) - 1:]
        return full

    def input(self, name: str, shape: Shape, dtype: str = "act") -> Proxy:
        self.graph.add_tensor(name, shape, dtype, kind="input")
        self.graph.inputs.append(name)
        return Proxy(name, shape, dtype, self)

    def param(self, spec: ParamSpec) -> Proxy:
        if spec.name not in self.graph.params:
            self.graph.params[spec.name] = spec
        return Proxy(spec.name, spec.shape, spec.dtype, self)

    def emit(self, kind: str, inputs: Sequence[Optional[Proxy]], out_specs: Sequence[Optional[Tuple[str, Shape, str]]], **attrs) -> List[Optional[Proxy]]:
        outs: List[Optional[Proxy]] = []
        names: List[Optional[str]] = []
        for spec in out_specs:
            if spec is None:
                outs.append(None)
                names.append(None)
                continue
            n, shape, dtype = spec
            real = self.graph.add_tensor(self.qualify(n), shape, dtype)
            names.append(real)
            outs.append(Proxy(real, shape, dtype, self))
        self.graph.add_op(kind, [p.name if p is not None else None for p in inputs], names, **attrs)
        return outs


def current_tracer() -> Tracer:
    if not _TRACE_STACK:
        raise RuntimeError("[E010] DSL ops may only be called while tracing (inside Model.trace())")
    return _TRACE_STACK[-1]


@contextlib.contextmanager
def tracing(tracer: Tracer):
    _TRACE_STACK.append(tracer)
    try:
        yield tracer
    finally:
        _TRACE_STACK.pop()


class Module:
    """Base class: holds parameter declarations and child modules."""

    #: maps qualified local names to canonical names (applied to params and activations)
    _name_remap_: Dict[str, str] = {}

    def __init__(self):
        object.__setattr__(self, "_params", {})
        object.__setattr__(self, "_children", {})
        object.__setattr__(self, "_name", "")

    def __setattr__(self, key, value):
        if isinstance(value, Module):
            self._children[key] = value
            object.__setattr__(value, "_name", key)
        object.__setattr__(self, key, value)

    # -- declaration ----------------------------------------------------------
    def declare_param(self, name: str, shape: Sequence[int], *, init: str = "normal", decay: Optional[bool] = None,
                      hf: Any = None, lora_targets=None, quantizable: bool = False, dtype: str = "param") -> None:
        shape = tuple(int(s) for s in shape)
        if decay is None:
            decay = len(shape) >= 2
        self._params[name] = dict(shape=shape, init=init, decay=decay, hf=hf, lora_targets=lora_targets,
                                  quantizable=quantizable, dtype=dtype)

    def p(self, name: str) -> Proxy:
        """Reference a declared parameter inside forward()."""
        t = current_tracer()
        d = self._params[name]
        qn = t.qualify(name)
        return t.param(ParamSpec(qn, d["shape"], d["dtype"], d["init"], d["decay"], d["hf"], d["lora_targets"], d["quantizable"]))

    # -- tracing ------------------------------------------------------------------
    def __call__(self, *args, **kwargs):
        t = current_tracer()
        pushed = bool(self._name)
        if pushed:
            t.scope.append(self._name)
        try:
            return self.forward(*args, **kwargs)
        finally:
            if pushed:
                t.scope.pop()

    def forward(self, *args, **kwargs):  # pragma: no cover - abstract
        raise NotImplementedError

    def named_modules(self, prefix: str = "") -> Iterable[Tuple[str, "Module"]]:
        yield prefix, self
        for k, c in self._children.items():
            yield from c.named_modules(f"{prefix}.{k}" if prefix else k)


class Block(Module):
    """One repeated transformer layer; forward(x, residual, position_ids) -> (x, residual)."""

    def trace_block(self, d_model: int, extra_inputs: Sequence[Tuple[str, Shape, str]] = ()) -> Graph:
        g = Graph(type(self).__name__)
        tr = Tracer(g)
        tr.remap = dict(self._name_remap_)
        with tracing(tr):
            x = tr.input("x", ("B", "T", d_model))
            res = tr.input("residual", ("B", "T", d_model))
            pos = tr.input("position_ids", ("B", "T"), "int32")
            extras = [tr.input(n, s, d) for n, s, d in extra_inputs]
            out = self.forward(x, res, pos, *extras)
        outs = list(out) if isinstance(out, (tuple, list)) else [out]
        g.outputs = [o.name for o in outs]
        g.validate()
        return g


class BlockStack(Module):
    """``n_layers`` copies of one block class (same structure, separate parameters)."""

    def __init__(self, n_layers: int, block_cls: Type[Block], **block_kwargs):
        super().__init__()
        self.n_layers = n_layers
        self.layer_types = [block_cls.__name__] * n_layers
        self.block_protos: Dict[str, Block] = {block_cls.__name__: block_cls(**block_kwargs)}

    def forward(self, x: Proxy, residual: Proxy, position_ids: Proxy):
        t = current_tracer()
        d_model = x.shape[-1]
        aux_names = []
        for name, proto in self.block_protos.items():
            bg = proto.trace_block(d_model)
            t.graph.subgraphs[name] = bg
            for extra in bg.outputs[2:]:
                if extra not in aux_names:
                    aux_names.append(extra)
        outs = t.emit(
            "block_stack", [x, residual, position_ids],
            [("xN", x.shape, x.dtype), ("residualN", residual.shape, residual.dtype)]
            + [(f"stack_{n}", (), "fp32") for n in aux_names],
            n_layers=self.n_layers, layer_types=list(self.layer_types), aux=aux_names,
        )
        if aux_names:
            return outs[0], outs[1], outs[2:]
        return outs[0], outs[1]


class HybridBlockStack(BlockStack):
    """Layer stack with a per-layer choice among several block classes (e.g. dense/MoE interleave)."""

    def __init__(self, layer_types: Sequence[str], block_classes: Dict[str, Tuple[Type[Block], Dict[str, Any]]]):
        Module.__init__(self)
        self.n_layers = len(layer_types)
        self.layer_types = list(layer_types)
        self.block_protos = {name: cls(**kw) for name, (cls, kw) in block_classes.items()}


class Model(Module):
    """Top-level model: forward(token_ids, position_ids, targets) -> loss."""

    hf_config_map: Dict[str, str] = {}
    hf_architecture: str = ""
    hf_model_type: str = ""
    #: model-level HF names; block-level ones come from the param declarations
    _hf_block_mappings_: Dict[str, Any] = {}

    def trace(self) -> Graph:
        g = Graph(type(self).__name__)
        tr = Tracer(g)
        tr.remap = dict(self._name_remap_)
        with tracing(tr):
            tok = tr.input("token_ids", ("B", "T"), "int32")
            pos = tr.input("position_ids", ("B", "T"), "int32")
            tgt = tr.input("targets", ("B", "T"), "int32")
            out = self.forward(tok, pos, tgt)
        outs = list(out) if isinstance(out, (tuple, list)) else [out]
        g.outputs = [o.name for o in outs]
        g.meta.update(self.describe())
        g.validate()
        return g

    def describe(self) -> Dict[str, Any]:
        return {k: v for k, v in vars(self).items() if isinstance(v, (int, float, str, bool))}

    @classmethod
    def from_hf_config(cls, cfg: Dict[str, Any], **overrides) -> "Model":
        kw = {}
        aliases = {"num_experts": ("num_local_experts", "n_routed_experts"), "head_dim": ("head_size",)}  # spellings used by other writers of config.json
        def lookup(path: str):
            node = cfg
            for part in path.split("."):  # "text_config.hidden_size" reaches into a nested sub-config
                if not isinstance(node, dict) or part not in node:
                    return None
                node = node[part]
            return node

        for mine, theirs in cls.hf_config_map.items():
            for key in (theirs,) + aliases.get(theirs, ()):
                val = lookup(key)
                if val is not None:
                    kw[mine] = val
                    break
        rp = cfg.get("rope_parameters") or cfg.get("rope_scaling")
        if "rope_theta" not in kw and isinstance(rp, dict) and rp.get("rope_theta") is not None:
            kw["rope_theta"] = rp["rope_theta"]  # newer config.json files keep the RoPE base inside rope_parameters
        kw.update(overrides)
        import inspect

        accepted = set()
        for klass in cls.__mro__:  # a subclass may forward **kwargs to its parent: collect the names along the chain
            init = klass.__dict__.get("__init__")
            if init is None:
                continue
            params = inspect.signature(init).parameters
            accepted |= {n for n, p in params.items() if p.kind in (p.POSITIONAL_OR_KEYWORD, p.KEYWORD_ONLY)}
            if not any(p.kind == p.VAR_KEYWORD for p in params.values()):
                break
        return cls(**{k: v for k, v in kw.items() if k in accepted})


_MODEL_REGISTRY: Dict[str, Type[Model]] = {}


def hf_config(architecture: str, model_type: str, **field_map: str) -> Callable[[Type[Model]], Type[Model]]:
    """Class decorator: bind a Model class to an HF architecture and map config.json keys to ctor args."""

    def deco(cls: Type[Model]) -> Type[Model]:
        cls.hf_config_map = dict(field_map)
        cls.hf_architecture = architecture
        cls.hf_model_type = model_type
        _MODEL_REGISTRY[architecture] = cls
        _MODEL_REGISTRY[model_type] = cls
        return cls

    return deco


def model_class_for(name: str) -> Type[Model]:
    if name not in _MODEL_REGISTRY:
        raise KeyError(f"[E020] no DSL model registered for architecture/model_type '{name}' (known: {sorted(_MODEL_REGISTRY)})")
    return _MODEL_REGISTRY[name]


def registered_models() -> Dict[str, Type[Model]]:
    return dict(_MODEL_REGISTRY)


def registered_architectures() -> List[str]:
    """HF ``architectures`` names (those ending in ForCausalLM / ForConditionalGeneration) that have a DSL model."""
    return sorted(k for k in _MODEL_REGISTRY if k[:1].isupper())
