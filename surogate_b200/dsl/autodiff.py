"""Ahead-of-time reverse-mode differentiation of a traced forward graph.

``derive_backward_graph`` walks the forward ops in reverse and, for each op with
a live output gradient, asks the op's rule to emit explicit backward ops.  The
result is an ordinary :class:`Graph` whose inputs are the output gradients, the
parameters and whichever forward tensors the backward ops read ("saved"
tensors).  Nothing is differentiated at run time.

Parameter gradients are written under the reserved name ``grad::<param>``; the
executor routes those to the gradient store, accumulating across micro-steps and
across multiple uses of a tied parameter.

Parity: csrc/src/runtime/dsl/autodiff.cpp:184 (derive_backward_graph) and the
REGISTER_AUTODIFF rules in csrc/src/runtime/ops/*.cpp.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

from .ir import Graph, OpNode

GRAD_PREFIX = "grad::"

Rule = Callable[["BackwardBuilder", OpNode, List[Optional[str]]], Dict[str, str]]
_RULES: Dict[str, Rule] = {}


def register_autodiff(kind: str):
    def deco(fn: Rule) -> Rule:
        _RULES[kind] = fn
        return fn

    return deco


def has_rule(kind: str) -> bool:
    return kind in _RULES


class BackwardBuilder:
    def __init__(self, fwd: Graph):
        self.fwd = fwd
        self.g = Graph(fwd.name + "_backward")
        self.g.params = dict(fwd.params)
        self.saved: List[str] = []

    def fwd_tensor(self, name: Optional[str]) -> Optional[str]:
        """Declare that the backward graph reads forward tensor ``name``."""
        if name is None:
            return None
        if name not in self.fwd.params and name not in self.saved:
            self.saved.append(name)
        return name

    def new_grad(self, of: str) -> str:
        spec = self.fwd.tensors.get(of)
        shape = spec.shape if spec is not None else self.fwd.params[of].shape
        dtype = spec.dtype if spec is not None else "act"
        return self.g.add_tensor(f"d_{of}", shape, dtype, kind="grad")

    def param_grad(self, param: Optional[str]) -> Optional[str]:
        if param is None:
            return None
        return GRAD_PREFIX + param

    def is_param(self, name: Optional[str]) -> bool:
        return name is not None and name in self.fwd.params

    def emit(self, kind: str, inputs: Sequence[Optional[str]], outputs: Sequence[Optional[str]], **attrs) -> OpNode:
        return self.g.add_op(kind, inputs, outputs, **attrs)


def derive_backward_graph(fwd: Graph, wrt_inputs: Optional[Sequence[str]] = None) -> Graph:
    """Return the backward graph of ``fwd``.

    Backward-graph inputs: ``d_<out>`` for each forward output, then saved forward
    tensors (``meta['saved']``).  Outputs: ``d_<in>`` for each requested forward
    input that receives a gradient (``meta['input_grads']`` maps input -> grad)."""
    b = BackwardBuilder(fwd)
    grads: Dict[str, str] = {}
    for o in fwd.outputs:
        name = b.g.add_tensor(f"d_{o}", fwd.tensors[o].shape, fwd.tensors[o].dtype, kind="input")
        b.g.inputs.append(name)
        grads[o] = name

    for op in reversed(fwd.ops):
        out_grads = [grads.get(o) if o is not None else None for o in op.outputs]
        if not any(g is not None for g in out_grads):
            continue
        rule = _RULES.get(op.kind)
        if rule is None:
            raise NotImplementedError(f"[E015] no autodiff rule for op '{op.kind}'")
        contrib = rule(b, op, out_grads)
        for tensor, g in contrib.items():
            if b.is_param(tensor):
                continue  # rule already wrote grad::<param>
            if tensor in grads:
                acc = b.new_grad(tensor)
                b.emit("add", [grads[tensor], g], [acc])
                grads[tensor] = acc
            else:
                grads[tensor] = g

    wrt = list(wrt_inputs) if wrt_inputs is not None else [i for i in fwd.inputs if fwd.tensors[i].dtype not in ("int32", "opaque")]
    input_grads = {i: grads[i] for i in wrt if i in grads}
    b.g.outputs = list(input_grads.values())
    b.g.inputs += b.saved
    b.g.meta = {"saved": list(b.saved), "input_grads": input_grads, "out_grads": {o: grads[o] for o in fwd.outputs}}
    for s in b.saved:
        if s in fwd.tensors:
            fwd.tensors[s].save = True
    return b.g


# ------------------------------------------------------------------------------- rules

@register_autodiff("zeros")
def _zeros(b, op, dy):
    return {}


@register_autodiff("add")
def _add(b, op, dy):
    a, c = op.inputs
    return {a: dy[0], c: dy[0]} if a != c else {a: dy[0]}


@register_autodiff("scale")
def _scale(b, op, dy):
    g = b.new_grad(op.inputs[0])
    b.emit("scale", [dy[0]], [g], factor=op.attrs["factor"])
    return {op.inputs[0]: g}


@register_autodiff("mul")
def _mul(b, op, dy):
    x, y = op.inputs
    gx, gy = b.new_grad(x), b.new_grad(y)
    b.emit("mul", [dy[0], b.fwd_tensor(y)], [gx])
    b.emit("mul", [dy[0], b.fwd_tensor(x)], [gy])
    return {x: gx, y: gy}


@register_autodiff("view")
def _view(b, op, dy):
    x = op.inputs[0]
    g = b.new_grad(x)
    b.emit("view", [dy[0]], [g], shape=list(b.fwd.tensors[x].shape))
    return {x: g}


@register_autodiff("embedding")
def _embedding(b, op, dy):
    tok, w = op.inputs
    b.emit("embedding_backward", [dy[0], b.fwd_tensor(tok)], [b.param_grad(w)])
    return {}


@register_autodiff("rmsnorm")
def _rmsnorm(b, op, dy):
    x, w = op.inputs
    y, rstd = op.outputs
    gx = b.new_grad(x)
    b.emit("rmsnorm_backward", [dy[0], b.fwd_tensor(x), w, b.fwd_tensor(rstd), None], [gx, b.param_grad(w)], eps=op.attrs["eps"])
    return {x: gx}


@register_autodiff("fused_residual_rmsnorm")
def _fused_residual_rmsnorm(b, op, dy):
    res, x, w = op.inputs
    res_out, y, rstd = op.outputs
    d_res_out, d_y, _ = dy
    g = b.new_grad(x)
    if d_y is None:
        # only the residual stream carries gradient
        return {res: d_res_out, x: d_res_out}
    # d(res_out) = d_res_out + rmsnorm_bwd(d_y); both `residual` and `x` receive it unchanged
    b.emit("rmsnorm_backward", [d_y, b.fwd_tensor(res_out), w, b.fwd_tensor(rstd), d_res_out], [g, b.param_grad(w)], eps=op.attrs["eps"])
    return {res: g, x: g}


@register_autodiff("matmul")
def _matmul(b, op, dy):
    x, w, bias = op.inputs
    gx = b.new_grad(x)
    b.emit("matmul_backward", [dy[0], b.fwd_tensor(x), w], [gx, b.param_grad(w), b.param_grad(bias)],
           role=op.attrs.get("role", ""), fwd_out=op.outputs[0])
    return {x: gx}


@register_autodiff("qkv_qk_norm_rope")
def _qknr(b, op, dy):
    qkv, qw, kw, pos = op.inputs
    out, q_rstd, k_rstd = op.outputs
    g = b.new_grad(qkv)
    b.emit("qkv_qk_norm_rope_backward",
           [dy[0], b.fwd_tensor(qkv), qw, kw, b.fwd_tensor(q_rstd), b.fwd_tensor(k_rstd), b.fwd_tensor(pos)],
           [g, b.param_grad(qw), b.param_grad(kw)], **op.attrs)
    return {qkv: g}


@register_autodiff("flash_attention")
def _fa(b, op, dy):
    qkv = op.inputs[0]
    att, lse = op.outputs
    g = b.new_grad(qkv)
    b.emit("flash_attention_backward", [dy[0], b.fwd_tensor(qkv), b.fwd_tensor(att), b.fwd_tensor(lse)], [g], **op.attrs)
    return {qkv: g}


@register_autodiff("swiglu")
def _swiglu(b, op, dy):
    x = op.inputs[0]
    g = b.new_grad(x)
    b.emit("swiglu_backward", [dy[0], b.fwd_tensor(x)], [g])
    return {x: g}


@register_autodiff("tiled_mlp")
def _tiled_mlp(b, op, dy):
    x, up_w, down_w = op.inputs
    g = b.new_grad(x)
    b.emit("tiled_mlp_backward", [dy[0], b.fwd_tensor(x), up_w, down_w], [g, b.param_grad(up_w), b.param_grad(down_w)], **op.attrs)
    return {x: g}


@register_autodiff("silu")
def _silu(b, op, dy):
    x = op.inputs[0]
    g = b.new_grad(x)
    b.emit("silu_backward", [dy[0], b.fwd_tensor(x)], [g])
    return {x: g}


@register_autodiff("gelu")
def _gelu(b, op, dy):
    x = op.inputs[0]
    g = b.new_grad(x)
    b.emit("gelu_backward", [dy[0], b.fwd_tensor(x)], [g])
    return {x: g}


@register_autodiff("fused_lm_head_loss")
def _lmhead(b, op, dy):
    x, w, tgt = op.inputs
    g = b.new_grad(x)
    # the forward op (in training mode) already produced d_x and accumulated d_w; backward just hands d_x over
    b.emit("fused_lm_head_loss_backward", [dy[0], b.fwd_tensor(x), w, b.fwd_tensor(tgt), b.fwd_tensor(op.outputs[0])],
           [g, b.param_grad(w)], **op.attrs)
    return {x: g}


@register_autodiff("block_stack")
def _block_stack(b, op, dy):
    x, res, pos = op.inputs
    gx, gr = b.new_grad(x), b.new_grad(res)
    b.emit("block_stack_backward", [dy[0], dy[1]] + list(dy[2:]), [gx, gr], **op.attrs)
    return {x: gx, res: gr}


@register_autodiff("torch_fn")
def _torch_fn(b, op, dy):
    """Backward = replay under autograd: inputs are re-read (saved tensors / parameters), gradients flow to every floating
    input; parameter gradients go to ``grad::<param>``."""
    ins = list(op.inputs)
    grads, outs, contrib = [], [], {}
    for n in ins:
        if n is None:
            grads.append(None)
            continue
        if b.is_param(n):
            grads.append(b.param_grad(n))
        else:
            spec = b.fwd.tensors.get(n)
            if spec is not None and spec.dtype in ("int32", "opaque"):
                grads.append(None)
            else:
                g = b.new_grad(n)
                grads.append(g)
                contrib[n] = g
    b.emit("torch_fn_backward", list(dy) + [b.fwd_tensor(n) if (n is not None and not b.is_param(n)) else n for n in ins], grads,
           **{**op.attrs, "n_in": len(ins)})
    return contrib


# ---- MoE

@register_autodiff("moe_router")
def _moe_router(b, op, dy):
    x, rw = op.inputs
    tw, ti, aux = op.outputs
    g = b.new_grad(x)
    b.emit("moe_router_backward", [dy[0], dy[2], b.fwd_tensor(x), rw, b.fwd_tensor(tw), b.fwd_tensor(ti)],
           [g, b.param_grad(rw)], **op.attrs)
    return {x: g}


@register_autodiff("moe_permute")
def _moe_permute(b, op, dy):
    x, idx = op.inputs
    xp, plan = op.outputs
    g = b.new_grad(x)
    b.emit("moe_permute_backward", [dy[0], b.fwd_tensor(plan)], [g], **op.attrs)
    return {x: g}


@register_autodiff("ep_dispatch")
def _ep_dispatch(b, op, dy):
    xp, plan = op.inputs
    y, plan2 = op.outputs
    g = b.new_grad(xp)
    b.emit("ep_combine", [dy[0], b.fwd_tensor(plan2)], [g], backward=True)
    return {xp: g}


@register_autodiff("ep_combine")
def _ep_combine(b, op, dy):
    y, plan = op.inputs
    g = b.new_grad(y)
    b.emit("ep_dispatch_backward", [dy[0], b.fwd_tensor(plan)], [g])
    return {y: g}


@register_autodiff("moe_grouped_gemm")
def _moe_gg(b, op, dy):
    x, w, plan = op.inputs
    g = b.new_grad(x)
    b.emit("moe_grouped_gemm_backward", [dy[0], b.fwd_tensor(x), w, b.fwd_tensor(plan)], [g, b.param_grad(w)], role=op.attrs.get("role", ""),
           fwd_out=op.outputs[0])
    return {x: g}


@register_autodiff("moe_expert_bias_add")
def _moe_bias_add(b, op, dy):
    y, bias, plan = op.inputs
    g = b.new_grad(y)
    b.emit("moe_expert_bias_add_backward", [dy[0], bias, b.fwd_tensor(plan)], [g, b.param_grad(bias)])
    return {y: g}


@register_autodiff("moe_unpermute")
def _moe_unpermute(b, op, dy):
    y, tw, plan = op.inputs
    gy, gw = b.new_grad(y), b.new_grad(tw)
    b.emit("moe_unpermute_backward", [dy[0], b.fwd_tensor(y), b.fwd_tensor(tw), b.fwd_tensor(plan)], [gy, gw])
    return {y: gy, tw: gw}
