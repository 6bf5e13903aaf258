"""FP8-hybrid recipe: E4M3 activations and weights in forward, E5M2 output gradients in backward,
per-tensor delayed scaling with an abs-max history.

Every GEMM of a block (qkv, out, mlp_up, mlp_down) runs on the tcgen05 FP8 path (kind::f8f6f4):

* forward  : x(e4m3) . W(e4m3)^T
* dgrad    : dy(e5m2) . W(e4m3)          (W read MN-major: no transposed weight copy)
* wgrad    : dy(e5m2)^T . x(e4m3)        (both read MN-major: no transposed activation copies)

The expert projections of MoE layers run the same three GEMMs as grouped FP8 GEMMs (``recipes/grouped_fp8.py``).

Activations are quantised where they are produced (RMSNorm and SwiGLU kernels emit FP8 next to
recording the abs-max), weights once per optimizer step into a per-layer FP8 cache, and the FP8 copy
of an activation is what is saved for backward.  Scales follow the delayed-scaling rule: the scale
used at step t is derived from the maximum abs-max over the last ``history`` steps; a quantiser with
no history yet (first step) measures its abs-max just in time.

Parity: csrc/src/recipes/fp8_hybrid/fp8_hybrid_recipe.cpp:56-604, runtime/core/fp8_scaling_config.h,
recipes/fp8_hybrid/kernels/{quant,delayed_scaling}.cu.
"""
from __future__ import annotations

import os

from typing import Dict, Tuple

import torch

from ..runtime.ops_cuda import Fp8Tensor, gemm
from .base import Recipe
from .grouped_fp8 import GroupedFp8Mixin

E4M3_MAX = 448.0
E5M2_MAX = 57344.0
QUANT_ROLES = ("qkv", "out", "mlp_up", "mlp_down")


class FP8HybridRecipe(GroupedFp8Mixin, Recipe):
    name = "fp8_hybrid"

    def __init__(self, cm, device, history: int = 16, margin: int = 0, skip_first_layers: int = 0, skip_last_layers: int = 0,
                 fp8_lm_head: bool = True):
        self.device = device
        self.fp8_lm_head = bool(fp8_lm_head) and os.environ.get("SUROGATE_FP8_LM_HEAD", "1") != "0"
        self.history = history
        self.margin = margin
        self.n_layers = cm.n_layers
        self.skip = set(range(skip_first_layers)) | set(range(cm.n_layers - skip_last_layers, cm.n_layers))
        # quantiser slots: (layer, role, kind) with kind in x (e4m3) / w (e4m3) / dy (e5m2)
        self.index: Dict[Tuple[int, str, str], int] = {}
        fmax = []
        for L in range(cm.n_layers):
            for role in QUANT_ROLES:
                for kind in ("x", "w", "dy"):
                    self.index[(L, role, kind)] = len(fmax)
                    fmax.append(E5M2_MAX if kind == "dy" else E4M3_MAX)
        Q = len(fmax)
        self.fmax = torch.tensor(fmax, dtype=torch.float32, device=device)
        self.amax_hist = torch.zeros(history, Q, dtype=torch.float32, device=device)
        self.amax_cur = torch.zeros(Q, dtype=torch.float32, device=device)
        self.scale = torch.ones(Q, dtype=torch.float32, device=device)
        self.scale_inv = torch.ones(Q, dtype=torch.float32, device=device)
        self.have_history = False
        self.weight_cache: Dict[Tuple[int, str], Fp8Tensor] = {}
        self.expert_weight_cache: Dict[Tuple[int, str], tuple] = {}
        self.weight_version = 0

    # ------------------------------------------------------------------ scaling state
    def slot(self, layer: int, role: str, kind: str) -> int:
        return self.index[(layer, role, kind)]

    def _quantize(self, ext, x: torch.Tensor, q: int, e5m2: bool) -> Fp8Tensor:
        """Quantise with the delayed scale (recording abs-max), or just-in-time when no history exists."""
        x = x.contiguous()
        if not self.have_history:
            am = self.amax_cur[q:q + 1]
            ext.amax(x, am)
            # scale = fmax / amax (amax > 0), computed on the device: no host sync
            s = torch.where(am > 0, self.fmax[q:q + 1] / am / (2.0 ** self.margin), torch.ones_like(am))
            self.scale[q:q + 1] = s
            self.scale_inv[q:q + 1] = 1.0 / s
            data = ext.quantize_fp8(x, self.scale[q:q + 1], None, e5m2)
        else:
            data = ext.quantize_fp8(x, self.scale[q:q + 1], self.amax_cur[q:q + 1], e5m2)
        return Fp8Tensor(data, self.scale_inv[q:q + 1])

    def end_step(self) -> None:
        """Roll the abs-max history and derive next step's scales (a handful of tiny tensor ops)."""
        self.amax_hist = torch.roll(self.amax_hist, 1, 0)
        self.amax_hist[0] = self.amax_cur
        amax = self.amax_hist.max(0).values
        s = torch.where(amax > 0, self.fmax / amax / (2.0 ** self.margin), self.scale)
        s = torch.where(torch.isfinite(s), s, self.scale)
        self.scale.copy_(s)
        self.scale_inv.copy_(1.0 / s)
        self.amax_cur.zero_()
        self.have_history = True
        self.grouped_end_step()

    def on_weights_updated(self, store) -> None:
        self.weight_cache.clear()
        self.expert_weight_cache.clear()
        self.weight_version += 1

    def state_dict(self):
        return {"amax_hist": self.amax_hist, "scale": self.scale, "have_history": self.have_history}

    def load_state_dict(self, sd) -> None:
        self.amax_hist.copy_(sd["amax_hist"])
        self.scale.copy_(sd["scale"])
        self.scale_inv.copy_(1.0 / self.scale)
        self.have_history = bool(sd["have_history"])

    # ------------------------------------------------------------------ which ops produce FP8
    _CONSUMER_ROLE = {"ln1": "qkv", "ln2": "mlp_up", "swiglu": "mlp_down"}

    def _active(self, ctx, role: str) -> bool:
        return ctx.layer is not None and ctx.layer not in self.skip and role in QUANT_ROLES

    def wants_fp8_activation(self, ctx, op, out_index: int) -> bool:
        name = op.outputs[out_index]
        if ctx.layer is None or ctx.layer in self.skip or name not in self._CONSUMER_ROLE:
            return False
        return self._only_fp8_matmuls_read(ctx.graph, name)

    def _only_fp8_matmuls_read(self, graph, name: str) -> bool:
        """An activation is emitted as FP8 only when every op that reads it is a matmul of a quantised role: in MoE blocks the
        second norm feeds the router and the token permutation, which want bf16."""
        if graph is None:
            return True
        compiled = graph.meta.get("consumers")      # written by the graph compiler (dsl/graph_compiler.py: annotate_consumers)
        if compiled is not None and name in compiled:
            return bool(compiled[name]["quant_only"])
        cache = self.__dict__.setdefault("_fp8_reader_cache", {})
        key = (id(graph), name)
        ok = cache.get(key)
        if ok is None:
            readers = [o for o in graph.ops if name in o.inputs]
            ok = bool(readers) and all(o.kind == "matmul" and o.attrs.get("role", "") in QUANT_ROLES for o in readers)
            cache[key] = ok
        return ok

    def swiglu_backward_fp8(self, ctx, op, ext, dy, x):
        """d(MLP-up output) straight as E5M2 when its only reader is the FP8 backward of the up projection (no bias gradient, no
        adapter): the bf16 gradient is never written and the separate quantise pass disappears.  None = take the bf16 path."""
        if not self.have_history or ctx.layer is None or ctx.layer in self.skip or ctx.lora is not None or ctx.graph is None:
            return None
        cache = self.__dict__.setdefault("_fp8_grad_reader_cache", {})
        key = (id(ctx.graph), op.outputs[0])
        ok = cache.get(key)
        if ok is None:
            readers = [o for o in ctx.graph.ops if op.outputs[0] in o.inputs]
            ok = cache[key] = (len(readers) == 1 and readers[0].kind == "matmul_backward" and readers[0].attrs.get("role", "") == "mlp_up"
                               and readers[0].inputs[0] == op.outputs[0] and readers[0].outputs[2] is None)
        if not ok or getattr(x, "_sg_rows", None) is not None:
            return None
        q = self.slot(ctx.layer, "mlp_up", "dy")
        d8 = ext.swiglu_bwd_fp8(dy.contiguous(), x, self.scale[q:q + 1], self.amax_cur[q:q + 1])
        return Fp8Tensor(d8, self.scale_inv[q:q + 1])

    def norm_forward(self, ctx, op, ext, x, residual, w):
        role = self._CONSUMER_ROLE[op.outputs[1 if residual is not None or len(op.outputs) == 3 else 0]]
        q = self.slot(ctx.layer, role, "x")
        if not self.have_history:
            res, y, rstd, _ = ext.rmsnorm_fwd(x, residual, w, op.attrs["eps"], True, None, None, False)
            return res, self._quantize(ext, y, q, False), rstd
        res, _, rstd, y8 = ext.rmsnorm_fwd(x, residual, w, op.attrs["eps"], False, self.scale[q:q + 1], self.amax_cur[q:q + 1], True)
        return res, Fp8Tensor(y8, self.scale_inv[q:q + 1]), rstd

    def swiglu_forward(self, ctx, op, ext, x):
        q = self.slot(ctx.layer, "mlp_down", "x")
        if not self.have_history:
            y = ext.swiglu_fwd(x, True, None, None, False)[0]
            return self._quantize(ext, y, q, False)
        _, y8 = ext.swiglu_fwd(x, False, self.scale[q:q + 1], self.amax_cur[q:q + 1], True)
        return Fp8Tensor(y8, self.scale_inv[q:q + 1])

    # ------------------------------------------------------------------ LM head
    def quantize_now(self, ext, x: torch.Tensor):
        """E4M3 with the scale of this very tensor (one abs-max pass): used where no amax history exists (LM-head input)."""
        am = torch.zeros(1, dtype=torch.float32, device=x.device)
        ext.amax(x, am)
        s = torch.where(am > 0, 448.0 / am, torch.ones_like(am))
        return ext.quantize_fp8(x, s, None, False), 1.0 / s

    def lm_head_weight(self, ext, w: torch.Tensor):
        """E4M3 copy of the LM-head matrix, rebuilt once per optimizer step (dropped by on_weights_updated)."""
        c = self.weight_cache.get(("lm_head", w.data_ptr()))
        if c is None:
            c = self.weight_cache[("lm_head", w.data_ptr())] = self.quantize_now(ext, w)
        return c

    # ------------------------------------------------------------------ GEMMs
    def quantizes(self, layer, role: str) -> bool:
        return layer is not None and layer not in self.skip and role in QUANT_ROLES

    def _weight(self, ctx, ext, role: str, w: torch.Tensor, pname: str = "") -> Fp8Tensor:
        pre = ctx.ex.store.get_fp8(ctx.full_name(pname)) if pname else None
        if pre is not None:   # already E4M3: written by the quantise-on-gather kernel with this tensor's scale
            return Fp8Tensor(pre[0], pre[1])
        key = (ctx.layer, role)
        cached = self.weight_cache.get(key)
        if cached is not None:
            return cached
        q = self.slot(ctx.layer, role, "w")
        if self.have_history:
            # delayed scaling like the activations: one pass that quantises with the scale derived from the earlier steps' abs-max and
            # records this step's (weights move by a learning-rate-sized step, so last step's abs-max is a tight bound)
            data = ext.quantize_fp8(w, self.scale[q:q + 1], self.amax_cur[q:q + 1], False)
            t = Fp8Tensor(data, self.scale_inv[q:q + 1])
            self.weight_cache[key] = t
            return t
        am = self.amax_cur[q:q + 1]
        am.zero_()
        ext.amax(w, am)
        s = torch.where(am > 0, self.fmax[q:q + 1] / am / (2.0 ** self.margin), torch.ones_like(am))
        self.scale[q:q + 1] = s
        self.scale_inv[q:q + 1] = 1.0 / s
        data = ext.quantize_fp8(w, self.scale[q:q + 1], None, False)
        t = Fp8Tensor(data, self.scale_inv[q:q + 1].clone())
        self.weight_cache[key] = t
        return t

    def forward_matmul(self, ctx, op, x, w, bias):
        role = op.attrs.get("role", "")
        if not self._active(ctx, role) or w.dtype != torch.bfloat16:
            if isinstance(x, Fp8Tensor):
                raise RuntimeError("FP8 activation reached a non-FP8 matmul")
            return None
        from ..ops import ext as _ext

        ext = _ext()
        K = x.shape[-1]
        lead = tuple(x.shape[:-1])
        if not isinstance(x, Fp8Tensor):
            x = self._quantize(ext, x.reshape(-1, K), self.slot(ctx.layer, role, "x"), False)
            ctx.stash[("fp8x", ctx.layer, op.outputs[0])] = x
        x2 = x.reshape(-1, K)
        w8 = self._weight(ctx, ext, role, w, op.inputs[1])
        y = gemm(x2.data, w8.data, scale_a=x2.scale_inv, scale_b=w8.scale_inv)
        y = y.reshape(*lead, w.shape[0])
        if bias is not None:
            y += bias
        return y

    def backward_matmul(self, ctx, op, dy2, x2, w):
        role = op.attrs.get("role", "")
        if not self._active(ctx, role) or w.dtype != torch.bfloat16:
            return None
        from ..ops import ext as _ext

        ext = _ext()
        if not isinstance(x2, Fp8Tensor):
            saved = ctx.stash.pop(("fp8x", ctx.layer, op.attrs.get("fwd_out")), None)
            x2 = saved if saved is not None else self._quantize(ext, x2, self.slot(ctx.layer, role, "x"), False)
        dy8 = dy2 if isinstance(dy2, Fp8Tensor) else self._quantize(ext, dy2, self.slot(ctx.layer, role, "dy"), True)
        w8 = self._weight(ctx, ext, role, w, op.inputs[2])
        dx = gemm(dy8.data, w8.data, a_mn=False, b_mn=True, scale_a=dy8.scale_inv, scale_b=w8.scale_inv)
        tgt, acc = ctx.grad_target(op.outputs[1])
        if tgt is not None:
            gemm(dy8.data, x2.data, tgt, a_mn=True, b_mn=True, accumulate=acc, scale_a=dy8.scale_inv, scale_b=x2.scale_inv)
        return dx, None
