"""FP8 grouped GEMMs for the experts of MoE layers (shared by the FP8-hybrid and NVFP4 recipes).

Per expert projection (``experts_gate_up``, ``experts_down``) the three grouped GEMMs run on the tcgen05 FP8 path with the
device-side tile scheduler over the experts' row offsets:

* forward : x (e4m3) . W[e] (e4m3)^T              rows grouped by expert
* dgrad   : dy (e5m2) . W[e] (e4m3)               W read MN-major, no transposed copy
* wgrad   : dy[e] (e5m2)^T . x[e] (e4m3)          contraction grouped by expert, both operands read MN-major

Scales are per tensor and delayed by one step: the quantise pass records the abs-max from which the next step's scale is derived
(the first step measures its abs-max just in time).  The expert buffers of an expert-parallel step are sized for the worst case;
every pass stops at the device-side count of rows in use.  The whole stack of a layer's expert matrices shares one scale.  Padding rows between experts are zero
in every operand, so they add nothing to any product.

Parity: csrc/src/kernels/moe/moe_fp8_grouped_gemm.cu, csrc/src/kernels/moe_cudnn.cpp:315,513 (the reference's FP8 / FP4
grouped expert GEMMs).
"""
from __future__ import annotations

import torch

E4M3_MAX = 448.0
E5M2_MAX = 57344.0
EXPERT_ROLES = ("experts_gate_up", "experts_down")


class GroupedFp8Mixin:
    """Needs ``self.skip`` (set of layers left in bf16), ``self.n_layers`` and a per-step ``self.expert_weight_cache`` dict cleared by
    ``on_weights_updated``; the recipe calls ``grouped_end_step()`` from its ``end_step``."""

    quantize_experts = True
    _KINDS = {"x": 0, "w": 1, "dy": 2}

    # ------------------------------------------------------------------ scaling state (delayed, one slot per layer / role / operand)
    def _gstate(self, device):
        st = self.__dict__.get("_g_state")
        if st is None:
            Q = max(1, int(getattr(self, "n_layers", 1))) * len(EXPERT_ROLES) * 3
            fmax = torch.full((Q,), E4M3_MAX, dtype=torch.float32, device=device)
            fmax[2::3] = E5M2_MAX
            st = self.__dict__["_g_state"] = {"scale": torch.ones(Q, dtype=torch.float32, device=device), "inv": torch.ones(Q, dtype=torch.float32, device=device),
                                              "amax": torch.zeros(Q, dtype=torch.float32, device=device), "fmax": fmax, "have": False}
        return st

    def _gslot(self, layer: int, role: str, kind: str) -> int:
        return (layer * len(EXPERT_ROLES) + EXPERT_ROLES.index(role)) * 3 + self._KINDS[kind]

    def grouped_end_step(self) -> None:
        """Next step's scales from this step's abs-max values (three vector ops for all slots); slots not used this step keep theirs."""
        st = self.__dict__.get("_g_state")
        if st is None:
            return
        comm = self.__dict__.get("ep_group_comm")
        if comm is not None and self.dispatch_in_fp8:
            # rows quantised by different ranks meet in one receive buffer: every rank of the expert group must derive the same scale
            comm.all_reduce(st["amax"], "max")
        s = torch.where(st["amax"] > 0, st["fmax"] / st["amax"], st["scale"])
        st["scale"].copy_(torch.where(torch.isfinite(s), s, st["scale"]))
        st["inv"].copy_(1.0 / st["scale"])
        st["amax"].zero_()
        st["have"] = True

    def _gq(self, ext, x: torch.Tensor, e5m2: bool, used, q: int):
        """(fp8 data, de-scale) of ``x``.  With a scale from the previous step: one pass that quantises and records the abs-max for the
        next step; without (first step): an abs-max pass first.  ``used``: device row count in use (or None)."""
        st = self._gstate(x.device)
        x2 = x.contiguous().reshape(-1, x.shape[-1])
        sc, inv, am = st["scale"][q:q + 1], st["inv"][q:q + 1], st["amax"][q:q + 1]
        if not st["have"]:
            am.zero_()
            ext.amax(x2, am, used)
            sc.copy_(torch.where(am > 0, st["fmax"][q:q + 1] / am, torch.ones_like(am)))
            inv.copy_(1.0 / sc)
            return ext.quantize_fp8(x2, sc, None, e5m2, used), inv
        return ext.quantize_fp8(x2, sc, am, e5m2, used), inv

    def _expert_weight(self, ctx, ext, role: str, w: torch.Tensor):
        """E4M3 copy of a layer's expert stack.  Kept for the whole optimizer step (forward and backward read it) when all layers'
        copies together stay below a twentieth of the device memory; a rank that holds many experts (small expert-parallel degree)
        quantises at each use instead and holds one layer's copy at a time."""
        key = (ctx.layer, role)
        c = self.expert_weight_cache.get(key)
        if c is not None:
            return c
        q, inv = self._gq(ext, w.reshape(-1, w.shape[-1]), False, None, self._gslot(ctx.layer, role, "w"))
        c = (q.reshape(w.shape), inv)
        keep = self.__dict__.get("_keep_expert_copies")
        if keep is None:
            n_layers = max(1, int(getattr(self, "n_layers", 1)))
            total = torch.cuda.get_device_properties(w.device).total_memory
            keep = self.__dict__["_keep_expert_copies"] = 3 * w.numel() * n_layers < total // 20   # gate_up + down of every layer, one byte each
        if keep:
            self.expert_weight_cache[key] = c
        return c

    def _grouped_active(self, ctx, op, x, w) -> bool:
        role = op.attrs.get("role", "")
        return (self.quantize_experts and ctx.layer is not None and ctx.layer not in self.skip and role in EXPERT_ROLES and torch.is_tensor(x)
                and (x.dtype == torch.bfloat16 or self._arrived_fp8(x)) and w.dtype == torch.bfloat16 and w.dim() == 3 and w.shape[1] % 16 == 0
                and w.shape[2] % 16 == 0)

    # ------------------------------------------------------------------ rows that crossed NVLink already quantised
    import os as _os

    dispatch_in_fp8 = _os.environ.get("SUROGATE_EP_FP8_DISPATCH", "1") == "1"    # 0: bf16 rows cross NVLink and the owner quantises them

    @staticmethod
    def _arrived_fp8(x) -> bool:
        return x.dtype == torch.float8_e4m3fn and getattr(x, "_sg_inv", None) is not None

    def dispatch_fp8(self, ctx, x):
        """(scale, de-scale, abs-max slot) when the expert-parallel dispatch of this layer may send E4M3 rows: the first expert GEMM
        then reads them as they arrive and the bf16 rows are never stored on the receiving side.  Needs a scale from an earlier step
        (the same on every rank of the expert group, see ``grouped_end_step``) and no adapter reading the rows in bf16."""
        st = self.__dict__.get("_g_state")
        if (not self.dispatch_in_fp8 or st is None or not st["have"] or not self.quantize_experts or ctx.layer is None or ctx.layer in self.skip
                or getattr(ctx, "lora", None) is not None or x.dtype != torch.bfloat16 or x.shape[-1] % 16 != 0
                or getattr(getattr(ctx, "ex", None), "offload", None) is not None):   # parked saved tensors come back without their scale tag
            return None
        q = self._gslot(ctx.layer, "experts_gate_up", "x")
        return st["scale"][q:q + 1], st["inv"][q:q + 1], st["amax"][q:q + 1]

    def forward_grouped(self, ctx, op, x, w, plan):
        if not self._grouped_active(ctx, op, x, w):
            return None
        from ..ops import ext as _ext

        ext = _ext()
        role = op.attrs["role"]
        used = getattr(x, "_sg_rows", None)
        if self._arrived_fp8(x):
            x8, x_inv = x, x._sg_inv
        else:
            x8, x_inv = self._gq(ext, x, False, used, self._gslot(ctx.layer, role, "x"))
        w8, w_inv = self._expert_weight(ctx, ext, role, w)
        y = (torch.empty if used is not None else torch.zeros)(x.shape[0], w.shape[1], dtype=torch.bfloat16, device=x.device)
        ext.gemm_grouped(x8, w8, y, plan.offsets, 1, False, False, 1.0, x_inv, w_inv, ext.error_flag_tensor())
        if used is not None:
            y._sg_rows = used
        self.__dict__["_grouped_calls"] = self.__dict__.get("_grouped_calls", 0) + 1
        return y

    def backward_grouped(self, ctx, op, dy, x, w, plan):
        if not self._grouped_active(ctx, op, x, w):
            return None
        from ..ops import ext as _ext

        ext = _ext()
        err = ext.error_flag_tensor()
        role = op.attrs["role"]
        used = getattr(dy, "_sg_rows", None)
        if used is None:
            used = getattr(x, "_sg_rows", None)
        dy8, dy_inv = self._gq(ext, dy, True, used, self._gslot(ctx.layer, role, "dy"))
        w8, w_inv = self._expert_weight(ctx, ext, role, w)
        dx = (torch.empty if used is not None else torch.zeros)(x.shape, dtype=torch.bfloat16, device=x.device)
        ext.gemm_grouped(dy8, w8, dx, plan.offsets, 1, True, False, 1.0, dy_inv, w_inv, err)          # dy [R, N] . W[e] [N, K]
        if used is not None:
            dx._sg_rows = used
        tgt, acc = ctx.grad_target(op.outputs[1])
        if tgt is not None:
            # re-quantised from the saved bf16 rows with the scale the forward used: a second FP8 copy per layer is not kept
            if self._arrived_fp8(x):
                x8, x_inv = x, x._sg_inv
            else:
                x8, x_inv = self._gq(ext, x, False, used, self._gslot(ctx.layer, role, "x"))
            ext.gemm_grouped(dy8, x8, tgt, plan.offsets, 2, True, acc, 1.0, dy_inv, x_inv, err)         # dW[e] (+)= dy[e]^T . x[e]
            if not acc:
                ext.zero_empty_groups(tgt, plan.offsets)
        return dx
