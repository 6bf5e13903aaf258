"""LoRA on the fused projection weights and on the per-expert matrices of MoE layers.

Each target module (q/k/v/o/gate/up/down) is a row slice of a fused internal weight.  For one fused matmul
with input ``x`` the adapters of all its targets share the first GEMM: ``h = x . A_cat^T`` with
``A_cat = [A_q; A_k; A_v]`` (N = targets * rank), then each target adds ``h_t . B_t^T * (alpha/r)`` into its
column slice of the output through the GEMM's accumulate epilogue on a strided view.  Backward mirrors it
with four small GEMMs.  On a GPU every one of these runs on the tcgen05 GEMM (small-N / small-K shapes use
its zero-filled tiles); on CPU plain matmuls.

Expert stacks ([E, N, K] parameters: ``experts_gate_up`` with the up / gate slices, ``experts_down``) get one adapter pair per expert,
stored as [E, r, K] / [E, rows, r]; their forward and backward run as grouped GEMMs over the same expert row offsets as the base
projections (csrc/src/runtime/lora/fast_expert_lora.h in the reference), and they export under
``...layers.L.mlp.experts.E.up_proj.lora_A.weight`` style keys.

Adapters are replicated across data-parallel ranks; their gradients are summed with one all-reduce of a flat
buffer, and the optimizer (AdamW fp32 or 8-bit state) runs on that flat buffer.  Masters are fp32 by default.

Export is PEFT-compatible: ``adapter_model.safetensors`` with
``base_model.model.model.layers.L.self_attn.q_proj.lora_A.weight`` style keys and ``adapter_config.json``.

Parity: csrc/src/runtime/lora/ (ModularLoRAConfig lora_config.h:39, lora_weights_manager.cpp,
lora_grads_manager.cpp:369-372), runtime/dsl/dsl_model_lora.cpp:41-63 (PEFT export), surogate/utils/lora_compat.py.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch

_MODULE_PATH = {"q_proj": "self_attn.q_proj", "k_proj": "self_attn.k_proj", "v_proj": "self_attn.v_proj", "o_proj": "self_attn.o_proj",
                "gate_proj": "mlp.gate_proj", "up_proj": "mlp.up_proj", "down_proj": "mlp.down_proj"}


@dataclass
class _Target:
    name: str  # q_proj ...
    row_off: int
    rows: int
    a_off: int  # offsets into the flat buffer
    b_off: int


class _Group:
    """All adapters attached to one fused weight of one layer."""

    def __init__(self, layer: int, param: str, in_features: int, targets: List[_Target], experts: int = 0):
        self.layer, self.param, self.in_features, self.targets = layer, param, in_features, targets
        self.experts = experts   # > 0: a stack of per-expert matrices [E, N, K]; every expert has its own A [r, K] and B [rows, r]


class LoRAManager:
    def __init__(self, cm, cfg: Dict[str, Any], device, comm, dtype=torch.bfloat16):
        self.cm, self.device, self.comm = cm, device, comm
        self.rank_dim = int(cfg.get("rank", 16))
        self.alpha = float(cfg.get("alpha", 32))
        self.dropout = float(cfg.get("dropout", 0.0))
        self.rslora = bool(cfg.get("rslora", False))
        self.train_router = bool(cfg.get("train_router", False))
        self.wanted = list(cfg.get("targets") or _MODULE_PATH)
        self.master_dtype = torch.float32 if cfg.get("dtype", "fp32") in ("fp32", "float32") else torch.bfloat16
        self.compute_dtype = dtype if device.type == "cuda" else torch.float32
        self.scaling = self.alpha / (math.sqrt(self.rank_dim) if self.rslora else self.rank_dim)
        self.groups: Dict[Tuple[int, str], _Group] = {}
        r = self.rank_dim
        n = 0
        for p in cm.params:
            if p.layer is None or not p.spec.lora_targets or len(p.spec.shape) not in (2, 3):
                continue
            E = p.spec.shape[0] if len(p.spec.shape) == 3 else 0   # expert stacks: one adapter pair per expert, stored [E, r, K] / [E, rows, r]
            K = p.spec.shape[-1]
            tl = []
            for tname, off, rows in p.spec.lora_targets:
                if tname not in self.wanted:
                    continue
                a_off = n
                n += max(1, E) * r * K
                b_off = n
                n += max(1, E) * rows * r
                tl.append(_Target(tname, off, rows, a_off, b_off))
            if tl:
                self.groups[(p.layer, p.local)] = _Group(p.layer, p.local, K, tl, experts=E)
        self.numel = (n + 127) // 128 * 128
        self.master = torch.zeros(self.numel, dtype=self.master_dtype, device=device)
        self.grad = torch.zeros(self.numel, dtype=torch.float32, device=device)
        self.work = self.master if self.master_dtype == self.compute_dtype else torch.zeros(self.numel, dtype=self.compute_dtype, device=device)
        self.opt_state: Optional[Dict[str, torch.Tensor]] = None
        self._written: set = set()
        self.use_kernels = device.type == "cuda"

    # ------------------------------------------------------------------ policy
    def freezes(self, name: str) -> bool:
        """Base parameters are frozen under LoRA (optionally except the MoE router)."""
        if self.train_router and name.endswith("router_weight"):
            return False
        return True

    # ------------------------------------------------------------------ weights
    def _A(self, buf, g: _Group, t: _Target):
        return buf[t.a_off:t.a_off + self.rank_dim * g.in_features].view(self.rank_dim, g.in_features)

    def _B(self, buf, t: _Target):
        return buf[t.b_off:t.b_off + t.rows * self.rank_dim].view(t.rows, self.rank_dim)

    def _EA(self, buf, g: _Group, t: _Target):
        return buf[t.a_off:t.a_off + g.experts * self.rank_dim * g.in_features].view(g.experts, self.rank_dim, g.in_features)

    def _EB(self, buf, g: _Group, t: _Target):
        return buf[t.b_off:t.b_off + g.experts * t.rows * self.rank_dim].view(g.experts, t.rows, self.rank_dim)

    def _A_cat(self, buf, g: _Group):
        """A matrices of one group are contiguous in the flat buffer only if interleaved B's are skipped: build views."""
        return [self._A(buf, g, t) for t in g.targets]

    def init_weights(self, seed: int = 0) -> None:
        """A ~ Kaiming-uniform(a=sqrt(5)) (bound 1/sqrt(in)), B = 0: the adapted model starts identical to the base."""
        gen = torch.Generator(device="cpu").manual_seed(seed + 7919)
        flat = torch.zeros(self.numel, dtype=torch.float32)
        for g in self.groups.values():
            bound = 1.0 / math.sqrt(g.in_features)
            for t in g.targets:
                n = max(1, g.experts) * self.rank_dim * g.in_features
                flat[t.a_off:t.a_off + n] = (torch.rand(n, generator=gen) * 2 - 1) * bound
        self.master.copy_(flat.to(self.master_dtype))
        self.sync_work()

    def sync_work(self) -> None:
        if self.work is not self.master:
            self.work.copy_(self.master)

    # ------------------------------------------------------------------ forward / backward hooks (called by the matmul ops)
    def _mm(self, a, b_t):
        """a @ b_t^T with b_t stored [N, K]."""
        if self.use_kernels and a.dtype == torch.bfloat16:
            from .ops_cuda import gemm

            return gemm(a, b_t)
        return a @ b_t.t()

    def forward(self, ctx, op, x, y):
        g = self.groups.get((ctx.layer, op.inputs[1])) if ctx.layer is not None else None
        if g is None or g.experts:
            return y
        if hasattr(x, "scale_inv"):
            x = x.hp if x.hp is not None else x.dequantize()
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        if self.dropout > 0 and ctx.training:
            mask = (torch.rand(x2.shape, device=x2.device) >= self.dropout).to(x2.dtype) / (1 - self.dropout)
            ctx.stash[("lora_mask", ctx.layer, op.outputs[0])] = mask
            x2 = x2 * mask
        y2 = y.reshape(-1, y.shape[-1])
        r = self.rank_dim
        a_cat = torch.cat(self._A_cat(self.work, g), dim=0)  # [targets*r, K]
        h = self._mm(x2, a_cat)  # [M, targets*r]
        ctx.stash[("lora_h", ctx.layer, op.outputs[0])] = h
        for i, t in enumerate(g.targets):
            ht = h[:, i * r:(i + 1) * r]
            Bt = self._B(self.work, t)
            ys = y2[:, t.row_off:t.row_off + t.rows]
            if self.use_kernels and ht.dtype == torch.bfloat16:
                from .ops_cuda import gemm

                gemm(ht, Bt, ys, accumulate=True, alpha=self.scaling)
            else:
                ys += (ht @ Bt.t()) * self.scaling
        return y

    def backward(self, ctx, op, dy2, x2):
        """Accumulates adapter gradients; returns the extra d_x contribution (or None)."""
        g = self.groups.get((ctx.layer, op.inputs[2])) if ctx.layer is not None else None
        if g is None or g.experts:
            return None
        if hasattr(x2, "scale_inv"):
            x2 = x2.hp if x2.hp is not None else x2.dequantize()
        key = op.attrs.get("fwd_out")
        mask = ctx.stash.pop(("lora_mask", ctx.layer, key), None)
        if mask is not None:
            x2 = x2 * mask
        h = ctx.stash.pop(("lora_h", ctx.layer, key), None)
        r = self.rank_dim
        if h is None:  # recompute path dropped it
            h = self._mm(x2, torch.cat(self._A_cat(self.work, g), dim=0))
        dh = torch.empty_like(h)
        a_list = self._A_cat(self.work, g)
        a_cat = torch.cat(a_list, dim=0)
        if self.use_kernels and h.dtype == torch.bfloat16 and dy2.dtype == torch.bfloat16:
            from .ops_cuda import gemm

            for i, t in enumerate(g.targets):
                dys = dy2[:, t.row_off:t.row_off + t.rows]
                # d_h_t = s * dy_slice . B_t   (B_t stored [rows, r] = [contraction, N])
                gemm(dys, self._B(self.work, t), dh[:, i * r:(i + 1) * r], b_mn=True, alpha=self.scaling)
                # dB_t += s * dy_slice^T . h_t  and  dA_t += d_h_t^T . x, straight into the fp32 gradient buffer
                gemm(dys, h[:, i * r:(i + 1) * r], self._B(self.grad, t), a_mn=True, b_mn=True, accumulate=True, alpha=self.scaling)
            for i, t in enumerate(g.targets):
                gemm(dh[:, i * r:(i + 1) * r], x2, self._A(self.grad, g, t), a_mn=True, b_mn=True, accumulate=True)
            dx = gemm(dh, a_cat, b_mn=True)
        else:
            for i, t in enumerate(g.targets):
                dys = dy2[:, t.row_off:t.row_off + t.rows]
                Bt = self._B(self.work, t)
                dh[:, i * r:(i + 1) * r] = (dys @ Bt) * self.scaling
                self._acc(t.b_off, (dys.t() @ h[:, i * r:(i + 1) * r]) * self.scaling)
            dA = dh.t() @ x2
            for i, t in enumerate(g.targets):
                self._acc(t.a_off, dA[i * r:(i + 1) * r])
            dx = dh @ a_cat
        if mask is not None:
            dx = dx * mask
        return dx

    # ------------------------------------------------------------------ per-expert adapters (grouped GEMM ops of MoE layers)
    def _local_expert_range(self, ctx, g: _Group, groups: int):
        """Global ids [e0, e0 + groups) of the experts whose rows this rank's grouped GEMM sees.  Adapters are kept for all experts on
        every rank (their gradients are summed like the dense adapters'); under expert parallelism a rank trains its own experts'
        slices, which assumes the identity expert placement (adapters do not travel with re-placed experts)."""
        ep = getattr(ctx, "ep", None)
        if ep is None or groups == g.experts:
            return 0
        if getattr(ep, "placement", None):
            raise RuntimeError("per-expert LoRA under expert parallelism needs the identity expert placement (ep_plan_refresh_interval: 0)")
        return ep.rank * groups

    def _ggemm(self, a, b, out, offsets, mode, b_mn=False, accumulate=False, alpha=1.0):
        from ..ops import ext

        e = ext()
        e.gemm_grouped(a.contiguous(), b.contiguous(), out, offsets, mode, b_mn, accumulate, float(alpha), None, None, e.error_flag_tensor())
        return out

    def forward_grouped(self, ctx, op, x, y, plan):
        """y[rows of expert e, slice t] += s * (x A_e,t^T) B_e,t^T for every adapted slice of an expert stack."""
        g = self.groups.get((ctx.layer, op.inputs[1])) if ctx.layer is not None else None
        if g is None or not g.experts:
            return y
        p = getattr(plan, "ep_plan", None) or getattr(plan, "local", None) or plan
        offsets = p.offsets
        G = offsets.numel() - 1 if not hasattr(p, "layout") else (p.layout.numel() - 2) // 2
        offsets = offsets[:G + 1]
        e0 = self._local_expert_range(ctx, g, G)
        r, T = self.rank_dim, len(g.targets)
        a_cat = torch.cat([self._EA(self.work, g, t)[e0:e0 + G] for t in g.targets], dim=1)     # [G, T*r, K]
        kernels = self.use_kernels and x.dtype == torch.bfloat16 and a_cat.dtype == torch.bfloat16
        if kernels:
            h = self._ggemm(x, a_cat, torch.zeros(x.shape[0], T * r, dtype=x.dtype, device=x.device), offsets, 1)
            for i, t in enumerate(g.targets):
                d = self._ggemm(h[:, i * r:(i + 1) * r], self._EB(self.work, g, t)[e0:e0 + G], torch.zeros(x.shape[0], t.rows, dtype=x.dtype, device=x.device),
                                offsets, 1, alpha=self.scaling)
                y[:, t.row_off:t.row_off + t.rows] += d
        else:
            off = offsets.tolist()   # host sync: reference path only
            h = torch.zeros(x.shape[0], T * r, dtype=x.dtype, device=x.device)
            for e in range(G):
                s0, s1 = off[e], off[e + 1]
                if s1 <= s0:
                    continue
                h[s0:s1] = x[s0:s1] @ a_cat[e].to(x.dtype).t()
                for i, t in enumerate(g.targets):
                    y[s0:s1, t.row_off:t.row_off + t.rows] += (h[s0:s1, i * r:(i + 1) * r] @ self._EB(self.work, g, t)[e0 + e].to(x.dtype).t()) * self.scaling
        ctx.stash[("lora_gh", ctx.layer, op.outputs[0])] = h
        return y

    def backward_grouped(self, ctx, op, dy, x, plan):
        """Adapter gradients of an expert stack; returns the extra d_x (or None)."""
        g = self.groups.get((ctx.layer, op.inputs[2])) if ctx.layer is not None else None
        if g is None or not g.experts:
            return None
        p = getattr(plan, "ep_plan", None) or getattr(plan, "local", None) or plan
        offsets = p.offsets
        G = offsets.numel() - 1 if not hasattr(p, "layout") else (p.layout.numel() - 2) // 2
        offsets = offsets[:G + 1]
        e0 = self._local_expert_range(ctx, g, G)
        r, T = self.rank_dim, len(g.targets)
        a_cat = torch.cat([self._EA(self.work, g, t)[e0:e0 + G] for t in g.targets], dim=1)
        h = ctx.stash.pop(("lora_gh", ctx.layer, op.attrs.get("fwd_out")), None)
        kernels = self.use_kernels and x.dtype == torch.bfloat16 and a_cat.dtype == torch.bfloat16 and dy.dtype == torch.bfloat16
        if kernels:
            if h is None:
                h = self._ggemm(x, a_cat, torch.zeros(x.shape[0], T * r, dtype=x.dtype, device=x.device), offsets, 1)
            dh = torch.zeros_like(h)
            for i, t in enumerate(g.targets):
                dys = dy[:, t.row_off:t.row_off + t.rows].contiguous()
                ht = h[:, i * r:(i + 1) * r].contiguous()
                dh_t = self._ggemm(dys, self._EB(self.work, g, t)[e0:e0 + G], torch.zeros(x.shape[0], r, dtype=x.dtype, device=x.device), offsets, 1,
                                   b_mn=True, alpha=self.scaling)                                    # s * dy_slice . B_e
                dh[:, i * r:(i + 1) * r] = dh_t
                self._ggemm(dys, ht, self._EB(self.grad, g, t)[e0:e0 + G], offsets, 2, b_mn=True, accumulate=True, alpha=self.scaling)   # dB_e += s dy^T h
                self._ggemm(dh_t, x, self._EA(self.grad, g, t)[e0:e0 + G], offsets, 2, b_mn=True, accumulate=True)                        # dA_e += dh^T x
            return self._ggemm(dh, a_cat, torch.zeros_like(x), offsets, 1, b_mn=True)
        off = offsets.tolist()
        dx = torch.zeros_like(x)
        for e in range(G):
            s0, s1 = off[e], off[e + 1]
            if s1 <= s0:
                continue
            xe = x[s0:s1]
            he = h[s0:s1] if h is not None else xe @ a_cat[e].to(x.dtype).t()
            dhe = torch.zeros_like(he)
            for i, t in enumerate(g.targets):
                dys = dy[s0:s1, t.row_off:t.row_off + t.rows]
                Be = self._EB(self.work, g, t)[e0 + e].to(dy.dtype)
                dhe[:, i * r:(i + 1) * r] = (dys @ Be) * self.scaling
                self._EB(self.grad, g, t)[e0 + e] += ((dys.t() @ he[:, i * r:(i + 1) * r]) * self.scaling).float()
                self._EA(self.grad, g, t)[e0 + e] += (dhe[:, i * r:(i + 1) * r].t() @ xe).float()
            dx[s0:s1] = dhe @ a_cat[e].to(x.dtype)
        return dx

    def _acc(self, off: int, g: torch.Tensor) -> None:
        self.grad[off:off + g.numel()] += g.reshape(-1).float()

    # ------------------------------------------------------------------ step plumbing
    def reduce_grads(self) -> None:
        if self.comm.world > 1:
            self.comm.all_reduce(self.grad, "sum")

    def grad_sumsq(self) -> torch.Tensor:
        return self.grad.pow(2).sum()

    def optimizer_step(self, hp: torch.Tensor, hp_host) -> None:
        lr, b1, b2, eps, wd, bc1, bc2 = hp_host
        if self.opt_state is None:
            self.opt_state = {"m": torch.zeros(self.numel, dtype=torch.float32, device=self.device),
                              "v": torch.zeros(self.numel, dtype=torch.float32, device=self.device)}
        if self.use_kernels:
            from ..ops import ext

            ext().adamw_step(self.master, self.grad, self.opt_state["m"], self.opt_state["v"], None, hp)
        elif float(hp[7]) != 0.0:  # a zero clip scale marks a skipped update (non-finite gradient norm)
            g = self.grad * hp[7]
            m, v = self.opt_state["m"], self.opt_state["v"]
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            p = self.master.float() - lr * (m / bc1) / ((v / bc2).sqrt() + eps)
            self.master.copy_(p.to(self.master.dtype))
        self.grad.zero_()
        self.sync_work()

    # ------------------------------------------------------------------ persistence
    def _hf_key(self, layer: int, target: str, which: str) -> str:
        return f"base_model.model.model.layers.{layer}.{_MODULE_PATH[target]}.lora_{which}.weight"

    def _hf_expert_key(self, layer: int, expert: int, target: str, which: str) -> str:
        return f"base_model.model.model.layers.{layer}.mlp.experts.{expert}.{target}.lora_{which}.weight"

    def adapter_tensors(self) -> Dict[str, torch.Tensor]:
        out = {}
        for g in self.groups.values():
            if g.experts:
                for t in g.targets:
                    A, B = self._EA(self.master, g, t).detach().float().cpu(), self._EB(self.master, g, t).detach().float().cpu()
                    for e in range(g.experts):
                        out[self._hf_expert_key(g.layer, e, t.name, "A")] = A[e].contiguous()
                        out[self._hf_expert_key(g.layer, e, t.name, "B")] = B[e].contiguous()
                continue
            for t in g.targets:
                out[self._hf_key(g.layer, t.name, "A")] = self._A(self.master, g, t).detach().float().cpu().contiguous()
                out[self._hf_key(g.layer, t.name, "B")] = self._B(self.master, t).detach().float().cpu().contiguous()
        return out

    def named_grads(self):
        """(PEFT key, gradient view) of every adapter matrix, over the flat fp32 gradient buffer (for debugging tools)."""
        for g in self.groups.values():
            for t in g.targets:
                if g.experts:
                    yield f"base_model.model.model.layers.{g.layer}.mlp.experts.*.{t.name}.lora_A.weight", self._EA(self.grad, g, t)
                    yield f"base_model.model.model.layers.{g.layer}.mlp.experts.*.{t.name}.lora_B.weight", self._EB(self.grad, g, t)
                else:
                    yield self._hf_key(g.layer, t.name, "A"), self._A(self.grad, g, t)
                    yield self._hf_key(g.layer, t.name, "B"), self._B(self.grad, t)

    def export_peft(self, out_dir: str, base_model: str = "", write: bool = True) -> None:
        if not write:
            return
        from safetensors.torch import save_file

        os.makedirs(out_dir, exist_ok=True)
        save_file(self.adapter_tensors(), os.path.join(out_dir, "adapter_model.safetensors"), metadata={"format": "pt"})
        cfg = {"peft_type": "LORA", "task_type": "CAUSAL_LM", "base_model_name_or_path": base_model, "r": self.rank_dim,
               "lora_alpha": self.alpha, "lora_dropout": self.dropout, "target_modules": sorted({t.name for g in self.groups.values() for t in g.targets}),
               "bias": "none", "use_rslora": self.rslora, "fan_in_fan_out": False, "inference_mode": True, "modules_to_save": None,
               "init_lora_weights": True}
        with open(os.path.join(out_dir, "adapter_config.json"), "w") as f:
            json.dump(cfg, f, indent=1)

    def load_peft(self, path: str) -> None:
        from safetensors import safe_open

        fn = os.path.join(path, "adapter_model.safetensors") if os.path.isdir(path) else path
        with safe_open(fn, framework="pt") as f:
            keys = set(f.keys())
            for g in self.groups.values():
                if g.experts:
                    for t in g.targets:
                        for e in range(g.experts):
                            ka, kb = self._hf_expert_key(g.layer, e, t.name, "A"), self._hf_expert_key(g.layer, e, t.name, "B")
                            if ka in keys:
                                self._EA(self.master, g, t)[e].copy_(f.get_tensor(ka).to(self.master.dtype))
                            if kb in keys:
                                self._EB(self.master, g, t)[e].copy_(f.get_tensor(kb).to(self.master.dtype))
                    continue
                for t in g.targets:
                    ka, kb = self._hf_key(g.layer, t.name, "A"), self._hf_key(g.layer, t.name, "B")
                    if ka in keys:
                        self._A(self.master, g, t).copy_(f.get_tensor(ka).to(self.master.dtype))
                    if kb in keys:
                        self._B(self.master, t).copy_(f.get_tensor(kb).to(self.master.dtype))
        self.sync_work()

    def save_state(self, d: str, rank: int) -> None:
        if rank != 0:
            return
        from safetensors.torch import save_file

        save_file(self.adapter_tensors(), os.path.join(d, "adapter_model.safetensors"))
        if self.opt_state is not None:
            save_file({k: v.cpu() for k, v in self.opt_state.items()}, os.path.join(d, "lora.adam.safetensors"))

    def load_state(self, d: str, rank: int) -> None:
        self.load_peft(d)
        fn = os.path.join(d, "lora.adam.safetensors")
        if os.path.exists(fn):
            from safetensors import safe_open

            with safe_open(fn, framework="pt") as f:
                self.opt_state = {k: f.get_tensor(k).to(self.device) for k in f.keys()}

    def merge_into(self, store) -> None:
        """W += s * B A for every adapted slice (writes the store's master shards)."""
        for g in self.groups.values():
            name = f"blocks.{g.layer}.{g.param}"
            w = store.full_tensor(name).float().clone()
            for t in g.targets:
                if g.experts:   # [E, rows, r] x [E, r, K]
                    w[:, t.row_off:t.row_off + t.rows] += self.scaling * torch.bmm(self._EB(self.master, g, t).float(), self._EA(self.master, g, t).float())
                    continue
                w[t.row_off:t.row_off + t.rows] += self.scaling * (self._B(self.master, t).float() @ self._A(self.master, g, t).float())
            store.load_tensor(name, w.cpu())
        store.sync_work_from_master()
