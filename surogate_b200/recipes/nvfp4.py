"""NVFP4 recipe: E2M1 values, one UE4M3 scale per 16 elements of the contraction, one fp32 scale per tensor.

Per dense projection (qkv, out, mlp_up, mlp_down) all three GEMMs run on the block-scaled tcgen05 kernel:

Round-to-nearest operands use four-over-six block scaling (``fp4_four_over_six``, on by default): each block of 16 is quantised with
its abs-max mapped to 6 and to 4 and the better reconstruction is kept (tensor encode factor 1536; arXiv 2512.02010).

* forward : x (row-wise blocks along K, round-to-nearest) . W (16x16 blocks) ^T
* dgrad   : dy (blocks along N, stochastic rounding) . W^T (the transposed quantisation of the same 16x16 blocks)
* wgrad   : dy^T . x^T with both operands passed through the same 16x16 random Hadamard transform along the token
            dimension before quantisation (dy with stochastic rounding), which spreads outliers without changing
            the product.

Weights are quantised once per optimizer step (both orientations, cached); activations and gradients just in time
from an abs-max pass.  The expert projections of MoE layers run as grouped FP8 GEMMs (E4M3 forward, E5M2 gradients, per-tensor
current scaling; ``recipes/grouped_fp8.py``): their rows arrive grouped by expert with device-side offsets, which the FP8 grouped
kernel schedules directly.  The LM head and the router stay in bf16.  Shapes whose contraction is not a multiple of 256 fall
back to bf16.

Parity: csrc/src/recipes/nvfp4/nvfp4_recipe.cpp:629-1131, recipes/nvfp4/kernels/*.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from .base import Recipe
from .grouped_fp8 import GroupedFp8Mixin

QUANT_ROLES = ("qkv", "out", "mlp_up", "mlp_down")
ENCODE = 2688.0          # 448 * 6: tensor encode factor of plain NVFP4
ENCODE_4O6 = 1536.0      # 256 * 6 = 384 * 4: with four-over-six both block-scale choices stay inside UE4M3
HADAMARD_SIGNS = 0b1011001110001101


class Fp4Tensor:
    __slots__ = ("q", "sf", "inv_ge")

    def __init__(self, q, sf, inv_ge):
        self.q, self.sf, self.inv_ge = q, sf, inv_ge


class NVFP4Recipe(GroupedFp8Mixin, Recipe):
    name = "nvfp4"

    def __init__(self, cm, device, skip_first_layers: int = 0, skip_last_layers: int = 0, hadamard: bool = True, stochastic: bool = True,
                 four_over_six: bool = True):
        from ..ops import ext

        self.ext = ext()
        self.device = device
        self.n_layers = cm.n_layers
        self.skip = set(range(skip_first_layers)) | set(range(cm.n_layers - skip_last_layers, cm.n_layers))
        self.hadamard, self.stochastic = hadamard, stochastic
        # round-to-nearest operands (activations and weights in forward, x^T in wgrad) pick, per block of 16, whichever of the two
        # mappings abs-max -> 6 and abs-max -> 4 reconstructs the block better; stochastically rounded gradients keep the plain mapping
        self.four_over_six = bool(four_over_six)
        self.weight_cache: Dict[Tuple[int, str, bool], Fp4Tensor] = {}
        self.expert_weight_cache: Dict[Tuple[int, str], tuple] = {}
        self.step = 0
        self.calls = 0

    def begin_step(self, step: int) -> None:
        self.step = step
        self.calls = 0

    def end_step(self) -> None:
        self.grouped_end_step()

    def on_weights_updated(self, store) -> None:
        self.weight_cache.clear()
        self.expert_weight_cache.clear()

    # ------------------------------------------------------------------ helpers
    def _amax(self, x: torch.Tensor) -> torch.Tensor:
        am = torch.zeros(1, dtype=torch.float32, device=x.device)
        self.ext.amax(x, am)
        return am

    def _seed(self) -> int:
        self.calls += 1
        return (self.step * 7919 + self.calls * 104729) & 0x7FFFFFFF

    def _q_rows(self, x: torch.Tensor, sr: bool = False, block2d: bool = False) -> Fp4Tensor:
        x = x.contiguous()
        am = self._amax(x)
        fos = self.four_over_six and not sr
        q, sf = self.ext.nvfp4_quantize(x, am, sr, self._seed() if sr else 0, block2d, fos)
        return Fp4Tensor(q, sf, am / (ENCODE_4O6 if fos else ENCODE))

    def _q_transpose(self, x: torch.Tensor, sr: bool, rht: bool) -> Fp4Tensor:
        x = x.contiguous()
        am = self._amax(x)
        fos = self.four_over_six and not sr
        q, sf = self.ext.nvfp4_quantize_transpose(x, am, sr, rht, self._seed() if sr else 0, HADAMARD_SIGNS, fos)
        return Fp4Tensor(q, sf, am * (2.0 if rht else 1.0) / (ENCODE_4O6 if fos else ENCODE))

    def _weight(self, ctx, role: str, w: torch.Tensor, transposed: bool) -> Fp4Tensor:
        key = (ctx.layer, role, transposed)
        t = self.weight_cache.get(key)
        if t is None:
            t = self._q_transpose(w, False, False) if transposed else self._q_rows(w, False, block2d=True)
            self.weight_cache[key] = t
        return t

    def _gemm(self, a: Fp4Tensor, b: Fp4Tensor, out=None, accumulate=False, M=None, N=None):
        if out is None:
            out = torch.empty(a.q.shape[0], b.q.shape[0], dtype=torch.bfloat16, device=a.q.device)
        self.ext.gemm_nvfp4(a.q, a.sf, b.q, b.sf, out, accumulate, 1.0, a.inv_ge, b.inv_ge, self.ext.error_flag_tensor())
        return out

    def _active(self, ctx, role: str, w, K: int, Ncontract: int = 256, M: int = 256) -> bool:
        return (ctx.layer is not None and ctx.layer not in self.skip and role in QUANT_ROLES and w.dtype == torch.bfloat16
                and K % 256 == 0 and Ncontract % 256 == 0 and M % 256 == 0 and w.shape[0] % 64 == 0)

    # ------------------------------------------------------------------ GEMMs
    def forward_matmul(self, ctx, op, x, w, bias):
        role = op.attrs.get("role", "")
        K = x.shape[-1]
        if not self._active(ctx, role, w, K):
            return None
        lead = tuple(x.shape[:-1])
        xq = self._q_rows(x.reshape(-1, K))
        y = self._gemm(xq, self._weight(ctx, role, w, False)).reshape(*lead, w.shape[0])
        if bias is not None:
            y += bias
        return y

    def backward_matmul(self, ctx, op, dy2, x2, w):
        role = op.attrs.get("role", "")
        N, K = w.shape
        M = dy2.shape[0]
        if not self._active(ctx, role, w, K, N, M):
            return None
        dyq = self._q_rows(dy2, sr=self.stochastic)
        dx = self._gemm(dyq, self._weight(ctx, role, w, True))              # [M, N] . (W^T [K, N])^T
        tgt, acc = ctx.grad_target(op.outputs[1])
        if tgt is not None:
            a = self._q_transpose(dy2, self.stochastic, self.hadamard)       # dy^T [N, M]
            b = self._q_transpose(x2, False, self.hadamard)                  # x^T  [K, M]
            self._gemm(a, b, tgt, accumulate=acc)
        return dx, None
