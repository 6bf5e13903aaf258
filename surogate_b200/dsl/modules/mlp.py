"""Gated MLP with the up and gate projections fused into one GEMM ([up; gate] rows, up first).

Parity: surogate/dsl/modules/mlp.py:19-225 (GenericMLP).
"""
from __future__ import annotations

from dataclasses import dataclass

from .. import functional as F
from .. import hf
from ..nn import Module


@dataclass
class MLPConfig:
    activation: str = "swiglu"
    tile_rows: int = 0  # > 0: evaluate the MLP over row tiles of this many tokens and recompute each tile in backward (long context)


class GenericMLP(Module):
    def __init__(self, d_model: int, d_ff: int, config: MLPConfig | None = None, prefix: str = "model.layers.{L}.mlp",
                 names: tuple = ("up_proj", "gate_proj", "down_proj")):
        super().__init__()
        self.cfg = config or MLPConfig()
        m = prefix
        up_n, gate_n, down_n = names  # checkpoint leaf names of the up / gate / down projections
        self.declare_param("up_weight", (2 * d_ff, d_model), quantizable=True,
                           hf=hf.fuse([f"{m}.{up_n}.weight", f"{m}.{gate_n}.weight"], sizes=[d_ff, d_ff]),
                           lora_targets=[("up_proj", 0, d_ff), ("gate_proj", d_ff, d_ff)])
        self.declare_param("down_weight", (d_model, d_ff), quantizable=True, hf=hf.direct(f"{m}.{down_n}.weight"),
                           lora_targets=[("down_proj", 0, d_model)])

    def forward(self, x):
        if self.cfg.tile_rows > 0:
            return F.tiled_mlp(x, self.p("up_weight"), self.p("down_weight"), self.cfg.tile_rows)
        up = F.matmul(x, self.p("up_weight"), name="mlp_up", role="mlp_up")
        if self.cfg.activation == "geglu":  # gelu(gate) * up with the tanh approximation (Gemma family)
            act = F.torch_fn("geglu", [up], [("geglu", up.shape[:-1] + (up.shape[-1] // 2,), "act")], approximate="tanh")
        else:
            act = F.swiglu(up)
        return F.matmul(act, self.p("down_weight"), name="mlp_down", role="mlp_down")
