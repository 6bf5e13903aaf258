"""Recipe interface.

A recipe decides, per matmul, the precision of the three GEMMs (forward, dgrad,
wgrad) and owns the quantisation state.  Returning ``None`` from a hook means
"use the backend's plain bf16/fp32 path".

Parity: csrc/src/recipes/recipe.h:62-318, recipe_factory.cpp.
"""
from __future__ import annotations


class Recipe:
    name = "base"

    def wants_fp8_activation(self, ctx, op, out_index: int) -> bool:
        return False

    def forward_matmul(self, ctx, op, x, w, bias):
        return None

    def backward_matmul(self, ctx, op, dy2, x2, w):
        return None

    def begin_step(self, step: int) -> None:
        pass

    def end_step(self) -> None:
        pass

    def on_weights_updated(self, store) -> None:
        pass

    def state_dict(self):
        return {}

    def load_state_dict(self, sd) -> None:
        pass


class BF16Recipe(Recipe):
    name = "bf16"


def make_recipe(name: str, cm, device, **kw) -> Recipe:
    name = (name or "bf16").replace("-", "_").lower()
    if name == "bf16" or device.type != "cuda":
        return BF16Recipe()
    if name == "fp8_hybrid":
        from .fp8_hybrid import FP8HybridRecipe

        return FP8HybridRecipe(cm, device, **kw)
    if name == "nvfp4":
        from .nvfp4 import NVFP4Recipe

        return NVFP4Recipe(cm, device, **kw)
    raise ValueError(f"unknown recipe '{name}' (bf16 | fp8_hybrid | nvfp4)")
