"""Precision recipes: who quantises what, and which GEMM runs.  Parity: csrc/src/recipes/recipe.h:62-318."""
from .base import Recipe, BF16Recipe, make_recipe
from .fp8_hybrid import FP8HybridRecipe

__all__ = ["Recipe", "BF16Recipe", "FP8HybridRecipe", "make_recipe"]
