"""Regression harness: a matrix of (model x recipe x distribution x storage) cases, run and compared as JSON artifacts."""
from .runner import Case, compare, default_matrix, run_case  # noqa: F401
