"""Knowledge distillation from teacher top-K log-probabilities stored in ``.kd`` sidecar files."""
from .sidecar import KD_MAGIC, SidecarReader, SidecarWriter  # noqa: F401
