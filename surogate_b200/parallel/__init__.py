"""Multi-GPU plumbing: process groups, collectives, symmetric memory, expert parallelism."""
from .dist import TorchComm, init_distributed, DistInfo

__all__ = ["TorchComm", "init_distributed", "DistInfo"]
