"""Rollout transports between the orchestrator (producer) and the trainer ranks (consumers)."""
from .filesystem import FilesystemTransport  # noqa: F401


def make_transport(kind: str, **kw):
    if kind == "filesystem":
        return FilesystemTransport(kw["directory"])
    if kind == "zmq":
        from .zmq import ZmqTransport

        return ZmqTransport(kw["endpoint"], role=kw.get("role", "consumer"))
    raise ValueError(f"unknown transport '{kind}' (filesystem | zmq)")
