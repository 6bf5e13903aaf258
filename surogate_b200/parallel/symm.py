"""Symmetric-memory data plane: peer-addressable buffers and the fused collective kernels that use them.

``maybe_enable`` switches a parameter store from library collectives to the hand-written peer-memory
kernels when symmetric memory can be set up on this node; it returns False (leaving NCCL in place) otherwise.
"""
from __future__ import annotations


def maybe_enable(store, comm, required: bool = False) -> bool:
    try:
        from .symm_comm import SymmComm

        sc = SymmComm.create(comm, store.device)
    except Exception as e:  # noqa: BLE001
        if required:
            raise
        return False
    if sc is None:
        if required:
            raise RuntimeError("symmetric memory is not available on this node")
        return False
    store.comm = sc
    return True
