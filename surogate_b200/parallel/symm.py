"""Symmetric-memory data plane: peer-addressable buffers and the fused collective kernels that use them.

``try_create`` wraps a library communicator into a :class:`~surogate_b200.parallel.symm_comm.SymmComm` when
symmetric memory can be set up on this node (one NVSwitch/NVLink domain, 2..8 ranks); otherwise it returns the
communicator unchanged, leaving NCCL as the data plane.
"""
from __future__ import annotations


def try_create(comm, device, required: bool = False):
    try:
        from .symm_comm import SymmComm

        sc = SymmComm.create(comm, device)
    except Exception:  # noqa: BLE001
        if required:
            raise
        return comm
    if sc is None:
        if required:
            raise RuntimeError("symmetric memory is not available for this communicator")
        return comm
    return sc
