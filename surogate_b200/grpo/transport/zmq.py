"""ZeroMQ transport (PUSH/PULL): lower latency than the filesystem when orchestrator and trainer share a network.

The producer binds, rank 0 of the trainer connects and re-broadcasts to the other ranks through the training
communicator.  Messages are ``[json header, npz bytes]``.  Needs ``pyzmq``; importing this module without it raises.

Parity: surogate/grpo/transport/zmq.py.
"""
from __future__ import annotations

import io
import json
from typing import Dict, Optional

import numpy as np

try:
    import zmq  # type: ignore
except ImportError as e:  # pragma: no cover - optional dependency
    raise ImportError("the zmq transport needs the `pyzmq` package; use transport: filesystem") from e


class ZmqTransport:
    def __init__(self, endpoint: str, role: str = "consumer", hwm: int = 8):
        self.ctx = zmq.Context.instance()
        if role == "producer":
            self.sock = self.ctx.socket(zmq.PUSH)
            self.sock.set_hwm(hwm)
            self.sock.bind(endpoint)
        else:
            self.sock = self.ctx.socket(zmq.PULL)
            self.sock.set_hwm(hwm)
            self.sock.connect(endpoint)
        self.pending: Dict[int, tuple] = {}

    def send(self, step: int, arrays: Dict[str, np.ndarray], meta: Optional[Dict] = None):
        buf = io.BytesIO()
        np.savez(buf, **arrays)
        self.sock.send_multipart([json.dumps({"step": step, "meta": meta or {}}).encode(), buf.getvalue()])

    def receive(self, step: int, timeout_s: float = 3600.0, poll_s: float = 0.05):
        while step not in self.pending:
            if not self.sock.poll(int(timeout_s * 1000)):
                raise TimeoutError(f"no rollout batch for step {step} within {timeout_s}s")
            head, body = self.sock.recv_multipart()
            h = json.loads(head.decode())
            with np.load(io.BytesIO(body)) as z:
                self.pending[h["step"]] = ({k: z[k] for k in z.files}, h["meta"])
        return self.pending.pop(step)

    def ack(self, step: int) -> None:
        pass

    def cleanup(self, keep_from: int) -> None:
        pass
