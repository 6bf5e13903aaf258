"""Publishing updated policy weights from the trainer to the inference engine.

* ``filesystem`` — rank 0 writes the adapter (LoRA) or the full HF model to ``<dir>/v<version>/`` and then a ``LATEST``
  marker; the inference server polls the marker and (re)loads.  Old versions are pruned.
* ``nccl`` — trainer rank 0 and the inference workers share a second process group; tensors are broadcast one by one
  (name list first), so no file I/O is involved.
* ``colocate`` — trainer and inference engine share the GPU: tensors are handed over as CUDA IPC handles through a
  multiprocessing queue, the engine maps them and copies into its own weights.

Parity: surogate/grpo/weight_broadcast.py, colocate.py.
"""
from __future__ import annotations

import json
import os
import shutil
import time
from typing import Dict, Iterable, Optional, Tuple

import torch


class FilesystemBroadcast:
    def __init__(self, directory: str, keep: int = 2, noise=None, total_steps: int = 0):
        """``noise``: a ``grpo.noise.NoiseConfig``; with it every published version carries exploration noise on its normalisation
        weights (full models) or at least the sigma in force (adapters), following the schedule over ``total_steps`` versions."""
        self.dir, self.keep, self.noise, self.total_steps = directory, keep, noise, total_steps
        os.makedirs(directory, exist_ok=True)

    def publish(self, trainer, version: int, hf_config: Optional[Dict] = None) -> str:
        out = os.path.join(self.dir, f"v{version:06d}")
        if trainer.rank == 0:
            os.makedirs(out, exist_ok=True)
        if trainer.lora is not None:
            trainer.export_adapter(out)
        else:
            trainer.export_model(out, hf_config)
        if trainer.rank == 0 and self.noise is not None and self.noise.enabled:
            from .noise import add_noise_to_directory, sigma_at

            add_noise_to_directory(out, sigma_at(version, self.total_steps, self.noise), seed=self.noise.seed + version)
        if trainer.rank == 0:
            with open(os.path.join(self.dir, "LATEST.tmp"), "w") as f:
                json.dump({"version": version, "path": out, "time": time.time(), "kind": "adapter" if trainer.lora is not None else "model"}, f)
            os.replace(os.path.join(self.dir, "LATEST.tmp"), os.path.join(self.dir, "LATEST"))
            old = sorted(d for d in os.listdir(self.dir) if d.startswith("v") and d[1:].isdigit())
            for d in old[:-self.keep]:
                shutil.rmtree(os.path.join(self.dir, d), ignore_errors=True)
        return out

    def latest(self) -> Optional[Dict]:
        try:
            with open(os.path.join(self.dir, "LATEST")) as f:
                return json.load(f)
        except (FileNotFoundError, json.JSONDecodeError):
            return None

    def wait_for(self, version: int, timeout_s: float = 3600.0, poll_s: float = 0.1) -> Dict:
        t0 = time.time()
        while True:
            cur = self.latest()
            if cur is not None and cur["version"] >= version:
                return cur
            if time.time() - t0 > timeout_s:
                raise TimeoutError(f"policy version {version} was not published within {timeout_s}s")
            time.sleep(poll_s)


class NCCLBroadcast:
    """Sender side lives in trainer rank 0; receivers call ``receive`` with the same group."""

    def __init__(self, group, src: int = 0):
        self.group, self.src = group, src

    def publish_tensors(self, named: Iterable[Tuple[str, torch.Tensor]], version: int) -> None:
        import torch.distributed as dist

        named = list(named)
        header = [{"name": n, "shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", "")} for n, t in named]
        dist.broadcast_object_list([{"version": version, "tensors": header}], src=self.src, group=self.group)
        for _, t in named:
            dist.broadcast(t.contiguous(), src=self.src, group=self.group)

    def receive(self, device) -> Tuple[int, Dict[str, torch.Tensor]]:
        import torch.distributed as dist

        box = [None]
        dist.broadcast_object_list(box, src=self.src, group=self.group)
        out = {}
        for h in box[0]["tensors"]:
            t = torch.empty(h["shape"], dtype=getattr(torch, h["dtype"]), device=device)
            dist.broadcast(t, src=self.src, group=self.group)
            out[h["name"]] = t
        return box[0]["version"], out


class ColocateBroadcast:
    """Same-GPU hand-over through CUDA IPC handles (torch.multiprocessing's tensor reductions) on a queue."""

    def __init__(self, queue):
        self.queue = queue

    def publish_tensors(self, named: Iterable[Tuple[str, torch.Tensor]], version: int) -> None:
        from torch.multiprocessing.reductions import reduce_tensor

        handles = {n: reduce_tensor(t.detach()) for n, t in named}
        self.queue.put({"version": version, "handles": handles})

    def receive(self, timeout_s: float = 600.0) -> Tuple[int, Dict[str, torch.Tensor]]:
        msg = self.queue.get(timeout=timeout_s)
        tensors = {n: fn(*args) for n, (fn, args) in msg["handles"].items()}
        return msg["version"], tensors
