"""Worker-side weight receivers for the rollout engine (vLLM ``--worker-extension-cls``).

vLLM instantiates every worker with the mix-in named by ``worker_extension_cls`` and lets the server call its methods on all workers
with ``collective_rpc``.  The three receivers correspond to the trainer's three ways of publishing weights
(``grpo/weight_broadcast.py``):

``FilesystemWeightReceiver``   ``update_weights_from_path(path)``: read the safetensors files of a published version and hand the
                               tensors to the model's own ``load_weights`` (which knows vLLM's fused / sharded parameter layout).
``NCCLWeightReceiver``         ``init_weight_group(host, port, world, rank)`` once, then ``receive_weights()`` per version: tensors
                               arrive by broadcast from trainer rank 0 over a process group of their own (no file I/O).
``ColocateWeightReceiver``     ``receive_ipc_handles(payload)``: the trainer shares the GPU; tensors arrive as CUDA IPC handles,
                               are mapped and copied into the engine's weights.

Nothing here imports vLLM: the classes only rely on the attributes vLLM's GPU worker has (``self.model_runner.model`` with
``load_weights(weights=iterable of (name, tensor))``, ``self.device``), so they are tested against a stand-in worker.

Parity: surogate/grpo/inference/vllm/worker/{filesystem,nccl,colocate}.py, surogate/grpo/orchestrator/patches.py.
"""
from __future__ import annotations

import os
from typing import Any, Dict, Iterable, Iterator, List, Optional, Tuple

import torch

WORKER_EXTENSIONS = {
    "filesystem": "surogate_b200.grpo.vllm_worker.FilesystemWeightReceiver",
    "nccl": "surogate_b200.grpo.vllm_worker.NCCLWeightReceiver",
    "colocate": "surogate_b200.grpo.vllm_worker.ColocateWeightReceiver",
}


def _model_of(worker):
    runner = getattr(worker, "model_runner", None)
    model = getattr(runner, "model", None)
    if model is None or not hasattr(model, "load_weights"):
        raise RuntimeError("this worker has no model_runner.model.load_weights: not a vLLM GPU worker?")
    return model


def _load(worker, named: Iterable[Tuple[str, torch.Tensor]]) -> int:
    model = _model_of(worker)
    count = {"n": 0}

    def counted() -> Iterator[Tuple[str, torch.Tensor]]:
        for name, t in named:
            count["n"] += 1
            yield name, t

    model.load_weights(weights=counted())
    return count["n"]


class FilesystemWeightReceiver:
    def update_weights_from_path(self, path: str) -> Dict[str, Any]:
        from safetensors import safe_open

        files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
        if not files:
            raise FileNotFoundError(f"no safetensors files under {path}")

        def stream():
            for fn in files:
                with safe_open(os.path.join(path, fn), framework="pt", device=str(getattr(self, "device", "cpu"))) as f:
                    for k in f.keys():
                        yield k, f.get_tensor(k)

        n = _load(self, stream())
        sigma = None
        try:
            from .noise import read_sigma

            sigma = (read_sigma(path) or {}).get("sigma")
        except Exception:  # noqa: BLE001
            pass
        self._weights_version = getattr(self, "_weights_version", 0) + 1
        return {"tensors": n, "version": self._weights_version, "noise_sigma": sigma}


class NCCLWeightReceiver:
    def init_weight_group(self, host: str, port: int, world_size: int, rank: int, backend: Optional[str] = None) -> bool:
        """A process group of its own (trainer rank 0 = rank 0, engine workers = 1 ..), separate from the engine's tensor-parallel
        group and from the trainer's training group."""
        import torch.distributed as dist
        from torch.distributed import TCPStore

        backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        store = TCPStore(host, port, world_size, is_master=(rank == 0), wait_for_workers=False)
        # a second default group cannot exist in one process: build the group object directly on the store
        pg_cls = dist.ProcessGroupNCCL if backend == "nccl" else dist.ProcessGroupGloo
        self._weight_group = pg_cls(dist.PrefixStore("surogate_weights", store), rank, world_size)
        self._weight_rank, self._weight_world = rank, world_size
        return True

    def receive_weights(self, header: List[Dict[str, Any]]) -> Dict[str, Any]:
        """``header``: [{name, shape, dtype}] in the order trainer rank 0 broadcasts the tensors."""
        g = self._weight_group
        dev = getattr(self, "device", "cpu")

        def stream():
            for h in header:
                t = torch.empty(h["shape"], dtype=getattr(torch, h["dtype"]), device=dev)
                g.broadcast([t], _bcast_opts(0)).wait()
                yield h["name"], t

        return {"tensors": _load(self, stream())}


def _bcast_opts(root: int):
    import torch.distributed as dist

    o = dist.BroadcastOptions()
    o.rootRank, o.rootTensor = root, 0
    return o


class ColocateWeightReceiver:
    def receive_ipc_handles(self, payload: Dict[str, Any]) -> Dict[str, Any]:
        """``payload`` = {"version": v, "handles": {name: (rebuild_fn, args)}} as produced by ``ColocateBroadcast.publish_tensors``."""
        tensors = ((n, fn(*args)) for n, (fn, args) in payload["handles"].items())
        return {"tensors": _load(self, tensors), "version": payload.get("version")}
