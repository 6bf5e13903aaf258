"""Launcher of the rollout engine (``surogate grpo-infer``): a vLLM OpenAI server with LoRA hot-swapping, plus the
watcher that loads each newly published policy version into it.

The server is an external process (``python -m vllm.entrypoints.openai.api_server``); nothing from vLLM runs inside the
trainer.  When vLLM is not installed the launcher raises with the command it would have run.

Parity: surogate/grpo/inference/vllm/* (server + worker patches), surogate/grpo/split.py (split-GPU runner).
"""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys
import time
import urllib.request
from typing import List, Optional

from .config import InferenceConfig
from .weight_broadcast import FilesystemBroadcast


def server_command(cfg: InferenceConfig) -> List[str]:
    frac = os.environ.get("SUROGATE_ENGINE_MEMORY_FRACTION")   # set by the colocate runner: the trainer shares these GPUs
    if frac:
        cfg.gpu_memory_utilization = min(cfg.gpu_memory_utilization, float(frac))
    cmd = [sys.executable, "-m", "vllm.entrypoints.openai.api_server", "--model", cfg.model, "--host", cfg.host, "--port", str(cfg.port),
           "--tensor-parallel-size", str(cfg.tensor_parallel_size), "--gpu-memory-utilization", str(cfg.gpu_memory_utilization)]
    if cfg.data_parallel_size > 1:
        cmd += ["--data-parallel-size", str(cfg.data_parallel_size)]
    if cfg.api_server_count > 1:
        cmd += ["--api-server-count", str(cfg.api_server_count)]
    if cfg.dtype and cfg.dtype != "auto":
        cmd += ["--dtype", cfg.dtype]
    # valued options: passed only when set, so the engine keeps its own defaults otherwise
    for flag, value in (("--max-model-len", cfg.max_model_len), ("--max-num-seqs", cfg.max_num_seqs), ("--kv-cache-dtype", cfg.kv_cache_dtype),
                        ("--attention-backend", cfg.attention_backend), ("--reasoning-parser", cfg.reasoning_parser), ("--all2all-backend", cfg.all2all_backend)):
        if value:
            cmd += [flag, str(value)]
    if cfg.rope_scaling:
        cmd += ["--rope-scaling", cfg.rope_scaling if isinstance(cfg.rope_scaling, str) else json.dumps(cfg.rope_scaling)]
    if cfg.seed:
        cmd += ["--seed", str(cfg.seed)]
    for flag, on in (("--enforce-eager", cfg.enforce_eager), ("--trust-remote-code", cfg.trust_remote_code), ("--enable-expert-parallel", cfg.enable_expert_parallel),
                     ("--enable-eplb", cfg.enable_eplb)):
        if on:
            cmd.append(flag)
    if cfg.enable_auto_tool_choice:
        cmd += ["--enable-auto-tool-choice"] + (["--tool-call-parser", cfg.tool_call_parser] if cfg.tool_call_parser else [])
    if cfg.enable_prefix_caching is not None:
        cmd.append("--enable-prefix-caching" if cfg.enable_prefix_caching else "--no-enable-prefix-caching")
    if cfg.enable_lora:
        cmd += ["--enable-lora", "--max-loras", str(cfg.max_loras), "--max-cpu-loras", str(cfg.max_cpu_loras)]
        if cfg.max_lora_rank is not None:
            cmd += ["--max-lora-rank", str(cfg.max_lora_rank)]
    from .vllm_worker import WORKER_EXTENSIONS

    ext = WORKER_EXTENSIONS.get(getattr(cfg, "weight_broadcast", "filesystem"))
    if ext:   # the workers gain update_weights_from_path / receive_weights / receive_ipc_handles, callable through collective_rpc
        cmd += ["--worker-extension-cls", ext]
    return cmd + list(cfg.extra_args)


def launch_server(cfg: InferenceConfig, gpus: Optional[str] = None) -> subprocess.Popen:
    try:
        import vllm  # noqa: F401
    except ImportError as e:
        raise RuntimeError("vLLM is not installed; the rollout server command would be: " + " ".join(server_command(cfg))) from e
    env = dict(os.environ, VLLM_ALLOW_RUNTIME_LORA_UPDATING="True")
    if gpus is not None:
        env["CUDA_VISIBLE_DEVICES"] = gpus
    return subprocess.Popen(server_command(cfg), env=env)


def load_adapter(base_url: str, name: str, path: str, timeout_s: float = 120.0) -> None:
    """vLLM's runtime LoRA endpoint: unload the previous adapter of that name (ignored if absent), load the new one."""
    root = base_url.rstrip("/").rsplit("/v1", 1)[0]
    for route, body in (("/v1/unload_lora_adapter", {"lora_name": name}), ("/v1/load_lora_adapter", {"lora_name": name, "lora_path": path})):
        req = urllib.request.Request(root + route, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
        try:
            urllib.request.urlopen(req, timeout=timeout_s).read()
        except Exception:  # noqa: BLE001
            if route.endswith("load_lora_adapter") and "unload" not in route:
                raise


def watch_and_reload(cfg: InferenceConfig, base_url: str, adapter_name: str = "policy", poll_s: float = 0.5, stop_after: Optional[int] = None) -> int:
    """Poll the weight directory; push every new adapter version into the running server.  Returns the last version loaded."""
    b = FilesystemBroadcast(cfg.weight_dir)
    seen = -1
    while stop_after is None or seen < stop_after:
        cur = b.latest()
        if cur is not None and cur["version"] > seen and cur.get("kind") == "adapter":
            load_adapter(base_url, adapter_name, cur["path"])
            seen = cur["version"]
        time.sleep(poll_s)
    return seen
