"""System diagnostics printed at start-up and by ``surogate info``.

Parity: surogate/utils/system_info.py, csrc/src/utilities/system_info.cpp.
"""
from __future__ import annotations

import os
import platform
from typing import Any, Dict


def system_info() -> Dict[str, Any]:
    import torch

    info: Dict[str, Any] = {"python": platform.python_version(), "platform": platform.platform(), "torch": torch.__version__,
                            "cuda_runtime": torch.version.cuda, "cpu_count": os.cpu_count()}
    try:
        import psutil

        vm = psutil.virtual_memory()
        info["host_memory_gb"] = round(vm.total / 2 ** 30, 1)
    except Exception:  # noqa: BLE001
        pass
    gpus = []
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            gpus.append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "memory_gb": round(p.total_memory / 2 ** 30, 1), "sms": p.multi_processor_count})
    info["gpus"] = gpus
    try:
        from ..ops import host

        t = host().query_gpu(0)
        if t["ok"]:
            info["gpu0_telemetry"] = {k: t[k] for k in ("sm_clock_mhz", "sm_clock_max_mhz", "power_w", "power_limit_w", "temperature_c")}
    except Exception:  # noqa: BLE001
        pass
    from ..ops import _build

    info["cuda_extension_built"] = os.path.exists(_build._so_path())
    info["host_extension_built"] = os.path.exists(_build._host_so())
    try:
        import torch.distributed as dist

        info["nccl"] = ".".join(map(str, torch.cuda.nccl.version())) if dist.is_nccl_available() else None
    except Exception:  # noqa: BLE001
        info["nccl"] = None
    return info
