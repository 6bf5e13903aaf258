"""GPU telemetry through NVML (read-only: clocks, power, temperature, throttle reasons, PCIe counters).

Nothing here changes a GPU setting.  Parity: csrc/src/utilities/gpu_info*.cpp.
"""
from __future__ import annotations

from typing import Any, Dict


def gpu_info(device=None, nvml=None) -> Dict[str, Any]:
    """``nvml`` may be injected (tests use a fake); defaults to pynvml."""
    try:
        if nvml is None:
            import pynvml as nvml
        nvml.nvmlInit()
        idx = getattr(device, "index", None) or 0
        h = nvml.nvmlDeviceGetHandleByIndex(idx)
        mem = nvml.nvmlDeviceGetMemoryInfo(h)
        util = nvml.nvmlDeviceGetUtilizationRates(h)
        out = {
            "name": nvml.nvmlDeviceGetName(h),
            "clock_sm_mhz": nvml.nvmlDeviceGetClockInfo(h, nvml.NVML_CLOCK_SM),
            "clock_sm_max_mhz": nvml.nvmlDeviceGetMaxClockInfo(h, nvml.NVML_CLOCK_SM),
            "clock_mem_mhz": nvml.nvmlDeviceGetClockInfo(h, nvml.NVML_CLOCK_MEM),
            "power_w": nvml.nvmlDeviceGetPowerUsage(h) / 1000.0,
            "power_limit_w": nvml.nvmlDeviceGetEnforcedPowerLimit(h) / 1000.0,
            "temperature_c": nvml.nvmlDeviceGetTemperature(h, nvml.NVML_TEMPERATURE_GPU),
            "mem_used": mem.used, "mem_total": mem.total, "gpu_util": util.gpu, "mem_util": util.memory,
            "throttle_reasons": int(nvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)),
        }
        try:
            out["pcie_tx_kbs"] = nvml.nvmlDeviceGetPcieThroughput(h, nvml.NVML_PCIE_UTIL_TX_BYTES)
            out["pcie_rx_kbs"] = nvml.nvmlDeviceGetPcieThroughput(h, nvml.NVML_PCIE_UTIL_RX_BYTES)
        except Exception:  # noqa: BLE001
            pass
        return out
    except Exception as e:  # noqa: BLE001
        return {"error": str(e)}
