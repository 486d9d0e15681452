"""Device inventory for `describe` / `--list-devices` (reference: src/v2/app/commands/DescribeCommand.cpp,
src/v2/backends/DeviceRegistry.cpp).  Read-only: nothing here changes a GPU setting."""
from __future__ import annotations

import os
import platform


def describe_devices() -> dict:
    import torch
    out = {"host": platform.node(), "cpu": {"logical_cores": os.cpu_count(), "machine": platform.machine()}, "gpus": []}
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            free, total = torch.cuda.mem_get_info(i)
            out["gpus"].append({"id": f"cuda:{i}", "name": p.name, "sm": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                                "memory_total_gb": round(total / 1e9, 1), "memory_free_gb": round(free / 1e9, 1),
                                "peer_access": [j for j in range(torch.cuda.device_count())
                                                if j != i and torch.cuda.can_device_access_peer(i, j)]})
        try:
            import pynvml
            pynvml.nvmlInit()
            for i, g in enumerate(out["gpus"]):
                h = pynvml.nvmlDeviceGetHandleByIndex(i)
                g["clocks_sm_mhz"] = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
                g["clocks_sm_max_mhz"] = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
                g["power_limit_w"] = pynvml.nvmlDeviceGetEnforcedPowerLimit(h) / 1000.0
        except Exception:
            pass
    try:                                            # is the compiled extension in place for the sources of this checkout?
        from ..ops import build as ops_build
        out["extension"] = {"path": str(ops_build.so_path()), "built_for_these_sources": bool(ops_build.is_built()),
                            "arch": "sm_100a"}
    except Exception as exc:
        out["extension"] = {"error": f"{type(exc).__name__}: {exc}"}
    return out
