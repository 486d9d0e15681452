"""Device inventory for `describe` / `--list-devices` (reference: src/v2/app/commands/DescribeCommand.cpp,
src/v2/backends/DeviceRegistry.cpp) and the device micro-benchmarks behind `describe --device-benchmark` (bandwidth, matrix
throughput, peer-to-peer; reference: src/v2/backends/benchmarks/CUDABenchmark.cu).  Read-only: nothing here changes a GPU
setting."""
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


def _timed(fn, device, reps: int) -> float:
    """Seconds per call of ``fn`` after one warm-up call: CUDA events on a GPU, the wall clock on the CPU."""
    import time

    import torch
    fn()
    if device.type == "cuda":
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.device(device):
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
        torch.cuda.synchronize(device)
        return e0.elapsed_time(e1) / 1e3 / reps
    t0 = time.perf_counter()
    for _ in range(reps):
        fn()
    return (time.perf_counter() - t0) / reps


def benchmark_device(device, copy_bytes: int = 1 << 30, gemm_n: int = 8192, reps: int = 10) -> dict:
    """Copy bandwidth (read + write of a buffer larger than the L2) and dense bf16 matrix throughput of one device: the two
    denominators every kernel summary of this package is quoted against."""
    import torch
    device = torch.device(device)
    n = copy_bytes // 4
    src = torch.empty(n, dtype=torch.float32, device=device).fill_(1.0)
    dst = torch.empty_like(src)
    t = _timed(lambda: dst.copy_(src), device, reps)
    dt = torch.bfloat16 if device.type == "cuda" else torch.float32
    a = torch.randn(gemm_n, gemm_n, device=device, dtype=dt)
    b = torch.randn(gemm_n, gemm_n, device=device, dtype=dt)
    tg = _timed(lambda: torch.matmul(a, b), device, reps)
    return {"device": str(device), "copy_gbs": round(2 * n * 4 / t / 1e9, 1), "copy_bytes": n * 4,
            "matmul_tflops": round(2 * gemm_n ** 3 / tg / 1e12, 2), "matmul_dtype": str(dt).replace("torch.", ""), "matmul_n": gemm_n}


def benchmark_devices(copy_bytes: int = 1 << 30, gemm_n: int = 8192, p2p_bytes: int = 1 << 28) -> dict:
    """`benchmark_device` for every visible GPU (or the CPU when there is none) and, between every pair of GPUs with peer
    access, the one-directional copy bandwidth of a device-to-device copy."""
    import torch
    if not torch.cuda.is_available():
        return {"devices": [benchmark_device("cpu", copy_bytes=min(copy_bytes, 1 << 26), gemm_n=min(gemm_n, 512), reps=3)], "p2p": []}
    n_dev = torch.cuda.device_count()
    out = {"devices": [benchmark_device(f"cuda:{i}", copy_bytes, gemm_n) for i in range(n_dev)], "p2p": []}
    for i in range(n_dev):
        for j in range(n_dev):
            if i == j or not torch.cuda.can_device_access_peer(i, j):
                continue
            src = torch.empty(p2p_bytes // 4, dtype=torch.float32, device=f"cuda:{i}").fill_(1.0)
            dst = torch.empty(p2p_bytes // 4, dtype=torch.float32, device=f"cuda:{j}")
            t = _timed(lambda: dst.copy_(src), torch.device(f"cuda:{i}"), 10)
            torch.cuda.synchronize(j)
            out["p2p"].append({"from": f"cuda:{i}", "to": f"cuda:{j}", "gbs": round(p2p_bytes / t / 1e9, 1)})
    return out
