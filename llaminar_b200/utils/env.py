"""Central registry of the LLAMINAR_* environment switches.

Every switch is declared once here with its type, default and meaning; the rest of the package asks
`debug_env()` and never reads `os.environ` for a LLAMINAR_* name itself (a unit test greps for that, as the
reference does with its static check; reference: src/v2/utils/DebugEnv.h, scripts/check_no_direct_getenv.sh).
"""
from __future__ import annotations

import os
from dataclasses import dataclass


@dataclass(frozen=True)
class EnvVar:
    name: str
    kind: type
    default: object
    help: str


REGISTRY: tuple[EnvVar, ...] = (
    EnvVar("LLAMINAR_LOG_LEVEL", str, "INFO", "log level of the package logger"),
    EnvVar("LLAMINAR_PROFILING", bool, False, "time engine phases and kernels categories with CUDA events"),
    EnvVar("LLAMINAR_PERF_STATS_JSON", str, "", "write the perf-stats records as JSON to this path at exit"),
    EnvVar("LLAMINAR_PERF_STATS_CSV", str, "", "write the perf-stats records as CSV to this path at exit"),
    EnvVar("LLAMINAR_PERF_STATS_TABLE", bool, False, "print the perf-stats table at exit"),
    EnvVar("LLAMINAR_PERF_STATS_FILTER", str, "", "only keep records whose domain/name contains this text"),
    EnvVar("LLAMINAR_TP_FUSED", bool, True, "fuse the row-parallel GEMM with its all-reduce over peer memory"),
    EnvVar("LLAMINAR_ALLREDUCE_PRECISION", str, "auto", "payload of the NCCL tensor-parallel all-reduce: fp32, bf16, fp16 or auto (bf16 for more than 32 rows, fp32 below)"),
    EnvVar("LLAMINAR_PP_PAYLOAD", str, "auto", "residual stream between pipeline stages: bf16, fp32 or auto (bf16 on GPUs, fp32 on the CPU back end)"),
    EnvVar("LLAMINAR_TP_SPIN_LIMIT", int, 64_000_000, "iterations of the bounded in-kernel wait for a peer (64 ns apiece: about four seconds, so that a host hiccup of one rank does not end the step)"),
    EnvVar("LLAMINAR_COLLECTIVE_ORDER_CHECK", bool, False, "audit that all ranks issue the same collectives in the same order"),
    EnvVar("LLAMINAR_VERIFY_COLLECTIVES", bool, False, "after every all-reduce compare a checksum of the result across ranks (and count NaN/Inf)"),
    EnvVar("LLAMINAR_SKIP_ALLREDUCE", bool, False, "debug: skip tensor-parallel all-reduces (results are wrong; isolates compute time)"),
    EnvVar("LLAMINAR_VALIDATE_TENSORS", bool, False, "check every index of a step's inputs on the host before launch; scan activations for NaN/Inf after every layer"),
    EnvVar("LLAMINAR_PDL", bool, True, "launch the decode-path kernels with programmatic dependent launch (prologues overlap the previous kernel)"),
    EnvVar("LLAMINAR_ATTN_TC", bool, True, "long prefill chunks (head_dim 128) run attention on the tcgen05 kernel instead of the mma.sync kernel"),
    EnvVar("LLAMINAR_TUNING_FILE", str, "", "JSON table of measured kernel launch parameters (written by python -m llaminar_b200.ops.tuning)"),
    EnvVar("LLAMINAR_NO_CUDA_GRAPHS", bool, False, "run decode steps eagerly instead of replaying CUDA graphs"),
    EnvVar("LLAMINAR_HEARTBEAT_S", float, 2.0, "interval of the per-rank heartbeat"),
    EnvVar("LLAMINAR_WATCHDOG_TIMEOUT_S", float, 60.0, "a rank whose heartbeat is older than this is reported dead"),
    EnvVar("LLAMINAR_STEP_TIMEOUT_S", float, 0.0, "abort the process group when one engine step takes longer (0 = off)"),
    EnvVar("LLAMINAR_STAGE_DUMP_DIR", str, "", "dump per-layer hidden states of the next forward pass into this directory"),
    EnvVar("LLAMINAR_BOUNDS_CHECK", bool, False, "build and load the kernels' debug variant with explicit index checks (status word instead of a fault)"),
    EnvVar("LLAMINAR_EXTENSION_REQUIRED", bool, True, "fail instead of falling back when the CUDA extension is missing on a GPU host"),
)
_BY_NAME = {e.name: e for e in REGISTRY}
_TRUE = {"1", "true", "yes", "on"}


class DebugEnv:
    def __init__(self, environ=None):
        self._env = os.environ if environ is None else environ

    def get(self, name: str):
        spec = _BY_NAME.get(name)
        if spec is None:
            raise KeyError(f"{name} is not a registered environment switch")
        raw = self._env.get(name)
        if raw is None or raw == "":
            return spec.default
        if spec.kind is bool:
            return raw.strip().lower() in _TRUE
        try:
            return spec.kind(raw)
        except ValueError as exc:
            raise ValueError(f"{name}={raw!r}: expected {spec.kind.__name__}") from exc

    def __getattr__(self, short: str):
        return self.get("LLAMINAR_" + short.upper())

    def describe(self) -> str:
        return "\n".join(f"{e.name:36s} {e.kind.__name__:5s} default={e.default!r:10}  {e.help}" for e in REGISTRY)

    def unknown(self) -> list[str]:
        """LLAMINAR_* names present in the environment but not registered (typos)."""
        return sorted(k for k in self._env if k.startswith("LLAMINAR_") and k not in _BY_NAME)


_env = DebugEnv()


def debug_env() -> DebugEnv:
    return _env
