"""Offline tuning table for the kernels' launch parameters.

The kernels choose their split-K factor (decode GEMV, small-batch GEMM) from built-in heuristics.  A table of measured
choices, keyed by (kernel, weight format, N, K, rows), overrides the heuristic where a sweep found a faster value:

    python -m llaminar_b200.ops.tuning --model qwen3-32b --formats Q4_K,Q6_K --tp 1,2,4,8 --out tuning.json    # on a B200
    LLAMINAR_TUNING_FILE=tuning.json python -m llaminar_b200 serve ...

An entry is kept only when it beats the heuristic by more than 3 %, so an empty or missing file changes nothing.  This
replaces the reference's learned tile heuristics (ONNX / decision-tree models trained from benchmark sweeps:
src/v2/kernels/cuda/python/, cmake/CudaGemmPipeline.cmake, python/train_*) with a plain lookup for the one target GPU.
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

DEFAULT_FILE = Path(__file__).with_name("tuning_b200.json")
MIN_GAIN = 0.03
GEMV_KSPLITS = (0, 1, 2, 3, 4, 6, 8, 12)


def key(kernel: str, fmt: int, n: int, k: int, rows: int) -> str:
    return f"{kernel}:{fmt}:{n}x{k}:m{rows}"


class TuningTable:
    def __init__(self, entries: dict | None = None, source: str = ""):
        self.entries = dict(entries or {})
        self.source = source

    @classmethod
    def load(cls, path: str | os.PathLike | None = None) -> "TuningTable":
        """The file named by LLAMINAR_TUNING_FILE, else the table shipped beside this module, else an empty table."""
        if path is None:
            from ..utils.env import debug_env
            path = debug_env().tuning_file or (DEFAULT_FILE if DEFAULT_FILE.exists() else None)
        if not path:
            return cls()
        p = Path(path)
        if not p.exists():
            raise FileNotFoundError(f"tuning file {p} does not exist")
        doc = json.loads(p.read_text())
        if not isinstance(doc, dict) or not isinstance(doc.get("entries", {}), dict):
            raise ValueError(f"tuning file {p}: expected an object with an 'entries' object")
        for name, e in doc.get("entries", {}).items():
            if not isinstance(e, dict) or not isinstance(e.get("ksplit", 0), int) or e.get("ksplit", 0) < 0:
                raise ValueError(f"tuning file {p}: bad entry {name!r}")
        return cls(doc.get("entries", {}), str(p))

    def ksplit(self, kernel: str, fmt: int, n: int, k: int, rows: int) -> int:
        """Measured split-K factor, or 0 (let the kernel's heuristic decide)."""
        e = self.entries.get(key(kernel, fmt, n, k, rows))
        return int(e["ksplit"]) if e else 0

    def record(self, kernel: str, fmt: int, n: int, k: int, rows: int, timings_us: dict[int, float]) -> bool:
        """Keep the fastest ksplit of a sweep if it beats the heuristic (ksplit 0) by more than MIN_GAIN."""
        base = timings_us[0]
        best = min(timings_us, key=timings_us.get)
        name = key(kernel, fmt, n, k, rows)
        if best != 0 and timings_us[best] < base * (1.0 - MIN_GAIN):
            self.entries[name] = {"ksplit": int(best), "us": round(timings_us[best], 2), "heuristic_us": round(base, 2)}
            return True
        self.entries.pop(name, None)
        return False

    def dump(self, path: str | os.PathLike, meta: dict | None = None) -> None:
        Path(path).write_text(json.dumps({"meta": meta or {}, "entries": self.entries}, indent=1, sort_keys=True) + "\n")


_table: TuningTable | None = None


def table() -> TuningTable:
    global _table
    if _table is None:
        _table = TuningTable.load()
    return _table


def reset(new: TuningTable | None = None) -> None:
    """Replace (or drop) the cached table; tests and the sweep use it."""
    global _table
    _table = new


def projection_shapes(cfg, tp: int = 1) -> list[tuple[str, int, int]]:
    """(name, N, K) of the per-rank decoder projections of a dense model under tensor parallelism."""
    hd = cfg.head_dim
    q, kv = cfg.n_heads * hd // tp, max(cfg.n_kv_heads // tp, 1) * hd
    return [("qkv", q + 2 * kv, cfg.d_model), ("wo", cfg.d_model, q), ("gate_up", 2 * cfg.d_ff // tp, cfg.d_model),
            ("down", cfg.d_model, cfg.d_ff // tp)]


def _sweep_gemv(ops, pw_list, x, out, norm_w, sc, ksplit: int, iters: int = 30) -> float:
    import torch
    for i in range(4):
        ops.gemv(pw_list[i % len(pw_list)], x, out, norm_w=norm_w, scratch=sc, ksplit=ksplit, tuned=False)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        ops.gemv(pw_list[i % len(pw_list)], x, out, norm_w=norm_w, scratch=sc, ksplit=ksplit, tuned=False)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def main() -> int:
    """Sweep the decode GEMV's split-K factor over a model's projection shapes on this GPU and write the table."""
    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--model", default="qwen3-32b")
    ap.add_argument("--formats", default="Q4_K,Q6_K", help="weight formats to sweep (comma separated)")
    ap.add_argument("--tp", default="1", help="tensor-parallel degrees whose shard shapes are swept (comma separated)")
    ap.add_argument("--rows", default="1", help="GEMV row counts (1..4, comma separated)")
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    import torch
    from .. import ops
    from ..gguf import GGMLType
    from ..gguf.constants import BLOCK_GEOMETRY
    from ..models.config import SHAPES
    from .layout import FMT_IDS
    cfg = SHAPES[args.model]
    dev = torch.device("cuda")
    sc = ops.scratch_for(dev)
    tab = TuningTable()
    for fmt_name in args.formats.split(","):
        qt = GGMLType[fmt_name]
        e_, b_ = BLOCK_GEOMETRY[qt]
        for tp in (int(t) for t in args.tp.split(",")):
            for name, n, k in projection_shapes(cfg, tp):
                if n % 128 or k % 256:
                    continue
                wb = n * k // e_ * b_
                pws = []
                for c in range(max(2, min(16, int(300e6 // wb) + 1))):       # rotate copies so that weights come from HBM
                    raw = torch.randint(0, 256, (wb,), dtype=torch.uint8, device=dev)
                    raw.view(torch.int16).bitwise_and_(0x1FFF)
                    pws.append(ops.pack_matrix(raw, qt, n, k))
                for rows in (int(r) for r in args.rows.split(",")):
                    x = torch.randn(rows, k, device=dev)
                    nw = torch.ones(k, device=dev)
                    out = torch.zeros(rows, n, dtype=torch.float32, device=dev)
                    t = {ks: _sweep_gemv(ops, pws, x, out, nw, sc, ks) for ks in GEMV_KSPLITS if ks <= max(1, k // 256 // 2)}
                    kept = tab.record("gemv", FMT_IDS[qt], n, k, rows, t)
                    print(f"{fmt_name} tp{tp} {name} {n}x{k} m{rows}: " + " ".join(f"ks{a}={b:.1f}" for a, b in t.items()) +
                          (f"  -> ksplit {tab.ksplit('gemv', FMT_IDS[qt], n, k, rows)}" if kept else "  -> heuristic"), flush=True)
                del pws
    tab.dump(args.out, {"model": args.model, "device": torch.cuda.get_device_name(0), "min_gain": MIN_GAIN})
    print(f"wrote {len(tab.entries)} entries to {args.out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
