"""Performance regression gate for the hot kernels.

    python -m llaminar_b200.ops.perf_gate               # on a B200: run the profile cases, compare with the baseline, exit 1 on a regression
    python -m llaminar_b200.ops.perf_gate --update      # rewrite the baseline from this run

Each case of ``ops/profile_cases.py`` runs in a child process; its time is compared with ``perf_baseline_b200.json``
(microseconds, CUDA events) under a per-case tolerance.  Only slow-downs fail the gate; a case that got faster than
its tolerance is reported so that the baseline can be refreshed.  Counterpart of the reference's pre-commit benchmark
check (.githooks/run_benchmark_check.sh against .githooks/benchmark_baseline.json, 5-25 % thresholds).
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
from pathlib import Path

BASELINE = Path(__file__).with_name("perf_baseline_b200.json")


def extract_us(case: str, rec: dict) -> dict[str, float]:
    """The timed quantities of one profile-case record, by name."""
    if case == "attn_prefill":
        return {f"attn_prefill.{k}": float(rec[k]["us"]) for k in ("mma_sync", "tcgen05") if k in rec}
    if case == "moe":
        return {"moe": float(rec["us_three_launches"])}
    return {case: float(rec["us"])}


def compare(baseline: dict, measured: dict[str, float]) -> tuple[list[str], list[str]]:
    """(regressions, notes).  ``baseline``: name -> {"us": float, "tolerance": fraction}."""
    bad, notes = [], []
    for name, spec in sorted(baseline.items()):
        if name not in measured:
            bad.append(f"{name}: not measured")
            continue
        us, ref, tol = measured[name], float(spec["us"]), float(spec.get("tolerance", 0.15))
        ratio = us / ref
        if ratio > 1.0 + tol:
            bad.append(f"{name}: {us:.1f} us vs baseline {ref:.1f} us (+{(ratio - 1) * 100:.0f} %, tolerance {tol * 100:.0f} %)")
        elif ratio < 1.0 - tol:
            notes.append(f"{name}: {us:.1f} us, {(1 - ratio) * 100:.0f} % faster than the baseline {ref:.1f} us: refresh it with --update")
        else:
            notes.append(f"{name}: {us:.1f} us (baseline {ref:.1f} us)")
    for name in sorted(set(measured) - set(baseline)):
        notes.append(f"{name}: {measured[name]:.1f} us (no baseline)")
    return bad, notes


def run_case(case: str, iters: int) -> dict:
    r = subprocess.run([sys.executable, "-m", "llaminar_b200.ops.profile_cases", "--case", case, "--iters", str(iters)],
                       capture_output=True, text=True, timeout=600)
    if r.returncode != 0:
        raise RuntimeError(f"profile case {case} failed:\n{r.stderr[-2000:]}")
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    return json.loads(lines[-1])


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--cases", default="gemv,gemm_small,gemm_large,attn_decode,attn_prefill,moe")
    ap.add_argument("--iters", type=int, default=9)
    ap.add_argument("--baseline", default=str(BASELINE))
    ap.add_argument("--update", action="store_true", help="write this run's times as the new baseline (tolerances are kept)")
    args = ap.parse_args()
    doc = json.loads(Path(args.baseline).read_text()) if Path(args.baseline).exists() else {"cases": {}}
    measured: dict[str, float] = {}
    for case in args.cases.split(","):
        measured.update(extract_us(case, run_case(case, args.iters)))
    if args.update:
        for name, us in measured.items():
            doc["cases"][name] = {"us": round(us, 1), "tolerance": doc["cases"].get(name, {}).get("tolerance", 0.15)}
        Path(args.baseline).write_text(json.dumps(doc, indent=1, sort_keys=True) + "\n")
        print(f"baseline written to {args.baseline}")
        return 0
    wanted = {k: v for k, v in doc["cases"].items() if k.split(".")[0] in args.cases.split(",")}
    bad, notes = compare(wanted, measured)
    for n in notes:
        print("ok   " + n)
    for b in bad:
        print("FAIL " + b)
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
