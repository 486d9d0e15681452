"""Perf-stats collector, environment-switch registry, collective-order checker, device inventory."""
import json

import pytest

from llaminar_b200.utils.perfstats import PerfStats
from tests.mp_utils import run_ranks


def test_perfstats_records_export_and_filter():
    p = PerfStats(enabled=True)
    p.set_phase("prefill")
    with p.timer("engine", "step", device="cpu", tags=("bs4",)):
        sum(range(1000))
    with p.timer("engine", "step", device="cpu", tags=("bs4",)):
        pass
    p.set_phase("decode")
    p.count("kv", "pages_allocated", 3)
    p.count("kv", "pages_allocated", 2)
    p.gauge("kv", "free_pages", 17)
    rows = p.rows()
    step = next(r for r in rows if r["name"] == "step")
    assert step["count"] == 2 and step["phase"] == "prefill" and step["tags"] == "bs4" and step["total_ms"] >= step["max_ms"] > 0
    pages = next(r for r in rows if r["name"] == "pages_allocated")
    assert pages["value"] == 5 and pages["phase"] == "decode"
    assert json.loads(p.to_json("kv")) and all(r["domain"] == "kv" for r in json.loads(p.to_json("kv")))
    csv = p.to_csv()
    assert csv.splitlines()[0].startswith("domain,name,phase,device,tags") and "free_pages" in csv
    assert "pages_allocated" in p.table()
    off = PerfStats(enabled=False)
    with off.timer("a", "b"):
        pass
    off.count("a", "c")
    assert off.rows() == []


def test_env_registry_types_and_unknown_names():
    from llaminar_b200.utils.env import DebugEnv
    env = DebugEnv({"LLAMINAR_PROFILING": "true", "LLAMINAR_TP_SPIN_LIMIT": "1000", "LLAMINAR_STAGE_DUMP_DIR": "/x"})
    assert env.profiling is True and env.tp_spin_limit == 1000 and env.stage_dump_dir == "/x" and env.pdl is True
    with pytest.raises(KeyError):
        env.get("LLAMINAR_NOT_A_SWITCH")
    with pytest.raises(ValueError):
        DebugEnv({"LLAMINAR_TP_SPIN_LIMIT": "many"}).tp_spin_limit
    assert "LLAMINAR_TP_FUSED" in env.describe()


def _order_check(rank, world, diverge):
    import torch
    from llaminar_b200.parallel.collective_check import CollectiveOrderChecker, CollectiveOrderMismatch
    chk = CollectiveOrderChecker(None, interval=1000)
    x = torch.zeros(4, 8)
    for i in range(5):
        chk.record("all_reduce", x)
    if diverge and rank == 1:
        chk.record("all_gather_vocab", x[:, :4])       # rank 1 issues a different collective
    else:
        chk.record("all_reduce", x)
    try:
        chk.verify()
        return "same"
    except CollectiveOrderMismatch as exc:
        return str(exc)


def test_collective_order_checker_names_the_divergence():
    assert run_ranks(_order_check, 2, False) == ["same", "same"]
    res = run_ranks(_order_check, 2, True)
    assert all("diverged" in r and "all_gather_vocab" in r for r in res)


def test_device_inventory_shape():
    from llaminar_b200.utils.devices import describe_devices as describe
    d = describe()
    assert "cpu" in d and "gpus" in d and isinstance(d["gpus"], list)


def test_tuning_table_keeps_only_clear_wins_and_validates_files(tmp_path):
    from llaminar_b200.ops import tuning
    t = tuning.TuningTable()
    assert t.ksplit("gemv", 0, 5120, 8192, 1) == 0                       # nothing measured: the kernel's heuristic decides
    assert t.record("gemv", 0, 5120, 8192, 1, {0: 20.0, 2: 19.8, 4: 17.0}) is True
    assert t.ksplit("gemv", 0, 5120, 8192, 1) == 4
    assert t.record("gemv", 0, 10240, 5120, 1, {0: 20.0, 2: 19.8}) is False    # 1 % is noise, not a win
    assert t.ksplit("gemv", 0, 10240, 5120, 1) == 0
    f = tmp_path / "tune.json"
    t.dump(f, {"device": "test"})
    back = tuning.TuningTable.load(f)
    assert back.entries == t.entries and back.ksplit("gemv", 0, 5120, 8192, 1) == 4
    bad = tmp_path / "bad.json"
    bad.write_text('{"entries": {"gemv:0:1x1:m1": {"ksplit": -3}}}')
    import pytest
    with pytest.raises(ValueError):
        tuning.TuningTable.load(bad)
    with pytest.raises(FileNotFoundError):
        tuning.TuningTable.load(tmp_path / "missing.json")
    from llaminar_b200.models.config import SHAPES
    shapes = dict((n, (a, b)) for n, a, b in tuning.projection_shapes(SHAPES["qwen3-32b"], tp=2))
    assert shapes["qkv"] == (5120, 5120) and shapes["down"] == (5120, 12800) and shapes["gate_up"] == (25600, 5120)


def test_perf_gate_flags_only_slowdowns_beyond_the_tolerance():
    from llaminar_b200.ops import perf_gate
    base = {"gemv": {"us": 40.0, "tolerance": 0.2}, "gemm_large": {"us": 500.0, "tolerance": 0.15}, "moe": {"us": 300.0}}
    bad, notes = perf_gate.compare(base, {"gemv": 47.0, "gemm_large": 580.0, "moe": 250.0, "extra": 1.0})
    assert len(bad) == 1 and bad[0].startswith("gemm_large") and "+16 %" in bad[0]
    assert any(n.startswith("moe") and "faster" in n for n in notes) and any(n.startswith("extra") for n in notes)
    bad, _ = perf_gate.compare(base, {"gemv": 40.0})
    assert sorted(b.split(":")[0] for b in bad) == ["gemm_large", "moe"]
    rec = {"mma_sync": {"us": 570.0, "tflops": 1.0}, "tcgen05": {"us": 480.0, "tflops": 1.0}}
    assert perf_gate.extract_us("attn_prefill", rec) == {"attn_prefill.mma_sync": 570.0, "attn_prefill.tcgen05": 480.0}
    assert perf_gate.extract_us("moe", {"us_three_launches": 315.0}) == {"moe": 315.0}
    import json
    doc = json.loads(perf_gate.BASELINE.read_text())
    assert {"gemv", "gemm_small", "gemm_large", "attn_decode", "moe"} <= set(doc["cases"])
