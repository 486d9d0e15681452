"""Flag parsing, validation rules, the placement planner, the CLI commands and SPMD command replication."""
import json
import subprocess
import sys

import pytest

from llaminar_b200.config.orchestration import ConfigError, parse_args
from llaminar_b200.models.config import SHAPES
from llaminar_b200.planning import build_plan
from tests.mp_utils import run_ranks


def test_defaults_and_explicit_set():
    c = parse_args(["oneshot", "--synthetic", "tiny-qwen3", "-n", "7"])
    assert c.command == "oneshot" and c.values["n_predict"] == 7 and "n_predict" in c.explicitly_set
    assert c.layout()["world"] == 1 and c.layout()["pp"] == 1


def test_yaml_config_and_cli_override(tmp_path):
    p = tmp_path / "c.yaml"
    p.write_text("synthetic: tiny-qwen3\nctx-size: 256\nbatch_size: 3\n")
    c = parse_args(["serve", "--config", str(p), "-c", "128"])
    assert c.values["ctx_size"] == 128 and c.values["batch_size"] == 3 and c.values["synthetic"] == "tiny-qwen3"
    p.write_text("no_such_key: 1\n")
    with pytest.raises(ConfigError):
        parse_args(["serve", "--config", str(p)])


def test_device_modes_are_mutually_exclusive():
    with pytest.raises(ConfigError) as e:
        parse_args(["oneshot", "--synthetic", "tiny-qwen3", "-d", "cuda:0", "--tp-devices", "cuda:0,cuda:1"])
    assert "mutually exclusive" in str(e.value)


def test_pp_layout_and_rules():
    argv = ["plan", "--synthetic", "qwen3-32b", "--define-domain", "a=cuda:0,cuda:1,cuda:2,cuda:3",
            "--define-domain", "b=cuda:4,cuda:5,cuda:6,cuda:7", "--pp-stage", "0=a:0-31", "--pp-stage", "1=b:32-63"]
    lay = parse_args(argv).layout()
    assert lay["pp"] == 2 and lay["tp"] == 4 and lay["world"] == 8 and lay["stages"][1][2:] == (32, 63)
    bad = argv[:-1] + ["1=b:40-63"]
    with pytest.raises(ConfigError) as e:
        parse_args(bad)
    assert "must continue at 32" in str(e.value)
    with pytest.raises(ConfigError):
        parse_args(["plan", "--synthetic", "qwen3-32b", "--pp-stage", "0=a:0-31"])


def test_unsupported_and_bad_values_are_named():
    with pytest.raises(ConfigError) as e:
        parse_args(["oneshot", "--synthetic", "tiny-qwen3", "--kv-cache-precision", "tq4"])
    assert "turbo-quantised KV" in str(e.value)
    with pytest.raises(ConfigError) as e:
        parse_args(["oneshot", "--synthetic", "tiny-qwen3", "-d", "cpu", "--kv-cache-precision", "q8_0"])
    assert "CUDA feature" in str(e.value)
    parse_args(["oneshot", "--synthetic", "tiny-qwen3", "--kv-cache-precision", "q8_0"])       # accepted for GPUs
    with pytest.raises(ConfigError):
        parse_args(["oneshot", "--synthetic", "tiny-qwen3", "--tp-devices", "rocm:0,rocm:1"])
    with pytest.raises(ConfigError):
        parse_args(["oneshot", "--synthetic", "tiny-qwen3", "--mtp-draft-tokens", "5"])
    with pytest.raises(ConfigError):
        parse_args(["oneshot"])


def test_planner_memory_and_errors():
    lay = {"pp": 2, "tp": 4, "world": 8, "stages": [("a", [f"cuda:{i}" for i in range(4)], 0, 31), ("b", [f"cuda:{i}" for i in range(4, 8)], 32, 63)]}
    plan = build_plan(SHAPES["qwen3-32b"], lay, ctx_size=4096, batch_size=8)
    assert not plan.errors and len(plan.ranks) == 8
    assert all(2e9 < r.total_bytes < 30e9 for r in plan.ranks)
    assert "stage" in plan.table()
    lay3 = {"pp": 1, "tp": 3, "world": 3, "stages": [("d", ["cuda:0", "cuda:1", "cuda:2"], 0, -1)]}
    assert build_plan(SHAPES["qwen3-8b"], lay3, ctx_size=4096, batch_size=1).errors


def _cli(*args):
    r = subprocess.run([sys.executable, "-m", "llaminar_b200", *args], capture_output=True, text=True, timeout=300)
    return r.returncode, r.stdout, r.stderr


def test_cli_oneshot_benchmark_plan_describe(tmp_path):
    rc, out, err = _cli("oneshot", "--synthetic", "tiny-qwen3", "--synthetic-recipe", "Q8_0", "-d", "cpu", "-p", "hello", "-n", "5")
    assert rc == 0, err
    out_json = tmp_path / "b.json"
    rc, out, err = _cli("benchmark", "--synthetic", "tiny-qwen3", "--synthetic-recipe", "Q8_0", "-d", "cpu", "--bench-runs", "1",
                        "--bench-prompt-tokens", "64", "-n", "8", "--bench-json", str(out_json))
    assert rc == 0, err
    j = json.loads(out_json.read_text())
    assert j["decode_tok_s"] > 0 and j["prefill_tok_s"] > 0 and j["ttft_ms_p50"] > 0
    rc, out, err = _cli("plan", "--synthetic", "qwen3-8b", "--tp-devices", "cuda:0,cuda:1")
    assert rc == 0 and "weight_bytes" in out
    rc, out, err = _cli("describe")
    assert rc == 0 and "cpu" in out
    rc, out, err = _cli("oneshot", "--synthetic", "nope")
    assert rc != 0 and "unknown shape" in (out + err)
    rc, out, err = _cli("oneshot", "--synthetic", "tiny-qwen3", "-d", "cpu", "-c", "8192", "-p", "x", "-n", "1")
    assert rc != 0 and "trained context" in (out + err)


def _spmd_run(rank, world):
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.parallel.spmd import ControlChannel, ReplicatedEngine, worker_loop
    from llaminar_b200.parallel.tp import TPContext
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=0)
    tp = TPContext.create(device="cpu")
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=128, tp=tp)
    ch = ControlChannel()
    if rank != 0:
        worker_loop(eng, ch)
        return eng.stats["decode_tokens"]
    drive = ReplicatedEngine(eng, ch)
    r = drive.add_request(list(range(3, 20)), SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    r2 = drive.add_request(list(range(30, 50)), SamplingParams(temperature=0.0, max_tokens=50, ignore_eos=True))
    n = 0
    while r.state != "finished":
        drive.step()
        n += 1
        if n == 2:
            drive.abort(r2.rid)
    drive.shutdown_workers()
    return eng.stats["decode_tokens"]


def test_spmd_workers_mirror_rank0():
    res = run_ranks(_spmd_run, 2)
    assert res[0] == res[1] and res[0] > 0


def test_cli_chat_reads_turns_from_stdin():
    r = subprocess.run([sys.executable, "-m", "llaminar_b200", "chat", "--synthetic", "tiny-qwen3", "--synthetic-recipe", "Q8_0",
                        "-d", "cpu", "-n", "4", "-c", "256", "--system-prompt", "be brief"],
                       input="hello\n/reset\nagain\n/exit\n", capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert r.stdout.count("> ") >= 3


def test_precision_flags_are_checked_against_the_device():
    with pytest.raises(ConfigError) as e:
        parse_args(["oneshot", "--synthetic", "tiny-qwen3", "--kv-cache-precision", "fp16"])
    assert "bf16" in str(e.value)
    c = parse_args(["oneshot", "--synthetic", "tiny-qwen3", "-d", "cpu", "--kv-cache-precision", "fp16"])
    assert c.values["kv_cache_precision"] == "fp16"
    rc, out, err = _cli("oneshot", "--synthetic", "tiny-qwen3", "--synthetic-recipe", "Q8_0", "-d", "cpu", "--kv-cache-precision", "bf16",
                        "-p", "hi", "-n", "3")
    assert rc == 0, err


def test_suggest_layout_from_synthetic_inventories():
    """Placement scenarios on made-up device inventories (no hardware): the planner is pure."""
    from llaminar_b200.planning import suggest_layout
    GB = 10 ** 9
    # a 32B Q4_K_S model fits one 180 GB device
    lay, plan = suggest_layout(SHAPES["qwen3-32b"], 8, "Q4_K_S", ctx_size=4096, batch_size=32)
    assert (lay["pp"], lay["tp"], lay["world"]) == (1, 1, 1) and not plan.errors
    # on 16 GB devices it needs several; tensor parallelism is preferred to pipeline stages when the heads divide
    lay, plan = suggest_layout(SHAPES["qwen3-32b"], 8, "Q4_K_S", ctx_size=2048, batch_size=1, hbm_bytes=16 * GB)
    assert lay is not None and lay["world"] in (2, 4) and lay["pp"] == 1 and max(r.total_bytes for r in plan.ranks) < 16 * GB
    # three devices: 64 heads cannot be split three ways, so the answer is three pipeline stages (or fewer devices)
    lay, plan = suggest_layout(SHAPES["qwen3-32b"], 3, "Q4_K_S", ctx_size=2048, batch_size=1, hbm_bytes=10 * GB)
    assert lay is None or lay["tp"] in (1, 2)
    # a mixed inventory: every rank must fit the smallest device that takes part
    lay, plan = suggest_layout(SHAPES["qwen3-32b"], 4, "Q4_K_S", ctx_size=2048, batch_size=1, hbm_bytes=[180 * GB, 12 * GB, 12 * GB, 12 * GB])
    assert lay["world"] == 1
    # nothing fits: the reasons say why
    lay, reasons = suggest_layout(SHAPES["qwen3-32b"], 2, "Q4_K_S", ctx_size=2048, batch_size=1, hbm_bytes=4 * GB)
    assert lay is None and reasons and "GB" in reasons[0]
    # the MoE model splits its experts
    lay, plan = suggest_layout(SHAPES["qwen3-30b-a3b"], 8, "IQ3_S_MOE", ctx_size=1024, batch_size=64, hbm_bytes=8 * GB)
    assert lay is not None and lay["world"] >= 2
    rc, out, err = _cli("plan", "--synthetic", "qwen3-32b", "--synthetic-recipe", "Q4_K_S", "--suggest-layout", "8")
    assert rc == 0 and "suggested layout: pp=1 x tp=1" in out and "flags: -d cuda:0" in out


def test_topology_tree_string_and_file(tmp_path):
    """--topology / --topology-file: a parallelism tree becomes domains and evenly split pipeline stages."""
    from llaminar_b200.config.orchestration import parse_topology, topology_to_layout
    c = parse_args(["plan", "--synthetic", "qwen3-32b", "--topology", "PP(global, TP(a, cuda:0, cuda:1), TP(b, cuda:2, cuda:3))"])
    lay = c.layout()
    assert (lay["pp"], lay["tp"], lay["world"]) == (2, 2, 4) and [s[0] for s in lay["stages"]] == ["a", "b"]
    plan = build_plan(SHAPES["qwen3-32b"], lay)
    assert not plan.errors and [(r.first_layer, r.last_layer) for r in plan.ranks] == [(0, 31), (0, 31), (32, 63), (32, 63)]
    lay = parse_args(["plan", "--synthetic", "qwen3-8b", "--topology", "tp(g, cuda:0, cuda:1, cuda:2, cuda:3)"]).layout()
    assert (lay["pp"], lay["tp"]) == (1, 4)
    lay = parse_args(["plan", "--synthetic", "qwen3-8b", "--topology", "PP(g, cuda:0, cuda:1, cuda:2)"]).layout()
    assert (lay["pp"], lay["tp"], lay["world"]) == (3, 1, 3)
    y = tmp_path / "t.yaml"
    y.write_text("topology:\n  type: pp\n  name: global\n  children:\n    - {type: tp, name: s1, rank: 1, devices: ['cuda:2', 'cuda:3']}\n"
                 "    - {type: tp, name: s0, rank: 0, backend: nccl, devices: ['cuda:0', 'cuda:1']}\n")
    c = parse_args(["plan", "--synthetic", "qwen3-32b", "--topology-file", str(y)])
    assert [s[0] for s in c.layout()["stages"]] == ["s0", "s1"] and c.domains[0].backend == "nccl"
    for bad in ("PP(global", "XX(a, cuda:0)", "TP(a)", "PP(g, TP(a, cuda:0), TP(b, cuda:0))", "TP(a, cuda:0) junk", "TP(a, TP(b, cuda:0))",
                "PP(g, TP(a, cuda:0, cuda:1), TP(b, cuda:2))"):
        with pytest.raises(ConfigError):
            parse_args(["plan", "--synthetic", "qwen3-32b", "--topology", bad])
    with pytest.raises(ConfigError):
        parse_args(["plan", "--synthetic", "qwen3-32b", "--topology", "TP(a, cuda:0, cuda:1)", "--tp-devices", "cuda:0,cuda:1"])
    tree = parse_topology("PP(x, TP(y, cuda:0))")
    assert tree["children"][0]["devices"] == ["cuda:0"] and topology_to_layout(tree)[1][0].domain == "y"


def test_device_map_is_an_explicit_rank_to_device_mapping():
    c = parse_args(["plan", "--synthetic", "qwen3-32b", "--device-map", "1=cuda:3, 0=cuda:2"])
    assert c.layout()["stages"][0][1] == ["cuda:2", "cuda:3"] and c.layout()["tp"] == 2
    for bad in ("0=cuda:0,2=cuda:1", "a=cuda:0", "0=cuda:0,0=cuda:1"):
        with pytest.raises(ConfigError):
            parse_args(["plan", "--synthetic", "qwen3-32b", "--device-map", bad])
    with pytest.raises(ConfigError):
        parse_args(["plan", "--synthetic", "qwen3-32b", "--device-map", "0=cuda:0", "-d", "cuda:0"])


def test_cli_moe_stats_and_expert_placement(tmp_path):
    stats = tmp_path / "stats.json"
    base = ["oneshot", "--synthetic", "tiny-qwen3moe", "--synthetic-recipe", "Q8_0", "-d", "cpu", "-p", "hello world", "-n", "5"]
    rc, out1, err = _cli(*base, "--moe-stats-out", str(stats))
    assert rc == 0 and json.loads(stats.read_text())["n_experts"] == SHAPES["tiny-qwen3moe"].n_experts, err
    rc, out2, err = _cli(*base, "--moe-expert-placement", str(stats))
    assert rc == 0 and out2.strip().splitlines()[-1] == out1.strip().splitlines()[-1], err      # same model function
    rc, out, err = _cli("oneshot", "--synthetic", "tiny-qwen3", "-d", "cpu", "-p", "x", "-n", "2", "--moe-expert-placement", str(stats))
    assert rc != 0 and "mixture-of-experts" in (out + err)
    rc, out, err = _cli(*base, "--moe-rebalance")
    assert rc != 0 and "--moe-expert-placement" in (out + err)


def test_describe_env_lists_the_switch_registry(capsys):
    from llaminar_b200.app import main
    assert main(["describe", "--env"]) == 0
    out = capsys.readouterr().out
    assert "LLAMINAR_TP_FUSED" in out and "LLAMINAR_ATTN_TC" in out


def test_planner_counts_resident_bytes_for_formats_without_a_packed_layout():
    """A 2-bit checkpoint is re-encoded as Q8_0 at load, so the plan must budget those bytes, not the file's; packed
    formats are budgeted at their file size, unquantised tensors as bf16."""
    from llaminar_b200.gguf.constants import GGMLType
    from llaminar_b200.models.config import SHAPES, QuantRecipe
    from llaminar_b200.planning import _bytes, build_plan
    assert _bytes(GGMLType.Q4_K, 256) == 144 and _bytes(GGMLType.IQ3_S, 256) == 110
    assert _bytes(GGMLType.IQ2_XS, 256) == 272 and _bytes(GGMLType.IQ2_XS, 256, expert=True) == 272
    assert _bytes(GGMLType.BF16, 256) == 512 and _bytes(GGMLType.F32, 256) == 512
    cfg = SHAPES["qwen3-32b"]
    layout = {"tp": 1, "stages": [("main", ["cuda:0"], 0, cfg.n_layers - 1)]}
    low = build_plan(cfg, layout, QuantRecipe(GGMLType.IQ2_XS, {}, "IQ2_XS"), 4096, 1)
    q4 = build_plan(cfg, layout, "Q4_K_S", 4096, 1)
    assert low.ranks[0].weight_bytes > 1.7 * q4.ranks[0].weight_bytes


def test_plan_of_a_checkpoint_budgets_the_formats_in_the_file(tmp_path, capsys):
    from llaminar_b200.app import main
    from llaminar_b200.gguf import GGUFFile
    from llaminar_b200.gguf.constants import GGMLType
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.planning import FileRecipe, build_plan
    sizes = {}
    for recipe in ("Q8_0", "Q4_K_M"):
        path = str(tmp_path / f"{recipe}.gguf")
        synthesize(SHAPES["tiny-qwen3"], recipe, seed=0).save_gguf(path)
        gf = GGUFFile(path)
        fr = FileRecipe(gf)
        assert fr.for_tensor("blk.0.attn_q.weight") == gf["blk.0.attn_q.weight"].qtype
        assert fr.for_tensor("blk.99.attn_q.weight") == fr.default and fr.default == (GGMLType.Q8_0 if recipe == "Q8_0" else GGMLType.Q4_K)
        layout = {"tp": 1, "stages": [("main", ["cuda:0"], 0, SHAPES["tiny-qwen3"].n_layers - 1)]}
        sizes[recipe] = build_plan(SHAPES["tiny-qwen3"], layout, fr).ranks[0].weight_bytes
        nominal = build_plan(SHAPES["tiny-qwen3"], layout, recipe).ranks[0].weight_bytes
        assert abs(sizes[recipe] - nominal) <= 0.1 * nominal      # a tied head takes the embedding's format, not the recipe's
        gf.close()
    assert sizes["Q8_0"] > 1.5 * sizes["Q4_K_M"]
    assert main(["plan", "-m", str(tmp_path / "Q8_0.gguf"), "-d", "cuda:0"]) == 0
    assert "weight" in capsys.readouterr().out


def test_describe_device_benchmark_reports_copy_and_matrix_rates(capsys):
    """`describe --device-benchmark`: on a host without GPUs the CPU is measured (small sizes), the JSON keeps its shape."""
    import json
    from llaminar_b200.app import main
    assert main(["describe", "--device-benchmark"]) == 0
    out = json.loads(capsys.readouterr().out)
    d = out["benchmark"]["devices"][0]
    assert d["copy_gbs"] > 0 and d["matmul_tflops"] > 0 and d["matmul_dtype"] in ("float32", "bfloat16")
    assert isinstance(out["benchmark"]["p2p"], list)
