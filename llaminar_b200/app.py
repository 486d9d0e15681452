"""Application commands: oneshot, serve, benchmark, plan, describe.

Start-up sequence of `serve` / `oneshot` / `benchmark` (reference call stack: src/v2/app/AppLifecycle.cpp:17,
src/v2/app/commands/ServeCommand.cpp:24, src/v2/app/RuntimeInitPhase.cpp:30, src/v2/execution/runner/
OrchestrationRunner.cpp:739-922): parse flags -> validate -> (re-launch one process per GPU when the layout
needs several) -> build the plan, check memory -> load and shard weights -> engine -> tokenizer and chat
template -> mode.  The reference re-executes itself under `mpirun`; here the launcher is torch.distributed.run.
"""
from __future__ import annotations

import json
import os
import statistics
import subprocess
import sys
import time

import torch

from .config.orchestration import ConfigError, OrchestrationConfig, help_by_category, parse_args
from .utils.log import get_logger

log = get_logger("app")


# ---------------------------------------------------------------------------------------------------------
# process launch
# ---------------------------------------------------------------------------------------------------------
def maybe_relaunch(cfg: OrchestrationConfig, argv: list[str]) -> int | None:
    """Spawn one process per device when the layout has more than one and we are not yet under a launcher."""
    world = cfg.layout()["world"]
    if world <= 1 or "RANK" in os.environ or cfg.values.get("dry_run") or cfg.command in ("plan", "describe"):
        return None
    port = 29500 + (os.getpid() % 2000)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "llaminar_b200", *argv]
    log.info("launching %d ranks: %s", world, " ".join(cmd))
    return subprocess.call(cmd)


def init_distributed(cfg: OrchestrationConfig):
    """Returns (rank, world, device, tp_context or None, layout)."""
    import torch.distributed as dist
    layout = cfg.layout()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    devs = [d for st in layout["stages"] for d in st[1]]
    want_cpu = all(d.startswith("cpu") for d in devs) or not torch.cuda.is_available()
    if world == 1:
        dev = torch.device("cpu") if want_cpu else torch.device(devs[0] if devs else "cuda:0")
        if dev.type == "cuda":
            torch.cuda.set_device(dev)
        return 0, 1, dev, None, layout
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if want_cpu:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    else:
        dev = torch.device(devs[rank]) if rank < len(devs) else torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", device_id=dev)
    from .parallel.tp import TPContext
    tp_size = layout["tp"]
    group = dist.group.WORLD
    if layout["pp"] > 1:
        stage = rank // tp_size
        groups = [dist.new_group(list(range(s * tp_size, (s + 1) * tp_size))) for s in range(layout["pp"])]
        group = groups[stage]
    backend = cfg.values.get("backend", "auto")
    fused = None if backend == "auto" else (backend == "fused")
    tp = TPContext.create(group, dev, fused=fused) if tp_size > 1 else None
    if tp is not None:
        tp.moe_mode = cfg.values.get("moe_expert_mode") or "expert-parallel"
    if tp is not None and cfg.values.get("check_collectives"):
        from .parallel.collective_check import CollectiveOrderChecker
        tp.order_check = CollectiveOrderChecker(group)
    return rank, world, dev, tp, layout


# ---------------------------------------------------------------------------------------------------------
# model / engine construction
# ---------------------------------------------------------------------------------------------------------
def load_weights(cfg: OrchestrationConfig, device):
    from .models.config import SHAPES
    from .models.synth import synthesize
    from .models.weights import ModelWeights
    v = cfg.values
    if v.get("synthetic"):
        if v["synthetic"] not in SHAPES:
            raise ConfigError([f"--synthetic: unknown shape '{v['synthetic']}' (known: {', '.join(SHAPES)})"])
        shape = SHAPES[v["synthetic"]]
        if v.get("mtp"):
            shape = shape.with_(nextn_layers=1)
        return synthesize(shape, v.get("synthetic_recipe") or "Q4_K_M", seed=0,
                          device=device if torch.device(device).type == "cuda" else "cpu")
    return ModelWeights.from_gguf(v["model"], device="cpu")


def build_engine(cfg: OrchestrationConfig):
    from .engine.engine import LLMEngine
    from .engine.prefix_cache import PrefixCache, PrefixCacheConfig
    from .planning import build_plan
    from .tokenizer.bpe import BPETokenizer
    from .tokenizer.chat_template import ChatTemplate
    v = cfg.values
    rank, world, dev, tp, layout = init_distributed(cfg)
    t0 = time.time()
    weights = load_weights(cfg, dev)
    mcfg = weights.config
    if v.get("moe_expert_placement"):
        from .models.expert_placement import ExpertStats, apply_placement, range_loads
        try:
            loads = ExpertStats.load(v["moe_expert_placement"])
            perms = apply_placement(weights, loads, layout["tp"])
        except (OSError, ValueError) as exc:
            raise ConfigError([f"--moe-expert-placement: {exc}"]) from exc
        if rank == 0 and perms:
            l0 = min(perms)
            before = range_loads(loads[l0], list(range(mcfg.n_experts)), layout["tp"])
            after = range_loads(loads[l0], perms[l0], layout["tp"])
            log.info("expert placement from %s: %d layers renumbered; layer %d load per rank %s -> %s", v["moe_expert_placement"],
                     len(perms), l0, [int(x) for x in before], [int(x) for x in after])
    if v["ctx_size"] > mcfg.context_length:
        # positions beyond the trained maximum are extrapolated RoPE angles: refuse rather than degrade silently
        raise ConfigError([f"--ctx-size {v['ctx_size']} exceeds the model's trained context of {mcfg.context_length} tokens"])
    from .planning import FileRecipe
    plan = build_plan(mcfg, layout, FileRecipe.from_weights(weights), ctx_size=v["ctx_size"], batch_size=v["batch_size"])
    if plan.errors:
        raise ConfigError(plan.errors)
    if rank == 0:
        log.info("model %s (%s): %d layers, d=%d, heads %d/%d, vocab %d", mcfg.name, mcfg.arch, mcfg.n_layers, mcfg.d_model,
                 mcfg.n_heads, mcfg.n_kv_heads, mcfg.vocab_size)
        log.info("placement\n%s", plan.table())
    if mcfg.is_hybrid:
        # the gated attention blocks append bf16 K/V
        if v.get("kv_cache_precision") in ("q8_0", "q8_1"):
            raise ConfigError([f"--kv-cache-precision q8_0 is not available for hybrid (linear-attention) models such as {mcfg.arch}"])
    prefix = None
    if v.get("prefix_cache"):
        prefix = PrefixCache(PrefixCacheConfig.from_values(v), fingerprint=_fingerprint(mcfg, layout, v))
    mtp = None
    if v.get("mtp"):
        from .engine.mtp import MTPConfig, MTPDecoder
        mtp = MTPDecoder(MTPConfig.from_values(v))
    tok = None
    if "tokenizer.ggml.tokens" in weights.metadata:
        tok = BPETokenizer.from_metadata(weights.metadata)
    eos = tok.eos_id if tok is not None else None
    kw = dict(device=dev, max_batch=v["batch_size"], max_context=v["ctx_size"], prefix_cache=prefix, mtp=mtp, tp=tp,
              eos_token_id=eos)
    if torch.device(dev).type == "cpu" and "kv_cache_precision" in cfg.explicitly_set:
        kw["kv_dtype"] = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[v["kv_cache_precision"]]
    elif v.get("kv_cache_precision") in ("q8_0", "q8_1"):
        from .engine.kv_cache import Q8
        kw["kv_dtype"] = Q8           # int8 values with an fp16 scale per 32 (the reference's q8_1 also stores block sums, which this layout does not need)
    if layout["pp"] > 1:
        from .parallel.pp import build_pipeline_engine
        engine = build_pipeline_engine(weights, layout, rank, **kw)
    else:
        engine = LLMEngine(weights, **kw)
    if v.get("moe_stats_out") and mcfg.is_moe and rank == 0:
        import atexit
        from .models.expert_placement import ExpertStats
        stats = ExpertStats(mcfg.n_layers, mcfg.n_experts)
        target = getattr(engine.model, "inner", engine.model)
        target.expert_stats = stats
        engine.use_graphs = False                      # the router hook reads the chosen experts on the host
        atexit.register(lambda: stats.dump(v["moe_stats_out"], mcfg.name))
    template = None
    if tok is not None:
        template = ChatTemplate.resolve(v.get("chat_template"), tok.chat_template,
                                        bos_token=tok.tokens[tok.bos_id] if tok.bos_id is not None else "",
                                        eos_token=tok.tokens[tok.eos_id] if tok.eos_id is not None else "")
    if rank == 0:
        log.info("engine ready in %.1f s on %s (world %d, tp %d, pp %d)", time.time() - t0, dev, world, layout["tp"], layout["pp"])
    return engine, tok, template, rank, world


def _fingerprint(mcfg, layout, v) -> str:
    return json.dumps({"model": mcfg.to_dict(), "tp": layout["tp"], "pp": layout["pp"], "kv": v.get("kv_cache_precision"),
                       "act": v.get("activation_precision"), "moe": v.get("moe_expert_mode"), "mtp": bool(v.get("mtp"))}, sort_keys=True)


def cli_sampling(cfg: OrchestrationConfig):
    from .engine.sampling import SamplingParams
    v = cfg.values
    return SamplingParams(temperature=v["temperature"], top_k=v["top_k"], top_p=v["top_p"], seed=v["seed"],
                          presence_penalty=v["presence_penalty"], frequency_penalty=v["frequency_penalty"],
                          max_tokens=v["n_predict"])


def _spmd(engine, rank, world):
    """(engine to drive on rank 0, worker entry for the others)."""
    if world == 1:
        return engine, None
    from .parallel.spmd import ControlChannel, ReplicatedEngine, worker_loop
    from .parallel.watchdog import Heartbeat, StepWatchdog, abort_process_group
    import torch.distributed as dist
    ch = ControlChannel()
    # failure detection: heartbeats through the rendezvous store; a dead or failed peer aborts the communicators so
    # that nobody stays blocked in a collective
    def peer_failed(r, why):
        log.error("rank %d reported dead or failed (%s); aborting the process group", r, why)
        abort_process_group()
    hb = Heartbeat(dist.distributed_c10d._get_default_store(), rank, world, on_failure=peer_failed).start()
    engine.heartbeat = hb
    engine.step_watchdog = StepWatchdog(heartbeat=hb)
    if rank == 0:
        return ReplicatedEngine(engine, ch), None
    return None, (lambda: worker_loop(engine, ch))


# ---------------------------------------------------------------------------------------------------------
# commands
# ---------------------------------------------------------------------------------------------------------
def cmd_oneshot(cfg: OrchestrationConfig) -> int:
    engine, tok, template, rank, world = build_engine(cfg)
    drive, worker = _spmd(engine, rank, world)
    if worker:
        worker()
        return 0
    v = cfg.values
    prompt = v.get("prompt") or "Hello"
    sp = cli_sampling(cfg)
    if tok is None:
        ids = [int(x) for x in prompt.split()] if prompt.replace(" ", "").isdigit() else [1, 2, 3]
    elif template is not None and not v.get("raw"):
        ids = tok.encode(template.render([{"role": "user", "content": prompt}]), add_special=True)
    else:
        ids = tok.encode(prompt, add_special=True)
    if tok is not None and tok.eos_id is not None:
        sp.stop_token_ids = (tok.eos_id,)
    t0 = time.perf_counter()
    req = drive.add_request(ids, sp)
    n_out = 0
    from .tokenizer.bpe import StreamDecoder
    dec = StreamDecoder(tok) if tok is not None else None
    t_first = None
    while req.state != "finished":
        for o in drive.step():
            if o.rid == req.rid and o.new_tokens:
                t_first = t_first or time.perf_counter()
                n_out += len(o.new_tokens)
                text = "".join(dec.push(t) for t in o.new_tokens) if dec else " ".join(map(str, o.new_tokens)) + " "
                sys.stdout.write(text)
                sys.stdout.flush()
    if dec:
        sys.stdout.write(dec.flush())
    t1 = time.perf_counter()
    sys.stdout.write("\n")
    log.info("prompt %d tok, ttft %.1f ms, %d tokens in %.2f s (%.1f tok/s)", len(ids), (t_first - t0) * 1e3, n_out,
             t1 - t0, n_out / max(t1 - (t_first or t0), 1e-9))
    if world > 1:
        drive.shutdown_workers()
    return 0


def cmd_chat(cfg: OrchestrationConfig) -> int:
    """Interactive multi-turn chat on the terminal: one line per user turn, `/reset` clears the history, `/exit` or
    end-of-input leaves (the reference's interactive mode is a full-screen TUI: src/v2/app/modes/InteractiveChatMode.cpp;
    this is its line-oriented equivalent)."""
    from .tokenizer.bpe import StreamDecoder
    from .tokenizer.chat_template import ThinkSplitter
    engine, tok, template, rank, world = build_engine(cfg)
    drive, worker = _spmd(engine, rank, world)
    if worker:
        worker()
        return 0
    if tok is None or template is None:
        raise ConfigError(["the checkpoint has no embedded tokenizer; `chat` needs tokenizer.ggml.* metadata"])
    v = cfg.values
    if v.get("tui"):
        from .tui import ChatSession, run
        session = ChatSession(drive, tok, template, v["ctx_size"], lambda: cli_sampling(cfg), v.get("system_prompt"))
        try:
            run(session, engine.cfg.name)
        finally:
            if world > 1:
                drive.shutdown_workers()
        return 0
    history: list[dict] = []
    if v.get("system_prompt"):
        history.append({"role": "system", "content": v["system_prompt"]})
    base = list(history)
    eos = tuple(i for i in (tok.eos_id, tok.vocab.get("<|im_end|>"), tok.vocab.get("<|endoftext|>")) if i is not None)
    while True:
        try:
            line = input("> ")
        except EOFError:
            break
        line = line.strip()
        if line in ("/exit", "/quit"):
            break
        if line == "/reset":
            history = list(base)
            drive.clear_cache()
            continue
        if not line:
            continue
        history.append({"role": "user", "content": line})
        ids = tok.encode(template.render(history), add_special=True)
        if len(ids) + 2 >= v["ctx_size"]:
            print("[context window exhausted; /reset to start over]")
            history.pop()
            continue
        sp = cli_sampling(cfg)
        sp.max_tokens = min(sp.max_tokens, v["ctx_size"] - len(ids) - 1)
        sp.stop_token_ids = tuple(dict.fromkeys(eos))
        req = drive.add_request(ids, sp)
        dec, split, answer = StreamDecoder(tok), ThinkSplitter(), []
        while req.state != "finished":
            for o in drive.step():
                if o.rid != req.rid:
                    continue
                for t in o.new_tokens:
                    _, content = split.push(dec.push(t))
                    if content:
                        answer.append(content)
                        sys.stdout.write(content)
                        sys.stdout.flush()
        _, content = split.push(dec.flush())
        tail = content + split.flush()[1]
        answer.append(tail)
        sys.stdout.write(tail + "\n")
        drive.requests.pop(req.rid, None)
        history.append({"role": "assistant", "content": "".join(answer)})
    if world > 1:
        drive.shutdown_workers()
    return 0


def cmd_serve(cfg: OrchestrationConfig) -> int:
    from .serve.chat_handler import ChatCompletionHandler
    from .serve.engine_loop import EngineLoop
    from .serve.server import Server
    engine, tok, template, rank, world = build_engine(cfg)
    drive, worker = _spmd(engine, rank, world)
    if worker:
        worker()
        return 0
    if tok is None or template is None:
        raise ConfigError(["the checkpoint has no embedded tokenizer; `serve` needs tokenizer.ggml.* metadata"])
    v = cfg.values
    loop = EngineLoop(drive)
    eos = tuple(i for i in (tok.eos_id, tok.vocab.get("<|im_end|>"), tok.vocab.get("<|endoftext|>")) if i is not None)
    chat = ChatCompletionHandler(loop, tok, template, engine.cfg.arch, v["ctx_size"], model_name=engine.cfg.name,
                                 cli_sampling=cli_sampling(cfg), eos_ids=tuple(dict.fromkeys(eos)))
    srv = Server(chat, v["host"], v["port"], verbose=v.get("verbose", False), api_key=v.get("api_key"))
    try:
        import resource
        rss = resource.getrusage(resource.RUSAGE_SELF).ru_maxrss / 1024
        log.info("[ServerReady] http://%s:%d  (max RSS %.0f MiB)", v["host"], srv.port, rss)
    except Exception:
        log.info("[ServerReady] http://%s:%d", v["host"], srv.port)
    try:
        srv.serve_forever()
    finally:
        if world > 1:
            drive.shutdown_workers()
    return 0


def run_benchmark(drive, vocab: int, prompt_tokens: int, decode_tokens: int, runs: int, batch: int = 1, is_cuda: bool = True,
                  shared_prefix: int = 0, keep_cache: bool = False) -> dict:
    """The reference protocol: built-in ~512-token prompt, 128 greedy decode tokens, 1 warm-up + N measured runs
    averaged, cache cleared between runs (reference: src/v2/utils/BenchmarkRunner.cpp:451-457, :1059-1065, :1125-1256)."""
    from .engine.sampling import SamplingParams
    g = torch.Generator().manual_seed(1234)
    common = torch.randint(0, vocab, (min(shared_prefix, prompt_tokens),), generator=g).tolist()
    def make_prompts():                         # a fresh unique tail per run: only the common prefix can hit the prefix cache
        return [common + torch.randint(0, vocab, (prompt_tokens - len(common),), generator=g).tolist() for _ in range(batch)]
    prompts = make_prompts()
    sp = SamplingParams(temperature=0.0, max_tokens=decode_tokens, ignore_eos=True)
    sync = (lambda: torch.cuda.synchronize()) if is_cuda else (lambda: None)
    res = []
    for run in range(runs + 1):
        if not keep_cache:                      # with keep_cache the prefix cache stays warm between runs
            drive.clear_cache()
        elif run > 0:
            prompts = make_prompts()
        sync()
        t0 = time.perf_counter()
        reqs = [drive.add_request(p, sp) for p in prompts]
        while any(not r.output for r in reqs):
            drive.step()
        sync()
        t1 = time.perf_counter()
        while any(r.state != "finished" for r in reqs):
            drive.step()
        sync()
        t2 = time.perf_counter()
        for r in reqs:
            drive.requests.pop(r.rid, None)
        if run > 0:
            res.append((t1 - t0, t2 - t1))
    pre = [batch * prompt_tokens / a for a, _ in res]
    dec = [batch * (decode_tokens - 1) / b for _, b in res]
    ttft = [a * 1e3 for a, _ in res]
    return {"prefill_tok_s": statistics.mean(pre), "decode_tok_s": statistics.mean(dec), "ttft_ms_p50": statistics.median(ttft),
            "runs": runs, "prompt_tokens": prompt_tokens, "decode_tokens": decode_tokens, "batch": batch}


def cmd_benchmark(cfg: OrchestrationConfig) -> int:
    engine, tok, template, rank, world = build_engine(cfg)
    drive, worker = _spmd(engine, rank, world)
    if worker:
        worker()
        return 0
    v = cfg.values
    out = run_benchmark(drive, engine.cfg.vocab_size, v["bench_prompt_tokens"], v["n_predict"], v["bench_runs"],
                        batch=v["batch_size"], is_cuda=engine.is_cuda, shared_prefix=v.get("bench_shared_prefix_tokens", 0),
                        keep_cache=bool(v.get("prefix_cache")) and v.get("bench_shared_prefix_tokens", 0) > 0)
    out.update(model=engine.cfg.name, world=world, stats={k: (round(x, 4) if isinstance(x, float) else x) for k, x in engine.stats.items()})
    if getattr(engine, "prefix_cache", None) is not None:
        out["prefix_cache"] = engine.prefix_cache.stats()
    if getattr(engine, "mtp", None) is not None:
        out["mtp"] = engine.mtp.stats()
    print(json.dumps(out, indent=2))
    if v.get("bench_json"):
        with open(v["bench_json"], "w") as f:
            json.dump(out, f, indent=2)
    if world > 1:
        drive.shutdown_workers()
    return 0


def cmd_plan(cfg: OrchestrationConfig) -> int:
    import yaml
    from .models.config import SHAPES, ModelConfig
    from .planning import build_plan
    v = cfg.values
    recipe = v.get("synthetic_recipe") or "Q4_K_M"
    if v.get("synthetic"):
        mcfg = SHAPES[v["synthetic"]]
    else:
        from .gguf import GGUFFile
        from .planning import FileRecipe
        gf = GGUFFile(v["model"])
        mcfg = ModelConfig.from_gguf(gf)
        recipe = FileRecipe(gf)                 # budget the formats the file really stores
        gf.close()
    if v.get("suggest_layout"):
        from .planning import suggest_layout
        layout, plan = suggest_layout(mcfg, int(v["suggest_layout"]), recipe, v["ctx_size"], v["batch_size"])
        if layout is None:
            for r in plan:
                print(f"error: {r}", file=sys.stderr)
            return 1
        flags = []
        if layout["pp"] == 1:
            flags = ["--tp-devices", ",".join(layout["stages"][0][1])] if layout["tp"] > 1 else ["-d", "cuda:0"]
        else:
            for name, devs, first, last in layout["stages"]:
                flags += ["--define-domain", f"{name}={','.join(devs)}"]
            for i, (name, devs, first, last) in enumerate(layout["stages"]):
                flags += ["--pp-stage", f"{i}={name}:{first}-{last}"]
        print(f"suggested layout: pp={layout['pp']} x tp={layout['tp']} on {layout['world']} device(s)")
        print("flags: " + " ".join(flags))
    else:
        plan = build_plan(mcfg, cfg.layout(), recipe, v["ctx_size"], v["batch_size"])
    print(plan.table())
    print(yaml.safe_dump(plan.to_dict(), sort_keys=False))
    return 1 if plan.errors else 0


def cmd_describe(cfg: OrchestrationConfig) -> int:
    if cfg.values.get("env"):
        from .utils.env import debug_env
        print(debug_env().describe())
        return 0
    from .utils.devices import benchmark_devices, describe_devices
    out = describe_devices()
    if cfg.values.get("device_benchmark"):
        out["benchmark"] = benchmark_devices()
    print(json.dumps(out, indent=2))
    return 0


def print_help() -> None:
    print("usage: python -m llaminar_b200 {oneshot|chat|serve|benchmark|plan|describe} [options]\n")
    for cat, opts in help_by_category().items():
        print(f"[{cat}]")
        for o in opts:
            tag = " (accepted, ignored)" if o.deprecated else (" (not supported on this build)" if o.unsupported else "")
            default = "" if o.default in (None, False, []) else f" [default: {o.default}]"
            print(f"  {', '.join(o.flags):34s} {o.help}{default}{tag}")
        print()


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help", "help"):
        print_help()
        return 0
    try:
        cfg = parse_args(argv)
    except ConfigError as exc:
        for e in exc.errors:
            print(f"error: {e}", file=sys.stderr)
        return 2
    v = cfg.values
    if v.get("list_devices"):
        return cmd_describe(cfg)
    if v.get("dry_run") or v.get("explain_placement") or v.get("validate_only"):
        if v.get("validate_only") and not (v.get("model") or v.get("synthetic")):
            print("configuration is valid")
            return 0
        return cmd_plan(cfg)
    rc = maybe_relaunch(cfg, argv)
    if rc is not None:
        return rc
    try:
        return {"oneshot": cmd_oneshot, "chat": cmd_chat, "serve": cmd_serve, "benchmark": cmd_benchmark, "plan": cmd_plan,
                "describe": cmd_describe}[cfg.command](cfg)
    except ConfigError as exc:
        for e in exc.errors:
            print(f"error: {e}", file=sys.stderr)
        return 2
