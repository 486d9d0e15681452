"""Command-line / YAML configuration: the declarative option table, the parsed `OrchestrationConfig`,
domain and pipeline-stage definitions, and the validation rules between the device-selection modes.

The flag names, defaults and mutual-exclusion rules follow the reference's CLI (reference:
src/v2/config/OrchestrationConfigParser.cpp:890-2130 option table, src/v2/config/OrchestrationConfig.h:129-229
`DomainDefinition` / `PPStageDefinition`, src/v2/config/ConfigValidator.cpp:225-436).  Options that only make
sense for the reference's CPU / ROCm / MPI back ends are accepted and reported as not supported on this build.
"""
from __future__ import annotations

import argparse
import re
from dataclasses import dataclass, field
from typing import Any

SUBCOMMANDS = ("oneshot", "chat", "serve", "benchmark", "plan", "describe")


@dataclass
class OptionSpec:
    flags: tuple[str, ...]
    dest: str
    type: Any = str
    default: Any = None
    help: str = ""
    category: str = "general"
    choices: tuple | None = None
    action: str | None = None           # "store_true" / "append"
    deprecated: bool = False            # accepted, ignored (kept so old command lines keep working)
    unsupported: str | None = None      # accepted; raises at validation time with this reason when set by the user


def _o(*flags, **kw) -> OptionSpec:
    dest = kw.pop("dest", None) or flags[-1].lstrip("-").replace("-", "_")
    return OptionSpec(tuple(flags), dest, **kw)


OPTIONS: list[OptionSpec] = [
    # -- model / general ------------------------------------------------------------------------------------
    _o("-m", "--model", help="path to the .gguf checkpoint (first part of a split checkpoint)", category="model"),
    _o("-c", "--ctx-size", dest="ctx_size", type=int, default=4096, help="context window in tokens", category="model"),
    _o("--batch-size", type=int, default=1, help="concurrent request lanes (decode batch)", category="model"),
    _o("-p", "--prompt", help="prompt text (oneshot)", category="model"),
    _o("-n", "--n-predict", dest="n_predict", type=int, default=128, help="tokens to generate", category="model"),
    _o("--config", help="YAML file with base values; command-line flags override it", category="general"),
    _o("--chat-template", help="override the checkpoint's chat template (Jinja file or built-in name)", category="model"),
    _o("--synthetic", help="use a random-init model of this shape instead of -m (e.g. tiny-qwen3, qwen3-8b)", category="model"),
    _o("--synthetic-recipe", default="Q4_K_M", help="quantisation recipe of --synthetic", category="model"),
    # -- server ---------------------------------------------------------------------------------------------
    _o("--host", default="127.0.0.1", help="HTTP bind address", category="server"),
    _o("--port", type=int, default=8080, help="HTTP port", category="server"),
    _o("--api-key", default=None, help="serve: require `Authorization: Bearer <key>` on the /v1 endpoints", category="server"),
    # -- sampling -------------------------------------------------------------------------------------------
    _o("-t", "--temperature", dest="temperature", type=float, default=0.8, category="sampling"),
    _o("--top-k", type=int, default=40, category="sampling"),
    _o("--top-p", type=float, default=0.9, category="sampling"),
    _o("-s", "--seed", dest="seed", type=int, default=None, category="sampling"),
    _o("--presence-penalty", type=float, default=0.0, category="sampling"),
    _o("--frequency-penalty", type=float, default=0.0, category="sampling"),
    # -- devices / parallelism ------------------------------------------------------------------------------
    _o("-d", "--device", dest="device", help="single device: cuda:N or cpu", category="devices"),
    _o("-tp", "--tensor-parallel", dest="tp", type=int, default=None, help="tensor-parallel degree over cuda:0..tp-1", category="devices"),
    _o("--tp-devices", help="comma-separated devices of one tensor-parallel group, e.g. cuda:0,cuda:1", category="devices"),
    _o("--tp-weights", help="proportional split weights for --tp-devices", category="devices",
       unsupported="heterogeneous proportional splits are not built (homogeneous B200 ranks only)"),
    _o("--define-domain", action="append", default=[], help="name=dev,dev[;backend=nccl] : a named tensor-parallel domain", category="devices"),
    _o("--pp-stage", action="append", default=[], help="id=domain:first-last : a pipeline stage (layer range on a domain)", category="devices"),
    _o("--device-map", category="devices", help='explicit rank -> device mapping of one tensor-parallel group, e.g. "0=cuda:0,1=cuda:1"'),
    _o("--topology", category="devices",
       help='parallelism tree, e.g. "PP(global, TP(a, cuda:0, cuda:1), TP(b, cuda:2, cuda:3))" or "TP(g, cuda:0, cuda:1)"; layers are split evenly'),
    _o("--topology-file", category="devices", help="YAML file with a `topology:` tree (type pp/tp, name, children / devices)"),
    _o("--backend", default="auto", choices=("auto", "nccl", "fused", "gloo", "mpi", "rccl", "host"),
       help="collective backend: fused = in-kernel NVLink collectives (default on GPU), nccl = library baseline", category="devices"),
    _o("--list-devices", action="store_true", category="devices"),
    _o("--dry-run", action="store_true", help="plan and validate, then exit", category="devices"),
    _o("--explain-placement", action="store_true", category="devices"),
    _o("--env", action="store_true", category="debug", help="describe: list the LLAMINAR_* environment switches instead of the devices"),
    _o("--device-benchmark", action="store_true", category="debug",
       help="describe: also measure every device (copy bandwidth, bf16 matrix throughput, peer-to-peer copy bandwidth)"),
    _o("--validate-only", action="store_true", category="devices"),
    _o("--suggest-layout", type=int, default=None, category="devices",
       help="plan: find the smallest pp x tp placement on up to N GPUs that fits their memory and print its flags"),
    # -- precision ------------------------------------------------------------------------------------------
    _o("--activation-precision", default="bf16", choices=("bf16", "fp32", "fp16"), category="precision"),
    _o("--kv-cache-precision", default="bf16", choices=("bf16", "fp16", "fp32", "q8_0", "q8_1", "tq4", "tq8"), category="precision"),
    # -- MoE ------------------------------------------------------------------------------------------------
    _o("--moe-expert-mode", default="expert-parallel", choices=("expert-parallel", "expert-parallel-a2a", "tensor-parallel", "replicated"), category="moe"),
    _o("--moe-overlay", category="moe", unsupported="CPU/GPU expert overlay tiers are not built"),
    _o("--moe-rebalance", action="store_true", category="moe",
       unsupported="experts are not moved while serving; measure with --moe-stats-out and place them with --moe-expert-placement"),
    _o("--moe-stats-out", category="moe", help="write per-layer router statistics (tokens per expert) to this JSON file at exit"),
    _o("--moe-expert-placement", category="moe",
       help="statistics file of --moe-stats-out: renumber every layer's experts so that the expert-parallel ranks carry balanced load"),
    # -- prefix cache ---------------------------------------------------------------------------------------
    _o("--prefix-cache", action="store_true", category="prefix-cache"),
    _o("--prefix-cache-storage", default="tiered", choices=("ram", "device", "tiered"), category="prefix-cache"),
    _o("--prefix-cache-block-size", type=int, default=64, category="prefix-cache"),
    _o("--prefix-cache-vram-budget-mb", type=int, default=256, category="prefix-cache"),
    _o("--prefix-cache-ram-budget-mb", type=int, default=4096, category="prefix-cache"),
    _o("--prefix-cache-disk-budget-mb", type=int, default=0, category="prefix-cache"),
    _o("--prefix-cache-disk-dir", category="prefix-cache"),
    _o("--prefix-cache-terminal-state", default="auto", choices=("off", "auto", "always"), category="prefix-cache"),
    _o("--prefix-cache-state-stride", type=int, default=0, category="prefix-cache",
       help="hybrid models: also snapshot the recurrent state every N prompt tokens (a multiple of the block size; 0 = only at "
            "the last block boundary of a prompt), so that prompts sharing a shorter prefix can resume from it"),
    _o("--prefix-cache-moe-policy", default="placement-fingerprint",
       choices=("disabled", "placement-fingerprint", "invalidate-on-rebalance"), category="prefix-cache"),
    # -- MTP / speculative decode -----------------------------------------------------------------------------
    _o("--mtp", action="store_true", category="mtp"),
    _o("--mtp-draft-tokens", type=int, default=1, category="mtp"),
    _o("--mtp-verify-mode", default="greedy", choices=("greedy", "speculative-sampling"), category="mtp"),
    _o("--mtp-depth-policy", default="fixed", choices=("fixed", "observe", "dynamic"), category="mtp"),
    _o("--mtp-depth-window", type=int, default=16, category="mtp"),
    _o("--mtp-depth-min-samples", type=int, default=4, category="mtp"),
    _o("--mtp-depth-cooldown", type=int, default=8, category="mtp"),
    _o("--mtp-depth-promote-windows", type=int, default=3, category="mtp"),
    _o("--mtp-depth-demote-zero-accept", type=float, default=0.30, category="mtp"),
    _o("--mtp-depth-demote-acceptance", type=float, default=0.55, category="mtp"),
    _o("--mtp-force-accept", action="store_true", help="benchmark aid: treat every draft as accepted (random weights)", category="mtp"),
    # -- benchmark ------------------------------------------------------------------------------------------
    _o("--bench-runs", type=int, default=3, category="benchmark"),
    _o("--tui", action="store_true", help="chat: full-screen interface (scroll-back, input history, status bar)", category="generation"),
    _o("--system-prompt", default=None, help="system message of `chat` / `oneshot`", category="generation"),
    _o("--bench-prompt-tokens", type=int, default=512, category="benchmark"),
    _o("--bench-shared-prefix-tokens", type=int, default=0, help="the first N prompt tokens are common to all requests of the batch", category="benchmark"),
    _o("--bench-json", help="write the benchmark result JSON here", category="benchmark"),
    # -- debugging --------------------------------------------------------------------------------------------
    _o("-v", "--verbose", dest="verbose", action="store_true", category="debug"),
    _o("--debug-dump", help="directory for per-layer tensor dumps", category="debug"),
    _o("--check-collectives", action="store_true", help="hash and compare the collective sequence across ranks", category="debug"),
    # -- accepted for compatibility, ignored --------------------------------------------------------------------
    _o("--no-mpi-bootstrap", action="store_true", deprecated=True),
    _o("--threads", type=int, deprecated=True),
    _o("--numa", deprecated=True),
    _o("--mlock", action="store_true", deprecated=True),
    _o("--no-mmap", action="store_true", deprecated=True),
]

_DEVICE_RE = re.compile(r"^(cuda:\d+|cpu(:\d+)?|rocm:\d+)$")


@dataclass
class DomainDefinition:
    """``name=dev,dev[;weights=..][;backend=..][;scope=..][;owner=..][;ranks=..]``"""
    name: str
    devices: list[str]
    backend: str = "auto"
    weights: list[float] | None = None
    scope: str = "local"
    extras: dict = field(default_factory=dict)

    @staticmethod
    def parse(text: str) -> "DomainDefinition":
        if "=" not in text:
            raise ValueError(f"--define-domain '{text}': expected name=dev,dev[;key=value]")
        name, rest = text.split("=", 1)
        parts = rest.split(";")
        devices = [d.strip() for d in parts[0].split(",") if d.strip()]
        if not name.strip() or not devices:
            raise ValueError(f"--define-domain '{text}': empty name or device list")
        for d in devices:
            if not _DEVICE_RE.match(d):
                raise ValueError(f"--define-domain '{text}': bad device '{d}'")
        dom = DomainDefinition(name.strip(), devices)
        for kv in parts[1:]:
            if not kv.strip():
                continue
            if "=" not in kv:
                raise ValueError(f"--define-domain '{text}': bad option '{kv}'")
            k, v = (s.strip() for s in kv.split("=", 1))
            if k == "backend":
                dom.backend = v
            elif k == "weights":
                dom.weights = [float(x) for x in v.split(",")]
            elif k == "scope":
                dom.scope = v
            elif k in ("owner", "ranks"):
                dom.extras[k] = v
            else:
                raise ValueError(f"--define-domain '{text}': unknown key '{k}'")
        return dom


@dataclass
class PPStageDefinition:
    """``id=domain:first-last`` (inclusive layer range)"""
    stage_id: int
    domain: str
    first_layer: int
    last_layer: int

    @staticmethod
    def parse(text: str) -> "PPStageDefinition":
        m = re.match(r"^\s*(\d+)\s*=\s*([\w.-]+)\s*:\s*(\d+)\s*-\s*(\d+)\s*$", text)
        if not m:
            raise ValueError(f"--pp-stage '{text}': expected id=domain:first-last")
        sid, dom, a, b = int(m.group(1)), m.group(2), int(m.group(3)), int(m.group(4))
        if b < a:
            raise ValueError(f"--pp-stage '{text}': last layer before first layer")
        return PPStageDefinition(sid, dom, a, b)


def parse_device_map(text: str) -> list[str]:
    """``rank=device,...`` -> devices in rank order (reference: --device-map, src/v2/config/OrchestrationConfigParser.cpp:1190).
    Ranks must be 0..n-1 without gaps; the ranks form one tensor-parallel group, rank r on the r-th device."""
    pairs = {}
    for item in text.split(","):
        m = re.match(r"^\s*(\d+)\s*=\s*([\w:.-]+)\s*$", item)
        if not m:
            raise ValueError(f"--device-map '{text}': expected rank=device, got '{item.strip()}'")
        r = int(m.group(1))
        if r in pairs:
            raise ValueError(f"--device-map '{text}': rank {r} appears twice")
        pairs[r] = m.group(2)
    if sorted(pairs) != list(range(len(pairs))):
        raise ValueError(f"--device-map '{text}': ranks must be 0..{len(pairs) - 1} without gaps")
    return [pairs[r] for r in range(len(pairs))]


def _topology_tokens(text: str) -> list[str]:
    return re.findall(r"[A-Za-z_][\w.:-]*|[(),]", text)


def parse_topology(text: str) -> dict:
    """``KIND(name, child, ...)`` with KIND in {PP, TP} and children either nested nodes or devices -> a tree of dicts
    {'type', 'name', 'children' | 'devices'} (the form the YAML file has).  Reference syntax:
    src/v2/config/ParallelismTreeParser.h:25-28 (the reference parses the tree but does not run it yet)."""
    toks = _topology_tokens(text)
    if "".join(toks) != re.sub(r"\s+", "", text):
        raise ValueError(f"--topology '{text}': unexpected characters")
    pos = 0

    def node() -> dict:
        nonlocal pos
        kind = toks[pos].lower() if pos < len(toks) else ""
        if kind not in ("pp", "tp") or pos + 1 >= len(toks) or toks[pos + 1] != "(":
            raise ValueError(f"--topology '{text}': expected PP(...) or TP(...) at token {pos}")
        pos += 2
        if pos >= len(toks) or toks[pos] in "(),":
            raise ValueError(f"--topology '{text}': a node needs a name")
        out = {"type": kind, "name": toks[pos], "children": [], "devices": []}
        pos += 1
        while pos < len(toks) and toks[pos] == ",":
            pos += 1
            if pos + 1 < len(toks) and toks[pos + 1] == "(":
                out["children"].append(node())
            elif pos < len(toks) and toks[pos] not in "(),":
                out["devices"].append(toks[pos])
                pos += 1
            else:
                raise ValueError(f"--topology '{text}': dangling ','")
        if pos >= len(toks) or toks[pos] != ")":
            raise ValueError(f"--topology '{text}': missing ')'")
        pos += 1
        return out

    tree = node()
    if pos != len(toks):
        raise ValueError(f"--topology '{text}': trailing input after the root node")
    return tree


def topology_to_layout(tree: dict) -> tuple[list["DomainDefinition"], list["PPStageDefinition"]]:
    """Domains and pipeline stages of a parallelism tree.  A TP root is one domain; a PP root has one stage per child
    (a TP node, or a bare device = a stage of one GPU).  Stages carry no layer ranges: the layers are split evenly."""
    kind = str(tree.get("type", "")).lower()
    if kind == "tp":
        if tree.get("children"):
            raise ValueError(f"topology node '{tree.get('name')}': a TP node holds devices, not nodes")
        devs = [str(d) for d in tree.get("devices") or []]
        if not devs:
            raise ValueError(f"topology node '{tree.get('name')}': a TP node needs devices")
        dom = DomainDefinition(str(tree["name"]), devs)
        if tree.get("backend"):
            dom.backend = str(tree["backend"])
        return [dom], []
    if kind != "pp":
        raise ValueError(f"topology node '{tree.get('name')}': type must be pp or tp")
    domains, stages = [], []
    kids = list(tree.get("children") or []) + [{"type": "tp", "name": f"{tree['name']}_{d.replace(':', '')}", "devices": [d]}
                                               for d in tree.get("devices") or []]
    if not kids:
        raise ValueError(f"topology node '{tree.get('name')}': a PP node needs stages")
    kids.sort(key=lambda k: k.get("rank", 0))                 # the YAML form may give explicit stage ranks; stable otherwise
    for i, k in enumerate(kids):
        if str(k.get("type", "")).lower() != "tp":
            raise ValueError(f"topology node '{k.get('name')}': stages of a PP node must be TP nodes or devices")
        d, _ = topology_to_layout(k)
        domains += d
        stages.append(PPStageDefinition(i, d[0].name, -1, -1))
    return domains, stages


@dataclass
class OrchestrationConfig:
    command: str = "oneshot"
    values: dict = field(default_factory=dict)
    explicitly_set: set = field(default_factory=set)
    domains: list[DomainDefinition] = field(default_factory=list)
    pp_stages: list[PPStageDefinition] = field(default_factory=list)

    def __getattr__(self, name):
        vals = self.__dict__.get("values", {})
        if name in vals:
            return vals[name]
        raise AttributeError(name)

    # -- derived layout -------------------------------------------------------------------------------------
    def tp_devices_list(self) -> list[str]:
        v = self.values
        if v.get("device_map"):
            return parse_device_map(v["device_map"])
        if v.get("tp_devices"):
            return [d.strip() for d in v["tp_devices"].split(",") if d.strip()]
        if v.get("tp"):
            return [f"cuda:{i}" for i in range(int(v["tp"]))]
        if v.get("device"):
            return [v["device"]]
        return []

    def layout(self) -> dict:
        """{'pp': n_stages, 'tp': ranks per stage, 'stages': [(domain, devices, first, last)], 'world': n}"""
        if self.pp_stages:
            doms = {d.name: d for d in self.domains}
            stages = []
            for st in sorted(self.pp_stages, key=lambda s: s.stage_id):
                stages.append((st.domain, doms[st.domain].devices, st.first_layer, st.last_layer))
            tp = len(stages[0][1])
            return {"pp": len(stages), "tp": tp, "stages": stages, "world": sum(len(s[1]) for s in stages)}
        if self.domains:
            d = self.domains[0]
            return {"pp": 1, "tp": len(d.devices), "stages": [(d.name, d.devices, 0, -1)], "world": len(d.devices)}
        devs = self.tp_devices_list() or ["cuda:0"]
        return {"pp": 1, "tp": len(devs), "stages": [("default", devs, 0, -1)], "world": len(devs)}


class ConfigError(ValueError):
    def __init__(self, errors: list[str]):
        super().__init__("; ".join(errors))
        self.errors = errors


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="llaminar_b200", add_help=True, allow_abbrev=False,
                                 description="Blackwell-native GGUF inference engine (oneshot | chat | serve | benchmark | plan | describe)")
    ap.add_argument("command", nargs="?", default="oneshot", choices=SUBCOMMANDS)
    groups: dict[str, Any] = {}
    for o in OPTIONS:
        g = groups.setdefault(o.category, ap.add_argument_group(o.category))
        kw: dict[str, Any] = {"dest": o.dest, "help": o.help or None, "default": argparse.SUPPRESS}
        if o.action == "store_true":
            kw["action"] = "store_true"
        elif o.action == "append":
            kw["action"] = "append"
            kw["type"] = o.type
        else:
            kw["type"] = o.type
            if o.choices:
                kw["choices"] = o.choices
        g.add_argument(*o.flags, **kw)
    return ap


def _load_yaml(path: str) -> dict:
    import yaml
    with open(path) as f:
        data = yaml.safe_load(f) or {}
    if not isinstance(data, dict):
        raise ConfigError([f"--config {path}: top level must be a mapping"])
    return {str(k).replace("-", "_"): v for k, v in data.items()}


def parse_args(argv: list[str]) -> OrchestrationConfig:
    ns = build_parser().parse_args(argv)
    given = dict(vars(ns))
    command = given.pop("command")
    values = {o.dest: (list(o.default) if isinstance(o.default, list) else o.default)
              for o in OPTIONS if o.action != "store_true"}
    values.update({o.dest: False for o in OPTIONS if o.action == "store_true"})
    explicitly = set()
    if given.get("config"):
        base = _load_yaml(given["config"])
        known = {o.dest for o in OPTIONS}
        unknown = [k for k in base if k not in known]
        if unknown:
            raise ConfigError([f"--config: unknown keys {unknown}"])
        values.update(base)
        explicitly |= set(base)
    values.update(given)
    explicitly |= set(given)
    cfg = OrchestrationConfig(command, values, explicitly)
    try:
        cfg.domains = [DomainDefinition.parse(t) for t in values.get("define_domain") or []]
        cfg.pp_stages = [PPStageDefinition.parse(t) for t in values.get("pp_stage") or []]
        if values.get("device_map"):
            parse_device_map(values["device_map"])
        tree = None
        if values.get("topology"):
            tree = parse_topology(values["topology"])
        elif values.get("topology_file"):
            doc = _load_yaml(values["topology_file"])
            tree = doc.get("topology", doc)
        if tree is not None:
            if cfg.domains or cfg.pp_stages:
                raise ValueError("--topology cannot be combined with --define-domain / --pp-stage")
            cfg.domains, cfg.pp_stages = topology_to_layout(tree)
    except ValueError as exc:
        raise ConfigError([str(exc)]) from exc
    errors = validate(cfg)
    if errors:
        raise ConfigError(errors)
    return cfg


def validate(cfg: OrchestrationConfig) -> list[str]:
    """Rules between the device-selection modes and co-requirements of the other flags."""
    v, ex = cfg.values, cfg.explicitly_set
    errs: list[str] = []
    modes = [name for name, on in (("-d", "device" in ex), ("-tp", "tp" in ex), ("--tp-devices", "tp_devices" in ex),
                                   ("--define-domain", bool(cfg.domains) and not ({"topology", "topology_file"} & ex)),
                                   ("--device-map", "device_map" in ex), ("--topology", "topology" in ex),
                                   ("--topology-file", "topology_file" in ex)) if on]
    if len(modes) > 1 and not (set(modes) == {"--define-domain"}):
        errs.append(f"device selection flags are mutually exclusive, got {' and '.join(modes)}")
    for o in OPTIONS:
        if o.unsupported and o.dest in ex:
            errs.append(f"{o.flags[-1]}: not supported on this build ({o.unsupported})")
    if cfg.pp_stages and not cfg.domains:
        errs.append("--pp-stage needs the domains it names (--define-domain)")
    if cfg.pp_stages:
        names = {d.name for d in cfg.domains}
        ids = [s.stage_id for s in cfg.pp_stages]
        if sorted(ids) != list(range(len(ids))):
            errs.append(f"--pp-stage ids must be 0..{len(ids) - 1} without gaps, got {sorted(ids)}")
        for s in cfg.pp_stages:
            if s.domain not in names:
                errs.append(f"--pp-stage {s.stage_id}: unknown domain '{s.domain}'")
        st = sorted(cfg.pp_stages, key=lambda s: s.stage_id)
        implicit = all(s.last_layer < 0 for s in st)          # stages of a topology tree: layers are split evenly
        for a, b in zip(st, st[1:]):
            if not implicit and b.first_layer != a.last_layer + 1:
                errs.append(f"--pp-stage {b.stage_id}: layers must continue at {a.last_layer + 1}, got {b.first_layer}")
        if st and not implicit and st[0].first_layer != 0:
            errs.append("--pp-stage 0 must start at layer 0")
        sizes = {len(d.devices) for d in cfg.domains if d.name in {s.domain for s in cfg.pp_stages}}
        if len(sizes) > 1:
            errs.append("all pipeline stages must have the same tensor-parallel degree")
        used = [dev for d in cfg.domains for dev in d.devices]
        if len(used) != len(set(used)):
            errs.append("a device appears in more than one domain")
    if len({d.name for d in cfg.domains}) != len(cfg.domains):
        errs.append("duplicate domain name")
    for dev in cfg.tp_devices_list():
        if not _DEVICE_RE.match(dev):
            errs.append(f"bad device '{dev}' (expected cuda:N or cpu)")
        elif dev.startswith("rocm"):
            errs.append(f"device '{dev}': ROCm devices are not supported on this build")
    devs = cfg.tp_devices_list()
    if len(devs) != len(set(devs)):
        errs.append("--tp-devices lists a device twice")
    if v.get("tp") is not None and int(v["tp"]) < 1:
        errs.append("-tp must be >= 1")
    if v.get("backend") in ("mpi", "rccl", "host"):
        errs.append(f"--backend {v['backend']}: not supported on this build (NCCL / fused NVLink / gloo only)")
    on_cpu = str(v.get("device") or "").startswith("cpu") or (cfg.tp_devices_list() and all(d.startswith("cpu") for d in cfg.tp_devices_list())) \
        or (cfg.domains and all(dev.startswith("cpu") for d in cfg.domains for dev in d.devices))
    if not on_cpu and v.get("kv_cache_precision") in ("fp16", "fp32") and "kv_cache_precision" in ex:
        errs.append(f"--kv-cache-precision {v['kv_cache_precision']}: the CUDA kernels keep the KV cache in bf16 (fp16 / fp32 are available with -d cpu)")
    if not on_cpu and v.get("activation_precision") in ("fp16", "fp32") and "activation_precision" in ex:
        errs.append(f"--activation-precision {v['activation_precision']}: the CUDA path uses bf16 GEMM operands with an fp32 residual stream (fp32 is available with -d cpu)")
    if v.get("kv_cache_precision") in ("tq4", "tq8"):
        errs.append(f"--kv-cache-precision {v['kv_cache_precision']}: the turbo-quantised KV caches are not built (bf16 / q8_0 on GPUs, bf16 / fp16 / fp32 with -d cpu)")
    if on_cpu and v.get("kv_cache_precision") in ("q8_0", "q8_1"):
        errs.append(f"--kv-cache-precision {v['kv_cache_precision']}: the 8-bit KV cache is a CUDA feature (bf16 / fp16 / fp32 with -d cpu)")
    if not 1 <= int(v.get("mtp_draft_tokens") or 1) <= 3:
        errs.append("--mtp-draft-tokens must be between 1 and 3")
    if int(v.get("prefix_cache_block_size") or 64) % 64:
        errs.append("--prefix-cache-block-size must be a multiple of 64 (the KV page size)")
    if v.get("prefix_cache_disk_budget_mb") and not v.get("prefix_cache_disk_dir"):
        errs.append("--prefix-cache-disk-budget-mb needs --prefix-cache-disk-dir")
    if int(v.get("batch_size") or 1) < 1 or int(v.get("ctx_size") or 1) < 16:
        errs.append("--batch-size must be >= 1 and -c >= 16")
    if cfg.command in ("oneshot", "chat", "serve", "benchmark") and not (v.get("model") or v.get("synthetic")) \
            and not (v.get("dry_run") or v.get("list_devices") or v.get("validate_only")):
        errs.append("a model is required (-m file.gguf, or --synthetic SHAPE)")
    return errs


def help_by_category() -> dict[str, list[OptionSpec]]:
    out: dict[str, list[OptionSpec]] = {}
    for o in OPTIONS:
        out.setdefault(o.category, []).append(o)
    return out
