"""Placement and memory planning: which rank holds what, and whether it fits.

A deterministic function of (model config, layout, limits), so `plan` / `--dry-run` / `--explain-placement`
need no devices (reference: src/v2/execution/mpi_orchestration/ExecutionPlanBuilder.cpp, src/v2/planning/*.cpp,
`validateMemoryPlan` src/v2/execution/runner/OrchestrationRunner.cpp:12310).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field

from .gguf.constants import BLOCK_GEOMETRY, GGMLType
from .models.config import RECIPES, ModelConfig, QuantRecipe
from .parallel.tp_plan import TPPlan

B200_HBM_BYTES = 180 * 10 ** 9


def _bytes(qt: GGMLType, n: int, expert: bool = False) -> float:
    """Device-resident bytes of ``n`` weights stored as ``qt`` in the file: formats with a packed device layout stay as
    they are, the other block formats are re-encoded as Q8_0 at load, and unquantised tensors become bf16."""
    from .ops.layout import FMT_IDS
    if qt in (GGMLType.F32, GGMLType.F16, GGMLType.BF16):
        return n * 2.0
    if qt not in FMT_IDS:
        qt = GGMLType.Q8_0
    e, b = BLOCK_GEOMETRY[qt]
    return n / e * b


class FileRecipe:
    """The formats a parsed checkpoint really stores, in the shape of a quantisation recipe: the planner then budgets
    the file that will be loaded instead of a nominal recipe (the reference's estimator reads the tensor types from the
    GGUF header the same way; reference: src/v2/planning/WeightMemoryEstimator.cpp)."""

    def __init__(self, gguf_file=None, entries=None):
        """``gguf_file``: a parsed GGUFFile; or ``entries``: (name, qtype, n_dims, n_bytes) tuples."""
        if entries is None:
            entries = [(t.name, t.qtype, len(t.shape), t.nbytes) for t in gguf_file]
        self.types = {name: qt for name, qt, _, _ in entries}
        counts: dict = {}
        for _, qt, nd, nb in entries:
            if nd >= 2:
                counts[qt] = counts.get(qt, 0) + nb
        self.default = max(counts, key=counts.get) if counts else GGMLType.Q8_0
        self.name = f"file ({self.default.name} mostly)"

    @staticmethod
    def from_weights(weights) -> "FileRecipe":
        """The same view of weights that are already loaded (or synthesised)."""
        return FileRecipe(entries=[(n, t.qtype, len(t.shape), t.raw.numel()) for n, t in weights.tensors.items()])

    def for_tensor(self, tensor_name: str, layer: int | None = None, n_layers: int = 0) -> GGMLType:
        qt = self.types.get(tensor_name)
        if qt is None and tensor_name == "output.weight":          # tied head
            qt = self.types.get("token_embd.weight")
        return qt if qt is not None else self.default


@dataclass
class RankPlan:
    rank: int
    device: str
    stage: int
    tp_rank: int
    first_layer: int
    last_layer: int
    has_embedding: bool
    has_head: bool
    tp: dict
    weight_bytes: int = 0
    kv_bytes: int = 0
    activation_bytes: int = 0
    workspace_bytes: int = 0

    @property
    def total_bytes(self) -> int:
        return self.weight_bytes + self.kv_bytes + self.activation_bytes + self.workspace_bytes


@dataclass
class ExecutionPlan:
    model: str
    layout: dict
    ranks: list[RankPlan] = field(default_factory=list)
    errors: list[str] = field(default_factory=list)

    def to_dict(self) -> dict:
        return {"model": self.model, "pp": self.layout["pp"], "tp": self.layout["tp"], "world": self.layout["world"],
                "ranks": [dict(asdict(r), total_bytes=r.total_bytes) for r in self.ranks], "errors": self.errors}

    def table(self) -> str:
        rows = [f"{'rank':>4} {'device':>8} {'stage':>5} {'layers':>9} {'weights':>10} {'kv':>10} {'act+ws':>10} {'total':>10}"]
        gb = lambda x: f"{x / 1e9:8.2f}GB"
        for r in self.ranks:
            rows.append(f"{r.rank:>4} {r.device:>8} {r.stage:>5} {r.first_layer:>4}-{r.last_layer:<4} {gb(r.weight_bytes)} "
                        f"{gb(r.kv_bytes)} {gb(r.activation_bytes + r.workspace_bytes)} {gb(r.total_bytes)}")
        return "\n".join(rows)


def layer_weight_bytes(cfg: ModelConfig, recipe: QuantRecipe, layer: int, tp: TPPlan) -> float:
    d, D = cfg.d_model, cfg.head_dim
    t = lambda name: recipe.for_tensor(f"blk.{layer}.{name}.weight", layer, cfg.n_layers)
    if cfg.is_gdn_layer(layer):
        # linear-attention block: q | k of every key head, this rank's value heads of v and z, alpha / b, output projection
        nv, ds = tp.gdn_v_stop - tp.gdn_v_start, cfg.ssm_state
        tot = _bytes(t("attn_qkv"), (2 * cfg.gdn_key_dim + nv * ds) * d) + _bytes(t("attn_gate"), nv * ds * d)
        tot += 2 * _bytes(t("ssm_alpha"), nv * d) + _bytes(t("ssm_out"), d * nv * ds)
        tot += 4 * (2 * cfg.gdn_key_dim + nv * ds) * cfg.ssm_conv_kernel
    else:
        tot = _bytes(t("attn_q"), tp.n_heads_local * D * d * (2 if cfg.attn_gate else 1)) + 2 * _bytes(t("attn_k"), tp.n_kv_local * D * d)
        tot += _bytes(t("attn_output"), d * tp.n_heads_local * D)
    if cfg.is_moe:
        n_e = tp.expert_stop - tp.expert_start
        tot += n_e * (2 * _bytes(t("ffn_gate_exps"), cfg.expert_ff * d, True) + _bytes(t("ffn_down_exps"), cfg.expert_ff * d, True))
        tot += 2 * cfg.n_experts * d
        if cfg.shared_expert_ff:            # replicated on every rank
            tot += 2 * _bytes(t("ffn_gate_shexp"), cfg.shared_expert_ff * d) + _bytes(t("ffn_down_shexp"), cfg.shared_expert_ff * d)
    else:
        ff = tp.ff_stop - tp.ff_start
        tot += 2 * _bytes(t("ffn_gate"), ff * d) + _bytes(t("ffn_down"), ff * d)
    return tot + 4 * (2 * d + 2 * D)


def build_plan(cfg: ModelConfig, layout: dict, recipe: QuantRecipe | str = "Q4_K_M", ctx_size: int = 4096,
               batch_size: int = 1, max_prefill_tokens: int = 8192, hbm_bytes: int = B200_HBM_BYTES) -> ExecutionPlan:
    if isinstance(recipe, str):
        recipe = RECIPES[recipe]
    plan = ExecutionPlan(cfg.name, layout)
    tp_n = layout["tp"]
    errs = TPPlan.validate(cfg, tp_n)
    if errs:
        plan.errors.extend(errs)
        return plan
    stages = layout["stages"]
    n_stages = len(stages)
    rank = 0
    for si, (dom, devices, first, last) in enumerate(stages):
        if last < 0:
            # even split of the layers when the stage gives no explicit range
            first = cfg.n_layers * si // n_stages
            last = cfg.n_layers * (si + 1) // n_stages - 1
        if last >= cfg.n_layers:
            plan.errors.append(f"stage {si}: layer {last} beyond the model's {cfg.n_layers} layers")
            last = cfg.n_layers - 1
        for ti, dev in enumerate(devices):
            tp = TPPlan.build(cfg, tp_n, ti)
            rp = RankPlan(rank, dev, si, ti, first, last, si == 0, si == n_stages - 1, asdict(tp))
            w = sum(layer_weight_bytes(cfg, recipe, l, tp) for l in range(first, last + 1))
            if rp.has_embedding:
                w += _bytes(recipe.for_tensor("token_embd.weight"), cfg.vocab_size * cfg.d_model)
            if rp.has_head:
                w += _bytes(recipe.for_tensor("output.weight"), (tp.vocab_stop - tp.vocab_start) * cfg.d_model)
            rp.weight_bytes = int(w)
            pages = batch_size * ((ctx_size + 63) // 64 + 1) + 64
            stage_layers = range(first, last + 1)
            rp.kv_bytes = int(pages * len(cfg.kv_layers(stage_layers)) * 2 * tp.n_kv_local * 64 * cfg.head_dim * 2)
            if cfg.is_hybrid:
                # one fp32 state slot per batch lane (+1 scratch) for every linear-attention layer of the stage
                from .engine.kv_cache import HybridState
                nv = tp.gdn_v_stop - tp.gdn_v_start
                rp.kv_bytes += (batch_size + 1) * HybridState.bytes_per_slot(len(cfg.gdn_layers(stage_layers)), 2 * cfg.gdn_key_dim + nv * cfg.ssm_state,
                                                                             cfg.ssm_conv_kernel, nv, cfg.ssm_state)
            T = max(max_prefill_tokens, batch_size * 4)
            ff = (tp.ff_stop - tp.ff_start) if not cfg.is_moe else cfg.expert_ff
            rp.activation_bytes = int(T * (cfg.d_model * (4 + 2) + (tp.n_heads_local + 2 * tp.n_kv_local) * cfg.head_dim * 2
                                           + 2 * tp.n_heads_local * cfg.head_dim * 2 + ff * 2))
            rp.workspace_bytes = int(256 * 65536 * 4 + (1 << 22) * 4 + batch_size * 4 * (tp.vocab_stop - tp.vocab_start) * 4)
            if rp.total_bytes > hbm_bytes * 0.95:
                plan.errors.append(f"rank {rank} ({dev}): needs {rp.total_bytes / 1e9:.1f} GB, device has {hbm_bytes / 1e9:.0f} GB")
            plan.ranks.append(rp)
            rank += 1
    if last != cfg.n_layers - 1 and not plan.errors:
        plan.errors.append(f"pipeline stages end at layer {last}, model has {cfg.n_layers} layers")
    return plan


def suggest_layout(cfg: ModelConfig, n_devices: int, recipe: QuantRecipe | str = "Q4_K_M", ctx_size: int = 4096,
                   batch_size: int = 1, hbm_bytes: int | list[int] = B200_HBM_BYTES, max_prefill_tokens: int = 8192):
    """Smallest placement of ``cfg`` on up to ``n_devices`` identical GPUs that fits their memory.

    Candidates are (pp, tp) with tp a degree the model can be split by and pp * tp <= n_devices; fewer devices win, then
    tensor parallelism wins over pipeline stages (one NVSwitch domain: TP has the lower latency), then the plan with the
    most head-room.  ``hbm_bytes`` may be a list (an inventory of device memories): every rank must fit the smallest
    device it could land on.  Returns (layout, plan) or (None, reasons).  The reference's planner answers the same
    question from a cluster inventory (src/v2/planning/, tests/v2/integration/orchestration/scenarios/).
    """
    caps = sorted(hbm_bytes)[::-1] if isinstance(hbm_bytes, (list, tuple)) else [hbm_bytes] * n_devices
    n_devices = min(n_devices, len(caps))
    reasons, best = [], None
    for world in range(1, n_devices + 1):
        cap = caps[world - 1]                                   # the smallest of the `world` largest devices
        for pp in range(1, world + 1):
            if world % pp:
                continue
            tp = world // pp
            if TPPlan.validate(cfg, tp) or pp > cfg.n_layers:
                continue
            stages = [(f"s{i}", [f"cuda:{i * tp + j}" for j in range(tp)], cfg.n_layers * i // pp, cfg.n_layers * (i + 1) // pp - 1)
                      for i in range(pp)]
            layout = {"pp": pp, "tp": tp, "world": world, "stages": stages}
            plan = build_plan(cfg, layout, recipe, ctx_size, batch_size, max_prefill_tokens, cap)
            if plan.errors:
                reasons.append(f"pp={pp} x tp={tp}: {plan.errors[0]}")
                continue
            head_room = cap - max(r.total_bytes for r in plan.ranks)
            cand = (pp, -head_room, layout, plan)
            if best is None or cand[:2] < best[:2]:
                best = cand
        if best is not None:
            return best[2], best[3]
    return None, reasons or [f"{cfg.name} cannot be split over 1..{n_devices} devices"]
