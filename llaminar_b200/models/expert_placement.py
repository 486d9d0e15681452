"""Load-aware placement of MoE experts on expert-parallel ranks.

Expert parallelism gives every rank a contiguous range of expert ids.  Router statistics are skewed, so contiguous ranges of
the checkpoint's own numbering leave some ranks with several hot experts.  Because an expert's id is only a label (router
row e selects expert e), the experts of a layer can be renumbered freely: router rows and the stacked expert tensors are
permuted together and the model computes exactly the same function, but the contiguous ranges now hold balanced load.

    python -m llaminar_b200 benchmark -m model.gguf -d cuda:0 --moe-stats-out stats.json          # measure
    python -m llaminar_b200 serve -m model.gguf --tp-devices cuda:0,...,cuda:7 --moe-expert-placement stats.json

This is the static form of the reference's expert rebalancing (`--moe-rebalance`; src/v2/execution/moe/ExpertRebalancer.cpp,
ExpertPlacementMap.cpp, DecodeExpertHistogram.cpp): the statistics come from a profiling run instead of being refreshed
while serving.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch


class ExpertStats:
    """Tokens routed to every expert, per layer (filled by the models' router hooks)."""

    def __init__(self, n_layers: int, n_experts: int):
        self.counts = torch.zeros(n_layers, n_experts, dtype=torch.int64)

    def record(self, layer: int, expert_ids: torch.Tensor) -> None:
        ids = expert_ids.detach().reshape(-1).to("cpu", torch.int64)
        self.counts[layer] += torch.bincount(ids, minlength=self.counts.shape[1])[: self.counts.shape[1]]

    def dump(self, path: str, model: str = "") -> None:
        Path(path).write_text(json.dumps({"model": model, "n_experts": int(self.counts.shape[1]),
                                          "layers": {str(i): row.tolist() for i, row in enumerate(self.counts)}}) + "\n")

    @staticmethod
    def load(path: str) -> dict[int, list[int]]:
        doc = json.loads(Path(path).read_text())
        if not isinstance(doc, dict) or not isinstance(doc.get("layers"), dict):
            raise ValueError(f"{path}: expected an object with a 'layers' object (written by --moe-stats-out)")
        return {int(k): [int(x) for x in v] for k, v in doc["layers"].items()}


def balanced_permutation(load: list[float], n_ranks: int) -> list[int]:
    """``perm`` such that new expert j is old expert perm[j] and the n_ranks contiguous ranges of equal size carry nearly
    equal load: longest-processing-time greedy into bins of fixed capacity; inside a bin the old order is kept."""
    n = len(load)
    if n_ranks < 1 or n % n_ranks:
        raise ValueError(f"{n} experts cannot be split evenly over {n_ranks} ranks")
    cap = n // n_ranks
    bins: list[list[int]] = [[] for _ in range(n_ranks)]
    tot = [0.0] * n_ranks
    for e in sorted(range(n), key=lambda i: (-load[i], i)):
        r = min((r for r in range(n_ranks) if len(bins[r]) < cap), key=lambda r: (tot[r], r))
        bins[r].append(e)
        tot[r] += load[e]
    return [e for b in bins for e in sorted(b)]


def range_loads(load: list[float], perm: list[int], n_ranks: int) -> list[float]:
    cap = len(perm) // n_ranks
    return [float(sum(load[e] for e in perm[r * cap:(r + 1) * cap])) for r in range(n_ranks)]


def _take(qt, perm: list[int]):
    """Rows (2-D) or expert slices (3-D) of a quantised tensor in the order ``perm``."""
    from .weights import QTensor
    n = qt.shape[0]
    raw = qt.raw.reshape(n, -1)
    idx = torch.as_tensor(perm, dtype=torch.long, device=raw.device)
    return QTensor(qt.qtype, qt.shape, raw.index_select(0, idx).reshape(-1).contiguous())


def apply_placement(weights, layer_loads: dict[int, list[float]], n_ranks: int) -> dict[int, list[int]]:
    """Renumber the experts of every layer that has statistics, in place; returns the permutations used."""
    cfg = weights.config
    if not cfg.is_moe:
        raise ValueError("expert placement needs a mixture-of-experts model")
    used = {}
    for layer in range(cfg.n_layers):
        load = layer_loads.get(layer)
        if load is None:
            continue
        if len(load) != cfg.n_experts:
            raise ValueError(f"layer {layer}: statistics for {len(load)} experts, the model has {cfg.n_experts}")
        perm = balanced_permutation(load, n_ranks)
        p = f"blk.{layer}."
        for name in ("ffn_gate_inp.weight", "ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight"):
            weights.tensors[p + name] = _take(weights.tensors[p + name], perm)
        used[layer] = perm
    return used
