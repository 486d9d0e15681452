"""Layer-by-layer parity report of the runtime model against the fp32 oracle.

    python -m llaminar_b200.parity --synthetic tiny-qwen3 --synthetic-recipe Q4_K_M -d cuda:0 --prompt-tokens 200 --csv parity.csv
    python -m llaminar_b200.parity -m model.gguf -d cpu

Both models read the same (quantised) weights: the oracle dequantises them to fp32 and runs plain PyTorch, the runtime
model runs the engine's kernels (or the CPU runner).  One prefill over a random prompt and a few decode steps are compared:
per-layer cosine similarity and relative L2 error of the hidden state, then KL divergence, top-1 agreement and top-5 overlap
of the logits.  The exit code is 1 when a gate fails.  Counterpart of the reference's PyTorch parity suite
(tests/v2/integration/parity/, python/reference/generate_*_snapshots.py: per-stage snapshots of the same GGUF, cosine
>= 0.99-0.999 per layer, LM-head KL, top-1/5, CSV per run).
"""
from __future__ import annotations

import argparse
import csv
import sys

import torch

GATES = {"layer_cosine": 0.99, "logit_top1": 0.90, "logit_kl": 0.05}


def _cos(a: torch.Tensor, b: torch.Tensor) -> float:
    return torch.nn.functional.cosine_similarity(a.double().flatten(), b.double().flatten(), dim=0).item()


def _rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    return ((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30)).item()


def logit_metrics(test: torch.Tensor, ref: torch.Tensor) -> dict:
    """KL(ref || test) of the softmax rows (mean), top-1 agreement and mean top-5 overlap."""
    lt, lr = test.double().log_softmax(-1), ref.double().log_softmax(-1)
    kl = (lr.exp() * (lr - lt)).sum(-1).mean().item()
    top1 = (test.argmax(-1) == ref.argmax(-1)).double().mean().item()
    t5, r5 = test.topk(5, -1).indices, ref.topk(5, -1).indices
    overlap = torch.stack([torch.isin(t5[i], r5[i]).double().mean() for i in range(t5.shape[0])]).mean().item()
    return {"kl": kl, "top1": top1, "top5_overlap": overlap}


def compare(weights, device: str, prompt_tokens: int = 96, decode_steps: int = 4, seed: int = 1) -> tuple[list[dict], list[str]]:
    """Rows of the report and the list of failed gates."""
    from .engine.cuda_model import ForwardBatch
    from .engine.kv_cache import PagedKVCache
    from .models.reference import ReferenceModel
    dev = torch.device(device)
    cfg = weights.config
    if dev.type == "cuda":
        from .engine.cuda_model import CudaModel
        model = CudaModel(weights, dev, max_tokens=max(prompt_tokens, 64))
        kv_dtype = torch.bfloat16
    else:
        from .engine.torch_model import TorchPagedModel
        model = TorchPagedModel(weights, dev)
        kv_dtype = torch.float32
    ref = ReferenceModel(weights)
    total = prompt_tokens + decode_steps
    pages = (total + 63) // 64
    kv = PagedKVCache(getattr(model, "n_kv_layers", cfg.n_layers + cfg.nextn_layers), model.n_kv_local, cfg.head_dim, pages + 2, dev,
                      dtype=kv_dtype)
    slots = None
    if getattr(model, "hybrid_dims", None):                  # linear-attention layers: one state slot for the one sequence
        from .engine.kv_cache import HybridState
        kv.hybrid = HybridState(n_slots=1, device=dev, **model.hybrid_dims)
        slots = torch.zeros(1, dtype=torch.int32, device=dev)
    g = torch.Generator().manual_seed(seed)
    prompt = torch.randint(0, cfg.vocab_size, (prompt_tokens,), generator=g)
    it = lambda x: torch.as_tensor(x, dtype=torch.int32, device=dev)
    bt = it([list(range(1, pages + 1))])
    rows, failed = [], []

    def one_pass(phase: str, tokens: torch.Tensor, fb: ForwardBatch, ref_kv):
        model.taps, ref_taps = {}, {}
        logits, _ = model.forward(fb, kv)
        ref_logits, _, ref_kv = ref.forward(tokens, ref_kv, taps=ref_taps)
        for name in sorted(ref_taps, key=lambda s: int(s[5:])):
            t, r = model.taps[name].cpu(), ref_taps[name].cpu()
            row = {"phase": phase, "stage": name, "cosine": _cos(t, r), "rel_l2": _rel_l2(t, r)}
            rows.append(row)
            if row["cosine"] < GATES["layer_cosine"]:
                failed.append(f"{phase} {name}: cosine {row['cosine']:.5f} < {GATES['layer_cosine']}")
        model.taps = None
        lm = logit_metrics(logits.float().cpu(), ref_logits.float().cpu()[-logits.shape[0]:])
        rows.append({"phase": phase, "stage": "logits", **lm})
        if lm["top1"] < GATES["logit_top1"]:
            failed.append(f"{phase} logits: top-1 agreement {lm['top1']:.3f} < {GATES['logit_top1']}")
        if lm["kl"] > GATES["logit_kl"]:
            failed.append(f"{phase} logits: KL {lm['kl']:.4f} > {GATES['logit_kl']}")
        return ref_logits, ref_kv

    n = prompt_tokens
    fb = ForwardBatch(tokens=it(prompt.tolist()), positions=it(list(range(n))), seq_ids=it([0] * n), block_table=bt,
                      cu_q=it([0, n]), ctx_lens=it([0]), max_q_len=n, state_slots=slots)
    ref_logits, ref_kv = one_pass("prefill", prompt, fb, None)
    nxt = int(ref_logits[-1].argmax())
    for step in range(decode_steps):                     # teacher-forced with the oracle's greedy tokens
        pos = n + step
        fb = ForwardBatch(tokens=it([nxt]), positions=it([pos]), seq_ids=it([0]), block_table=bt, seq_lens=it([pos + 1]),
                          state_slots=slots)
        ref_logits, ref_kv = one_pass(f"decode{step}", torch.tensor([nxt]), fb, ref_kv)
        nxt = int(ref_logits[-1].argmax())
    return rows, failed


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("-m", "--model", help="GGUF file")
    ap.add_argument("--synthetic", help="random-init model of a known shape instead of a file")
    ap.add_argument("--synthetic-recipe", default="Q4_K_M")
    ap.add_argument("-d", "--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--prompt-tokens", type=int, default=96)
    ap.add_argument("--decode-steps", type=int, default=4)
    ap.add_argument("--csv", help="write the report rows to this file")
    args = ap.parse_args(argv)
    if bool(args.model) == bool(args.synthetic):
        ap.error("give exactly one of --model and --synthetic")
    if args.synthetic:
        from .models.config import SHAPES
        from .models.synth import synthesize
        weights = synthesize(SHAPES[args.synthetic], args.synthetic_recipe, seed=0)
    else:
        from .models.weights import ModelWeights
        weights = ModelWeights.from_gguf(args.model, device="cpu")
    rows, failed = compare(weights, args.device, args.prompt_tokens, args.decode_steps)
    for r in rows:
        if r["stage"] == "logits":
            print(f"{r['phase']:9s} logits   KL {r['kl']:.5f}  top-1 {r['top1']:.3f}  top-5 overlap {r['top5_overlap']:.3f}")
        else:
            print(f"{r['phase']:9s} {r['stage']:8s} cosine {r['cosine']:.6f}  rel-L2 {r['rel_l2']:.5f}")
    if args.csv:
        keys = ["phase", "stage", "cosine", "rel_l2", "kl", "top1", "top5_overlap"]
        with open(args.csv, "w", newline="") as f:
            wr = csv.DictWriter(f, fieldnames=keys)
            wr.writeheader()
            for r in rows:
                wr.writerow({k: r.get(k, "") for k in keys})
    for msg in failed:
        print("FAIL " + msg, file=sys.stderr)
    return 1 if failed else 0


if __name__ == "__main__":
    raise SystemExit(main())
