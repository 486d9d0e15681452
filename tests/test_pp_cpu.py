"""Pipeline parallelism on CPU ranks (gloo): PP=2 and PP=2 x TP=2 reproduce the single-rank tokens."""
import dataclasses

import torch

from llaminar_b200.models.config import SHAPES
from llaminar_b200.parallel.pp import stage_layer_ranges
from tests.mp_utils import run_ranks


def _prompts():
    g = torch.Generator().manual_seed(5)
    return [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (17, 90)]


def _pp_generate(rank, world, tp_size, mtp, payload="auto"):
    import os
    import torch.distributed as dist
    os.environ.update({"LLAMINAR_PP_PAYLOAD": payload})       # a child process of its own: set before the stage model reads it
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.parallel.pp import build_pipeline_engine
    from llaminar_b200.parallel.tp import TPContext
    shape = SHAPES["tiny-qwen3"]
    if mtp:
        shape = dataclasses.replace(shape, nextn_layers=1)
    w = synthesize(shape, "Q8_0", seed=0)
    pp = world // tp_size
    layout = {"pp": pp, "tp": tp_size, "world": world,
              "stages": [(f"s{i}", ["cpu"] * tp_size, None, None) for i in range(pp)]}
    groups = [dist.new_group(list(range(s * tp_size, (s + 1) * tp_size))) for s in range(pp)]
    tp = TPContext.create(groups[rank // tp_size], "cpu") if tp_size > 1 else None
    dec = None
    if mtp:
        from llaminar_b200.engine.mtp import MTPConfig, MTPDecoder
        dec = MTPDecoder(MTPConfig(draft_tokens=2))
    eng = build_pipeline_engine(w, layout, rank, microbatch_tokens=32, device="cpu", max_batch=2, max_context=256, tp=tp, mtp=dec)
    outs = eng.generate(_prompts(), SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    return outs, eng.model.stats, len(eng.model.inner.layers)


def _single(mtp=False):
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.synth import synthesize
    shape = SHAPES["tiny-qwen3"]
    if mtp:
        shape = dataclasses.replace(shape, nextn_layers=1)
    eng = LLMEngine(synthesize(shape, "Q8_0", seed=0), device="cpu", max_batch=2, max_context=256)
    return eng.generate(_prompts(), SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))


def test_pp2_matches_single_rank():
    ref = _single()
    res = run_ranks(_pp_generate, 2, 1, False)
    assert res[0][0] == ref and res[1][0] == ref
    assert res[0][1]["sent_bytes"] > 0 and res[1][1]["recv_bytes"] == res[0][1]["sent_bytes"]
    # only token ids cross the stages after sampling: one 4-byte id per sampled row, no full-vocabulary rows
    assert res[0][1]["token_syncs"] > 0 and res[0][1]["bcast_bytes"] == res[1][1]["bcast_bytes"] < 1024
    assert res[0][2] + res[1][2] == SHAPES["tiny-qwen3"].n_layers


def test_pp2_bf16_payload_halves_the_bytes_and_ranks_agree():
    """The residual stream between the stages as bf16: both stages emit the same tokens (the last stage's draw is
    broadcast), half the bytes cross; the tokens may differ from the fp32 run by a rounding."""
    fp32 = run_ranks(_pp_generate, 2, 1, False)
    bf16 = run_ranks(_pp_generate, 2, 1, False, "bf16")
    assert bf16[0][0] == bf16[1][0] and all(len(o) == 6 for o in bf16[0][0])
    assert bf16[0][1]["sent_bytes"] * 2 == fp32[0][1]["sent_bytes"]


def test_pp2_tp2_with_mtp_matches_single_rank():
    ref = _single(mtp=True)
    res = run_ranks(_pp_generate, 4, 2, True)
    assert all(r[0] == ref for r in res)


def test_stage_ranges():
    lay = {"pp": 3, "stages": [("a", [], None, None)] * 3}
    assert stage_layer_ranges(10, lay) == [(0, 3), (3, 6), (6, 10)]
    lay = {"pp": 2, "stages": [("a", [], 0, 5), ("b", [], 6, 9)]}
    assert stage_layer_ranges(10, lay) == [(0, 6), (6, 10)]
