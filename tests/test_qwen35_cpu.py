"""The hybrid Gated-DeltaNet family (qwen35) on the CPU: the chunk-parallel delta rule against the token-by-token form, the
fp32 oracle against the `transformers` implementation of the architecture (weights converted the way GGUF files store them:
norm gains as 1 + w, ssm_a = -exp(A_log), value heads in tiled order), and the engine's runner against the oracle."""
import pytest
import torch

from llaminar_b200.gguf import GGMLType
from llaminar_b200.models import gdn
from llaminar_b200.models.config import SHAPES, ModelConfig
from llaminar_b200.models.reference import ReferenceModel
from llaminar_b200.models.synth import synthesize
from llaminar_b200.models.weights import ModelWeights, qtensor_from_float


def test_chunked_delta_rule_matches_token_by_token():
    torch.manual_seed(0)
    T, H, d = 150, 4, 32
    q = gdn.l2norm(torch.randn(T, H, d)) * d ** -0.5
    k = gdn.l2norm(torch.randn(T, H, d))
    v = torch.randn(T, H, d)
    g, beta = -torch.rand(T, H) * 3, torch.rand(T, H)
    S0 = torch.randn(H, d, d) * 0.1
    S1, S2 = S0.clone(), S0.clone()
    o1 = gdn.delta_rule_recurrent(q, k, v, g, beta, S1)
    o2 = gdn.delta_rule_chunked(q, k, v, g, beta, S2, chunk=64)
    assert (o1 - o2).abs().max() < 1e-5 and (S1 - S2).abs().max() < 1e-5


def test_convolution_state_carries_across_calls():
    torch.manual_seed(1)
    x, w = torch.randn(11, 6), torch.randn(6, 4)
    y, _ = gdn.causal_conv_silu(x, torch.zeros(6, 3), w)
    y1, st = gdn.causal_conv_silu(x[:5], torch.zeros(6, 3), w)
    y2, _ = gdn.causal_conv_silu(x[5:], st, w)
    assert torch.allclose(y, torch.cat([y1, y2]), atol=1e-6)


def _hf_model(moe: bool = False):
    tf = pytest.importorskip("transformers")
    try:
        if moe:
            from transformers.models.qwen3_5_moe.modeling_qwen3_5_moe import Qwen3_5MoeForCausalLM as Qwen3_5ForCausalLM
            from transformers.models.qwen3_5_moe.modeling_qwen3_5_moe import Qwen3_5MoeTextConfig as Qwen3_5TextConfig
        else:
            from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5ForCausalLM, Qwen3_5TextConfig
    except Exception as e:                                    # an older transformers without the family
        pytest.skip(f"transformers has no qwen3_5: {e}")
    extra = dict(num_experts=6, num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=48) if moe else {}
    cfg = Qwen3_5TextConfig(**extra, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                            intermediate_size=128, vocab_size=128, rms_norm_eps=1e-6, max_position_embeddings=512,
                            layer_types=["linear_attention"] * 3 + ["full_attention"], full_attention_interval=4,
                            linear_key_head_dim=16, linear_value_head_dim=16, linear_num_key_heads=2, linear_num_value_heads=4,
                            linear_conv_kernel_dim=4, tie_word_embeddings=False,
                            rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.25,
                                             "mrope_section": [2, 1, 1]})
    cfg._attn_implementation = "eager"
    torch.manual_seed(3)
    m = Qwen3_5ForCausalLM(cfg).float().eval()
    with torch.no_grad():                                      # make every learned vector non-trivial
        for n, p in m.named_parameters():
            if p.dim() == 1:
                p.copy_(torch.randn_like(p) * 0.3)
            if n.endswith("A_log"):
                p.copy_(torch.log(torch.rand_like(p) * 6 + 0.5))
            if n.endswith("linear_attn.norm.weight"):
                p.copy_(torch.rand_like(p) + 0.5)
            if "experts." in n or "mlp.gate.weight" in n or "shared_expert_gate" in n:
                p.copy_(torch.randn_like(p) * 0.2)           # left uninitialised / zero by the constructor
    return cfg, m


def _tiled_value_heads(n_k: int, n_v: int) -> list[int]:
    """GGUF value head i = r * n_k + kh holds the transformers value head kh * rep + r (so that head i reads key head
    i mod n_k where transformers reads key head j div rep)."""
    rep = n_v // n_k
    return [(i % n_k) * rep + i // n_k for i in range(n_v)]


def _convert(cfg, m) -> ModelWeights:
    n_k, n_v, d = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim
    moe = hasattr(cfg, "num_experts")
    moe_kw = dict(n_experts=cfg.num_experts, n_experts_used=cfg.num_experts_per_tok, expert_ff=cfg.moe_intermediate_size,
                  shared_expert_ff=cfg.shared_expert_intermediate_size) if moe else {}
    ours = ModelConfig(name="hf-tiny-qwen35", arch="qwen35moe" if moe else "qwen35", n_layers=cfg.num_hidden_layers, d_model=cfg.hidden_size,
                       n_heads=cfg.num_attention_heads, n_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, **moe_kw,
                       d_ff=0 if moe else cfg.intermediate_size, vocab_size=cfg.vocab_size, rope_theta=10000.0, rms_eps=cfg.rms_norm_eps,
                       tie_embeddings=False, full_attention_interval=4, ssm_conv_kernel=4, ssm_state=d, ssm_k_heads=n_k,
                       ssm_v_heads=n_v, rope_dim=int(cfg.head_dim * 0.25), attn_gate=True)
    sd = {k: v.detach().float() for k, v in m.state_dict().items()}
    perm = torch.tensor(_tiled_value_heads(n_k, n_v))
    rows = (perm[:, None] * d + torch.arange(d)[None, :]).reshape(-1)           # value-head blocks of d rows
    t = {}
    put = lambda name, x: t.__setitem__(name, qtensor_from_float(x.contiguous(), GGMLType.F32))
    put("token_embd.weight", sd["model.embed_tokens.weight"])
    put("output.weight", sd["lm_head.weight"])
    put("output_norm.weight", 1 + sd["model.norm.weight"])
    for i in range(cfg.num_hidden_layers):
        s, p = f"model.layers.{i}.", f"blk.{i}."
        put(p + "attn_norm.weight", 1 + sd[s + "input_layernorm.weight"])
        put(p + "post_attention_norm.weight", 1 + sd[s + "post_attention_layernorm.weight"])
        if moe:
            ff = cfg.moe_intermediate_size
            put(p + "ffn_gate_inp.weight", sd[s + "mlp.gate.weight"])
            put(p + "ffn_gate_exps.weight", sd[s + "mlp.experts.gate_up_proj"][:, :ff])
            put(p + "ffn_up_exps.weight", sd[s + "mlp.experts.gate_up_proj"][:, ff:])
            put(p + "ffn_down_exps.weight", sd[s + "mlp.experts.down_proj"])
            for a, b in (("gate", "gate_proj"), ("up", "up_proj"), ("down", "down_proj")):
                put(p + f"ffn_{a}_shexp.weight", sd[s + f"mlp.shared_expert.{b}.weight"])
            put(p + "ffn_gate_inp_shexp.weight", sd[s + "mlp.shared_expert_gate.weight"].reshape(-1))
        else:
            for a, b in (("gate", "gate_proj"), ("up", "up_proj"), ("down", "down_proj")):
                put(p + f"ffn_{a}.weight", sd[s + f"mlp.{b}.weight"])
        if cfg.layer_types[i] == "linear_attention":
            la = s + "linear_attn."
            kd = n_k * d
            qkv = sd[la + "in_proj_qkv.weight"]
            put(p + "attn_qkv.weight", torch.cat([qkv[:2 * kd], qkv[2 * kd:][rows]]))
            put(p + "attn_gate.weight", sd[la + "in_proj_z.weight"][rows])
            put(p + "ssm_alpha.weight", sd[la + "in_proj_a.weight"][perm])
            put(p + "ssm_beta.weight", sd[la + "in_proj_b.weight"][perm])
            conv = sd[la + "conv1d.weight"].squeeze(1)
            put(p + "ssm_conv1d.weight", torch.cat([conv[:2 * kd], conv[2 * kd:][rows]]))
            put(p + "ssm_dt.bias", sd[la + "dt_bias"][perm])
            put(p + "ssm_a", -torch.exp(sd[la + "A_log"][perm]))
            put(p + "ssm_norm.weight", sd[la + "norm.weight"])
            put(p + "ssm_out.weight", sd[la + "out_proj.weight"][:, rows])
        else:
            sa = s + "self_attn."
            put(p + "attn_q.weight", sd[sa + "q_proj.weight"])
            put(p + "attn_k.weight", sd[sa + "k_proj.weight"])
            put(p + "attn_v.weight", sd[sa + "v_proj.weight"])
            put(p + "attn_output.weight", sd[sa + "o_proj.weight"])
            put(p + "attn_q_norm.weight", 1 + sd[sa + "q_norm.weight"])
            put(p + "attn_k_norm.weight", 1 + sd[sa + "k_norm.weight"])
    return ModelWeights(ours, t)


@pytest.mark.parametrize("moe", [False, True], ids=["dense", "moe-with-shared-expert"])
def test_oracle_matches_the_transformers_model(moe):
    cfg, m = _hf_model(moe)
    w = _convert(cfg, m)
    toks = torch.randint(0, cfg.vocab_size, (37,), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        want = m(input_ids=toks[None]).logits[0]
    ref = ReferenceModel(w)
    got, _, kv = ref.forward(toks)
    assert (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))
    # the same rows fed in pieces (prefill chunk, second chunk, single tokens): the carried state must give the same logits
    a, _, kv = ref.forward(toks[:20])
    b, _, kv = ref.forward(toks[20:33], kv)
    rest = [ref.forward(toks[i:i + 1], kv)[0] for i in range(33, 37)]
    assert (torch.cat([a, b] + rest) - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))


def test_gguf_round_trip_keeps_the_hybrid_configuration(tmp_path):
    w = synthesize(SHAPES["tiny-qwen35"], "Q8_0", seed=2)
    path = str(tmp_path / "h.gguf")
    w.save_gguf(path)
    back = ModelWeights.from_gguf(path)
    c0, c1 = w.config, back.config
    for f in ("arch", "n_layers", "full_attention_interval", "ssm_conv_kernel", "ssm_state", "ssm_k_heads", "ssm_v_heads",
              "rope_dim", "attn_gate", "qk_norm", "head_dim"):
        assert getattr(c0, f) == getattr(c1, f), f
    assert [c1.is_gdn_layer(i) for i in range(8)] == [True, True, True, False] * 2
    assert back["blk.0.ssm_conv1d.weight"].shape == (c0.gdn_conv_dim, 4)


def _prompt(n, seed, vocab=1024):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def test_engine_on_the_hybrid_model_matches_the_oracle_with_batching_and_chunked_prefill():
    """Continuous batching over state slots: three prompts of different lengths, prefill split into chunks (the recurrent
    state carries from chunk to chunk), decode steps batched; every sequence must emit the oracle's greedy tokens."""
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    w = synthesize(SHAPES["tiny-qwen35"], "Q8_0", seed=7)
    ref = ReferenceModel(w)
    prompts = [_prompt(70, 1), _prompt(9, 2), _prompt(33, 3)]
    want = [ref.generate_greedy(torch.tensor(p), 8)[0] for p in prompts]
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=256, max_prefill_tokens=48)
    got = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    assert got == want
    assert sorted(eng.kv.hybrid.free) == [0, 1]                       # every slot came back
    assert eng.kv.allocator.n_free == eng.kv.n_pages - 1


def test_hybrid_model_rejects_speculation_and_the_8bit_cache_by_name():
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.mtp import MTPDecoder
    w = synthesize(SHAPES["tiny-qwen35"], "Q8_0", seed=7)
    with pytest.raises(ValueError, match="mtp"):
        LLMEngine(w, device="cpu", max_batch=2, max_context=128, mtp=MTPDecoder())


def _chat_turns(eng):
    """Two 'turns': the second prompt extends the first prompt and its answer.  Returns both outputs."""
    from llaminar_b200.engine.sampling import SamplingParams
    p = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    first = _prompt(150, 21)
    a = eng.generate([first], p)[0]
    second = first + a + _prompt(40, 22)
    return a, eng.generate([second], p)[0]


def test_prefix_cache_resumes_a_hybrid_model_from_a_state_snapshot():
    """The second prompt shares 156 tokens with the first request; the cached chain is cut back to the boundary where the
    first prompt's recurrent state was snapshotted (128 = the last block boundary that left a token to run), the state
    slot is restored from it, and the answers equal those of an engine without a cache."""
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.prefix_cache import PrefixCache
    w = synthesize(SHAPES["tiny-qwen35"], "Q8_0", seed=7)
    plain = _chat_turns(LLMEngine(w, device="cpu", max_batch=2, max_context=512, max_prefill_tokens=96))
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=512, max_prefill_tokens=96, prefix_cache=PrefixCache())
    cached = _chat_turns(eng)
    assert cached == plain
    assert eng.stats["prefix_hit_tokens"] == 128
    st = eng.prefix_cache.stats()
    assert st["state_snapshots"] == 2 and st["terminal_stored"] == 0      # one per prompt (at 128 and at 192)
    assert sorted(eng.kv.hybrid.free) == [0, 1]


def _tp_chat(rank, world):
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.prefix_cache import PrefixCache
    from llaminar_b200.parallel.tp import TPContext
    w = synthesize(SHAPES["tiny-qwen35"], "Q8_0", seed=7)
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=512, tp=TPContext.create(device="cpu"), prefix_cache=PrefixCache())
    return _chat_turns(eng), eng.stats["prefix_hit_tokens"]


def test_tp2_ranks_agree_on_the_snapshot_boundary():
    from llaminar_b200.engine.engine import LLMEngine
    from tests.mp_utils import run_ranks
    w = synthesize(SHAPES["tiny-qwen35"], "Q8_0", seed=7)
    plain = _chat_turns(LLMEngine(w, device="cpu", max_batch=2, max_context=512))
    res = run_ranks(_tp_chat, 2)
    assert res[0] == (plain, 128) and res[1] == (plain, 128)


def _tp_generate(rank, world):
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.parallel.tp import TPContext
    w = synthesize(SHAPES["tiny-qwen35"], "Q8_0", seed=0)
    tp = TPContext.create(device="cpu")
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=128, tp=tp, max_prefill_tokens=32)
    outs = eng.generate([_prompt(17, 5), _prompt(40, 6)], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    return outs, eng.model.hybrid_dims


def test_tp2_shards_the_value_heads_and_matches_a_single_rank():
    """Two gloo ranks: each holds two of the four value heads (with all key heads, read in tiled order from the rank's
    first global head), the output projection is row-parallel; tokens must equal the single-rank engine's."""
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from tests.mp_utils import run_ranks
    w = synthesize(SHAPES["tiny-qwen35"], "Q8_0", seed=0)
    ref = LLMEngine(w, device="cpu", max_batch=2, max_context=128, max_prefill_tokens=32).generate(
        [_prompt(17, 5), _prompt(40, 6)], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    res = run_ranks(_tp_generate, 2)
    assert res[0][0] == ref and res[1][0] == ref
    assert res[0][1]["n_v_heads"] == 2 and res[0][1]["conv_dim"] == 2 * 64 + 2 * 32


def _pp_generate(rank, world):
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.parallel.pp import build_pipeline_engine
    w = synthesize(SHAPES["tiny-qwen35"], "Q8_0", seed=0)
    layout = {"pp": 2, "tp": 1, "world": 2, "stages": [("s0", ["cpu"], 0, 2), ("s1", ["cpu"], 3, 7)]}
    eng = build_pipeline_engine(w, layout, rank, microbatch_tokens=32, device="cpu", max_batch=2, max_context=256)
    outs = eng.generate([_prompt(17, 5), _prompt(90, 6)], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    return outs, eng.model.n_kv_layers, eng.model.hybrid_dims["n_layers"]


def test_pp2_with_a_stage_of_linear_attention_only_matches_a_single_rank():
    """Stage 0 holds layers 0-2 (no softmax block, hence no KV layer at all), stage 1 the rest."""
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from tests.mp_utils import run_ranks
    w = synthesize(SHAPES["tiny-qwen35"], "Q8_0", seed=0)
    ref = LLMEngine(w, device="cpu", max_batch=2, max_context=256).generate(
        [_prompt(17, 5), _prompt(90, 6)], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    res = run_ranks(_pp_generate, 2)
    assert res[0][0] == ref and res[1][0] == ref
    assert (res[0][1], res[0][2]) == (0, 3) and (res[1][1], res[1][2]) == (2, 3)


def _moe_tp_generate(rank, world):
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.parallel.tp import TPContext
    w = synthesize(SHAPES["tiny-qwen35moe"], "Q8_0", seed=11, std=0.05)
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=128, tp=TPContext.create(device="cpu"))
    return eng.generate([_prompt(17, 5), _prompt(40, 6)], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))


def test_hybrid_moe_engine_matches_the_oracle_and_expert_parallel_ranks_agree():
    """qwen35moe: linear-attention blocks, routed experts and the always-on shared expert with its sigmoid gate.  Single
    rank against the oracle; two expert-parallel ranks (the shared expert replicated, added after the experts' sum)
    against the single rank."""
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from tests.mp_utils import run_ranks
    w = synthesize(SHAPES["tiny-qwen35moe"], "Q8_0", seed=11, std=0.05)
    assert "blk.0.ffn_gate_inp_shexp.weight" in w and w.config.shared_expert_ff == 256
    ref = ReferenceModel(w)
    prompts = [_prompt(17, 5), _prompt(40, 6)]
    want = [ref.generate_greedy(torch.tensor(p), 6)[0] for p in prompts]
    got = LLMEngine(w, device="cpu", max_batch=2, max_context=128).generate(
        prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    assert got == want
    assert any(len(set(o)) > 1 for o in got)                   # not a degenerate repeat
    res = run_ranks(_moe_tp_generate, 2)
    assert res[0] == got and res[1] == got


def test_batched_paged_decode_attention_matches_a_per_sequence_loop():
    """The shape-static decode attention used for head sizes without a kernel (256 in the published hybrid checkpoints):
    three sequences of different lengths on shuffled pages, GQA 4:2, against plain attention over each sequence's rows."""
    from llaminar_b200.engine.cuda_model import paged_decode_attention_torch
    torch.manual_seed(2)
    B, H, Hk, D, P = 3, 4, 2, 256, 3
    kv = torch.randn(12, 2, Hk, 64, D)
    bt = torch.tensor([[5, 2, 9], [1, 7, 0], [3, 11, 4]], dtype=torch.int32)
    lens = torch.tensor([130, 1, 64], dtype=torch.int32)
    q = torch.randn(B, H, D)
    got = paged_decode_attention_torch(q, kv, bt, lens, D ** -0.5)
    for b in range(B):
        n = int(lens[b])
        K = kv[bt[b].long(), 0].permute(1, 0, 2, 3).reshape(Hk, P * 64, D)[:, :n].repeat_interleave(H // Hk, 0)
        V = kv[bt[b].long(), 1].permute(1, 0, 2, 3).reshape(Hk, P * 64, D)[:, :n].repeat_interleave(H // Hk, 0)
        p = torch.softmax(torch.einsum("hd,hld->hl", q[b], K) * D ** -0.5, -1)
        assert torch.allclose(got[b], torch.einsum("hl,hld->hd", p, V), atol=1e-5)


def test_deferred_rows_and_commit_equal_feeding_the_accepted_rows_one_by_one():
    torch.manual_seed(0)
    B, R, n_k, n_v, d, K = 3, 4, 2, 4, 16, 4
    C = 2 * n_k * d + n_v * d
    conv_w, ssm_a, dt, nw = torch.randn(C, K) * 0.4, -(torch.rand(n_v) * 3 + 0.2), torch.rand(n_v) * 2 - 1, torch.rand(d) + 0.5
    conv, rec = torch.randn(6, C, K - 1) * 0.5, torch.randn(6, n_v, d, d) * 0.1
    slots, acc = torch.tensor([4, 1, 2]), torch.tensor([1, 4, 2])
    qkv, z, al, bb = torch.randn(B, R, C), torch.randn(B, R, n_v * d), torch.randn(B, R, n_v), torch.randn(B, R, n_v)
    c2, r2 = conv.clone(), rec.clone()
    rows, stash = gdn.gdn_rows_deferred(qkv, z, al, bb, conv_w, ssm_a, dt, nw, c2, r2, slots, n_k, n_v, d, 1e-6, 1)
    assert torch.equal(c2, conv) and torch.equal(r2, rec)              # nothing committed yet
    gdn.commit_rows(stash, c2, r2, slots, acc)
    c3, r3 = conv.clone(), rec.clone()
    for i in range(B):
        s = int(slots[i])
        for j in range(int(acc[i])):
            o, c3[s] = gdn.gdn_mix(qkv[i, j:j + 1], z[i, j:j + 1], al[i, j:j + 1], bb[i, j:j + 1], conv_w, ssm_a, dt, nw,
                                   c3[s], r3[s], n_k, n_v, d, 1e-6, 1)
            assert torch.allclose(o[0], rows[i * R + j], atol=1e-5)
    assert torch.allclose(c2, c3, atol=1e-6) and torch.allclose(r2, r3, atol=1e-6)


@pytest.mark.parametrize("force", [False, True], ids=["verified", "all-drafts-accepted"])
def test_speculative_decoding_on_the_hybrid_model(force):
    """NextN drafts verified by the hybrid trunk: the verification pass leaves the recurrent state alone and it is advanced
    by the accepted rows only.  Verified drafts must reproduce plain greedy decoding token for token; with every draft
    force-accepted (a throughput switch, not lossless) the state must still advance by all rows, which the run's length
    and the returned slots show."""
    import dataclasses
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.mtp import MTPConfig, MTPDecoder
    from llaminar_b200.engine.sampling import SamplingParams
    cfg = dataclasses.replace(SHAPES["tiny-qwen35"], nextn_layers=1, name="tiny-qwen35-mtp")
    w = synthesize(cfg, "Q8_0", seed=9)
    prompts = [_prompt(40, 3), _prompt(70, 4)]
    p = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    plain = LLMEngine(w, device="cpu", max_batch=2, max_context=256).generate(prompts, p)
    dec = MTPDecoder(MTPConfig(draft_tokens=2, force_accept=force))
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=256, mtp=dec)
    got = eng.generate(prompts, p)
    assert all(len(o) == 12 for o in got)
    if not force:
        assert got == plain
    st = dec.stats()
    assert st["drafted"] > 0 and (st["accepted"] == st["drafted"] if force else True)
    assert sorted(eng.kv.hybrid.free) == [0, 1] and not eng.kv.hybrid.stash


def test_per_layer_head_count_arrays_in_gguf_metadata_are_accepted(tmp_path):
    """Converters of hybrid checkpoints may write `attention.head_count_kv` (and the FFN width) as one entry per layer, with
    0 for the linear-attention layers; the configuration takes the softmax blocks' value."""
    w = synthesize(SHAPES["tiny-qwen35"], "Q8_0", seed=2)
    path = str(tmp_path / "arr.gguf")
    c = w.config
    per_layer = [0 if c.is_gdn_layer(i) else c.n_kv_heads for i in range(c.n_layers)]
    w.save_gguf(path, extra_metadata={"qwen35.attention.head_count_kv": per_layer,
                                      "qwen35.feed_forward_length": [c.d_ff] * c.n_layers})
    back = ModelWeights.from_gguf(path).config
    assert back.n_kv_heads == c.n_kv_heads and back.d_ff == c.d_ff and back.full_attention_interval == 4


def test_preemption_on_the_hybrid_model_gives_the_slot_back_and_recomputes_the_state():
    """A cache that holds about half of three long generations: preempted sequences return their pages and their state slot,
    come back with their tokens folded into the prompt, and the prefill that rebuilds their K/V rebuilds the recurrent
    state from position 0; outputs equal those of an engine with room for everything."""
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    w = synthesize(SHAPES["tiny-qwen35"], "Q8_0", seed=7)
    prompts = [_prompt(60, s) for s in (1, 2, 3)]
    sp = SamplingParams(temperature=0.0, max_tokens=120, ignore_eos=True)
    want = LLMEngine(w, device="cpu", max_batch=3, max_context=256).generate(prompts, sp)
    small = LLMEngine(w, device="cpu", max_batch=3, max_context=256, kv_pages=7)          # 6 usable pages of 64 tokens
    reqs = [small.add_request(p, sp) for p in prompts]
    while small.has_unfinished():
        small.step()
    assert small.stats["preemptions"] >= 1
    assert [r.output for r in reqs] == want
    assert small.kv.allocator.n_free == small.kv.n_pages - 1 and sorted(small.kv.hybrid.free) == [0, 1, 2]


def test_equal_length_sequences_evaluated_together_match_one_at_a_time():
    """A packed prefill batch with three 70-row sequences (one of them continuing from an earlier state), one 9-row and one
    3-row sequence: the grouped evaluation must equal running every sequence alone."""
    torch.manual_seed(4)
    n_k, n_v, d, K = 2, 4, 16, 4
    C = 2 * n_k * d + n_v * d
    conv_w, ssm_a, dt, nw = torch.randn(C, K) * 0.4, -(torch.rand(n_v) * 3 + 0.2), torch.rand(n_v) * 2 - 1, torch.rand(d) + 0.5
    conv, rec = torch.randn(7, C, K - 1) * 0.5, torch.randn(7, n_v, d, d) * 0.1
    lens, slots, fresh = [70, 9, 70, 3, 70], [5, 0, 2, 6, 1], [True, True, False, False, True]
    T = sum(lens)
    qkv, z, al, bb = torch.randn(T, C), torch.randn(T, n_v * d), torch.randn(T, n_v), torch.randn(T, n_v)
    seqs, r0 = [], 0
    for n, s, f in zip(lens, slots, fresh):
        seqs.append((r0, r0 + n, s, f))
        r0 += n
    c1, r1 = conv.clone(), rec.clone()
    got = gdn.gdn_block_rows(qkv, z, al, bb, seqs, c1, r1, conv_w, ssm_a, dt, nw, n_k, n_v, d, 1e-6, 1)
    c2, r2 = conv.clone(), rec.clone()
    want = torch.cat([gdn.gdn_block_rows(qkv[a:b_], z[a:b_], al[a:b_], bb[a:b_], [(0, b_ - a, s, f)], c2, r2, conv_w, ssm_a, dt, nw,
                                         n_k, n_v, d, 1e-6, 1) for a, b_, s, f in seqs])
    assert torch.allclose(got, want, atol=2e-5)
    assert torch.allclose(c1, c2, atol=1e-6) and torch.allclose(r1, r2, atol=2e-5)


def test_parity_report_and_memory_plan_cover_hybrid_models():
    """The layer-by-layer parity tool runs a hybrid model (it owns one state slot), and the memory planner counts the
    recurrent state of every batch lane and KV pages for the softmax blocks only."""
    from llaminar_b200.parity import compare
    from llaminar_b200.planning import build_plan
    rows, failed = compare(synthesize(SHAPES["tiny-qwen35"], "Q8_0", seed=1), "cpu", prompt_tokens=40, decode_steps=2)
    assert not failed and sum(r["stage"] == "logits" for r in rows) == 3
    lay = {"pp": 1, "tp": 2, "world": 2, "stages": [("s0", ["cuda:0", "cuda:1"], 0, -1)]}
    cfg = SHAPES["qwen3.5-27b"]
    plan = build_plan(cfg, lay, "Q4_K_M", ctx_size=8192, batch_size=32)
    assert not plan.errors
    r0 = plan.ranks[0]
    pages = 32 * (8192 // 64 + 1) + 64
    kv_only = pages * 16 * 2 * 2 * 64 * 256 * 2                       # 16 softmax blocks, 2 of 4 KV heads per rank
    state = 33 * 4 * 48 * ((2 * 2048 + 24 * 128) * 3 + 24 * 128 * 128)  # 33 slots, 48 blocks, 24 value heads per rank
    assert r0.kv_bytes == kv_only + state
    # the dense 32B shape at the same settings holds four times the KV layers
    dense = build_plan(SHAPES["qwen3-32b"], lay, "Q4_K_M", ctx_size=8192, batch_size=32).ranks[0]
    assert dense.kv_bytes > r0.kv_bytes - state


def test_state_stride_lets_prompts_with_a_shorter_common_prefix_resume():
    """Two different prompts that share their first 130 tokens: with a snapshot every 64 tokens the second one resumes at
    128; with the default (one snapshot at the end of a prompt) it finds pages but no state and starts over."""
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.prefix_cache import PrefixCache, PrefixCacheConfig
    from llaminar_b200.engine.sampling import SamplingParams
    w = synthesize(SHAPES["tiny-qwen35"], "Q8_0", seed=7)
    shared = _prompt(130, 31)
    prompts = [shared + _prompt(90, 32), shared + _prompt(70, 33)]
    p = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    plain = [LLMEngine(w, device="cpu", max_batch=2, max_context=512).generate([q], p)[0] for q in prompts]
    for stride, want_hit in ((64, 128), (0, 0)):
        eng = LLMEngine(w, device="cpu", max_batch=2, max_context=512, prefix_cache=PrefixCache(PrefixCacheConfig(state_stride=stride)))
        got = [eng.generate([q], p)[0] for q in prompts]
        assert got == plain and eng.stats["prefix_hit_tokens"] == want_hit, stride


def test_prefix_cache_and_speculation_together_on_the_hybrid_model():
    """Chat turns with both switches on: the second turn resumes from the first prompt's snapshot and decodes with NextN
    drafts; answers equal those of a plain engine."""
    import dataclasses
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.mtp import MTPConfig, MTPDecoder
    from llaminar_b200.engine.prefix_cache import PrefixCache
    cfg = dataclasses.replace(SHAPES["tiny-qwen35"], nextn_layers=1, name="tiny-qwen35-mtp")
    w = synthesize(cfg, "Q8_0", seed=9)
    plain = _chat_turns(LLMEngine(w, device="cpu", max_batch=2, max_context=512))
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=512, prefix_cache=PrefixCache(), mtp=MTPDecoder(MTPConfig(draft_tokens=2)))
    assert _chat_turns(eng) == plain
    assert eng.stats["prefix_hit_tokens"] == 128 and eng.mtp.stats()["drafted"] > 0


def _pp_chat(rank, world):
    from llaminar_b200.engine.prefix_cache import PrefixCache
    from llaminar_b200.parallel.pp import build_pipeline_engine
    w = synthesize(SHAPES["tiny-qwen35"], "Q8_0", seed=7)
    layout = {"pp": 2, "tp": 1, "world": 2, "stages": [("s0", ["cpu"], 0, 2), ("s1", ["cpu"], 3, 7)]}
    eng = build_pipeline_engine(w, layout, rank, microbatch_tokens=64, device="cpu", max_batch=2, max_context=512, prefix_cache=PrefixCache())
    return _chat_turns(eng), eng.stats["prefix_hit_tokens"]


def test_pipeline_stages_agree_on_the_snapshot_boundary_of_a_hybrid_model():
    """Stage 0 holds linear-attention blocks only (no KV layer, three state layers), stage 1 the rest: both must cut the
    second turn's prefix hit back to the same snapshot boundary."""
    from llaminar_b200.engine.engine import LLMEngine
    from tests.mp_utils import run_ranks
    w = synthesize(SHAPES["tiny-qwen35"], "Q8_0", seed=7)
    plain = _chat_turns(LLMEngine(w, device="cpu", max_batch=2, max_context=512))
    res = run_ranks(_pp_chat, 2)
    assert res[0] == (plain, 128) and res[1] == (plain, 128)


def test_packed_prefill_attention_over_pages_matches_plain_attention():
    """Two sequences in one packed batch, head size 256, GQA 4:2: a fresh 70-row prompt and a 30-row chunk behind 100 cached
    positions, pages shuffled; against softmax attention written out per sequence."""
    from llaminar_b200.engine.cuda_model import paged_attention_torch
    torch.manual_seed(6)
    H, Hk, D = 4, 2, 256
    kv = torch.randn(9, 2, Hk, 64, D)
    bt = torch.tensor([[4, 1, 0], [7, 2, 5]], dtype=torch.int32)
    sid = torch.tensor([0] * 70 + [1] * 30, dtype=torch.int32)
    pos = torch.tensor(list(range(70)) + list(range(100, 130)), dtype=torch.int32)
    q = torch.randn(100, H, D)
    got = paged_attention_torch(q, kv, bt, sid, pos, D ** -0.5)
    for b, rows in ((0, range(0, 70)), (1, range(70, 100))):
        K = kv[bt[b].long(), 0].permute(1, 0, 2, 3).reshape(Hk, 192, D).repeat_interleave(H // Hk, 0)
        V = kv[bt[b].long(), 1].permute(1, 0, 2, 3).reshape(Hk, 192, D).repeat_interleave(H // Hk, 0)
        for r in rows:
            n = int(pos[r]) + 1
            p = torch.softmax(torch.einsum("hd,hld->hl", q[r], K[:, :n]) * D ** -0.5, -1)
            assert torch.allclose(got[r], torch.einsum("hl,hld->hd", p, V[:, :n]), atol=2e-5), r
