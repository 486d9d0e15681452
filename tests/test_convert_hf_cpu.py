"""Hugging Face checkpoint -> GGUF conversion: for every family the engine runs, a tiny random model saved with
`save_pretrained` is converted, loaded back from the GGUF file and run through the fp32 oracle; logits must equal the
`transformers` model's.  Plus the tokenizer carry-over."""
import json

import pytest
import torch

from llaminar_b200.models.convert_hf import config_from_hf, convert_directory, tokenizer_metadata
from llaminar_b200.models.reference import ReferenceModel
from llaminar_b200.models.weights import ModelWeights

tf = pytest.importorskip("transformers")


def _tiny(family: str):
    common = dict(hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, vocab_size=128,
                  max_position_embeddings=512, rms_norm_eps=1e-6, tie_word_embeddings=False)
    hybrid = dict(head_dim=32, layer_types=["linear_attention"] * 3 + ["full_attention"], full_attention_interval=4,
                  linear_key_head_dim=16, linear_value_head_dim=16, linear_num_key_heads=2, linear_num_value_heads=4,
                  linear_conv_kernel_dim=4,
                  rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.25, "mrope_section": [2, 1, 1]})
    try:
        if family == "qwen2":
            from transformers import Qwen2Config, Qwen2ForCausalLM
            return Qwen2ForCausalLM(Qwen2Config(**common, intermediate_size=256))
        if family == "qwen3":
            from transformers import Qwen3Config, Qwen3ForCausalLM
            return Qwen3ForCausalLM(Qwen3Config(**common, head_dim=16, intermediate_size=256))
        if family == "qwen3_moe":
            from transformers import Qwen3MoeConfig, Qwen3MoeForCausalLM
            return Qwen3MoeForCausalLM(Qwen3MoeConfig(**common, head_dim=16, intermediate_size=256, moe_intermediate_size=32, num_experts=6,
                                                      num_experts_per_tok=2, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[]))
        if family == "qwen3_5":
            from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5ForCausalLM, Qwen3_5TextConfig
            return Qwen3_5ForCausalLM(Qwen3_5TextConfig(**common, **hybrid, intermediate_size=256))
        from transformers.models.qwen3_5_moe.modeling_qwen3_5_moe import Qwen3_5MoeForCausalLM, Qwen3_5MoeTextConfig
        return Qwen3_5MoeForCausalLM(Qwen3_5MoeTextConfig(**common, **hybrid, num_experts=6, num_experts_per_tok=2,
                                                          moe_intermediate_size=32, shared_expert_intermediate_size=48))
    except ImportError as e:
        pytest.skip(f"this transformers has no {family}: {e}")


@pytest.mark.parametrize("family", ["qwen2", "qwen3", "qwen3_moe", "qwen3_5", "qwen3_5_moe"])
def test_converted_checkpoint_reproduces_the_transformers_logits(family, tmp_path):
    torch.manual_seed(7)
    m = _tiny(family).float().eval()
    m.config._attn_implementation = "eager"
    with torch.no_grad():
        for n, p in m.named_parameters():                       # nothing left at its constructor value (zeros, ones, empty)
            p.copy_(torch.randn_like(p) * (0.3 if p.dim() == 1 else 0.08))
            if n.endswith("A_log"):
                p.copy_(torch.log(torch.rand_like(p) * 6 + 0.5))
    src, out = tmp_path / "hf", str(tmp_path / "m.gguf")
    m.save_pretrained(src, safe_serialization=True)
    convert_directory(str(src), out, "F32")
    w = ModelWeights.from_gguf(out)
    assert w.config.arch == {"qwen2": "qwen2", "qwen3": "qwen3", "qwen3_moe": "qwen3moe", "qwen3_5": "qwen35", "qwen3_5_moe": "qwen35moe"}[family]
    toks = torch.randint(0, 128, (33,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = m(input_ids=toks[None]).logits[0]
    got, _, _ = ReferenceModel(w).forward(toks)
    assert (got - want).abs().max() < 3e-4 * max(1.0, float(want.abs().max()))


def test_quantised_recipe_and_config_mapping(tmp_path):
    m = _tiny("qwen3_5").float().eval()
    src, out = tmp_path / "hf", str(tmp_path / "q.gguf")
    m.save_pretrained(src, safe_serialization=True)
    w = convert_directory(str(src), out, "Q8_0")
    assert w["blk.0.attn_qkv.weight"].qtype.name == "Q8_0" and w["blk.0.ssm_a"].qtype.name == "F32"
    c = config_from_hf(json.load(open(src / "config.json")))
    assert (c.full_attention_interval, c.ssm_k_heads, c.ssm_v_heads, c.ssm_state, c.rope_dim, c.attn_gate) == (4, 2, 4, 16, 8, True)
    with pytest.raises(ValueError, match="model_type"):
        config_from_hf({"model_type": "llama"})


def test_tokenizer_files_become_gguf_tokenizer_metadata(tmp_path):
    from llaminar_b200.tokenizer.bpe import BPETokenizer, byte_alphabet
    alpha = byte_alphabet()
    vocab = {alpha[b]: b for b in range(256)}
    he = alpha[ord("h")] + alpha[ord("e")]
    vocab[he] = 256
    rx = r"[\p{L}\p{M}]+|\p{N}|\s+|[^\s\p{L}\p{M}\p{N}]+"
    tj = {"model": {"type": "BPE", "vocab": vocab, "merges": [[alpha[ord("h")], alpha[ord("e")]]]},
          "pre_tokenizer": {"type": "Sequence", "pretokenizers": [{"type": "Split", "pattern": {"Regex": rx}, "behavior": "Isolated"},
                                                                  {"type": "ByteLevel", "add_prefix_space": False}]},
          "added_tokens": [{"id": 257, "content": "<|im_end|>", "special": True}, {"id": 259, "content": "<tool>", "special": False}]}
    json.dump(tj, open(tmp_path / "tokenizer.json", "w"))
    json.dump({"eos_token": {"content": "<|im_end|>"}, "chat_template": "{{ messages }}"}, open(tmp_path / "tokenizer_config.json", "w"))
    md = tokenizer_metadata(str(tmp_path))
    assert len(md["tokenizer.ggml.tokens"]) == 260 and md["tokenizer.ggml.token_type"][257] == 3
    assert md["tokenizer.ggml.token_type"][258] == 5 and md["tokenizer.ggml.token_type"][259] == 4
    assert md["tokenizer.ggml.eos_token_id"] == 257 and md["tokenizer.chat_template"] == "{{ messages }}"
    assert md["tokenizer.llaminar.split_regex"] == rx and md["tokenizer.ggml.pre"] == "qwen35"      # the file's own expression
    tok = BPETokenizer.from_metadata(md)
    assert tok._split_re.pattern == rx
    ids = tok.encode("hehe<|im_end|>")
    assert ids == [256, 256, 257] and tok.decode(ids[:2]) == "hehe"
    assert tokenizer_metadata(str(tmp_path / "nowhere")) == {}


def test_requantising_a_gguf_file_keeps_the_model_function(tmp_path):
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.convert_hf import main
    from llaminar_b200.models.synth import synthesize
    src, dst = str(tmp_path / "a.gguf"), str(tmp_path / "b.gguf")
    w = synthesize(SHAPES["tiny-qwen35"], "F32", seed=3)
    w.save_gguf(src)
    assert main([src, dst, "--recipe", "Q8_0"]) == 0
    back = ModelWeights.from_gguf(dst)
    assert back["blk.0.attn_qkv.weight"].qtype.name == "Q8_0" and back["blk.0.ssm_conv1d.weight"].qtype.name == "F32"
    assert back.metadata.get("tokenizer.ggml.model") == "gpt2"
    toks = torch.randint(0, 1024, (24,), generator=torch.Generator().manual_seed(2))
    a, _, _ = ReferenceModel(w).forward(toks)
    b, _, _ = ReferenceModel(back).forward(toks)
    assert torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0) > 0.995      # Q8_0 rounding through eight blocks


def test_multi_token_prediction_blocks_of_a_checkpoint_become_nextn_blocks():
    """Checkpoints keep the NextN head under `mtp.` (shared projection and norms + one decoder block per depth); the library
    model drops it on load, so the tensors are fabricated here from block 3 of a tiny hybrid model.  The converted file
    must describe one NextN layer, and an engine that drafts with it must decode exactly like one that does not."""
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.mtp import MTPConfig, MTPDecoder
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.convert_hf import convert_state_dict
    torch.manual_seed(5)
    m = _tiny("qwen3_5").float().eval()
    sd = {k: v.detach().clone() for k, v in m.state_dict().items()}
    for k in [k for k in sd if k.startswith("model.layers.3.")]:
        sd["mtp.layers.0." + k[len("model.layers.3."):]] = torch.randn_like(sd[k]) * 0.05
    d = m.config.hidden_size
    sd.update({"mtp.fc.weight": torch.randn(d, 2 * d) * 0.05, "mtp.norm.weight": torch.zeros(d),
               "mtp.pre_fc_norm_embedding.weight": torch.zeros(d), "mtp.pre_fc_norm_hidden.weight": torch.randn(d) * 0.1})
    w = convert_state_dict(config_from_hf(m.config.to_dict()), sd, "F32")
    c = w.config
    assert c.nextn_layers == 1 and w["blk.4.nextn.eh_proj.weight"].shape == (d, 2 * d)
    assert torch.equal(w["blk.4.nextn.enorm.weight"].to_float(), torch.ones(d))            # zero-centred gain stored as 1 + w
    assert "blk.4.attn_q.weight" in w and "blk.4.post_attention_norm.weight" in w and "blk.4.attn_qkv.weight" not in w
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 128, (n,), generator=g).tolist() for n in (30, 50)]
    p = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    plain = LLMEngine(w, device="cpu", max_batch=2, max_context=128).generate(prompts, p)
    spec = LLMEngine(w, device="cpu", max_batch=2, max_context=128, mtp=MTPDecoder(MTPConfig(draft_tokens=2)))
    assert spec.generate(prompts, p) == plain and spec.mtp.stats()["drafted"] > 0


def test_converted_tokenizer_encodes_like_the_tokenizers_library(tmp_path):
    """A byte-level BPE vocabulary trained with the `tokenizers` library (Qwen-style pre-tokeniser with combining marks
    counted as letters, two special tokens), written as tokenizer.json, carried into GGUF metadata: this package's tokenizer
    must give the library's ids on mixed text, and decode them back."""
    tk = pytest.importorskip("tokenizers")
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers
    from llaminar_b200.tokenizer.bpe import BPETokenizer, SPLIT_BY_NAME
    t = Tokenizer(models.BPE())
    t.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(SPLIT_BY_NAME["qwen35"]), behavior="isolated"),
                                               pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    t.decoder = decoders.ByteLevel()
    corpus = ["The quick brown fox jumps over the lazy dog. " * 3, "def add(a, b):\\n    return a + b\\n", "Zwölf Boxkämpfer jagen Viktor quer",
              "über den großen Sylter Deich 12345 67890", "naïve café déjà vu — “quotes” and… ellipses", "它们是中文字符，日本語のテキスト",
              "I'm sure they've said we'll go; it's what he'd do.", "été with combining marks"] * 4
    t.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=420, special_tokens=["<|im_start|>", "<|im_end|>"],
                                                      initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False))
    t.save(str(tmp_path / "tokenizer.json"))
    ours = BPETokenizer.from_metadata(tokenizer_metadata(str(tmp_path)))
    samples = ["Hello, world! It's 2026.", "<|im_start|>user\\nZwölf   Boxkämpfer\\n\\n<|im_end|>", "  leading and trailing  ", "tabs\\tand\\r\\nnewlines",
               "été naïve 中文 12 345", "x = {'a': [1, 2, 3]}  # comment"]
    for text in samples:
        want = t.encode(text, add_special_tokens=False).ids
        got = ours.encode(text)
        assert got == want, text
        assert ours.decode(got) == text


@pytest.mark.parametrize("family", ["qwen2", "qwen3", "qwen3_moe", "qwen3_5", "qwen3_5_moe"])
def test_engine_on_a_converted_checkpoint_generates_what_transformers_generates(family, tmp_path):
    """End to end: converter, GGUF file, loader, CPU runner, paged cache (and state slots for the hybrid families), scheduler
    and greedy sampler against `generate(do_sample=False)` of the library model, two prompts batched."""
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    torch.manual_seed(11)
    m = _tiny(family).float().eval()
    m.config._attn_implementation = "eager"
    with torch.no_grad():
        for n, p in m.named_parameters():
            p.copy_(torch.randn_like(p) * (0.3 if p.dim() == 1 else 0.1))
            if n.endswith("A_log"):
                p.copy_(torch.log(torch.rand_like(p) * 6 + 0.5))
    src, out = tmp_path / "hf", str(tmp_path / "m.gguf")
    m.save_pretrained(src, safe_serialization=True)
    convert_directory(str(src), out, "F32")
    eng = LLMEngine(ModelWeights.from_gguf(out), device="cpu", max_batch=2, max_context=128, max_prefill_tokens=24)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 128, (n,), generator=g).tolist() for n in (19, 40)]
    got = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for pr, o in zip(prompts, got):
        with torch.no_grad():
            want = m.generate(torch.tensor([pr]), max_new_tokens=10, do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(pr):].tolist()
        assert o == want
