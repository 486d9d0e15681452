"""Byte-level BPE from GGUF metadata: merges, special tokens, streaming decode of split UTF-8."""
from llaminar_b200.tokenizer.bpe import BPETokenizer, StreamDecoder, byte_alphabet


def _tok():
    alpha = list(byte_alphabet())
    sp = alpha[ord(" ")]
    merges = ["h e", "l l", "he ll", "hell o", f"{sp} w", "o r", f"{sp}w or", "l d", f"{sp}wor ld"]
    tokens = alpha + ["he", "ll", "hell", "hello", f"{sp}w", "or", f"{sp}wor", "ld", f"{sp}world", "<|im_start|>", "<|im_end|>"]
    types = [1] * (len(tokens) - 2) + [3, 3]
    return BPETokenizer(tokens, merges, types, bos_id=None, eos_id=len(tokens) - 1)


def test_merges_apply_in_rank_order():
    t = _tok()
    ids = t.encode("hello world")
    assert [t.tokens[i] for i in ids] == ["hello", byte_alphabet()[ord(" ")] + "world"]
    assert t.decode(ids) == "hello world"


def test_special_tokens_are_atomic_and_optional():
    t = _tok()
    ids = t.encode("<|im_start|>hello<|im_end|>")
    assert t.tokens[ids[0]] == "<|im_start|>" and t.tokens[ids[-1]] == "<|im_end|>" and len(ids) == 3
    plain = t.encode("<|im_end|>", parse_special=False)
    assert len(plain) > 1 and t.decode(plain) == "<|im_end|>"
    assert t.decode(ids, skip_special=True) == "hello"
    assert t.is_special(ids[0]) and not t.is_special(ids[1])


def test_round_trip_unicode_and_stream_decoder():
    t = _tok()
    text = "héllo wörld ✓ 你好"
    ids = t.encode(text)
    assert t.decode(ids) == text
    dec = StreamDecoder(t)
    out = "".join(dec.push(i) for i in ids) + dec.flush()
    assert out == text                                           # multi-byte characters only appear once complete


def test_from_metadata_of_a_synthetic_model():
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.synth import synthesize
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=0)
    t = BPETokenizer.from_metadata(w.metadata)
    assert t.vocab_size == SHAPES["tiny-qwen3"].vocab_size and t.chat_template
    assert t.decode(t.encode("plain ascii text")) == "plain ascii text"
