"""Byte-level BPE from GGUF metadata: merges, special tokens, streaming decode of split UTF-8."""
import pytest

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


def test_chat_template_rendering_matches_the_transformers_renderer():
    """The same Jinja source rendered here and by `transformers` (its sandbox, filters and whitespace options): a Qwen3-style
    template with tool definitions, tool calls, tool results, thinking content and the generation prompt."""
    cu = pytest.importorskip("transformers.utils.chat_template_utils")
    from llaminar_b200.models.synth import CHATML_TEMPLATE
    from llaminar_b200.tokenizer.chat_template import ChatTemplate
    qwen3_like = (
        "{%- if tools %}{{- '<|im_start|>system\\n' }}{%- if messages[0].role == 'system' %}{{- messages[0].content + '\\n\\n' }}{%- endif %}"
        "{{- '# Tools\\n<tools>' }}{%- for tool in tools %}{{- '\\n' }}{{- tool | tojson }}{%- endfor %}{{- '\\n</tools><|im_end|>\\n' }}"
        "{%- elif messages[0].role == 'system' %}{{- '<|im_start|>system\\n' + messages[0].content + '<|im_end|>\\n' }}{%- endif %}"
        "{%- set ns = namespace(last_user=-1) %}"
        "{%- for m in messages %}{%- if m.role == 'user' %}{%- set ns.last_user = loop.index0 %}{%- endif %}{%- endfor %}"
        "{%- for message in messages %}"
        "{%- if message.role == 'user' or (message.role == 'system' and not loop.first) %}"
        "{{- '<|im_start|>' + message.role + '\\n' + message.content + '<|im_end|>\\n' }}"
        "{%- elif message.role == 'assistant' %}"
        "{%- set content = message.content or '' %}"
        "{%- if '</think>' in content %}{%- set content = content.split('</think>')[-1].lstrip('\\n') %}{%- endif %}"
        "{{- '<|im_start|>assistant\\n' + content }}"
        "{%- for tc in message.tool_calls or [] %}{{- '\\n<tool_call>\\n{\"name\": \"' + tc.function.name + '\", \"arguments\": ' }}"
        "{{- tc.function.arguments | tojson }}{{- '}\\n</tool_call>' }}{%- endfor %}{{- '<|im_end|>\\n' }}"
        "{%- elif message.role == 'tool' %}{{- '<|im_start|>user\\n<tool_response>\\n' + message.content + '\\n</tool_response><|im_end|>\\n' }}"
        "{%- endif %}{%- endfor %}"
        "{%- if add_generation_prompt %}{{- '<|im_start|>assistant\\n' }}"
        "{%- if enable_thinking is defined and enable_thinking is false %}{{- '<think>\\n\\n</think>\\n\\n' }}{%- endif %}{%- endif %}")
    tools = [{"type": "function", "function": {"name": "get_weather", "description": 'Weather for a <city> & country — "now"',
                                               "parameters": {"type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"]}}}]
    msgs = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "Wetter in Köln?"},
            {"role": "assistant", "content": "<think>\nneed a tool\n</think>\n\nLet me check.",
             "tool_calls": [{"type": "function", "function": {"name": "get_weather", "arguments": {"city": "Köln", "n": 2}}}]},
            {"role": "tool", "content": '{"temp": 7}'}, {"role": "user", "content": "thanks"}]
    for source in (CHATML_TEMPLATE, qwen3_like):
        for tl in (None, tools):
            for think in (True, False):
                want = cu.render_jinja_template([msgs], tools=tl, chat_template=source, add_generation_prompt=True, enable_thinking=think)[0]
                if isinstance(want, list):
                    want = want[0]
                got = ChatTemplate(source).render(msgs, tools=tl, add_generation_prompt=True, enable_thinking=think)
                assert got == want
