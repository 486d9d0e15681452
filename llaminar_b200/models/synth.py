"""Random-init checkpoints of a given shape, quantised to a GGUF recipe.

There are no downloadable checkpoints in the build/test environment, so every test and
benchmark model is drawn here: matrices N(0, 0.02) from a fixed seed, norm gains 1.0, then
encoded block by block with the codecs in :mod:`llaminar_b200.gguf.quants`.  Tensor names are
the GGUF names the reference maps (reference: src/v2/models/qwen/Qwen2Schema.h,
src/v2/execution/mtp/MTPWeightManifest.cpp:55-100).
"""
from __future__ import annotations

import torch

from ..gguf import GGMLType
from ..gguf.constants import BLOCK_GEOMETRY
from .config import RECIPES, ModelConfig, QuantRecipe
from .weights import ModelWeights, QTensor, qtensor_from_float


def _fit_type(qtype: GGMLType, cols: int) -> GGMLType:
    """Fall back to a finer-grained format when the row length does not fit the block size."""
    if cols % BLOCK_GEOMETRY[qtype][0] == 0:
        return qtype
    if cols % 32 == 0:
        return GGMLType.Q8_0
    return GGMLType.F16


def synthesize(cfg: ModelConfig, recipe: QuantRecipe | str = "Q8_0", seed: int = 0,
               device: str | torch.device = "cpu", std: float = 0.02,
               with_tokenizer: bool = True) -> ModelWeights:
    if isinstance(recipe, str):
        recipe = RECIPES[recipe]
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    tensors: dict[str, QTensor] = {}

    def mat(name: str, *shape: int, layer: int | None = None) -> None:
        qt = _fit_type(recipe.for_tensor(name, layer, cfg.n_layers), shape[-1])
        rows = 1
        for s in shape[:-1]:
            rows *= s
        # draw + encode in row chunks so multi-GB tensors never materialise in fp32 at once
        chunk_rows = max(1, (1 << 26) // shape[-1])
        parts = []
        for r0 in range(0, rows, chunk_rows):
            r1 = min(rows, r0 + chunk_rows)
            x = torch.randn(r1 - r0, shape[-1], generator=gen, device=dev, dtype=torch.float32) * std
            parts.append(qtensor_from_float(x, qt).raw)
        raw = parts[0] if len(parts) == 1 else torch.cat(parts)
        tensors[name] = QTensor(qt, tuple(shape), raw)

    def vec(name: str, n: int, value: float | None = 1.0) -> None:
        if value is None:
            x = torch.randn(n, generator=gen, device=dev, dtype=torch.float32) * std
        else:
            x = torch.full((n,), value, device=dev, dtype=torch.float32)
        tensors[name] = qtensor_from_float(x, GGMLType.F32)

    d, qd, kvd = cfg.d_model, cfg.q_dim, cfg.kv_dim
    mat("token_embd.weight", cfg.vocab_size, d)
    vec("output_norm.weight", d)
    if not cfg.tie_embeddings:
        mat("output.weight", cfg.vocab_size, d)

    def rand_vec(name: str, n: int, lo: float, hi: float, sign: float = 1.0) -> None:
        x = (torch.rand(n, generator=gen, device=dev, dtype=torch.float32) * (hi - lo) + lo) * sign
        tensors[name] = qtensor_from_float(x, GGMLType.F32)

    def gdn_layer(i: int) -> None:
        """Linear-attention block of the hybrid family (names: src/v2/models/qwen35/Qwen35Schema.h:107-134 of the reference).
        ssm_a holds -exp(A_log); the convolution taps are a [channels, kernel] matrix; value heads are in tiled order
        (value head j reads key head j mod n_k)."""
        p = f"blk.{i}."
        vec(p + "attn_norm.weight", d)
        mat(p + "attn_qkv.weight", cfg.gdn_conv_dim, d, layer=i)
        mat(p + "attn_gate.weight", cfg.gdn_value_dim, d, layer=i)
        mat(p + "ssm_alpha.weight", cfg.ssm_v_heads, d, layer=i)
        mat(p + "ssm_beta.weight", cfg.ssm_v_heads, d, layer=i)
        x = torch.randn(cfg.gdn_conv_dim, cfg.ssm_conv_kernel, generator=gen, device=dev, dtype=torch.float32) * 0.3
        tensors[p + "ssm_conv1d.weight"] = qtensor_from_float(x, GGMLType.F32)
        rand_vec(p + "ssm_dt.bias", cfg.ssm_v_heads, -1.0, 1.0)
        rand_vec(p + "ssm_a", cfg.ssm_v_heads, 0.5, 8.0, sign=-1.0)
        vec(p + "ssm_norm.weight", cfg.ssm_state)
        mat(p + "ssm_out.weight", d, cfg.gdn_value_dim, layer=i)
        vec(p + cfg.ffn_norm_name, d)
        ffn(i)

    def ffn(i: int) -> None:
        p = f"blk.{i}."
        if cfg.is_moe:
            mat(p + "ffn_gate_inp.weight", cfg.n_experts, d, layer=i)
            mat(p + "ffn_gate_exps.weight", cfg.n_experts, cfg.expert_ff, d, layer=i)
            mat(p + "ffn_up_exps.weight", cfg.n_experts, cfg.expert_ff, d, layer=i)
            mat(p + "ffn_down_exps.weight", cfg.n_experts, d, cfg.expert_ff, layer=i)
            if cfg.shared_expert_ff:
                mat(p + "ffn_gate_shexp.weight", cfg.shared_expert_ff, d, layer=i)
                mat(p + "ffn_up_shexp.weight", cfg.shared_expert_ff, d, layer=i)
                mat(p + "ffn_down_shexp.weight", d, cfg.shared_expert_ff, layer=i)
                x = torch.randn(d, generator=gen, device=dev, dtype=torch.float32) * 0.2
                tensors[p + "ffn_gate_inp_shexp.weight"] = qtensor_from_float(x, GGMLType.F32)
        else:
            mat(p + "ffn_gate.weight", cfg.d_ff, d, layer=i)
            mat(p + "ffn_up.weight", cfg.d_ff, d, layer=i)
            mat(p + "ffn_down.weight", d, cfg.d_ff, layer=i)

    def decoder_layer(i: int) -> None:
        if cfg.is_gdn_layer(i):
            return gdn_layer(i)
        p = f"blk.{i}."
        vec(p + "attn_norm.weight", d)
        mat(p + "attn_q.weight", qd * (2 if cfg.attn_gate else 1), d, layer=i)
        mat(p + "attn_k.weight", kvd, d, layer=i)
        mat(p + "attn_v.weight", kvd, d, layer=i)
        mat(p + "attn_output.weight", d, qd, layer=i)
        if cfg.qkv_bias:
            vec(p + "attn_q.bias", qd, None)
            vec(p + "attn_k.bias", kvd, None)
            vec(p + "attn_v.bias", kvd, None)
        if cfg.qk_norm:
            vec(p + "attn_q_norm.weight", cfg.head_dim)
            vec(p + "attn_k_norm.weight", cfg.head_dim)
        vec(p + cfg.ffn_norm_name, d)
        ffn(i)

    for i in range(cfg.n_layers):
        decoder_layer(i)
    for j in range(cfg.nextn_layers):
        i = cfg.n_layers + j
        decoder_layer(i)
        p = f"blk.{i}.nextn."
        mat(p + "eh_proj.weight", d, 2 * d, layer=i)
        vec(p + "enorm.weight", d)
        vec(p + "hnorm.weight", d)
        vec(p + "shared_head_norm.weight", d)

    md = {}
    if with_tokenizer:
        md.update(byte_tokenizer_metadata(cfg.vocab_size))
    return ModelWeights(cfg, tensors, md)


def byte_tokenizer_metadata(vocab_size: int) -> dict:
    """A self-contained byte-level BPE vocabulary for synthetic checkpoints.

    Tokens 0..255 are the GPT-2 byte alphabet, the last five ids are chat control tokens, the
    rest are filler pieces that never result from a merge.  Enough for `serve`/`oneshot` to run
    end-to-end on a random-weight model.
    """
    from ..tokenizer.bpe import byte_alphabet
    alphabet = byte_alphabet()
    tokens = [alphabet[b] for b in range(256)]
    n_special = 5
    while len(tokens) < vocab_size - n_special:
        tokens.append(f"<|filler_{len(tokens)}|>")
    specials = ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>"]
    types = [1] * len(tokens)
    for s in specials:
        tokens.append(s)
        types.append(3)
    tokens, types = tokens[:vocab_size], types[:vocab_size]
    for i in range(256, max(256, vocab_size - n_special)):
        if i < len(types):
            types[i] = 5          # unused
    eos = tokens.index("<|im_end|>") if "<|im_end|>" in tokens else 0
    bos = tokens.index("<|endoftext|>") if "<|endoftext|>" in tokens else 0
    return {
        "tokenizer.ggml.model": "gpt2",
        "tokenizer.ggml.pre": "qwen2",
        "tokenizer.ggml.tokens": tokens,
        "tokenizer.ggml.token_type": types,
        "tokenizer.ggml.merges": [],
        "tokenizer.ggml.eos_token_id": eos,
        "tokenizer.ggml.bos_token_id": bos,
        "tokenizer.ggml.padding_token_id": bos,
        "tokenizer.chat_template": CHATML_TEMPLATE,
    }


CHATML_TEMPLATE = (
    "{%- if tools %}{{- '<|im_start|>system\\n' }}"
    "{%- if messages[0].role == 'system' %}{{- messages[0].content + '\\n\\n' }}{%- endif %}"
    "{{- '# Tools\\n\\nYou may call one or more functions to assist with the user query.\\n\\n"
    "You are provided with function signatures within <tools></tools> XML tags:\\n<tools>' }}"
    "{%- for tool in tools %}{{- '\\n' }}{{- tool | tojson }}{%- endfor %}"
    "{{- '\\n</tools>\\n\\nFor each function call, return a json object with function name and arguments "
    "within <tool_call></tool_call> XML tags:\\n<tool_call>\\n{\\\"name\\\": <function-name>, "
    "\\\"arguments\\\": <args-json-object>}\\n</tool_call><|im_end|>\\n' }}"
    "{%- elif messages[0].role == 'system' %}"
    "{{- '<|im_start|>system\\n' + messages[0].content + '<|im_end|>\\n' }}{%- endif %}"
    "{%- for message in messages %}"
    "{%- if message.role == 'system' and loop.first %}"
    "{%- else %}{{- '<|im_start|>' + message.role + '\\n' + (message.content or '') + '<|im_end|>\\n' }}{%- endif %}"
    "{%- endfor %}"
    "{%- if add_generation_prompt %}{{- '<|im_start|>assistant\\n' }}"
    "{%- if enable_thinking is defined and enable_thinking is false %}{{- '<think>\\n\\n</think>\\n\\n' }}{%- endif %}"
    "{%- endif %}"
)
