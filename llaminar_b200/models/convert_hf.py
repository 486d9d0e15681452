"""Hugging Face checkpoint (config.json + *.safetensors) -> GGUF, for the families this engine runs.

    python -m llaminar_b200.models.convert_hf <model directory> <out.gguf> [--recipe Q4_K_M]
    python -m llaminar_b200.models.convert_hf <in.gguf> <out.gguf> --recipe Q4_K_M        # re-encode an existing GGUF file

Tensor names, metadata keys and storage conventions are the ones GGUF files of these families use (and the loader here and
the reference expect: src/v2/models/qwen/Qwen2Schema.h, src/v2/models/qwen35/Qwen35Schema.h:107-134,
python/reference/qwen35.py:13-19 of the reference):

* qwen2 / qwen3 / qwen3_moe: projections and norms under their GGUF names; the experts of a MoE block as three stacked
  tensors (`ffn_{gate,up,down}_exps`).
* qwen3_5 / qwen3_5_moe (hybrid): zero-centred RMSNorm gains are stored as ``1 + w``; ``ssm_a`` holds ``-exp(A_log)``; the
  convolution taps as a [channels, kernel] matrix; the value heads of the linear-attention blocks in *tiled* order (GGUF value
  head ``r * n_k + kh`` is the checkpoint's value head ``kh * rep + r``, so that head j reads key head j mod n_k), applied to
  every per-value-head tensor; q and gate of a softmax block stay interleaved per head in ``attn_q``; the shared expert's gate
  vector as ``ffn_gate_inp_shexp``.

Weights are re-encoded to the chosen recipe with the block encoders of `llaminar_b200.gguf.quants` (norms, biases and the
small state-space vectors stay fp32).  The tokenizer (``tokenizer.json`` byte-level BPE, special tokens, chat template) is
carried over when the directory has one.
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Mapping

import torch

from ..gguf import GGMLType
from ..gguf.constants import BLOCK_GEOMETRY
from .config import RECIPES, ModelConfig, QuantRecipe
from .weights import ModelWeights, QTensor, qtensor_from_float

_ARCH = {"qwen2": "qwen2", "qwen3": "qwen3", "qwen3_moe": "qwen3moe", "qwen3_5": "qwen35", "qwen3_5_text": "qwen35",
         "qwen3_5_moe": "qwen35moe", "qwen3_5_moe_text": "qwen35moe"}


def config_from_hf(hf: dict) -> ModelConfig:
    """`config.json` (or its `text_config` for the multimodal wrappers) -> ModelConfig."""
    hf = hf.get("text_config", hf)
    mt = hf.get("model_type", "")
    if mt not in _ARCH:
        raise ValueError(f"model_type '{mt}' is not one of {sorted(_ARCH)}")
    arch = _ARCH[mt]
    rope = hf.get("rope_parameters") or {}
    n_heads = hf["num_attention_heads"]
    head_dim = hf.get("head_dim") or hf["hidden_size"] // n_heads
    kw = dict(arch=arch, name=hf.get("_name_or_path") or mt, n_layers=hf["num_hidden_layers"], d_model=hf["hidden_size"],
              n_heads=n_heads, n_kv_heads=hf.get("num_key_value_heads", n_heads), head_dim=head_dim,
              d_ff=hf.get("intermediate_size", 0), vocab_size=hf["vocab_size"],
              rope_theta=float(rope.get("rope_theta", hf.get("rope_theta", 10000.0))), rms_eps=float(hf.get("rms_norm_eps", 1e-6)),
              context_length=int(hf.get("max_position_embeddings", 4096)), tie_embeddings=bool(hf.get("tie_word_embeddings", False)),
              qk_norm=arch != "qwen2", qkv_bias=arch == "qwen2")
    if arch in ("qwen3moe", "qwen35moe"):
        kw.update(n_experts=hf.get("num_experts", hf.get("num_local_experts", 0)), n_experts_used=hf["num_experts_per_tok"],
                  expert_ff=hf["moe_intermediate_size"], d_ff=0)
        if hf.get("mlp_only_layers") or hf.get("decoder_sparse_step", 1) != 1:
            raise ValueError("checkpoints that mix dense and MoE FFN blocks are not supported")
    if arch.startswith("qwen35"):
        types = hf.get("layer_types") or []
        interval = int(hf.get("full_attention_interval", 4))
        if types and types != ["full_attention" if (i + 1) % interval == 0 else "linear_attention" for i in range(len(types))]:
            raise ValueError("layer_types does not follow full_attention_interval")
        kw.update(full_attention_interval=interval, ssm_conv_kernel=hf.get("linear_conv_kernel_dim", 4),
                  ssm_state=hf["linear_key_head_dim"], ssm_k_heads=hf["linear_num_key_heads"], ssm_v_heads=hf["linear_num_value_heads"],
                  rope_dim=int(head_dim * float(rope.get("partial_rotary_factor", hf.get("partial_rotary_factor", 1.0)))), attn_gate=True)
        if hf["linear_key_head_dim"] != hf["linear_value_head_dim"]:
            raise ValueError("linear_key_head_dim != linear_value_head_dim is not supported")
        if arch == "qwen35moe":
            kw["shared_expert_ff"] = hf.get("shared_expert_intermediate_size", 0)
    return ModelConfig(**kw)


def tiled_value_heads(n_k: int, n_v: int) -> list[int]:
    """GGUF value head i holds the checkpoint's value head (i mod n_k) * rep + i div n_k."""
    rep = n_v // n_k
    return [(i % n_k) * rep + i // n_k for i in range(n_v)]


def _fit(qt: GGMLType, cols: int) -> GGMLType:
    if cols % BLOCK_GEOMETRY[qt][0] == 0:
        return qt
    return GGMLType.Q8_0 if cols % 32 == 0 else GGMLType.F16


def convert_state_dict(cfg: ModelConfig, sd: Mapping[str, torch.Tensor], recipe: QuantRecipe | str = "F32") -> ModelWeights:
    """Tensors of a `...ForCausalLM` state dict (any floating dtype) -> ModelWeights in GGUF conventions."""
    if isinstance(recipe, str):
        recipe = RECIPES[recipe]
    emb_key = next(k for k in sd if k.endswith("embed_tokens.weight"))
    root = emb_key[:-len("embed_tokens.weight")]                  # "model." or "model.language_model."
    get = lambda name: sd[name].detach().float()
    hybrid = cfg.arch.startswith("qwen35")
    gain = (lambda x: 1.0 + x) if hybrid else (lambda x: x)       # zero-centred norm gains are stored as 1 + w
    out: dict[str, QTensor] = {}

    def mat(name: str, x: torch.Tensor, layer: int | None = None) -> None:
        qt = _fit(recipe.for_tensor(name, layer, cfg.n_layers), x.shape[-1])
        out[name] = qtensor_from_float(x.contiguous(), qt)

    def vec(name: str, x: torch.Tensor) -> None:
        out[name] = qtensor_from_float(x.contiguous(), GGMLType.F32)

    mat("token_embd.weight", get(emb_key))
    vec("output_norm.weight", gain(get(root + "norm.weight")))
    if not cfg.tie_embeddings:
        head = next((k for k in ("lm_head.weight", root.replace("model.", "", 1) + "lm_head.weight") if k in sd), None)
        if head is None:
            raise KeyError("lm_head.weight is missing and tie_word_embeddings is false")
        mat("output.weight", get(head))
    d, n_k, n_v = cfg.ssm_state, cfg.ssm_k_heads, cfg.ssm_v_heads
    if hybrid:
        perm = torch.tensor(tiled_value_heads(n_k, n_v))
        vrows = (perm[:, None] * d + torch.arange(d)[None, :]).reshape(-1)
    def block(s: str, i: int) -> None:
        """One decoder block: checkpoint prefix ``s`` -> GGUF block ``i``."""
        p = f"blk.{i}."
        vec(p + "attn_norm.weight", gain(get(s + "input_layernorm.weight")))
        vec(p + cfg.ffn_norm_name, gain(get(s + "post_attention_layernorm.weight")))
        if cfg.is_gdn_layer(i):
            la, kd = s + "linear_attn.", cfg.gdn_key_dim
            qkv, conv = get(la + "in_proj_qkv.weight"), get(la + "conv1d.weight").squeeze(1)
            mat(p + "attn_qkv.weight", torch.cat([qkv[:2 * kd], qkv[2 * kd:][vrows]]), i)
            mat(p + "attn_gate.weight", get(la + "in_proj_z.weight")[vrows], i)
            mat(p + "ssm_alpha.weight", get(la + "in_proj_a.weight")[perm], i)
            mat(p + "ssm_beta.weight", get(la + "in_proj_b.weight")[perm], i)
            vec(p + "ssm_conv1d.weight", torch.cat([conv[:2 * kd], conv[2 * kd:][vrows]]))
            vec(p + "ssm_dt.bias", get(la + "dt_bias")[perm])
            vec(p + "ssm_a", -torch.exp(get(la + "A_log")[perm]))
            vec(p + "ssm_norm.weight", get(la + "norm.weight"))
            mat(p + "ssm_out.weight", get(la + "out_proj.weight")[:, vrows], i)
        else:
            sa = s + "self_attn."
            for g, h in (("q", "q_proj"), ("k", "k_proj"), ("v", "v_proj"), ("output", "o_proj")):
                mat(p + f"attn_{g}.weight", get(sa + h + ".weight"), i)
                if cfg.qkv_bias and g != "output":
                    vec(p + f"attn_{g}.bias", get(sa + h + ".bias"))
            if cfg.qk_norm:
                vec(p + "attn_q_norm.weight", gain(get(sa + "q_norm.weight")))
                vec(p + "attn_k_norm.weight", gain(get(sa + "k_norm.weight")))
        m = s + "mlp."
        if cfg.is_moe:
            mat(p + "ffn_gate_inp.weight", get(m + "gate.weight"), i)
            if m + "experts.gate_up_proj" in sd:                               # stacked [E, 2 ff, d] / [E, d, ff]
                gu, ff = get(m + "experts.gate_up_proj"), cfg.expert_ff
                ge, ue, de = gu[:, :ff], gu[:, ff:], get(m + "experts.down_proj")
            else:                                                              # one module per expert
                ge, ue, de = (torch.stack([get(f"{m}experts.{e}.{n}.weight") for e in range(cfg.n_experts)])
                              for n in ("gate_proj", "up_proj", "down_proj"))
            mat(p + "ffn_gate_exps.weight", ge, i)
            mat(p + "ffn_up_exps.weight", ue, i)
            mat(p + "ffn_down_exps.weight", de, i)
            if cfg.shared_expert_ff:
                for g in ("gate", "up", "down"):
                    mat(p + f"ffn_{g}_shexp.weight", get(m + f"shared_expert.{g}_proj.weight"), i)
                vec(p + "ffn_gate_inp_shexp.weight", get(m + "shared_expert_gate.weight").reshape(-1))
        else:
            for g in ("gate", "up", "down"):
                mat(p + f"ffn_{g}.weight", get(m + f"{g}_proj.weight"), i)

    for i in range(cfg.n_layers):
        block(f"{root}layers.{i}.", i)
    # multi-token-prediction (NextN) blocks, kept by checkpoints under `mtp.`: every GGUF NextN block carries the shared
    # projection and norms beside its own decoder block (names: src/v2/execution/mtp/MTPWeightManifest.cpp:55-100 of the reference)
    n_mtp = len({k.split(".")[2] for k in sd if k.startswith("mtp.layers.")})
    for j in range(n_mtp):
        i = cfg.n_layers + j
        block(f"mtp.layers.{j}.", i)
        mat(f"blk.{i}.nextn.eh_proj.weight", get("mtp.fc.weight"), i)
        vec(f"blk.{i}.nextn.enorm.weight", gain(get("mtp.pre_fc_norm_embedding.weight")))
        vec(f"blk.{i}.nextn.hnorm.weight", gain(get("mtp.pre_fc_norm_hidden.weight")))
        vec(f"blk.{i}.nextn.shared_head_norm.weight", gain(get("mtp.norm.weight")))
    if n_mtp:
        cfg = cfg.with_(nextn_layers=n_mtp)
    return ModelWeights(cfg, out)


def tokenizer_metadata(model_dir: str) -> dict:
    """`tokenizer.json` (byte-level BPE) + `tokenizer_config.json` -> the `tokenizer.ggml.*` keys; {} without a tokenizer."""
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.exists(path):
        return {}
    tj = json.load(open(path, encoding="utf-8"))
    model = tj.get("model", {})
    if model.get("type") != "BPE":
        raise ValueError(f"tokenizer model '{model.get('type')}' is not BPE")
    vocab = dict(model["vocab"])
    added = {a["content"]: a for a in tj.get("added_tokens", [])}
    for content, a in added.items():
        vocab.setdefault(content, a["id"])
    n = max(vocab.values()) + 1
    tokens, types = [f"[PAD{i}]" for i in range(n)], [5] * n          # unused ids keep a placeholder of type "unused"
    for t, i in vocab.items():
        tokens[i] = t
        types[i] = 3 if t in added and added[t].get("special", True) else (4 if t in added else 1)     # control / user-defined / normal
    merges = [m if isinstance(m, str) else " ".join(m) for m in model.get("merges", [])]
    md = {"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.pre": "qwen2", "tokenizer.ggml.tokens": tokens,
          "tokenizer.ggml.token_type": types, "tokenizer.ggml.merges": merges}
    # the pre-tokeniser's expression itself, when the file states one: exact for any byte-level BPE vocabulary
    pre = tj.get("pre_tokenizer") or {}
    for part in (pre.get("pretokenizers") or [pre]):
        rx = (part.get("pattern") or {}).get("Regex") if part.get("type") == "Split" else None
        if rx:
            md["tokenizer.llaminar.split_regex"] = rx
            if "\\p{M}" in rx:
                md["tokenizer.ggml.pre"] = "qwen35"
            break
    cfg_path = os.path.join(model_dir, "tokenizer_config.json")
    if os.path.exists(cfg_path):
        tc = json.load(open(cfg_path, encoding="utf-8"))
        text = lambda v: v.get("content") if isinstance(v, dict) else v
        for key, field in (("eos_token_id", "eos_token"), ("bos_token_id", "bos_token"), ("padding_token_id", "pad_token")):
            t = text(tc.get(field))
            if t in vocab:
                md[f"tokenizer.ggml.{key}"] = vocab[t]
        if tc.get("chat_template"):
            md["tokenizer.chat_template"] = tc["chat_template"]
    return md


class _LazyTensors(Mapping):
    """Tensor name -> tensor over the `.safetensors` files of a directory; a tensor is read when it is asked for, so a
    conversion never holds the whole unquantised checkpoint."""

    def __init__(self, model_dir: str):
        from safetensors import safe_open
        self._files, self._where = {}, {}
        for name in sorted(os.listdir(model_dir)):
            if name.endswith(".safetensors"):
                f = safe_open(os.path.join(model_dir, name), framework="pt")
                self._files[name] = f
                for k in f.keys():
                    self._where[k] = name
        if not self._where:
            raise FileNotFoundError(f"no .safetensors file in {model_dir}")

    def __getitem__(self, key: str) -> torch.Tensor:
        return self._files[self._where[key]].get_tensor(key)

    def __iter__(self):
        return iter(self._where)

    def __len__(self) -> int:
        return len(self._where)


def load_checkpoint(model_dir: str) -> tuple[dict, Mapping]:
    """(config.json as a dict, {tensor name: tensor}, read lazily) of a directory with one or several `.safetensors` files."""
    hf = json.load(open(os.path.join(model_dir, "config.json"), encoding="utf-8"))
    return hf, _LazyTensors(model_dir)


def requantize(w: ModelWeights, recipe: QuantRecipe | str) -> ModelWeights:
    """The same checkpoint with every matrix re-encoded to ``recipe`` (decode, then encode; vectors and metadata are kept).
    Going from a coarser to a finer format does not bring precision back."""
    if isinstance(recipe, str):
        recipe = RECIPES[recipe]
    cfg, out = w.config, {}
    for name, t in w.tensors.items():
        layer = int(name.split(".")[1]) if name.startswith("blk.") else None
        if len(t.shape) < 2 or "ssm_conv1d" in name:
            out[name] = t
        else:
            out[name] = t.transcoded(_fit(recipe.for_tensor(name, layer, cfg.n_layers), t.shape[-1]))
    return ModelWeights(cfg, out, dict(w.metadata))


def convert_directory(model_dir: str, out_path: str, recipe: str = "Q8_0") -> ModelWeights:
    hf, sd = load_checkpoint(model_dir)
    cfg = config_from_hf(hf)
    w = convert_state_dict(cfg, sd, recipe)
    w.metadata.update(tokenizer_metadata(model_dir))
    w.save_gguf(out_path)
    return w


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("model_dir")
    ap.add_argument("out")
    ap.add_argument("--recipe", default="Q8_0", choices=sorted(RECIPES))
    a = ap.parse_args(argv)
    if os.path.isfile(a.model_dir):
        w = requantize(ModelWeights.from_gguf(a.model_dir), a.recipe)
        w.save_gguf(a.out)
    else:
        w = convert_directory(a.model_dir, a.out, a.recipe)
    c = w.config
    print(f"{a.out}: {c.arch}, {c.n_layers} layers, d={c.d_model}, {len(w.tensors)} tensors, {w.nbytes() / 1e9:.2f} GB ({a.recipe})")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
