"""Model hyper-parameters read from GGUF metadata, plus the named benchmark shapes.

Keys follow the ``<arch>.*`` convention the reference extracts (reference:
src/v2/loaders/ModelLoader.cpp:2548-2652) and the MoE / NextN keys it uses
(src/v2/models/qwen35moe/Qwen35MoEGraphConfigBuilder.cpp:37-45,
src/v2/execution/mtp/MTPWeightManifest.cpp:141-156).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field, replace

from ..gguf.constants import GGMLType

SUPPORTED_ARCHS = ("qwen2", "qwen3", "qwen3moe", "qwen35", "qwen35moe")


@dataclass
class ModelConfig:
    arch: str = "qwen3"
    n_layers: int = 2
    d_model: int = 256
    n_heads: int = 4
    n_kv_heads: int = 2
    head_dim: int = 64
    d_ff: int = 768
    vocab_size: int = 1024
    rope_theta: float = 1e6
    rms_eps: float = 1e-6
    context_length: int = 4096
    qk_norm: bool = True            # qwen3 / qwen3moe: per-head RMSNorm on Q and K
    qkv_bias: bool = False          # qwen2: biases on the Q/K/V projections
    tie_embeddings: bool = True
    # MoE
    n_experts: int = 0
    n_experts_used: int = 0
    expert_ff: int = 0
    norm_topk_prob: bool = True
    shared_expert_ff: int = 0       # qwen35moe: one always-on expert of this width, scaled by sigmoid(x . ffn_gate_inp_shexp)
    # multi-token prediction (NextN) head: number of extra decoder layers stored after the trunk
    nextn_layers: int = 0
    # hybrid layout (qwen35): every `full_attention_interval`-th layer is softmax attention over the KV cache, the others are
    # Gated-DeltaNet linear attention (short causal convolution + one recurrent d_k x d_v state per value head)
    # (reference: src/v2/models/qwen35/Qwen35GraphConfigBuilder.cpp:56-137)
    full_attention_interval: int = 0     # 0: every layer is full attention
    ssm_conv_kernel: int = 4
    ssm_state: int = 0                   # d_k = d_v of the linear-attention heads
    ssm_k_heads: int = 0
    ssm_v_heads: int = 0
    rope_dim: int = 0                    # leading dims of each head that are rotated (0: all of head_dim)
    attn_gate: bool = False              # attn_q holds [q | gate] per head; the attention output is scaled by sigmoid(gate)
    name: str = "tiny-qwen3"

    @property
    def is_moe(self) -> bool:
        return self.n_experts > 0

    @property
    def is_hybrid(self) -> bool:
        return self.full_attention_interval > 0

    def is_gdn_layer(self, i: int) -> bool:
        """Trunk layer i is linear attention (NextN layers, i >= n_layers, are always full attention)."""
        return self.is_hybrid and i < self.n_layers and (i + 1) % self.full_attention_interval != 0

    def kv_layers(self, layer_ids) -> list[int]:
        """Of the given layers, the ones that own a KV-cache layer (all but the linear-attention ones)."""
        return [i for i in layer_ids if not self.is_gdn_layer(i)]

    def gdn_layers(self, layer_ids) -> list[int]:
        return [i for i in layer_ids if self.is_gdn_layer(i)]

    @property
    def gdn_key_dim(self) -> int:
        return self.ssm_k_heads * self.ssm_state

    @property
    def gdn_value_dim(self) -> int:
        return self.ssm_v_heads * self.ssm_state

    @property
    def gdn_conv_dim(self) -> int:
        return 2 * self.gdn_key_dim + self.gdn_value_dim

    @property
    def rotary_dim(self) -> int:
        return self.rope_dim or self.head_dim

    @property
    def ffn_norm_name(self) -> str:
        """GGUF name of the second norm of a block: qwen35 files call it post_attention_norm."""
        return "post_attention_norm.weight" if self.arch.startswith("qwen35") else "ffn_norm.weight"

    @property
    def q_dim(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    def to_dict(self) -> dict:
        return asdict(self)

    def with_(self, **kw) -> "ModelConfig":
        return replace(self, **kw)

    # -- GGUF metadata ---------------------------------------------------------------------
    @staticmethod
    def from_gguf(gf) -> "ModelConfig":
        arch = gf.architecture
        if arch not in SUPPORTED_ARCHS:
            raise ValueError(f"unsupported GGUF architecture '{arch}' (supported: {', '.join(SUPPORTED_ARCHS)}; "
                             "qwen35 / qwen35moe are the hybrid Gated-DeltaNet families)")
        a = gf.arch_key

        def scalar(v):
            """Hybrid checkpoints may store per-layer arrays (0 for the linear-attention layers): the softmax blocks' value."""
            if isinstance(v, (list, tuple)):
                vals = [int(x) for x in v if int(x) > 0]
                return max(vals) if vals else 0
            return v

        d_model = int(a("embedding_length"))
        n_heads = int(scalar(a("attention.head_count")))
        n_kv = int(scalar(a("attention.head_count_kv", n_heads)))
        head_dim = int(a("attention.key_length", d_model // n_heads))
        tokens = gf.get("tokenizer.ggml.tokens")
        if tokens is not None:
            vocab = len(tokens)
        elif "token_embd.weight" in gf:
            vocab = gf["token_embd.weight"].shape[0]
        else:
            vocab = int(a("vocab_size"))
        nextn = int(a("nextn_predict_layers", 0))
        n_blocks = int(a("block_count"))
        hybrid = {}
        first_attn = 0                                  # first block with softmax attention (QK-norm / bias probes look there)
        if arch in ("qwen35", "qwen35moe"):
            interval = int(a("full_attention_interval", 4))
            first_attn = interval - 1
            hybrid = dict(full_attention_interval=interval, ssm_conv_kernel=int(a("ssm.conv_kernel", 4)),
                          ssm_state=int(a("ssm.state_size")), ssm_k_heads=int(a("ssm.group_count")),
                          ssm_v_heads=int(a("ssm.time_step_rank")), rope_dim=int(a("rope.dimension_count", 0) or 0),
                          attn_gate=True)
            if int(a("ssm.inner_size", hybrid["ssm_v_heads"] * hybrid["ssm_state"])) != hybrid["ssm_v_heads"] * hybrid["ssm_state"]:
                raise ValueError("qwen35: ssm.inner_size is not ssm.time_step_rank x ssm.state_size")
        return ModelConfig(
            arch=arch,
            n_layers=n_blocks - nextn,
            d_model=d_model,
            n_heads=n_heads,
            n_kv_heads=n_kv,
            head_dim=head_dim,
            d_ff=int(scalar(a("feed_forward_length", 0)) or 0),
            vocab_size=vocab,
            rope_theta=float(a("rope.freq_base", 10000.0)),
            rms_eps=float(a("attention.layer_norm_rms_epsilon", 1e-6)),
            context_length=int(a("context_length", 4096)),
            qk_norm=f"blk.{first_attn}.attn_q_norm.weight" in gf,
            qkv_bias=f"blk.{first_attn}.attn_q.bias" in gf,
            tie_embeddings="output.weight" not in gf,
            n_experts=int(a("expert_count", 0) or 0),
            n_experts_used=int(a("expert_used_count", 0) or 0),
            expert_ff=int(a("expert_feed_forward_length", 0) or 0),
            norm_topk_prob=True,
            shared_expert_ff=(gf["blk.0.ffn_gate_shexp.weight"].shape[0] if "blk.0.ffn_gate_shexp.weight" in gf else 0),
            nextn_layers=nextn,
            name=str(gf.get("general.name", arch)),
            **hybrid,
        )

    def gguf_metadata(self) -> dict:
        a = self.arch
        md = {
            "general.architecture": a,
            "general.name": self.name,
            f"{a}.block_count": self.n_layers + self.nextn_layers,
            f"{a}.context_length": self.context_length,
            f"{a}.embedding_length": self.d_model,
            f"{a}.feed_forward_length": self.d_ff,
            f"{a}.attention.head_count": self.n_heads,
            f"{a}.attention.head_count_kv": self.n_kv_heads,
            f"{a}.attention.key_length": self.head_dim,
            f"{a}.attention.value_length": self.head_dim,
            f"{a}.rope.freq_base": float(self.rope_theta),
            f"{a}.attention.layer_norm_rms_epsilon": float(self.rms_eps),
        }
        if self.is_moe:
            md[f"{a}.expert_count"] = self.n_experts
            md[f"{a}.expert_used_count"] = self.n_experts_used
            md[f"{a}.expert_feed_forward_length"] = self.expert_ff
            if self.shared_expert_ff:
                md[f"{a}.expert_shared_count"] = 1
        if self.nextn_layers:
            md[f"{a}.nextn_predict_layers"] = self.nextn_layers
        if self.is_hybrid:
            md[f"{a}.full_attention_interval"] = self.full_attention_interval
            md[f"{a}.ssm.conv_kernel"] = self.ssm_conv_kernel
            md[f"{a}.ssm.state_size"] = self.ssm_state
            md[f"{a}.ssm.group_count"] = self.ssm_k_heads
            md[f"{a}.ssm.time_step_rank"] = self.ssm_v_heads
            md[f"{a}.ssm.inner_size"] = self.gdn_value_dim
            if self.rope_dim:
                md[f"{a}.rope.dimension_count"] = self.rope_dim
        return md


@dataclass
class QuantRecipe:
    """Which GGUF block format each weight role is stored in."""
    default: GGMLType = GGMLType.Q8_0
    overrides: dict = field(default_factory=dict)     # substring of tensor name -> GGMLType
    name: str = "Q8_0"

    def for_tensor(self, tensor_name: str, layer: int | None = None, n_layers: int = 0) -> GGMLType:
        for key, t in self.overrides.items():
            if key == "ffn_down:some":
                # Q4_K_M rule of thumb: a subset of the down projections is kept in Q6_K
                if "ffn_down" in tensor_name and layer is not None and _more_bits(layer, n_layers):
                    return t
            elif key == "ffn_down:first8th":
                # Q4_K_S: the down projections of the first eighth of the layers get one more bit
                if "ffn_down" in tensor_name and "_exps" not in tensor_name and layer is not None and layer < n_layers // 8:
                    return t
            elif key == "attn_v:first4":
                if "attn_v" in tensor_name and layer is not None and layer < 4:
                    return t
            elif key == "output.weight":
                # the LM head only: "blk.N.attn_output.weight" contains the same text and is an ordinary projection
                if tensor_name == "output.weight":
                    return t
            elif key in tensor_name:
                return t
        return self.default


def _more_bits(i_layer: int, n_layers: int) -> bool:
    return i_layer < n_layers // 8 or i_layer >= 7 * n_layers // 8 or (i_layer - n_layers // 8) % 3 == 2


RECIPES = {
    "Q8_0": QuantRecipe(GGMLType.Q8_0, {}, "Q8_0"),
    "Q4_0": QuantRecipe(GGMLType.Q4_0, {}, "Q4_0"),
    # llama.cpp's Q4_K_S mix: Q4_K everywhere, Q5_K for attn_v of the first four layers and ffn_down of the first eighth,
    # Q6_K for the LM head
    "Q4_K_S": QuantRecipe(GGMLType.Q4_K, {"output.weight": GGMLType.Q6_K, "token_embd": GGMLType.Q4_K, "attn_v:first4": GGMLType.Q5_K,
                                          "ffn_down:first8th": GGMLType.Q5_K}, "Q4_K_S"),
    "Q4_K_M": QuantRecipe(GGMLType.Q4_K, {"output.weight": GGMLType.Q6_K, "attn_v": GGMLType.Q6_K,
                                          "ffn_down:some": GGMLType.Q6_K}, "Q4_K_M"),
    "Q5_K": QuantRecipe(GGMLType.Q5_K, {"output.weight": GGMLType.Q6_K}, "Q5_K"),
    "Q6_K": QuantRecipe(GGMLType.Q6_K, {}, "Q6_K"),
    "IQ3_S_MOE": QuantRecipe(GGMLType.Q4_K, {"_exps": GGMLType.IQ3_S, "output.weight": GGMLType.Q6_K,
                                             "ffn_gate_inp": GGMLType.F32}, "IQ3_S-experts/Q4_K-attn"),
    "BF16": QuantRecipe(GGMLType.BF16, {}, "BF16"),
    "F32": QuantRecipe(GGMLType.F32, {}, "F32"),
}

# The benchmark shapes (random-init stand-ins for the named public models).
SHAPES = {
    "tiny-qwen3": ModelConfig(name="tiny-qwen3"),
    "tiny-qwen2": ModelConfig(name="tiny-qwen2", arch="qwen2", qk_norm=False, qkv_bias=True),
    "tiny-qwen3moe": ModelConfig(name="tiny-qwen3moe", arch="qwen3moe", n_experts=8, n_experts_used=2,
                                 expert_ff=256, d_ff=0),
    # hybrid: layers 0-2 and 4-6 linear attention, 3 and 7 softmax attention with an output gate and partial RoPE;
    # twice as many value heads as key heads (the 4B / 27B ratio)
    "tiny-qwen35": ModelConfig(name="tiny-qwen35", arch="qwen35", n_layers=8, head_dim=64, rope_dim=16, attn_gate=True,
                               full_attention_interval=4, ssm_state=32, ssm_k_heads=2, ssm_v_heads=4, rope_theta=1e7),
    "tiny-qwen35moe": ModelConfig(name="tiny-qwen35moe", arch="qwen35moe", n_layers=4, head_dim=64, rope_dim=16, attn_gate=True,
                                  full_attention_interval=4, ssm_state=32, ssm_k_heads=2, ssm_v_heads=4, rope_theta=1e7,
                                  n_experts=8, n_experts_used=2, expert_ff=256, shared_expert_ff=256, d_ff=0),
    "qwen3.5-35b-a3b": ModelConfig(name="qwen3.5-35b-a3b", arch="qwen35moe", n_layers=40, d_model=2048, n_heads=16, n_kv_heads=2,
                                   head_dim=256, rope_dim=64, attn_gate=True, d_ff=0, vocab_size=248320, tie_embeddings=False,
                                   full_attention_interval=4, ssm_state=128, ssm_k_heads=16, ssm_v_heads=32, rope_theta=1e7,
                                   n_experts=256, n_experts_used=8, expert_ff=512, shared_expert_ff=512, context_length=262144),
    "qwen3.5-27b": ModelConfig(name="qwen3.5-27b", arch="qwen35", n_layers=64, d_model=5120, n_heads=24, n_kv_heads=4,
                               head_dim=256, rope_dim=64, attn_gate=True, d_ff=17408, vocab_size=248320,
                               tie_embeddings=False, full_attention_interval=4, ssm_state=128, ssm_k_heads=16,
                               ssm_v_heads=48, rope_theta=1e7, context_length=262144),
    "qwen3-8b": ModelConfig(name="qwen3-8b", n_layers=36, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128,
                            d_ff=12288, vocab_size=151936, tie_embeddings=False, context_length=40960),
    "qwen3-32b": ModelConfig(name="qwen3-32b", n_layers=64, d_model=5120, n_heads=64, n_kv_heads=8, head_dim=128,
                             d_ff=25600, vocab_size=151936, tie_embeddings=False, context_length=40960),
    "qwen3-30b-a3b": ModelConfig(name="qwen3-30b-a3b", arch="qwen3moe", n_layers=48, d_model=2048, n_heads=32,
                                 n_kv_heads=4, head_dim=128, d_ff=0, vocab_size=151936, tie_embeddings=False,
                                 n_experts=128, n_experts_used=8, expert_ff=768, context_length=40960),
    "qwen2.5-7b": ModelConfig(name="qwen2.5-7b", arch="qwen2", n_layers=28, d_model=3584, n_heads=28, n_kv_heads=4,
                              head_dim=128, d_ff=18944, vocab_size=152064, tie_embeddings=False, qk_norm=False,
                              qkv_bias=True, context_length=32768),
}
