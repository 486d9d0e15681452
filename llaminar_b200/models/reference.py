"""Plain PyTorch fp32 decoder: the numerical oracle and the CPU execution path.

Implements the block order the reference builds for qwen2 / qwen3 (RMSNorm -> QKV(+bias) ->
per-head QK RMSNorm -> split-half RoPE -> causal GQA attention -> Wo; RMSNorm -> SwiGLU FFN or
softmax-top-k MoE; reference: src/v2/models/qwen/QwenStandardGraph.cpp:103-203,
src/v2/models/qwen/QwenGraphBase.cpp:1974-2176) and the NextN multi-token-prediction head
(src/v2/models/qwen35/Qwen35Graph.cpp:403-610) on dequantised weights.  The hybrid qwen35 family adds linear-attention
blocks (models/gdn.py) and, in its softmax blocks, a per-head output gate and partial rotation
(src/v2/models/qwen35/Qwen35Graph.cpp:980-990).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import gdn
from .config import ModelConfig
from .weights import ModelWeights


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps) * w


def rope_split_half(x: torch.Tensor, positions: torch.Tensor, theta: float, rotary_dim: int = 0) -> torch.Tensor:
    """x: [T, H, D]; rotates pairs (i, i + R/2) of the first R = rotary_dim (default D) values by pos * theta^(-2i/R); the
    rest of each head passes through."""
    if rotary_dim and rotary_dim < x.shape[-1]:
        return torch.cat([rope_split_half(x[..., :rotary_dim], positions, theta), x[..., rotary_dim:]], dim=-1)
    D = x.shape[-1]
    half = D // 2
    inv = theta ** (-torch.arange(half, device=x.device, dtype=torch.float32) * 2.0 / D)
    ang = positions.to(torch.float32)[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def moe_route(logits: torch.Tensor, k: int, renorm: bool = True):
    """softmax over all experts, top-k with lower-index tie-break, optional renormalisation."""
    probs = torch.softmax(logits.float(), dim=-1)
    # stable descending sort keeps the lower index first among equals
    order = torch.sort(probs, dim=-1, descending=True, stable=True)
    idx, w = order.indices[..., :k], order.values[..., :k]
    if renorm:
        w = w / w.sum(dim=-1, keepdim=True)
    return idx, w


class KVState:
    """Per-layer contiguous K/V history for the oracle."""

    def __init__(self, n_layers: int):
        self.k = [None] * n_layers
        self.v = [None] * n_layers
        self.conv = {}                  # linear-attention layers: last K-1 convolution inputs [C, K-1]
        self.rec = {}                   # ... and the recurrent matrices [n_v, d, d]
        self.seen = 0                   # tokens fed so far

    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor):
        self.k[layer] = k if self.k[layer] is None else torch.cat([self.k[layer], k], dim=0)
        self.v[layer] = v if self.v[layer] is None else torch.cat([self.v[layer], v], dim=0)
        return self.k[layer], self.v[layer]

    def length(self) -> int:
        return self.seen

    def truncate(self, n: int) -> None:
        if self.rec and n != self.seen:
            raise ValueError("a recurrent state cannot be rolled back")
        self.seen = n
        for i in range(len(self.k)):
            if self.k[i] is not None:
                self.k[i], self.v[i] = self.k[i][:n], self.v[i][:n]


class ReferenceModel:
    def __init__(self, weights: ModelWeights | None = None, cfg: ModelConfig | None = None,
                 float_weights: dict | None = None, device="cpu"):
        self.cfg = cfg or weights.config
        self.w = float_weights if float_weights is not None else weights.float_dict(device)
        self.device = torch.device(device)

    # -- pieces ------------------------------------------------------------------------------
    def embed(self, tokens: torch.Tensor) -> torch.Tensor:
        return self.w["token_embd.weight"][tokens.long()]

    def lm_head(self, h: torch.Tensor, norm_name: str = "output_norm.weight") -> torch.Tensor:
        x = rmsnorm(h, self.w[norm_name], self.cfg.rms_eps)
        out = self.w.get("output.weight", self.w["token_embd.weight"])
        return x @ out.T

    def attention(self, i: int, x: torch.Tensor, positions: torch.Tensor, kv: KVState, kv_layer: int):
        c, w, p = self.cfg, self.w, f"blk.{i}."
        T = x.shape[0]
        q = x @ w[p + "attn_q.weight"].T
        k = x @ w[p + "attn_k.weight"].T
        v = x @ w[p + "attn_v.weight"].T
        if c.qkv_bias:
            q, k, v = q + w[p + "attn_q.bias"], k + w[p + "attn_k.bias"], v + w[p + "attn_v.bias"]
        gate = None
        if c.attn_gate:                 # every head's rows are [query | gate]
            q, gate = q.view(T, c.n_heads, 2, c.head_dim).unbind(dim=2)
            gate = gate.reshape(T, c.q_dim)
        q = q.reshape(T, c.n_heads, c.head_dim)
        k = k.view(T, c.n_kv_heads, c.head_dim)
        v = v.view(T, c.n_kv_heads, c.head_dim)
        if c.qk_norm:
            q = rmsnorm(q, w[p + "attn_q_norm.weight"], c.rms_eps)
            k = rmsnorm(k, w[p + "attn_k_norm.weight"], c.rms_eps)
        q = rope_split_half(q, positions, c.rope_theta, c.rotary_dim)
        k = rope_split_half(k, positions, c.rope_theta, c.rotary_dim)
        K, V = kv.append(kv_layer, k, v)
        S = K.shape[0]
        past = S - T
        g = c.n_heads // c.n_kv_heads
        Kh = K.repeat_interleave(g, dim=1)
        Vh = V.repeat_interleave(g, dim=1)
        scores = torch.einsum("thd,shd->hts", q, Kh) / (c.head_dim ** 0.5)
        key_pos = torch.arange(S, device=x.device)[None, :]
        qry_pos = (past + torch.arange(T, device=x.device))[:, None]
        scores = scores.masked_fill((key_pos > qry_pos)[None], float("-inf"))
        o = torch.einsum("hts,shd->thd", torch.softmax(scores, dim=-1), Vh).reshape(T, c.q_dim)
        if gate is not None:
            o = o * torch.sigmoid(gate)
        return o @ w[p + "attn_output.weight"].T

    def linear_attention(self, i: int, x: torch.Tensor, kv: KVState) -> torch.Tensor:
        c, w, p = self.cfg, self.w, f"blk.{i}."
        if i not in kv.rec:
            kv.conv[i] = torch.zeros(c.gdn_conv_dim, c.ssm_conv_kernel - 1, device=x.device)
            kv.rec[i] = torch.zeros(c.ssm_v_heads, c.ssm_state, c.ssm_state, device=x.device)
        rows, kv.conv[i] = gdn.gdn_mix(x @ w[p + "attn_qkv.weight"].T, x @ w[p + "attn_gate.weight"].T,
                                       x @ w[p + "ssm_alpha.weight"].T, x @ w[p + "ssm_beta.weight"].T,
                                       w[p + "ssm_conv1d.weight"], w[p + "ssm_a"], w[p + "ssm_dt.bias"], w[p + "ssm_norm.weight"],
                                       kv.conv[i], kv.rec[i], c.ssm_k_heads, c.ssm_v_heads, c.ssm_state, c.rms_eps)
        return rows @ w[p + "ssm_out.weight"].T

    def ffn(self, i: int, x: torch.Tensor) -> torch.Tensor:
        c, w, p = self.cfg, self.w, f"blk.{i}."
        if not c.is_moe:
            g = x @ w[p + "ffn_gate.weight"].T
            u = x @ w[p + "ffn_up.weight"].T
            return (F.silu(g) * u) @ w[p + "ffn_down.weight"].T
        logits = x @ w[p + "ffn_gate_inp.weight"].T
        idx, wt = moe_route(logits, c.n_experts_used, c.norm_topk_prob)
        out = torch.zeros_like(x)
        Wg, Wu, Wd = w[p + "ffn_gate_exps.weight"], w[p + "ffn_up_exps.weight"], w[p + "ffn_down_exps.weight"]
        for e in idx.unique().tolist():
            tok, slot = (idx == e).nonzero(as_tuple=True)
            xe = x[tok]
            ye = (F.silu(xe @ Wg[e].T) * (xe @ Wu[e].T)) @ Wd[e].T
            out.index_add_(0, tok, ye * wt[tok, slot].unsqueeze(-1))
        if c.shared_expert_ff:          # always-on expert, scaled per token by sigmoid(x . gate vector)
            sh = (F.silu(x @ w[p + "ffn_gate_shexp.weight"].T) * (x @ w[p + "ffn_up_shexp.weight"].T)) @ w[p + "ffn_down_shexp.weight"].T
            out = out + torch.sigmoid(x @ w[p + "ffn_gate_inp_shexp.weight"].reshape(-1, 1)) * sh
        return out

    def layer(self, i: int, h: torch.Tensor, positions: torch.Tensor, kv: KVState, kv_layer: int | None = None):
        c, w, p = self.cfg, self.w, f"blk.{i}."
        kv_layer = i if kv_layer is None else kv_layer
        x = rmsnorm(h, w[p + "attn_norm.weight"], c.rms_eps)
        h = h + (self.linear_attention(i, x, kv) if c.is_gdn_layer(i) else self.attention(i, x, positions, kv, kv_layer))
        h = h + self.ffn(i, rmsnorm(h, w[p + c.ffn_norm_name], c.rms_eps))
        return h

    # -- full passes -------------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, kv: KVState | None = None, taps: dict | None = None):
        """Returns (logits [T, vocab], final hidden [T, d] before the output norm, kv)."""
        c = self.cfg
        kv = kv or KVState(c.n_layers)
        tokens = tokens.to(self.device)
        pos = kv.length() + torch.arange(tokens.shape[0], device=self.device)
        h = self.embed(tokens).float()
        for i in range(c.n_layers):
            h = self.layer(i, h, pos, kv)
            if taps is not None:
                taps[f"layer{i}"] = h.clone()
        kv.seen += tokens.shape[0]
        return self.lm_head(h), h, kv

    @torch.no_grad()
    def mtp_forward(self, next_tokens: torch.Tensor, hidden: torch.Tensor, kv: KVState | None = None,
                    depth: int = 0):
        """NextN head: row t predicts token t+2 from (embedding of token t+1, trunk hidden of t)."""
        c, w = self.cfg, self.w
        i = c.n_layers + depth
        p = f"blk.{i}.nextn."
        kv = kv or KVState(1)
        e = rmsnorm(self.embed(next_tokens.to(self.device)).float(), w[p + "enorm.weight"], c.rms_eps)
        hn = rmsnorm(hidden.float(), w[p + "hnorm.weight"], c.rms_eps)
        x = torch.cat([e, hn], dim=-1) @ w[p + "eh_proj.weight"].T
        pos = kv.length() + torch.arange(x.shape[0], device=self.device)
        h = self.layer(i, x, pos, kv, kv_layer=0)
        kv.seen += x.shape[0]
        return self.lm_head(h, p + "shared_head_norm.weight"), h, kv

    @torch.no_grad()
    def generate_greedy(self, prompt: torch.Tensor, n_new: int):
        logits, _, kv = self.forward(prompt)
        out, all_logits = [], [logits[-1]]
        tok = int(logits[-1].argmax())
        out.append(tok)
        for _ in range(n_new - 1):
            logits, _, kv = self.forward(torch.tensor([tok]), kv)
            all_logits.append(logits[-1])
            tok = int(logits[-1].argmax())
            out.append(tok)
        return out, torch.stack(all_logits)
