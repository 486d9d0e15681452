"""GPU model runner: GGUF weights in chunk layout + the per-layer kernel sequence.

Per decoder layer (dense), small batches (<= 4 rows, the GEMV path) launch
    QKV GEMV (RMSNorm fused in the prologue) -> QK-norm + RoPE + KV append -> paged attention
    -> Wo GEMV (residual add in the epilogue) -> gate|up GEMV (RMSNorm prologue, SwiGLU epilogue)
    -> down GEMV (residual epilogue)
and larger batches / prefill run the same sequence on the tcgen05 GEMM with a separate RMSNorm.
The order of operations is the one the reference graph builds (reference:
src/v2/models/qwen/QwenStandardGraph.cpp:103-203, src/v2/models/qwen/QwenGraphBase.cpp:1974-2176);
the residual stream is kept in fp32, activations in bf16.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import ops
from ..gguf.constants import GGMLType
from ..models.config import ModelConfig
from ..models.weights import ModelWeights, QTensor
from ..ops.layout import PackedWeight, can_pack, interleave_gate_up, pack_experts, pack_matrix, q4k_scales_in_range
from .kv_cache import PAGE_SIZE, PagedKVCache


_FLOAT_TYPES = (GGMLType.F32, GGMLType.F16, GGMLType.BF16)


def for_kernels(t: QTensor) -> QTensor:
    """A weight matrix in a format the quantised GEMV / GEMM kernels can read.  Block formats without a packed device
    layout (Q2_K, Q3_K, Q4_1, Q5_0/1, IQ4_*, IQ3_XXS, IQ2_*, IQ1_*) are re-encoded as Q8_0 once at load: half the bytes
    of a bf16 copy and the same kernels as every other layer.  Unquantised tensors, and matrices whose K is not a whole
    number of 256-column chunks, are left alone and run as dense bf16."""
    k = t.shape[-1]
    if t.qtype == GGMLType.Q4_K and can_pack(t.qtype, k) and not q4k_scales_in_range(t.raw):
        return t.transcoded(GGMLType.Q8_0)          # block scales beyond the Q4_K conversion's range (never seen in practice)
    if can_pack(t.qtype, k) or t.qtype in _FLOAT_TYPES or not can_pack(GGMLType.Q8_0, k):
        return t
    return t.transcoded(GGMLType.Q8_0)


def expert_tensors_for_packing(w: ModelWeights, prefix: str) -> tuple[QTensor, QTensor, QTensor]:
    """Gate, up and down expert stacks of a layer in formats the grouped expert kernels can read.  The grouped kernels
    have no dense path, so a stack whose format has no packed device layout (the 1- to 3-bit codebook formats, Q2_K, Q3_K,
    ...) is re-encoded as Q8_0 once; gate and up must share a format because their rows are interleaved."""
    ge, ue, de = (w[prefix + n] for n in ("ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight"))
    _, ff, d = ge.shape
    if not (can_pack(ge.qtype, d) and ge.qtype == ue.qtype):
        for name, key in (("gate", "ffn_gate_exps.weight"), ("up", "ffn_up_exps.weight")):
            t = w[prefix + key]
            if t.qtype != GGMLType.Q8_0:
                w.tensors[prefix + key] = t.transcoded(GGMLType.Q8_0)      # cached: expert-parallel slabs share the result
        ge, ue = w[prefix + "ffn_gate_exps.weight"], w[prefix + "ffn_up_exps.weight"]
    if not can_pack(de.qtype, ff):
        w.tensors[prefix + "ffn_down_exps.weight"] = de = de.transcoded(GGMLType.Q8_0)
    return ge, ue, de


@dataclass
class ForwardBatch:
    """Device-side description of one forward call (all int32 tensors on the model's device)."""
    tokens: torch.Tensor            # [T]
    positions: torch.Tensor         # [T]
    seq_ids: torch.Tensor           # [T] row of block_table
    block_table: torch.Tensor       # [B, max_pages]
    # decode-style attention (few rows per sequence)
    seq_lens: torch.Tensor | None = None     # [B] cache length including this step's rows
    rows_per_seq: int = 1
    n_splits: int = 1
    # prefill-style attention
    cu_q: torch.Tensor | None = None         # [B + 1]
    ctx_lens: torch.Tensor | None = None     # [B]
    max_kv_len: int = 0                      # prefill: longest context + chunk of the batch (0: unknown, assume the table width)
    max_q_len: int = 0
    # which hidden rows get logits (None: all rows)
    logit_rows: torch.Tensor | None = None
    embeds: torch.Tensor | None = None       # optional fp32 [T, d] input instead of token embeddings
    state_slots: torch.Tensor | None = None  # [B] hybrid models: the state slot of every sequence (row of block_table)
    defer_state: bool = False                # hybrid models, speculative verification: equal rows per sequence, the recurrent
                                             # state is advanced later by `HybridState.commit` for the accepted rows only

    @property
    def is_decode(self) -> bool:
        return self.seq_lens is not None

    def index_errors(self, vocab: int, n_pages: int, max_positions: int) -> list[str]:
        """Every index the kernels will dereference, checked against its range on the host (one synchronisation; a debug
        aid behind LLAMINAR_VALIDATE_TENSORS, never inside graph capture).  The kernels themselves trust these arrays: an
        out-of-range page id or sequence id would be an out-of-bounds access on the device, so the check runs before any
        launch and reports instead."""
        errs = []

        def rng(name, t, lo, hi):
            if t is not None and t.numel():
                mn, mx = int(t.min()), int(t.max())
                if mn < lo or mx >= hi:
                    errs.append(f"{name}: values in [{mn}, {mx}], allowed [{lo}, {hi})")

        T = self.tokens.shape[0] if self.embeds is None else self.embeds.shape[0]
        B, P = self.block_table.shape
        if self.embeds is None:
            rng("tokens", self.tokens, 0, vocab)
        rng("positions", self.positions, 0, max_positions)
        rng("seq_ids", self.seq_ids, 0, B)
        rng("block_table", self.block_table, 0, n_pages)
        if self.positions.shape[0] != T or self.seq_ids.shape[0] != T:
            errs.append(f"positions / seq_ids have {self.positions.shape[0]} / {self.seq_ids.shape[0]} rows for {T} tokens")
        cap = P * PAGE_SIZE
        if self.is_decode:
            rng("seq_lens", self.seq_lens, 1, cap + 1)
            if self.seq_lens.shape[0] * self.rows_per_seq < T and self.seq_lens.shape[0] != B:
                errs.append(f"seq_lens has {self.seq_lens.shape[0]} entries for {B} block-table rows")
        else:
            if self.cu_q is None or self.ctx_lens is None:
                errs.append("prefill batch without cu_q / ctx_lens")
            else:
                cu = self.cu_q.tolist()
                if cu[0] != 0 or cu[-1] != T or any(b < a for a, b in zip(cu, cu[1:])):
                    errs.append(f"cu_q {cu[:4]}...{cu[-1]} is not a non-decreasing partition of {T} rows")
                elif max(b - a for a, b in zip(cu, cu[1:])) > self.max_q_len:
                    errs.append(f"max_q_len {self.max_q_len} is smaller than the longest query of the batch")
                end = [c + (b - a) for c, a, b in zip(self.ctx_lens.tolist(), cu, cu[1:])]
                if end and max(end) > cap:
                    errs.append(f"context + query reaches {max(end)} tokens, the block table holds {cap}")
        rng("logit_rows", self.logit_rows, 0, max(T, 1))
        return errs


class _HiddenRows:
    """The hidden rows a sequence-sharded forward pass brought to every rank, indexed by their global row number (the
    other rows of the residual stream live on their owners only)."""

    def __init__(self, rows: torch.Tensor, values: torch.Tensor | None):
        self._pos = {int(r): i for i, r in enumerate(rows.tolist())} if values is not None else {}
        self._values = values

    def __getitem__(self, row):
        return self._values[self._pos[int(row)]]


class QLinear:
    """A (possibly multi-part) quantised linear layer: parts may differ in block format."""

    def __init__(self, parts: list[tuple[PackedWeight | torch.Tensor, int]], n_out: int, k: int, bias: torch.Tensor | None = None):
        self.parts = parts          # (weight, first output column); torch.Tensor = dense bf16 fallback [n, k]
        self.n_out, self.k, self.bias = n_out, k, bias

    @staticmethod
    def from_qtensors(qts: list[QTensor], device, bias: torch.Tensor | None = None) -> "QLinear":
        """Row-concatenate matrices; consecutive matrices of one format share a launch."""
        parts, col = [], 0
        i = 0
        qts = [for_kernels(q) for q in qts]
        k = qts[0].shape[1]
        while i < len(qts):
            j = i
            while j + 1 < len(qts) and qts[j + 1].qtype == qts[i].qtype:
                j += 1
            group = qts[i:j + 1]
            n = sum(q.shape[0] for q in group)
            qt = group[0].qtype
            raw = torch.cat([q.raw.to(device).reshape(-1) for q in group]) if len(group) > 1 else group[0].raw.to(device)
            if can_pack(qt, k):
                parts.append((pack_matrix(raw, qt, n, k), col))          # rows are padded to whole 128-row tiles
            else:
                from ..gguf import dequantize
                parts.append((dequantize(raw, qt, (n, k)).to(torch.bfloat16), col))
            col += n
            i = j + 1
        return QLinear(parts, col, k, bias)

    def nbytes(self) -> int:
        return sum(p.nbytes() if isinstance(p, PackedWeight) else p.numel() * 2 for p, _ in self.parts)

    def __call__(self, x: torch.Tensor, out: torch.Tensor, *, norm_w=None, eps=1e-6, epi=ops.EPI_STORE, scratch=None,
                 xn: torch.Tensor | None = None) -> None:
        """x: bf16 rows, or the fp32 residual rows when ``norm_w`` is given (GEMV path only).
        ``xn``: pre-normalised bf16 rows for the GEMM path."""
        rows = x.shape[0]
        for w, col in self.parts:
            n = w.n if isinstance(w, PackedWeight) else w.shape[0]
            if epi == ops.EPI_SWIGLU:
                o = out
            else:
                o = out[:, col:col + n] if (col or n != out.shape[1]) else out
            b = self.bias[col:col + n] if self.bias is not None else None
            if not isinstance(w, PackedWeight):
                src = xn if xn is not None else x
                y = src.to(torch.bfloat16) @ w.T
                if b is not None:
                    y = y + b
                if epi == ops.EPI_RESID:
                    o += y.float()
                else:
                    o.copy_(y)
                continue
            if rows <= ops.GEMV_MAX_ROWS and xn is None:
                ops.gemv(w, x, o, norm_w=norm_w, eps=eps, epi=epi, bias=b, scratch=scratch)
            else:
                ops.gemm(w, xn if xn is not None else x, o, epi=epi, bias=b, scratch=scratch)


def _expert_view_for_tests(pw: PackedWeight, e: int) -> PackedWeight:
    """Expert ``e`` of a packed expert slab as a matrix of its own (tests dequantise it for their fp32 references)."""
    return PackedWeight(pw.fmt, pw.qtype, pw.n, pw.k, pw.n_tiles, pw.k_blocks, pw.data[e])


def _f32(t: QTensor | None, device) -> torch.Tensor | None:
    return None if t is None else t.to_float().to(device=device, dtype=torch.float32).contiguous()


class CudaLayer:
    pass


def paged_attention_torch(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor, seq_ids: torch.Tensor,
                          positions: torch.Tensor, scale: float) -> torch.Tensor:
    """Causal GQA attention of a packed batch over the paged cache, any head size, one sequence at a time through
    `scaled_dot_product_attention` (no [rows x keys] score matrix in memory, whatever the context length).  Rows of a
    sequence are consecutive with consecutive positions; its keys are positions 0 .. last row's position.
    q: [T, H, D]; kv_layer: [n_pages, 2, Hk, 64, D]; returns fp32 [T, H, D].  (One host synchronisation for the row ranges:
    this is the prefill path of head sizes without an attention kernel.)"""
    T, H, D = q.shape
    Hk = kv_layer.shape[2]
    sid, pos = seq_ids.tolist(), positions.tolist()
    out = torch.empty(T, H, D, dtype=torch.float32, device=q.device)
    r0 = 0
    for r in range(1, T + 1):
        if r < T and sid[r] == sid[r0]:
            continue
        n_keys = pos[r - 1] + 1
        n_pages = (n_keys + 63) // 64
        pages = block_table[sid[r0], :n_pages].long()
        K = kv_layer[pages, 0].permute(1, 0, 2, 3).reshape(1, Hk, n_pages * 64, D)[:, :, :n_keys]
        V = kv_layer[pages, 1].permute(1, 0, 2, 3).reshape(1, Hk, n_pages * 64, D)[:, :, :n_keys]
        qs = q[r0:r].to(K.dtype).transpose(0, 1).unsqueeze(0)                       # [1, H, rows, D]
        allowed = None
        if pos[r0] != 0:                                                            # rows behind cached context: explicit mask
            allowed = torch.arange(n_keys, device=q.device)[None, :] <= positions[r0:r].long()[:, None]
        try:
            o = torch.nn.functional.scaled_dot_product_attention(qs, K, V, attn_mask=allowed, is_causal=allowed is None, scale=scale,
                                                                 enable_gqa=H != Hk)[0]
        except RuntimeError:
            # no fused backend took the shape: the same attention written out (materialises the rows x keys scores)
            g = H // Hk
            sc = torch.einsum("htd,hsd->hts", qs[0].float(), K[0].float().repeat_interleave(g, 0)) * scale
            if allowed is None:
                allowed = torch.arange(n_keys, device=q.device)[None, :] <= positions[r0:r].long()[:, None]
            o = torch.einsum("hts,hsd->htd", torch.softmax(sc.masked_fill(~allowed[None], float("-inf")), -1),
                             V[0].float().repeat_interleave(g, 0))
        out[r0:r] = o.transpose(0, 1).float()
        r0 = r
    return out


def paged_decode_attention_torch(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor,
                                 scale: float) -> torch.Tensor:
    """One query row per sequence against the paged cache, any head size, as one batched expression with static shapes
    (every sequence's whole page-table row is gathered and the positions past its length are masked), so a CUDA graph can
    capture it.  q: [B, H, D]; kv_layer: [n_pages, 2, Hk, 64, D]; block_table: [B, P]; seq_lens: [B] (>= 1, the new
    token included).  Returns fp32 [B, H, D].  The gather reads P x 64 positions per sequence whatever its length: a
    stand-in for head sizes without a decode kernel, not a fast path."""
    B, H, D = q.shape
    P, Hk = block_table.shape[1], kv_layer.shape[2]
    pages = kv_layer[block_table.long()]                                        # [B, P, 2, Hk, 64, D]
    K = pages[:, :, 0].permute(0, 2, 1, 3, 4).reshape(B, Hk, P * 64, D)
    V = pages[:, :, 1].permute(0, 2, 1, 3, 4).reshape(B, Hk, P * 64, D)
    qg = q.reshape(B, Hk, H // Hk, D).to(K.dtype)
    s = torch.einsum("bkgd,bkld->bkgl", qg, K).float() * scale
    dead = torch.arange(P * 64, device=q.device)[None, :] >= seq_lens.long()[:, None]
    p = torch.softmax(s.masked_fill(dead[:, None, None, :], float("-inf")), dim=-1)
    return torch.einsum("bkgl,bkld->bkgd", p.to(V.dtype), V).float().reshape(B, H, D)


class CudaModel:
    def __init__(self, weights: ModelWeights, device="cuda", max_tokens: int = 4096, tp=None, layer_range=None,
                 with_head: bool = True, with_embed: bool = True, with_mtp: bool = True):
        self.cfg: ModelConfig = weights.config
        self.device = torch.device(device)
        self.tp = tp
        self.max_tokens = max_tokens
        c = self.cfg
        self.scratch = ops.scratch_for(self.device)
        dev = self.device
        self.layer_ids = list(range(*layer_range)) if layer_range else list(range(c.n_layers))
        # ---- tensor-parallel slicing plan (replicated when tp is None) ----
        from ..parallel.tp_plan import TPPlan
        self.plan = TPPlan.build(c, tp.size if tp else 1, tp.rank if tp else 0, getattr(tp, "moe_mode", "expert-parallel"))
        pl = self.plan
        self.n_heads_local, self.n_kv_local = pl.n_heads_local, pl.n_kv_local
        self.q_dim, self.kv_dim = pl.n_heads_local * c.head_dim, pl.n_kv_local * c.head_dim
        self.qkv_dim = self.q_dim + 2 * self.kv_dim
        self.ff_local = pl.ff_stop - pl.ff_start

        if with_embed:
            emb = weights["token_embd.weight"]
            self.embed = self._pack_or_dense(emb)
        else:
            self.embed = None
        self.head = None
        if with_head:
            self.out_norm = _f32(weights["output_norm.weight"], dev)
            head_t = weights.get("output.weight") or weights["token_embd.weight"]
            v0, v1 = pl.vocab_start, pl.vocab_stop
            self.head = QLinear.from_qtensors([head_t.rows(v0, v1)], dev)
            self.vocab_local = v1 - v0
        self._kv_ids, self._gdn_ids = c.kv_layers(self.layer_ids), c.gdn_layers(self.layer_ids)
        self.gdn_v_local = pl.gdn_v_stop - pl.gdn_v_start
        self.gdn_conv_local = 2 * c.gdn_key_dim + self.gdn_v_local * c.ssm_state
        # hybrid models whose softmax blocks have a head size without an attention kernel here (qwen3.5 checkpoints use 256)
        # run attention on PyTorch ops: decode steps as one batched, shape-static expression that CUDA graphs capture,
        # prefill chunks sequence by sequence
        self.torch_attention = c.is_hybrid and c.head_dim not in (64, 128)
        self.graph_safe = True
        self.layers = [self._build_layer(weights, i) for i in self.layer_ids]
        self.mtp_layers = []
        self.mtp_kv_base = len(self._kv_ids)            # the NextN layers' K/V follow this stage's own layers in the cache
        self.n_kv_layers = len(self._kv_ids) + (c.nextn_layers if with_mtp else 0)
        self.hybrid_dims = None
        if self._gdn_ids:
            self.hybrid_dims = dict(n_layers=len(self._gdn_ids), conv_dim=self.gdn_conv_local, conv_kernel=c.ssm_conv_kernel,
                                    n_v_heads=self.gdn_v_local, d=c.ssm_state)
        for j in range(c.nextn_layers if with_mtp else 0):
            i = c.n_layers + j
            lay = self._build_layer(weights, i)
            p = f"blk.{i}.nextn."
            lay.eh_proj = QLinear.from_qtensors([weights[p + "eh_proj.weight"]], dev)
            lay.enorm = _f32(weights[p + "enorm.weight"], dev)
            lay.hnorm = _f32(weights[p + "hnorm.weight"], dev)
            lay.shared_head_norm = _f32(weights[p + "shared_head_norm.weight"], dev)
            self.mtp_layers.append(lay)
        self._alloc_workspace(max_tokens)

    # ---------------------------------------------------------------------------------------
    def _pack_or_dense(self, t: QTensor):
        t = for_kernels(t)
        n, k = t.shape
        if can_pack(t.qtype, k):
            return pack_matrix(t.raw.to(self.device), t.qtype, n, k)
        return t.to_float().to(self.device)

    def _build_layer(self, w: ModelWeights, i: int) -> CudaLayer:
        c, dev, pl = self.cfg, self.device, self.plan
        p = f"blk.{i}."
        L = CudaLayer()
        L.index = i
        L.attn_norm = _f32(w[p + "attn_norm.weight"], dev)
        L.ffn_norm = _f32(w[p + c.ffn_norm_name], dev)
        L.is_gdn = c.is_gdn_layer(i)
        L.kv_index = self._kv_ids.index(i) if i in self._kv_ids else (self.mtp_kv_base + i - c.n_layers if i >= c.n_layers else None)
        if L.is_gdn:
            self._build_gdn(L, w, p)
            self._build_ffn(L, w, p)
            return L
        D = c.head_dim
        qw = 2 if c.attn_gate else 1                            # rows of a head: [query | gate]
        q = w[p + "attn_q.weight"].rows(pl.q_head_start * D * qw, pl.q_head_stop * D * qw)
        k = w[p + "attn_k.weight"].rows(pl.kv_head_start * D, pl.kv_head_stop * D)
        v = w[p + "attn_v.weight"].rows(pl.kv_head_start * D, pl.kv_head_stop * D)
        bias = None
        if c.qkv_bias:
            bq = _f32(w[p + "attn_q.bias"], dev)[pl.q_head_start * D:pl.q_head_stop * D]
            bk = _f32(w[p + "attn_k.bias"], dev)[pl.kv_head_start * D:pl.kv_head_stop * D]
            bv = _f32(w[p + "attn_v.bias"], dev)[pl.kv_head_start * D:pl.kv_head_stop * D]
            bias = torch.cat([bq, bk, bv]).contiguous()
        L.qkv = QLinear.from_qtensors([q, k, v], dev, bias)
        L.q_norm = _f32(w.get(p + "attn_q_norm.weight"), dev) if c.qk_norm else None
        L.k_norm = _f32(w.get(p + "attn_k_norm.weight"), dev) if c.qk_norm else None
        L.wo = QLinear.from_qtensors([w[p + "attn_output.weight"].cols(pl.q_head_start * D, pl.q_head_stop * D)], dev)
        self._build_ffn(L, w, p)
        return L

    def _build_ffn(self, L: CudaLayer, w: ModelWeights, p: str) -> None:
        c, dev, pl = self.cfg, self.device, self.plan
        if c.is_moe:
            L.router = w[p + "ffn_gate_inp.weight"].to_float().to(dev).to(torch.bfloat16).contiguous()
            e0, e1 = pl.expert_start, pl.expert_stop
            L.experts = self._pack_expert_slab(w, p, e0, e1)
            L.gate_up = L.down = None
            L.shared = None
            if c.shared_expert_ff:
                # the always-on expert of the hybrid MoE family: replicated on every rank and added after the routed experts'
                # sum (its width is one or two K blocks, too narrow to shard)
                sh = CudaLayer()
                sh.gate_up = self._pack_gate_up(w[p + "ffn_gate_shexp.weight"], w[p + "ffn_up_shexp.weight"])
                sh.down = QLinear.from_qtensors([w[p + "ffn_down_shexp.weight"]], dev)
                sh.gate_w = w[p + "ffn_gate_inp_shexp.weight"].to_float().to(dev).reshape(-1, 1).to(torch.bfloat16).contiguous()
                L.shared = sh
        else:
            f0, f1 = pl.ff_start, pl.ff_stop
            g = w[p + "ffn_gate.weight"].rows(f0, f1)
            u = w[p + "ffn_up.weight"].rows(f0, f1)
            L.gate_up = self._pack_gate_up(g, u)
            L.down = QLinear.from_qtensors([w[p + "ffn_down.weight"].cols(f0, f1)], dev)

    def _build_gdn(self, L: CudaLayer, w: ModelWeights, p: str) -> None:
        """Linear-attention block.  One input projection produces q | k (all key heads) | v (this rank's value heads) | z |
        alpha | b in one launch; `wo` is the row-parallel output projection over this rank's value heads
        (sharding as in the reference: src/v2/models/qwen35/Qwen35Schema.h:107-134)."""
        c, dev, pl = self.cfg, self.device, self.plan
        d, kd = c.ssm_state, c.gdn_key_dim
        v0, v1 = pl.gdn_v_start, pl.gdn_v_stop
        qkv, z = w[p + "attn_qkv.weight"], w[p + "attn_gate.weight"]
        L.gdn_index = self._gdn_ids.index(L.index)
        L.qkv = QLinear.from_qtensors([qkv.rows(0, 2 * kd), qkv.rows(2 * kd + v0 * d, 2 * kd + v1 * d), z.rows(v0 * d, v1 * d),
                                       w[p + "ssm_alpha.weight"].rows(v0, v1), w[p + "ssm_beta.weight"].rows(v0, v1)], dev)
        L.z_off = self.gdn_conv_local
        L.ab_off = L.z_off + (v1 - v0) * d
        rows = torch.cat([torch.arange(2 * kd), 2 * kd + torch.arange(v0 * d, v1 * d)])
        L.conv_w = _f32(w[p + "ssm_conv1d.weight"], dev)[rows.to(dev)].contiguous()
        L.ssm_a = _f32(w[p + "ssm_a"], dev)[v0:v1].contiguous()
        L.dt_bias = _f32(w[p + "ssm_dt.bias"], dev)[v0:v1].contiguous()
        L.ssm_norm = _f32(w[p + "ssm_norm.weight"], dev)
        L.wo = QLinear.from_qtensors([w[p + "ssm_out.weight"].cols(v0 * d, v1 * d)], dev)

    def _pack_gate_up(self, g: QTensor, u: QTensor) -> QLinear:
        dev = self.device
        g, u = for_kernels(g), for_kernels(u)
        n, k = g.shape
        if g.qtype == u.qtype and can_pack(g.qtype, k) and n % 16 == 0:
            raw, qt, n2, _ = interleave_gate_up(g.raw.to(dev), u.raw.to(dev), g.qtype, n, k)
            lin = QLinear([(pack_matrix(raw, qt, n2, k), 0)], n2, k)
            lin.fused_swiglu = True
            return lin
        lin = QLinear.from_qtensors([g, u], dev)
        lin.fused_swiglu = False
        return lin

    def _pack_expert_slab(self, w: ModelWeights, p: str, e0: int, e1: int):
        dev = self.device
        ge, ue, de = expert_tensors_for_packing(w, p)
        E, ff, d = ge.shape
        slab = CudaLayer()
        gu_parts = []
        for e in range(e0, e1):
            g, u = ge.expert(e), ue.expert(e)
            raw, qt, n2, _ = interleave_gate_up(g.raw.to(dev), u.raw.to(dev), g.qtype, ff, d)
            gu_parts.append(raw)
        slab.gate_up = pack_experts(torch.cat(gu_parts), ge.qtype, e1 - e0, 2 * ff, d)
        dn = torch.cat([de.expert(e).raw.to(dev) for e in range(e0, e1)])
        slab.down = pack_experts(dn, de.qtype, e1 - e0, d, ff)
        slab.e0, slab.n_local = e0, e1 - e0
        return slab

    def weight_bytes(self) -> int:
        tot = 0
        for L in self.layers + self.mtp_layers:
            tot += L.qkv.nbytes() + L.wo.nbytes()
            if L.gate_up is not None:
                tot += L.gate_up.nbytes() + L.down.nbytes()
            else:
                tot += L.experts.gate_up.nbytes() + L.experts.down.nbytes()
                if getattr(L, "shared", None) is not None:
                    tot += L.shared.gate_up.nbytes() + L.shared.down.nbytes()
        if self.head is not None:
            tot += self.head.nbytes()
        return tot

    def _alloc_workspace(self, T: int) -> None:
        c, dev = self.cfg, self.device
        bf, f32 = torch.bfloat16, torch.float32
        e = lambda *s, dt=bf: torch.empty(*s, dtype=dt, device=dev)
        self.ws_h = e(T, c.d_model, dt=f32)
        self.ws_xn = e(T, c.d_model)
        gdn_in = self.gdn_conv_local + self.gdn_v_local * c.ssm_state + 2 * self.gdn_v_local if self._gdn_ids else 0
        self.ws_qkv = e(T, max(self.qkv_dim + (self.q_dim if c.attn_gate else 0), (gdn_in + 63) // 64 * 64))
        self.ws_q = e(T, self.n_heads_local, c.head_dim)
        self.ws_o = e(T, self.q_dim)
        self.ws_gdn_o = e(T, self.gdn_v_local * c.ssm_state) if self._gdn_ids else None      # input of the block's output projection
        self.ws_gdn_y = e(T, self.gdn_conv_local, dt=f32) if self._gdn_ids else None
        ff = max(self.ff_local, c.expert_ff if c.is_moe else 0)
        self.ws_act = e(T, ff)
        self.ws_shared = e(T, c.d_model, dt=f32) if c.shared_expert_ff else None
        self.ws_sh_gu = e(T, 2 * c.shared_expert_ff) if c.shared_expert_ff else None
        self.ws_sh_act = e(T, c.shared_expert_ff) if c.shared_expert_ff else None
        self.ws_gu = e(T, 2 * ff) if any(getattr(L.gate_up, "fused_swiglu", True) is False for L in self.layers if L.gate_up) else None
        self.ws_partial = e(T, c.d_model, dt=f32) if self.tp is not None else None

    # ---------------------------------------------------------------------------------------
    def embed_tokens(self, tokens: torch.Tensor, out: torch.Tensor) -> None:
        if isinstance(self.embed, PackedWeight):
            ops.gather_rows(self.embed, tokens, out)
        else:
            out.copy_(self.embed[tokens.long()])

    def _attention(self, L: CudaLayer, fb: ForwardBatch, kv_layer: torch.Tensor, T: int) -> torch.Tensor:
        c = self.cfg
        qkv, q, o = self.ws_qkv[:T], self.ws_q[:T], self.ws_o[:T]
        ops.rope_kv(qkv, q, kv_layer, L.q_norm, L.k_norm, fb.positions, fb.seq_ids, fb.block_table,
                    self.n_heads_local, self.n_kv_local, c.head_dim, c.rope_theta, c.rms_eps)
        scale = 1.0 / math.sqrt(c.head_dim)
        o3 = o.view(T, self.n_heads_local, c.head_dim)
        if fb.is_decode:
            ops.attn_decode(q, kv_layer, o3, fb.block_table, fb.seq_lens, self.n_heads_local, self.n_kv_local,
                            c.head_dim, fb.rows_per_seq, scale, fb.n_splits, self.scratch)
        else:
            kv_bf16, btab = self._kv_for_prefill(fb, kv_layer)
            ops.attn_prefill(q, kv_bf16, o3, btab, fb.cu_q, fb.ctx_lens, self.n_heads_local,
                             self.n_kv_local, c.head_dim, scale, fb.max_q_len, scratch=self.scratch)
        return o

    def _linear_attention(self, L: CudaLayer, fb: ForwardBatch, inp: torch.Tensor, T: int) -> torch.Tensor:
        """Between the input and output projections of a Gated-DeltaNet block.  Decode steps (one row per sequence) run
        the two step kernels on the sequences' state slots; prefill chunks run the chunk-parallel form on PyTorch ops,
        sequence by sequence (one host synchronisation per forward pass for the row ranges)."""
        c, hs = self.cfg, self._kv.hybrid
        d, nv = c.ssm_state, self.gdn_v_local
        o = self.ws_gdn_o[:T]
        conv, rec = hs.conv[L.gdn_index], hs.rec[L.gdn_index]
        from ..models import gdn
        if fb.defer_state:
            B = fb.state_slots.shape[0]
            x = inp.float().view(B, T // B, -1)
            C = self.gdn_conv_local
            rows, hs.stash[L.gdn_index] = gdn.gdn_rows_deferred(
                x[..., :C], x[..., L.z_off:L.z_off + nv * d], x[..., L.ab_off:L.ab_off + nv], x[..., L.ab_off + nv:L.ab_off + 2 * nv],
                L.conv_w, L.ssm_a, L.dt_bias, L.ssm_norm, conv, rec, fb.state_slots.long(), c.ssm_k_heads, nv, d, c.rms_eps,
                self.plan.gdn_v_start)
            hs.stash_slots = fb.state_slots.long()
            o.copy_(rows)
            return o
        if fb.is_decode and fb.rows_per_seq == 1:
            ops.gdn_step(inp, self.gdn_conv_local, L.z_off, L.ab_off, L.conv_w, L.ssm_a, L.dt_bias, L.ssm_norm, conv, rec,
                         fb.state_slots, self.ws_gdn_y[:T], o, c.ssm_k_heads, self.plan.gdn_v_start, c.rms_eps)
            return o
        seqs = getattr(fb, "_gdn_seqs", None)
        if seqs is None:
            seqs = fb._gdn_seqs = gdn.batch_sequences(fb.seq_ids, fb.positions, fb.state_slots)
        C = self.gdn_conv_local
        x = inp.float()
        rows = gdn.gdn_block_rows(x[:, :C], x[:, L.z_off:L.z_off + nv * d], x[:, L.ab_off:L.ab_off + nv],
                                  x[:, L.ab_off + nv:L.ab_off + 2 * nv], seqs, conv, rec, L.conv_w, L.ssm_a, L.dt_bias, L.ssm_norm,
                                  c.ssm_k_heads, nv, d, c.rms_eps, self.plan.gdn_v_start)
        o.copy_(rows)
        return o

    def _attention_gated(self, L: CudaLayer, fb: ForwardBatch, kv_layer: torch.Tensor, qkv: torch.Tensor, T: int) -> torch.Tensor:
        """Softmax block of the hybrid family: every head's projection rows are [query | gate], only the first `rotary_dim`
        values of a head are rotated, and the attention output is scaled by sigmoid(gate) before the output projection.
        The split, QK-norm, rotation and cache append are PyTorch ops (a dozen small launches per block, one block in
        four); attention itself runs the paged kernels for head sizes 64 and 128 and PyTorch otherwise."""
        from ..models.reference import rmsnorm, rope_split_half
        c = self.cfg
        H, Hk, D = self.n_heads_local, self.n_kv_local, c.head_dim
        if kv_layer.dtype == torch.uint8:
            raise NotImplementedError("the 8-bit KV cache is not available for the gated-attention blocks of hybrid models")
        qw = 2 if c.attn_gate else 1
        qg = qkv[:, :H * D * qw].view(T, H, qw, D)
        q = qg[:, :, 0].float()
        gate = qg[:, :, 1].reshape(T, H * D).float() if c.attn_gate else None
        k = qkv[:, H * D * qw:H * D * qw + Hk * D].view(T, Hk, D).float()
        v = qkv[:, H * D * qw + Hk * D:H * D * qw + 2 * Hk * D].view(T, Hk, D)
        if L.q_norm is not None:
            q, k = rmsnorm(q, L.q_norm, c.rms_eps), rmsnorm(k, L.k_norm, c.rms_eps)
        pos = fb.positions.long()
        q = rope_split_half(q, pos, c.rope_theta, c.rotary_dim)
        k = rope_split_half(k, pos, c.rope_theta, c.rotary_dim)
        page = fb.block_table.long()[fb.seq_ids.long(), pos // 64]
        off = pos % 64
        kv_layer[page, 0, :, off] = k.to(kv_layer.dtype)
        kv_layer[page, 1, :, off] = v.to(kv_layer.dtype)
        o = self.ws_o[:T]
        o3 = o.view(T, H, D)
        scale = 1.0 / math.sqrt(D)
        if self.torch_attention and fb.is_decode and fb.rows_per_seq == 1:
            o3.copy_(paged_decode_attention_torch(q, kv_layer, fb.block_table, fb.seq_lens, scale))
        elif self.torch_attention:
            o3.copy_(self._attention_torch(q, fb, kv_layer, scale))
        else:
            qb = self.ws_q[:T]
            qb.copy_(q)
            if fb.is_decode:
                ops.attn_decode(qb, kv_layer, o3, fb.block_table, fb.seq_lens, H, Hk, D, fb.rows_per_seq, scale, fb.n_splits, self.scratch)
            else:
                ops.attn_prefill(qb, kv_layer, o3, fb.block_table, fb.cu_q, fb.ctx_lens, H, Hk, D, scale, fb.max_q_len, scratch=self.scratch)
        if gate is not None:
            o.copy_(o.float() * torch.sigmoid(gate))
        return o

    def _attention_torch(self, q: torch.Tensor, fb: ForwardBatch, kv_layer: torch.Tensor, scale: float) -> torch.Tensor:
        return paged_attention_torch(q, kv_layer, fb.block_table, fb.seq_ids, fb.positions, scale)

    def _kv_for_prefill(self, fb: ForwardBatch, kv_layer: torch.Tensor):
        """The prefill kernels read bf16 pages.  With the 8-bit cache the pages of the chunk's sequences (context and the rows
        just appended) are expanded into a staging pool that is reused layer after layer, and the kernels get a block table
        into that pool.  Decode reads the 8-bit pages directly."""
        if kv_layer.dtype != torch.uint8:
            return kv_layer, fb.block_table
        c = self.cfg
        B, P = fb.block_table.shape
        if fb.max_kv_len:
            P = min(P, (fb.max_kv_len + 63) // 64)
        st = getattr(self, "_q8_prefill", None)
        if st is None or st["fb"] is not fb:
            n_tok = (fb.ctx_lens + (fb.cu_q[1:] - fb.cu_q[:-1])).to(torch.int32)
            st = {"fb": fb, "n_tok": n_tok, "bt": fb.block_table[:, :P].contiguous(),
                  "bt2": torch.arange(B * P, dtype=torch.int32, device=self.device).view(B, P)}
            self._q8_prefill = st
        need = B * P
        pool = getattr(self, "_q8_pool", None)
        if pool is None or pool.shape[0] < need:
            pool = torch.empty(need, 2, self.n_kv_local, 64, c.head_dim, dtype=torch.bfloat16, device=self.device)
            self._q8_pool = pool
        ops.kv_dequant_pages(kv_layer, st["bt"], st["n_tok"], self.n_kv_local, c.head_dim, pool)
        return pool, st["bt2"]

    def _row_parallel_resid(self, lin: QLinear, x: torch.Tensor, h: torch.Tensor) -> None:
        """h += x @ W^T, summed over tensor-parallel ranks."""
        if self.tp is None or self.tp.size == 1:
            lin(x, h, epi=ops.EPI_RESID, scratch=self.scratch, xn=x if x.shape[0] > ops.GEMV_MAX_ROWS else None)
            return
        self.tp.row_parallel_resid(lin, x, h, self)
        if self.tp.verify_checksums and not torch.cuda.is_current_stream_capturing():
            # debug: after the (fused or NCCL) reduction every rank must hold the same residual rows, bit for bit
            self.tp.verify_replicated(h, "row-parallel projection + all-reduce")

    def _layer(self, L: CudaLayer, fb: ForwardBatch, kv_layer: torch.Tensor, T: int) -> None:
        c, sc = self.cfg, self.scratch
        h = self.ws_h[:T]
        small = T <= ops.GEMV_MAX_ROWS
        qkv = self.ws_qkv[:T, :L.qkv.n_out]
        if small:
            L.qkv(h, qkv, norm_w=L.attn_norm, eps=c.rms_eps, scratch=sc)
        else:
            xn = self.ws_xn[:T]
            ops.rmsnorm(h, L.attn_norm, xn, c.rms_eps)
            L.qkv(xn, qkv, scratch=sc, xn=xn)
        if getattr(L, "is_gdn", False):
            o = self._linear_attention(L, fb, qkv, T)
        elif c.attn_gate or c.rotary_dim != c.head_dim or self.torch_attention:
            o = self._attention_gated(L, fb, kv_layer, qkv, T)
        else:
            o = self._attention(L, fb, kv_layer, T)
        self._row_parallel_resid(L.wo, o, h)
        if c.is_moe:
            self._moe(L, h, T)
            return
        act = self.ws_act[:T, :self.ff_local]
        if small:
            if L.gate_up.fused_swiglu:
                L.gate_up(h, act, norm_w=L.ffn_norm, eps=c.rms_eps, epi=ops.EPI_SWIGLU, scratch=sc)
            else:
                gu = self.ws_gu[:T, :2 * self.ff_local]
                L.gate_up(h, gu, norm_w=L.ffn_norm, eps=c.rms_eps, scratch=sc)
                act.copy_((torch.nn.functional.silu(gu[:, :self.ff_local].float()) * gu[:, self.ff_local:].float()).to(act.dtype))
        else:
            xn = self.ws_xn[:T]
            ops.rmsnorm(h, L.ffn_norm, xn, c.rms_eps)
            if L.gate_up.fused_swiglu:
                L.gate_up(xn, act, epi=ops.EPI_SWIGLU, scratch=sc, xn=xn)
            else:
                gu = self.ws_gu[:T, :2 * self.ff_local]
                L.gate_up(xn, gu, scratch=sc, xn=xn)
                act.copy_((torch.nn.functional.silu(gu[:, :self.ff_local].float()) * gu[:, self.ff_local:].float()).to(act.dtype))
        self._row_parallel_resid(L.down, act, h)

    def _debug_hooks(self):
        """Per-layer checks behind environment switches (never inside CUDA-graph capture):
        LLAMINAR_VALIDATE_TENSORS scans the residual stream for NaN/Inf after every layer (reference: the stage verifier,
        src/v2/graph/StageVerifier.cpp); LLAMINAR_STAGE_DUMP_DIR writes it to `<dir>/layer_<n>_call_<k>.pt`
        (reference: src/v2/execution/debug/StageDumper.h)."""
        from ..utils.env import debug_env
        env = debug_env()
        validate, dump_dir = env.validate_tensors, env.stage_dump_dir
        if not (validate or dump_dir) or torch.cuda.is_current_stream_capturing():
            return None
        self._dump_calls = getattr(self, "_dump_calls", 0) + 1
        call = self._dump_calls

        def hook(layer: int, h: torch.Tensor) -> None:
            if validate:
                n_nan, n_inf = ops.nan_scan(h)
                if n_nan or n_inf:
                    raise FloatingPointError(f"layer {layer}: {n_nan} NaN and {n_inf} Inf values in the residual stream")
            if dump_dir:
                import os
                os.makedirs(dump_dir, exist_ok=True)
                torch.save(h.detach().float().cpu(), os.path.join(dump_dir, f"layer_{layer:03d}_call_{call:05d}.pt"))
        return hook

    def _moe(self, L: CudaLayer, h: torch.Tensor, T: int) -> None:
        from .moe import moe_forward
        shared = self._shared_expert(L, h, T) if getattr(L, "shared", None) is not None else None
        moe_forward(self, L, h, T)
        if shared is not None:
            h += shared

    def _shared_expert(self, L: CudaLayer, h: torch.Tensor, T: int) -> torch.Tensor:
        """sigmoid(x . g) * FFN_shared(x) for the normed rows x of `h`, as fp32 rows in a workspace (read before the routed
        experts update `h` in place)."""
        c, sc, sh = self.cfg, self.scratch, L.shared
        xn = self.ws_xn[:T]
        ops.rmsnorm(h, L.ffn_norm, xn, c.rms_eps)
        big = xn if T > ops.GEMV_MAX_ROWS else None
        act = self.ws_sh_act[:T]
        if sh.gate_up.fused_swiglu:
            sh.gate_up(xn, act, epi=ops.EPI_SWIGLU, scratch=sc, xn=big)
        else:
            gu = self.ws_sh_gu[:T]
            sh.gate_up(xn, gu, scratch=sc, xn=big)
            f = c.shared_expert_ff
            act.copy_((torch.nn.functional.silu(gu[:, :f].float()) * gu[:, f:].float()).to(act.dtype))
        y = self.ws_shared[:T]
        sh.down(act, y, scratch=sc, xn=act if T > ops.GEMV_MAX_ROWS else None)
        y.mul_(torch.sigmoid((xn @ sh.gate_w).float()))
        return y

    def _final_logits(self, h_rows: torch.Tensor, out: torch.Tensor | None, norm_w: torch.Tensor) -> torch.Tensor:
        rows = h_rows.shape[0]
        if out is None:
            out = torch.empty(rows, self.vocab_local, dtype=torch.float32, device=self.device)
        if rows <= ops.GEMV_MAX_ROWS:
            self.head(h_rows, out, norm_w=norm_w, eps=self.cfg.rms_eps, scratch=self.scratch)
        else:
            xn = torch.empty(rows, self.cfg.d_model, dtype=torch.bfloat16, device=self.device)
            ops.rmsnorm(h_rows.contiguous(), norm_w, xn, self.cfg.rms_eps)
            self.head(xn, out, scratch=self.scratch, xn=xn)
        return out

    # -- sequence-sharded tensor-parallel prefill: fused GEMM -> reduce-scatter and all-gather -> GEMM ---------------------
    SEQ_SHARD_MIN_ROWS = 64          # per rank; below that the replicated path (small-batch kernels, fused all-reduce) is faster

    def _seq_shard_arena(self, fb: ForwardBatch, T: int):
        """The arena of the sequence-sharded path when this forward call can take it, else None.  It serves prefill chunks
        of a dense model under fused tensor parallelism: every weight in a packed format, no pipeline input, no debug taps,
        no consumer of the full hidden state (the engine turns ``seq_shard`` off when a NextN head needs all rows)."""
        tp = self.tp
        if (tp is None or tp.size == 1 or not tp.fused or not getattr(self, "seq_shard", True) or fb.is_decode or fb.embeds is not None
                or self.cfg.is_moe or self.cfg.is_hybrid or getattr(self, "taps", None) is not None or T < self.SEQ_SHARD_MIN_ROWS * tp.size
                or self.cfg.d_model % 128 or self.cfg.d_model > 8192 or not isinstance(self.embed, PackedWeight)):
            return None
        if getattr(self, "_ss_ok", None) is None:
            lins = [l for L in self.layers for l in (L.qkv, L.wo, L.gate_up, L.down)]
            self._ss_ok = (all(isinstance(w, PackedWeight) for l in lins for w, _ in l.parts)
                           and all(len(L.wo.parts) == 1 and len(L.down.parts) == 1 and L.gate_up.fused_swiglu for L in self.layers))
        if not self._ss_ok:
            return None
        if getattr(self, "_ss_arena", None) is None:
            from ..parallel.symm import SeqShardArena
            rows_cap = (self.max_tokens + tp.size - 1) // tp.size
            self._ss_arena = SeqShardArena(tp.group, self.device, rows_cap, self.cfg.d_model)
        return self._ss_arena

    def _column_parallel_gathered(self, lin: QLinear, arena, T: int, tw: int, out: torch.Tensor, epi=ops.EPI_STORE) -> None:
        """out = gather(x) @ W_shard^T: the first part's launch pulls the rows from their owners while it multiplies; further
        parts (another block format) read the staged copy."""
        for i, (w, col) in enumerate(lin.parts):
            o = out if epi == ops.EPI_SWIGLU else (out[:, col:col + w.n] if (col or w.n != out.shape[1]) else out)
            b = lin.bias[col:col + w.n] if lin.bias is not None else None
            if i == 0:
                arena.ag.gemm(w, T, tw, o, epi=epi, bias=b)
            else:
                ops.gemm(w, arena.ag.gathered(T, lin.k), o, epi=epi, bias=b, scratch=self.scratch)

    def _forward_seq_sharded(self, arena, fb: ForwardBatch, kv: PagedKVCache, T: int, logits_out, want_logits: bool, kv_layer_offset: int):
        c, tp = self.cfg, self.tp
        tw = arena.rows_per_rank(T)
        r0, mine = arena.my_rows(T, tw)
        h = self.ws_h[:mine]                                   # this rank's rows of the residual stream
        if mine:
            self.embed_tokens(fb.tokens[r0:r0 + mine], h)
            ops.rmsnorm(h, self.layers[0].attn_norm, arena.ag.own_rows(tw, c.d_model)[:mine], c.rms_eps)
        n_layers = len(self.layers)
        for li, L in enumerate(self.layers):
            qkv = self.ws_qkv[:T]
            self._column_parallel_gathered(L.qkv, arena, T, tw, qkv)
            o = self._attention(L, fb, kv.layers[kv_layer_offset + li], T)
            arena.gemm_reduce_scatter(L.wo.parts[0][0], o, tw)
            arena.reduce_norm(h, T, tw, c.d_model, L.ffn_norm, arena.ag.own_rows(tw, c.d_model)[:mine] if mine else None, c.rms_eps)
            act = self.ws_act[:T, :self.ff_local]
            self._column_parallel_gathered(L.gate_up, arena, T, tw, act, epi=ops.EPI_SWIGLU)
            arena.gemm_reduce_scatter(L.down.parts[0][0], act, tw)
            nxt = self.layers[li + 1].attn_norm if li + 1 < n_layers else None
            arena.reduce_norm(h, T, tw, c.d_model, nxt, (arena.ag.own_rows(tw, c.d_model)[:mine] if mine else None) if nxt is not None else None,
                              c.rms_eps)
            tp.stats["fused_calls"] += 4
        # the rows that get logits (and whose hidden state the caller keeps) are brought to every rank: each is owned by
        # one rank, the others contribute zeros to a small all-reduce
        rows = fb.logit_rows if fb.logit_rows is not None else torch.arange(T, dtype=torch.int32, device=self.device)
        logits, sel = None, None
        if want_logits and rows.numel():
            idx = rows.long() - r0
            ok = (idx >= 0) & (idx < mine)
            sel = torch.zeros(rows.numel(), c.d_model, dtype=torch.float32, device=self.device)
            if mine:
                sel[ok] = h.index_select(0, idx.clamp(0, max(mine - 1, 0)))[ok]
            tp.all_reduce(sel)
            if self.head is not None:
                logits = self._final_logits(sel, logits_out, self.out_norm)
        return logits, _HiddenRows(rows, sel)

    @torch.no_grad()
    def forward(self, fb: ForwardBatch, kv: PagedKVCache, logits_out: torch.Tensor | None = None,
                want_logits: bool = True, kv_layer_offset: int = 0):
        """Runs the layers of this model (stage) over the batch; returns (logits or None, hidden [T, d] fp32 view)."""
        T = fb.tokens.shape[0] if fb.embeds is None else fb.embeds.shape[0]
        assert T <= self.max_tokens, f"{T} tokens exceed the workspace ({self.max_tokens})"
        debug = self._debug_hooks()
        arena = self._seq_shard_arena(fb, T) if debug is None else None
        if arena is not None:
            return self._forward_seq_sharded(arena, fb, kv, T, logits_out, want_logits, kv_layer_offset)
        if debug is not None:
            errs = fb.index_errors(self.cfg.vocab_size, kv.n_pages, self.cfg.context_length)
            if errs:
                raise IndexError("forward batch rejected before launch: " + "; ".join(errs))
        h = self.ws_h[:T]
        if fb.embeds is not None:
            h.copy_(fb.embeds)
        else:
            self.embed_tokens(fb.tokens, h)
        self._kv = kv
        for li, L in enumerate(self.layers):
            self._layer(L, fb, kv.layers[kv_layer_offset + L.kv_index] if L.kv_index is not None else None, T)
            if debug is not None:
                debug(self.layer_ids[li], h)
            if getattr(self, "taps", None) is not None:       # per-layer hidden states for the parity report
                self.taps[f"layer{self.layer_ids[li]}"] = h.float().clone()
        logits = None
        if want_logits and self.head is not None:
            rows = h if fb.logit_rows is None else h.index_select(0, fb.logit_rows.long())
            logits = self._final_logits(rows, logits_out, self.out_norm)
        return logits, h

    @torch.no_grad()
    def mtp_forward(self, fb: ForwardBatch, hidden: torch.Tensor, kv: PagedKVCache, depth: int = 0,
                    logits_out: torch.Tensor | None = None):
        """NextN head: fb.tokens are the *next* tokens, ``hidden`` the trunk's final hidden rows (fp32 [T, d]).
        Uses KV layer ``n_layers + depth`` of the cache."""
        c = self.cfg
        L = self.mtp_layers[depth]
        T = fb.tokens.shape[0]
        emb = torch.empty(T, c.d_model, dtype=torch.float32, device=self.device)
        self.embed_tokens(fb.tokens, emb)
        cat = torch.empty(T, 2 * c.d_model, dtype=torch.bfloat16, device=self.device)
        ops.mtp_concat_norm(emb, hidden.float().contiguous(), L.enorm, L.hnorm, cat, c.rms_eps)
        x0 = torch.empty(T, c.d_model, dtype=torch.float32, device=self.device)
        L.eh_proj(cat, x0, scratch=self.scratch, xn=cat if T > ops.GEMV_MAX_ROWS else None)
        h = self.ws_h[:T]
        h.copy_(x0)
        self._layer(L, fb, kv.layers[self.mtp_kv_base + depth], T)
        rows = h if fb.logit_rows is None else h.index_select(0, fb.logit_rows.long())
        logits = self._final_logits(rows, logits_out, L.shared_head_norm)
        return logits, h
