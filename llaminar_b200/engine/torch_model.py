"""Pure-PyTorch model runner with the same interface as :class:`CudaModel` (paged KV, ForwardBatch).

It is the CPU execution path (``-d cpu``) and lets the scheduler, prefix cache, speculative
decoding and the parallel layouts be tested without a GPU.  Math is fp32 on dequantised weights;
tensor-parallel ranks hold the same slices the GPU runner would (see parallel/tp_plan.py) and
sum the row-parallel partial results with ``torch.distributed`` (gloo on CPU).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..models import gdn
from ..models.config import ModelConfig
from ..models.reference import moe_route, rmsnorm, rope_split_half
from ..models.weights import ModelWeights
from ..parallel.tp_plan import TPPlan
from .cuda_model import ForwardBatch
from .kv_cache import PAGE_SIZE, PagedKVCache


class TorchPagedModel:
    def __init__(self, weights: ModelWeights, device="cpu", max_tokens: int = 4096, tp=None, layer_range=None,
                 with_head: bool = True, with_embed: bool = True, with_mtp: bool = True):
        self.cfg: ModelConfig = weights.config
        self.device = torch.device(device)
        self.tp = tp
        self.max_tokens = max_tokens
        c = self.cfg
        pl = self.plan = TPPlan.build(c, tp.size if tp else 1, tp.rank if tp else 0, getattr(tp, "moe_mode", "expert-parallel"))
        self.n_heads_local, self.n_kv_local = pl.n_heads_local, pl.n_kv_local
        self.layer_ids = list(range(*layer_range)) if layer_range else list(range(c.n_layers))
        D = c.head_dim
        f = lambda name: weights[name].to_float().to(self.device)
        self.embed = f("token_embd.weight") if with_embed else None
        self.head = None
        if with_head:
            self.out_norm = f("output_norm.weight")
            head = weights.get("output.weight") or weights["token_embd.weight"]
            self.head = head.rows(pl.vocab_start, pl.vocab_stop).to_float().to(self.device)
            self.vocab_local = pl.vocab_stop - pl.vocab_start

        kv_ids, gdn_ids = c.kv_layers(self.layer_ids), c.gdn_layers(self.layer_ids)

        def ffn(L, p):
            if c.is_moe:
                L["router"] = f(p + "ffn_gate_inp.weight")
                e0, e1 = pl.expert_start, pl.expert_stop
                L["e0"], L["e1"] = e0, e1
                L["wg"] = f(p + "ffn_gate_exps.weight")[e0:e1]
                L["wu"] = f(p + "ffn_up_exps.weight")[e0:e1]
                L["wd"] = f(p + "ffn_down_exps.weight")[e0:e1]
                if c.shared_expert_ff:                      # replicated on every rank, added after the experts' sum
                    L["sh"] = (f(p + "ffn_gate_shexp.weight"), f(p + "ffn_up_shexp.weight"), f(p + "ffn_down_shexp.weight"),
                               f(p + "ffn_gate_inp_shexp.weight").reshape(-1, 1))
                return
            L["wg"] = f(p + "ffn_gate.weight")[pl.ff_start:pl.ff_stop]
            L["wu"] = f(p + "ffn_up.weight")[pl.ff_start:pl.ff_stop]
            L["wd"] = f(p + "ffn_down.weight")[:, pl.ff_start:pl.ff_stop]

        def gdn_layer(i):
            """Linear-attention block: all key heads (q and k rows) plus this rank's value heads."""
            p = f"blk.{i}."
            L = {"attn_norm": f(p + "attn_norm.weight"), "ffn_norm": f(p + c.ffn_norm_name), "index": i,
                 "gdn_index": gdn_ids.index(i)}
            d, kd = c.ssm_state, c.gdn_key_dim
            v0, v1 = pl.gdn_v_start, pl.gdn_v_stop
            rows = torch.cat([torch.arange(2 * kd), 2 * kd + torch.arange(v0 * d, v1 * d)])
            L["wqkv"] = f(p + "attn_qkv.weight")[rows]
            L["conv_w"] = f(p + "ssm_conv1d.weight")[rows]
            L["wz"] = f(p + "attn_gate.weight")[v0 * d:v1 * d]
            L["walpha"], L["wbeta"] = f(p + "ssm_alpha.weight")[v0:v1], f(p + "ssm_beta.weight")[v0:v1]
            L["ssm_a"], L["dt_bias"] = f(p + "ssm_a")[v0:v1], f(p + "ssm_dt.bias")[v0:v1]
            L["ssm_norm"] = f(p + "ssm_norm.weight")
            L["wout"] = f(p + "ssm_out.weight")[:, v0 * d:v1 * d]
            ffn(L, p)
            return L

        def layer(i):
            if c.is_gdn_layer(i):
                return gdn_layer(i)
            p = f"blk.{i}."
            L = {"attn_norm": f(p + "attn_norm.weight"), "ffn_norm": f(p + c.ffn_norm_name), "index": i,
                 "kv_index": kv_ids.index(i) if i in kv_ids else None}
            qs, qe, ks, ke = pl.q_head_start * D, pl.q_head_stop * D, pl.kv_head_start * D, pl.kv_head_stop * D
            qw = 2 if c.attn_gate else 1                       # rows of a head: [query | gate]
            L["wq"], L["wk"], L["wv"] = f(p + "attn_q.weight")[qs * qw:qe * qw], f(p + "attn_k.weight")[ks:ke], f(p + "attn_v.weight")[ks:ke]
            L["wo"] = f(p + "attn_output.weight")[:, qs:qe]
            if c.qkv_bias:
                L["bq"], L["bk"], L["bv"] = f(p + "attn_q.bias")[qs:qe], f(p + "attn_k.bias")[ks:ke], f(p + "attn_v.bias")[ks:ke]
            if c.qk_norm:
                L["qn"], L["kn"] = f(p + "attn_q_norm.weight"), f(p + "attn_k_norm.weight")
            ffn(L, p)
            return L

        self.layers = [layer(i) for i in self.layer_ids]
        self.mtp_layers = []
        self.mtp_kv_base = len(kv_ids)                  # the NextN layers' K/V follow this stage's own layers in the cache
        self.n_kv_layers = len(kv_ids) + (c.nextn_layers if with_mtp else 0)
        # what the engine needs to size the linear-attention state pools of this stage (None: no such layers)
        self.hybrid_dims = None
        if gdn_ids:
            nv = pl.gdn_v_stop - pl.gdn_v_start
            self.hybrid_dims = dict(n_layers=len(gdn_ids), conv_dim=2 * c.gdn_key_dim + nv * c.ssm_state,
                                    conv_kernel=c.ssm_conv_kernel, n_v_heads=nv, d=c.ssm_state)
        for j in range(c.nextn_layers if with_mtp else 0):
            i = c.n_layers + j
            L = layer(i)
            p = f"blk.{i}.nextn."
            for k in ("eh_proj", "enorm", "hnorm", "shared_head_norm"):
                L[k] = f(p + k + ".weight")
            self.mtp_layers.append(L)

    def weight_bytes(self) -> int:
        return 0

    # ---------------------------------------------------------------------------------------
    def _sum_ranks(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp is not None and self.tp.size > 1:
            self.tp.all_reduce(x)
        return x

    def _attention(self, L, x, fb: ForwardBatch, kvl: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        T, D = x.shape[0], c.head_dim
        q, k, v = x @ L["wq"].T, x @ L["wk"].T, x @ L["wv"].T
        if c.qkv_bias:
            q, k, v = q + L["bq"], k + L["bk"], v + L["bv"]
        gate = None
        if c.attn_gate:
            q, gate = q.view(T, self.n_heads_local, 2, D).unbind(dim=2)
            gate = gate.reshape(T, -1)
        q = q.reshape(T, self.n_heads_local, D)
        k = k.view(T, self.n_kv_local, D)
        v = v.view(T, self.n_kv_local, D)
        if c.qk_norm:
            q, k = rmsnorm(q, L["qn"], c.rms_eps), rmsnorm(k, L["kn"], c.rms_eps)
        pos = fb.positions.long()
        q, k = rope_split_half(q, pos, c.rope_theta, c.rotary_dim), rope_split_half(k, pos, c.rope_theta, c.rotary_dim)
        sid = fb.seq_ids.long()
        page = fb.block_table.long()[sid, pos // PAGE_SIZE]
        off = pos % PAGE_SIZE
        kvl[page, 0, :, off] = k.to(kvl.dtype)
        kvl[page, 1, :, off] = v.to(kvl.dtype)
        g = self.n_heads_local // self.n_kv_local
        out = torch.empty(T, self.n_heads_local, D, dtype=torch.float32, device=x.device)
        scale = 1.0 / math.sqrt(D)
        for b in sid.unique().tolist():
            rows = (sid == b).nonzero(as_tuple=True)[0]
            last = int(pos[rows].max())
            n_pages = last // PAGE_SIZE + 1
            pages = fb.block_table.long()[b, :n_pages]
            K = kvl[pages, 0].permute(1, 0, 2, 3).reshape(self.n_kv_local, n_pages * PAGE_SIZE, D)[:, :last + 1].float()
            V = kvl[pages, 1].permute(1, 0, 2, 3).reshape(self.n_kv_local, n_pages * PAGE_SIZE, D)[:, :last + 1].float()
            K, V = K.repeat_interleave(g, 0), V.repeat_interleave(g, 0)
            s = torch.einsum("thd,hsd->hts", q[rows], K) * scale
            mask = torch.arange(last + 1, device=x.device)[None, :] > pos[rows][:, None]
            s = s.masked_fill(mask[None], float("-inf"))
            out[rows] = torch.einsum("hts,hsd->thd", torch.softmax(s, -1), V)
        out = out.reshape(T, -1)
        if gate is not None:
            out = out * torch.sigmoid(gate)
        return out @ L["wo"].T

    def _linear_attention(self, L, x, fb: ForwardBatch, kv: PagedKVCache) -> torch.Tensor:
        c, hs, gi = self.cfg, kv.hybrid, L["gdn_index"]
        nv = self.plan.gdn_v_stop - self.plan.gdn_v_start
        if fb.defer_state:                       # speculative verification: R rows per sequence, state committed afterwards
            B = fb.state_slots.shape[0]
            sh = lambda t: t.view(B, x.shape[0] // B, -1)
            rows, hs.stash[gi] = gdn.gdn_rows_deferred(sh(x @ L["wqkv"].T), sh(x @ L["wz"].T), sh(x @ L["walpha"].T), sh(x @ L["wbeta"].T),
                                                       L["conv_w"], L["ssm_a"], L["dt_bias"], L["ssm_norm"], hs.conv[gi], hs.rec[gi],
                                                       fb.state_slots.long(), c.ssm_k_heads, nv, c.ssm_state, c.rms_eps,
                                                       self.plan.gdn_v_start)
            hs.stash_slots = fb.state_slots.long()
            return rows @ L["wout"].T
        seqs = gdn.batch_sequences(fb.seq_ids, fb.positions, fb.state_slots)
        rows = gdn.gdn_block_rows(x @ L["wqkv"].T, x @ L["wz"].T, x @ L["walpha"].T, x @ L["wbeta"].T, seqs,
                                  hs.conv[gi], hs.rec[gi], L["conv_w"], L["ssm_a"], L["dt_bias"], L["ssm_norm"],
                                  c.ssm_k_heads, self.plan.gdn_v_stop - self.plan.gdn_v_start, c.ssm_state, c.rms_eps,
                                  self.plan.gdn_v_start)
        return rows @ L["wout"].T

    def _ffn(self, L, x: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        if not c.is_moe:
            return (F.silu(x @ L["wg"].T) * (x @ L["wu"].T)) @ L["wd"].T
        idx, wt = moe_route(x @ L["router"].T, c.n_experts_used, c.norm_topk_prob)
        if getattr(self, "expert_stats", None) is not None:
            self.expert_stats.record(L["index"], idx)
        out = torch.zeros_like(x)
        for e in range(L["e0"], L["e1"]):
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            le = e - L["e0"]
            xe = x[tok]
            ye = (F.silu(xe @ L["wg"][le].T) * (xe @ L["wu"][le].T)) @ L["wd"][le].T
            out.index_add_(0, tok, ye * wt[tok, slot].unsqueeze(-1))
        return out

    def _layer(self, L, h, fb, kvl, kv=None):
        c = self.cfg
        x = rmsnorm(h, L["attn_norm"], c.rms_eps)
        h = h + self._sum_ranks(self._linear_attention(L, x, fb, kv) if "gdn_index" in L else self._attention(L, x, fb, kvl))
        xn = rmsnorm(h, L["ffn_norm"], c.rms_eps)
        y = self._ffn(L, xn)
        if not (c.is_moe and getattr(self.tp, "moe_mode", "expert-parallel") == "replicated"):
            y = self._sum_ranks(y)               # replicated experts: every rank already has the full sum
        if "sh" in L:
            wg, wu, wd, gate = L["sh"]
            y = y + torch.sigmoid(xn @ gate) * ((F.silu(xn @ wg.T) * (xn @ wu.T)) @ wd.T)
        return h + y

    def _logits(self, h_rows, norm_w, out):
        lg = rmsnorm(h_rows, norm_w, self.cfg.rms_eps) @ self.head.T
        if out is not None:
            out[:lg.shape[0]].copy_(lg)
            return out[:lg.shape[0]]
        return lg

    @torch.no_grad()
    def forward(self, fb: ForwardBatch, kv: PagedKVCache, logits_out=None, want_logits=True, kv_layer_offset: int = 0):
        h = fb.embeds.float() if fb.embeds is not None else self.embed[fb.tokens.long()].float()
        for li, L in enumerate(self.layers):
            kvl = kv.layers[kv_layer_offset + L["kv_index"]] if L.get("kv_index") is not None else None
            h = self._layer(L, h, fb, kvl, kv)
            if getattr(self, "taps", None) is not None:       # per-layer hidden states for the parity report
                self.taps[f"layer{li}"] = h.float().clone()
        logits = None
        if want_logits and self.head is not None:
            rows = h if fb.logit_rows is None else h.index_select(0, fb.logit_rows.long())
            logits = self._logits(rows, self.out_norm, logits_out)
        return logits, h

    @torch.no_grad()
    def mtp_forward(self, fb: ForwardBatch, hidden: torch.Tensor, kv: PagedKVCache, depth: int = 0, logits_out=None):
        c = self.cfg
        L = self.mtp_layers[depth]
        e = rmsnorm(self.embed[fb.tokens.long()].float(), L["enorm"], c.rms_eps)
        hn = rmsnorm(hidden.float(), L["hnorm"], c.rms_eps)
        x = torch.cat([e, hn], dim=-1) @ L["eh_proj"].T
        h = self._layer(L, x, fb, kv.layers[self.mtp_kv_base + depth])
        rows = h if fb.logit_rows is None else h.index_select(0, fb.logit_rows.long())
        return self._logits(rows, L["shared_head_norm"], logits_out), h
