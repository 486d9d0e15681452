"""Pipeline parallelism: contiguous layer ranges per stage, each stage a tensor-parallel group.

Every rank runs the same scheduler on the same requests (commands are replicated, `parallel.spmd`), so all
ranks build identical batches and call `forward` in lock step.  A stage's `forward` receives the residual
stream from the stage before it, runs its own layers and sends the result on; the last stage computes the
logits and gathers the vocabulary shards inside its tensor-parallel group.  Every rank runs the same sampler on the
same request state, but only the last stage has real logits: it samples, and the chosen token ids (a few bytes, not
the 19 MB of full-vocabulary rows of a 32-row step) are broadcast to the other stages, which drop what they drew
from their placeholder rows (`sync_sampled`).  Full rows are still broadcast for the steps that need them on every
rank (log-probabilities, speculative verification).  Between stages the residual stream travels as bf16 on GPUs
(`LLAMINAR_PP_PAYLOAD`).  Sends and receives are stream-ordered NCCL point-to-point
operations between ranks with the same tensor-parallel index, so a long prompt that the engine feeds in chunks
of ``microbatch_tokens`` rows pipelines by itself: stage 0 starts chunk i+1 while stage 1 still works on chunk i
(reference: src/v2/execution/pipeline/PipelineStageRunner.cpp, src/v2/execution/runner/OrchestrationRunner.cpp:850-922;
the reference moves activations with MPI or host-staged copies between its stage runners).
"""
from __future__ import annotations

from dataclasses import replace

import torch
import torch.distributed as dist

from ..engine.cuda_model import ForwardBatch


def stage_layer_ranges(n_layers: int, layout: dict) -> list[tuple[int, int]]:
    """[first, stop) per stage; explicit ranges from the layout win, otherwise an even split."""
    pp = layout["pp"]
    out = []
    explicit = all(s[3] is not None and s[3] >= 0 for s in layout["stages"])
    for i, s in enumerate(layout["stages"]):
        if explicit:
            out.append((int(s[2]), int(s[3]) + 1))
        else:
            out.append((n_layers * i // pp, n_layers * (i + 1) // pp))
    if out[0][0] != 0 or out[-1][1] != n_layers or any(out[i][1] != out[i + 1][0] for i in range(pp - 1)):
        raise ValueError(f"pipeline stages must cover layers 0..{n_layers - 1} contiguously, got {out}")
    return out


class PipelineStageModel:
    """Wraps one stage's model so that the engine sees an ordinary model returning full-vocabulary logits."""

    returns_full_vocab = True

    def __init__(self, inner, stage: int, n_stages: int, tp_index: int, tp_size: int, pp_group, tp=None):
        self.inner, self.stage, self.n_stages = inner, stage, n_stages
        self.first, self.last = stage == 0, stage == n_stages - 1
        self.cfg, self.device, self.tp = inner.cfg, inner.device, tp
        self.n_kv_local, self.n_heads_local = inner.n_kv_local, inner.n_heads_local
        self.n_kv_layers = inner.n_kv_layers
        self.hybrid_dims = getattr(inner, "hybrid_dims", None)     # linear-attention state of this stage's layers (or None)
        self.graph_safe = getattr(inner, "graph_safe", True)
        self.vocab_local = inner.cfg.vocab_size
        self.mtp_layers = [object()] * inner.cfg.nextn_layers        # only their count is read outside the last stage
        self.pp_group = pp_group                                       # ranks with this tensor-parallel index, one per stage
        self.prev = (stage - 1) * tp_size + tp_index
        self.next = (stage + 1) * tp_size + tp_index
        self.last_rank = (n_stages - 1) * tp_size + tp_index
        self.scratch = getattr(inner, "scratch", None)
        self.stats = {"sent_bytes": 0, "recv_bytes": 0, "bcast_bytes": 0, "token_syncs": 0}
        d = self.cfg.d_model
        from ..utils.env import debug_env
        mode = str(debug_env().pp_payload).lower()
        if mode not in ("auto", "bf16", "fp32"):
            raise ValueError(f"LLAMINAR_PP_PAYLOAD={mode!r}: expected auto, bf16 or fp32")
        self.payload_dtype = torch.bfloat16 if (mode == "bf16" or (mode == "auto" and self.device.type == "cuda")) else torch.float32
        rows = getattr(inner, "max_tokens", 4096)
        self._recv = torch.empty(rows, d, dtype=torch.float32, device=self.device)
        self._wire = torch.empty(rows, d, dtype=self.payload_dtype, device=self.device) if self.payload_dtype != torch.float32 else None
        # set by the engine before a forward pass whose rows will be sampled: True = only token ids cross the stages
        self.token_sync = False
        self._placeholder = None

    def weight_bytes(self) -> int:
        return self.inner.weight_bytes()

    def _n_rows(self, fb: ForwardBatch) -> int:
        return fb.tokens.shape[0]

    def sync_sampled(self, tokens: list[int]) -> list[int]:
        """The last stage's draw is everybody's: one small broadcast per sampled step."""
        t = torch.tensor(tokens, dtype=torch.int32, device=self.device)
        dist.broadcast(t, src=self.last_rank, group=self.pp_group)
        self.stats["token_syncs"] += 1
        self.stats["bcast_bytes"] += t.numel() * 4
        return t.tolist()

    def _bcast_logits(self, logits, n_rows: int, logits_out):
        V = self.cfg.vocab_size
        if self.token_sync:
            if self.last:
                full = logits if self.tp is None or self.tp.size == 1 else self.tp.all_gather_vocab(logits, V)
                return full.contiguous()
            if self._placeholder is None:
                self._placeholder = torch.zeros(1, V, dtype=torch.float32, device=self.device)
            return self._placeholder.expand(n_rows, V)           # never read for its values: `sync_sampled` replaces the draw
        if self.last:
            full = logits if self.tp is None or self.tp.size == 1 else self.tp.all_gather_vocab(logits, V)
            full = full.contiguous()
            if logits_out is not None and full.data_ptr() != logits_out.data_ptr():
                logits_out[:n_rows].copy_(full)
                full = logits_out[:n_rows]
        else:
            full = logits_out[:n_rows] if logits_out is not None else torch.empty(n_rows, V, dtype=torch.float32, device=self.device)
        dist.broadcast(full, src=self.last_rank, group=self.pp_group)
        self.stats["bcast_bytes"] += full.numel() * 4
        return full

    @torch.no_grad()
    def forward(self, fb: ForwardBatch, kv, logits_out=None, want_logits: bool = True):
        T = self._n_rows(fb)
        if not self.first:
            buf = self._recv[:T]
            if self._wire is None:
                dist.recv(buf, src=self.prev)
            else:
                dist.recv(self._wire[:T], src=self.prev)
                buf.copy_(self._wire[:T])
            self.stats["recv_bytes"] += buf.numel() * self.payload_dtype.itemsize
            fb = replace(fb, embeds=buf)
        # the vocabulary shard of the last stage goes through its own buffer; `logits_out` holds full rows
        logits, h = self.inner.forward(fb, kv, want_logits=want_logits and self.last)
        if not self.last:
            out = h[:T].contiguous() if self._wire is None else h[:T].to(self.payload_dtype)
            dist.send(out, dst=self.next)
            self.stats["sent_bytes"] += out.numel() * self.payload_dtype.itemsize
        if want_logits:
            n_rows = T if fb.logit_rows is None else fb.logit_rows.shape[0]
            logits = self._bcast_logits(logits, n_rows, logits_out)
        return logits, h

    @torch.no_grad()
    def mtp_forward(self, fb: ForwardBatch, hidden, kv, depth: int = 0, logits_out=None):
        """The NextN head lives on the last stage; the other stages only receive its logits."""
        T = self._n_rows(fb)
        n_rows = T if fb.logit_rows is None else fb.logit_rows.shape[0]
        if self.last:
            logits, h = self.inner.mtp_forward(fb, hidden, kv, depth=depth)
        else:
            logits, h = None, torch.zeros(T, self.cfg.d_model, dtype=torch.float32, device=self.device)
        return self._bcast_logits(logits, n_rows, logits_out), h


def build_pipeline_engine(weights, layout: dict, rank: int, microbatch_tokens: int = 1024, **kw):
    """Engine for this rank's stage.  ``kw`` are `LLMEngine` keyword arguments (device, tp, prefix_cache, mtp, ...)."""
    from ..engine.engine import LLMEngine
    cfg = weights.config
    tp_size, pp = layout["tp"], layout["pp"]
    stage, tp_index = rank // tp_size, rank % tp_size
    ranges = stage_layer_ranges(cfg.n_layers, layout)
    device = torch.device(kw.get("device") or "cpu")
    last = stage == pp - 1
    # one group per tensor-parallel index, spanning the stages (every rank must create all of them, in the same order)
    pp_groups = [dist.new_group([s * tp_size + j for s in range(pp)]) for j in range(tp_size)]
    tp = kw.get("tp")
    max_tokens = max(microbatch_tokens, kw.get("max_batch", 32) * 4)
    args = dict(tp=tp, layer_range=ranges[stage], with_head=last, with_embed=(stage == 0) or (last and cfg.nextn_layers > 0),
                with_mtp=last, max_tokens=max_tokens)
    if device.type == "cuda":
        from ..engine.cuda_model import CudaModel
        inner = CudaModel(weights, device, **args)
    else:
        from ..engine.torch_model import TorchPagedModel
        inner = TorchPagedModel(weights, device, **args)
    model = PipelineStageModel(inner, stage, pp, tp_index, tp_size, pp_groups[tp_index], tp=tp)
    kw = dict(kw)
    kw["max_prefill_tokens"] = microbatch_tokens
    kw.setdefault("use_graphs", False)           # point-to-point transfers stay outside CUDA graphs
    kw.setdefault("agree_group", dist.group.WORLD)   # all stages schedule in lock step: one KV page count for everybody
    eng = LLMEngine(weights, model=model, **kw)
    eng.pp_stage, eng.pp_size = stage, pp
    return eng
