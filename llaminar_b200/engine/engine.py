"""Request scheduler + step loop: continuous batching over a paged KV cache.

The reference serves one request at a time through `prefill` / `decodeStep`
(reference: src/v2/execution/runner/OrchestrationRunner.cpp:1028-1297, :10910-11317); here the same
two phases run over up to ``max_batch`` lanes.  Decode steps replay a CUDA graph captured per
batch bucket (inputs live in one static int32 buffer that is refreshed with a single pinned
host-to-device copy per step).  The first generated token is sampled from the prefill logits, as in
the reference (OrchestrationRunner.cpp:1289-1294).
"""
from __future__ import annotations

import itertools
import time
from dataclasses import dataclass, field

import torch

from ..models.config import ModelConfig
from ..models.weights import ModelWeights
from .cuda_model import ForwardBatch
from .kv_cache import HybridState, PAGE_SIZE, OutOfPages, PagedKVCache, SequenceKV
from .kv_cache import Q8 as KV_Q8
from .sampling import SamplingParams, apply_penalties, sample_row
from ..utils.env import debug_env
from ..utils.perfstats import perf_stats

BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128)


@dataclass
class Request:
    rid: int
    prompt: list[int]
    params: SamplingParams
    kv: SequenceKV = field(default_factory=SequenceKV)
    output: list[int] = field(default_factory=list)
    state: str = "waiting"              # waiting -> running -> finished
    finish_reason: str | None = None
    prefix_hit_tokens: int = 0
    t_arrival: float = 0.0
    t_first_token: float | None = None
    forced: list[int] = field(default_factory=list)     # tokens to emit instead of sampling (forceDecodeToken)
    hidden: torch.Tensor | None = None                   # last trunk hidden row (MTP input)
    draft: list[int] = field(default_factory=list)
    step_count: int = 0
    terminal: object = None                               # prefix-cache terminal state: the forward pass is skipped
    logprobs: list = field(default_factory=list)          # one (token, logprob, [(token, logprob), ...]) per output token
    n_folded: int = 0                                     # leading output tokens that a preemption appended to `prompt`
    slot: int = -1                                        # hybrid models: state slot held from admission to the end

    @property
    def all_tokens(self) -> list[int]:
        return self.prompt + self.output[self.n_folded:]

    @property
    def n_tokens(self) -> int:
        return len(self.prompt) + len(self.output) - self.n_folded


@dataclass
class StepOutput:
    rid: int
    new_tokens: list[int]
    finished: bool
    finish_reason: str | None = None
    logprobs: list | None = None        # entries of Request.logprobs for new_tokens, when the request asked for them


class LLMEngine:
    def __init__(self, weights: ModelWeights, device: str | torch.device | None = None, max_batch: int = 32,
                 max_context: int = 4096, kv_pages: int | None = None, max_prefill_tokens: int = 8192,
                 use_graphs: bool = True, prefix_cache=None, mtp=None, tp=None, eos_token_id: int | None = None,
                 model=None, kv_memory_fraction: float = 0.85, kv_dtype: torch.dtype | None = None, agree_group=None):
        self.cfg: ModelConfig = weights.config if weights is not None else model.cfg
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        self.is_cuda = self.device.type == "cuda"
        self.max_batch, self.max_context = max_batch, max_context
        self.max_prefill_tokens = max_prefill_tokens
        self.tp = tp
        self.eos_token_id = eos_token_id
        c = self.cfg
        if model is not None:
            self.model = model
        elif self.is_cuda:
            from .cuda_model import CudaModel
            self.model = CudaModel(weights, self.device, max_tokens=max(max_prefill_tokens, max_batch * 4), tp=tp)
        else:
            from .torch_model import TorchPagedModel
            self.model = TorchPagedModel(weights, self.device, tp=tp)
        if kv_dtype == KV_Q8 and not self.is_cuda:
            raise ValueError("the 8-bit KV cache is a CUDA feature (the CPU back end takes bf16 / fp16 / fp32)")
        self.max_pages_per_seq = (max_context + PAGE_SIZE - 1) // PAGE_SIZE + 1
        # hybrid models: one state slot per lane for the linear-attention layers, allocated before the KV cache is sized so
        # that the page count is taken from what is left
        hybrid = None
        hd = getattr(self.model, "hybrid_dims", None)
        if hd:
            if kv_dtype == KV_Q8:
                raise ValueError("the 8-bit KV cache is not available for hybrid (linear-attention) models: their gated "
                                 "attention blocks append to a bf16 cache")
            hybrid = HybridState(n_slots=max(1, max_batch), device=self.device, **hd)
        n_kv_layers = getattr(self.model, "n_kv_layers", c.n_layers + c.nextn_layers)
        if kv_pages is None:
            need = max_batch * self.max_pages_per_seq + 64
            if self.is_cuda:
                free, _ = torch.cuda.mem_get_info(self.device)
                per_page = max(1, PagedKVCache.bytes_per_page(n_kv_layers, self.model.n_kv_local, c.head_dim, 17 / 16 if kv_dtype == KV_Q8 else 2))
                kv_pages = int(min(need * 2, max(need // 4, int(free * kv_memory_fraction) // per_page)))
            else:
                kv_pages = need
        # Every rank of a multi-process engine runs the same scheduler and must reach the same admission, eviction and
        # preemption decisions, so all of them use the smallest page count any rank could afford (free memory differs
        # between GPUs).  `agree_group`: the ranks that step together (default: the tensor-parallel group).
        self._agree_group = agree_group if agree_group is not None else (tp.group if tp is not None and tp.size > 1 else None)
        kv_pages = self._agree_kv_pages(kv_pages, self._agree_group)
        self.kv = PagedKVCache(n_kv_layers, self.model.n_kv_local, c.head_dim, kv_pages, self.device,
                               dtype=(KV_Q8 if kv_dtype == KV_Q8 else torch.bfloat16) if self.is_cuda else (kv_dtype or torch.float32))
        self.kv.hybrid = hybrid
        self.use_graphs = use_graphs and self.is_cuda and not debug_env().no_cuda_graphs and getattr(self.model, "graph_safe", True)
        self.perf = perf_stats()
        self._graphs: dict = {}
        self.launches_per_graph: dict = {}      # kernels of this package inside each captured decode graph
        self.step_events = None                 # optional list of (start, end) CUDA events, one pair consumed per decode step
        self._rid = itertools.count()
        self.waiting: list[Request] = []
        self.running: list[Request] = []
        self.requests: dict[int, Request] = {}
        self.prefix_cache = prefix_cache
        if prefix_cache is not None:
            prefix_cache.attach(self)
        self.mtp = mtp
        if mtp is not None:
            mtp.attach(self)
            self.model.seq_shard = False            # the NextN head reads the hidden state of every prompt row
        self._dropped: list[StepOutput] = []       # sequences that a decode step had to end because the cache is full
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "prefill_s": 0.0, "decode_s": 0.0, "steps": 0,
                      "prefix_hit_tokens": 0, "graph_replays": 0, "preemptions": 0}
        self._vocab = c.vocab_size
        if self.is_cuda:
            self._init_static_buffers()

    # -- construction helpers ------------------------------------------------------------------
    def _agree_kv_pages(self, kv_pages: int, group) -> int:
        import torch.distributed as dist
        if group is None or not dist.is_initialized() or dist.get_world_size(group) == 1:
            return kv_pages
        dev = self.device if dist.get_backend(group) == "nccl" else "cpu"
        t = torch.tensor([kv_pages, -kv_pages], dtype=torch.int64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
        lo, hi = int(t[0]), -int(t[1])
        self.kv_pages_per_rank = (lo, hi)              # smallest and largest proposal, for the start-up log
        return lo

    def _agree_min(self, value: int) -> int:
        """The smallest `value` over the ranks that step together.  Cache decisions go through it: what a prefix lookup finds
        depends on each rank's own RAM / disk tiers and eviction history, and ranks that reuse different numbers of pages
        build different batches and meet in different collectives (reference: PrefixCacheCoordinator.cpp:61-96)."""
        import torch.distributed as dist
        group = getattr(self, "_agree_group", None)
        if group is None or not dist.is_initialized() or dist.get_world_size(group) == 1:
            return value
        dev = self.device if dist.get_backend(group) == "nccl" else "cpu"
        t = torch.tensor([value], dtype=torch.int64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
        self.stats["agreements"] = self.stats.get("agreements", 0) + 1
        return int(t[0])

    @staticmethod
    def from_gguf(path: str, **kw) -> "LLMEngine":
        dev = kw.get("device") or ("cuda" if torch.cuda.is_available() else "cpu")
        w = ModelWeights.from_gguf(path, device="cpu")
        eng = LLMEngine(w, **kw)
        eng.metadata = w.metadata
        return eng

    # -- static decode buffers ---------------------------------------------------------------------
    def _init_static_buffers(self) -> None:
        B, P = max(self.max_batch, 1), self.max_pages_per_seq
        bmax = next(b for b in BUCKETS if b >= B) if B <= BUCKETS[-1] else B
        self._bmax = bmax
        R = 4                                   # up to 4 rows per sequence (speculative verify)
        n_int = bmax * R * 2 + bmax + bmax * P + bmax * 3 * R + bmax
        self._dec_host = torch.zeros(n_int, dtype=torch.int32).pin_memory()
        self._dec_dev = torch.zeros(n_int, dtype=torch.int32, device=self.device)
        self._fl_host = torch.zeros(bmax * R * 2, dtype=torch.float32).pin_memory()
        self._fl_dev = torch.zeros(bmax * R * 2, dtype=torch.float32, device=self.device)
        self._seed_host = torch.zeros(bmax * R, dtype=torch.int64).pin_memory()
        self._seed_dev = torch.zeros(bmax * R, dtype=torch.int64, device=self.device)
        self._tok_dev = torch.zeros(bmax * R, dtype=torch.int32, device=self.device)
        self._tok_host = torch.zeros(bmax * R, dtype=torch.int32).pin_memory()
        self._logits = torch.empty(bmax * R, self.model.vocab_local, dtype=torch.float32, device=self.device)
        # per-shard argmax candidates (value bits, global index) and their all-gathered copies: greedy sampling over a
        # vocabulary-sharded head exchanges 8 bytes per row instead of the logits
        ws = self.tp.size if self.tp is not None else 1
        self._pairs = torch.zeros(bmax * R, 2, dtype=torch.int32, device=self.device)
        self._pairs_all = torch.zeros(ws, bmax * R, 2, dtype=torch.int32, device=self.device)
        # top-k / top-p sampling over a sharded head: every rank contributes its SAMPLE_CANDIDATES best entries per row
        # (the sampling kernel never looks beyond that many), 8 KB per row and rank instead of the logits
        # presence / frequency penalties inside the captured step: per-lane penalty values and (allocated on first use) a
        # dense table of token counts per lane over this rank's vocabulary shard, advanced on the device after sampling
        self._pen_host = torch.zeros(2 * bmax, dtype=torch.float32).pin_memory()
        self._pen_dev = torch.zeros(2 * bmax, dtype=torch.float32, device=self.device)
        self._pen_counts = None
        self._pen_lanes: list = [None] * bmax          # per lane: (request id, tokens of its history that the table holds)
        self._cand = self._cand_all = None
        if ws > 1 and self.is_cuda:
            kc = min(self.SAMPLE_CANDIDATES, self.model.vocab_local)
            self._cand = torch.zeros(bmax * R, kc, 2, dtype=torch.int32, device=self.device)
            self._cand_all = torch.zeros(ws * bmax * R * kc * 2, dtype=torch.int32, device=self.device)

    def _dec_views(self, bucket: int, R: int):
        """Slices of the static int buffer for a (bucket, rows-per-seq) decode shape."""
        P = self.max_pages_per_seq
        T = bucket * R
        o = 0
        d, h = self._dec_dev, self._dec_host
        def take(n):
            nonlocal o
            s = slice(o, o + n)
            o += n
            return s
        s_tok, s_pos, s_len, s_bt = take(T), take(T), take(bucket), take(bucket * P)
        s_topk, s_step, s_sid = take(T), take(T), take(T)
        s_slot = take(bucket)                           # hybrid models: state slot per lane
        return {"tok": s_tok, "pos": s_pos, "len": s_len, "bt": s_bt, "topk": s_topk, "step": s_step, "sid": s_sid,
                "slot": s_slot, "n": o}

    # -- public API ---------------------------------------------------------------------------------
    def add_request(self, prompt: list[int], params: SamplingParams | None = None) -> Request:
        if not prompt:
            raise ValueError("empty prompt")
        params = params or SamplingParams()
        if len(prompt) + 1 > self.max_context:
            raise ValueError(f"prompt of {len(prompt)} tokens exceeds the context window of {self.max_context}")
        r = Request(next(self._rid), list(prompt), params, t_arrival=time.perf_counter())
        self.requests[r.rid] = r
        self.waiting.append(r)
        return r

    def _status_words(self) -> list[torch.Tensor]:
        """The device status words that kernels set when a bounded wait runs out (split-K scratch, fused TP arena)."""
        words = []
        sc = getattr(self.model, "scratch", None)
        if sc is not None:
            words.append(sc.status)
        symm = getattr(self.tp, "symm", None) if self.tp is not None else None
        if symm is not None:
            words.append(symm.status)
        return words

    def _queue_health(self) -> None:
        """Enqueue the copy of the status words into pinned memory behind the step's kernels; the step's own
        synchronisation then makes them readable at no extra cost (`_finish_health`)."""
        if not self.is_cuda:
            return
        if getattr(self, "_health_host", None) is None:
            self._health_host = torch.zeros(8, dtype=torch.int32).pin_memory()
        words = self._status_words()
        for i, w in enumerate(words):
            self._health_host[i:i + 1].copy_(w[:1], non_blocking=True)
        self._health_host[7:8].copy_(self._group_failed(words), non_blocking=True)
        self._health_queued = True

    def _group_failed(self, words: list[torch.Tensor]) -> torch.Tensor:
        """Device word: 1 if ANY rank of the tensor-parallel group has a status word set after this step (MAX over the group,
        enqueued behind the step's kernels).  A wait that runs out on one rank (its peer stalled) leaves the arrival counters
        of the fused kernels out of step on every rank, so all of them have to see the failure and resynchronise together;
        the rank that caused it may have nothing in its own words."""
        flag = torch.stack([w[0] for w in words]).ne(0).any().to(torch.int32).view(1) if words else torch.zeros(1, dtype=torch.int32, device=self.device)
        tp = self.tp
        if tp is not None and getattr(tp, "size", 1) > 1 and getattr(tp, "symm", None) is not None:
            import torch.distributed as dist
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=tp.group)
        return flag

    def _finish_health(self) -> None:
        """After the step has synchronised: raise if any status word was set.  The scratch is reset first, the failure is
        posted to the heartbeat (so that the other ranks stop too) and the caller fails the running requests."""
        if not self.is_cuda:
            return
        if getattr(self, "_health_queued", False):
            self._health_queued = False
            vals = self._health_host[:len(self._status_words())].tolist()
            group_failed = bool(self._health_host[7])
        else:
            words = self._status_words()
            group_failed = bool(int(self._group_failed(words)[0]))       # every rank calls check_health at the same point
            vals = [int(w[0]) for w in words]
        if not any(vals) and not group_failed:
            return
        symm0 = getattr(self.tp, "symm", None) if self.tp is not None else None
        detail = ""
        if symm0 is not None and int(symm0.status[0]) != 0:
            t, seen, want = (int(v) for v in symm0.status[1:4])
            detail = f"; fused tensor-parallel wait: tile {t & 0xffff}{' (second phase)' if t & 0x10000 else ''} saw count {seen}, wanted {want}"
        sc = getattr(self.model, "scratch", None)
        if sc is not None:
            sc.reset()
        symm = getattr(self.tp, "symm", None) if self.tp is not None else None
        if symm is not None:
            symm.status.zero_()
            if getattr(self.tp, "verify_checksums", False) and hasattr(symm, "check_canaries"):
                symm.check_canaries()
            if group_failed and getattr(self.tp, "size", 1) > 1 and hasattr(symm, "resync"):
                # all ranks of the group are here (the flag was agreed): bring the fused kernels' counters back in step, so that
                # the next step can run instead of timing out again on the counts this step left behind
                symm.resync()
        if not any(vals):
            detail += "; reported by another rank of the tensor-parallel group"
        msg = f"a kernel gave up a bounded wait (status words {vals}{detail}); scratch buffers were reset"
        hb = getattr(self, "heartbeat", None)
        if hb is not None:
            hb.post_error(msg)
        raise RuntimeError(msg)

    def check_health(self) -> None:
        """Raise if a kernel reported a bounded wait that ran out (a peer rank stalled); the scratch is reset first.
        `step()` runs this check itself after every step; it is public for callers that drive `model.forward` directly."""
        if self.is_cuda:
            torch.cuda.current_stream(self.device).synchronize()
        self._finish_health()

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def abort(self, rid: int) -> None:
        r = self.requests.get(rid)
        if r is None or r.state == "finished":
            return
        self._finish(r, "abort")
        if r in self.waiting:
            self.waiting.remove(r)

    def force_token(self, rid: int, token: int) -> None:
        """Make the next decode step of a request emit ``token`` instead of sampling (thinking-budget stop)."""
        self.requests[rid].forced.append(token)

    def clear_cache(self) -> None:
        for r in list(self.running):
            self._finish(r, "abort")
        if self.prefix_cache is not None:
            self.prefix_cache.clear()

    def generate(self, prompts: list[list[int]], params: SamplingParams | list[SamplingParams] | None = None) -> list[list[int]]:
        plist = params if isinstance(params, list) else [params or SamplingParams()] * len(prompts)
        reqs = [self.add_request(p, sp) for p, sp in zip(prompts, plist)]
        while any(r.state != "finished" for r in reqs):
            self.step()
        outs = [r.output for r in reqs]
        for r in reqs:
            self.requests.pop(r.rid, None)
        return outs

    # -- scheduling -----------------------------------------------------------------------------------
    def step(self) -> list[StepOutput]:
        """One scheduler iteration: admit + prefill waiting requests if lanes are free, else one decode step."""
        if not self.perf.enabled:
            outs = self._step()
            self._finish_health()
            return outs
        kind = "prefill" if self.waiting and len(self.running) < self.max_batch else "decode"
        self.perf.set_phase(kind)
        with self.perf.timer("engine", "step", device=str(self.device)), self.perf.cuda_timer("engine", "step_device", device=self.device):
            outs = self._step()
        self._finish_health()
        self.perf.count("engine", "tokens", sum(len(o.new_tokens) for o in outs), device=str(self.device))
        return outs

    def _step(self) -> list[StepOutput]:
        self.stats["steps"] += 1
        if self.waiting and len(self.running) < self.max_batch:
            batch, budget = [], self.max_prefill_tokens
            while self.waiting and len(self.running) + len(batch) < self.max_batch:
                r = self.waiting[0]
                cost = len(r.prompt)
                if batch and cost > budget:
                    break
                if self.kv.hybrid is not None:
                    r.slot = self.kv.hybrid.alloc()            # at most max_batch sequences are admitted: a slot is free
                try:
                    self._admit(r, len(batch))
                except OutOfPages:
                    self._release_slot(r)
                    if not batch and not self.running:
                        # the whole cache is free and the prompt still does not fit: this request can never run.  It
                        # ends with finish reason "cache_full" (the server answers 400); the queue behind it goes on.
                        self.waiting.pop(0)
                        self._finish(r, "cache_full")
                        return [StepOutput(r.rid, [], True, "cache_full", [] if r.params.wants_logprobs else None)]
                    break
                self.waiting.pop(0)
                batch.append(r)
                budget -= cost
            if batch:
                return self._prefill(batch)
        if self.running:
            self._dropped = []
            outs = self.mtp.decode_step(self, list(self.running)) if self.mtp is not None else self._decode(list(self.running))
            return outs + self._dropped
        return []

    def _admit(self, r: Request, pending: int = 0) -> None:
        """Pages for the prompt (shared with the prefix cache where it hits).  ``pending``: sequences admitted earlier in
        the same scheduler step, which count as running for the watermark."""
        if r.n_folded and self.running:
            # a preempted sequence comes back only when it fits with room to grow beside the running ones: re-admitting
            # it into a full cache would recompute its whole prefix just to be preempted again
            need = (r.n_tokens + PAGE_SIZE) // PAGE_SIZE + len(self.running) + 1
            if self._available_pages() < need:
                raise OutOfPages("waiting for pages after a preemption")
        hit_pages, hit_tokens = [], 0
        hybrid = self.cfg.is_hybrid                          # a model property: every rank takes the same branches below
        if self.prefix_cache is not None:
            term = None if hybrid else self.prefix_cache.lookup_terminal(r.prompt)
            if not self._agree_min(1 if term is not None else 0):
                term = None                                   # some rank does not have it: nobody uses it
            if term is not None:
                try:
                    if self.prefix_cache.restore_terminal(self, r, term):
                        r.terminal, r.prefix_hit_tokens = term, len(r.prompt)
                        self._ensure_pages(r, len(r.prompt) + 1)
                        self.stats["prefix_hit_tokens"] += len(r.prompt)
                        return
                except OutOfPages:
                    self.kv.free_sequence(r.kv)
                    r.kv = SequenceKV()
            held, hit_tokens = self.prefix_cache.lookup(r.prompt)      # `held`: one reference per page, dropped below
            agreed = self._agree_min(hit_tokens)                       # every rank reuses the same number of pages
            if hybrid:
                # a linear-attention state can only be resumed where a snapshot of it is held: cut the hit back to the
                # longest such boundary that leaves a token to run, the same one on every rank
                limit = min(agreed, len(r.prompt) - 1) // PAGE_SIZE * PAGE_SIZE
                local = self.kv.hybrid is not None           # a pipeline stage may hold softmax blocks only
                b = self._agree_min(self.prefix_cache.state_boundary(r.prompt, limit) if local else limit)
                have = b == 0 or not local or self.prefix_cache.state_at(r.prompt, b) is not None
                agreed = b if self._agree_min(1 if have else 0) else 0
                if agreed and local:
                    self.kv.hybrid.restore(r.slot, self.prefix_cache.state_at(r.prompt, agreed))
            hit_pages = list(held)[:agreed // PAGE_SIZE]
            hit_tokens = len(hit_pages) * PAGE_SIZE if agreed < hit_tokens else hit_tokens
        else:
            held = []
        try:
            if hit_tokens >= len(r.prompt):               # keep at least one token to run for the logits
                drop = (hit_tokens - len(r.prompt)) // PAGE_SIZE + 1
                hit_pages = hit_pages[:len(hit_pages) - drop]
                hit_tokens = len(hit_pages) * PAGE_SIZE
            r.kv = self.kv.fork_prefix(hit_pages, hit_tokens) if hit_pages else SequenceKV()
        finally:
            if held:
                self.prefix_cache.release_pages(held)
        r.prefix_hit_tokens = hit_tokens
        try:
            self._ensure_pages(r, len(r.prompt) + 1)
            others = len(self.running) + pending
            if others and self._available_pages() < others + 1:
                # admission watermark: every running sequence must still be able to take its next page, otherwise the
                # newcomer's prefill would be thrown away by a preemption a few steps later
                raise OutOfPages("admission would leave the running sequences no room to grow")
        except OutOfPages:
            self.kv.free_sequence(r.kv)
            r.kv = SequenceKV()
            r.prefix_hit_tokens = 0
            raise
        self.stats["prefix_hit_tokens"] += hit_tokens

    def _available_pages(self) -> int:
        """Free pages plus the pages that the prefix cache would give back on demand."""
        n = self.kv.allocator.n_free
        if self.prefix_cache is not None:
            n += self.prefix_cache.evictable_pages()
        return n

    def _ensure_pages(self, r: Request, n_tokens: int) -> None:
        try:
            self.kv.ensure_capacity(r.kv, n_tokens)
        except OutOfPages:
            if self.prefix_cache is None or not self.prefix_cache.evict_for(self, n_tokens - r.kv.capacity()):
                raise
            self.kv.ensure_capacity(r.kv, n_tokens)

    def _release_slot(self, r: Request) -> None:
        if r.slot >= 0:
            self.kv.hybrid.release(r.slot)
            r.slot = -1

    def _finish(self, r: Request, reason: str) -> None:
        if r.state == "finished":
            return
        if self.prefix_cache is not None and reason != "abort":
            self.prefix_cache.insert(self, r)
        r.state, r.finish_reason = "finished", reason
        if r in self.running:
            self.running.remove(r)
        self.kv.free_sequence(r.kv)
        self._release_slot(r)
        if self.prefix_cache is not None:
            self.prefix_cache.trim()                  # pages the request pinned can now leave the device tier
        if self.mtp is not None:
            self.mtp.release(r)

    def _check_stop(self, r: Request, tok: int) -> str | None:
        p = r.params
        if tok in p.stop_token_ids:
            return "stop"
        if not p.ignore_eos and self.eos_token_id is not None and tok == self.eos_token_id:
            return "stop"
        if len(r.output) >= p.max_tokens:
            return "length"
        if r.n_tokens + 1 >= self.max_context:
            return "length"
        return None

    def _emit(self, r: Request, toks: list[int]) -> StepOutput:
        new = []
        for t in toks:
            r.output.append(t)
            new.append(t)
            if r.t_first_token is None:
                r.t_first_token = time.perf_counter()
            reason = self._check_stop(r, t)
            if reason:
                self._finish(r, reason)
                return StepOutput(r.rid, new, True, reason, self._new_logprobs(r, len(new)))
        return StepOutput(r.rid, new, False, None, self._new_logprobs(r, len(new)))

    @staticmethod
    def _new_logprobs(r: Request, n: int) -> list | None:
        if not r.params.wants_logprobs:
            return None
        return r.logprobs[len(r.logprobs) - n:] if n else []

    @staticmethod
    def _record_logprobs(logits: torch.Tensor, reqs: list[Request], toks: list[int]) -> None:
        """Log-probabilities of the model's own distribution (full-vocabulary rows, before penalties, temperature and
        truncation) for the requests that asked: the emitted token and the k likeliest ones."""
        rows = [i for i, r in enumerate(reqs) if r.params.wants_logprobs]
        if not rows:
            return
        lp = torch.log_softmax(logits[rows].float(), dim=-1)
        k = max(reqs[i].params.logprobs for i in rows)
        chosen = lp.gather(1, torch.tensor([[toks[i]] for i in rows], device=lp.device)).view(-1).tolist()
        top_v, top_i = (lp.topk(k, dim=-1) if k else (lp[:, :0], lp[:, :0].long()))
        top_v, top_i = top_v.tolist(), top_i.tolist()
        for j, i in enumerate(rows):
            kk = reqs[i].params.logprobs
            reqs[i].logprobs.append((int(toks[i]), float(chosen[j]), list(zip(top_i[j][:kk], top_v[j][:kk]))))

    # -- sampling -----------------------------------------------------------------------------------
    def _sample_rows(self, logits: torch.Tensor, reqs: list[Request]) -> list[int]:
        """Eager sampling of one row per request (prefill tail, penalties, CPU backend)."""
        all_greedy = all(r.params.is_greedy and not r.params.needs_penalties and not r.forced for r in reqs)
        want_lp = any(r.params.wants_logprobs for r in reqs)
        if all_greedy and not want_lp and self._sharded_vocab() and logits.shape[0] <= self._pairs.shape[0]:
            tok = torch.empty(len(reqs), dtype=torch.int32, device=self.device)
            self._sharded_argmax(logits.contiguous(), len(reqs), tok)
            return tok.tolist()
        logits = self._gather_vocab(logits)
        out = self._sample_full_rows(logits, reqs, all_greedy)
        if getattr(self.model, "token_sync", False):
            out = self.model.sync_sampled(out)            # pipeline stages: the last stage's draw is everybody's
        if want_lp:
            self._record_logprobs(logits, reqs, out)
        return out

    def _sample_full_rows(self, logits: torch.Tensor, reqs: list[Request], all_greedy: bool) -> list[int]:
        out = []
        if all_greedy:
            if self.is_cuda:
                from .. import ops
                tok = torch.empty(len(reqs), dtype=torch.int32, device=self.device)
                ops.argmax(logits.contiguous(), tok)
                return tok.tolist()
            return logits.argmax(-1).tolist()
        for i, r in enumerate(reqs):
            if r.forced:
                out.append(r.forced.pop(0))
                continue
            row = apply_penalties(logits[i], r.all_tokens, r.params)
            if self.is_cuda and not r.params.is_greedy:
                from .. import ops
                dev = self.device
                seed = r.params.seed if r.params.seed is not None else (r.rid * 7919 + 17)
                tok = torch.empty(1, dtype=torch.int32, device=dev)
                ops.sample(row.view(1, -1).contiguous(), torch.tensor([r.params.temperature], device=dev),
                           torch.tensor([r.params.top_k], dtype=torch.int32, device=dev),
                           torch.tensor([r.params.top_p], device=dev), torch.tensor([seed], dtype=torch.int64, device=dev),
                           torch.tensor([len(r.output)], dtype=torch.int32, device=dev), tok)
                out.append(int(tok))
            else:
                # never the global generator: every rank of a multi-process engine must draw the same token
                seed = r.params.seed if r.params.seed is not None else (r.rid * 7919 + 17)
                gen = torch.Generator().manual_seed(seed * 1000003 + len(r.output))
                out.append(sample_row(row, r.params, gen))
        return out

    def _sharded_vocab(self) -> bool:
        return self.is_cuda and self.tp is not None and self.tp.size > 1 and not getattr(self.model, "returns_full_vocab", False)

    def _sharded_argmax(self, logits: torch.Tensor, rows: int, tokens: torch.Tensor) -> None:
        """Greedy token over a vocabulary-sharded head: per-shard argmax, all-gather of (value, index), merge."""
        from .. import ops
        ws = self.tp.size
        pairs = self._pairs[:rows]
        ops.argmax(logits, None, pairs=pairs, idx_offset=self.model.plan.vocab_start)
        gathered = self._pairs_all.view(-1)[:ws * rows * 2].view(ws, rows, 2)
        self.tp.all_gather_flat(gathered, pairs)
        ops.argmax_merge(gathered, ws, rows, tokens)

    SAMPLE_CANDIDATES = 1024      # the sampling kernel's candidate cap (top_k = 0 means "the best 1024")

    def _sharded_sample(self, logits: torch.Tensor, rows: int, temperature, top_k, top_p, seeds, step, tokens) -> None:
        """Top-k / top-p sampling over a vocabulary-sharded head: per-shard candidates, all-gather, one merged draw.
        Every rank draws the same token, and it is the token a single rank would draw from the gathered logits
        (reference: DeviceSampler's per-shard candidate merge, src/v2/execution/local_execution/orchestrators/DeviceSampler.cpp)."""
        from .. import ops
        ws = self.tp.size
        cand = self._cand[:rows]
        kc = cand.shape[1]
        ops.sample_candidates(logits, self.model.plan.vocab_start, cand)
        gathered = self._cand_all[:ws * rows * kc * 2].view(ws, rows, kc, 2)
        self.tp.all_gather_flat(gathered, cand)
        ops.sample_merged(gathered, temperature, top_k, top_p, seeds, step, tokens)

    def _gather_vocab(self, logits: torch.Tensor) -> torch.Tensor:
        """Vocab-parallel logits shards -> full rows (a no-op without tensor parallelism)."""
        if self.tp is None or self.tp.size == 1 or getattr(self.model, "returns_full_vocab", False):
            return logits
        return self.tp.all_gather_vocab(logits, self.cfg.vocab_size)

    # -- prefill ---------------------------------------------------------------------------------------
    def _set_token_sync(self, reqs: list[Request]) -> None:
        """Pipeline stages: whether only the sampled ids cross the stages in this pass (not with speculative decoding, which
        verifies full rows on every rank, nor when a request wants log-probabilities from the rows)."""
        if hasattr(self.model, "sync_sampled"):
            self.model.token_sync = self.mtp is None and not any(r.params.wants_logprobs for r in reqs)

    def _prefill(self, batch: list[Request]) -> list[StepOutput]:
        t0 = time.perf_counter()
        dev = self.device
        self._set_token_sync(batch)
        # split long prompts into chunks of at most max_prefill_tokens rows per forward
        pending = {r.rid: r.prefix_hit_tokens for r in batch}
        final_logits: dict[int, torch.Tensor] = {}
        final_hidden: dict[int, torch.Tensor] = {}
        for r in batch:
            if r.terminal is not None:            # exact repeat of a cached prompt: logits and hidden row come from the cache
                final_logits[r.rid], final_hidden[r.rid] = r.terminal.logits, r.terminal.hidden
        # hybrid models with a prefix cache: one snapshot of the linear-attention state per prompt, at the last block boundary
        # that leaves a token to run (where a follow-up prompt that extends this one can resume)
        snap_at: dict[int, list[int]] = {}
        if self.prefix_cache is not None and self.kv.hybrid is not None:
            snap_at = {r.rid: self.prefix_cache.snapshot_points(len(r.prompt), pending[r.rid]) for r in batch}
        while any(pending[r.rid] < len(r.prompt) for r in batch):
            toks, pos, sid, cu, ctx, rows_for, chunks = [], [], [], [0], [], [], []
            budget = self.max_prefill_tokens
            btab_rows = []
            for r in batch:
                done = pending[r.rid]
                if done >= len(r.prompt) or budget <= 0:
                    continue
                n = min(len(r.prompt) - done, budget)
                nxt = next((b for b in snap_at.get(r.rid, ()) if b > done), None)
                if nxt is not None:                          # a chunk ends where the prefix cache wants the recurrent state
                    n = min(n, nxt - done)
                budget -= n
                b = len(ctx)
                toks.extend(r.prompt[done:done + n])
                pos.extend(range(done, done + n))
                sid.extend([b] * n)
                cu.append(cu[-1] + n)
                ctx.append(done)
                btab_rows.append(r.kv.pages)
                pending[r.rid] = done + n
                chunks.append((r, done, n))
                rows_for.append((r, cu[-1] - 1 if done + n == len(r.prompt) else None))
            P = max(len(p) for p in btab_rows)
            bt = torch.zeros(len(btab_rows), P, dtype=torch.int32)
            for i, p in enumerate(btab_rows):
                bt[i, :len(p)] = torch.tensor(p, dtype=torch.int32)
            it = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
            logit_rows = [row for _, row in rows_for if row is not None]
            fb = ForwardBatch(tokens=it(toks), positions=it(pos), seq_ids=it(sid), block_table=bt.to(dev), cu_q=it(cu),
                              ctx_lens=it(ctx), max_q_len=max(cu[i + 1] - cu[i] for i in range(len(ctx))),
                              max_kv_len=max(ctx[i] + cu[i + 1] - cu[i] for i in range(len(ctx))),
                              logit_rows=it(logit_rows) if logit_rows else None,
                              state_slots=it([r.slot for r, _, _ in chunks]) if self.kv.hybrid is not None else None)
            logits, h = self.model.forward(fb, self.kv, want_logits=bool(logit_rows))
            for r, done, n in chunks:
                if done + n in snap_at.get(r.rid, ()):
                    self.prefix_cache.store_state(r.prompt[:done + n], self.kv.hybrid.snapshot(r.slot))
            if self.mtp is not None:
                keep = {r.rid: h[row].clone() for r, row in rows_for if row is not None}
                self.mtp.on_prefill_chunk(self, fb, h, chunks)
            j = 0
            for r, row in rows_for:
                if row is not None:
                    final_logits[r.rid] = logits[j]
                    final_hidden[r.rid] = keep[r.rid] if self.mtp is not None else h[row].clone()
                    j += 1
            self.stats["prefill_tokens"] += len(toks)
        outs = []
        lg = torch.stack([final_logits[r.rid] for r in batch])
        toks = self._sample_rows(lg, batch)
        for r, t in zip(batch, toks):
            r.kv.length = len(r.prompt)
            r.hidden = final_hidden[r.rid]
            r.state = "running"
            self.running.append(r)
            if self.prefix_cache is not None:
                self.prefix_cache.insert(self, r)
                if r.terminal is None and not self.cfg.is_hybrid:
                    self.prefix_cache.store_terminal(self, r, final_logits[r.rid], final_hidden[r.rid])
            if self.mtp is not None:
                self.mtp.on_prefill_done(self, r, t, final_hidden[r.rid])
            outs.append(self._emit(r, [t]))
        if self.is_cuda:
            torch.cuda.synchronize(dev)
        self.stats["prefill_s"] += time.perf_counter() - t0
        return outs

    # -- decode ----------------------------------------------------------------------------------------
    def _decode(self, reqs: list[Request]) -> list[StepOutput]:
        t0 = time.perf_counter()
        reqs = self._reserve_decode_pages(reqs)
        if not reqs:
            return []
        # presence / frequency penalties run inside the graph (device-side count table); DRY, forced tokens and logprobs
        # need the host and take the eager path
        eager = (not self.use_graphs) or any(r.params.dry_multiplier > 0.0 or r.forced or r.params.wants_logprobs for r in reqs)
        if self.is_cuda:
            toks = self._decode_cuda(reqs, eager)
        else:
            toks = self._decode_eager(reqs)
        outs = []
        for r, t in zip(reqs, toks):
            r.kv.length = r.n_tokens          # the fed token's K/V are now cached
            r.step_count += 1
            outs.append(self._emit(r, [t]))
        self.stats["decode_tokens"] += len(reqs)
        self.stats["decode_s"] += time.perf_counter() - t0
        return outs

    def _reserve_decode_pages(self, reqs: list[Request], extra: int = 0) -> list[Request]:
        """Gives every running sequence the pages its next token (plus ``extra`` speculative rows) needs.  When the cache
        is exhausted (and the prefix cache has nothing left to evict) the most recently admitted sequences are preempted
        until the others fit; a single sequence that does not fit is ended with finish reason "length"."""
        live = list(reqs)
        i = 0
        while i < len(live):
            try:
                self._ensure_pages(live[i], live[i].n_tokens + extra)
                i += 1
            except OutOfPages:
                if len(live) == 1:
                    # nobody left to preempt: the cache cannot hold this one sequence any further.  It ends here with
                    # what it has produced (finish reason "length") instead of failing the step for every request.
                    r = live.pop()
                    self._finish(r, "length")
                    self._dropped.append(StepOutput(r.rid, [], True, "length", [] if r.params.wants_logprobs else None))
                else:
                    self._preempt(live.pop())
        return live

    def _preempt(self, r: Request) -> None:
        """Recompute preemption: the sequence gives its pages back and returns to the head of the waiting queue with
        its generated tokens appended to the prompt; the next prefill rebuilds the cache and samples the next token
        with the same step index a decode step would have used, so the output continues where it stopped."""
        self.running.remove(r)
        if self.prefix_cache is not None:
            self.prefix_cache.insert(self, r)          # its full pages stay reusable until someone needs the space
        self.kv.free_sequence(r.kv)
        self._release_slot(r)                          # the next prefill starts from position 0 and so from a zero state
        if self.mtp is not None:
            self.mtp.release(r)
        r.kv = SequenceKV()
        r.draft = []
        r.prompt = r.prompt + r.output[r.n_folded:]
        r.n_folded = len(r.output)
        r.state, r.hidden, r.terminal, r.prefix_hit_tokens = "waiting", None, None, 0
        self.waiting.insert(0, r)
        self.stats["preemptions"] += 1

    def _decode_batch_tensors(self, reqs: list[Request]):
        dev = self.device
        B = len(reqs)
        it = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
        P = max(len(r.kv.pages) for r in reqs)
        bt = torch.zeros(B, P, dtype=torch.int32)
        for i, r in enumerate(reqs):
            bt[i, :len(r.kv.pages)] = torch.tensor(r.kv.pages, dtype=torch.int32)
        return ForwardBatch(tokens=it([r.output[-1] for r in reqs]), positions=it([r.n_tokens - 1 for r in reqs]),
                            seq_ids=it(list(range(B))), block_table=bt.to(dev), seq_lens=it([r.n_tokens for r in reqs]),
                            rows_per_seq=1, n_splits=self._splits_for(B),
                            state_slots=it([r.slot for r in reqs]) if self.kv.hybrid is not None else None)

    def _splits_for(self, bucket: int) -> int:
        if not self.is_cuda:
            return 1
        s = max(1, min(16, 296 // max(1, bucket * self.model.n_kv_local)))
        return min(s, max(1, self.max_pages_per_seq // 2))

    def _decode_eager(self, reqs: list[Request]) -> list[int]:
        self._set_token_sync(reqs)
        fb = self._decode_batch_tensors(reqs)
        evp = self.step_events.pop() if self.step_events else None
        if evp:
            evp[0].record()
        logits, h = self.model.forward(fb, self.kv)
        if evp:
            evp[1].record()
        for i, r in enumerate(reqs):
            r.hidden = h[i].clone()
        return self._sample_rows(logits, reqs)

    def _fill_decode_host(self, reqs: list[Request], bucket: int, v: dict) -> None:
        """Writes the step's inputs into the pinned staging buffer (numpy views; one slice assignment per field).  Lanes
        keep their contents between steps: while the set of running requests is unchanged only the token, position and
        length of every lane, and the page-table rows that grew, are rewritten."""
        import numpy as np
        if getattr(self, "_np_dec", None) is None:
            self._np_dec = self._dec_host.numpy()
            self._np_fl = self._fl_host.numpy()
            self._np_seed = self._seed_host.numpy()
            self._lane_sig = None
        h = self._np_dec
        P = self.max_pages_per_seq
        B = len(reqs)
        tok, pos, ln = h[v["tok"]], h[v["pos"]], h[v["len"]]
        bt = h[v["bt"]].reshape(bucket, P)
        n_tok = np.fromiter((r.n_tokens for r in reqs), dtype=np.int32, count=B)
        tok[:B] = np.fromiter((r.output[-1] for r in reqs), dtype=np.int32, count=B)
        pos[:B] = n_tok - 1
        ln[:B] = n_tok
        h[v["step"]][:B] = np.fromiter((len(r.output) for r in reqs), dtype=np.int32, count=B)
        if self.kv.hybrid is not None:                  # padded lanes work on the scratch slot
            sl = h[v["slot"]]
            sl[:B] = np.fromiter((r.slot for r in reqs), dtype=np.int32, count=B)
            sl[B:bucket] = self.kv.hybrid.scratch_slot
        sig = (bucket, tuple(r.rid for r in reqs))
        if sig != self._lane_sig:
            self._lane_sig = sig
            self._lane_pages = [0] * B
            h[v["sid"]] = np.arange(bucket, dtype=np.int32)        # a decode batch uses block-table rows 0..bucket-1
            h[v["topk"]][:B] = np.fromiter((r.params.top_k for r in reqs), dtype=np.int32, count=B)
            temp, topp = self._np_fl[:bucket], self._np_fl[bucket:2 * bucket]
            temp[:B] = [0.0 if r.params.is_greedy else r.params.temperature for r in reqs]
            topp[:B] = [r.params.top_p for r in reqs]
            self._np_seed[:B] = [r.params.seed if r.params.seed is not None else (r.rid * 7919 + 17) for r in reqs]
            if B < bucket:                              # padded lanes point at the scratch page
                tok[B:bucket] = 0
                pos[B:bucket] = 0
                ln[B:bucket] = 1
                bt[B:bucket] = 0
                temp[B:bucket] = 0.0
        for i, r in enumerate(reqs):
            npg = len(r.kv.pages)
            if npg != self._lane_pages[i]:
                bt[i, :npg] = r.kv.pages
                self._lane_pages[i] = npg

    def _decode_cuda(self, reqs: list[Request], eager: bool) -> list[int]:
        from .. import ops
        B = len(reqs)
        bucket = next((b for b in BUCKETS if b >= B), B)
        if eager or bucket > self._bmax:
            return self._decode_eager(reqs)
        v = self._dec_views(bucket, 1)
        self._fill_decode_host(reqs, bucket, v)
        greedy = all(r.params.is_greedy for r in reqs)
        pen = any(r.params.presence_penalty != 0.0 or r.params.frequency_penalty != 0.0 for r in reqs)
        n = v["n"]
        self._dec_dev[:n].copy_(self._dec_host[:n], non_blocking=True)
        if not greedy:
            self._fl_dev[:2 * bucket].copy_(self._fl_host[:2 * bucket], non_blocking=True)
            self._seed_dev[:bucket].copy_(self._seed_host[:bucket], non_blocking=True)
        key = (bucket, greedy, pen)
        g = self._graphs.get(key)
        if g is None:
            if pen and self._pen_counts is None:
                self._pen_counts = torch.zeros(self._bmax, self._vocab_window()[1], dtype=torch.int16, device=self.device)
            g = self._capture_decode(bucket, greedy, v, pen)     # its warm-up runs dirty the count table: synced below
            self._graphs[key] = g
        if pen:
            self._sync_penalty_tables(reqs, bucket)
            for i, r in enumerate(reqs):              # the graph counts the token it samples
                self._pen_lanes[i] = (r.rid, r.n_tokens + 1)
        evp = self.step_events.pop() if self.step_events else None
        if evp:
            evp[0].record()
        g.replay()
        if evp:
            evp[1].record()
        self.stats["graph_replays"] += 1
        self._tok_host[:bucket].copy_(self._tok_dev[:bucket], non_blocking=True)
        self._queue_health()
        torch.cuda.current_stream(self.device).synchronize()
        return self._tok_host[:B].tolist()

    def _vocab_window(self) -> tuple[int, int]:
        """[first token id, number of ids) of the logits rows this rank samples from."""
        if self._sharded_vocab():
            return self.model.plan.vocab_start, self.model.vocab_local
        return 0, self._logits.shape[1]

    def _sync_penalty_tables(self, reqs: list[Request], bucket: int) -> None:
        """Bring the device-side count table in line with the lanes of this step.  A lane whose request changed, or whose
        request took steps outside the graph since the table last saw it, is rebuilt from the request's tokens (one row
        memset plus a small scatter); otherwise the table is already current, the previous graph replay has counted the
        token it sampled."""
        import numpy as np
        v0, V = self._vocab_window()
        if self._pen_counts is None:
            self._pen_counts = torch.zeros(self._bmax, V, dtype=torch.int16, device=self.device)
        ph, B = self._pen_host.numpy(), len(reqs)
        ph[:bucket] = 0.0
        ph[self._bmax:self._bmax + bucket] = 0.0
        for i, r in enumerate(reqs):
            ph[i], ph[self._bmax + i] = r.params.presence_penalty, r.params.frequency_penalty
            if self._pen_lanes[i] != (r.rid, r.n_tokens):
                toks = np.asarray(r.all_tokens, dtype=np.int64) - v0
                u, c = np.unique(toks[(toks >= 0) & (toks < V)], return_counts=True)
                row = self._pen_counts[i]
                row.zero_()
                if len(u):
                    row.index_copy_(0, torch.from_numpy(u).to(self.device),
                                    torch.from_numpy(np.minimum(c, 32767).astype(np.int16)).to(self.device))
        for i in range(B, bucket):
            self._pen_lanes[i] = None
        self._pen_dev.copy_(self._pen_host, non_blocking=True)

    def _decode_body(self, bucket: int, greedy: bool, v: dict, pen: bool = False) -> None:
        from .. import ops
        d = self._dec_dev
        P = self.max_pages_per_seq
        fb = ForwardBatch(tokens=d[v["tok"]], positions=d[v["pos"]], seq_ids=d[v["sid"]],
                          block_table=d[v["bt"]].view(bucket, P), seq_lens=d[v["len"]], rows_per_seq=1,
                          n_splits=self._splits_for(bucket),
                          state_slots=d[v["slot"]] if self.kv.hybrid is not None else None)
        logits, _ = self.model.forward(fb, self.kv, logits_out=self._logits[:bucket])
        tok = self._tok_dev[:bucket]
        if pen:
            ops.penalties_dense(logits, self._pen_counts[:bucket], self._pen_dev[:bucket], self._pen_dev[self._bmax:self._bmax + bucket])
        if greedy and self._sharded_vocab():
            self._sharded_argmax(logits, bucket, tok)
        elif not greedy and self._sharded_vocab() and self._cand is not None:
            self._sharded_sample(logits, bucket, self._fl_dev[:bucket], d[v["topk"]], self._fl_dev[bucket:2 * bucket],
                                 self._seed_dev[:bucket], d[v["step"]], tok)
        else:
            logits = self._gather_vocab(logits)
            if greedy:
                ops.argmax(logits, tok)
            else:
                ops.sample(logits, self._fl_dev[:bucket], d[v["topk"]], self._fl_dev[bucket:2 * bucket],
                           self._seed_dev[:bucket], d[v["step"]], tok)
        if pen:
            v0, V = self._vocab_window()
            ops.count_tokens(self._pen_counts[:bucket], tok, v0, V)

    def _capture_decode(self, bucket: int, greedy: bool, v: dict, pen: bool = False):
        torch.cuda.synchronize(self.device)
        if self.kv.hybrid is not None:
            # the warm-up runs are real steps, and a recurrent state (unlike a K/V row) is not the same after being advanced
            # twice with one token: they work on the scratch slot, the lanes' own slots come back with the staged inputs
            self._dec_dev[v["slot"]].fill_(self.kv.hybrid.scratch_slot)
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):                          # warm-up: lazy initialisation must not happen in capture
                self._decode_body(bucket, greedy, v, pen)
            if pen:                                     # the warm-up runs counted tokens: every lane's table is rebuilt below
                self._pen_lanes = [None] * self._bmax
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        from .. import ops
        n0 = ops.launch_count()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._decode_body(bucket, greedy, v, pen)
        self.launches_per_graph[(bucket, greedy, pen) if pen else (bucket, greedy)] = ops.launch_count() - n0
        if self.kv.hybrid is not None:
            self._dec_dev[:v["n"]].copy_(self._dec_host[:v["n"]], non_blocking=True)
        return g
