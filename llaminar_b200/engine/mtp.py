"""Multi-token prediction (NextN head) speculative decoding.

Each decode step drafts up to three tokens with the model's NextN layer, verifies them with ONE trunk forward
over ``draft + 1`` rows per sequence and emits the accepted prefix plus the trunk's own next token
(reference: src/v2/execution/runner/OrchestrationRunner.cpp:2244-2253 for the verify step,
src/v2/execution/mtp/MTPDepthController.h for the depth policy, src/v2/execution/mtp/MTPSpecVerifier.h for
the rejection sampler).  The whole running batch is drafted and verified together.

Bookkeeping per request.  With tokens t_0..t_{n-1} known, the trunk has cached K/V for positions 0..n-2 and
``hidden[p]`` is the trunk's final residual row at position p.  The NextN layer at position p consumes
(embedding of t_{p+1}, hidden[p]) and predicts t_{p+2}; it has its own K/V layer in the paged cache, so it must
visit every position once with exact inputs.  Rows it has not seen yet are queued in ``catch``; the first draft
call of a step processes the queue (variable rows per sequence, prefill-style attention) and its last row's
logits give draft 1.  Further drafts chain the layer on its own hidden output; the K/V written by those
approximate rows is overwritten when the exact rows arrive through the queue.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field

import torch

from .cuda_model import ForwardBatch
from .kv_cache import PAGE_SIZE


@dataclass
class MTPConfig:
    draft_tokens: int = 1
    verify_mode: str = "greedy"            # greedy | speculative-sampling
    depth_policy: str = "fixed"            # fixed | observe | dynamic
    depth_window: int = 16
    depth_min_samples: int = 4
    depth_cooldown: int = 8
    depth_promote_windows: int = 3
    demote_zero_accept: float = 0.30
    demote_acceptance: float = 0.55
    force_accept: bool = False

    @staticmethod
    def from_values(v: dict) -> "MTPConfig":
        return MTPConfig(int(v.get("mtp_draft_tokens") or 1), v.get("mtp_verify_mode", "greedy"),
                         v.get("mtp_depth_policy", "fixed"), int(v.get("mtp_depth_window", 16)),
                         int(v.get("mtp_depth_min_samples", 4)), int(v.get("mtp_depth_cooldown", 8)),
                         int(v.get("mtp_depth_promote_windows", 3)), float(v.get("mtp_depth_demote_zero_accept", 0.30)),
                         float(v.get("mtp_depth_demote_acceptance", 0.55)), bool(v.get("mtp_force_accept")))


class DepthController:
    """Sliding-window draft-depth policy: demote when drafts mostly miss, promote after sustained full accepts."""

    def __init__(self, cfg: MTPConfig):
        self.cfg = cfg
        self.max_depth = cfg.draft_tokens
        self.depth = cfg.draft_tokens
        self.window: deque = deque(maxlen=cfg.depth_window)      # (accepted, drafted) per sequence-step
        self.cooldown = 0
        self.good_windows = 0
        self.history: list[tuple[int, int]] = []                   # (step, new depth)
        self.steps = 0

    def observe(self, accepted: int, drafted: int) -> None:
        if drafted > 0:
            self.window.append((accepted, drafted))

    def end_step(self) -> int:
        self.steps += 1
        c = self.cfg
        if c.depth_policy != "dynamic" or len(self.window) < max(c.depth_min_samples, 1):
            return self.depth
        if self.cooldown > 0:
            self.cooldown -= 1
            return self.depth
        zero = sum(1 for a, _ in self.window if a == 0) / len(self.window)
        rate = sum(a for a, _ in self.window) / max(1, sum(d for _, d in self.window))
        if self.depth > 1 and (zero > c.demote_zero_accept or rate < c.demote_acceptance):
            self._set(self.depth - 1)
        elif self.depth < self.max_depth and len(self.window) == self.window.maxlen:
            full = all(a == d for a, d in self.window)
            self.good_windows = self.good_windows + 1 if full else 0
            if self.good_windows >= c.depth_promote_windows:
                self._set(self.depth + 1)
        return self.depth

    def _set(self, d: int) -> None:
        self.depth = d
        self.history.append((self.steps, d))
        self.window.clear()
        self.cooldown = self.cfg.depth_cooldown
        self.good_windows = 0


@dataclass
class _SeqState:
    catch: list = field(default_factory=list)      # (position, next token, trunk hidden row) not yet seen by the NextN layer


class MTPDecoder:
    def __init__(self, cfg: MTPConfig | None = None):
        self.cfg = cfg or MTPConfig()
        self.ctl = DepthController(self.cfg)
        self.seq: dict[int, _SeqState] = {}
        self._stats = {"steps": 0, "drafted": 0, "accepted": 0, "emitted": 0, "seq_steps": 0, "draft_s": 0.0, "verify_s": 0.0,
                       "accept_hist": [0, 0, 0, 0]}

    # -- wiring ---------------------------------------------------------------------------------------------
    def attach(self, engine) -> None:
        if engine.cfg.nextn_layers < 1 or not getattr(engine.model, "mtp_layers", None):
            raise ValueError("--mtp needs a model with a NextN (multi-token prediction) layer")
        self.engine = engine

    def release(self, req) -> None:
        self.seq.pop(req.rid, None)

    def stats(self) -> dict:
        s = dict(self._stats)
        s["acceptance_rate"] = s["accepted"] / s["drafted"] if s["drafted"] else 0.0
        s["tokens_per_step"] = s["emitted"] / s["seq_steps"] if s["seq_steps"] else 0.0   # per sequence
        s["depth"] = self.ctl.depth
        s["depth_changes"] = list(self.ctl.history)
        return s

    # -- prefill hook: run the NextN layer over the prompt so its K/V layer is complete ----------------------------
    def on_prefill_chunk(self, engine, fb: ForwardBatch, hidden: torch.Tensor, chunks: list) -> None:
        """``chunks``: (request, first position, n rows) in the row order of ``fb``."""
        nxt = []
        for r, start, n in chunks:
            seqtok = r.prompt[start + 1:start + n + 1]
            nxt.extend(seqtok + [0] * (n - len(seqtok)))          # the prompt's last row is redone with the sampled token
        T = len(nxt)
        fb2 = ForwardBatch(tokens=torch.tensor(nxt, dtype=torch.int32, device=engine.device), positions=fb.positions,
                           seq_ids=fb.seq_ids, block_table=fb.block_table, cu_q=fb.cu_q, ctx_lens=fb.ctx_lens,
                           max_q_len=fb.max_q_len, logit_rows=torch.zeros(1, dtype=torch.int32, device=engine.device))
        engine.model.mtp_forward(fb2, hidden[:T].clone(), engine.kv, depth=0)

    def on_prefill_done(self, engine, req, first_token: int, hidden_last: torch.Tensor) -> None:
        self.seq[req.rid] = _SeqState([(len(req.prompt) - 1, first_token, hidden_last)])

    # -- one speculative decode step over the running batch ----------------------------------------------------------
    def decode_step(self, engine, reqs: list) -> list:
        t0 = time.perf_counter()
        dev = engine.device
        it = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
        special = any(r.forced or r.params.needs_penalties or r.params.wants_logprobs for r in reqs)     # plain steps: one row each
        sampling = self.cfg.verify_mode == "speculative-sampling" and not all(r.params.is_greedy for r in reqs)
        if self.cfg.verify_mode == "greedy" and not all(r.params.is_greedy for r in reqs):
            special = True                                 # argmax verification would override the requested sampler
        k = 0 if special else self.ctl.depth
        k = min(k, min(engine.max_context - r.n_tokens - 2 for r in reqs))
        k = max(k, 0)
        reqs = engine._reserve_decode_pages(reqs, extra=k + 1)     # may preempt the youngest sequences
        if not reqs:
            return []
        B = len(reqs)
        n0 = [r.n_tokens for r in reqs]
        for r in reqs:
            if r.rid not in self.seq:                      # admitted through a terminal-state hit: only the last row is known
                self.seq[r.rid] = _SeqState([(r.n_tokens - 2, r.output[-1], r.hidden)])
        P = max(len(r.kv.pages) for r in reqs)
        bt = torch.zeros(B, P, dtype=torch.int32)
        for i, r in enumerate(reqs):
            bt[i, :len(r.kv.pages)] = torch.tensor(r.kv.pages, dtype=torch.int32)
        bt = bt.to(dev)

        # 1. catch-up + draft 1 (always runs, so the NextN K/V layer never falls behind)
        toks, pos, sid, cu, ctx, hid = [], [], [], [0], [], []
        for i, r in enumerate(reqs):
            rows = self.seq[r.rid].catch
            ctx.append(rows[0][0])
            for p, t, h in rows:
                toks.append(t)
                pos.append(p)
                sid.append(i)
                hid.append(h)
            cu.append(cu[-1] + len(rows))
            self.seq[r.rid].catch = []
        fb = ForwardBatch(tokens=it(toks), positions=it(pos), seq_ids=it(sid), block_table=bt, cu_q=it(cu), ctx_lens=it(ctx),
                          max_q_len=max(cu[i + 1] - cu[i] for i in range(B)), logit_rows=it([c - 1 for c in cu[1:]]))
        drafts: list[list[int]] = [[] for _ in reqs]
        p_draft = []
        if k > 0:
            logits, hm = engine.model.mtp_forward(fb, torch.stack(hid).float(), engine.kv, depth=0)
            hm = hm.index_select(0, fb.logit_rows.long()).clone()
            d = self._draft_tokens(engine, logits, reqs, sampling, p_draft, 0)
            for i in range(B):
                drafts[i].append(d[i])
            # 2. chained drafts 2..k: one row per sequence on the NextN layer's own hidden output
            n_mtp = len(engine.model.mtp_layers)
            for j in range(1, k):
                fbj = ForwardBatch(tokens=it([drafts[i][-1] for i in range(B)]), positions=it([n0[i] - 1 + (j - 1) for i in range(B)]),
                                   seq_ids=it(list(range(B))), block_table=bt, seq_lens=it([n0[i] + j - 1 for i in range(B)]),
                                   rows_per_seq=1, n_splits=1)
                logits, hm2 = engine.model.mtp_forward(fbj, hm, engine.kv, depth=min(j, n_mtp - 1) if n_mtp > 1 else 0)
                hm = hm2[:B].clone()
                d = self._draft_tokens(engine, logits, reqs, sampling, p_draft, j)
                for i in range(B):
                    drafts[i].append(d[i])
        else:
            engine.model.mtp_forward(fb, torch.stack(hid).float(), engine.kv, depth=0)
        t1 = time.perf_counter()

        # 3. verify: one trunk forward over k + 1 rows per sequence
        R = k + 1
        vt, vp = [], []
        for i, r in enumerate(reqs):
            vt.extend([r.output[-1]] + drafts[i])
            vp.extend(range(n0[i] - 1, n0[i] + k))
        G = engine.cfg.n_heads // engine.cfg.n_kv_heads
        if G * R <= 16:
            fbv = ForwardBatch(tokens=it(vt), positions=it(vp), seq_ids=it([i for i in range(B) for _ in range(R)]), block_table=bt,
                               seq_lens=it([n0[i] + k for i in range(B)]), rows_per_seq=R, n_splits=engine._splits_for(B))
        else:
            fbv = ForwardBatch(tokens=it(vt), positions=it(vp), seq_ids=it([i for i in range(B) for _ in range(R)]), block_table=bt,
                               cu_q=it([i * R for i in range(B + 1)]), ctx_lens=it([n0[i] - 1 for i in range(B)]), max_q_len=R)
        hybrid = engine.kv.hybrid
        if hybrid is not None:
            # linear-attention layers: with drafts in flight the pass leaves the recurrent state alone and a stash behind;
            # the state is advanced below by the accepted rows only
            fbv.state_slots = it([r.slot for r in reqs])
            fbv.defer_state = k > 0
        raw_logits, h = engine.model.forward(fbv, engine.kv)
        device_verify = (k > 0 and not sampling and engine.is_cuda and engine._sharded_vocab() and B * R <= engine._pairs.shape[0])
        logits = raw_logits if (k == 0 or device_verify) else engine._gather_vocab(raw_logits)
        h = h[:B * R].clone()

        # 4. accept
        if k == 0:
            out_tokens = [[t] for t in engine._sample_rows(raw_logits, reqs)]
            n_acc = [0] * B
        elif sampling:
            out_tokens, n_acc = self._verify_sampling(engine, logits.view(B, R, -1), torch.stack(p_draft, 1), drafts, reqs)
        else:
            if engine.is_cuda:
                # greedy verification on the device: per-shard argmax of the B x R target rows (8 bytes per row and rank
                # cross the wire instead of the logits), then one kernel compares drafts and targets and writes the
                # accepted prefix; only the counts and the tokens come back to the host
                from .. import ops
                tgt_dev = torch.empty(B * R, dtype=torch.int32, device=dev)
                if engine._sharded_vocab() and B * R <= engine._pairs.shape[0]:
                    engine._sharded_argmax(raw_logits.contiguous(), B * R, tgt_dev)
                else:
                    ops.argmax(logits.contiguous(), tgt_dev)
                n_acc_dev = torch.empty(B, dtype=torch.int32, device=dev)
                out_dev = torch.empty(B, R, dtype=torch.int32, device=dev)
                ops.spec_verify_greedy(it(drafts).view(B, k), tgt_dev.view(B, R), n_acc_dev, out_dev)
                acc_host, out_host, tgt = n_acc_dev.tolist(), out_dev.tolist(), tgt_dev.view(B, R).tolist()
            else:
                tgt = logits.argmax(-1).view(B, R).tolist()
                acc_host = out_host = None
            out_tokens, n_acc = [], []
            for i in range(B):
                if acc_host is not None:
                    a = acc_host[i]
                else:
                    a = 0
                    while a < k and drafts[i][a] == tgt[i][a]:
                        a += 1
                if self.cfg.force_accept:
                    a = k
                    out_tokens.append(drafts[i] + [tgt[i][k]])
                else:
                    out_tokens.append(out_host[i][:a + 1] if out_host is not None else tgt[i][:a + 1])
                n_acc.append(a)
        if hybrid is not None and k > 0:
            hybrid.commit([a + 1 for a in n_acc])
        outs = []
        for i, r in enumerate(reqs):
            a = n_acc[i]
            seqs = out_tokens[i]
            st = self.seq[r.rid]
            st.catch = [(n0[i] - 1 + j, seqs[j], h[i * R + j]) for j in range(a + 1)]
            r.hidden = h[i * R + a]
            r.step_count += 1
            out = engine._emit(r, seqs)
            if not out.finished:
                r.kv.length = r.n_tokens - 1
            outs.append(out)
            if k > 0:
                self.ctl.observe(a, k)
                self._stats["drafted"] += k
                self._stats["accepted"] += a
                self._stats["accept_hist"][a] += 1
            self._stats["emitted"] += len(out.new_tokens)
            self._stats["seq_steps"] += 1
        self.ctl.end_step()
        if engine.is_cuda:
            torch.cuda.synchronize(dev)
        t2 = time.perf_counter()
        self._stats["steps"] += 1
        self._stats["draft_s"] += t1 - t0
        self._stats["verify_s"] += t2 - t1
        engine.stats["decode_tokens"] += sum(len(o.new_tokens) for o in outs)
        engine.stats["decode_s"] += t2 - t0
        return outs

    # -- helpers --------------------------------------------------------------------------------------------------------
    def _draft_tokens(self, engine, logits, reqs, sampling: bool, p_draft: list, j: int) -> list[int]:
        if not sampling and engine.is_cuda and engine._sharded_vocab() and logits.shape[0] <= engine._pairs.shape[0]:
            tok = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
            engine._sharded_argmax(logits.contiguous(), logits.shape[0], tok)      # per-shard argmax + merge: no logits gather
            return tok.tolist()
        logits = engine._gather_vocab(logits)
        if not sampling:
            return logits.argmax(-1).tolist()
        temp = torch.tensor([max(r.params.temperature, 1e-3) if not r.params.is_greedy else 1e-3 for r in reqs],
                            device=logits.device).unsqueeze(1)
        p = torch.softmax(logits.float() / temp, -1)
        gens = []
        for i, r in enumerate(reqs):
            g = torch.Generator(device="cpu").manual_seed(((r.params.seed or r.rid * 7919 + 17) * 1000003 + len(r.output)) * 8 + j)
            gens.append(int(torch.multinomial(p[i].cpu(), 1, generator=g)))
        p_draft.append(p)
        return gens

    def _verify_sampling(self, engine, logits, p_draft, drafts, reqs):
        """Rejection sampling (accept draft x with probability min(1, p_target(x) / p_draft(x)); on reject resample from
        the normalised positive part of p_target - p_draft), which leaves the output distribution equal to the trunk's."""
        from .sampling import filtered_probs
        B, R, V = logits.shape
        k = R - 1
        p_t = torch.stack([torch.stack([filtered_probs(logits[i, j], r.params) for j in range(R)]) for i, r in enumerate(reqs)])
        dev = logits.device
        if engine.is_cuda:
            from .. import ops
            dr = torch.tensor(drafts, dtype=torch.int32, device=dev)
            seeds = torch.tensor([r.params.seed if r.params.seed is not None else r.rid * 7919 + 17 for r in reqs], dtype=torch.int64, device=dev)
            step = torch.tensor([len(r.output) for r in reqs], dtype=torch.int32, device=dev)
            n_acc = torch.empty(B, dtype=torch.int32, device=dev)
            out = torch.empty(B, R, dtype=torch.int32, device=dev)
            ops.spec_verify_reject(p_t.contiguous(), p_draft.contiguous().float(), dr, seeds, step, n_acc, out)
            n_acc = n_acc.tolist()
            out = out.tolist()
            return [out[i][:n_acc[i] + 1] for i in range(B)], n_acc
        outs, accs = [], []
        for i, r in enumerate(reqs):
            g = torch.Generator().manual_seed((r.params.seed or r.rid * 7919 + 17) * 1000003 + len(r.output) + 77)
            a, seq = 0, []
            while a < k:
                x = drafts[i][a]
                pt, pd = float(p_t[i, a, x]), float(p_draft[i, a, x])
                u = float(torch.rand(1, generator=g))
                if not (pt > 0 if pd <= 0 else u * pd < pt):
                    break
                seq.append(x)
                a += 1
            resid = p_t[i, a].clone()
            if a < k:
                resid = (resid - p_draft[i, a]).clamp_min(0)
                if float(resid.sum()) <= 0:
                    resid = p_t[i, a].clone()
            seq.append(int(torch.multinomial(resid.cpu() / resid.sum().cpu(), 1, generator=g)))
            outs.append(seq)
            accs.append(a)
        return outs, accs
