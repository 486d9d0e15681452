"""Gated-DeltaNet linear attention in plain PyTorch: the pieces of the hybrid (qwen35) blocks.

A linear-attention block keeps, per sequence, the last ``K - 1`` inputs of a short causal convolution and one
``d_k x d_v`` matrix per value head.  Per token t and head:

    a_t = exp(g_t)                      g_t = ssm_a * softplus(alpha_t + dt_bias)        (ssm_a = -exp(A_log) < 0)
    S   = a_t * S                       decay
    u_t = beta_t * (v_t - S^T k_t)      delta-rule correction, beta_t = sigmoid(b_t)
    S   = S + k_t u_t^T
    o_t = S^T q_t                       q, k L2-normalised, q scaled by d_k^-1/2

(reference: the recurrence and chunk kernels of src/v2/kernels/cuda/gdn/CUDAGatedDeltaNetKernels.cu and the stage that
drives them, src/v2/execution/compute_stages/stages/GDNRecurrenceStage.cpp; value head j reads key head j mod n_k, the
tiled order GGUF files store).  Two evaluators of the same recurrence are given: token by token (decode, and the oracle of
the other), and chunk-parallel for prefill, which turns a chunk of C tokens into one unit-lower-triangular solve and three
matrix products per head.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def causal_conv_silu(x: torch.Tensor, state: torch.Tensor, w: torch.Tensor):
    """Depth-wise causal convolution + SiLU over one sequence.  x: [T, C] new inputs, state: [C, K-1] the inputs before
    them (zeros at the start of a sequence), w: [C, K] taps (tap K-1 multiplies the newest input).  Returns
    (y [T, C], new state [C, K-1])."""
    T, C = x.shape
    K = w.shape[1]
    xp = torch.cat([state.t().to(x.dtype), x], dim=0)                    # [K-1+T, C]
    y = torch.zeros(T, C, dtype=x.dtype, device=x.device)
    for j in range(K):
        y += xp[j:j + T] * w[:, j]
    return F.silu(y), xp[T:].t().contiguous()


def gates(alpha: torch.Tensor, b: torch.Tensor, ssm_a: torch.Tensor, dt_bias: torch.Tensor):
    """Log-decay g (<= 0) and write strength beta of every (token, value head).  alpha, b: [T, H]."""
    return ssm_a.float() * F.softplus(alpha.float() + dt_bias.float()), torch.sigmoid(b.float())


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(dim=-1, keepdim=True) + eps)


def expand_key_heads(x: torch.Tensor, n_v: int, v_head_offset: int = 0) -> torch.Tensor:
    """[T, n_k, d] -> [T, n_v, d]: value head j (global index j + v_head_offset) reads key head (j + offset) mod n_k."""
    n_k = x.shape[1]
    idx = (torch.arange(n_v, device=x.device) + v_head_offset) % n_k
    return x.index_select(1, idx)


def delta_rule_recurrent(q, k, v, g, beta, S):
    """Token-by-token evaluation.  q, k: [T, H, dk] (already normalised / scaled), v: [T, H, dv], g, beta: [T, H],
    S: [H, dk, dv] float32 (updated in place).  Returns o [T, H, dv]."""
    T = q.shape[0]
    o = torch.empty_like(v, dtype=torch.float32)
    for t in range(T):
        S.mul_(torch.exp(g[t])[:, None, None])
        u = (v[t] - torch.einsum("hkv,hk->hv", S, k[t])) * beta[t][:, None]
        S.add_(torch.einsum("hk,hv->hkv", k[t], u))
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o


def delta_rule_chunked(q, k, v, g, beta, S, chunk: int = 64):
    """Chunk-parallel evaluation of the same recurrence (same arguments and result as `delta_rule_recurrent`).

    Inside a chunk let G_t be the running sum of g and M[t, i] = exp(G_t - G_i) for i <= t (0 above the diagonal).  The
    corrections solve (I + A) U = beta * (V - exp(G) * K S0) with A[t, i] = beta_t M[t, i] (k_t . k_i) for i < t; then
    O = exp(G) * Q S0 + (M * Q K^T) U and S_C = exp(G_C) S0 + K^T (exp(G_C - G) * U).  Every exponent is <= 0."""
    T, H, dk = q.shape
    o = torch.empty(T, H, v.shape[-1], dtype=torch.float32, device=q.device)
    for c0 in range(0, T, chunk):
        c1 = min(T, c0 + chunk)
        C = c1 - c0
        qc, kc, vc = (x[c0:c1].float().transpose(0, 1) for x in (q, k, v))          # [H, C, d]
        gc, bc = g[c0:c1].float().t(), beta[c0:c1].float().t()                      # [H, C]
        G = torch.cumsum(gc, dim=1)
        low = torch.tril(torch.ones(C, C, dtype=torch.bool, device=q.device))
        M = torch.exp((G[:, :, None] - G[:, None, :]).masked_fill(~low, float("-inf")))       # [H, C, C], 0 above the diagonal
        eG = torch.exp(G)[:, :, None]
        A = (kc @ kc.transpose(1, 2)) * M * bc[:, :, None]
        A = A.masked_fill(torch.eye(C, dtype=torch.bool, device=q.device), 0.0)               # strictly lower
        rhs = (vc - eG * (kc @ S)) * bc[:, :, None]
        U = torch.linalg.solve_triangular(A + torch.eye(C, device=q.device), rhs, upper=False, unitriangular=True)
        o[c0:c1] = (eG * (qc @ S) + ((qc @ kc.transpose(1, 2)) * M) @ U).transpose(0, 1)
        last = torch.exp(G[:, -1:, None] - G[:, :, None])                                     # [H, C, 1]
        S.mul_(torch.exp(G[:, -1])[:, None, None]).add_(kc.transpose(1, 2) @ (last * U))
    return o


def gated_rmsnorm(o: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over each head's d_v values, then * SiLU(z).  o, z: [T, H, dv]; w: [dv]."""
    of = o.float()
    return of * torch.rsqrt(of.pow(2).mean(dim=-1, keepdim=True) + eps) * w.float() * F.silu(z.float())


def gdn_mix(qkv: torch.Tensor, z: torch.Tensor, alpha: torch.Tensor, b: torch.Tensor, conv_w, ssm_a, dt_bias, norm_w,
            conv_state: torch.Tensor, S: torch.Tensor, n_k: int, n_v: int, d: int, eps: float,
            v_head_offset: int = 0, chunk: int = 64) -> tuple[torch.Tensor, torch.Tensor]:
    """Everything between the input projections and the output projection of one linear-attention block, for the new
    tokens of ONE sequence.  qkv: [T, 2 n_k d + n_v d], z: [T, n_v d], alpha, b: [T, n_v]; conv_state [C, K-1] and
    S [n_v, d, d] are the sequence's state before these tokens.  Returns (rows [T, n_v d] for the output projection,
    new conv state); S is updated in place."""
    T = qkv.shape[0]
    y, conv_state = causal_conv_silu(qkv.float(), conv_state, conv_w.float())
    q, k, v = torch.split(y, [n_k * d, n_k * d, n_v * d], dim=-1)
    q = expand_key_heads(l2norm(q.view(T, n_k, d)) * d ** -0.5, n_v, v_head_offset)
    k = expand_key_heads(l2norm(k.view(T, n_k, d)), n_v, v_head_offset)
    g, beta = gates(alpha, b, ssm_a, dt_bias)
    if T <= 4:
        o = delta_rule_recurrent(q, k, v.view(T, n_v, d), g, beta, S)
    else:
        o = delta_rule_chunked(q, k, v.view(T, n_v, d), g, beta, S, chunk)
    return gated_rmsnorm(o, z.view(T, n_v, d), norm_w, eps).reshape(T, n_v * d), conv_state


def gdn_block_rows(qkv, z, alpha, b, seqs, conv_pool, rec_pool, conv_w, ssm_a, dt_bias, norm_w, n_k: int, n_v: int, d: int,
                   eps: float, v_head_offset: int = 0) -> torch.Tensor:
    """The linear-attention mix for a packed batch.  ``seqs``: (first row, end row, state slot, fresh) per sequence, rows of
    a sequence being consecutive; ``fresh`` sequences start from a zero state.  conv_pool [slots, C, K-1] and
    rec_pool [slots, n_v, d, d] are one layer's state pools and are updated.  Returns fp32 rows [T, n_v d].
    Sequences with the same number of rows (the usual prefill batch of equal prompts or equal chunks) are evaluated
    together, their heads stacked into one batch axis, so the number of small launches does not grow with the batch."""
    out = torch.empty(qkv.shape[0], n_v * d, dtype=torch.float32, device=qkv.device)
    by_len: dict[int, list] = {}
    for sq in seqs:
        if sq[3]:
            conv_pool[sq[2]].zero_()
            rec_pool[sq[2]].zero_()
        by_len.setdefault(sq[1] - sq[0], []).append(sq)
    for T, group in by_len.items():
        if len(group) == 1 or T <= 4:
            for r0, r1, slot, _ in group:
                out[r0:r1], conv_pool[slot] = gdn_mix(qkv[r0:r1], z[r0:r1], alpha[r0:r1], b[r0:r1], conv_w, ssm_a, dt_bias, norm_w,
                                                     conv_pool[slot], rec_pool[slot], n_k, n_v, d, eps, v_head_offset)
            continue
        G = len(group)
        rows = torch.cat([torch.arange(r0, r1, device=qkv.device) for r0, r1, _, _ in group])
        slots = torch.tensor([sq[2] for sq in group], device=qkv.device)
        pick = lambda t: t.index_select(0, rows).float().view(G, T, -1)
        x, K = pick(qkv), conv_w.shape[1]
        xp = torch.cat([conv_pool[slots].transpose(1, 2), x], dim=1)                          # [G, K-1+T, C]
        y = torch.zeros_like(x)
        for j in range(K):
            y += xp[:, j:j + T] * conv_w.float()[:, j]
        conv_pool[slots] = xp[:, T:].transpose(1, 2)
        q, k, v = torch.split(F.silu(y), [n_k * d, n_k * d, n_v * d], dim=-1)
        idx = (torch.arange(n_v, device=qkv.device) + v_head_offset) % n_k
        # [G, T, heads, d] -> [T, G * n_v, d]: every (sequence, value head) is one row of the batch axis of the chunk form
        fold = lambda t: t.permute(1, 0, 2, 3).reshape(T, G * n_v, d)
        q = fold((l2norm(q.view(G, T, n_k, d)) * d ** -0.5).index_select(2, idx))
        k = fold(l2norm(k.view(G, T, n_k, d)).index_select(2, idx))
        g, beta = gates(pick(alpha), pick(b), ssm_a, dt_bias)                                 # [G, T, n_v]
        S = rec_pool[slots].reshape(G * n_v, d, d)
        o = delta_rule_chunked(q, k, fold(v.view(G, T, n_v, d)), g.permute(1, 0, 2).reshape(T, G * n_v),
                               beta.permute(1, 0, 2).reshape(T, G * n_v), S)
        rec_pool[slots] = S.view(G, n_v, d, d)
        o = o.view(T, G, n_v, d).permute(1, 0, 2, 3).reshape(G * T, n_v, d)
        out[rows] = gated_rmsnorm(o, pick(z).reshape(G * T, n_v, d), norm_w, eps).reshape(G * T, n_v * d)
    return out


def batch_sequences(seq_ids, positions, state_slots) -> list[tuple[int, int, int, bool]]:
    """(first row, end row, slot, fresh) of every sequence of a packed batch (host lists; one synchronisation on a GPU)."""
    sid, pos, slots = seq_ids.tolist(), positions.tolist(), state_slots.tolist()
    out, r0 = [], 0
    for r in range(1, len(sid) + 1):
        if r == len(sid) or sid[r] != sid[r0]:
            out.append((r0, r, slots[sid[r0]], pos[r0] == 0))
            r0 = r
    return out


def gdn_rows_deferred(qkv, z, alpha, b, conv_w, ssm_a, dt_bias, norm_w, conv_pool, rec_pool, slots, n_k: int, n_v: int, d: int,
                      eps: float, v_head_offset: int = 0):
    """R new rows for each of B sequences (speculative verification) WITHOUT touching the state pools: the outputs are what
    feeding the rows one by one would give, and the returned stash holds what `commit_rows` needs to advance each
    sequence's state by however many of its rows are accepted afterwards (the per-row decay, key and correction, and the
    convolution inputs), a few KB per row instead of a copy of the state per row.
    qkv: [B, R, C], z: [B, R, n_v d], alpha, b: [B, R, n_v]; slots: [B] int64.  Returns (rows [B * R, n_v d] fp32, stash).
    (reference: the verifier's state capture rows, src/v2/models/qwen35/Qwen35Graph.cpp:886-887.)"""
    B, R, C = qkv.shape
    K = conv_w.shape[1]
    xp = torch.cat([conv_pool[slots].transpose(1, 2), qkv.float()], dim=1)                     # [B, K-1+R, C]
    y = torch.zeros(B, R, C, dtype=torch.float32, device=qkv.device)
    for j in range(K):
        y += xp[:, j:j + R] * conv_w.float()[:, j]
    y = F.silu(y)
    q, k, v = torch.split(y, [n_k * d, n_k * d, n_v * d], dim=-1)
    idx = (torch.arange(n_v, device=qkv.device) + v_head_offset) % n_k
    q = (l2norm(q.view(B, R, n_k, d)) * d ** -0.5).index_select(2, idx)
    k = l2norm(k.view(B, R, n_k, d)).index_select(2, idx)
    v = v.view(B, R, n_v, d)
    g, beta = gates(alpha, b, ssm_a, dt_bias)                                                 # [B, R, n_v]
    S = rec_pool[slots].clone()                                                               # [B, n_v, d, d]
    o = torch.empty(B, R, n_v, d, dtype=torch.float32, device=qkv.device)
    u_all = torch.empty_like(o)
    for j in range(R):
        S = S * torch.exp(g[:, j])[:, :, None, None]
        u = (v[:, j] - torch.einsum("bhkv,bhk->bhv", S, k[:, j])) * beta[:, j][..., None]
        S = S + torch.einsum("bhk,bhv->bhkv", k[:, j], u)
        o[:, j] = torch.einsum("bhkv,bhk->bhv", S, q[:, j])
        u_all[:, j] = u
    rows = gated_rmsnorm(o.view(B * R, n_v, d), z.reshape(B * R, n_v, d), norm_w, eps).reshape(B * R, n_v * d)
    return rows, (g, k, u_all, xp)


def commit_rows(stash, conv_pool, rec_pool, slots, n_rows) -> None:
    """Advance the state of sequence i (slot ``slots[i]``) by its first ``n_rows[i]`` stashed rows (>= 1)."""
    g, k, u, xp = stash
    B, R = g.shape[:2]
    Km1 = conv_pool.shape[-1]
    S = rec_pool[slots]
    n_rows = n_rows.to(g.device)
    for j in range(R):
        live = (n_rows > j)[:, None, None, None]
        S = torch.where(live, S * torch.exp(g[:, j])[:, :, None, None] + torch.einsum("bhk,bhv->bhkv", k[:, j], u[:, j]), S)
    rec_pool[slots] = S
    # the convolution window ends at the last accepted row: inputs n .. n + K - 2 of xp (xp starts with the old window)
    win = torch.stack([xp[i, int(n):int(n) + Km1] for i, n in enumerate(n_rows.tolist())])    # [B, K-1, C]
    conv_pool[slots] = win.transpose(1, 2)
