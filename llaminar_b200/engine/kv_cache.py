"""Paged KV cache: fixed 64-token pages, ref-counted so prefix-cache hits can share pages.

The reference keeps a per-sequence ring buffer per layer and *copies* cached prefix blocks back
in on a hit (reference: src/v2/kernels/cuda/kvcache/CUDARingKVCache.cu, src/v2/execution/
prefix_cache/PrefixStateCache.h).  Here a sequence is a list of page ids; a prefix hit just
appends the cached page ids to the new sequence's table and bumps their reference counts.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

PAGE_SIZE = 64


class OutOfPages(RuntimeError):
    pass


class PageAllocator:
    """Free-list allocator with reference counts (host side, O(1) per page)."""

    def __init__(self, n_pages: int, reserved: int = 1):
        # page 0 is kept as a scratch page that padded batch lanes point at
        self.n_pages = n_pages
        self.reserved = reserved
        self.free = list(range(n_pages - 1, reserved - 1, -1))
        self.refs = [0] * n_pages

    def alloc(self) -> int:
        if not self.free:
            raise OutOfPages("KV cache exhausted")
        p = self.free.pop()
        self.refs[p] = 1
        return p

    def retain(self, page: int) -> None:
        assert self.refs[page] > 0
        self.refs[page] += 1

    def release(self, page: int) -> None:
        assert self.refs[page] > 0, f"double free of page {page}"
        self.refs[page] -= 1
        if self.refs[page] == 0:
            self.free.append(page)

    @property
    def n_free(self) -> int:
        return len(self.free)


@dataclass
class SequenceKV:
    """Page table of one sequence."""
    pages: list[int] = field(default_factory=list)
    length: int = 0                  # tokens whose K/V are in the cache

    def capacity(self) -> int:
        return len(self.pages) * PAGE_SIZE


class HybridState:
    """Per-sequence state of the linear-attention layers of a hybrid model: for every such layer and every state slot the
    last K-1 inputs of the short convolution and one d x d matrix per value head (fp32).  A running sequence owns one slot
    from admission to its end; slot ``n_slots`` is scratch for the padded lanes of a captured decode step.  (The
    reference keeps these beside its ring KV cache: src/v2/kernels/cuda/kvcache/CUDAHybridRingKVCache.h.)"""

    def __init__(self, n_layers: int, n_slots: int, conv_dim: int, conv_kernel: int, n_v_heads: int, d: int, device):
        self.n_slots, self.scratch_slot = n_slots, n_slots
        self.conv = torch.zeros(n_layers, n_slots + 1, conv_dim, conv_kernel - 1, dtype=torch.float32, device=device)
        self.rec = torch.zeros(n_layers, n_slots + 1, n_v_heads, d, d, dtype=torch.float32, device=device)
        self.free = list(range(n_slots - 1, -1, -1))
        self.stash: dict = {}                  # layer -> what a deferred (speculative) pass left for `commit`
        self.stash_slots = None

    def commit(self, n_rows: list[int]) -> None:
        """After a deferred pass over R rows per sequence: advance every layer's state of sequence i by its first
        ``n_rows[i]`` rows (the accepted ones) and drop the stash."""
        from ..models.gdn import commit_rows
        n = torch.tensor(n_rows, dtype=torch.int64)
        for layer, st in self.stash.items():
            commit_rows(st, self.conv[layer], self.rec[layer], self.stash_slots, n)
        self.stash.clear()
        self.stash_slots = None

    def alloc(self) -> int:
        if not self.free:
            raise OutOfPages("no free state slot")
        return self.free.pop()

    def release(self, slot: int) -> None:
        assert 0 <= slot < self.n_slots and slot not in self.free
        self.free.append(slot)

    def snapshot(self, slot: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Copy of one slot's state over all layers (kept by the prefix cache at a block boundary of a prompt)."""
        return self.conv[:, slot].clone(), self.rec[:, slot].clone()

    def restore(self, slot: int, snap: tuple[torch.Tensor, torch.Tensor]) -> None:
        self.conv[:, slot].copy_(snap[0])
        self.rec[:, slot].copy_(snap[1])

    @property
    def slot_bytes(self) -> int:
        return 4 * (self.conv[:, 0].numel() + self.rec[:, 0].numel())

    @staticmethod
    def bytes_per_slot(n_layers: int, conv_dim: int, conv_kernel: int, n_v_heads: int, d: int) -> int:
        return 4 * n_layers * (conv_dim * (conv_kernel - 1) + n_v_heads * d * d)


Q8 = "q8_0"          # 8-bit cache: int8 values with one fp16 scale per 32 (CUDA back end; reference: CUDARingKVCache.cu:405)


class PagedKVCache:
    def __init__(self, n_layers: int, n_kv_heads: int, head_dim: int, n_pages: int, device, dtype=torch.bfloat16):
        self.n_layers, self.n_kv_heads, self.head_dim, self.n_pages = n_layers, n_kv_heads, head_dim, n_pages
        self.device = torch.device(device)
        self.q8 = dtype == Q8
        if self.q8:
            # a page is [2][n_kv_heads][64][head_dim] int8 followed by [2][n_kv_heads][64][head_dim / 32] fp16 block scales;
            # zero bytes decode to zeros, so untouched positions stay finite
            if head_dim % 32:
                raise ValueError("the 8-bit KV cache needs a head dimension that is a multiple of 32")
            data = 2 * n_kv_heads * PAGE_SIZE * head_dim
            self.layers = [torch.zeros(n_pages, data + data // 16, dtype=torch.uint8, device=device) for _ in range(n_layers)]
        else:
            # zero-filled: masked-out positions are multiplied by zero probabilities, so they must stay finite
            self.layers = [torch.zeros(n_pages, 2, n_kv_heads, PAGE_SIZE, head_dim, dtype=dtype, device=device)
                           for _ in range(n_layers)]
        self.allocator = PageAllocator(n_pages)
        self.hybrid: HybridState | None = None          # set by the engine for models with linear-attention layers

    @staticmethod
    def bytes_per_page(n_layers: int, n_kv_heads: int, head_dim: int, itemsize: float = 2) -> int:
        return int(n_layers * 2 * n_kv_heads * PAGE_SIZE * head_dim * itemsize)

    def ensure_capacity(self, seq: SequenceKV, n_tokens: int) -> None:
        """Grow the page table so that ``n_tokens`` positions fit."""
        while seq.capacity() < n_tokens:
            seq.pages.append(self.allocator.alloc())

    def free_sequence(self, seq: SequenceKV) -> None:
        for p in seq.pages:
            self.allocator.release(p)
        seq.pages.clear()
        seq.length = 0

    def truncate(self, seq: SequenceKV, n_tokens: int) -> None:
        """Roll a sequence back to ``n_tokens`` (speculative-decode rejection); frees whole spare pages."""
        keep = (n_tokens + PAGE_SIZE - 1) // PAGE_SIZE
        while len(seq.pages) > max(keep, 0):
            self.allocator.release(seq.pages.pop())
        seq.length = min(seq.length, n_tokens)

    def fork_prefix(self, pages: list[int], n_tokens: int) -> SequenceKV:
        """New sequence that shares the given full pages (prefix-cache hit)."""
        assert n_tokens == len(pages) * PAGE_SIZE
        for p in pages:
            self.allocator.retain(p)
        return SequenceKV(list(pages), n_tokens)

    # -- page payload movement for the RAM / disk prefix tiers -------------------------------
    def export_page(self, page: int) -> torch.Tensor:
        if not self.layers:                      # a pipeline stage of linear-attention blocks only: pages carry no bytes here
            return torch.empty(0)
        return torch.stack([l[page] for l in self.layers]).to("cpu", non_blocking=False)

    def import_page(self, page: int, payload: torch.Tensor) -> None:
        for i, l in enumerate(self.layers):
            l[page].copy_(payload[i].to(self.device, non_blocking=True))
