"""Prefix cache over the paged KV cache: chained block hashes, device / RAM / disk tiers, LRU, terminal states.

Keying follows the reference: every 64-token block is hashed together with its parent's hash and a
fingerprint of everything that changes the KV contents (model, runtime precision, topology, MoE placement,
MTP) (reference: src/v2/execution/prefix_cache/BlockHash.cpp, PrefixCacheKey.h, PrefixCacheFingerprint.h).
Where the reference *copies* cached KV blocks back into a sequence's ring buffer on a hit
(PrefixStateCache.h, PrefixStorageBackend.h), the device tier here shares pages: a hit appends the cached
page ids to the new sequence's page table and bumps reference counts.  Evicted pages spill to pinned host
memory and optionally to disk, and are re-imported on a later hit.  A *terminal state* (first-token logits,
final hidden row and a copy of the partial tail page) lets an exact repeat of a prompt skip the forward pass
(reference: src/v2/execution/runner/OrchestrationRunner.cpp:1207-1214).

Hybrid models (linear-attention layers with a recurrent state) can resume a cached prefix only where that state is
known.  The engine snapshots it once per prompt, at the last block boundary that leaves a token to run, and a hit is cut
back to the longest cached chain that ends at a boundary with a snapshot (`store_state`, `state_boundary`; the reference
stores the hybrid state in its block payloads: src/v2/execution/prefix_cache/PrefixPayloadLayout.h).  A follow-up prompt
that extends an earlier one (a chat turn) therefore reuses the earlier prompt up to that boundary.
"""
from __future__ import annotations

import hashlib
import os
import struct
from collections import OrderedDict
from dataclasses import dataclass, field

import torch

from .kv_cache import PAGE_SIZE, OutOfPages, SequenceKV


@dataclass
class PrefixCacheConfig:
    storage: str = "tiered"              # ram | device | tiered
    block_size: int = PAGE_SIZE
    vram_budget_mb: int = 256
    ram_budget_mb: int = 4096
    disk_budget_mb: int = 0
    disk_dir: str | None = None
    terminal_state: str = "auto"         # off | auto | always
    moe_policy: str = "placement-fingerprint"
    state_stride: int = 0                # hybrid models: extra recurrent-state snapshots every this many prompt tokens (0: none)

    @staticmethod
    def from_values(v: dict) -> "PrefixCacheConfig":
        return PrefixCacheConfig(v.get("prefix_cache_storage", "tiered"), int(v.get("prefix_cache_block_size", 64)),
                                 int(v.get("prefix_cache_vram_budget_mb", 256)), int(v.get("prefix_cache_ram_budget_mb", 4096)),
                                 int(v.get("prefix_cache_disk_budget_mb", 0)), v.get("prefix_cache_disk_dir"),
                                 v.get("prefix_cache_terminal_state", "auto"), v.get("prefix_cache_moe_policy", "placement-fingerprint"),
                                 int(v.get("prefix_cache_state_stride") or 0))


def chain_hashes(tokens: list[int], salt: bytes, block: int = PAGE_SIZE) -> list[bytes]:
    """Hash of every *full* block, each chained through its parent's hash."""
    out, parent = [], salt
    for i in range(0, len(tokens) - len(tokens) % block, block):
        h = hashlib.blake2b(parent + struct.pack(f"<{block}i", *tokens[i:i + block]), digest_size=16).digest()
        out.append(h)
        parent = h
    return out


@dataclass
class TerminalState:
    n_tokens: int
    tail_tokens: int
    tail_payload: torch.Tensor | None     # [layers, 2, kv_heads, 64, D] copy of the partial last page (device)
    logits: torch.Tensor
    hidden: torch.Tensor | None


class PrefixCache:
    def __init__(self, cfg: PrefixCacheConfig | None = None, fingerprint: str = ""):
        self.cfg = cfg or PrefixCacheConfig()
        self.salt = hashlib.blake2b(fingerprint.encode(), digest_size=16).digest()
        self.device: "OrderedDict[bytes, int]" = OrderedDict()          # hash -> page id (cache holds one reference)
        self.ram: "OrderedDict[bytes, torch.Tensor]" = OrderedDict()    # hash -> pinned host payload
        self.disk: "OrderedDict[bytes, int]" = OrderedDict()            # hash -> bytes on disk
        self.terminal: "OrderedDict[bytes, TerminalState]" = OrderedDict()
        self.states: "OrderedDict[bytes, tuple]" = OrderedDict()        # hash of the block that ends at a boundary -> state snapshot
        self.max_states = 0
        self.engine = None
        self.page_bytes = 0
        self._stats = {"lookups": 0, "hits": 0, "hit_tokens": 0, "inserted_blocks": 0, "evicted_to_ram": 0,
                       "evicted_to_disk": 0, "dropped": 0, "promoted": 0, "terminal_hits": 0, "terminal_stored": 0,
                       "state_snapshots": 0}
        self.file_prefix = self.salt.hex()[:8]           # completed by attach(): the shard of the cache this process holds

    # -- wiring ---------------------------------------------------------------------------------------------
    def attach(self, engine) -> None:
        self.engine = engine
        kv = engine.kv
        el = kv.layers[0].element_size() if kv.layers else 2
        self.page_bytes = kv.n_layers * 2 * kv.n_kv_heads * PAGE_SIZE * kv.head_dim * el
        if kv.hybrid is not None:
            # state snapshots live on the device; between 1 and 64 of them, within the device budget of the cache
            self.max_states = max(1, min(64, self.cfg.vram_budget_mb * (1 << 20) // max(kv.hybrid.slot_bytes, 1)))
        # Disk-tier files are private to one shard of the cache: every rank of a multi-process engine holds other KV heads
        # (tensor parallelism) or other layers (pipeline stages) of the same block hash.  The file prefix therefore names
        # the model fingerprint AND this process's rank / world size and page geometry, so that a rank never reads a
        # payload that another rank, or an earlier run with another layout, wrote.
        import torch.distributed as dist
        rank, world = (dist.get_rank(), dist.get_world_size()) if dist.is_available() and dist.is_initialized() else (0, 1)
        shard = f"{rank}/{world}/{kv.n_layers}/{kv.n_kv_heads}/{kv.head_dim}/{kv.layers[0].dtype if kv.layers else None}"
        self.file_prefix = self.salt.hex()[:8] + hashlib.blake2b(shard.encode(), digest_size=4).hexdigest()
        if self.cfg.disk_dir and self.cfg.disk_budget_mb > 0:
            os.makedirs(self.cfg.disk_dir, exist_ok=True)
            for name in sorted(os.listdir(self.cfg.disk_dir)):          # blocks persisted by an earlier process
                if name.endswith(".kvblk") and name.startswith(self.file_prefix + "_"):
                    self.disk[bytes.fromhex(name[len(self.file_prefix) + 1:-6])] = os.path.getsize(os.path.join(self.cfg.disk_dir, name))

    @property
    def max_device_pages(self) -> int:
        if self.cfg.storage == "ram":
            return 0
        return max(1, self.cfg.vram_budget_mb * (1 << 20) // max(self.page_bytes, 1))

    def stats(self) -> dict:
        s = dict(self._stats)
        s.update(device_blocks=len(self.device), ram_blocks=len(self.ram), disk_blocks=len(self.disk),
                 terminal_states=len(self.terminal))
        return s

    def clear(self) -> None:
        if self.engine is not None:
            for page in self.device.values():
                self.engine.kv.allocator.release(page)
        self.device.clear()
        self.ram.clear()
        self.terminal.clear()
        self.states.clear()

    # -- lookup -----------------------------------------------------------------------------------------------
    def lookup(self, prompt: list[int]) -> tuple[list[int], int]:
        """Longest cached chain of full blocks -> (page ids, tokens covered).  RAM / disk hits are re-imported.

        Every returned page carries one extra reference that belongs to the caller: promoting a later block of the chain
        may have to evict, and a page that only the cache held could otherwise be evicted and handed straight back for
        the new block while it is already part of this result.  The caller drops the references with `release_pages`
        once the sequence has taken its own (`fork_prefix`)."""
        self._stats["lookups"] += 1
        kv = self.engine.kv
        pages: list[int] = []
        for h in chain_hashes(prompt, self.salt, self.cfg.block_size):
            page = self.device.get(h)
            if page is None:
                payload = self._fetch_lower(h)
                if payload is None:
                    break
                try:
                    page = self._alloc_page()
                except OutOfPages:
                    break
                kv.import_page(page, payload)
                self._register_device(h, page)
                self._stats["promoted"] += 1
            else:
                self.device.move_to_end(h)
            kv.allocator.retain(page)
            pages.append(page)
        if pages:
            self._stats["hits"] += 1
            self._stats["hit_tokens"] += len(pages) * PAGE_SIZE
        return pages, len(pages) * PAGE_SIZE

    # -- recurrent-state snapshots of hybrid models ----------------------------------------------------------
    def store_state(self, prompt_prefix: list[int], snap: tuple) -> None:
        """Keep the state a sequence has after exactly ``prompt_prefix`` (a whole number of blocks)."""
        hs = chain_hashes(prompt_prefix, self.salt, self.cfg.block_size)
        if not hs or len(prompt_prefix) % self.cfg.block_size or self.max_states == 0:
            return
        self.states[hs[-1]] = snap
        self.states.move_to_end(hs[-1])
        self._stats["state_snapshots"] += 1
        while len(self.states) > self.max_states:
            self.states.popitem(last=False)

    def snapshot_points(self, n_prompt: int, done: int) -> list[int]:
        """Where prefill of an ``n_prompt``-token prompt, ``done`` tokens of which are cached already, should leave a snapshot:
        the last block boundary that leaves a token to run, and every `state_stride` tokens before it."""
        if self.max_states == 0:
            return []
        blk = self.cfg.block_size
        last = (n_prompt - 1) // blk * blk
        stride = self.cfg.state_stride // blk * blk
        pts = set(range(stride, last + 1, stride)) if stride > 0 else set()
        pts.add(last)
        return sorted(p for p in pts if p > done)

    def state_boundary(self, prompt: list[int], limit_tokens: int) -> int:
        """Largest block boundary <= ``limit_tokens`` at which a snapshot of this prompt's state is held (0: none)."""
        hs = chain_hashes(prompt[:limit_tokens - limit_tokens % self.cfg.block_size], self.salt, self.cfg.block_size)
        for i in range(len(hs), 0, -1):
            if hs[i - 1] in self.states:
                return i * self.cfg.block_size
        return 0

    def state_at(self, prompt: list[int], n_tokens: int):
        hs = chain_hashes(prompt[:n_tokens], self.salt, self.cfg.block_size)
        snap = self.states.get(hs[-1]) if hs and n_tokens % self.cfg.block_size == 0 else None
        if snap is not None:
            self.states.move_to_end(hs[-1])
        return snap

    def release_pages(self, pages: list[int]) -> None:
        """Drop the references `lookup` took on the caller's behalf."""
        for p in pages:
            self.engine.kv.allocator.release(p)

    def lookup_terminal(self, prompt: list[int]) -> TerminalState | None:
        if self.cfg.terminal_state == "off":
            return None
        t = self.terminal.get(self._terminal_key(prompt))
        if t is not None:
            self.terminal.move_to_end(self._terminal_key(prompt))
        return t

    def _terminal_key(self, prompt: list[int]) -> bytes:
        return hashlib.blake2b(self.salt + struct.pack(f"<{len(prompt)}i", *prompt), digest_size=16).digest()

    def _fetch_lower(self, h: bytes):
        if h in self.ram:
            self.ram.move_to_end(h)
            return self.ram[h]
        if h in self.disk:
            path = self._disk_path(h)
            try:
                return torch.load(path, map_location="cpu")
            except Exception:
                self.disk.pop(h, None)
        return None

    # -- insert -----------------------------------------------------------------------------------------------
    def insert(self, engine, req) -> None:
        """Register every full block of the request whose K/V is in the cache and not known yet."""
        n_cached = req.kv.length
        toks = req.all_tokens[:n_cached]
        for i, h in enumerate(chain_hashes(toks, self.salt, self.cfg.block_size)):
            if h in self.device:
                self.device.move_to_end(h)
                continue
            if i >= len(req.kv.pages):
                break
            page = req.kv.pages[i]
            if self.max_device_pages == 0:
                self._spill(h, engine.kv.export_page(page))
            else:
                engine.kv.allocator.retain(page)
                self._register_device(h, page)
            self._stats["inserted_blocks"] += 1
        self._trim_device()

    def store_terminal(self, engine, req, logits: torch.Tensor, hidden: torch.Tensor | None) -> None:
        mode = self.cfg.terminal_state
        n = len(req.prompt)
        if mode == "off" or (mode == "auto" and n < 2 * PAGE_SIZE):
            return
        tail = n % PAGE_SIZE
        payload = None
        if tail:
            page = req.kv.pages[n // PAGE_SIZE]
            payload = torch.stack([l[page] for l in engine.kv.layers]).clone()
        self.terminal[self._terminal_key(req.prompt)] = TerminalState(n, tail, payload, logits.detach().clone(),
                                                                        None if hidden is None else hidden.detach().clone())
        self._stats["terminal_stored"] += 1
        while len(self.terminal) > 64:
            self.terminal.popitem(last=False)

    def restore_terminal(self, engine, req, term: TerminalState) -> bool:
        """Rebuild the sequence's pages for an exact prompt repeat; False if the full blocks are gone."""
        held, covered = self.lookup(req.prompt)
        need_full = term.n_tokens - term.tail_tokens
        if covered < need_full:
            self.release_pages(held)
            return False
        try:
            pages = held[:need_full // PAGE_SIZE]
            req.kv = engine.kv.fork_prefix(pages, need_full) if pages else SequenceKV()
            if term.tail_tokens:
                page = self._alloc_page()
                for i, l in enumerate(engine.kv.layers):
                    l[page].copy_(term.tail_payload[i])
                req.kv.pages.append(page)
        finally:
            self.release_pages(held)
        req.kv.length = term.n_tokens
        self._stats["terminal_hits"] += 1
        return True

    # -- eviction ---------------------------------------------------------------------------------------------
    def _alloc_page(self) -> int:
        kv = self.engine.kv
        try:
            return kv.allocator.alloc()
        except OutOfPages:
            if not self.evict_for(self.engine, PAGE_SIZE):
                raise
            return kv.allocator.alloc()

    def _register_device(self, h: bytes, page: int) -> None:
        self.device[h] = page
        self.device.move_to_end(h)

    def trim(self) -> None:
        self._trim_device()

    def _trim_device(self) -> None:
        while len(self.device) > self.max_device_pages:
            if not self._evict_one():
                break

    def _evict_one(self) -> bool:
        kv = self.engine.kv
        for h, page in self.device.items():                 # oldest first
            if kv.allocator.refs[page] == 1:                # only the cache still holds it
                if self.cfg.storage in ("ram", "tiered"):
                    self._spill(h, kv.export_page(page))
                else:
                    self._stats["dropped"] += 1
                del self.device[h]
                kv.allocator.release(page)
                return True
        return False

    def evictable_pages(self) -> int:
        """Device pages that only the cache still holds (they can be handed back to the allocator on demand)."""
        refs = self.engine.kv.allocator.refs
        return sum(1 for page in self.device.values() if refs[page] == 1)

    def evict_for(self, engine, n_tokens: int) -> bool:
        """Free at least ceil(n_tokens / 64) pages held only by the cache.  Returns False if nothing could be freed."""
        need = (n_tokens + PAGE_SIZE - 1) // PAGE_SIZE
        freed = 0
        while freed < need and self._evict_one():
            freed += 1
        return freed > 0

    def _spill(self, h: bytes, payload: torch.Tensor) -> None:
        if self.cfg.ram_budget_mb > 0:
            self.ram[h] = payload.pin_memory() if torch.cuda.is_available() else payload
            self._stats["evicted_to_ram"] += 1
            max_blocks = max(1, self.cfg.ram_budget_mb * (1 << 20) // max(self.page_bytes, 1))
            while len(self.ram) > max_blocks:
                old, pay = self.ram.popitem(last=False)
                self._to_disk(old, pay)
        else:
            self._to_disk(h, payload)

    def _disk_path(self, h: bytes) -> str:
        return os.path.join(self.cfg.disk_dir, f"{self.file_prefix}_{h.hex()}.kvblk")

    def _to_disk(self, h: bytes, payload: torch.Tensor) -> None:
        if not (self.cfg.disk_dir and self.cfg.disk_budget_mb > 0):
            self._stats["dropped"] += 1
            return
        path = self._disk_path(h)
        tmp = f"{path}.{os.getpid()}.tmp"                # a reader never sees a half-written file
        torch.save(payload.cpu(), tmp)
        os.replace(tmp, path)
        self.disk[h] = os.path.getsize(path)
        self._stats["evicted_to_disk"] += 1
        budget = self.cfg.disk_budget_mb * (1 << 20)
        while sum(self.disk.values()) > budget and len(self.disk) > 1:
            old, _ = self.disk.popitem(last=False)
            try:
                os.remove(self._disk_path(old))
            except OSError:
                pass
            self._stats["dropped"] += 1
