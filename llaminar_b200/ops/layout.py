"""Load-time reorder of GGUF block-quantised matrices into the tile-major layout the kernels read.

The bits of every block are preserved; only their order in memory changes.  A matrix
``W[N, K]`` (N padded to a multiple of 128, K a multiple of 256) becomes an array of
*chunks* indexed ``[n_tile][k_block]``, one chunk = 128 rows x 256 columns.  Inside a chunk
each field of the block struct is stored as its own *plane* (all 128 rows of ``qs``, then all
rows of ``scales`` ...), which makes every chunk and every plane 16-byte aligned even for the
110/210/34-byte block formats, so a chunk can be fetched with one bulk copy.  Planes with at
least 16 bytes per row are stored ``[4 row groups][16-byte unit][32 rows][16 bytes]``: one
warp-wide 16-byte load fetches the same unit of 32 consecutive rows (coalesced), and lane ==
row, so a GEMV needs no cross-lane reduction and a GEMM's dequant warps write 32 different rows
of the swizzled MMA operand tile without bank conflicts.  Smaller planes are ``[128 rows][R]``.

(The reference repacks GGUF blocks into its own "NativeVNNI" structure-of-arrays layout at load
time for the same reason: src/v2/kernels/cuda/gemm/CUDAWeightPacker.cpp:44-109.)
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..gguf.constants import BLOCK_GEOMETRY, GGMLType

TILE_N = 128
TILE_K = 256

# format ids shared with the CUDA side (csrc/formats.cuh)
FMT_IDS = {GGMLType.Q4_K: 0, GGMLType.Q5_K: 1, GGMLType.Q6_K: 2, GGMLType.Q8_0: 3, GGMLType.Q4_0: 4,
           GGMLType.IQ3_S: 5}

# planes per format: (byte offset inside the 256-element block group, bytes per row)
# for the 32-element formats the 8 blocks of a 256-column group are de-interleaved first
_PLANES = {
    GGMLType.Q4_K: [(16, 128), (0, 16)],                         # qs | d,dmin,scales[12]
    GGMLType.Q5_K: [(48, 128), (16, 32), (0, 16)],               # qs | qh | d,dmin,scales[12]
    GGMLType.Q6_K: [(0, 128), (128, 64), (192, 16), (208, 2)],   # ql | qh | scales | d
    GGMLType.IQ3_S: [(2, 64), (74, 32), (66, 8), (106, 4), (0, 2)],   # qs | signs | qh | scales | d
}


def chunk_bytes(qtype: GGMLType) -> int:
    e, b = BLOCK_GEOMETRY[qtype]
    return TILE_N * (TILE_K // e) * b


@dataclass
class PackedWeight:
    """A quantised matrix (or stack of expert matrices) in chunk layout on the device."""
    fmt: int                    # FMT_IDS value
    qtype: GGMLType
    n: int                      # logical rows
    k: int                      # logical columns
    n_tiles: int
    k_blocks: int
    data: torch.Tensor          # uint8 [experts?][n_tiles * k_blocks * chunk_bytes]
    n_experts: int = 0

    @property
    def chunk_bytes(self) -> int:
        return chunk_bytes(self.qtype)

    def nbytes(self) -> int:
        return self.data.numel()


def _planes_of(qtype: GGMLType, blocks: torch.Tensor) -> list[torch.Tensor]:
    """blocks: [N, KB, bytes per 256 columns] -> list of [N, KB, R] planes."""
    n, kb, _ = blocks.shape
    if qtype in _PLANES:
        return [blocks[:, :, off:off + r] for off, r in _PLANES[qtype]]
    if qtype == GGMLType.Q8_0:
        v = blocks.reshape(n, kb, 8, 34)
        return [v[..., 2:].reshape(n, kb, 256), v[..., :2].reshape(n, kb, 16)]
    if qtype == GGMLType.Q4_0:
        v = blocks.reshape(n, kb, 8, 18)
        return [v[..., 2:].reshape(n, kb, 128), v[..., :2].reshape(n, kb, 16)]
    raise NotImplementedError(qtype)


Q4K_MAX_D = 0.5 / 63          # the small-batch GEMM multiplies d * sc by 2^129 in bf16: d * sc must stay below 0.5


def q4k_scales_in_range(raw: torch.Tensor) -> bool:
    """Whether every super-block scale ``d`` of a Q4_K tensor is small enough for the small-batch GEMM's conversion
    (csrc/formats_smem.cuh: DequantAtomQ4KRt).  Real checkpoints are two orders of magnitude below the limit (it allows
    weights up to about +-7); a tensor that is not gets re-encoded by the loader instead of silently losing range."""
    d = raw.reshape(-1, 144)[:, :2].contiguous().view(torch.float16).float().abs()
    d = torch.nan_to_num(d, nan=float("inf"))
    return bool((d.max() <= Q4K_MAX_D).item()) if d.numel() else True


def can_pack(qtype: GGMLType, k: int) -> bool:
    return qtype in FMT_IDS and k % TILE_K == 0


def pack_matrix(raw: torch.Tensor, qtype: GGMLType, n: int, k: int) -> PackedWeight:
    """raw: flat uint8 GGUF bytes of W[n, k] (row-major blocks) -> chunk layout (same device)."""
    qtype = GGMLType(qtype)
    if not can_pack(qtype, k):
        raise ValueError(f"cannot tile {qtype.name} with k={k}")
    e, b = BLOCK_GEOMETRY[qtype]
    grp = TILE_K // e * b
    kb = k // TILE_K
    nt = (n + TILE_N - 1) // TILE_N
    blocks = raw.reshape(n, kb, grp)
    if nt * TILE_N != n:
        pad = torch.zeros(nt * TILE_N - n, kb, grp, dtype=torch.uint8, device=raw.device)
        blocks = torch.cat([blocks, pad], dim=0)
    outs = []
    for plane in _planes_of(qtype, blocks):
        r = plane.shape[-1]
        if r >= 16:
            p = plane.reshape(nt, 4, 32, kb, r // 16, 16).permute(0, 3, 1, 4, 2, 5)
        else:
            p = plane.reshape(nt, TILE_N, kb, r).permute(0, 2, 1, 3)
        outs.append(p.reshape(nt, kb, TILE_N * r))
    data = torch.cat(outs, dim=2).contiguous().reshape(-1)
    assert data.numel() == nt * kb * chunk_bytes(qtype)
    return PackedWeight(FMT_IDS[qtype], qtype, n, k, nt, kb, data)


def pack_experts(raw: torch.Tensor, qtype: GGMLType, n_experts: int, n: int, k: int) -> PackedWeight:
    per = raw.numel() // n_experts
    parts = [pack_matrix(raw[e * per:(e + 1) * per], qtype, n, k) for e in range(n_experts)]
    p0 = parts[0]
    data = torch.stack([p.data for p in parts])
    return PackedWeight(p0.fmt, p0.qtype, n, k, p0.n_tiles, p0.k_blocks, data, n_experts)


def concat_rows(parts: list[tuple[torch.Tensor, GGMLType, int, int]]) -> tuple[torch.Tensor, GGMLType, int, int]:
    """Stack several [n_i, k] matrices of the same format row-wise (fused QKV / gate|up weights)."""
    qt, k = parts[0][1], parts[0][3]
    for _, q, _, kk in parts:
        if q != qt or kk != k:
            raise ValueError("row-concatenated matrices must share format and K")
    return torch.cat([p[0].reshape(-1) for p in parts]), qt, sum(p[2] for p in parts), k


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, qtype: GGMLType, n: int, k: int):
    """Row order for the fused SwiGLU epilogue: 16 gate rows, then the 16 up rows of the same outputs.

    A kernel warp owns 32 consecutive fused rows (lane == row), so gate and up of one output column
    sit in lanes l and l + 16 of the same warp and are combined with one shuffle."""
    if n % 16:
        raise ValueError("gate/up row count must be a multiple of 16")
    e, b = BLOCK_GEOMETRY[qtype]
    rb = k // e * b
    g = gate.reshape(n // 16, 16, rb)
    u = up.reshape(n // 16, 16, rb)
    return torch.stack([g, u], dim=1).reshape(-1), qtype, 2 * n, k
