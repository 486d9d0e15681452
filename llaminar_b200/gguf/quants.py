"""Block codecs for GGUF quantised tensors, written with torch ops (CPU or CUDA).

Every codec works on a ``[n_blocks, block_bytes]`` uint8 tensor and produces /
consumes ``[n_blocks, block_elems]`` float32.  They are the numerical oracle for the
CUDA kernels and the quantisers behind the synthetic-model generator, so they run on
whatever device the input lives on.

Bit layouts are those of the ggml block structs (reference:
src/v2/tensors/BlockStructures.h:32-590; the reference's NumPy oracle lives in
python/reference/loaders/dequantize.py).  The quantisers here are simple
min/max-fit encoders: they emit valid blocks but do not reproduce ggml's iterative
scale search.
"""
from __future__ import annotations

import torch

from .constants import BLOCK_GEOMETRY, GGMLType
from .iq_tables import (IQ1_DELTA, IQ1_LEVELS, IQ1S_GRID_CODES, IQ2_LEVELS, IQ2S_GRID_CODES, IQ2XS_GRID_CODES, IQ2XXS_GRID_CODES,
                        IQ3_S_GRID, IQ3_XXS_GRID, IQ4_NL_VALUES, unpack_codes)

_TABLE_CACHE: dict[tuple[str, str], torch.Tensor] = {}


def _table(name: str, device: torch.device) -> torch.Tensor:
    key = (name, str(device))
    t = _TABLE_CACHE.get(key)
    if t is None:
        if name == "iq4nl":
            t = torch.tensor(IQ4_NL_VALUES, dtype=torch.float32, device=device)
        elif name in ("iq3s", "iq3xxs"):
            src = IQ3_S_GRID if name == "iq3s" else IQ3_XXS_GRID
            packed = torch.tensor(src, dtype=torch.int64, device=device)
            t = torch.stack([(packed >> (8 * i)) & 0xFF for i in range(4)], dim=-1).to(torch.float32)
        elif name in ("iq2xxs", "iq2xs", "iq2s", "iq1s"):
            src = {"iq2xxs": IQ2XXS_GRID_CODES, "iq2xs": IQ2XS_GRID_CODES, "iq2s": IQ2S_GRID_CODES, "iq1s": IQ1S_GRID_CODES}[name]
            t = torch.tensor(unpack_codes(src, IQ1_LEVELS if name == "iq1s" else IQ2_LEVELS), dtype=torch.float32, device=device)
        else:
            raise KeyError(name)
        _TABLE_CACHE[key] = t
    return t


def _f16_at(blocks: torch.Tensor, off: int) -> torch.Tensor:
    """Read the little-endian fp16 at byte offset ``off`` of every block -> float32 [n, 1]."""
    return blocks[:, off:off + 2].contiguous().view(torch.float16).to(torch.float32)


def _f16_bytes(x: torch.Tensor) -> torch.Tensor:
    """float32 [n] or [n, 1] -> uint8 [n, 2] holding the fp16 encoding."""
    return x.reshape(-1, 1).to(torch.float16).contiguous().view(torch.uint8).reshape(-1, 2)


def _i(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.int32)


# ----------------------------------------------------------------------------------------
# simple 32-element formats
# ----------------------------------------------------------------------------------------

def dequant_q8_0(b: torch.Tensor) -> torch.Tensor:
    d = _f16_at(b, 0)
    q = b[:, 2:34].contiguous().view(torch.int8).to(torch.float32)
    return d * q


def quant_q8_0(x: torch.Tensor) -> torch.Tensor:
    amax = x.abs().amax(dim=1, keepdim=True)
    d = amax / 127.0
    dh = d.to(torch.float16)
    inv = torch.where(dh > 0, 1.0 / dh.to(torch.float32), torch.zeros_like(d))
    q = torch.round(x * inv).clamp_(-127, 127).to(torch.int8)
    return torch.cat([dh.contiguous().view(torch.uint8).reshape(-1, 2), q.view(torch.uint8)], dim=1)


def dequant_q4_0(b: torch.Tensor) -> torch.Tensor:
    d = _f16_at(b, 0)
    qs = _i(b[:, 2:18])
    q = torch.cat([qs & 0xF, qs >> 4], dim=1).to(torch.float32) - 8.0
    return d * q


def quant_q4_0(x: torch.Tensor) -> torch.Tensor:
    idx = x.abs().argmax(dim=1, keepdim=True)
    mx = torch.gather(x, 1, idx)
    d = (mx / -8.0).to(torch.float16)
    df = d.to(torch.float32)
    inv = torch.where(df != 0, 1.0 / df, torch.zeros_like(df))
    q = torch.clamp(torch.floor(x * inv + 8.5), 0, 15).to(torch.uint8)
    packed = q[:, :16] | (q[:, 16:] << 4)
    return torch.cat([d.contiguous().view(torch.uint8).reshape(-1, 2), packed], dim=1)


def dequant_q4_1(b: torch.Tensor) -> torch.Tensor:
    d, m = _f16_at(b, 0), _f16_at(b, 2)
    qs = _i(b[:, 4:20])
    q = torch.cat([qs & 0xF, qs >> 4], dim=1).to(torch.float32)
    return d * q + m


def _q5_high_bits(b: torch.Tensor, off: int) -> torch.Tensor:
    qh = b[:, off:off + 4].to(torch.int64)
    word = qh[:, 0] | (qh[:, 1] << 8) | (qh[:, 2] << 16) | (qh[:, 3] << 24)
    shifts = torch.arange(32, device=b.device, dtype=torch.int64)
    return ((word[:, None] >> shifts[None, :]) & 1).to(torch.int32)


def dequant_q5_0(b: torch.Tensor) -> torch.Tensor:
    d = _f16_at(b, 0)
    hb = _q5_high_bits(b, 2)
    qs = _i(b[:, 6:22])
    q = torch.cat([qs & 0xF, qs >> 4], dim=1) | (hb << 4)
    return d * (q.to(torch.float32) - 16.0)


def dequant_q5_1(b: torch.Tensor) -> torch.Tensor:
    d, m = _f16_at(b, 0), _f16_at(b, 2)
    hb = _q5_high_bits(b, 4)
    qs = _i(b[:, 8:24])
    q = torch.cat([qs & 0xF, qs >> 4], dim=1) | (hb << 4)
    return d * q.to(torch.float32) + m


def dequant_iq4_nl(b: torch.Tensor) -> torch.Tensor:
    d = _f16_at(b, 0)
    qs = b[:, 2:18].to(torch.int64)
    idx = torch.cat([qs & 0xF, qs >> 4], dim=1)
    return d * _table("iq4nl", b.device)[idx]


# ----------------------------------------------------------------------------------------
# K-quants (256-element super-blocks)
# ----------------------------------------------------------------------------------------

def _unpack_k4_scales(sc12: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """12 packed bytes -> (8 six-bit scales, 8 six-bit mins), both int32 [n, 8]."""
    s = _i(sc12)
    sc_lo, m_lo = s[:, 0:4] & 63, s[:, 4:8] & 63
    sc_hi = (s[:, 8:12] & 0xF) | ((s[:, 0:4] >> 6) << 4)
    m_hi = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
    return torch.cat([sc_lo, sc_hi], dim=1), torch.cat([m_lo, m_hi], dim=1)


def _pack_k4_scales(sc: torch.Tensor, mn: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`_unpack_k4_scales`; inputs int32 [n, 8] in [0, 63]."""
    out = torch.empty(sc.shape[0], 12, dtype=torch.int32, device=sc.device)
    out[:, 0:4] = (sc[:, 0:4] & 63) | ((sc[:, 4:8] >> 4) << 6)
    out[:, 4:8] = (mn[:, 0:4] & 63) | ((mn[:, 4:8] >> 4) << 6)
    out[:, 8:12] = (sc[:, 4:8] & 0xF) | ((mn[:, 4:8] & 0xF) << 4)
    return out.to(torch.uint8)


def dequant_q4_k(b: torch.Tensor) -> torch.Tensor:
    n = b.shape[0]
    d, dmin = _f16_at(b, 0), _f16_at(b, 2)
    sc, mn = _unpack_k4_scales(b[:, 4:16])
    qs = _i(b[:, 16:144]).reshape(n, 4, 32)
    q = torch.stack([qs & 0xF, qs >> 4], dim=2).reshape(n, 8, 32).to(torch.float32)
    scale = (d * sc.to(torch.float32)).unsqueeze(-1)
    minv = (dmin * mn.to(torch.float32)).unsqueeze(-1)
    return (scale * q - minv).reshape(n, 256)


def _fit_k_scale_min(x: torch.Tensor, nmax: int):
    """Per-sub-block affine fit x ~= s*q - m with q in [0, nmax], m >= 0.  x: [n, 8, 32]."""
    lo = x.amin(dim=2).clamp(max=0.0)
    hi = x.amax(dim=2).clamp(min=0.0)
    s = (hi - lo) / float(nmax)
    return s, -lo


def _quant_k_affine(x: torch.Tensor, nmax: int):
    n = x.shape[0]
    xs = x.reshape(n, 8, 32)
    s, m = _fit_k_scale_min(xs, nmax)
    d = (s.amax(dim=1, keepdim=True) / 63.0).to(torch.float16)
    dmin = (m.amax(dim=1, keepdim=True) / 63.0).to(torch.float16)
    df, dmf = d.to(torch.float32), dmin.to(torch.float32)
    sc = torch.where(df > 0, torch.round(s / df.clamp(min=1e-30)), torch.zeros_like(s)).clamp_(0, 63)
    mn = torch.where(dmf > 0, torch.round(m / dmf.clamp(min=1e-30)), torch.zeros_like(m)).clamp_(0, 63)
    eff_s = (df * sc).unsqueeze(-1)
    eff_m = (dmf * mn).unsqueeze(-1)
    q = torch.where(eff_s > 0, torch.round((xs + eff_m) / eff_s.clamp(min=1e-30)), torch.zeros_like(xs))
    q = q.clamp_(0, nmax).to(torch.int32)
    return d, dmin, sc.to(torch.int32), mn.to(torch.int32), q


def quant_q4_k(x: torch.Tensor) -> torch.Tensor:
    n = x.shape[0]
    d, dmin, sc, mn, q = _quant_k_affine(x, 15)
    q = q.reshape(n, 4, 2, 32)
    qs = (q[:, :, 0, :] | (q[:, :, 1, :] << 4)).to(torch.uint8).reshape(n, 128)
    return torch.cat([_f16_bytes(d), _f16_bytes(dmin), _pack_k4_scales(sc, mn), qs], dim=1)


def dequant_q5_k(b: torch.Tensor) -> torch.Tensor:
    n = b.shape[0]
    d, dmin = _f16_at(b, 0), _f16_at(b, 2)
    sc, mn = _unpack_k4_scales(b[:, 4:16])
    qh = _i(b[:, 16:48])  # [n, 32]
    qs = _i(b[:, 48:176]).reshape(n, 4, 32)
    shifts = torch.arange(8, device=b.device, dtype=torch.int32)
    hb = ((qh[:, None, :] >> shifts[None, :, None]) & 1)  # [n, 8, 32]: bit s of qh[l] -> sub-block s
    q = torch.stack([qs & 0xF, qs >> 4], dim=2).reshape(n, 8, 32) | (hb << 4)
    scale = (d * sc.to(torch.float32)).unsqueeze(-1)
    minv = (dmin * mn.to(torch.float32)).unsqueeze(-1)
    return (scale * q.to(torch.float32) - minv).reshape(n, 256)


def quant_q5_k(x: torch.Tensor) -> torch.Tensor:
    n = x.shape[0]
    d, dmin, sc, mn, q = _quant_k_affine(x, 31)  # q: [n, 8, 32]
    lo = (q & 0xF).reshape(n, 4, 2, 32)
    qs = (lo[:, :, 0, :] | (lo[:, :, 1, :] << 4)).to(torch.uint8).reshape(n, 128)
    shifts = torch.arange(8, device=x.device, dtype=torch.int32)
    qh = (((q >> 4) & 1) << shifts[None, :, None]).sum(dim=1).to(torch.uint8)  # [n, 32]
    return torch.cat([_f16_bytes(d), _f16_bytes(dmin), _pack_k4_scales(sc, mn), qh, qs], dim=1)


def dequant_q6_k(b: torch.Tensor) -> torch.Tensor:
    n = b.shape[0]
    ql = _i(b[:, 0:128]).reshape(n, 2, 2, 32)   # [half, which 32-byte run, l]
    qh = _i(b[:, 128:192]).reshape(n, 2, 32)
    sc = b[:, 192:208].contiguous().view(torch.int8).to(torch.float32).reshape(n, 2, 8)
    d = _f16_at(b, 208)
    q1 = (ql[:, :, 0, :] & 0xF) | (((qh >> 0) & 3) << 4)
    q2 = (ql[:, :, 1, :] & 0xF) | (((qh >> 2) & 3) << 4)
    q3 = (ql[:, :, 0, :] >> 4) | (((qh >> 4) & 3) << 4)
    q4 = (ql[:, :, 1, :] >> 4) | (((qh >> 6) & 3) << 4)
    q = torch.stack([q1, q2, q3, q4], dim=2).to(torch.float32) - 32.0   # [n, 2, 4, 32]
    # 16-element sub-blocks: scale index inside a half = 2*group + (l // 16)
    scale = sc.reshape(n, 2, 4, 2).unsqueeze(-1).expand(n, 2, 4, 2, 16).reshape(n, 2, 4, 32)
    return (d.reshape(n, 1, 1, 1) * scale * q).reshape(n, 256)


def quant_q6_k(x: torch.Tensor) -> torch.Tensor:
    n = x.shape[0]
    xs = x.reshape(n, 16, 16)
    amax_idx = xs.abs().argmax(dim=2, keepdim=True)
    mx = torch.gather(xs, 2, amax_idx).squeeze(-1)           # signed extreme of each sub-block
    s = mx / -32.0                                           # per sub-block scale (signed)
    d = (s.abs().amax(dim=1, keepdim=True) / 127.0).to(torch.float16)
    df = d.to(torch.float32)
    sc = torch.where(df > 0, torch.round(s / df.clamp(min=1e-30)), torch.zeros_like(s)).clamp_(-128, 127)
    eff = (df * sc).unsqueeze(-1)
    q = torch.where(eff != 0, torch.round(xs / torch.where(eff != 0, eff, torch.ones_like(eff))),
                    torch.zeros_like(xs))
    q = (q.clamp_(-32, 31) + 32).to(torch.int32).reshape(n, 2, 4, 32)
    ql0 = (q[:, :, 0, :] & 0xF) | ((q[:, :, 2, :] & 0xF) << 4)
    ql1 = (q[:, :, 1, :] & 0xF) | ((q[:, :, 3, :] & 0xF) << 4)
    ql = torch.stack([ql0, ql1], dim=2).reshape(n, 128).to(torch.uint8)
    qh = ((q[:, :, 0, :] >> 4) | ((q[:, :, 1, :] >> 4) << 2) | ((q[:, :, 2, :] >> 4) << 4)
          | ((q[:, :, 3, :] >> 4) << 6)).reshape(n, 64).to(torch.uint8)
    return torch.cat([ql, qh, sc.to(torch.int8).view(torch.uint8), _f16_bytes(d)], dim=1)


def dequant_q2_k(b: torch.Tensor) -> torch.Tensor:
    n = b.shape[0]
    scales = _i(b[:, 0:16])
    qs = _i(b[:, 16:80]).reshape(n, 2, 32)
    d, dmin = _f16_at(b, 80), _f16_at(b, 82)
    shifts = torch.arange(4, device=b.device, dtype=torch.int32) * 2
    q = ((qs[:, :, None, :] >> shifts[None, None, :, None]) & 3).to(torch.float32)  # [n, 2, 4, 32]
    sc = (scales & 0xF).to(torch.float32).reshape(n, 2, 4, 2)
    mn = (scales >> 4).to(torch.float32).reshape(n, 2, 4, 2)
    sc = sc.unsqueeze(-1).expand(n, 2, 4, 2, 16).reshape(n, 2, 4, 32)
    mn = mn.unsqueeze(-1).expand(n, 2, 4, 2, 16).reshape(n, 2, 4, 32)
    d4, m4 = d.reshape(n, 1, 1, 1), dmin.reshape(n, 1, 1, 1)
    return (d4 * sc * q - m4 * mn).reshape(n, 256)


def dequant_q3_k(b: torch.Tensor) -> torch.Tensor:
    n = b.shape[0]
    hmask = _i(b[:, 0:32])
    qs = _i(b[:, 32:96]).reshape(n, 2, 32)
    s = _i(b[:, 96:108])
    d = _f16_at(b, 108)
    # 16 six-bit scales: low 4 bits in bytes 0..7 (two per byte), high 2 bits in bytes 8..11
    low = torch.cat([s[:, 0:8] & 0xF, s[:, 0:8] >> 4], dim=1)                        # [n, 16]
    hi_src = s[:, 8:12]
    high = torch.cat([(hi_src >> (2 * k)) & 3 for k in range(4)], dim=1)              # [n, 16]
    sc = ((low | (high << 4)) - 32).to(torch.float32)
    shifts = torch.arange(4, device=b.device, dtype=torch.int32) * 2
    q = (qs[:, :, None, :] >> shifts[None, None, :, None]) & 3                       # [n, 2, 4, 32]
    bit = torch.arange(8, device=b.device, dtype=torch.int32).reshape(1, 2, 4, 1)
    hb = (hmask[:, None, None, :] >> bit) & 1
    q = (q - torch.where(hb == 1, 0, 4)).to(torch.float32)
    scale = sc.reshape(n, 2, 4, 2).unsqueeze(-1).expand(n, 2, 4, 2, 16).reshape(n, 2, 4, 32)
    return (d.reshape(n, 1, 1, 1) * scale * q).reshape(n, 256)


# ----------------------------------------------------------------------------------------
# IQ formats
# ----------------------------------------------------------------------------------------

def dequant_iq4_xs(b: torch.Tensor) -> torch.Tensor:
    n = b.shape[0]
    d = _f16_at(b, 0)
    sh = _i(b[:, 2:3]) | (_i(b[:, 3:4]) << 8)             # scales_h, [n, 1]
    sl = _i(b[:, 4:8])                                     # [n, 4]
    qs = b[:, 8:136].to(torch.int64).reshape(n, 8, 16)
    ib = torch.arange(8, device=b.device, dtype=torch.int32)
    low = (sl[:, ib // 2] >> (4 * (ib % 2))[None, :]) & 0xF
    high = (sh >> (2 * ib)[None, :]) & 3
    dl = d * ((low | (high << 4)) - 32).to(torch.float32)  # [n, 8]
    idx = torch.cat([qs & 0xF, qs >> 4], dim=2)            # [n, 8, 32]
    return (dl.unsqueeze(-1) * _table("iq4nl", b.device)[idx]).reshape(n, 256)


def dequant_iq3_s(b: torch.Tensor) -> torch.Tensor:
    n = b.shape[0]
    dev = b.device
    d = _f16_at(b, 0)
    qs = b[:, 2:66].to(torch.int64).reshape(n, 8, 8)       # [sub-block of 32, 8 index bytes]
    qh = b[:, 66:74].to(torch.int64)                       # [n, 8]
    signs = b[:, 74:106].to(torch.int64).reshape(n, 8, 4)  # one sign byte per 8 elements
    scales = _i(b[:, 106:110])
    ib = torch.arange(8, device=dev, dtype=torch.int32)
    s4 = (scales[:, ib // 2] >> (4 * (ib % 2))[None, :]) & 0xF
    db = d * (1 + 2 * s4).to(torch.float32)                # [n, 8]
    bitpos = torch.arange(8, device=dev, dtype=torch.int64)
    hi = ((qh[:, :, None] >> bitpos[None, None, :]) & 1) << 8
    idx = qs | hi                                          # [n, 8, 8] nine-bit grid indices
    mag = _table("iq3s", dev)[idx]                         # [n, 8, 8, 4]
    mag = mag.reshape(n, 8, 4, 8)                          # two grid entries per sign byte
    sb = (signs[:, :, :, None] >> bitpos[None, None, None, :]) & 1
    sign = 1.0 - 2.0 * sb.to(torch.float32)
    return (db[:, :, None, None] * mag * sign).reshape(n, 256)


def quant_iq3_s(x: torch.Tensor) -> torch.Tensor:
    """Nearest-grid-point IQ3_S encoder (per 32-element sub-block scale fit)."""
    n = x.shape[0]
    dev = x.device
    xs = x.reshape(n, 8, 32)
    amax = xs.abs().amax(dim=2)                            # [n, 8]
    want = amax / 13.0                                     # map the extreme near the top grid value
    d = (want.amax(dim=1, keepdim=True) / 31.0).to(torch.float16)
    df = d.to(torch.float32)
    s4 = torch.where(df > 0, torch.round((want / df.clamp(min=1e-30) - 1.0) * 0.5),
                     torch.zeros_like(want)).clamp_(0, 15)
    db = df * (1 + 2 * s4)
    mags = (xs.abs() / db.clamp(min=1e-30).unsqueeze(-1)).reshape(n * 64, 4)
    grid = _table("iq3s", dev)                             # [512, 4]
    g2 = (grid * grid).sum(dim=1)
    idx = torch.empty(n * 64, dtype=torch.int64, device=dev)
    step = 1 << 20
    for s in range(0, n * 64, step):
        chunk = mags[s:s + step]
        idx[s:s + step] = (g2[None, :] - 2.0 * (chunk @ grid.T)).argmin(dim=1)
    idx = idx.reshape(n, 8, 8)
    qs = (idx & 0xFF).to(torch.uint8).reshape(n, 64)
    bitpos = torch.arange(8, device=dev, dtype=torch.int64)
    qh = (((idx >> 8) & 1) << bitpos[None, None, :]).sum(dim=2).to(torch.uint8)          # [n, 8]
    neg = (xs < 0).to(torch.int64).reshape(n, 8, 4, 8)
    signs = (neg << bitpos[None, None, None, :]).sum(dim=3).to(torch.uint8).reshape(n, 32)
    s4i = s4.to(torch.int32)
    scales = (s4i[:, 0::2] | (s4i[:, 1::2] << 4)).to(torch.uint8)
    return torch.cat([_f16_bytes(d), qs, qh, signs, scales], dim=1)


def dequant_iq3_xxs(b: torch.Tensor) -> torch.Tensor:
    n = b.shape[0]
    dev = b.device
    d = _f16_at(b, 0)
    qs = b[:, 2:66].to(torch.int64).reshape(n, 8, 8)
    aux = b[:, 66:98].to(torch.int64).reshape(n, 8, 4)
    word = aux[:, :, 0] | (aux[:, :, 1] << 8) | (aux[:, :, 2] << 16) | (aux[:, :, 3] << 24)
    db = d * (0.5 + (word >> 28).to(torch.float32)) * 0.5
    mag = _table("iq3xxs", dev)[qs].reshape(n, 8, 4, 8)
    l = torch.arange(4, device=dev, dtype=torch.int64)
    s7 = (word[:, :, None] >> (7 * l)[None, None, :]) & 127                       # [n, 8, 4]
    # the 8th sign bit makes the popcount even
    par = s7 ^ (s7 >> 4)
    par = par ^ (par >> 2)
    par = (par ^ (par >> 1)) & 1
    s8 = s7 | (par << 7)
    bitpos = torch.arange(8, device=dev, dtype=torch.int64)
    sb = (s8[:, :, :, None] >> bitpos[None, None, None, :]) & 1
    sign = 1.0 - 2.0 * sb.to(torch.float32)
    return (db[:, :, None, None] * mag * sign).reshape(n, 256)


# ----------------------------------------------------------------------------------------
# 2-bit and 1-bit codebook formats (eight elements per codebook entry)
# ----------------------------------------------------------------------------------------

def _u16(b: torch.Tensor) -> torch.Tensor:
    """uint8 [n, 2m] -> little-endian 16-bit words as int64 [n, m]."""
    w = b.to(torch.int64)
    return w[:, 0::2] | (w[:, 1::2] << 8)


def _signs_from_7bit(s7: torch.Tensor) -> torch.Tensor:
    """7 stored sign bits -> +-1.0 for eight elements [..., 8]; the eighth bit makes the number of set bits even."""
    par = s7 ^ (s7 >> 4)
    par = par ^ (par >> 2)
    par = (par ^ (par >> 1)) & 1
    return _signs_from_byte(s7 | (par << 7))


def _signs_from_byte(s8: torch.Tensor) -> torch.Tensor:
    bitpos = torch.arange(8, device=s8.device, dtype=torch.int64)
    return 1.0 - 2.0 * ((s8[..., None] >> bitpos) & 1).to(torch.float32)


def dequant_iq2_xxs(b: torch.Tensor) -> torch.Tensor:
    """66 bytes: fp16 d, then per 32 elements two 32-bit words: four 8-bit codebook indices; 4 x 7 sign bits + 4-bit scale."""
    n = b.shape[0]
    d = _f16_at(b, 0)
    w = _u16(b[:, 2:66]).reshape(n, 8, 4)
    idx = torch.stack([w[:, :, 0] & 0xFF, w[:, :, 0] >> 8, w[:, :, 1] & 0xFF, w[:, :, 1] >> 8], dim=-1)       # [n, 8, 4]
    hi = w[:, :, 2] | (w[:, :, 3] << 16)
    db = d * (0.5 + (hi >> 28).to(torch.float32)) * 0.25                                                       # [n, 8]
    l = torch.arange(4, device=b.device, dtype=torch.int64)
    sign = _signs_from_7bit((hi[:, :, None] >> (7 * l)) & 127)                                                 # [n, 8, 4, 8]
    return (db[:, :, None, None] * _table("iq2xxs", b.device)[idx] * sign).reshape(n, 256)


def dequant_iq2_xs(b: torch.Tensor) -> torch.Tensor:
    """74 bytes: fp16 d, 32 words (9-bit codebook index + 7 sign bits, one per 8 elements), 8 bytes of two 4-bit scales
    (low nibble: first 16 elements of the group of 32, high nibble: the other 16)."""
    n = b.shape[0]
    d = _f16_at(b, 0)
    q = _u16(b[:, 2:66]).reshape(n, 8, 4)
    sc = b[:, 66:74].to(torch.int64)
    ls = torch.stack([sc & 0xF, sc & 0xF, sc >> 4, sc >> 4], dim=-1).to(torch.float32)                         # [n, 8, 4]
    db = d[:, :, None] * (0.5 + ls) * 0.25
    return (db[..., None] * _table("iq2xs", b.device)[q & 511] * _signs_from_7bit(q >> 9)).reshape(n, 256)


def dequant_iq2_s(b: torch.Tensor) -> torch.Tensor:
    """82 bytes: fp16 d, 32 index low bytes, 32 full sign bytes, 8 bytes of index bits 8-9 (two per 8 elements), 8 bytes
    of two 4-bit scales."""
    n = b.shape[0]
    d = _f16_at(b, 0)
    lo = b[:, 2:34].to(torch.int64).reshape(n, 8, 4)
    sg = b[:, 34:66].to(torch.int64).reshape(n, 8, 4)
    qh = b[:, 66:74].to(torch.int64)
    sc = b[:, 74:82].to(torch.int64)
    l = torch.arange(4, device=b.device, dtype=torch.int64)
    idx = lo | (((qh[:, :, None] >> (2 * l)) & 3) << 8)
    ls = torch.stack([sc & 0xF, sc & 0xF, sc >> 4, sc >> 4], dim=-1).to(torch.float32)
    db = d[:, :, None] * (0.5 + ls) * 0.25
    return (db[..., None] * _table("iq2s", b.device)[idx] * _signs_from_byte(sg)).reshape(n, 256)


def dequant_iq1_s(b: torch.Tensor) -> torch.Tensor:
    """50 bytes: fp16 d, 32 index low bytes, 8 words: 4 x 3 index high bits, a 3-bit scale (bits 12-14) and the sign of the
    common offset (bit 15).  Elements are d * (2 s + 1) * (codebook value +- 1/8)."""
    n = b.shape[0]
    d = _f16_at(b, 0)
    lo = b[:, 2:34].to(torch.int64).reshape(n, 8, 4)
    qh = _u16(b[:, 34:50])                                                                                      # [n, 8]
    l = torch.arange(4, device=b.device, dtype=torch.int64)
    idx = lo | (((qh[:, :, None] >> (3 * l)) & 7) << 8)
    dl = d * (2.0 * ((qh >> 12) & 7).to(torch.float32) + 1.0)
    delta = torch.where((qh & 0x8000) != 0, -IQ1_DELTA, IQ1_DELTA)
    return (dl[:, :, None, None] * (_table("iq1s", b.device)[idx] + delta[:, :, None, None])).reshape(n, 256)


def dequant_iq1_m(b: torch.Tensor) -> torch.Tensor:
    """56 bytes, no separate d: 32 index low bytes; 16 bytes with, per nibble, 3 index high bits and an offset sign (one
    nibble per 8 elements); 4 scale words whose top nibbles spell the fp16 super-block scale and whose low 12 bits hold
    four 3-bit scales (one per 16 elements)."""
    n = b.shape[0]
    lo = b[:, 0:32].to(torch.int64).reshape(n, 16, 2)
    qh = b[:, 32:48].to(torch.int64)                                                                            # [n, 16]
    sc = _u16(b[:, 48:56])                                                                                      # [n, 4]
    dbits = (sc[:, 0] >> 12) | ((sc[:, 1] >> 8) & 0x00F0) | ((sc[:, 2] >> 4) & 0x0F00) | (sc[:, 3] & 0xF000)
    d = ((dbits ^ 0x8000) - 0x8000).to(torch.int16).view(torch.float16).to(torch.float32)[:, None]      # 16 bits -> fp16
    nib = torch.stack([qh & 0xF, qh >> 4], dim=-1)                                                              # [n, 16, 2]
    idx = lo | ((nib & 7) << 8)
    delta = torch.where((nib & 8) != 0, -IQ1_DELTA, IQ1_DELTA)
    sh = torch.arange(4, device=b.device, dtype=torch.int64) * 3
    s3 = ((sc[:, :, None] >> sh) & 7).reshape(n, 16)                                                            # one per 16 elements
    dl = d * (2.0 * s3.to(torch.float32) + 1.0)
    return (dl[:, :, None, None] * (_table("iq1s", b.device)[idx] + delta[..., None])).reshape(n, 256)


# ----------------------------------------------------------------------------------------
# registry + tensor-level helpers
# ----------------------------------------------------------------------------------------

_DEQUANT = {
    GGMLType.Q8_0: dequant_q8_0, GGMLType.Q4_0: dequant_q4_0, GGMLType.Q4_1: dequant_q4_1,
    GGMLType.Q5_0: dequant_q5_0, GGMLType.Q5_1: dequant_q5_1, GGMLType.IQ4_NL: dequant_iq4_nl,
    GGMLType.Q4_K: dequant_q4_k, GGMLType.Q5_K: dequant_q5_k, GGMLType.Q6_K: dequant_q6_k,
    GGMLType.Q2_K: dequant_q2_k, GGMLType.Q3_K: dequant_q3_k, GGMLType.IQ4_XS: dequant_iq4_xs,
    GGMLType.IQ3_S: dequant_iq3_s, GGMLType.IQ3_XXS: dequant_iq3_xxs,
    GGMLType.IQ2_XXS: dequant_iq2_xxs, GGMLType.IQ2_XS: dequant_iq2_xs, GGMLType.IQ2_S: dequant_iq2_s,
    GGMLType.IQ1_S: dequant_iq1_s, GGMLType.IQ1_M: dequant_iq1_m,
}
_QUANT = {
    GGMLType.Q8_0: quant_q8_0, GGMLType.Q4_0: quant_q4_0, GGMLType.Q4_K: quant_q4_k,
    GGMLType.Q5_K: quant_q5_k, GGMLType.Q6_K: quant_q6_k, GGMLType.IQ3_S: quant_iq3_s,
}

SUPPORTED_DEQUANT = tuple(_DEQUANT) + (GGMLType.F32, GGMLType.F16, GGMLType.BF16)
SUPPORTED_QUANT = tuple(_QUANT) + (GGMLType.F32, GGMLType.F16, GGMLType.BF16)


def dequantize(raw: torch.Tensor, qtype: GGMLType, shape: tuple[int, ...]) -> torch.Tensor:
    """Raw GGUF bytes (flat uint8) of a tensor with logical ``shape`` -> float32 tensor."""
    qtype = GGMLType(qtype)
    raw = raw.reshape(-1)
    if qtype == GGMLType.F32:
        return raw.view(torch.float32).reshape(shape).clone()
    if qtype == GGMLType.F16:
        return raw.view(torch.float16).to(torch.float32).reshape(shape)
    if qtype == GGMLType.BF16:
        return raw.view(torch.bfloat16).to(torch.float32).reshape(shape)
    if qtype not in _DEQUANT:
        raise NotImplementedError(f"no dequantiser for {qtype.name}")
    _, nbytes = BLOCK_GEOMETRY[qtype]
    blocks = raw.reshape(-1, nbytes)
    out = torch.empty(0)
    step = 1 << 18   # bound temporaries for multi-GB tensors
    if blocks.shape[0] <= step:
        out = _DEQUANT[qtype](blocks)
    else:
        out = torch.cat([_DEQUANT[qtype](blocks[s:s + step]) for s in range(0, blocks.shape[0], step)])
    return out.reshape(shape)


def quantize(x: torch.Tensor, qtype: GGMLType) -> torch.Tensor:
    """float tensor (last dim = row) -> flat uint8 tensor of GGUF bytes, rows in order."""
    qtype = GGMLType(qtype)
    if qtype == GGMLType.F32:
        return x.to(torch.float32).contiguous().view(torch.uint8).reshape(-1)
    if qtype == GGMLType.F16:
        return x.to(torch.float16).contiguous().view(torch.uint8).reshape(-1)
    if qtype == GGMLType.BF16:
        return x.to(torch.bfloat16).contiguous().view(torch.uint8).reshape(-1)
    if qtype not in _QUANT:
        raise NotImplementedError(f"no quantiser for {qtype.name}")
    elems, _ = BLOCK_GEOMETRY[qtype]
    if x.shape[-1] % elems:
        raise ValueError(f"{qtype.name}: row length {x.shape[-1]} not a multiple of {elems}")
    blocks = x.to(torch.float32).reshape(-1, elems)
    step = 1 << 18
    if blocks.shape[0] <= step:
        return _QUANT[qtype](blocks).reshape(-1)
    return torch.cat([_QUANT[qtype](blocks[s:s + step]) for s in range(0, blocks.shape[0], step)]).reshape(-1)
