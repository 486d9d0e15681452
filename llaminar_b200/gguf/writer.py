"""GGUF writer: metadata key/values + tensors (already-encoded bytes or float tensors to encode).

Used by the synthetic-model generator and the tests; produces files that the reader in this
package and ggml-compatible tools parse (little-endian, version 3, 32-byte data alignment;
reference for the layout rules: src/v2/loaders/ModelLoader.cpp:2245-2277, :530).
"""
from __future__ import annotations

import struct
from typing import Any

import torch

from .constants import (BLOCK_GEOMETRY, GGUF_DEFAULT_ALIGNMENT, GGUF_MAGIC, GGUF_VERSION,
                        SCALAR_STRUCT, GGMLType, GGUFValueType)
from .quants import quantize


def _pack_string(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _infer_type(v: Any) -> GGUFValueType:
    if isinstance(v, bool):
        return GGUFValueType.BOOL
    if isinstance(v, int):
        return GGUFValueType.UINT32 if 0 <= v < 2 ** 32 else GGUFValueType.INT64
    if isinstance(v, float):
        return GGUFValueType.FLOAT32
    if isinstance(v, str):
        return GGUFValueType.STRING
    if isinstance(v, (list, tuple)):
        return GGUFValueType.ARRAY
    raise TypeError(f"cannot store {type(v)} in GGUF metadata")


def _pack_value(v: Any, vtype: GGUFValueType | None = None) -> tuple[GGUFValueType, bytes]:
    vtype = GGUFValueType(vtype) if vtype is not None else _infer_type(v)
    if vtype == GGUFValueType.STRING:
        return vtype, _pack_string(v)
    if vtype == GGUFValueType.ARRAY:
        items = list(v)
        if items:
            etype = _infer_type(items[0])
            if etype == GGUFValueType.UINT32 and any(isinstance(x, int) and x < 0 for x in items):
                etype = GGUFValueType.INT32
        else:
            etype = GGUFValueType.UINT32
        body = b"".join(_pack_value(x, etype)[1] for x in items)
        return vtype, struct.pack("<IQ", int(etype), len(items)) + body
    return vtype, struct.pack("<" + SCALAR_STRUCT[vtype], v)


class GGUFWriter:
    def __init__(self, alignment: int = GGUF_DEFAULT_ALIGNMENT):
        self.alignment = alignment
        self._kv: list[tuple[str, GGUFValueType, bytes]] = []
        self._tensors: list[tuple[str, GGMLType, tuple[int, ...], torch.Tensor]] = []

    def add(self, key: str, value: Any, vtype: GGUFValueType | None = None) -> None:
        t, payload = _pack_value(value, vtype)
        self._kv.append((key, t, payload))

    def add_raw_tensor(self, name: str, qtype: GGMLType, shape: tuple[int, ...], raw: torch.Tensor) -> None:
        """``raw``: flat uint8 GGUF bytes; ``shape`` in torch order (slowest first)."""
        qtype = GGMLType(qtype)
        elems, nbytes = BLOCK_GEOMETRY[qtype]
        n = 1
        for s in shape:
            n *= s
        if raw.numel() != n // elems * nbytes:
            raise ValueError(f"{name}: {raw.numel()} bytes do not match shape {shape} as {qtype.name}")
        self._tensors.append((name, qtype, tuple(shape), raw.reshape(-1).cpu()))

    def add_tensor(self, name: str, x: torch.Tensor, qtype: GGMLType) -> None:
        self.add_raw_tensor(name, qtype, tuple(x.shape), quantize(x, qtype))

    def write(self, path: str) -> None:
        head = struct.pack("<IIQQ", GGUF_MAGIC, GGUF_VERSION, len(self._tensors), len(self._kv) + 1)
        kv = [_pack_string("general.alignment") + struct.pack("<II", int(GGUFValueType.UINT32), self.alignment)]
        for key, t, payload in self._kv:
            kv.append(_pack_string(key) + struct.pack("<I", int(t)) + payload)
        infos, rel = [], 0
        offsets = []
        for name, qtype, shape, raw in self._tensors:
            ne = tuple(reversed(shape))
            infos.append(_pack_string(name) + struct.pack("<I", len(ne))
                         + b"".join(struct.pack("<Q", d) for d in ne)
                         + struct.pack("<IQ", int(qtype), rel))
            offsets.append(rel)
            rel = (rel + raw.numel() + self.alignment - 1) // self.alignment * self.alignment
        with open(path, "wb") as f:
            f.write(head)
            for b in kv:
                f.write(b)
            for b in infos:
                f.write(b)
            pos = f.tell()
            pad = (-pos) % self.alignment
            f.write(b"\0" * pad)
            base = f.tell()
            for (name, qtype, shape, raw), off in zip(self._tensors, offsets):
                f.seek(base + off)
                f.write(raw.numpy().tobytes())
            end = base + rel
            f.seek(0, 2)
            if f.tell() < end:
                f.write(b"\0" * (end - f.tell()))
