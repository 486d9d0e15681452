"""Memory-mapped GGUF reader.

Parses the header, the key/value metadata (all value types incl. nested arrays) and the
tensor-info table, then exposes every tensor as a zero-copy uint8 view of the mapped file.
Multi-part checkpoints (``name-00001-of-0000N.gguf``) are opened together.

GGUF stores dimensions fastest-varying first (ne0 = columns); ``GGUFTensor.shape`` is
reported slowest-first (torch order), which is the swap the reference performs for 2-D
tensors (reference: src/v2/loaders/ModelLoader.cpp:2245-2277 header, :2490-2496 dim order,
:2658-2723 split files).
"""
from __future__ import annotations

import mmap
import os
import re
import struct
from dataclasses import dataclass
from typing import Any, Iterator

import numpy as np
import torch

from .constants import (BLOCK_GEOMETRY, GGUF_DEFAULT_ALIGNMENT, GGUF_MAGIC, SCALAR_STRUCT,
                        GGMLType, GGUFValueType)
from .quants import dequantize


class GGUFError(ValueError):
    pass


@dataclass
class GGUFTensor:
    name: str
    qtype: GGMLType
    shape: tuple[int, ...]      # torch order: (rows, cols) for 2-D, (experts, rows, cols) for 3-D
    offset: int                 # absolute byte offset inside its file
    nbytes: int
    _buf: Any = None            # the owning mmap (keeps it alive)

    def raw(self) -> torch.Tensor:
        """Zero-copy flat uint8 view of the tensor bytes (read-only mapping)."""
        arr = np.frombuffer(self._buf, dtype=np.uint8, count=self.nbytes, offset=self.offset)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")     # non-writable buffer warning: we never write
            return torch.from_numpy(arr)

    def to_float(self, device: str | torch.device = "cpu") -> torch.Tensor:
        return dequantize(self.raw().to(device), self.qtype, self.shape)

    @property
    def n_elements(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class _Cursor:
    def __init__(self, buf, pos: int = 0):
        self.buf, self.pos = buf, pos

    def unpack(self, fmt: str):
        size = struct.calcsize("<" + fmt)
        if self.pos + size > len(self.buf):
            raise GGUFError("truncated GGUF file")
        v = struct.unpack_from("<" + fmt, self.buf, self.pos)
        self.pos += size
        return v[0] if len(v) == 1 else v

    def string(self) -> str:
        n = self.unpack("Q")
        if self.pos + n > len(self.buf):
            raise GGUFError("truncated GGUF string")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, vtype: int):
        vtype = GGUFValueType(vtype)
        if vtype == GGUFValueType.STRING:
            return self.string()
        if vtype == GGUFValueType.ARRAY:
            etype = GGUFValueType(self.unpack("I"))
            count = self.unpack("Q")
            if etype in SCALAR_STRUCT and etype != GGUFValueType.BOOL:
                fmt = SCALAR_STRUCT[etype]
                size = struct.calcsize("<" + fmt) * count
                arr = np.frombuffer(self.buf, dtype=np.dtype("<" + fmt), count=count, offset=self.pos)
                self.pos += size
                return arr.tolist()
            return [self.value(etype) for _ in range(count)]
        return self.unpack(SCALAR_STRUCT[vtype])


_SPLIT_RE = re.compile(r"^(.*)-(\d{5})-of-(\d{5})\.gguf$")


def split_paths(path: str) -> list[str]:
    """All part files of a split checkpoint, in order (a single path if it is not split)."""
    m = _SPLIT_RE.match(path)
    if not m:
        return [path]
    stem, _, total = m.group(1), m.group(2), int(m.group(3))
    return [f"{stem}-{i:05d}-of-{total:05d}.gguf" for i in range(1, total + 1)]


class GGUFFile:
    """A parsed GGUF checkpoint (possibly several part files)."""

    def __init__(self, path: str):
        self.path = path
        self.metadata: dict[str, Any] = {}
        self.tensors: dict[str, GGUFTensor] = {}
        self._maps: list[mmap.mmap] = []
        self._files = []
        for i, p in enumerate(split_paths(path)):
            if not os.path.exists(p):
                raise FileNotFoundError(p)
            self._parse_one(p, first=(i == 0))

    # -- parsing -------------------------------------------------------------------------
    def _parse_one(self, path: str, first: bool) -> None:
        f = open(path, "rb")
        if os.fstat(f.fileno()).st_size < 24:
            raise GGUFError(f"{path}: too small to be a GGUF file")
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        self._files.append(f)
        self._maps.append(mm)
        cur = _Cursor(mm)
        magic = cur.unpack("I")
        if magic != GGUF_MAGIC:
            raise GGUFError(f"{path}: bad magic 0x{magic:08x}")
        version = cur.unpack("I")
        if version not in (2, 3):
            raise GGUFError(f"{path}: unsupported GGUF version {version}")
        n_tensors = cur.unpack("Q")
        n_kv = cur.unpack("Q")
        meta: dict[str, Any] = {}
        for _ in range(n_kv):
            key = cur.string()
            vtype = cur.unpack("I")
            meta[key] = cur.value(vtype)
        if first:
            self.metadata = meta
            self.version = version
        else:
            for k, v in meta.items():
                self.metadata.setdefault(k, v)
        alignment = int(meta.get("general.alignment", GGUF_DEFAULT_ALIGNMENT))
        infos = []
        for _ in range(n_tensors):
            name = cur.string()
            n_dims = cur.unpack("I")
            ne = [cur.unpack("Q") for _ in range(n_dims)]
            qtype = cur.unpack("I")
            rel = cur.unpack("Q")
            infos.append((name, ne, qtype, rel))
        data_start = (cur.pos + alignment - 1) // alignment * alignment
        for name, ne, qtype, rel in infos:
            try:
                qt = GGMLType(qtype)
            except ValueError as exc:
                raise GGUFError(f"{path}: tensor {name} has unknown type id {qtype}") from exc
            elems, nbytes = BLOCK_GEOMETRY[qt]
            n_el = 1
            for d in ne:
                n_el *= d
            if ne and ne[0] % elems:
                raise GGUFError(f"{name}: ne0={ne[0]} not a multiple of block size {elems}")
            size = n_el // elems * nbytes
            off = data_start + rel
            if off + size > len(mm):
                raise GGUFError(f"{path}: tensor {name} runs past end of file")
            self.tensors[name] = GGUFTensor(name, qt, tuple(reversed(ne)), off, size, mm)

    # -- access --------------------------------------------------------------------------
    def __contains__(self, name: str) -> bool:
        return name in self.tensors

    def __getitem__(self, name: str) -> GGUFTensor:
        return self.tensors[name]

    def __iter__(self) -> Iterator[GGUFTensor]:
        return iter(self.tensors.values())

    def get(self, key: str, default=None):
        return self.metadata.get(key, default)

    @property
    def architecture(self) -> str:
        return str(self.metadata.get("general.architecture", ""))

    def arch_key(self, suffix: str, default=None):
        """Metadata lookup under the ``<architecture>.`` prefix."""
        return self.metadata.get(f"{self.architecture}.{suffix}", default)

    def close(self) -> None:
        self.tensors.clear()
        for mm in self._maps:
            try:
                mm.close()
            except BufferError:
                pass        # a tensor view is still alive; the GC will release the map later
        for f in self._files:
            f.close()
        self._maps, self._files = [], []
