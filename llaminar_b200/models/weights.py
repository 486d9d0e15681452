"""In-memory checkpoint: tensors kept as raw GGUF block bytes + type + logical shape.

``ModelWeights`` is what both the torch reference model (after dequantisation) and the GPU
engine (after the load-time tile reorder) are built from.  It can come from a ``.gguf`` file
or from the synthetic generator, and can be written back to a ``.gguf``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..gguf import GGMLType, GGUFFile, GGUFWriter, dequantize, quantize
from ..gguf.constants import BLOCK_GEOMETRY
from .config import ModelConfig


@dataclass
class QTensor:
    qtype: GGMLType
    shape: tuple[int, ...]          # logical shape, torch order
    raw: torch.Tensor               # flat uint8

    def to_float(self) -> torch.Tensor:
        return dequantize(self.raw, self.qtype, self.shape)

    @property
    def row_bytes(self) -> int:
        e, b = BLOCK_GEOMETRY[self.qtype]
        return self.shape[-1] // e * b

    def rows(self, start: int, stop: int) -> "QTensor":
        """Row slice of a 2-D tensor (column-parallel / vocab-parallel shards)."""
        assert len(self.shape) == 2
        rb = self.row_bytes
        return QTensor(self.qtype, (stop - start, self.shape[1]), self.raw[start * rb:stop * rb])

    def cols(self, start: int, stop: int) -> "QTensor":
        """Column slice of a 2-D tensor on block boundaries (row-parallel shards)."""
        assert len(self.shape) == 2
        e, b = BLOCK_GEOMETRY[self.qtype]
        if start % e or stop % e:
            raise ValueError(f"column slice [{start},{stop}) is not aligned to {self.qtype.name} blocks of {e}")
        r = self.raw.reshape(self.shape[0], self.row_bytes)
        return QTensor(self.qtype, (self.shape[0], stop - start),
                       r[:, start // e * b: stop // e * b].contiguous().reshape(-1))

    def expert(self, e: int) -> "QTensor":
        assert len(self.shape) == 3
        n = self.raw.numel() // self.shape[0]
        return QTensor(self.qtype, self.shape[1:], self.raw[e * n:(e + 1) * n])

    def to(self, device) -> "QTensor":
        return QTensor(self.qtype, self.shape, self.raw.to(device))

    def transcoded(self, target: GGMLType = GGMLType.Q8_0) -> "QTensor":
        """The same values re-encoded in ``target`` (decode, then quantise; one leading slice at a time so that the fp32
        temporary stays small).  Used where a kernel needs a format with a packed device layout and the file's format has
        none: Q8_0 adds a rounding error of ~0.4 %, far below the error of the 1- to 3-bit formats it replaces."""
        if self.qtype == target:
            return self
        if len(self.shape) < 3:
            return QTensor(target, self.shape, quantize(self.to_float(), target))
        parts = [self.expert(e).transcoded(target).raw for e in range(self.shape[0])]
        return QTensor(target, self.shape, torch.cat(parts))


class ModelWeights:
    def __init__(self, config: ModelConfig, tensors: dict[str, QTensor], metadata: dict | None = None):
        self.config = config
        self.tensors = tensors
        self.metadata = metadata or {}

    def __getitem__(self, name: str) -> QTensor:
        return self.tensors[name]

    def __contains__(self, name: str) -> bool:
        return name in self.tensors

    def get(self, name: str):
        return self.tensors.get(name)

    def float_dict(self, device="cpu") -> dict[str, torch.Tensor]:
        """Every tensor dequantised to float32 (only sensible for small models)."""
        return {k: dequantize(v.raw.to(device), v.qtype, v.shape) for k, v in self.tensors.items()}

    def nbytes(self) -> int:
        return sum(t.raw.numel() for t in self.tensors.values())

    # -- file I/O ------------------------------------------------------------------------------
    @staticmethod
    def from_gguf(path: str, device="cpu") -> "ModelWeights":
        gf = GGUFFile(path)
        cfg = ModelConfig.from_gguf(gf)
        tensors = {}
        for t in gf:
            raw = t.raw()
            raw = raw.to(device) if str(device) != "cpu" else raw.clone()
            tensors[t.name] = QTensor(t.qtype, t.shape, raw)
        md = dict(gf.metadata)
        gf.close()
        return ModelWeights(cfg, tensors, md)

    def save_gguf(self, path: str, extra_metadata: dict | None = None) -> None:
        w = GGUFWriter()
        md = dict(self.config.gguf_metadata())
        for k, v in self.metadata.items():
            if k != "general.alignment":
                md.setdefault(k, v)
        md.update(extra_metadata or {})
        for k, v in md.items():
            w.add(k, v)
        for name, t in self.tensors.items():
            w.add_raw_tensor(name, t.qtype, t.shape, t.raw)
        w.write(path)


def qtensor_from_float(x: torch.Tensor, qtype: GGMLType) -> QTensor:
    return QTensor(GGMLType(qtype), tuple(x.shape), quantize(x, qtype))
