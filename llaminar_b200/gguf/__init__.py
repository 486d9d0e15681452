"""GGUF checkpoint format: reader, writer, block codecs."""
from .constants import BLOCK_GEOMETRY, GGMLType, GGUFValueType, row_bytes
from .quants import dequantize, quantize
from .reader import GGUFError, GGUFFile, GGUFTensor
from .writer import GGUFWriter

__all__ = ["BLOCK_GEOMETRY", "GGMLType", "GGUFValueType", "row_bytes", "dequantize", "quantize",
           "GGUFError", "GGUFFile", "GGUFTensor", "GGUFWriter"]
