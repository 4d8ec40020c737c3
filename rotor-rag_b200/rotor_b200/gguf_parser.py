"""GGUF container reader, mirroring the interface of the reference's ``src/rotor/gguf_parser.py``
(GGUFValueType :15-29, GGUFTensorType :32-65, GGUFTensor :68-74, GGUFReader :77-300) so that code
written against it keeps working: ``GGUFReader(path).read()``, ``.metadata``, ``.tensors``,
``.get_tensor``, ``.load_tensor_data``, ``.list_tensors``.

Behaviour kept from the reference: little-endian GGUF v2/v3 layout (magic, version, tensor count,
metadata count, key/value pairs, tensor infos, data section aligned to 32 bytes); dimensions in
file order; its own type codes for the ternary tensors (TQ1_0 = 30, TQ2_0 = 31), whose payload it
reads as the 2-bit packed format of this project -- four weights per byte, ``[dims[0], -1]`` --
i.e. exactly what ``TernaryLinear.load_from_bitnet`` takes.  F32 and F16 tensors come back as
arrays of their shape; other quantised types raise NotImplementedError.

Added here: ``load_linear`` hands a ternary tensor's bytes to the device repack kernel without an
int8 detour.  Parsing needs no GPU.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from enum import IntEnum
from typing import Dict, List, Optional

import numpy as np


class GGUFValueType(IntEnum):
    UINT8 = 0
    INT8 = 1
    UINT16 = 2
    INT16 = 3
    UINT32 = 4
    INT32 = 5
    FLOAT32 = 6
    BOOL = 7
    STRING = 8
    ARRAY = 9
    UINT64 = 10
    INT64 = 11
    FLOAT64 = 12


class GGUFTensorType(IntEnum):
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q8_1 = 9
    Q2_K = 10
    Q3_K = 11
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    Q8_K = 15
    IQ2_XXS = 16
    IQ2_XS = 17
    IQ3_XXS = 18
    IQ1_S = 19
    IQ4_NL = 20
    IQ3_S = 21
    IQ2_S = 22
    IQ4_XS = 23
    I8 = 24
    I16 = 25
    I32 = 26
    I64 = 27
    F64 = 28
    IQ1_M = 29
    TQ1_0 = 30
    TQ2_0 = 31


_SCALARS = {GGUFValueType.UINT8: "<B", GGUFValueType.INT8: "<b", GGUFValueType.UINT16: "<H",
            GGUFValueType.INT16: "<h", GGUFValueType.UINT32: "<I", GGUFValueType.INT32: "<i",
            GGUFValueType.FLOAT32: "<f", GGUFValueType.BOOL: "<?", GGUFValueType.UINT64: "<Q",
            GGUFValueType.INT64: "<q", GGUFValueType.FLOAT64: "<d"}
DATA_ALIGNMENT = 32
TERNARY_TYPES = (GGUFTensorType.TQ1_0, GGUFTensorType.TQ2_0)


@dataclass
class GGUFTensor:
    name: str
    dims: List[int]
    type: GGUFTensorType
    offset: int
    data: Optional[np.ndarray] = None


class _Cursor:
    """Sequential little-endian reads over a bytes-like object."""

    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt):
        size = struct.calcsize(fmt)
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += size
        return v

    def string(self):
        n = self.take("<Q")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8")
        self.pos += n
        return s

    def value(self, vtype):
        vtype = GGUFValueType(vtype)
        if vtype == GGUFValueType.STRING:
            return self.string()
        if vtype == GGUFValueType.ARRAY:
            inner = self.take("<I")
            count = self.take("<Q")
            return [self.value(inner) for _ in range(count)]
        return self.take(_SCALARS[vtype])


class GGUFReader:
    def __init__(self, filepath: str, verbose: bool = False):
        self.filepath = filepath
        self.verbose = verbose
        self.version = None
        self.tensor_count = 0
        self.metadata_count = 0
        self.metadata: Dict[str, object] = {}
        self.tensors: Dict[str, GGUFTensor] = {}
        self.data_offset = 0

    def read(self):
        with open(self.filepath, "rb") as f, mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) as mm:
            cur = _Cursor(mm)
            if bytes(mm[:4]) != b"GGUF":
                raise ValueError(f"Not a valid GGUF file: magic={bytes(mm[:4])!r}")
            cur.pos = 4
            self.version = cur.take("<I")
            self.tensor_count = cur.take("<Q")
            self.metadata_count = cur.take("<Q")
            for _ in range(self.metadata_count):
                key = cur.string()
                self.metadata[key] = cur.value(cur.take("<I"))
            for _ in range(self.tensor_count):
                name = cur.string()
                ndim = cur.take("<I")
                dims = [cur.take("<Q") for _ in range(ndim)]
                ttype = GGUFTensorType(cur.take("<I"))
                self.tensors[name] = GGUFTensor(name, dims, ttype, cur.take("<Q"))
            self.data_offset = -(-cur.pos // DATA_ALIGNMENT) * DATA_ALIGNMENT
        if self.verbose:
            print(f"GGUF v{self.version}: {self.tensor_count} tensors, {self.metadata_count} metadata entries")
        return self

    def get_tensor(self, name: str) -> Optional[GGUFTensor]:
        return self.tensors.get(name)

    def list_tensors(self) -> List[str]:
        return list(self.tensors)

    def load_tensor_data(self, name: str) -> np.ndarray:
        t = self.tensors.get(name)
        if t is None:
            raise ValueError(f"Tensor '{name}' not found")
        count = int(np.prod(t.dims))
        start = self.data_offset + t.offset
        if t.type in TERNARY_TYPES:
            raw = np.fromfile(self.filepath, dtype=np.uint8, count=(count + 3) // 4, offset=start)
            return raw.reshape(t.dims[0], -1) if len(t.dims) == 2 else raw
        if t.type == GGUFTensorType.F32:
            return np.fromfile(self.filepath, dtype=np.float32, count=count, offset=start).reshape(t.dims)
        if t.type == GGUFTensorType.F16:
            return np.fromfile(self.filepath, dtype=np.float16, count=count, offset=start).reshape(t.dims)
        raise NotImplementedError(f"Tensor type {t.type} not yet implemented")

    # -- device ingestion (no counterpart in the reference) -------------------------------------
    def load_linear(self, name: str, layer, scale: float = 1.0):
        """Packed bytes of ternary tensor ``name`` -> ``layer`` (a rotor_b200 TernaryLinear) through
        the device repack kernel.  The tensor must be [out_features, in_features]."""
        t = self.tensors.get(name)
        if t is None or t.type not in TERNARY_TYPES or len(t.dims) != 2:
            raise ValueError(f"'{name}' is not a two-dimensional ternary tensor")
        if (t.dims[0], t.dims[1]) != (layer.out_features, layer.in_features):
            raise ValueError(f"'{name}' has shape {t.dims}, layer expects {[layer.out_features, layer.in_features]}")
        layer.load_from_bitnet(self.load_tensor_data(name), scale)
        return layer

    def print_summary(self):
        print(f"GGUF version {self.version}: {self.tensor_count} tensors, {self.metadata_count} metadata entries")
        for key, value in list(self.metadata.items())[:10]:
            if isinstance(value, (str, int, float, bool)):
                print(f"  {key}: {value}")
        for name, t in list(self.tensors.items())[:10]:
            print(f"  {name}: {t.dims} {t.type.name}")
