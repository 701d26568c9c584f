"""Mirror of the reference's safetensors reader (packages/core/src/io/safetensor/parser.ts:35-170,
sharded.ts:20-97, dtypes.ts:14-60, io/tensor-loaders.ts:44-76) with one deliberate change for this
backend: BF16 tensors are NOT widened to float32 on load (the reference converts them because WebGPU
has no bf16); their 16-bit patterns go to the device as they are when the destination is bfloat16.

The same validation and the same error texts as the reference: header length fields, the 100 MB
header cap, JSON errors, unsupported dtypes, byte-size mismatches, missing shards / layers.
Files are memory-mapped; a tensor's bytes are touched only when it is loaded.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass, field

import numpy as np

from . import core
from .core import Tensor

SAFETENSORS_DTYPE_BYTES = {"F64": 8, "F32": 4, "F16": 2, "BF16": 2, "I64": 8, "I32": 4, "I16": 2, "I8": 1,
                           "U64": 8, "U32": 4, "U16": 2, "U8": 1, "BOOL": 1}
# dtypes.ts:14-28, except BF16 -> bfloat16 (kept native)
SAFETENSORS_DTYPE_MAP = {"F64": "float64", "F32": "float32", "F16": "float16", "BF16": "bfloat16", "I64": "int64", "I32": "int32",
                         "I16": "int16", "I8": "int8", "U64": "uint64", "U32": "uint32", "U16": "uint16", "U8": "uint8",
                         "BOOL": "bool"}
_NUMPY_VIEW = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I64": np.int64, "I32": np.int32,
               "I16": np.int16, "I8": np.int8, "U64": np.uint64, "U32": np.uint32, "U16": np.uint16, "U8": np.uint8,
               "BOOL": np.uint8}
MAX_HEADER_SIZE = 100 * 1024 * 1024


@dataclass
class SafetensorLayer:
    name: str
    dtype: str                 # logical dtype of this backend
    shape: tuple
    originalDtype: str         # safetensors dtype string
    file: "SafetensorFile"
    dataOffsets: tuple
    byteSize: int
    numel: int

    def raw(self) -> np.ndarray:
        """The stored values as a numpy view of the mapped file (BF16: uint16 bit patterns)."""
        start = self.file.dataOffset + self.dataOffsets[0]
        buf = self.file.mapped()[start:start + self.byteSize]
        return buf.view(_NUMPY_VIEW[self.originalDtype]).reshape(self.shape)

    def to_float32(self) -> np.ndarray:
        a = self.raw()
        if self.originalDtype == "BF16":     # dtypes.ts:46-58: bits << 16
            return (a.astype(np.uint32) << 16).view(np.float32)
        return a.astype(np.float32)


@dataclass
class SafetensorFile:
    path: str
    metadata: dict
    layers: dict
    dataOffset: int
    _map: np.ndarray | None = field(default=None, repr=False)

    def mapped(self) -> np.ndarray:
        if self._map is None:
            self._map = np.memmap(self.path, dtype=np.uint8, mode="r")
        return self._map

    def close(self) -> None:
        self._map = None


@dataclass
class SafetensorGroup:
    sharded: bool
    metadata: dict
    files: dict
    layers: dict
    totalSize: int | None = None

    def getLayer(self, name: str):
        return self.layers.get(name)

    def hasLayer(self, name: str) -> bool:
        return name in self.layers

    def close(self) -> None:
        for f in self.files.values():
            f.close()


def parseHeaderSize(buf: bytes) -> int:                      # parser.ts:35-51
    low, high = struct.unpack("<II", buf[:8])
    if high != 0:
        raise ValueError(f"Header size too large: exceeds safe integer limit (high bytes: {high})")
    if low > MAX_HEADER_SIZE:
        raise ValueError(f"Header size exceeds safe limit: {low} bytes (max: {MAX_HEADER_SIZE})")
    return low


def parseSafetensorFile(path: str) -> SafetensorFile:       # parser.ts:84-170
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise ValueError("Invalid safetensors: file too small to contain header size")
        header_size = parseHeaderSize(head)
        if header_size == 0:
            raise ValueError("Invalid safetensors: header size is 0")
        hb = f.read(header_size)
    if len(hb) < header_size:
        raise ValueError("Invalid safetensors: header data incomplete")
    try:
        header = json.loads(hb.decode("utf-8"))
    except (ValueError, UnicodeDecodeError) as e:
        raise ValueError(f"Invalid JSON in safetensors header: {e}") from None
    if not isinstance(header, dict):
        raise ValueError("Invalid JSON in safetensors header: not an object")
    meta = header.get("__metadata__") or {}
    file = SafetensorFile(path, meta, {}, 8 + header_size)
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        if not (isinstance(entry, dict) and isinstance(entry.get("dtype"), str) and isinstance(entry.get("shape"), list)
                and isinstance(entry.get("data_offsets"), list) and len(entry["data_offsets"]) == 2):
            continue                                           # parser.ts:126-129: entries of another kind are skipped
        st = entry["dtype"]
        if st not in SAFETENSORS_DTYPE_BYTES:
            raise ValueError(f"Unsupported safetensors dtype: {st}")
        numel = int(np.prod(entry["shape"], dtype=np.int64)) if entry["shape"] else 1
        b0, b1 = entry["data_offsets"]
        byte_size = b1 - b0
        expected = numel * SAFETENSORS_DTYPE_BYTES[st]
        if numel > 0 and byte_size != expected:
            raise ValueError(f"Data size mismatch for {name}: expected {expected} bytes, got {byte_size} bytes")
        # beyond the reference: a tensor must lie inside the file (a truncated download otherwise fails at read time)
        if b0 < 0 or file.dataOffset + b1 > size:
            raise ValueError(f"Data range of {name} [{b0}, {b1}) lies outside the file ({size} bytes)")
        file.layers[name] = SafetensorLayer(name, SAFETENSORS_DTYPE_MAP[st], tuple(entry["shape"]), st, file, (b0, b1), byte_size, numel)
    return file


def parseShardedIndex(path: str) -> SafetensorGroup:        # sharded.ts:20-97
    try:
        with open(path, "rb") as f:
            index = json.loads(f.read().decode("utf-8"))
    except ValueError as e:
        raise ValueError(f"Invalid index.json: {e}") from None
    wm = index.get("weight_map") if isinstance(index, dict) else None
    if not isinstance(wm, dict):
        raise ValueError("Invalid index.json: weight_map must be an object")
    base = os.path.dirname(os.path.abspath(path))
    files = {}
    for shard in sorted(set(wm.values())):
        sp = os.path.join(base, shard)
        if not os.path.exists(sp):
            raise ValueError(f"Shard file not found: {shard}")
        files[shard] = parseSafetensorFile(sp)
    layers = {}
    for layer_name, shard in wm.items():
        layer = files[shard].layers.get(layer_name)
        if layer is None:
            raise ValueError(f"Layer not found in shard {shard}: {layer_name}")
        layers[layer_name] = layer
    md = index.get("metadata") or {}
    metadata = {k: v for k, v in md.items() if isinstance(v, str)}
    return SafetensorGroup(True, metadata, files, layers, md.get("total_size"))


def loadSafetensor(path: str) -> SafetensorGroup:           # index.ts: one file, or an index.json of shards
    if path.endswith(".json"):
        return parseShardedIndex(path)
    f = parseSafetensorFile(path)
    return SafetensorGroup(False, f.metadata, {f.path: f}, dict(f.layers))


def tensorFromSafetensorLayer(layer: SafetensorLayer, dtype: str | None = None) -> Tensor:
    """io/tensor-loaders.ts:44-76.  dtype None keeps the stored type (BF16 stays bfloat16: 2 bytes per
    value cross PCIe instead of the reference's 4); float targets convert on the host."""
    target = dtype or layer.dtype
    if target == "bfloat16" and layer.originalDtype == "BF16":
        return Tensor(np.ascontiguousarray(layer.raw()), dtype="bfloat16")         # uint16 bit patterns, uploaded as they are
    if target in ("float32", "bfloat16", "float16"):
        return Tensor(layer.to_float32(), dtype=target)
    if target in ("int64", "int32", "uint8"):
        return Tensor(np.ascontiguousarray(layer.raw()).astype(target), dtype=target)
    if target == "bool":
        return Tensor(np.ascontiguousarray(layer.raw()) != 0, dtype="bool")
    raise TypeError(f"dtype {target} has no device representation in this backend")


def loadModuleFromSafetensor(module, group: SafetensorGroup, keyMapper=None, strict: bool = True) -> dict:
    """nn/module.ts:572-669 loadFromSafetensor: every parameter of `module` is filled from the layer
    of the same (mapped) name; returns {"loadedKeys", "missingKeys", "unexpectedKeys"}."""
    be = core._backend()
    own = module.stateDict()
    loaded, missing = [], []
    used = set()
    for name, param in own.items():
        key = keyMapper(name) if keyMapper else name
        layer = group.getLayer(key) if key is not None else None
        if layer is None:
            missing.append(name)
            continue
        if tuple(layer.shape) != tuple(param.shape):
            raise ValueError(f"shape mismatch for {name}: file has {tuple(layer.shape)}, module expects {tuple(param.shape)}")
        if param.dtype == "bfloat16" and layer.originalDtype == "BF16":
            be.upload(param._handle, np.ascontiguousarray(layer.raw()))            # native 16-bit upload
        else:
            be.upload(param._handle, layer.to_float32() if param.dtype in ("float32", "bfloat16", "float16") else layer.raw())
        loaded.append(name)
        used.add(key)
    unexpected = [k for k in group.layers if k not in used]
    if strict and missing:
        raise KeyError(f"missing keys in safetensors file: {missing[:5]}{'...' if len(missing) > 5 else ''}")
    return {"loadedKeys": loaded, "missingKeys": missing, "unexpectedKeys": unexpected}


class SafetensorStateDict:
    """Read-only mapping name -> float32 array over a SafetensorGroup, materialising one tensor at a
    time: what Qwen3Engine(cfg, weights, ...) and Module.loadStateDict take as `weights`.  bf16 values
    widen exactly, so the engine's re-rounding to bf16 gives back the stored bits."""

    def __init__(self, group: SafetensorGroup, keyMapper=None):
        self.group, self.keyMapper = group, keyMapper

    def _key(self, name):
        return self.keyMapper(name) if self.keyMapper else name

    def __contains__(self, name) -> bool:
        return self.group.hasLayer(self._key(name))

    def __getitem__(self, name) -> np.ndarray:
        layer = self.group.getLayer(self._key(name))
        if layer is None:
            raise KeyError(name)
        return layer.to_float32()

    def keys(self):
        return self.group.layers.keys()


def save_file(tensors: dict, path: str, metadata: dict | None = None) -> None:
    """Writes a safetensors file (the reference only reads them; this exists for tests and for
    exporting synthetic weights).  Values: numpy arrays; a (uint16 array, "BF16") tuple stores bf16 bits."""
    rev = {np.dtype(v): k for k, v in _NUMPY_VIEW.items() if k not in ("BF16", "BOOL")}
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, val in tensors.items():
        if isinstance(val, tuple):
            arr, st = np.ascontiguousarray(val[0]), val[1]
        else:
            arr = np.ascontiguousarray(val)
            st = rev[arr.dtype]
        b = arr.tobytes()
        header[name] = {"dtype": st, "shape": list(arr.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hb = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for b in blobs:
            f.write(b)
