"""GGUF container: reading the tensors of a Kogarashi checkpoint into a resident MoE layer.

The reference opens the file with `darask_formats::gguf::Gguf` (common/formats/src/gguf.rs: header, typed metadata,
tensor directory, data section aligned to `general.alignment`, 32 by default) and uploads every tensor as one device
buffer in 64 MiB pieces (engines/kogarashi/crates/kogarashi-engine/src/engine.rs:73-107), keeping `{data, ty, k, rows, ne}`.
This module does the same for the tensors of one layer's MoE block (`blk.<l>.ffn_*`, engine.rs:330, 530-632) and hands
them to `KogarashiMoeLayer.load`, which regroups Q6_K tensors once. `expert_block` gives the byte range of a block of
experts inside an `_exps` tensor (the expert index is the outermost dimension, so the residency of one rank under
expert parallelism is one contiguous range of the file).

`write` produces a file in the same container for tests and tools; nothing here touches a GPU until `load_layer`.
"""
from __future__ import annotations

import os
import struct
from dataclasses import dataclass

import numpy as np

from .formats import ggml_tensor_bytes

MAGIC = b"GGUF"
DEFAULT_ALIGNMENT = 32
PIECE = 64 << 20          # bytes per host -> device copy, as the reference uploads

# metadata value types of the container: id -> struct format (scalars)
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_STRING, _ARRAY = 8, 9


@dataclass
class TensorInfo:
    name: str
    ne: tuple        # GGML order: ne[0] is the innermost, contiguous dimension
    ty: int          # GGML type id (0 F32, 1 F16, 12 Q4_K, 14 Q6_K, 30 BF16)
    offset: int      # absolute file offset of the data

    @property
    def nbytes(self) -> int:
        return ggml_tensor_bytes(self.ty, self.ne)


class _Reader:
    def __init__(self, f):
        self.f = f

    def take(self, fmt):
        size = struct.calcsize(fmt)
        raw = self.f.read(size)
        if len(raw) != size:
            raise ValueError("truncated GGUF header")
        return struct.unpack(fmt, raw)[0]

    def string(self):
        n = self.take("<Q")
        raw = self.f.read(n)
        if len(raw) != n:
            raise ValueError("truncated GGUF header")
        return raw.decode("utf-8", errors="replace")

    def value(self, ty):
        if ty in _SCALARS:
            return self.take(_SCALARS[ty])
        if ty == _STRING:
            return self.string()
        if ty == _ARRAY:
            ety, n = self.take("<I"), self.take("<Q")
            return [self.value(ety) for _ in range(n)]
        raise ValueError(f"GGUF value type {ty}")


class GgufFile:
    """Header of a GGUF file (versions 2 and 3): `meta` and the tensor directory with absolute offsets."""

    def __init__(self, path):
        self.path = os.fspath(path)
        self.size = os.path.getsize(self.path)
        with open(self.path, "rb") as f:
            r = _Reader(f)
            if f.read(4) != MAGIC:
                raise ValueError(f"{self.path}: not a GGUF file")
            version = r.take("<I")
            if version not in (2, 3):
                raise ValueError(f"{self.path}: GGUF version {version}")
            n_tensors, n_kv = r.take("<Q"), r.take("<Q")
            self.meta = {}
            for _ in range(n_kv):
                key = r.string()
                self.meta[key] = r.value(r.take("<I"))
            infos = []
            for _ in range(n_tensors):
                name = r.string()
                nd = r.take("<I")
                ne = tuple(r.take("<Q") for _ in range(nd))
                infos.append((name, ne, r.take("<I"), r.take("<Q")))
            align = int(self.meta.get("general.alignment", DEFAULT_ALIGNMENT))
            data = -(-f.tell() // align) * align
        self.tensors = {}
        for name, ne, ty, rel in infos:
            t = TensorInfo(name, ne, ty, data + rel)
            if t.offset + t.nbytes > self.size:
                raise ValueError(f"{name}: tensor exceeds file")          # engine.rs:77-82
            self.tensors[name] = t

    def read(self, name, first_byte=0, nbytes=None) -> np.ndarray:
        """Bytes of a tensor (or of a byte range of it) as a read-only uint8 view of the file."""
        t = self.tensors[name]
        nbytes = t.nbytes - first_byte if nbytes is None else nbytes
        if first_byte < 0 or nbytes < 0 or first_byte + nbytes > t.nbytes:
            raise ValueError(f"{name}: byte range outside the tensor")
        return np.memmap(self.path, dtype=np.uint8, mode="r", offset=t.offset + first_byte, shape=(nbytes,))


def _put_string(out, s):
    raw = s.encode("utf-8")
    out += struct.pack("<Q", len(raw)) + raw


def _put_value(out, v):
    """Writes (type id, value) for the Python types the tests need."""
    if isinstance(v, bool):
        out += struct.pack("<I", 7) + struct.pack("<?", v)
    elif isinstance(v, int):
        out += (struct.pack("<I", 4) + struct.pack("<I", v)) if 0 <= v < 2 ** 32 else (struct.pack("<I", 11) + struct.pack("<q", v))
    elif isinstance(v, float):
        out += struct.pack("<I", 6) + struct.pack("<f", v)
    elif isinstance(v, str):
        out += struct.pack("<I", _STRING)
        _put_string(out, v)
    elif isinstance(v, (list, tuple)) and all(isinstance(e, str) for e in v):
        out += struct.pack("<I", _ARRAY) + struct.pack("<I", _STRING) + struct.pack("<Q", len(v))
        for e in v:
            _put_string(out, e)
    elif isinstance(v, (list, tuple)):
        out += struct.pack("<I", _ARRAY) + struct.pack("<I", 5) + struct.pack("<Q", len(v))
        for e in v:
            out += struct.pack("<i", int(e))
    else:
        raise TypeError(type(v))


def write(path, meta: dict, tensors: list, alignment: int = DEFAULT_ALIGNMENT, version: int = 3) -> None:
    """tensors: list of (name, ne in GGML order, GGML type id, bytes-like). Data is laid out in list order, each tensor
    aligned to `alignment`."""
    meta = dict(meta)
    if alignment != DEFAULT_ALIGNMENT:
        meta["general.alignment"] = alignment
    head = bytearray(MAGIC + struct.pack("<I", version) + struct.pack("<Q", len(tensors)) + struct.pack("<Q", len(meta)))
    for key, v in meta.items():
        _put_string(head, key)
        _put_value(head, v)
    rel, offsets = 0, []
    for name, ne, ty, raw in tensors:
        raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        if raw.size != ggml_tensor_bytes(ty, ne):
            raise ValueError(f"{name}: {raw.size} bytes given, {ggml_tensor_bytes(ty, ne)} expected")
        rel = -(-rel // alignment) * alignment
        offsets.append(rel)
        rel += raw.size
    for (name, ne, ty, _), off in zip(tensors, offsets):
        _put_string(head, name)
        head += struct.pack("<I", len(ne))
        for d in ne:
            head += struct.pack("<Q", int(d))
        head += struct.pack("<I", ty) + struct.pack("<Q", off)
    start = -(-len(head) // alignment) * alignment
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * (start - len(head)))
        pos = 0
        for (_, _, _, raw), off in zip(tensors, offsets):
            f.write(b"\0" * (off - pos))
            raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
            f.write(raw.tobytes())
            pos = off + raw.size


# tensors of one layer's MoE block (engine.rs:530-632) -> does the tensor have an expert dimension
LAYER_TENSORS = {"ffn_gate_inp.weight": False, "ffn_gate_exps.weight": True, "ffn_up_exps.weight": True, "ffn_down_exps.weight": True,
                 "ffn_gate_shexp.weight": False, "ffn_up_shexp.weight": False, "ffn_down_shexp.weight": False,
                 "ffn_gate_inp_shexp.weight": False}


def layer_shape(g: GgufFile, layer: int):
    """(hidden, inter, experts) from the tensor directory of block `layer`."""
    t = g.tensors[f"blk.{layer}.ffn_gate_exps.weight"]
    if len(t.ne) != 3:
        raise ValueError("ffn_gate_exps must be [hidden, inter, experts]")
    return int(t.ne[0]), int(t.ne[1]), int(t.ne[2])


def expert_block(t: TensorInfo, first: int, count: int):
    """Byte range and GGML shape of experts [first, first + count) of an `_exps` tensor."""
    experts = int(t.ne[-1])
    if first < 0 or count < 1 or first + count > experts:
        raise ValueError("expert block outside the tensor")
    per = t.nbytes // experts
    return first * per, count * per, tuple(t.ne[:-1]) + (count,)


def load_layer(path_or_file, layer: int, topk: int, max_tokens: int = 1, device="cuda"):
    """One layer's MoE block as a resident `KogarashiMoeLayer` (all experts on this GPU: decode layers do not shard)."""
    import torch

    from .kogarashi import KogarashiMoeLayer
    g = path_or_file if isinstance(path_or_file, GgufFile) else GgufFile(path_or_file)
    hidden, inter, total = layer_shape(g, layer)
    m = KogarashiMoeLayer(hidden, inter, total, topk, max_tokens, device=device)
    for suffix in LAYER_TENSORS:
        name = f"blk.{layer}.{suffix}"
        if name not in g.tensors:
            if "shexp" in suffix:
                continue                                   # a model without a shared expert
            raise KeyError(name)
        t = g.tensors[name]
        dst = torch.empty(t.nbytes, dtype=torch.uint8, device=device)
        for off in range(0, t.nbytes, PIECE):              # 64 MiB pieces, as engine.rs:73-96
            n = min(PIECE, t.nbytes - off)
            dst[off:off + n].copy_(torch.from_numpy(np.array(g.read(name, off, n))))
        m.load(suffix, dst, t.ty, t.ne)
    return m
