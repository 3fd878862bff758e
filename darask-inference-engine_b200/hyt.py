"""`.hyt` weight files (Hayate): header, tensor table and the assembly of one layer's expert images.

A `.hyt` file is a checkpoint pre-converted into the layout the kernels consume (reference: common/core/src/hyt.rs;
writer engines/hayate/python-tools/hayate_tools/hyt.py): a 64-byte little-endian header (magic "HYT0", format version
2, machine id, tensor count, table offset, 4 KiB-aligned data offset, 16 bytes of source hash), a table of entries
{name, quant tag / dtype / group, shape, offset relative to the data region (4 KiB aligned), byte count} and the data.
A layer's routed experts are the entries `mlp.experts.<e>.{gate,up,down}_proj.weight`; the device image of an expert
is those three tensors one after the other, each padded with zeros to a multiple of 256 bytes
(engines/hayate/crates/models/src/glm53/experts.rs:2607-2655 `read_image`), which is the layout
`hayate_glm_moe_gate_up` / `hayate_moe_layer` read in place. NVFP4 matrices are checked as the reference checks them
(glm53/mod.rs:119-133): exact size, no NaN scale codes, a finite positive tensor scale.
"""
from __future__ import annotations

import math
import os
import struct
from dataclasses import dataclass

import numpy as np

MAGIC = b"HYT0"
FORMAT_VERSION = 2
HEADER_LEN = 64
DATA_ALIGN = 4096
IMAGE_ALIGN = 256
MAX_RANK = 6
TAG_PLAIN, TAG_PER_TENSOR, TAG_NVFP4, TAG_MXFP8, TAG_Q4_BF16, TAG_INT8_ROW, TAG_LOWBIT, TAG_EXL3 = range(8)
_DTYPE_BITS = {0: 32, 1: 16, 2: 16, 3: 8, 4: 8, 5: 4, 6: 8, 7: 32, 8: 4}     # f32 bf16 f16 e4m3 e5m2 e2m1 i8 i32 i4


def _round_up(v: int, a: int) -> int:
    return -(-v // a) * a


def storage_bytes(shape, quant) -> int | None:
    """Bytes a tensor of `shape` occupies under quant = (tag, dtype, group), by the sizing rules of the reference's
    `TensorDesc::storage_bytes` (common/core/src/hyt.rs); None for LOWBIT, whose byte count is taken from the table."""
    shape = tuple(int(d) for d in shape)
    if len(shape) > MAX_RANK or any(d <= 0 for d in shape):
        raise ValueError("invalid shape")
    tag, dtype, group = quant
    n = math.prod(shape)
    cols = shape[-1] if shape else 1
    if tag in (TAG_PLAIN, TAG_PER_TENSOR):
        if dtype not in _DTYPE_BITS or group:
            raise ValueError("invalid quantization words")
        return (n * _DTYPE_BITS[dtype] + 7) // 8 + (4 if tag == TAG_PER_TENSOR else 0)
    if tag in (TAG_NVFP4, TAG_MXFP8):
        if dtype or group:
            raise ValueError("invalid quantization words")
        block = 16 if tag == TAG_NVFP4 else 32
        if cols % block:
            raise ValueError("last dimension is not a whole number of blocks")
        rows = shape[-2] if len(shape) > 1 else 1
        batch = n // (rows * cols)
        payload = (rows * cols * (4 if tag == TAG_NVFP4 else 8) + 7) // 8
        scales = _round_up(rows, 128) * _round_up(cols // block, 4)          # 128 x 4 scale tiles
        return batch * (payload + scales + (4 if tag == TAG_NVFP4 else 0))
    if tag == TAG_Q4_BF16:
        if dtype or group <= 0 or cols % group:
            raise ValueError("invalid block size")
        return (n * 4 + 7) // 8 + (n // cols) * (cols // group) * 2
    if tag == TAG_INT8_ROW:
        if dtype:
            raise ValueError("invalid quantization words")
        return n + (n // cols) * 4
    if tag == TAG_EXL3:                                  # dtype = twice the bits per weight, group = codebook
        ok = (2 <= dtype <= 16 and dtype % 2 == 0 and group in (0, 1, 2)) or (dtype in (3, 5, 7) and group == 2)
        if len(shape) != 2 or shape[0] % 128 or shape[1] % 128 or not ok:
            raise ValueError("invalid EXL3 matrix")
        return n * dtype // 16 + 2 * (shape[0] + shape[1])
    if tag == TAG_LOWBIT:
        return None
    raise ValueError(f"unknown quantization tag {tag}")


@dataclass
class Entry:
    name: str
    quant: tuple          # (tag, dtype, group)
    shape: tuple
    offset: int           # absolute file offset
    nbytes: int


class HytFile:
    """Header and tensor table of a `.hyt` file, validated as `HytFile::open` validates them (hyt.rs): magic, version,
    machine id (and, when `machine` is given, that the file was converted for that machine), regions in order and
    aligned, every entry's size equal to what its shape and quantization give, data ranges inside the file, no
    duplicate names, no overlapping ranges."""

    def __init__(self, path, machine=None):
        self.path = os.fspath(path)
        size = os.path.getsize(self.path)
        with open(self.path, "rb") as f:
            head = f.read(HEADER_LEN)
            if len(head) != HEADER_LEN or head[:4] != MAGIC:
                raise ValueError(f"{self.path}: not a .hyt file")
            version, self.machine, count, table_at, data_at = struct.unpack_from("<IIIQQ", head, 4)
            self.source_hash = head[32:48]
            if version != FORMAT_VERSION:
                raise ValueError(f"format version {version} != {FORMAT_VERSION}")
            if self.machine > 1 or (machine is not None and machine != self.machine):
                raise ValueError(f"machine id {self.machine} is unknown or not the one asked for")
            fits = table_at <= data_at if count == 0 else table_at < data_at
            if data_at % DATA_ALIGN or table_at < HEADER_LEN or not fits or data_at > size:
                raise ValueError("misaligned or overlapping regions")
            f.seek(table_at)
            table = f.read(data_at - table_at)
        self.entries, self.by_name = [], {}
        pos = 0

        def take(fmt):
            nonlocal pos
            n = struct.calcsize(fmt)
            if pos + n > len(table):
                raise ValueError("truncated tensor table")
            v = struct.unpack_from(fmt, table, pos)
            pos += n
            return v
        if count > len(table) // 37:                    # the smallest entry: a scalar with a one-byte name
            raise ValueError("tensor count exceeds table region")
        for _ in range(count):
            (name_len,) = take("<I")
            if name_len == 0 or pos + name_len > len(table):
                raise ValueError("invalid tensor name length")
            name = table[pos:pos + name_len].decode("utf-8")
            pos += name_len
            tag, dtype, group, rank = take("<IIII")
            if rank > MAX_RANK:
                raise ValueError(f"rank {rank} > {MAX_RANK}")
            shape = take(f"<{rank}Q") if rank else ()
            rel, nbytes = take("<QQ")
            expected = storage_bytes(shape, (tag, dtype, group))
            if rel % DATA_ALIGN or (expected is not None and expected != nbytes):
                raise ValueError(f"{name}: invalid size or alignment")
            if data_at + rel + nbytes > size:
                raise ValueError(f"{name}: tensor exceeds file")
            if name in self.by_name:
                raise ValueError(f"{name}: duplicate tensor name")
            e = Entry(name, (tag, dtype, group), tuple(shape), data_at + rel, nbytes)
            self.by_name[name] = e
            self.entries.append(e)
        spans = sorted((e.offset, e.offset + e.nbytes) for e in self.entries)
        if any(a[1] > b[0] for a, b in zip(spans, spans[1:])):
            raise ValueError("tensor data ranges overlap")

    def read(self, name, first_byte=0, nbytes=None) -> np.ndarray:
        """Bytes of a tensor, or of a byte range that lies inside it, as a read-only view of the file."""
        e = self.by_name[name]
        nbytes = e.nbytes - first_byte if nbytes is None else nbytes
        if first_byte < 0 or nbytes < 0 or first_byte + nbytes > e.nbytes:
            raise ValueError(f"{name}: byte range outside the tensor")
        if nbytes == 0:
            return np.zeros(0, np.uint8)
        return np.memmap(self.path, dtype=np.uint8, mode="r", offset=e.offset + first_byte, shape=(nbytes,))


def write(path, tensors, machine=0, source_hash=bytes(16)) -> None:
    """tensors: list of (name, shape, (tag, dtype, group), bytes-like). For tests and tools; data in list order."""
    rel, table, blobs = 0, bytearray(), []
    for name, shape, quant, raw in tensors:
        raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        expected = storage_bytes(shape, quant)
        if expected is not None and expected != raw.size:
            raise ValueError(f"{name}: {raw.size} bytes given, {expected} expected")
        label = name.encode("utf-8")
        table += struct.pack("<I", len(label)) + label + struct.pack("<IIII", *quant, len(shape))
        table += b"".join(struct.pack("<Q", int(d)) for d in shape) + struct.pack("<QQ", rel, raw.size)
        blobs.append((rel, raw))
        rel = _round_up(rel + raw.size, DATA_ALIGN)
    base = _round_up(HEADER_LEN + len(table), DATA_ALIGN)
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<IIIQQ", FORMAT_VERSION, machine, len(tensors), HEADER_LEN, base) + bytes(source_hash)[:16].ljust(16, b"\0")
                + bytes(16))
        f.write(table)
        for at, raw in blobs:
            f.seek(base + at)
            f.write(raw.tobytes())
        if not blobs:
            f.truncate(base)


def check_nvfp4(raw: np.ndarray, n: int, k: int, name="matrix") -> None:
    """The reference's checks of an NVFP4 matrix image: size, no NaN scale codes, finite positive tensor scale."""
    if raw.size != storage_bytes((n, k), (TAG_NVFP4, 0, 0)):
        raise ValueError(f"{name}: NVFP4 size")
    scales = raw[n * k // 2:raw.size - 4]
    g = np.frombuffer(np.ascontiguousarray(raw[raw.size - 4:]).tobytes(), np.float32)[0]
    if np.any((scales & 0x7F) == 0x7F) or not np.isfinite(g) or g <= 0:
        raise ValueError(f"{name}: invalid NVFP4 scales / layout")


def mlp_image(f: HytFile, stem: str) -> np.ndarray:
    """[gate | up | down] of `<stem>.{gate,up,down}_proj.weight`, each at the next multiple of 256 bytes, zero padded."""
    parts, total = [], 0
    for part in ("gate", "up", "down"):
        name = f"{stem}.{part}_proj.weight"
        if name not in f.by_name:
            raise KeyError(f"missing {name}")
        e = f.by_name[name]
        raw = np.array(f.read(name))
        if e.quant[0] == TAG_NVFP4:
            check_nvfp4(raw, int(e.shape[0]), int(e.shape[1]), name)
        elif e.quant[0] in (TAG_LOWBIT, TAG_EXL3):
            raise ValueError(f"{name}: LOWBIT / EXL3 expert formats have no kernel in this library")
        parts.append((total, raw))
        total = _round_up(total + raw.size, IMAGE_ALIGN)
    image = np.zeros(total, np.uint8)
    for at, raw in parts:
        image[at:at + raw.size] = raw
    return image


def expert_image(f: HytFile, expert: int) -> np.ndarray:
    """One routed expert's device image."""
    return mlp_image(f, f"mlp.experts.{expert}")


def layer_images(f: HytFile, experts: int, first: int = 0) -> np.ndarray:
    """uint8 [experts, image bytes] of experts [first, first + experts): what `HayateMoeLayer.load` takes as `images`
    (all experts resident), or one rank's block of an expert-parallel group."""
    images = [expert_image(f, first + e) for e in range(experts)]
    if len({im.size for im in images}) != 1:
        raise ValueError("expert images of one layer differ in size")
    return np.stack(images)


def plain_tensor(f: HytFile, name: str) -> np.ndarray:
    """A PLAIN f32 / bf16 / f16 tensor as float32 in its shape."""
    e = f.by_name[name]
    tag, dtype, _ = e.quant
    if tag != TAG_PLAIN or dtype not in (0, 1, 2):
        raise ValueError(f"{name}: not a plain f32 / bf16 / f16 tensor")
    raw = np.array(f.read(name))
    if dtype == 0:
        v = raw.view(np.float32)
    elif dtype == 1:
        v = (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
    else:
        v = raw.view(np.float16).astype(np.float32)
    return v.reshape(e.shape)


def load_layer(path_or_file, topk: int, scale: float = 2.5, max_tokens: int = 1, device="cuda"):
    """One layer file as a resident `HayateMoeLayer`: router (`mlp.gate.weight`), selection bias
    (`mlp.gate.e_score_correction_bias`), every routed expert's image and the shared expert's (`mlp.shared_experts`)."""
    import torch

    from .hayate import HayateMoeLayer
    f = path_or_file if isinstance(path_or_file, HytFile) else HytFile(path_or_file)
    router = plain_tensor(f, "mlp.gate.weight")
    experts, hidden = router.shape
    inter = int(f.by_name["mlp.experts.0.gate_proj.weight"].shape[0])
    m = HayateMoeLayer(hidden, inter, experts, topk, scale, max_tokens, device=device)
    m.load(torch.from_numpy(router), torch.from_numpy(plain_tensor(f, "mlp.gate.e_score_correction_bias")),
           torch.from_numpy(layer_images(f, experts)), torch.from_numpy(mlp_image(f, "mlp.shared_experts")))
    return m
