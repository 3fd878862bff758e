"""Host-side packing of a Tsumuji checkpoint's routed experts into the device layout the kernels read in place.

Mirrors `pack_experts` and `csf_decode` of the reference (engines/tsumuji/crates/tsumuji-engine/src/weights.rs:445-541):
per expert one block of 27/16 * F * H bytes

    [gate codes | up codes | down codes | gate scales | up scales | down scales]        (weights.rs:10-12, 334-336)

and three float32 global scales. The checkpoint stores every projection as two e2m1 codes per byte (low nibble first)
under `weight` (ModelOpt exports, global scale `weight_scale_2`, multiplied) or `weight_packed` (compressed-tensors
exports, `weight_global_scale`, divided), and its e4m3 block scales either plainly (`weight_scale`) or in the lossless
compressed form `weight_scale.nvfp4_csf_fixed` + `.nvfp4_csf_exceptions`.

`tensors` is any mapping name -> numpy array (a dict, or `SafetensorsSource` over the shards of a checkpoint); the
result goes to `TsumujiMoeLayer.load` unchanged. `csf_encode` exists for tests and tools: the reference only decodes.
"""
from __future__ import annotations

import numpy as np

PROJECTIONS = ("gate_proj", "up_proj", "down_proj")


def expert_stride(hidden: int, inter: int) -> int:
    return inter * hidden * 27 // 16


def csf_decode(fixed: np.ndarray, exceptions: np.ndarray, rows: int, ns: int) -> np.ndarray:
    """-> e4m3 scale bytes [rows, ns]. `fixed`: per 16 rows 16 base bytes (one per row), then each row's 4-bit offsets,
    low nibble first; scale byte = base + offset (mod 256). `exceptions`: little-endian u32 words, byte << 24 | flat
    index, holding the scale byte itself at that index."""
    fixed = np.ascontiguousarray(fixed, np.uint8).reshape(-1)
    stride = 16 + 16 * ns // 2
    if rows % 16 or ns % 2 or fixed.size != rows // 16 * stride:
        raise ValueError(f"CSF scales: {fixed.size} bytes for {rows} x {ns}")
    blk = fixed.reshape(rows // 16, stride)
    base = blk[:, :16].reshape(rows, 1)
    nib = blk[:, 16:].reshape(rows, ns // 2)
    out = np.empty((rows, ns), np.uint8)
    out[:, 0::2] = base + (nib & 15)                 # uint8 arithmetic wraps, as `wrapping_add`
    out[:, 1::2] = base + (nib >> 4)
    words = np.ascontiguousarray(exceptions, np.uint8).reshape(-1)
    if words.size % 4:
        raise ValueError("CSF exceptions: not a whole number of 32-bit words")
    words = words.view("<u4")
    at = (words & 0xFFFFFF).astype(np.int64)
    if at.size and at.max() >= rows * ns:
        raise ValueError(f"CSF exception index {int(at.max())} out of range")
    flat = out.reshape(-1)
    flat[at] = (words >> 24).astype(np.uint8)        # later entries win, as the reference's loop
    return out


def csf_encode(scales: np.ndarray):
    """Inverse of `csf_decode` for tests: base = the row's smallest byte, offsets up to 15, everything else an exception."""
    s = np.ascontiguousarray(scales, np.uint8)
    rows, ns = s.shape
    if rows % 16 or ns % 2:
        raise ValueError("CSF needs rows % 16 == 0 and an even number of scales per row")
    base = s.min(1, keepdims=True)
    off = (s - base).astype(np.uint8)
    exc = off > 15
    off = np.where(exc, 0, off).astype(np.uint8)
    nib = (off[:, 0::2] | (off[:, 1::2] << 4)).astype(np.uint8)
    fixed = np.concatenate([base.reshape(rows // 16, 16), nib.reshape(rows // 16, 16 * ns // 2)], 1).reshape(-1)
    at = np.flatnonzero(exc.reshape(-1)).astype(np.uint32)
    words = ((s.reshape(-1)[at].astype(np.uint32) << 24) | at).astype("<u4")
    return fixed, words.view(np.uint8)


def _get(tensors, name):
    try:
        return tensors[name]
    except KeyError:
        return None


def _check(a, name, dtype, shape):
    a = np.asarray(a)
    if a.dtype != dtype or tuple(a.shape) != tuple(shape):
        raise ValueError(f"{name}: {a.dtype}{list(a.shape)}, expected {np.dtype(dtype)}{list(shape)}")
    return a


def pack_experts(tensors, prefix: str, experts: int, hidden: int, inter: int, first: int = 0):
    """Routed experts [first, first + experts) under `prefix` (`...layers.<l>.mlp.experts`) ->
    (uint8 [experts * stride], float32 [experts, 3]); a rank of an expert-parallel group packs its own block only."""
    f, h = inter, hidden
    fh = f * h
    stride = expert_stride(h, f)
    buf = np.zeros(experts * stride, np.uint8)
    gs = np.zeros((experts, 3), np.float32)
    # (rows, cols, code offset, scale offset) per projection, weights.rs:459-463
    layout = ((f, h, 0, fh * 3 // 2), (f, h, fh // 2, fh * 3 // 2 + fh // 16), (h, f, fh, fh * 3 // 2 + fh // 8))
    for e in range(experts):
        base = e * stride
        for pi, (proj, (rows, cols, co, so)) in enumerate(zip(PROJECTIONS, layout)):
            p = f"{prefix}.{first + e}.{proj}"
            w = _get(tensors, f"{p}.weight_packed")
            packed = w is not None
            if not packed:
                w = _get(tensors, f"{p}.weight")
                if w is None:
                    raise KeyError(f"{p}.weight")
            w = _check(w, f"{p}.weight", np.uint8, (rows, cols // 2))
            buf[base + co:base + co + rows * cols // 2] = w.reshape(-1)
            fixed = _get(tensors, f"{p}.weight_scale.nvfp4_csf_fixed")
            if fixed is not None:
                fixed = _check(fixed, f"{p}.weight_scale.nvfp4_csf_fixed", np.uint8, (rows // 16, 16 + 16 * cols // 32))
                exc = _get(tensors, f"{p}.weight_scale.nvfp4_csf_exceptions")
                if exc is None:
                    raise KeyError(f"{p}.weight_scale.nvfp4_csf_exceptions")
                scales = csf_decode(fixed, exc, rows, cols // 16)
            else:
                s = _get(tensors, f"{p}.weight_scale")
                if s is None:
                    raise KeyError(f"{p}.weight_scale")
                s = np.asarray(s)
                if s.dtype.itemsize != 1 or tuple(s.shape) != (rows, cols // 16):
                    raise ValueError(f"{p}.weight_scale: expected e4m3 bytes [{rows}, {cols // 16}]")
                scales = s.view(np.uint8)
            buf[base + so:base + so + rows * cols // 16] = scales.reshape(-1)
            if packed:       # compressed-tensors divides by the global scale, ModelOpt multiplies (weights.rs:498-511)
                g = _get(tensors, f"{p}.weight_global_scale")
                if g is None:
                    raise KeyError(f"{p}.weight_global_scale")
                gs[e, pi] = np.float32(1.0) / np.asarray(g, np.float32).reshape(-1)[0]
            else:
                g = _get(tensors, f"{p}.weight_scale_2")
                if g is None:
                    raise KeyError(f"{p}.weight_scale_2")
                gs[e, pi] = np.asarray(g, np.float32).reshape(-1)[0]
    return buf, gs


class SafetensorsSource:
    """Mapping name -> numpy array over the `.safetensors` shards of a checkpoint directory (tensors are read on access;
    e4m3 tensors come back as their bytes)."""

    def __init__(self, paths):
        from safetensors import safe_open
        self._where, self._open = {}, safe_open
        for path in paths:
            with safe_open(path, framework="pt") as f:
                for name in f.keys():
                    self._where[name] = path

    def __getitem__(self, name):
        import torch
        path = self._where[name]                      # KeyError for an absent tensor
        with self._open(path, framework="pt") as f:
            t = f.get_tensor(name)
        if t.dtype in (torch.float8_e4m3fn,):
            return t.view(torch.uint8).numpy()
        if t.dtype == torch.bfloat16:
            return t.float().numpy()
        return t.numpy()

    def __contains__(self, name):
        return name in self._where
