"""Byte-size arithmetic of the weight layouts the kernels read (host side, no numerics).

Mirrors `tensor_bytes` (engines/kogarashi/crates/kogarashi-engine/src/config.rs:86-105) and
`QuantSpec::matrix_bytes` (common/core/src/dtype.rs:94-197) of the reference.
"""
from __future__ import annotations

GGML_F32, GGML_F16, GGML_Q4_K, GGML_Q6_K, GGML_BF16 = 0, 1, 12, 14, 30
_GGML = {GGML_F32: (1, 4), GGML_F16: (1, 2), GGML_BF16: (1, 2), GGML_Q4_K: (256, 144), GGML_Q6_K: (256, 210)}


def ggml_tensor_bytes(ty: int, ne) -> int:
    """Bytes of a contiguous GGML tensor; quantized rows must hold complete blocks."""
    if ty not in _GGML:
        raise ValueError(f"unsupported GGML type {ty}")
    block, size = _GGML[ty]
    ne = [int(d) for d in ne]
    if not ne or ne[0] == 0 or ne[0] % block or 0 in ne:
        raise ValueError("invalid tensor shape/block alignment")
    n = 1
    for d in ne:
        n *= d
    return n // block * size


def _align(v: int, a: int) -> int:
    return (v + a - 1) // a * a


def nvfp4_tiled_bytes(rows: int, cols: int) -> int:
    """Hayate NVFP4 matrix: e2m1 payload, e4m3 scales in 128x4 tiles, one float32."""
    if cols % 16:
        raise ValueError("NVFP4 K must be divisible by 16")
    return rows * cols // 2 + _align(rows, 128) * _align(cols // 16, 4) + 4


def nvfp4_expert_stride(hidden: int, inter: int) -> int:
    """256-byte aligned distance between gate | up | down of a Hayate expert image."""
    return _align(nvfp4_tiled_bytes(inter, hidden), 256)


def nvfp4_linear_expert_bytes(hidden: int, inter: int) -> int:
    """Tsumuji routed-expert block: three code planes then three scale planes."""
    return hidden * inter * 27 // 16


def fp8_block_bytes(rows: int, cols: int) -> int:
    return rows * cols + _align(rows, 128) // 128 * (_align(cols, 128) // 128) * 4


def q6k_r16_row_bytes(k: int) -> int:
    """Row bytes of the 16-byte aligned device layout of Q6_K (see darask_q6k_repack)."""
    return k // 256 * 208 + _align(2 * (k // 256), 16)
