"""Weight formats of the MoE hot path: byte layouts, decoders and quantizers (numpy).

Test infrastructure only (see the package docstring).  Every decoder restates a
formula of the reference engine and cites it; float32 rounding points are kept
where the reference has them (numpy float32 arithmetic rounds after every
operation and never contracts to FMA).
"""
from __future__ import annotations

import numpy as np

# ----------------------------------------------------------------------------
# scalar formats
# ----------------------------------------------------------------------------

E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)
#: code (0..15) -> value; bit 3 is the sign (tsumuji weights.rs:10-12, hayate math.cuh:42-48).
E2M1_TABLE = np.concatenate([E2M1_VALUES, -E2M1_VALUES]).astype(np.float32)
E2M1_MIDPOINTS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)


def _e4m3_table() -> np.ndarray:
    """e4m3 (no infinities; 0x7f / 0xff are NaN): hayate cu/glm53/math.cuh:17-22."""
    t = np.zeros(256, np.float32)
    for b in range(256):
        e, m = (b >> 3) & 15, b & 7
        if e == 15 and m == 7:
            v = np.nan
        elif e:
            v = np.ldexp(1.0 + m / 8.0, e - 7)
        else:
            v = np.ldexp(float(m), -9)
        t[b] = -v if b & 128 else v
    return t


E4M3_TABLE = _e4m3_table()
_E4M3_POS = E4M3_TABLE[:127].astype(np.float64)          # codes 0x00..0x7e, ascending
_E4M3_MID = (_E4M3_POS[:-1] + _E4M3_POS[1:]) / 2.0


def e4m3_decode(b: np.ndarray) -> np.ndarray:
    return E4M3_TABLE[np.asarray(b, np.uint8)]


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float -> e4m3 code, round to nearest even, saturating at +-448 (NaN -> 0x7f).

    Matches ``torch.Tensor.to(float8_e4m3fn)`` on inputs already clamped to
    [-448, 448] (hayate_tools/quant.py:55) and ``__nv_cvt_float_to_fp8(x,
    __NV_SATFINITE, __NV_E4M3)`` (tsumuji decode/quant.cu:104).
    """
    x = np.asarray(x, np.float32)
    a = np.abs(x).astype(np.float64)
    idx = np.searchsorted(_E4M3_MID, a, side="left")           # ties land on the lower code
    tie = (idx < 126) & (a == _E4M3_MID[np.minimum(idx, 125)])
    idx = np.where(tie & (idx % 2 == 1), idx + 1, idx)          # ... then move to the even one
    code = idx.astype(np.uint8) | (np.signbit(x).astype(np.uint8) << 7)
    return np.where(np.isnan(x), np.uint8(0x7F), code).astype(np.uint8)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest bf16 (ties to even), returned as float32. hayate math.cuh:23-30."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return u.view(np.float32)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    return (bf16_round(x).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


def bf16_from_bits(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def e2m1_encode(q: np.ndarray) -> np.ndarray:
    """Nearest e2m1 code of q (already divided by its scale); midpoint ties go to the even
    code, the sign bit follows signbit(q). hayate_tools/quant.py:58-64, tests/test_quant.py:135-145;
    the CUDA conversion used by tsumuji decode/quant.cu:111 rounds the same way."""
    q = np.asarray(q, np.float32)
    a = np.abs(q)
    idx = np.searchsorted(E2M1_MIDPOINTS, a, side="left").astype(np.uint8)
    idx = idx + ((a == 0.75) | (a == 1.75) | (a == 3.5)).astype(np.uint8)
    return (idx | (np.signbit(q).astype(np.uint8) << 3)).astype(np.uint8)


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """Element 2i in the low nibble, 2i+1 in the high nibble (row-major flattening)."""
    flat = np.asarray(codes, np.uint8).reshape(-1)
    return (flat[0::2] | (flat[1::2] << 4)).astype(np.uint8)


def unpack_nibbles(payload: np.ndarray) -> np.ndarray:
    p = np.asarray(payload, np.uint8).reshape(-1)
    return np.stack([p & 15, p >> 4], -1).reshape(-1)


# ----------------------------------------------------------------------------
# GGUF Q4_K / Q6_K  (kogarashi kernels/native.cu:21-41, 52-82; sizes config.rs:86-105)
# ----------------------------------------------------------------------------

GGML_F32, GGML_F16, GGML_Q4_K, GGML_Q6_K, GGML_BF16 = 0, 1, 12, 14, 30
Q4K_BLOCK_BYTES, Q6K_BLOCK_BYTES, QK_K = 144, 210, 256


def ggml_tensor_bytes(ty: int, ne) -> int:
    """Byte size of a contiguous GGML tensor; restates kogarashi config.rs:86-105."""
    block, size = {0: (1, 4), 1: (1, 2), 30: (1, 2), 12: (256, 144), 14: (256, 210)}[ty]
    if not ne or ne[0] == 0 or ne[0] % block or 0 in ne:
        raise ValueError("invalid tensor shape/block alignment")
    n = 1
    for d in ne:
        n *= int(d)
    return n // block * size


def q4k_decode(raw: np.ndarray) -> np.ndarray:
    """[..., 144] bytes -> [..., 256] float32, value = (d*sc)*q - dmin*m with every product
    rounded to float32 (native.cu:26-34)."""
    b = np.asarray(raw, np.uint8).reshape(-1, Q4K_BLOCK_BYTES)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)          # [nb,1]
    dmin = b[:, 2:4].copy().view(np.float16).astype(np.float32)
    s = b[:, 4:16].astype(np.int32)
    sc = np.empty((b.shape[0], 8), np.int32)
    mi = np.empty((b.shape[0], 8), np.int32)
    sc[:, :4] = s[:, 0:4] & 63
    mi[:, :4] = s[:, 4:8] & 63
    sc[:, 4:] = (s[:, 8:12] & 15) | ((s[:, 0:4] >> 6) << 4)
    mi[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
    qs = b[:, 16:144].reshape(-1, 4, 32)                                # byte (j/64)*32 + (j&31)
    q = np.stack([qs & 15, qs >> 4], 2).reshape(-1, 8, 32).astype(np.float32)   # sub-block g = 2*(j/64)+(g&1)
    dsc = (d * sc.astype(np.float32)).astype(np.float32)[:, :, None]
    dm = (dmin * mi.astype(np.float32)).astype(np.float32)[:, :, None]
    val = (dsc * q).astype(np.float32) - dm
    return val.astype(np.float32).reshape(*np.shape(raw)[:-1], QK_K)


def q6k_decode(raw: np.ndarray) -> np.ndarray:
    """[..., 210] bytes -> [..., 256] float32, value = (d*scale)*(q-32) (native.cu:35-40)."""
    b = np.asarray(raw, np.uint8).reshape(-1, Q6K_BLOCK_BYTES)
    nb = b.shape[0]
    ql = b[:, 0:128].reshape(nb, 2, 2, 32)        # [n][g&1][l]
    qh = b[:, 128:192].reshape(nb, 2, 32)         # [n][l]
    sc = b[:, 192:208].copy().view(np.int8).astype(np.float32)   # index j // 16
    d = b[:, 208:210].copy().view(np.float16).astype(np.float32)
    q = np.empty((nb, 2, 4, 32), np.int32)        # [n][g][l]
    for g in range(4):
        lo = (ql[:, :, g & 1, :].astype(np.int32) >> ((g // 2) * 4)) & 15
        hi = (qh.astype(np.int32) >> (g * 2)) & 3
        q[:, :, g, :] = lo | (hi << 4)
    q = q.reshape(nb, 16, 16)
    dsc = (d * sc).astype(np.float32)[:, :, None]
    val = (dsc * (q - 32).astype(np.float32)).astype(np.float32)
    return val.reshape(*np.shape(raw)[:-1], QK_K)


def _nearest_int(x):
    return np.floor(x + 0.5)


def q4k_quantize(w: np.ndarray) -> np.ndarray:
    """float32 [..., K] (K % 256 == 0) -> bytes [..., K/256*144].

    Written from the block layout that native.cu decodes; the reference has no Q4_K
    quantizer (weights arrive quantized by an un-vendored llama.cpp build), so the choice of
    scales below is this project's own: min/max per 32-element sub-block, 6-bit scales and
    mins against the super-block maxima. Parity of this function is unpinned.
    """
    w = np.asarray(w, np.float32)
    lead, k = w.shape[:-1], w.shape[-1]
    assert k % QK_K == 0
    x = w.reshape(-1, 8, 32)
    lo = np.minimum(x.min(-1), 0.0)
    hi = np.maximum(x.max(-1), 0.0)
    sub_scale = (hi - lo) / 15.0
    sub_min = np.float32(0) - lo          # +0 for an all-zero sub-block
    d = (sub_scale.max(-1) / 63.0).astype(np.float16)
    dmin = (sub_min.max(-1) / 63.0).astype(np.float16)
    df, dmf = d.astype(np.float32)[:, None], dmin.astype(np.float32)[:, None]
    sc = np.where(df > 0, _nearest_int(sub_scale / np.where(df > 0, df, 1)), 0).clip(0, 63).astype(np.int32)
    mi = np.where(dmf > 0, _nearest_int(sub_min / np.where(dmf > 0, dmf, 1)), 0).clip(0, 63).astype(np.int32)
    step = (df * sc.astype(np.float32)).astype(np.float32)[:, :, None]
    off = (dmf * mi.astype(np.float32)).astype(np.float32)[:, :, None]
    q = np.where(step > 0, _nearest_int((x + off) / np.where(step > 0, step, 1)), 0).clip(0, 15).astype(np.uint8)
    out = np.zeros((x.shape[0], Q4K_BLOCK_BYTES), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = dmin.view(np.uint8).reshape(-1, 2)
    s = np.zeros((x.shape[0], 12), np.int32)
    s[:, 0:4] = sc[:, :4] | ((sc[:, 4:] >> 4) << 6)
    s[:, 4:8] = mi[:, :4] | ((mi[:, 4:] >> 4) << 6)
    s[:, 8:12] = (sc[:, 4:] & 15) | ((mi[:, 4:] & 15) << 4)
    out[:, 4:16] = s.astype(np.uint8)
    qg = q.reshape(-1, 4, 2, 32)
    out[:, 16:144] = (qg[:, :, 0, :] | (qg[:, :, 1, :] << 4)).reshape(-1, 128)
    return out.reshape(*lead, k // QK_K * Q4K_BLOCK_BYTES)


def q6k_quantize(w: np.ndarray) -> np.ndarray:
    """float32 [..., K] -> bytes [..., K/256*210]; fresh quantizer (see q4k_quantize): one int8
    scale per 16 elements against the super-block maximum, symmetric 6-bit codes. Unpinned."""
    w = np.asarray(w, np.float32)
    lead, k = w.shape[:-1], w.shape[-1]
    assert k % QK_K == 0
    x = w.reshape(-1, 16, 16)
    sub = np.abs(x).max(-1) / 31.0
    d = (sub.max(-1) / 127.0).astype(np.float16)
    df = d.astype(np.float32)[:, None]
    sc = np.where(df > 0, _nearest_int(sub / np.where(df > 0, df, 1)), 0).clip(0, 127).astype(np.int32)
    step = (df * sc.astype(np.float32)).astype(np.float32)[:, :, None]
    q = (np.where(step > 0, _nearest_int(x / np.where(step > 0, step, 1)), 0).clip(-32, 31) + 32).astype(np.uint8)
    nb = x.shape[0]
    qv = q.reshape(nb, 2, 4, 32)                       # [n][g][l]
    out = np.zeros((nb, Q6K_BLOCK_BYTES), np.uint8)
    ql = np.zeros((nb, 2, 2, 32), np.uint8)
    qh = np.zeros((nb, 2, 32), np.uint8)
    for g in range(4):
        ql[:, :, g & 1, :] |= ((qv[:, :, g, :] & 15) << ((g // 2) * 4)).astype(np.uint8)
        qh |= ((qv[:, :, g, :] >> 4) << (g * 2)).astype(np.uint8)
    out[:, 0:128] = ql.reshape(nb, 128)
    out[:, 128:192] = qh.reshape(nb, 64)
    out[:, 192:208] = sc.astype(np.int8).view(np.uint8)
    out[:, 208:210] = d.view(np.uint8).reshape(-1, 2)
    return out.reshape(*lead, k // QK_K * Q6K_BLOCK_BYTES)


def ggml_decode(raw: np.ndarray, ty: int, k: int) -> np.ndarray:
    """Rows of a GGML tensor (any leading shape, last axis = row bytes) -> float32 [..., k]."""
    if ty == GGML_Q4_K:
        return q4k_decode(raw.reshape(*raw.shape[:-1], k // QK_K, Q4K_BLOCK_BYTES)).reshape(*raw.shape[:-1], k)
    if ty == GGML_Q6_K:
        return q6k_decode(raw.reshape(*raw.shape[:-1], k // QK_K, Q6K_BLOCK_BYTES)).reshape(*raw.shape[:-1], k)
    if ty == GGML_F32:
        return raw.view(np.float32).reshape(*raw.shape[:-1], k)
    if ty == GGML_F16:
        return raw.view(np.float16).astype(np.float32).reshape(*raw.shape[:-1], k)
    if ty == GGML_BF16:
        return bf16_from_bits(raw.view(np.uint16)).reshape(*raw.shape[:-1], k)
    raise ValueError(f"unsupported GGML type {ty}")


def ggml_quantize(w: np.ndarray, ty: int) -> np.ndarray:
    if ty == GGML_Q4_K:
        return q4k_quantize(w)
    if ty == GGML_Q6_K:
        return q6k_quantize(w)
    if ty == GGML_F32:
        return np.ascontiguousarray(w, np.float32).view(np.uint8)
    if ty == GGML_BF16:
        return bf16_bits(w).view(np.uint8)
    raise ValueError(f"unsupported GGML type {ty}")


# ----------------------------------------------------------------------------
# NVFP4, Hayate tiled layout (math.cuh:41-49, dtype.rs:85-105,160-197, quant.py:11-64)
# ----------------------------------------------------------------------------

def _align(v: int, a: int) -> int:
    return (v + a - 1) // a * a


def nvfp4_tiled_bytes(n: int, k: int) -> int:
    """codes n*k/2, scales pad128(n)*pad4(k/16), one float32 (dtype.rs:50-52,104,204-217)."""
    return n * k // 2 + _align(n, 128) * _align(k // 16, 4) + 4


def nvfp4_scale_offset(row, col, padded_cols):
    """Byte of scale (row, col) inside the tiled scale area (quant.py:11-12, math.cuh:45)."""
    return ((row // 128) * (padded_cols // 4) + col // 4) * 512 + (row % 32) * 16 + (row % 128 // 32) * 4 + col % 4


def _positive_scale(maximum, divisor):
    minimum = np.float32(np.finfo(np.float32).tiny) * np.float32(np.finfo(np.float32).eps)
    with np.errstate(divide="ignore", invalid="ignore"):
        v = np.maximum((maximum / np.float32(divisor)).astype(np.float32), minimum)
    return np.where(maximum == 0, np.float32(1.0), v).astype(np.float32)


def nvfp4_tiled_quantize(w: np.ndarray) -> np.ndarray:
    """float32 [n, k] -> Hayate NVFP4 matrix image (codes | tiled scales | global).
    Restates hayate_tools/quant.py:42-64 operation by operation in float32."""
    w = np.asarray(w, np.float32)
    n, k = w.shape
    assert k % 16 == 0
    x = w.reshape(n, k // 16, 16)
    ms = _positive_scale(np.abs(x).max().astype(np.float32), 6.0 * 448.0)
    bmax = np.abs(x).max(-1).astype(np.float32)
    sc = np.clip(((bmax / ms).astype(np.float32) / np.float32(6.0)).astype(np.float32), 0, 448)
    scode = e4m3_encode(sc)
    dec = e4m3_decode(scode)
    norm = ((x / ms).astype(np.float32) / np.where(dec == 0, np.float32(1), dec)[:, :, None]).astype(np.float32)
    codes = e2m1_encode(np.abs(norm)) | (np.signbit(x).astype(np.uint8) << 3)
    cols = _align(k // 16, 4)
    tiles = np.zeros(_align(n, 128) * cols, np.uint8)
    r, c = np.meshgrid(np.arange(n), np.arange(k // 16), indexing="ij")
    tiles[nvfp4_scale_offset(r, c, cols)] = scode
    return np.concatenate([pack_nibbles(codes), tiles, np.array([ms], np.float32).view(np.uint8)])


def nvfp4_tiled_parts(image: np.ndarray, n: int, k: int):
    """-> (codes uint8 [n,k], scale codes uint8 [n,k/16], global float32)."""
    image = np.asarray(image, np.uint8)
    codes = unpack_nibbles(image[: n * k // 2]).reshape(n, k)
    cols = _align(k // 16, 4)
    r, c = np.meshgrid(np.arange(n), np.arange(k // 16), indexing="ij")
    sc = image[n * k // 2 + nvfp4_scale_offset(r, c, cols)]
    at = n * k // 2 + _align(n, 128) * cols
    g = image[at:at + 4].copy().view(np.float32)[0]
    return codes, sc, g


def nvfp4_tiled_decode(image: np.ndarray, n: int, k: int, scaled: bool = True, rounded: bool = False) -> np.ndarray:
    """value = e2m1 * (e4m3 * global) as the decode kernels form it (dense.cuh:32-37,61-73);
    `rounded` applies the bf16 rounding of the FP8 / shared-expert path."""
    codes, sc, g = nvfp4_tiled_parts(image, n, k)
    mult = (e4m3_decode(sc) * (g if scaled else np.float32(1))).astype(np.float32)
    v = (E2M1_TABLE[codes].reshape(n, k // 16, 16) * mult[:, :, None]).astype(np.float32).reshape(n, k)
    return bf16_round(v) if rounded else v


def hayate_expert_stride(hidden: int, inter: int) -> int:
    """256-byte aligned stride between gate | up | down of one image (lowbit.cuh:9-13,
    experts.rs:68-74). With hidden and inter multiples of 256 all three strides agree."""
    return _align(nvfp4_tiled_bytes(inter, hidden), 256)


def hayate_expert_image(gate: np.ndarray, up: np.ndarray, down: np.ndarray) -> np.ndarray:
    inter, hidden = gate.shape
    stride = hayate_expert_stride(hidden, inter)
    assert _align(nvfp4_tiled_bytes(hidden, inter), 256) == stride
    img = np.zeros(3 * stride, np.uint8)
    for i, m in enumerate((gate, up, down)):
        q = nvfp4_tiled_quantize(m)
        img[i * stride:i * stride + q.size] = q
    return img


# ----------------------------------------------------------------------------
# NVFP4, Tsumuji linear layout (weights.rs:10-12,334-336,448-509; quant.cu:88-114)
# ----------------------------------------------------------------------------

def nvfp4_linear_quantize(w: np.ndarray):
    """bf16-valued float32 [rows, k] -> (codes uint8 [rows,k/2], scales uint8 [rows,k/16], global f32).
    Restates tsumuji decode/quant.cu:88-114: global = amax/(6*448) (1 if zero),
    scale = e4m3(blockmax/6/global), code = e2m1(x / (e4m3(scale)*global))."""
    w = bf16_round(np.asarray(w, np.float32))
    rows, k = w.shape
    x = w.reshape(rows, k // 16, 16)
    g = (np.abs(x).max().astype(np.float32) / (np.float32(6.0) * np.float32(448.0))).astype(np.float32)
    if g == 0:
        g = np.float32(1.0)
    a = np.abs(x).max(-1).astype(np.float32)
    scode = e4m3_encode(((a / np.float32(6.0)).astype(np.float32) / g).astype(np.float32))
    d = (e4m3_decode(scode) * g).astype(np.float32)[:, :, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(d > 0, (x / np.where(d > 0, d, 1)).astype(np.float32), np.float32(0))
    codes = e2m1_encode(q).reshape(rows, k)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return packed, scode, np.float32(g)


def nvfp4_linear_decode(packed: np.ndarray, scode: np.ndarray, g=None) -> np.ndarray:
    """-> float32 [rows, k] of e2m1 * e4m3 (exact), times `g` if given."""
    rows = packed.shape[0]
    codes = np.stack([packed & 15, packed >> 4], -1).reshape(rows, -1)
    v = (E2M1_TABLE[codes].reshape(rows, -1, 16) * e4m3_decode(scode)[:, :, None]).reshape(rows, -1)
    return v if g is None else (v * np.float32(g)).astype(np.float32)


def tsumuji_expert_block(gate, up, down):
    """One routed expert: [gate codes | up codes | down codes | gate sf | up sf | down sf],
    27/16*F*H bytes, plus the three global scales (weights.rs:10-12, gemv.cu:97-103,149-153)."""
    parts = [nvfp4_linear_quantize(m) for m in (gate, up, down)]
    block = np.concatenate([p[0].reshape(-1) for p in parts] + [p[1].reshape(-1) for p in parts])
    f, h = gate.shape
    assert block.size == f * h * 27 // 16
    return block, np.array([p[2] for p in parts], np.float32)


def tsumuji_block_decode(block: np.ndarray, gs: np.ndarray, h: int, f: int):
    """-> (gate [F,H], up [F,H], down [H,F]) float32 without the global scales applied,
    and gs; the dot kernels multiply by gs after the row sum (gemv.cu:104-105,153)."""
    fh = f * h
    cg, cu, cd = block[:fh // 2], block[fh // 2:fh], block[fh:fh * 3 // 2]
    s0 = fh * 3 // 2
    sg, su, sd = block[s0:s0 + fh // 16], block[s0 + fh // 16:s0 + fh // 8], block[s0 + fh // 8:s0 + fh * 3 // 16]
    gate = nvfp4_linear_decode(cg.reshape(f, h // 2), sg.reshape(f, h // 16))
    up = nvfp4_linear_decode(cu.reshape(f, h // 2), su.reshape(f, h // 16))
    down = nvfp4_linear_decode(cd.reshape(h, f // 2), sd.reshape(h, f // 16))
    return gate, up, down


# ----------------------------------------------------------------------------
# block FP8 (hayate cpu/glm53.rs:23-24,42-46,119-120; ops.cu:13-16; math.cuh:40)
# ----------------------------------------------------------------------------

def fp8_block_bytes(n: int, k: int) -> int:
    return n * k + ((n + 127) // 128) * ((k + 127) // 128) * 4


def fp8_block_quantize(w: np.ndarray):
    """float32 [n,k] -> (payload uint8 [n,k], scales float32 [ceil(n/128), ceil(k/128)]) with
    scale = absmax/448 per 128x128 block (1 for an all-zero block)."""
    w = np.asarray(w, np.float32)
    n, k = w.shape
    nb, kb = (n + 127) // 128, (k + 127) // 128
    pad = np.zeros((nb * 128, kb * 128), np.float32)
    pad[:n, :k] = w
    blk = pad.reshape(nb, 128, kb, 128)
    amax = np.abs(blk).max((1, 3)).astype(np.float32)
    scale = np.where(amax == 0, np.float32(1), (amax / np.float32(448.0)).astype(np.float32)).astype(np.float32)
    q = (blk / scale[:, None, :, None]).astype(np.float32).clip(-448, 448)
    payload = e4m3_encode(q).reshape(nb * 128, kb * 128)[:n, :k]
    return np.ascontiguousarray(payload), scale


def fp8_block_image(w: np.ndarray) -> np.ndarray:
    p, s = fp8_block_quantize(w)
    return np.concatenate([p.reshape(-1), s.reshape(-1).view(np.uint8)])


def fp8_block_decode(payload: np.ndarray, scale: np.ndarray, rounded: bool = True) -> np.ndarray:
    """weight = bf16(fp8(byte) * scale) on the Hayate decode path (math.cuh:40); `rounded=False`
    gives the raw product."""
    n, k = payload.shape
    s = np.repeat(np.repeat(scale, 128, 0)[:n], 128, 1)[:, :k]
    v = (e4m3_decode(payload) * s).astype(np.float32)
    return bf16_round(v) if rounded else v


def fp8_act_quantize(x: np.ndarray):
    """Activations -> (e4m3 codes [T,H], float32 scales [T,H/128]), scale = absmax/448 of each
    128-channel group of a token (1 where the group is zero); code = e4m3(x * (1/scale)) with the
    reciprocal rounded to float32 (one division per group, a multiplication per element)."""
    x = np.asarray(x, np.float32)
    t, h = x.shape
    g = x.reshape(t, h // 128, 128)
    amax = np.abs(g).max(-1).astype(np.float32)
    scale = np.where(amax == 0, np.float32(1), (amax / np.float32(448.0)).astype(np.float32)).astype(np.float32)
    inv = (np.float32(1.0) / scale).astype(np.float32)
    q = (g * inv[:, :, None]).astype(np.float32).clip(-448, 448)
    return e4m3_encode(q).reshape(t, h), scale
