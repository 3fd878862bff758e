"""The arithmetic of the one-token decode kernel, restated in numpy and held against the float64 value of the same
quantized weights: activations as 16-bit fixed point of the largest magnitude inside their own scale group (32 columns
for Q4_K, 16 for Q6_K), split into two signed bytes; exact integer sums of code x byte per group; 1 / S, the group scales,
the Q4_K minimum (through the group's activation sum) and the Q6_K offset 32 (through the group's integer sum) applied in
float32 (darask-inference-engine_b200/csrc/decode_fused.cuh: `split_bytes4`, `q4k_rows`, `q6k_rows`).  The point of the
test is the error bound for inputs a layer can meet: outliers, tiny values, empty groups."""
import numpy as np
import pytest

from oracle import formats as F

RANGE = np.float32(32000.0)


def fixed_point(x, group):
    """-> (hi, lo int8-valued int32 [.., k], inv float32 per group, integer sum per group) as the kernel forms them."""
    x = np.asarray(x, np.float32).reshape(-1, group)
    top = np.abs(x).max(1).astype(np.float32)
    s = np.where(top > 0, RANGE / np.where(top > 0, top, 1), 0).astype(np.float32)
    inv = (top * (np.float32(1.0) / RANGE)).astype(np.float32)
    xi = np.rint((x * s[:, None]).astype(np.float32)).astype(np.int32)
    lo = ((xi + 128) & 255) - 128
    hi = (xi - lo) >> 8
    assert np.all(np.abs(hi) <= 125) and np.all((lo >= -128) & (lo <= 127)) and np.array_equal(256 * hi + lo, xi)
    return hi, lo, inv, xi.sum(1)


def q4k_parts(raw):
    b = np.asarray(raw, np.uint8).reshape(-1, 144)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)[:, 0]
    dmin = b[:, 2:4].copy().view(np.float16).astype(np.float32)[:, 0]
    s = b[:, 4:16].astype(np.int32)
    sc = np.concatenate([s[:, 0:4] & 63, (s[:, 8:12] & 15) | ((s[:, 0:4] >> 6) << 4)], 1)
    mi = np.concatenate([s[:, 4:8] & 63, (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)], 1)
    qs = b[:, 16:144].reshape(-1, 4, 32)
    q = np.stack([qs & 15, qs >> 4], 2).reshape(-1, 8, 32).astype(np.int64)
    return d, dmin, sc, mi, q


def q4k_dot_fixed_point(raw, x):
    """One row of Q4_K blocks times x, the kernel's way; float32 sums per block row as the lanes keep them."""
    d, dmin, sc, mi, q = q4k_parts(raw)
    nb = d.size
    hi, lo, inv, xsum = fixed_point(x, 32)
    hi, lo = hi.reshape(nb, 8, 32), lo.reshape(nb, 8, 32)
    inv, xsum = inv.reshape(nb, 8), xsum.reshape(nb, 8)
    c_hi, c_lo = (q * hi).sum(2), (q * lo).sum(2)                              # exact integers, as the s32 accumulators
    assert np.abs(256 * c_hi + c_lo).max() < 2 ** 31
    raw_sum = ((256 * c_hi + c_lo).astype(np.float32) * inv).astype(np.float32)
    xs = (inv * xsum.astype(np.float32)).astype(np.float32)
    acc = np.float32(0)
    for b in range(nb):
        for g in range(8):
            acc = np.float32(acc + np.float32(d[b] * np.float32(sc[b, g])) * raw_sum[b, g])
            acc = np.float32(acc - np.float32(dmin[b] * np.float32(mi[b, g])) * xs[b, g])
    return acc


def q6k_dot_fixed_point(raw, x):
    b = np.asarray(raw, np.uint8).reshape(-1, 210)
    nb = b.shape[0]
    ql, qh = b[:, 0:128].reshape(nb, 2, 2, 32), b[:, 128:192].reshape(nb, 2, 32)
    sc = b[:, 192:208].copy().view(np.int8).astype(np.float32)
    d = b[:, 208:210].copy().view(np.float16).astype(np.float32)[:, 0]
    q = np.empty((nb, 2, 4, 32), np.int64)                                      # unsigned 6-bit codes, formats.q6k_decode's order
    for g in range(4):
        q[:, :, g, :] = ((ql[:, :, g & 1, :].astype(np.int64) >> ((g // 2) * 4)) & 15) | (((qh.astype(np.int64) >> (g * 2)) & 3) << 4)
    q = q.reshape(nb, 16, 16)
    hi, lo, inv, xsum = fixed_point(x, 16)
    hi, lo = hi.reshape(nb, 16, 16), lo.reshape(nb, 16, 16)
    inv, xsum = inv.reshape(nb, 16), xsum.reshape(nb, 16)
    c = 256 * (q * hi).sum(2) + (q * lo).sum(2)
    acc = np.float32(0)
    for bi in range(nb):
        for g in range(16):
            scale = np.float32(np.float32(d[bi] * inv[bi, g]) * sc[bi, g])
            acc = np.float32(acc + scale * np.float32(np.float32(-32.0) * np.float32(xsum[bi, g]) + np.float32(c[bi, g])))
    return acc


def activations(kind, k, rng):
    x = rng.standard_normal(k).astype(np.float32)
    if kind == "outliers":
        x[rng.integers(0, k, 4)] *= np.float32(3000.0)
    elif kind == "heavy_tail":
        x = (rng.standard_cauchy(k)).astype(np.float32)
    elif kind == "tiny":
        x *= np.float32(1e-30)
    elif kind == "empty_groups":
        x[64:160] = 0
        x[512:] = 0
    return x


@pytest.mark.parametrize("kind", ["normal", "outliers", "heavy_tail", "tiny", "empty_groups"])
@pytest.mark.parametrize("ty", [F.GGML_Q4_K, F.GGML_Q6_K])
def test_fixed_point_rows_against_float64(ty, kind):
    rng = np.random.default_rng(11)
    k, rows = 1024, 48
    w = F.ggml_quantize((rng.standard_normal((rows, k)) * 0.02).astype(np.float32), ty)
    x = activations(kind, k, rng)
    exact = F.ggml_decode(w, ty, k).astype(np.float64) @ x.astype(np.float64)
    dot = q4k_dot_fixed_point if ty == F.GGML_Q4_K else q6k_dot_fixed_point
    got = np.array([dot(w[r], x) for r in range(rows)], np.float64)
    err = np.linalg.norm(got - exact) / np.linalg.norm(exact)
    # a tenth of the layer tolerance (1e-3), whatever the shape of the activations
    assert err < 1e-4, err


def test_nvfp4_code_times_scale_is_exact_in_fp16_and_bf16():
    """The packed NVFP4 grouped GEMM multiplies e2m1 code by e4m3 block scale in fp16 and stores bf16 in front of the
    tensor core (csrc/grouped_nvfp4.cuh `expand8`): every one of the 16 x 254 finite products must be exactly
    representable in both, so that the tile holds the same weights the reference decodes (packed_grouped.cu:103-108)."""
    codes = F.E2M1_TABLE.astype(np.float64)                                  # 16 signed values
    scales = F.e4m3_decode(np.arange(256, dtype=np.uint8)).astype(np.float64)
    scales = scales[np.isfinite(scales)]
    prod = codes[:, None] * scales[None, :]
    assert np.array_equal(prod.astype(np.float16).astype(np.float64), prod)
    assert np.array_equal(F.bf16_round(prod.astype(np.float32)).astype(np.float64), prod)


def test_tags_of_the_one_token_kernel():
    """`make_tag` (csrc/decode_fused.cuh): the tag of a call is never zero (a cleared workspace) and never the bit pattern of
    -0.0f, and consecutive calls differ."""
    tag = lambda epoch: (0x80000001 + epoch % 0x7FFFFFFE) & 0xFFFFFFFF
    for e in (0, 1, 2, 0x7FFFFFFD, 0x7FFFFFFE, 0x7FFFFFFF, 0xFFFFFFFE, 0xFFFFFFFF):
        assert tag(e) not in (0, 0x80000000) and tag(e) >> 31 == 1
        assert tag(e) != tag((e + 1) & 0xFFFFFFFF)
