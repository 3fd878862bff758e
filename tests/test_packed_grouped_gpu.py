"""hayate_glm_grouped_packed_{gate_up,down}: ragged grouped GEMM on packed NVFP4 expert images read in place.

Tier A: the same calls into the reference's own launchers (cu/glm53/packed_grouped.cu compiled unmodified into
oracle/_ref/libhayate_ref.so) and into this library, same device buffers.  Tier B: a float64 restatement of the
reference's arithmetic (packed_grouped.cu:177-266) on the decoded images."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import formats as F
from tests import workloads as W

pytestmark = pytest.mark.gpu
HAYATE_SO = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "oracle", "_ref", "libhayate_ref.so")
P, U = ctypes.c_void_p, ctypes.c_uint


def build_case(seed, hidden, inter, rows_per_expert):
    import darask_inference_engine_b200 as D
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    stride = D.formats.nvfp4_expert_stride(hidden, inter)
    count = len(rows_per_expert)
    images = []
    for _ in range(count):
        buf = torch.zeros(3 * stride, dtype=torch.uint8, device=dev)
        for part, shp in enumerate(((inter, hidden), (inter, hidden), (hidden, inter))):
            m = D.quantize.nvfp4_tiled(torch.randn(shp, generator=gen, device=dev) * 0.05)
            buf[part * stride:part * stride + m.numel()] = m
        images.append(buf)
    table = torch.tensor([b.data_ptr() for b in images], dtype=torch.int64, device=dev)
    formats = torch.zeros(count * 8, dtype=torch.uint8, device=dev)
    offsets = np.concatenate([[0], np.cumsum(rows_per_expert)[:-1]])
    ranges = torch.tensor(np.stack([rows_per_expert, offsets], 1).astype(np.uint32).view(np.int32), dtype=torch.int32, device=dev)
    total = int(np.sum(rows_per_expert))
    x = torch.randn(total, hidden, generator=gen, device=dev).bfloat16()
    return dict(images=images, table=table, formats=formats, ranges=ranges, x=x, total=total, stride=stride, count=count,
                hidden=hidden, inter=inter, rows=list(rows_per_expert), offsets=offsets)


def run(lib, case):
    st = torch.cuda.current_stream().cuda_stream
    dev = case["x"].device
    # poisoned outputs: rows the kernels must not touch stay recognisable, rows they own must be overwritten
    product = torch.full((case["total"], case["inter"]), 7.0, dtype=torch.bfloat16, device=dev)
    out = torch.full((case["total"], case["hidden"]), 7.0, dtype=torch.bfloat16, device=dev)
    for name in ("hayate_glm_grouped_packed_gate_up", "hayate_glm_grouped_packed_down"):
        getattr(lib, name).argtypes, getattr(lib, name).restype = [P, P, P, P, P, U, U, U, P], ctypes.c_int
    assert lib.hayate_glm_grouped_packed_gate_up(product.data_ptr(), case["x"].data_ptr(), case["table"].data_ptr(), case["formats"].data_ptr(),
                                                 case["ranges"].data_ptr(), case["count"], case["hidden"], case["inter"], st) == 0, lib
    assert lib.hayate_glm_grouped_packed_down(out.data_ptr(), product.data_ptr(), case["table"].data_ptr(), case["formats"].data_ptr(),
                                              case["ranges"].data_ptr(), case["count"], case["hidden"], case["inter"], st) == 0
    torch.cuda.synchronize()
    return product.float().cpu().numpy(), out.float().cpu().numpy()


CASES = [(3, 512, 256, [5, 0, 130, 1, 77]), (4, 1024, 512, [300, 17, 0, 0, 128, 129, 64, 1, 255])]


@pytest.mark.skipif(not os.path.exists(HAYATE_SO), reason="oracle/_ref/libhayate_ref.so is built where the reference checkout is present")
@pytest.mark.parametrize("seed,hidden,inter,rows", CASES)
def test_packed_grouped_against_reference_launchers(seed, hidden, inter, rows):
    import darask_inference_engine_b200 as D
    case = build_case(seed, hidden, inter, rows)
    ref = ctypes.CDLL(HAYATE_SO)
    p_ref, o_ref = run(ref, case)
    p_mine, o_mine = run(D._lib.lib(), case)
    status = ctypes.c_uint(99)
    assert D._lib.lib().hayate_glm_grouped_packed_status(ctypes.byref(status), torch.cuda.current_stream().cuda_stream) == 0
    assert status.value == 0
    # bf16 outputs of float32 sums taken in a different order: one bf16 step of the largest value, 4e-3 in L2
    W.check_output(p_mine, p_ref, rel=4e-3, max_abs=2.0 ** -7)
    W.check_output(o_mine, o_ref, rel=4e-3, max_abs=2.0 ** -7)


def test_packed_grouped_against_oracle():
    import darask_inference_engine_b200 as D
    seed, hidden, inter, rows = CASES[0]
    case = build_case(seed, hidden, inter, rows)
    p_mine, o_mine = run(D._lib.lib(), case)
    x = case["x"].float().cpu().numpy().astype(np.float64)
    stride = case["stride"]
    for e, (r, off) in enumerate(zip(case["rows"], case["offsets"])):
        if r == 0:
            continue
        img = case["images"][e].cpu().numpy()
        mats = []
        for part, (n, k) in enumerate(((inter, hidden), (inter, hidden), (hidden, inter))):
            m = img[part * stride:part * stride + F.nvfp4_tiled_bytes(n, k)]
            _, _, g = F.nvfp4_tiled_parts(m, n, k)
            mats.append((F.nvfp4_tiled_decode(m, n, k, scaled=False).astype(np.float64), np.float32(g)))
        xe = x[off:off + r]
        gate = F.bf16_round((xe @ mats[0][0].T).astype(np.float32) * mats[0][1])
        up = F.bf16_round((xe @ mats[1][0].T).astype(np.float32) * mats[1][1])
        g10 = np.minimum(gate, np.float32(10))
        u10 = np.clip(up, -10, 10).astype(np.float32)
        silu = F.bf16_round((g10 / (1 + np.exp(-g10.astype(np.float64)))).astype(np.float32))
        prod = F.bf16_round(F.bf16_round(silu * u10))
        W.check_output(p_mine[off:off + r], prod, rel=4e-3, max_abs=2.0 ** -7)
        # the down projection on the product this library wrote (so that the first GEMM's rounding does not enter twice)
        down = F.bf16_round((p_mine[off:off + r].astype(np.float64) @ mats[2][0].T).astype(np.float32) * mats[2][1])
        W.check_output(o_mine[off:off + r], down, rel=4e-3, max_abs=2.0 ** -7)


def test_packed_grouped_other_formats_and_bad_arguments():
    """LOWBIT images are outside this library: such an expert gets zero rows and status bit 8; the argument checks are
    the reference's (packed_grouped.cu:297-301)."""
    import darask_inference_engine_b200 as D
    lib = D._lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    case = build_case(5, 512, 256, [40, 40])
    case["formats"][8] = 1            # expert 1: gate_up.format = LOWBIT
    product, _ = run(lib, case)
    status = ctypes.c_uint(0)
    assert lib.hayate_glm_grouped_packed_status(ctypes.byref(status), st) == 0
    assert status.value == 8
    assert np.abs(product[:40]).max() > 0 and np.all(product[40:] == 0)
    assert lib.hayate_glm_grouped_packed_status(ctypes.byref(status), st) == 0 and status.value == 0     # read clears
    x = case["x"]
    args = lambda **kw: [kw.get("out", x.data_ptr() + 2), x.data_ptr(), case["table"].data_ptr(), case["formats"].data_ptr(),
                         case["ranges"].data_ptr(), kw.get("count", 2), kw.get("hidden", 512), kw.get("inter", 256), st]
    assert lib.hayate_glm_grouped_packed_gate_up(*args(out=x.data_ptr())) == 1       # out == x
    assert lib.hayate_glm_grouped_packed_gate_up(*args(count=289)) == 1
    assert lib.hayate_glm_grouped_packed_down(*args(hidden=500)) == 1
    assert lib.hayate_glm_grouped_packed_down(*args(inter=8192)) == 1
    assert lib.hayate_glm_grouped_packed_set_config(3) == 0 and lib.hayate_glm_grouped_packed_set_config(4) == 1
