"""Hayate prefill launchers (reference names): NVFP4 restore, gather, scatter, copy and the grouped bf16 GEMM."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import formats as F
from tests import workloads as W

pytestmark = pytest.mark.gpu


def lib():
    import darask_inference_engine_b200 as D
    return D._lib.lib(), D._lib.check


def stream():
    return torch.cuda.current_stream().cuda_stream


def ref_restore(image, n, k, scaled):
    """bf16(((e2m1 * e4m3) * global)), the product order of the reference's `nvfp4` (cu/glm53/math.cuh:41-49)."""
    codes, sc, g = F.nvfp4_tiled_parts(image, n, k)
    v = (F.E2M1_TABLE[codes].reshape(n, k // 16, 16) * F.e4m3_decode(sc)[:, :, None]).astype(np.float32)
    if scaled:
        v = (v * np.float32(g)).astype(np.float32)
    return F.bf16_round(v.reshape(n, k)), g


@pytest.mark.parametrize("n,k", [(256, 512), (130, 80)])
def test_nvfp4_restore(n, k):
    l, check = lib()
    rng = W.rng_for(3)
    image = F.nvfp4_tiled_quantize(W.normal(rng, (n, k), 0.02))
    d = torch.from_numpy(image).cuda()
    out = torch.empty(n, k, dtype=torch.bfloat16, device="cuda")
    check(l.hayate_glm_nvfp4_restore(out.data_ptr(), d.data_ptr(), n, k, stream()), "restore")
    ref, g = ref_restore(image, n, k, True)
    assert np.array_equal(out.float().cpu().numpy(), ref)
    scale = torch.zeros(1, device="cuda")
    check(l.hayate_glm_nvfp4_restore_unscaled(out.data_ptr(), scale.data_ptr(), d.data_ptr(), n, k, stream()), "restore_unscaled")
    ref, g = ref_restore(image, n, k, False)
    assert np.array_equal(out.float().cpu().numpy(), ref) and scale.item() == g
    assert l.hayate_glm_nvfp4_restore(out.data_ptr(), d.data_ptr(), n, 24, stream()) != 0      # k % 16 as in the reference


@pytest.mark.parametrize("n,k", [(256, 384), (130, 200)])
def test_fp8_restore(n, k):
    l, check = lib()
    rng = W.rng_for(6)
    payload, scale = F.fp8_block_quantize(W.normal(rng, (n, k), 0.02))
    p_d, s_d = torch.from_numpy(payload).cuda(), torch.from_numpy(scale).cuda()
    out = torch.empty(n, k, dtype=torch.bfloat16, device="cuda")
    check(l.hayate_glm_restore(out.data_ptr(), p_d.data_ptr(), s_d.data_ptr(), n, k, stream()), "restore")
    assert np.array_equal(out.float().cpu().numpy(), F.fp8_block_decode(payload, scale, rounded=True))


def test_gather_scatter_copy():
    l, check = lib()
    rng = W.rng_for(4)
    tokens, hidden, topk = 37, 256, 8
    x = F.bf16_round(W.normal(rng, (tokens, hidden), 1.0))
    assignments = rng.permutation(tokens * topk)[:50].astype(np.uint32)
    a_d = torch.from_numpy(assignments.astype(np.int64)).to(torch.int32).cuda()
    x_d = torch.from_numpy(x).bfloat16().cuda()
    g = torch.empty(50, hidden, dtype=torch.bfloat16, device="cuda")
    check(l.hayate_glm_gather(g.data_ptr(), x_d.data_ptr(), a_d.data_ptr(), 50, hidden, stream()), "gather")
    assert np.array_equal(g.float().cpu().numpy(), x[assignments // topk])
    # scatter: one row per token per call, out = bf16(out + bf16(y * w[a]))
    one_per_token = np.array([t * topk + rng.integers(topk) for t in rng.permutation(tokens)[:20]], np.uint32)
    y = F.bf16_round(W.normal(rng, (20, hidden), 1.0))
    w = rng.random(tokens * topk, dtype=np.float32)
    out0 = F.bf16_round(W.normal(rng, (tokens, hidden), 1.0))
    out = torch.from_numpy(out0).bfloat16().cuda()
    y_d, w_d = torch.from_numpy(y).bfloat16().cuda(), torch.from_numpy(w).cuda()
    o_d = torch.from_numpy(one_per_token.astype(np.int64)).to(torch.int32).cuda()
    check(l.hayate_glm_scatter(out.data_ptr(), y_d.data_ptr(), w_d.data_ptr(), o_d.data_ptr(), 20, hidden, stream()), "scatter")
    ref = out0.copy()
    for i, a in enumerate(one_per_token):
        t = a // topk
        ref[t] = F.bf16_round(ref[t] + F.bf16_round(y[i] * w[a]))
    assert np.array_equal(out.float().cpu().numpy(), ref)
    z = torch.ones(64, dtype=torch.uint8, device="cuda")
    check(l.hayate_glm_copy(z.data_ptr(), None, 64, stream()), "copy")
    assert not z.any()
    check(l.hayate_glm_copy(z.data_ptr(), x_d.data_ptr(), 64, stream()), "copy")
    assert torch.equal(z, x_d.view(torch.uint8).reshape(-1)[:64])


@pytest.mark.parametrize("counts", [[128, 1, 0, 300], [5], [256, 256, 256, 256, 256, 256, 256, 256]])
@pytest.mark.parametrize("n,k", [(256, 128), (384, 448), (2048, 4096)])
def test_grouped_bf16(counts, n, k):
    """The rows buffer ends exactly at the last routed row: the kernel may not read past it."""
    if n * k > 1 << 20 and len(counts) > 4:
        counts = counts[:3]
    l, check = lib()
    rng = W.rng_for(9)
    groups, rows = len(counts), int(sum(counts))
    x = F.bf16_round(W.normal(rng, (rows, k), 1.0))
    w = F.bf16_round(W.normal(rng, (groups, n, k), k ** -0.5))
    offs = np.concatenate([[0], np.cumsum(counts)[:-1]])
    ranges = torch.from_numpy(np.stack([counts, offs], 1).astype(np.int32)).cuda()
    x_d, w_d = torch.from_numpy(x).bfloat16().cuda(), torch.from_numpy(w).bfloat16().cuda()
    out = torch.zeros(rows, n, dtype=torch.bfloat16, device="cuda")
    meta = torch.zeros(608, dtype=torch.uint8, device="cuda")
    check(l.hayate_glm_grouped(out.data_ptr(), x_d.data_ptr(), w_d.data_ptr(), ranges.data_ptr(), groups, n, k, meta.data_ptr(), stream()),
          "grouped")
    acc = torch.zeros(rows, n, dtype=torch.float32, device="cuda")
    out2 = torch.zeros(rows, n, dtype=torch.bfloat16, device="cuda")
    scales = rng.random(groups, dtype=np.float32) + 0.5
    s_d = torch.from_numpy(scales).cuda()
    check(l.hayate_glm_grouped_nvfp4(out2.data_ptr(), acc.data_ptr(), x_d.data_ptr(), w_d.data_ptr(), ranges.data_ptr(), groups, n, k,
                                     meta.data_ptr(), s_d.data_ptr(), max(counts), stream()), "grouped_nvfp4")
    torch.cuda.synchronize()
    got, got_acc, got2 = out.float().cpu().numpy(), acc.cpu().numpy(), out2.float().cpu().numpy()
    for g, (c, o) in enumerate(zip(counts, offs)):
        if not c:
            continue
        ref = x[o:o + c].astype(np.float64) @ w[g].astype(np.float64).T
        W.check_output(got_acc[o:o + c], ref.astype(np.float32), rel=1e-5, max_abs=1e-5)
        W.check_output(got[o:o + c], ref.astype(np.float32), rel=4e-3, max_abs=2 ** -8)            # bf16 store
        assert np.array_equal(got2[o:o + c], F.bf16_round(got_acc[o:o + c] * scales[g]))
    assert l.hayate_glm_grouped(out.data_ptr(), x_d.data_ptr(), w_d.data_ptr(), ranges.data_ptr(), 0, n, k, meta.data_ptr(), stream()) != 0
