"""Router top-k and dispatch permutation on the GPU against the oracle: ids, their order and the
permutation must match bit for bit on identical float32 logits."""
import numpy as np
import pytest
import torch

from oracle import routing as R

pytestmark = pytest.mark.gpu


def gpu_route(mode, logits, experts, topk, bias=None, scale=1.0):
    import darask_inference_engine_b200 as D
    lib = D._lib.lib()
    t, ld = logits.shape
    lg = torch.from_numpy(logits).cuda()
    ids = torch.full((t, topk), -1, dtype=torch.int32, device="cuda")
    w = torch.zeros((t, topk), dtype=torch.float32, device="cuda")
    sg = torch.zeros(t, dtype=torch.float32, device="cuda")
    b = torch.from_numpy(bias).cuda() if bias is not None else None
    rc = lib.darask_route_topk(mode, lg.data_ptr(), ld, experts, topk, t, b.data_ptr() if b is not None else None,
                               scale, ids.data_ptr(), w.data_ptr(), sg.data_ptr() if mode == 1 else None,
                               torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    return ids.cpu().numpy(), w.cpu().numpy(), sg.cpu().numpy()


def grid_logits(rng, t, e, step=2.0 ** -8, spread=6.0):
    """Logits on a coarse grid: distinct values differ by far more than any rounding of the key,
    equal values are exact ties (which must go to the lower id)."""
    return (np.round(rng.standard_normal((t, e)) * spread / step / 4) * step).astype(np.float32)


@pytest.mark.parametrize("experts,topk", [(64, 4), (128, 8), (256, 8), (288, 8), (512, 10), (1024, 32), (8, 8)])
def test_kogarashi_router(experts, topk):
    rng = np.random.default_rng(experts + topk)
    for logits in (grid_logits(rng, 33, experts), rng.standard_normal((17, experts)).astype(np.float32),
                   np.zeros((2, experts), np.float32)):
        ids, w, _ = gpu_route(0, logits, experts, topk)
        rid, rw = R.route_kogarashi(logits, topk)
        assert np.array_equal(ids, rid)
        assert np.allclose(w, rw, rtol=2e-6, atol=1e-9)


@pytest.mark.parametrize("experts,topk", [(64, 4), (128, 8), (256, 8), (512, 10), (1024, 32)])
def test_tsumuji_router(experts, topk):
    rng = np.random.default_rng(experts * 3 + topk)
    for logits in (grid_logits(rng, 40, experts + 1), np.zeros((3, experts + 1), np.float32)):
        ids, w, sg = gpu_route(1, logits, experts, topk)
        rid, rw, rsg = R.route_tsumuji(logits, experts, topk)
        assert np.array_equal(ids, rid)
        assert np.allclose(w, rw, rtol=1e-5, atol=1e-9) and np.allclose(sg, rsg, rtol=1e-6)
    # full-entropy logits: keys of distinct logits can round together; any difference from the
    # oracle must be explained by keys closer than 4 ulp
    logits = rng.uniform(-1, 1, (256, experts + 1)).astype(np.float32)
    ids, _, _ = gpu_route(1, logits, experts, topk)
    rid, _, _ = R.route_tsumuji(logits, experts, topk)
    keys = R.selection_keys(R.TSUMUJI, logits, experts)
    for t in np.nonzero((ids != rid).any(1))[0]:
        a, b = keys[t, ids[t]], keys[t, rid[t]]
        assert np.all(np.abs(a - b) <= 4 * np.spacing(np.maximum(a, b)))


@pytest.mark.parametrize("experts,topk,scale", [(64, 4, 1.8), (288, 8, 2.5), (256, 8, 2.5), (4, 2, 2.5)])
def test_hayate_router(experts, topk, scale):
    rng = np.random.default_rng(experts + 7)
    bias = (np.round(rng.standard_normal(experts) * 0.1 * 256) / 256).astype(np.float32)
    # logits whose sigmoid is separated well beyond approximate-math error, plus exact ties
    logits = (rng.integers(-24, 25, (48, experts)) * 0.25).astype(np.float32)
    ids, w, _ = gpu_route(2, logits, experts, topk, bias, scale)
    rid, rw = R.route_hayate(logits, bias, topk, scale)
    keys = R.selection_keys(R.HAYATE, logits, experts, bias)
    for t in range(logits.shape[0]):
        if not np.array_equal(ids[t], rid[t]):            # only near-equal keys may swap
            a, b = keys[t, ids[t]], keys[t, rid[t]]
            assert np.all(np.abs(a - b) <= 1e-6)
    assert np.mean(ids == rid) > 0.98
    same = (ids == rid).all(1)
    assert np.allclose(w[same], rw[same], rtol=2e-6 * 50, atol=1e-7)
    if experts == 4:      # reference test: bias only affects selection, weights all 1.25
        ids, w, _ = gpu_route(2, np.zeros((2, 4), np.float32), 4, 2, np.array([0, 3, 1, 2], np.float32), 2.5)
        assert ids.tolist() == [[1, 3], [1, 3]] and np.allclose(w, 1.25, rtol=1e-6)


def gpu_permute(ids, experts, topk, large=False):
    import darask_inference_engine_b200 as D
    lib = D._lib.lib()
    t = ids.size // topk
    d = torch.from_numpy(ids.astype(np.int32).reshape(-1)).cuda()
    asg = torch.full((t * topk,), 0xFFFFFFFF, dtype=torch.int64, device="cuda").to(torch.int32)
    ranges = torch.zeros(experts * 2, dtype=torch.int32, device="cuda")
    active = torch.full((experts,), -1, dtype=torch.int32, device="cuda")
    counters = torch.zeros(4, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    if large:
        scratch = torch.empty(lib.darask_moe_permute_scratch_bytes(t, topk, experts), dtype=torch.uint8, device="cuda")
        rc = lib.darask_moe_permute_large(d.data_ptr(), t, topk, experts, asg.data_ptr(), ranges.data_ptr(), active.data_ptr(),
                                          counters.data_ptr(), status.data_ptr(), scratch.data_ptr(), scratch.numel(),
                                          torch.cuda.current_stream().cuda_stream)
    else:
        rc = lib.darask_moe_permute(d.data_ptr(), t, topk, experts, asg.data_ptr(), ranges.data_ptr(), active.data_ptr(),
                                    counters.data_ptr(), status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    return (asg.cpu().numpy().view(np.uint32), ranges.cpu().numpy().reshape(experts, 2), active.cpu().numpy(),
            counters.cpu().numpy(), int(status.item()))


def test_permutation_golden_and_random():
    # reference golden: engines/hayate/crates/models/src/glm53/prefill.rs:490-502
    ids = np.array([7, 2, 3, 4, 5, 6, 1, 0, 8, 2, 3, 4, 5, 6, 1, 0])
    asg, ranges, active, counters, status = gpu_permute(ids, 288, 8)
    ra, rc, ro = R.permutation(ids, 288, 8)
    assert status == 0 and np.array_equal(asg, ra)
    assert np.array_equal(ranges[:, 0], rc) and np.array_equal(ranges[:, 1], ro)
    assert asg[ro[0]:ro[0] + 2].tolist() == [7, 15] and asg[ro[7]] == 0 and asg[ro[8]] == 8
    assert counters[0] == 9 and counters[1] == 16 and active[:9].tolist() == list(range(9))
    rng = np.random.default_rng(0)
    for t, e, k in [(1, 256, 8), (16, 256, 8), (256, 512, 10), (4096, 256, 8), (5, 7, 7), (1000, 1024, 3)]:
        ids = np.stack([rng.permutation(e)[:k] for _ in range(t)])
        asg, ranges, active, counters, status = gpu_permute(ids, e, k)
        ra, rc, ro = R.permutation(ids, e, k)
        assert status == 0 and np.array_equal(asg, ra) and np.array_equal(ranges[:, 0], rc)
        assert np.array_equal(ranges[:, 1], ro)
        assert np.array_equal(active[:counters[0]], np.nonzero(rc)[0])


def test_permutation_large_batches():
    """The multi-block permutation equals the host loop on prefill-sized and ragged batches, skewed and uniform."""
    rng = np.random.default_rng(1)
    for t, e, k, skew in [(4096, 256, 8, True), (4096, 256, 8, False), (1, 8, 2, False), (129, 1024, 5, False),
                          (1025, 64, 4, True), (8192, 512, 10, False)]:
        p = 1.0 / np.arange(1, e + 1) ** 1.1 if skew else np.ones(e)
        p = p / p.sum()
        ids = np.stack([rng.choice(e, size=k, replace=False, p=p) for _ in range(t)])
        asg, ranges, active, counters, status = gpu_permute(ids, e, k, large=True)
        ra, rc, ro = R.permutation(ids, e, k)
        assert status == 0 and np.array_equal(asg, ra)
        assert np.array_equal(ranges[:, 0], rc) and np.array_equal(ranges[:, 1], ro)
        assert np.array_equal(active[:counters[0]], np.nonzero(rc)[0]) and counters[1] == t * k
    _, _, _, counters, status = gpu_permute(np.array([2, 2, 3, 4, 5, 6, 1, 0] * 300), 288, 8, large=True)
    assert status & 2 and counters[1] == 7 * 300


def test_permutation_flags_bad_routes():
    # duplicate inside a token and an id >= experts are rejected by the reference (prefill.rs:18-20)
    _, _, _, counters, status = gpu_permute(np.array([2, 2, 3, 4, 5, 6, 1, 0]), 288, 8)
    assert status & 2 and counters[1] == 7
    _, _, _, counters, status = gpu_permute(np.array([288, 2, 3, 4, 5, 6, 1, 0]), 288, 8)
    assert status & 2 and counters[1] == 7
