"""Parity of the CUDA Hayate layer and of the reference-named one-token launchers with the oracle."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import formats as F
from oracle import layers as L
from oracle import routing as R
from tests import workloads as W

pytestmark = pytest.mark.gpu


def bf16_tensor(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).bfloat16()


def check_ids(ids, ref_ids, keys):
    """ids equal, except that experts whose selection keys are closer than 1e-6 may swap (approximate sigmoid)."""
    for t in np.nonzero((ids != ref_ids).any(1))[0]:
        a, b = keys[t, ids[t]], keys[t, ref_ids[t]]
        assert np.all(np.abs(a - b) <= 1e-6), (t, ids[t], ref_ids[t])
    return np.array_equal(ids, ref_ids)


def run_layer(layer, acts):
    import darask_inference_engine_b200 as D
    t = acts["x"].shape[0]
    m = D.HayateMoeLayer(layer.hidden, layer.inter, layer.experts, layer.topk, layer.scale, t)
    m.load(bf16_tensor(layer.router), torch.from_numpy(layer.bias), torch.from_numpy(layer.images.reshape(-1)),
           torch.from_numpy(layer.shared))
    out = m.forward(bf16_tensor(acts["x"]).cuda())
    torch.cuda.synchronize()
    return m, out.float().cpu().numpy()


def check_layer(layer, acts):
    m, out = run_layer(layer, acts)
    t = acts["x"].shape[0]
    logits = m.logits[:t].cpu().numpy()
    assert np.allclose(logits, L.hayate_logits(layer, acts["x"]), rtol=1e-4, atol=1e-4)
    ref = L.hayate_forward(layer, acts["x"], logits=logits)
    keys = R.selection_keys(R.HAYATE, logits, layer.experts, layer.bias)
    if not check_ids(m.ids[:t].cpu().numpy(), ref["ids"], keys):     # near-tie: compare on the device's own selection
        ref = L.hayate_forward(layer, acts["x"], logits=logits, ids=m.ids[:t].cpu().numpy())
    assert np.allclose(m.weights[:t].cpu().numpy(), ref["weights"], rtol=1e-4)
    # outputs are bf16: one rounding flip is 2^-8 of the value, so the max-abs bar is one bf16 step of max|ref|
    return W.check_output(out, ref["out"], rel=1e-3, max_abs=2.0 ** -8)


@pytest.mark.parametrize("tokens", [1, 3])
def test_small_layer(tokens):
    layer, acts = W.hayate_layer(41, hidden=512, inter=256, experts=16, topk=4, tokens=tokens, scale=2.5, pool=16)
    check_layer(layer, acts)


def test_many_tokens_per_expert():
    # 8 experts, top-4, 19 tokens: an expert serves about ten tokens (eight-token passes, a second pass, ragged groups)
    layer, acts = W.hayate_layer(42, hidden=512, inter=256, experts=8, topk=4, tokens=19, scale=2.5, pool=8)
    check_layer(layer, acts)


@pytest.mark.parametrize("tokens", [1, 8])
def test_config3_glm_decode(tokens):
    # hidden 2048, 64 experts, sigmoid + bias, top-4, scale 1.8, intermediate 1536, NVFP4, one shared expert, seed 2
    layer, acts = W.hayate_layer(2, 2048, 1536, 64, 4, tokens, scale=1.8, pool=8)
    check_layer(layer, acts)


def test_reference_named_decode_launchers():
    """route_decode -> gate_up -> down -> reduce with the reference's signatures, at a non-default shape."""
    import darask_inference_engine_b200 as D
    lib = D._lib.lib()
    H, Fi, E, K, scale = 1024, 512, 32, 4, 1.8
    layer, acts = W.hayate_layer(43, H, Fi, E, K, 1, scale=scale, pool=8)
    dev = torch.device("cuda")
    st = torch.cuda.current_stream().cuda_stream
    assert lib.hayate_glm_moe_set_shape(H, Fi, E, K, scale) == 0
    ws = torch.zeros(lib.hayate_glm_moe_workspace_bytes(H, Fi, E, K, 1), dtype=torch.uint8, device=dev)
    assert lib.hayate_glm_moe_set_workspace(ws.data_ptr(), ws.numel(), st) == 0
    x = bf16_tensor(acts["x"]).to(dev)
    router = bf16_tensor(layer.router).to(dev)
    bias = torch.from_numpy(layer.bias).to(dev)
    images = torch.from_numpy(layer.images).to(dev)
    shared = torch.from_numpy(layer.shared).to(dev)
    logits = torch.zeros(E, device=dev)
    weights = torch.zeros(K, device=dev)
    ids = torch.zeros(K, dtype=torch.int32, device=dev)
    assert lib.hayate_glm_route_decode(logits.data_ptr(), weights.data_ptr(), ids.data_ptr(), x.data_ptr(), router.data_ptr(),
                                       bias.data_ptr(), st) == 0
    torch.cuda.synchronize()
    ref = L.hayate_forward(layer, acts["x"], logits=logits.cpu().numpy()[None])
    keys = R.selection_keys(R.HAYATE, logits.cpu().numpy()[None], E, layer.bias)
    if not check_ids(ids.cpu().numpy()[None], ref["ids"], keys):
        ref = L.hayate_forward(layer, acts["x"], logits=logits.cpu().numpy()[None], ids=ids.cpu().numpy()[None])
    # the host looks the images up (all resident): device array of top-k pointers in route order
    table = torch.tensor([images.data_ptr() + int(e) * images.shape[1] for e in ids.cpu().numpy()], dtype=torch.int64, device=dev)
    stride = layer.stride
    dw = lambda part: D._lib.HayateDenseWeight(shared.data_ptr() + part * stride, None, 3)
    product = torch.zeros(K + 1, Fi, dtype=torch.bfloat16, device=dev)
    expert = torch.zeros(K + 1, H, dtype=torch.bfloat16, device=dev)
    out = torch.zeros(H, dtype=torch.bfloat16, device=dev)
    assert lib.hayate_glm_moe_gate_up(product.data_ptr(), x.data_ptr(), x.data_ptr(), table.data_ptr(), dw(0), dw(1), 1, 0, stride, st) == 0
    assert lib.hayate_glm_moe_down(expert.data_ptr(), product.data_ptr(), table.data_ptr(), dw(2), 1, 0, stride, st) == 0
    assert lib.hayate_glm_moe_reduce(out.data_ptr(), expert.data_ptr(), ids.data_ptr(), weights.data_ptr(), st) == 0
    torch.cuda.synchronize()
    W.check_output(out.float().cpu().numpy()[None], ref["out"], rel=1e-3, max_abs=2.0 ** -8)
    # validation failures return cudaErrorInvalidValue like the reference launchers
    assert lib.hayate_glm_moe_reduce(None, expert.data_ptr(), ids.data_ptr(), weights.data_ptr(), st) == 1
    assert lib.hayate_glm_moe_set_shape(4096, 2048, 288, 8, 2.5) == 0
    assert lib.hayate_glm_moe_set_workspace(None, 0, st) == 0


def test_reduction_order_golden():
    # reference test engines/hayate/crates/kernels/src/glm53.rs:1702: ids [287,0,17,42,8,256,3,4] are added in the
    # order [1,6,7,4,2,3,5,0]; with bf16 rounding after every add the order is visible in the result
    import darask_inference_engine_b200 as D
    lib = D._lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    assert lib.hayate_glm_moe_set_shape(4096, 2048, 288, 8, 2.5) == 0
    ids = np.array([287, 0, 17, 42, 8, 256, 3, 4], np.int32)
    rng = np.random.default_rng(9)
    y = F.bf16_round(rng.standard_normal((9, 4096)).astype(np.float32) * np.float32(3))
    w = rng.uniform(0.1, 0.9, 8).astype(np.float32)
    acc = np.zeros(4096, np.float32)
    for s in R.route_order(ids):
        acc = F.bf16_round(acc + F.bf16_round((y[s] * w[s]).astype(np.float32)))
    expect = F.bf16_round(acc + y[8])
    out = torch.zeros(4096, dtype=torch.bfloat16, device="cuda")
    y_d, ids_d, w_d = bf16_tensor(y).cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
    assert lib.hayate_glm_moe_reduce(out.data_ptr(), y_d.data_ptr(), ids_d.data_ptr(), w_d.data_ptr(), st) == 0
    torch.cuda.synchronize()
    assert np.array_equal(out.float().cpu().numpy(), expect)


def fp8_image(rng, n, k):
    """Block-FP8 matrix image as the reference lays it out (decode.cu:32-36): payload [n][k], then the float32 scales."""
    payload, scale = F.fp8_block_quantize(W.normal(rng, (n, k), 0.02))
    return payload, scale, np.concatenate([payload.reshape(-1), scale.reshape(-1).view(np.uint8)])


@pytest.mark.parametrize("nv", [0, 1])
def test_block_fp8_images(nv):
    """nv = 0: gate, up and down of the routed and the shared expert are block-FP8; nv = 1 with down_fp8: NVFP4 gate/up,
    block-FP8 down.  Weights are bf16(e4m3 * scale) as the reference's `scaled_fp8` forms them."""
    import darask_inference_engine_b200 as D
    lib = D._lib.lib()
    H, Fi, E, K, scale = 1024, 512, 32, 4, 1.8
    rng = W.rng_for(77 + nv)
    dev, st = torch.device("cuda"), torch.cuda.current_stream().cuda_stream
    assert lib.hayate_glm_moe_set_shape(H, Fi, E, K, scale) == 0
    ws = torch.zeros(lib.hayate_glm_moe_workspace_bytes(H, Fi, E, K, 1), dtype=torch.uint8, device=dev)
    assert lib.hayate_glm_moe_set_workspace(ws.data_ptr(), ws.numel(), st) == 0
    stride = max(F.hayate_expert_stride(H, Fi), (H * Fi + (H // 128) * (Fi // 128) * 4 + 255) // 256 * 256)

    def expert():
        """-> (image bytes [3*stride], dense (gate, up, down) float64 as the kernels must see them)"""
        img = np.zeros(3 * stride, np.uint8)
        dense = []
        for part, (n, k) in enumerate(((Fi, H), (Fi, H), (H, Fi))):
            if nv and part < 2:
                m = F.nvfp4_tiled_quantize(W.normal(rng, (n, k), 0.02))
                dense.append(("nv", m, n, k))
            else:
                p, s, m = fp8_image(rng, n, k)
                dense.append(("f8", (p, s), n, k))
            img[part * stride:part * stride + m.size] = m
        return img, dense

    def mats(dense, rounded_nv):
        out = []
        for kind, m, n, k in dense:
            out.append((F.nvfp4_tiled_decode(m, n, k, rounded=rounded_nv) if kind == "nv" else F.fp8_block_decode(m[0], m[1], rounded=True)).astype(np.float64))
        return out

    ids = rng.permutation(E)[:K].astype(np.int32)
    weights = (rng.random(K, dtype=np.float32) + 0.1).astype(np.float32)
    images = [expert() for _ in range(K)]
    shared_img, shared_dense = expert()
    x = F.bf16_round(W.normal(rng, (H,), 1.0))
    # oracle (decode.cu:37-59)
    xt = x.astype(np.float64)
    ys = []
    for img, dense in images + [(shared_img, shared_dense)]:
        g, u, d = mats(dense, rounded_nv=dense is shared_dense)
        p = L.hayate_swiglu(F.bf16_round((g @ xt).astype(np.float32)), F.bf16_round((u @ xt).astype(np.float32)))
        ys.append(F.bf16_round((d @ p.astype(np.float64)).astype(np.float32)))
    acc = np.zeros(H, np.float32)
    for a in R.route_order(ids):
        acc = F.bf16_round(acc + F.bf16_round((ys[a] * weights[a]).astype(np.float32)))
    ref = F.bf16_round((acc + ys[K]).astype(np.float32))
    # device
    imgs_d = [torch.from_numpy(img).to(dev) for img, _ in images]
    shared_d = torch.from_numpy(shared_img).to(dev)
    table = torch.tensor([t.data_ptr() for t in imgs_d], dtype=torch.int64, device=dev)
    DW = D._lib.HayateDenseWeight

    def dw(part):
        kind, m, n, k = shared_dense[part]
        base = shared_d.data_ptr() + part * stride
        return DW(base, None, 3) if kind == "nv" else DW(base, base + n * k, 1)

    x_d = bf16_tensor(x[None]).to(dev)
    product = torch.zeros(K + 1, Fi, dtype=torch.bfloat16, device=dev)
    expert_out = torch.zeros(K + 1, H, dtype=torch.bfloat16, device=dev)
    out = torch.zeros(H, dtype=torch.bfloat16, device=dev)
    ids_d, w_d = torch.from_numpy(ids).to(dev), torch.from_numpy(weights).to(dev)
    assert lib.hayate_glm_moe_gate_up(product.data_ptr(), x_d.data_ptr(), x_d.data_ptr(), table.data_ptr(), dw(0), dw(1), nv, 1 if nv else 0, stride, st) == 0
    assert lib.hayate_glm_moe_down(expert_out.data_ptr(), product.data_ptr(), table.data_ptr(), dw(2), nv, 1 if nv else 0, stride, st) == 0
    assert lib.hayate_glm_moe_reduce(out.data_ptr(), expert_out.data_ptr(), ids_d.data_ptr(), w_d.data_ptr(), st) == 0
    torch.cuda.synchronize()
    W.check_output(expert_out.float().cpu().numpy(), np.stack(ys), rel=4e-3, max_abs=2.0 ** -7)
    W.check_output(out.float().cpu().numpy()[None], ref[None], rel=4e-3, max_abs=2.0 ** -7)
    # formats that are not built answer like the reference answers bad arguments
    assert lib.hayate_glm_moe_down(expert_out.data_ptr(), product.data_ptr(), table.data_ptr(), DW(shared_d.data_ptr(), None, 0), nv, 1, stride, st) == 1
    assert lib.hayate_glm_moe_set_shape(4096, 2048, 288, 8, 2.5) == 0
    assert lib.hayate_glm_moe_set_workspace(None, 0, st) == 0
