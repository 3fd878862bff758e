"""The AVX2 + FMA row products of oracle/cpu_moe.c (used by the timed CPU baseline) against its scalar loops."""
import ctypes

import numpy as np

from oracle import build_ref
from oracle import formats as F
from tests import workloads as W


def test_simd_row_products_match_scalar_loops():
    import bench
    lib = ctypes.CDLL(str(build_ref.build_cpu()))
    lib.cpu_set_simd(1)
    if not lib.cpu_simd():
        import pytest
        pytest.skip("host without AVX2 / FMA")
    for down_ty in (F.GGML_Q6_K, F.GGML_Q4_K):
        layer, acts = W.kogarashi_layer(31, hidden=512, inter=256, experts=8, topk=2, tokens=3, pool=4, down_ty=down_ty)
        outs = []
        for simd in (0, 1):
            lib.cpu_set_simd(simd)
            L = bench.KogarashiCpu(layer.hidden, layer.inter, layer.experts, layer.topk, 3)
            keep = [np.ascontiguousarray(a) for a in (layer.router, layer.gate, layer.up, layer.down, layer.sh_gate, layer.sh_up, layer.sh_down,
                                                      layer.sh_inp, acts["n"])]
            L.router, L.gate, L.up, L.down, L.sh_gate, L.sh_up, L.sh_down, L.sh_inp, L.n = (a.ctypes.data for a in keep)
            L.gate_ty, L.up_ty, L.down_ty = layer.gate_ty, layer.up_ty, layer.down_ty
            x = acts["x"].copy()
            logits, ids, prob = np.zeros((3, 8), np.float32), np.zeros((3, 2), np.int32), np.zeros((3, 2), np.float32)
            L.x, L.logits, L.ids, L.prob = x.ctypes.data, logits.ctypes.data, ids.ctypes.data, prob.ctypes.data
            assert lib.cpu_kogarashi_layer(ctypes.byref(L), 2) == 0
            outs.append((x - acts["x"], ids.copy()))
        lib.cpu_set_simd(0)
        assert np.array_equal(outs[0][1], outs[1][1])
        W.check_output(outs[1][0], outs[0][0], rel=2e-5, max_abs=2e-5)


def test_c_fp8_layer_matches_the_numpy_oracle():
    """`cpu_fp8_layer` (the timed CPU baseline of the prefill workload) against `oracle.layers.fp8_forward`."""
    import bench
    from oracle import layers as L
    lib = ctypes.CDLL(str(build_ref.build_cpu()))
    layer, acts = W.fp8_layer(9, 256, 128, 8, 2, 24, pool=8, zipf=1.1)
    ref = L.fp8_forward(layer, acts["x"], acts["logits"])
    stack = lambda mats, j: np.ascontiguousarray(np.stack([m[j] for m in mats]))
    keep = [stack(layer.gate, 0), stack(layer.up, 0), stack(layer.down, 0), stack(layer.gate, 1), stack(layer.up, 1), stack(layer.down, 1),
            np.ascontiguousarray(acts["x"]), np.ascontiguousarray(acts["logits"]), np.zeros((24, 256), np.float32), np.zeros((24, 2), np.int32),
            np.zeros((24, 2), np.float32)]
    desc = bench.Fp8Cpu(256, 128, 8, 2, 24, *[a.ctypes.data for a in keep])
    assert lib.cpu_fp8_layer(ctypes.byref(desc), 2) == 0
    assert np.array_equal(keep[9], ref["ids"])
    np.testing.assert_allclose(keep[10], ref["prob"], rtol=1e-5, atol=1e-7)
    W.check_output(keep[8], ref["out"])


def hayate_c_layer(lib, layer, x, threads=2):
    import bench
    t = x.shape[0]
    keep = [bench.bf16_bits(layer.router), np.ascontiguousarray(layer.bias, np.float32), np.ascontiguousarray(layer.images),
            np.ascontiguousarray(layer.shared), bench.bf16_bits(x), np.zeros((t, layer.hidden), np.uint16),
            np.zeros((t, layer.experts), np.float32), np.zeros((t, layer.topk), np.int32), np.zeros((t, layer.topk), np.float32)]
    d = bench.HayateCpu(layer.hidden, layer.inter, layer.experts, layer.topk, t, layer.scale)
    d.router, d.bias, d.images, d.shared, d.x, d.out, d.logits, d.ids, d.weights = (a.ctypes.data for a in keep)
    d.stride = layer.stride
    assert lib.cpu_hayate_layer(ctypes.byref(d), threads) == 0
    out = (keep[5].astype(np.uint32) << 16).view(np.float32)
    return dict(out=out, logits=keep[6], ids=keep[7], weights=keep[8])


def test_c_hayate_layer_matches_the_numpy_oracle():
    """`cpu_hayate_layer` (the reference's CPU expert path restated in C: NVFP4 rows multiplied without decoding them to
    memory, at most four activation rows per pass, 128-row claims, two dispatches) against `oracle.layers.hayate_forward`,
    with vector instructions and without; 7 tokens over 8 experts so that experts meet more than four rows."""
    from oracle import layers as L
    lib = ctypes.CDLL(str(build_ref.build_cpu()))
    layer, acts = W.hayate_layer(12, hidden=512, inter=384, experts=8, topk=3, tokens=7, scale=1.8, pool=8)
    got = {}
    for simd in (0, 1):
        lib.cpu_set_simd(simd)
        if simd and not lib.cpu_simd():
            continue
        got[simd] = hayate_c_layer(lib, layer, acts["x"])
    lib.cpu_set_simd(0)
    for simd, g in got.items():
        assert np.allclose(g["logits"], L.hayate_logits(layer, acts["x"]), rtol=1e-4, atol=1e-5)
        ref = L.hayate_forward(layer, acts["x"], logits=g["logits"], ids=g["ids"])
        ids, _ = __import__("oracle.routing", fromlist=["x"]).route_hayate(g["logits"], layer.bias, layer.topk, layer.scale)
        assert np.array_equal(g["ids"], ids)
        np.testing.assert_allclose(g["weights"], ref["weights"], rtol=1e-5)
        W.check_output(g["out"], ref["out"], rel=4e-3, max_abs=2.0 ** -7)        # bf16 roundings at float32 against float64 sums
    if len(got) == 2:
        assert np.array_equal(got[0]["ids"], got[1]["ids"])
        W.check_output(got[1]["out"], got[0]["out"], rel=4e-3, max_abs=2.0 ** -7)


def test_c_tsumuji_layer_matches_the_numpy_oracle():
    """`cpu_tsumuji_layer` (linear-layout NVFP4 experts, float32 activations, dense bf16 shared expert) against
    `oracle.layers.tsumuji_forward`: router projection by the C code, and logits handed in."""
    import bench
    from oracle import layers as L
    from oracle import routing as R
    lib = ctypes.CDLL(str(build_ref.build_cpu()))
    for given in (False, True):
        layer, acts = W.tsumuji_layer(21, hidden=256, inter=128, experts=12, topk=3, tokens=9, pool=6, uniform_logits=given)
        t, e, k = 9, layer.experts, layer.topk
        logits = acts["logits"].copy() if given else np.zeros((t, e + 1), np.float32)
        keep = [bench.bf16_bits(layer.router), np.ascontiguousarray(layer.blocks), np.ascontiguousarray(layer.gs, np.float32),
                bench.bf16_bits(layer.shared_gu), bench.bf16_bits(layer.shared_down), np.ascontiguousarray(acts["x"], np.float32),
                np.zeros((t, layer.hidden), np.float32), logits, np.zeros((t, k), np.int32), np.zeros((t, k), np.float32), np.zeros(t, np.float32)]
        for simd in (0, 1):
            lib.cpu_set_simd(simd)
            d = bench.TsumujiCpu(layer.hidden, layer.inter, e, k, t)
            d.router, d.blocks, d.gs, d.shared_gu, d.shared_down, d.x, d.out, d.logits, d.ids, d.w, d.shared_gate = (a.ctypes.data for a in keep)
            d.given_logits = int(given)
            assert lib.cpu_tsumuji_layer(ctypes.byref(d), 2) == 0
            if not given:
                assert np.allclose(logits, L.tsumuji_logits(layer, acts["x"]), rtol=1e-4, atol=1e-5)
            ids, w, sgate = R.route_tsumuji(logits, e, k)
            assert np.array_equal(keep[8], ids)
            np.testing.assert_allclose(keep[9], w, rtol=1e-5)
            np.testing.assert_allclose(keep[10], sgate, rtol=1e-6)
            ref = L.tsumuji_forward(layer, acts["x"], logits=logits, ids=keep[8])
            W.check_output(keep[6], ref["out"])
    lib.cpu_set_simd(0)
