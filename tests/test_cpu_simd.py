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
