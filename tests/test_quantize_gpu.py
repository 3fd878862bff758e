"""Device quantizers against the oracle quantizers, byte for byte."""
import numpy as np
import pytest
import torch

from oracle import formats as F
from tests import workloads as W

pytestmark = pytest.mark.gpu


def _w(seed, shape, std=0.02):
    w = W.normal(W.rng_for(seed), shape, std)
    w[0, :16] = 0.0
    return w


@pytest.mark.parametrize("ty", [F.GGML_Q4_K, F.GGML_Q6_K])
def test_ggml_quantizers(ty):
    import darask_inference_engine_b200 as D
    w = _w(1, (96, 1024))
    w[3] = 0.0
    got = D.quantize.ggml(torch.from_numpy(w).cuda(), ty).cpu().numpy()
    ref = F.ggml_quantize(w, ty).reshape(-1)
    assert np.array_equal(got, ref)


def test_nvfp4_tiled_quantizer_matches_reference_fixture():
    import os
    import darask_inference_engine_b200 as D
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "hayate_quant.npz"))
    for name in "abc":                  # images produced by the reference's own Python quantizer
        w, img = g[f"nvfp4_{name}_w"], g[f"nvfp4_{name}_img"]
        got = D.quantize.nvfp4_tiled(torch.from_numpy(w).cuda()).cpu().numpy()
        assert np.array_equal(got, img), name
    w = np.zeros((128, 64), np.float32)
    assert np.array_equal(D.quantize.nvfp4_tiled(torch.from_numpy(w).cuda()).cpu().numpy(), F.nvfp4_tiled_quantize(w))


def test_nvfp4_linear_quantizer():
    import darask_inference_engine_b200 as D
    f, h = 128, 256
    gate, up, down = _w(2, (f, h)), _w(3, (f, h)), _w(4, (h, f))
    block, gs = D.quantize.nvfp4_linear_expert(*[torch.from_numpy(m).cuda() for m in (gate, up, down)])
    rb, rgs = F.tsumuji_expert_block(gate, up, down)
    assert np.array_equal(gs.cpu().numpy(), rgs)
    got = block.cpu().numpy()
    # +0 / -0 codes (0 vs 8) decode identically; everything else must be equal
    diff = got != rb
    assert diff.sum() == 0 or set(np.unique(np.concatenate([got[diff] ^ rb[diff]]))) <= {0x08, 0x80, 0x88}


def test_fp8_quantizers():
    import darask_inference_engine_b200 as D
    w = _w(5, (300, 384))
    p, s = D.quantize.fp8_block(torch.from_numpy(w).cuda())
    rp, rs = F.fp8_block_quantize(w)
    assert np.array_equal(p.cpu().numpy(), rp) and np.array_equal(s.cpu().numpy(), rs)
    x = F.bf16_round(W.normal(W.rng_for(6), (33, 256), 1.0))
    x[2, :128] = 0
    for t in (torch.from_numpy(x).cuda(), torch.from_numpy(x).cuda().bfloat16()):
        c, sc = D.quantize.fp8_act(t)
        rc, rsc = F.fp8_act_quantize(x)
        assert np.array_equal(c.cpu().numpy(), rc) and np.array_equal(sc.cpu().numpy(), rsc)
