"""Parity of the CUDA Tsumuji layer (through the C ABI) with the oracle."""
import numpy as np
import pytest
import torch

from oracle import layers as L
from tests import workloads as W

pytestmark = pytest.mark.gpu


def run(layer, acts, given_logits=False):
    import darask_inference_engine_b200 as D
    n = acts["x"].shape[0]
    m = D.TsumujiMoeLayer(layer.hidden, layer.inter, layer.experts, layer.topk, n)
    t = torch.from_numpy
    m.load(None if given_logits else t(layer.router), t(layer.blocks.reshape(-1)), t(layer.gs), t(layer.shared_gu), t(layer.shared_down))
    if given_logits:
        m.rlogits[:n].copy_(t(acts["logits"]))
    out = m.forward(t(acts["x"]).cuda())
    torch.cuda.synchronize()
    return m, out.cpu().numpy()


def check(layer, acts, given_logits=False):
    m, out = run(layer, acts, given_logits)
    n = acts["x"].shape[0]
    logits = m.rlogits[:n].cpu().numpy()
    if not given_logits:
        assert np.allclose(logits, L.tsumuji_logits(layer, acts["x"]), rtol=1e-4, atol=1e-4)
    ref = L.tsumuji_forward(layer, acts["x"], logits=logits)
    ids = m.sel[:n].cpu().numpy()
    if not np.array_equal(ids, ref["ids"]):          # only keys within 4 ulp of each other may swap (expf rounding)
        from oracle import routing as R
        keys = R.selection_keys(R.TSUMUJI, logits, layer.experts)
        for t in np.nonzero((ids != ref["ids"]).any(1))[0]:
            a, b = keys[t, ids[t]], keys[t, ref["ids"][t]]
            assert np.all(np.abs(a - b) <= 4 * np.spacing(np.maximum(a, b)))
        ref = L.tsumuji_forward(layer, acts["x"], logits=logits, ids=ids)     # compare on the device's own selection
    assert np.allclose(m.rw[:n].cpu().numpy(), ref["w"], rtol=1e-5)
    assert np.allclose(m.sgate[:n].cpu().numpy(), ref["shared_gate"], rtol=1e-6)
    return W.check_output(out, ref["out"])


@pytest.mark.parametrize("tokens", [1, 3, 8])
def test_small_layer(tokens):
    layer, acts = W.tsumuji_layer(31, hidden=512, inter=256, experts=32, topk=4, tokens=tokens, pool=32)
    check(layer, acts)


def test_logits_from_caller():
    layer, acts = W.tsumuji_layer(32, hidden=512, inter=256, experts=64, topk=6, tokens=5, pool=16, uniform_logits=True)
    check(layer, acts, given_logits=True)


def test_config5_shape_verify_window():
    # hidden 2048, 512 experts, top-10, intermediate 512, NVFP4, shared expert, uniform logits, seed 4;
    # one sequence's window of 4 tokens (1 + 3 drafts)
    layer, acts = W.tsumuji_layer(4, 2048, 512, 512, 10, 4, pool=8, uniform_logits=True)
    check(layer, acts, given_logits=True)


def test_config5_batched_verify_256_tokens():
    # 64 sequences x 4 tokens = 256 tokens in one call
    layer, acts = W.tsumuji_layer(4, 2048, 512, 512, 10, 256, pool=8, uniform_logits=True)
    check(layer, acts, given_logits=True)


@pytest.mark.parametrize("tokens,hidden,inter,experts,topk", [(17, 512, 256, 32, 4), (40, 512, 256, 160, 6), (256, 2048, 512, 512, 10)])
def test_window_router_projection(tokens, hidden, inter, experts, topk):
    """Windows of more than 16 tokens take the batched front end: rows split into bf16 hi + lo, the router projection as
    a tensor-core product against the E + 1 router rows (E + 1 is never a multiple of the 128-row weight tile here, so
    zero-filled tile rows are covered), top-k per token, the multi-block permutation. Activations are float32 values that
    bf16 cannot hold, so the lo half of the split carries information; logits and routes are checked against the oracle."""
    layer, _ = W.tsumuji_layer(33, hidden, inter, experts, topk, 1, pool=8)
    x = W.normal(W.rng_for(1000 + tokens), (tokens, hidden), 1.0)
    assert not np.array_equal(x, np.asarray(torch.from_numpy(x).bfloat16().float()))
    check(layer, dict(x=x, logits=None))
