"""The workspace-free entry point `kogarashi_moe_layer_static`.

Some hosts cannot give the layer a workspace because they have no device allocator where the
call is made (all device memory went to their own arena at start-up, or they run after the
point where their engine stops allocating).  For them the library carries a fixed 1 MiB scratch
array per GPU.  This test drives that entry point through the C ABI twice in a row and checks
both results against the ordinary entry point, which gets a caller-provided workspace.  The
file name sorts last so that a run that stops at the first failure has already run everything
else; the test does not depend on any state the other tests leave behind.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import formats as F
from tests import workloads as W

pytestmark = pytest.mark.gpu


def _descriptor(D, layer, bufs, t):
    d = D._lib.KogarashiMoe()
    d.hidden, d.inter, d.experts, d.topk, d.tokens = layer.hidden, layer.inter, layer.experts, layer.topk, t
    d.router_w, d.router_ty = bufs["router"].data_ptr(), F.GGML_F32
    d.gate_w, d.gate_ty = bufs["gate"].data_ptr(), layer.gate_ty
    d.up_w, d.up_ty = bufs["up"].data_ptr(), layer.up_ty
    d.down_w, d.down_ty = bufs["down"].data_ptr(), layer.down_ty
    d.sh_gate_w, d.sh_up_w = bufs["sh_gate"].data_ptr(), bufs["sh_up"].data_ptr()
    d.sh_down_w, d.sh_inp_w = bufs["sh_down"].data_ptr(), bufs["sh_inp"].data_ptr()
    d.n, d.x = bufs["n"].data_ptr(), bufs["x"].data_ptr()
    d.logits, d.ids, d.prob = bufs["logits"].data_ptr(), bufs["ids"].data_ptr(), bufs["prob"].data_ptr()
    return d


@pytest.mark.parametrize("t", [2, 1])          # two tokens: four launches; one token: the single persistent launch
def test_static_scratch_entry_matches_workspace_entry(t):
    import darask_inference_engine_b200 as D
    lib = D._lib.lib()
    dev = torch.device("cuda", 0)
    layer, acts = W.kogarashi_layer(21, hidden=768, inter=512, experts=16, topk=4, tokens=t, shared=True, pool=16)
    up8 = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(-1)).to(dev)
    st = torch.cuda.current_stream(dev).cuda_stream

    def q6(raw, rows, k):                     # Q6_K tensors go through the device regrouping first
        out = torch.empty(lib.darask_q6k_repacked_bytes(rows, k), dtype=torch.uint8, device=dev)
        assert lib.darask_q6k_repack(out.data_ptr(), up8(raw).data_ptr(), rows, k, 0, st) == 0
        return out

    bufs = dict(router=up8(layer.router), gate=up8(layer.gate), up=up8(layer.up),
                down=q6(layer.down, layer.experts * layer.hidden, layer.inter),
                sh_gate=up8(layer.sh_gate), sh_up=up8(layer.sh_up),
                sh_down=q6(layer.sh_down, layer.hidden, layer.inter), sh_inp=up8(layer.sh_inp),
                n=torch.from_numpy(acts["n"]).to(dev), x=None,
                logits=torch.empty(t, layer.experts, device=dev), ids=torch.empty(t, layer.topk, dtype=torch.int32, device=dev),
                prob=torch.empty(t, layer.topk, device=dev))

    # the ordinary entry point with a caller-provided workspace
    bufs["x"] = torch.from_numpy(acts["x"].copy()).to(dev)
    d = _descriptor(D, layer, bufs, t)
    need = lib.kogarashi_moe_workspace_bytes(layer.hidden, layer.inter, layer.experts, layer.topk, t)
    assert need <= lib.kogarashi_moe_static_scratch_bytes()
    ws = torch.zeros(need, dtype=torch.uint8, device=dev)
    d.workspace, d.workspace_bytes = ws.data_ptr(), need
    assert lib.kogarashi_moe_layer(ctypes.byref(d), st) == 0
    torch.cuda.synchronize()
    expected = bufs["x"].cpu().numpy()
    expected_ids = bufs["ids"].cpu().numpy().copy()

    # the workspace-free entry point, two calls in a row on the same stream
    for call in range(2):
        bufs["x"] = torch.from_numpy(acts["x"].copy()).to(dev)
        bufs["ids"].fill_(-1)
        d = _descriptor(D, layer, bufs, t)
        d.workspace, d.workspace_bytes = None, 0
        assert lib.kogarashi_moe_layer_static(ctypes.byref(d), st) == 0, call
        torch.cuda.synchronize()
        got = bufs["x"].cpu().numpy()
        assert np.array_equal(bufs["ids"].cpu().numpy(), expected_ids), call
        W.check_output(got.astype(np.float64) - acts["x"], expected.astype(np.float64) - acts["x"])
        assert np.array_equal(got, expected), call      # same kernels, same order: identical bits
        word = ctypes.c_uint(99)
        assert lib.kogarashi_moe_static_status(ctypes.byref(word), st) == 0 and word.value == 0

    # a shape whose scratch need exceeds the built-in array is refused, nothing is launched
    d.tokens = 64
    assert lib.kogarashi_moe_workspace_bytes(layer.hidden, layer.inter, layer.experts, layer.topk, 64) > lib.kogarashi_moe_static_scratch_bytes()
    assert lib.kogarashi_moe_layer_static(ctypes.byref(d), st) == 1
    torch.cuda.synchronize()
