"""Child process of tests/test_driver_context_gpu.py.

Plays the reference's host (common/cuda/src/lib.rs:57-76, 130-145, 395-402): `cuInit`, the device's primary context
retained and made current through the Driver API, memory from `cuMemAlloc`, a non-blocking stream from
`cuStreamCreate`; no runtime-API call and no torch CUDA call happens in this process before the library is entered.
Then one Kogarashi layer for one token and for three tokens through the C ABI, results printed as JSON."""
import ctypes
import json
import sys

import numpy as np
from cuda.bindings import driver as cu

from oracle import formats as F
from oracle import layers as L
from tests import workloads as W


def ok(res):
    err, *rest = res
    assert int(err) == 0, err
    return rest[0] if len(rest) == 1 else rest


def main():
    import darask_inference_engine_b200 as D
    ok(cu.cuInit(0))
    dev = ok(cu.cuDeviceGet(0))
    ctx = ok(cu.cuDevicePrimaryCtxRetain(dev))
    ok(cu.cuCtxSetCurrent(ctx))
    stream = ok(cu.cuStreamCreate(cu.CUstream_flags.CU_STREAM_NON_BLOCKING.value))
    lib = D._lib.lib()
    st = int(stream)
    held = []

    def upload(a):
        a = np.ascontiguousarray(a)
        p = ok(cu.cuMemAlloc(max(a.nbytes, 1)))
        held.append(p)
        ok(cu.cuMemcpyHtoD(p, a.view(np.uint8).reshape(-1), a.nbytes))
        return int(p)

    def alloc(nbytes):
        p = ok(cu.cuMemAlloc(nbytes))
        held.append(p)
        return int(p)

    def download(ptr, shape, dtype):
        out = np.empty(shape, dtype)
        ok(cu.cuMemcpyDtoH(out.view(np.uint8).reshape(-1), ptr, out.nbytes))
        return out

    report = {}
    for tokens in (1, 3):
        layer, acts = W.kogarashi_layer(21, hidden=512, inter=256, experts=16, topk=4, tokens=tokens, pool=16)
        d = D._lib.KogarashiMoe()
        d.hidden, d.inter, d.experts, d.topk, d.tokens = layer.hidden, layer.inter, layer.experts, layer.topk, tokens
        d.router_w, d.router_ty = upload(layer.router), F.GGML_F32
        d.gate_w, d.gate_ty = upload(layer.gate), layer.gate_ty
        d.up_w, d.up_ty = upload(layer.up), layer.up_ty

        def q6(raw, rows, k):        # Q6_K tensors go through the library's lossless regrouping
            src = upload(raw)
            dst = alloc(lib.darask_q6k_repacked_bytes(rows, k))
            assert lib.darask_q6k_repack(dst, src, rows, k, 0, st) == 0
            return dst
        assert layer.down_ty == F.GGML_Q6_K
        d.down_w, d.down_ty = q6(layer.down, layer.experts * layer.hidden, layer.inter), layer.down_ty
        d.sh_gate_w, d.sh_up_w = upload(layer.sh_gate), upload(layer.sh_up)
        d.sh_down_w = q6(layer.sh_down, layer.hidden, layer.inter)
        d.sh_inp_w = upload(layer.sh_inp)
        d.n, d.x = upload(acts["n"]), upload(acts["x"])
        d.logits, d.ids, d.prob = alloc(tokens * layer.experts * 4), alloc(tokens * layer.topk * 4), alloc(tokens * layer.topk * 4)
        need = lib.kogarashi_moe_workspace_bytes(layer.hidden, layer.inter, layer.experts, layer.topk, tokens)
        d.workspace, d.workspace_bytes = alloc(need), need
        assert lib.kogarashi_moe_workspace_init(d.workspace, need, st) == 0
        assert lib.kogarashi_moe_layer(ctypes.byref(d), st) == 0
        status = ctypes.c_uint(9)
        assert lib.kogarashi_moe_status(d.workspace, ctypes.byref(status), st) == 0
        ok(cu.cuStreamSynchronize(stream))
        out = download(d.x, acts["x"].shape, np.float32)
        logits = download(d.logits, (tokens, layer.experts), np.float32)
        ids = download(d.ids, (tokens, layer.topk), np.int32)
        ref = L.kogarashi_forward(layer, acts["x"], acts["n"], logits=logits)
        delta_ref = ref["out"].astype(np.float64) - acts["x"]
        delta_got = out.astype(np.float64) - acts["x"]
        report[str(tokens)] = dict(status=int(status.value), ids_equal=bool(np.array_equal(ids, ref["ids"])),
                                   rel_l2=float(W.rel_l2(delta_got, delta_ref)))
    for p in held:
        ok(cu.cuMemFree(p))
    ok(cu.cuStreamDestroy(stream))
    ok(cu.cuDevicePrimaryCtxRelease(dev))
    print(json.dumps(report))


if __name__ == "__main__":
    sys.exit(main())
