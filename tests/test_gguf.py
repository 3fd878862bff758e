"""GGUF container reader / writer (`darask_inference_engine_b200.gguf`) and loading a layer from a file.

The byte layout follows the reference's reader (common/formats/src/gguf.rs: magic, version 2 or 3, counts, typed
metadata, tensor directory, data aligned to `general.alignment`) and its upload loop (kogarashi engine.rs:73-107)."""
import struct

import numpy as np
import pytest
import torch

from oracle import formats as F
from oracle import layers as L
from tests import workloads as W


def layer_file(tmp_path, seed=41, hidden=512, inter=256, experts=8, topk=2, shared=True, alignment=32, block=3):
    import darask_inference_engine_b200 as D
    layer, acts = W.kogarashi_layer(seed, hidden, inter, experts, topk, 1, shared=shared, pool=experts)
    name = lambda s: f"blk.{block}.{s}"
    tensors = [(name("ffn_gate_inp.weight"), (hidden, experts), F.GGML_F32, layer.router),
               (name("ffn_gate_exps.weight"), (hidden, inter, experts), layer.gate_ty, layer.gate),
               (name("ffn_up_exps.weight"), (hidden, inter, experts), layer.up_ty, layer.up),
               (name("ffn_down_exps.weight"), (inter, hidden, experts), layer.down_ty, layer.down)]
    if shared:
        tensors += [(name("ffn_gate_shexp.weight"), (hidden, inter), layer.gate_ty, layer.sh_gate),
                    (name("ffn_up_shexp.weight"), (hidden, inter), layer.up_ty, layer.sh_up),
                    (name("ffn_down_shexp.weight"), (inter, hidden), layer.down_ty, layer.sh_down),
                    (name("ffn_gate_inp_shexp.weight"), (hidden,), F.GGML_F32, layer.sh_inp)]
    tensors.append(("token_embd.weight", (hidden, 5), F.GGML_F32, np.arange(5 * hidden, dtype=np.float32)))
    meta = {"general.architecture": "qwen35moe", "qwen35moe.expert_count": experts, "qwen35moe.expert_used_count": topk,
            "qwen35moe.attention.layer_norm_rms_epsilon": 1e-6, "tokenizer.ggml.tokens": ["a", "b"], "some.flag": True, "neg": -3}
    path = tmp_path / "layer.gguf"
    D.gguf.write(path, meta, tensors, alignment=alignment)
    return path, layer, acts, tensors


@pytest.mark.parametrize("alignment", [32, 64, 4096])
def test_header_round_trip(tmp_path, alignment):
    import darask_inference_engine_b200 as D
    path, layer, _, tensors = layer_file(tmp_path, alignment=alignment)
    g = D.gguf.GgufFile(path)
    assert g.meta["general.architecture"] == "qwen35moe" and g.meta["qwen35moe.expert_count"] == 8
    assert g.meta["tokenizer.ggml.tokens"] == ["a", "b"] and g.meta["some.flag"] is True and g.meta["neg"] == -3
    assert abs(g.meta["qwen35moe.attention.layer_norm_rms_epsilon"] - 1e-6) < 1e-12
    assert D.gguf.layer_shape(g, 3) == (512, 256, 8)
    for name, ne, ty, raw in tensors:
        t = g.tensors[name]
        assert t.ne == tuple(ne) and t.ty == ty and t.offset % alignment == 0
        assert np.array_equal(np.array(g.read(name)), np.ascontiguousarray(raw).view(np.uint8).reshape(-1))
    # a block of experts is one byte range of an `_exps` tensor
    t = g.tensors["blk.3.ffn_down_exps.weight"]
    lo, n, ne = D.gguf.expert_block(t, 2, 3)
    per = D.formats.ggml_tensor_bytes(t.ty, t.ne[:-1])
    assert (lo, n, ne) == (2 * per, 3 * per, (256, 512, 3))
    assert np.array_equal(np.array(g.read(t.name, lo, n)), np.ascontiguousarray(layer.down).view(np.uint8).reshape(-1)[lo:lo + n])
    with pytest.raises(ValueError):
        D.gguf.expert_block(t, 6, 3)


def test_rejects_what_the_reference_rejects(tmp_path):
    import darask_inference_engine_b200 as D
    path, *_ = layer_file(tmp_path)
    raw = path.read_bytes()
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + raw[4:])
    with pytest.raises(ValueError, match="not a GGUF"):
        D.gguf.GgufFile(bad)
    bad.write_bytes(raw[:4] + struct.pack("<I", 1) + raw[8:])
    with pytest.raises(ValueError, match="version"):
        D.gguf.GgufFile(bad)
    bad.write_bytes(raw[:len(raw) - 100])                       # the last tensor would run past the end of the file
    with pytest.raises(ValueError, match="exceeds file"):
        D.gguf.GgufFile(bad)
    bad.write_bytes(raw[:40])
    with pytest.raises(ValueError, match="truncated"):
        D.gguf.GgufFile(bad)
    with pytest.raises(ValueError):                               # Q4_K rows must hold whole 256-wide blocks (config.rs:86-105)
        D.gguf.write(tmp_path / "x.gguf", {}, [("t", (100, 2), F.GGML_Q4_K, np.zeros(10, np.uint8))])


@pytest.mark.gpu
@pytest.mark.parametrize("shared", [True, False])
def test_layer_loaded_from_file_matches_the_oracle(tmp_path, shared):
    import darask_inference_engine_b200 as D
    path, layer, acts, _ = layer_file(tmp_path, shared=shared)
    m = D.gguf.load_layer(path, 3, topk=2)
    x = torch.from_numpy(acts["x"].copy()).cuda()
    m.forward(x, torch.from_numpy(acts["n"]).cuda())
    torch.cuda.synchronize()
    assert m.status() == 0
    ref = L.kogarashi_forward(layer, acts["x"], acts["n"], logits=m.logits[:1].cpu().numpy())
    assert np.array_equal(m.ids[:1].cpu().numpy(), ref["ids"])
    W.check_output(x.cpu().numpy().astype(np.float64) - acts["x"], ref["out"].astype(np.float64) - acts["x"])
