"""Packing of Tsumuji checkpoint tensors into the device expert block (`tsumuji_loader.pack_experts`, `csf_decode`):
the reference's loader is engines/tsumuji/crates/tsumuji-engine/src/weights.rs:445-541."""
import numpy as np
import pytest

from oracle import formats as F
from tests import workloads as W


def checkpoint(experts, hidden, inter, style, csf, seed=3):
    """Tensors of `experts` routed experts in one of the two export styles, and the blocks the oracle builds from the same
    float matrices."""
    rng = W.rng_for(seed)
    tensors, blocks, gss = {}, [], []
    for e in range(experts):
        mats = [W.normal(rng, (inter, hidden), 0.02), W.normal(rng, (inter, hidden), 0.02), W.normal(rng, (hidden, inter), 0.02)]
        block, gs = F.tsumuji_expert_block(*mats)
        blocks.append(block), gss.append(gs)
        for proj, m in zip(("gate_proj", "up_proj", "down_proj"), mats):
            codes, scales, g = F.nvfp4_linear_quantize(m)
            p = f"model.layers.0.mlp.experts.{e}.{proj}"
            if style == "modelopt":
                tensors[f"{p}.weight"] = codes
                tensors[f"{p}.weight_scale_2"] = np.array([g], np.float32)
            else:
                tensors[f"{p}.weight_packed"] = codes
                tensors[f"{p}.weight_global_scale"] = np.array([np.float32(1.0) / g], np.float32)
            if csf:
                import darask_inference_engine_b200 as D
                fixed, exc = D.tsumuji_loader.csf_encode(scales)
                tensors[f"{p}.weight_scale.nvfp4_csf_fixed"] = fixed.reshape(m.shape[0] // 16, -1)
                tensors[f"{p}.weight_scale.nvfp4_csf_exceptions"] = exc
            else:
                tensors[f"{p}.weight_scale"] = scales
    return tensors, np.concatenate(blocks), np.stack(gss)


@pytest.mark.parametrize("style", ["modelopt", "compressed-tensors"])
@pytest.mark.parametrize("csf", [False, True])
def test_pack_experts_gives_the_oracle_block(style, csf):
    import darask_inference_engine_b200 as D
    tensors, blocks, gs = checkpoint(3, 256, 128, style, csf)
    buf, got = D.tsumuji_loader.pack_experts(tensors, "model.layers.0.mlp.experts", 3, 256, 128)
    assert buf.size == 3 * D.tsumuji_loader.expert_stride(256, 128) and np.array_equal(buf, blocks)
    if style == "modelopt":
        assert np.array_equal(got, gs)
    else:                      # 1 / (1 / g): one rounding each way
        np.testing.assert_allclose(got, gs, rtol=2e-7)


def test_pack_experts_of_one_rank_is_a_slice_of_the_whole():
    """Expert parallelism: rank g packs experts [g*E/G, (g+1)*E/G); the blocks are the same bytes as in the whole buffer."""
    import darask_inference_engine_b200 as D
    tensors, blocks, gs = checkpoint(4, 256, 128, "modelopt", False)
    stride = D.tsumuji_loader.expert_stride(256, 128)
    for rank in range(2):
        buf, got = D.tsumuji_loader.pack_experts(tensors, "model.layers.0.mlp.experts", 2, 256, 128, first=2 * rank)
        assert np.array_equal(buf, blocks[2 * rank * stride:(2 * rank + 2) * stride]) and np.array_equal(got, gs[2 * rank:2 * rank + 2])
    with pytest.raises(KeyError):
        D.tsumuji_loader.pack_experts(tensors, "model.layers.0.mlp.experts", 2, 256, 128, first=3)


def test_csf_scales_round_trip_with_exceptions_and_wrapping():
    import darask_inference_engine_b200 as D
    rng = np.random.default_rng(5)
    scales = (rng.integers(0x30, 0x3C, (32, 8))).astype(np.uint8)       # offsets within 4 bits of the row minimum
    scales[3, 5] = 0x7E                                                 # far from its row: an exception
    scales[17, 0] = 0x00                                                # a new row minimum: the others become exceptions
    fixed, exc = D.tsumuji_loader.csf_encode(scales)
    assert exc.size % 4 == 0 and exc.size > 0
    assert np.array_equal(D.tsumuji_loader.csf_decode(fixed, exc, 32, 8), scales)
    # base + offset wraps modulo 256, as the reference's wrapping_add
    blk = np.zeros(16 + 16 * 2 // 2, np.uint8)
    blk[0], blk[16] = 250, 0x9F                                         # row 0: base 250, offsets 15 and 9
    out = D.tsumuji_loader.csf_decode(blk, np.zeros(0, np.uint8), 16, 2)
    assert out[0, 0] == (250 + 15) % 256 and out[0, 1] == (250 + 9) % 256
    with pytest.raises(ValueError):
        D.tsumuji_loader.csf_decode(fixed[:-1], exc, 32, 8)
    bad = np.array([(1 << 24) | 32 * 8], "<u4").view(np.uint8)          # index one past the end
    with pytest.raises(ValueError, match="out of range"):
        D.tsumuji_loader.csf_decode(fixed, bad, 32, 8)


def test_pack_experts_reports_missing_and_misshaped_tensors():
    import darask_inference_engine_b200 as D
    tensors, _, _ = checkpoint(1, 256, 128, "modelopt", False)
    t = dict(tensors)
    del t["model.layers.0.mlp.experts.0.up_proj.weight_scale_2"]
    with pytest.raises(KeyError):
        D.tsumuji_loader.pack_experts(t, "model.layers.0.mlp.experts", 1, 256, 128)
    t = dict(tensors)
    t["model.layers.0.mlp.experts.0.down_proj.weight"] = t["model.layers.0.mlp.experts.0.down_proj.weight"].T.copy()
    with pytest.raises(ValueError):
        D.tsumuji_loader.pack_experts(t, "model.layers.0.mlp.experts", 1, 256, 128)


def test_safetensors_source(tmp_path):
    import torch
    from safetensors.torch import save_file
    import darask_inference_engine_b200 as D
    tensors, blocks, gs = checkpoint(2, 256, 128, "compressed-tensors", False)
    half = len(tensors) // 2
    names = sorted(tensors)
    for i, part in enumerate((names[:half], names[half:])):
        out = {}
        for n in part:
            a = torch.from_numpy(np.ascontiguousarray(tensors[n]))
            out[n] = a.view(torch.float8_e4m3fn) if n.endswith(".weight_scale") else a
        save_file(out, str(tmp_path / f"model-{i}.safetensors"))
    src = D.tsumuji_loader.SafetensorsSource(sorted(str(p) for p in tmp_path.glob("*.safetensors")))
    buf, got = D.tsumuji_loader.pack_experts(src, "model.layers.0.mlp.experts", 2, 256, 128)
    assert np.array_equal(buf, blocks)
    np.testing.assert_allclose(got, gs, rtol=2e-7)
