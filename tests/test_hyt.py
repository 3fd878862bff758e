"""`.hyt` container reader and the assembly of expert images (`darask_inference_engine_b200.hyt`).

Pinned on two files: the reference's own golden (python-tools/tests/golden.hyt, rebuilt from its recorded header and
table; with the values its Rust test
`shared_python_golden_loads_and_reads` asserts, common/core/src/hyt.rs:528-557, and the mutations of
`file_rejects_...`, hyt.rs:660-676) and a small layer file written with the reference's Python tools
(tests/golden/make_hyt_layer_golden.py). The image layout follows glm53/experts.rs `read_image`."""
import os
import struct

import numpy as np
import pytest

from oracle import formats as F

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def hyt():
    import darask_inference_engine_b200 as D
    return D.hyt


def reference_golden() -> bytes:
    """The reference's golden file: its header and table as recorded from the file, zero padding, and the three tensors
    with the bytes its Rust test states (hyt.rs:546-551); 12292 bytes."""
    head = np.load(os.path.join(GOLD, "hyt_layer_expected.npz"))["golden_head"].tobytes()
    raw = bytearray(12292)
    raw[:len(head)] = head
    raw[4096:4104] = bytes([0x00, 0x38, 0xB8, 0x7E, 0, 0, 0x80, 0x3F])
    raw[8192:8194] = bytes([0x00, 0x38])
    raw[12288:12292] = struct.pack("<f", 1.0)
    return bytes(raw)


def test_reference_golden_file(tmp_path):
    H = hyt()
    path = tmp_path / "golden.hyt"
    path.write_bytes(reference_golden())
    f = H.HytFile(path, machine=0)
    assert f.source_hash.hex() == "c5e8ba63157fbff9984d1f11bc7ac56a"
    got = [(e.name, e.quant, e.shape, e.offset - 4096, e.nbytes) for e in f.entries]
    assert got == [("重み", (H.TAG_PER_TENSOR, 3, 0), (2, 2), 0, 8), ("half", (H.TAG_PLAIN, 2, 0), (), 4096, 2),
                   ("float", (H.TAG_PLAIN, 0, 0), (1,), 8192, 4)]
    assert bytes(f.read("重み")) == bytes([0x00, 0x38, 0xB8, 0x7E, 0, 0, 0x80, 0x3F])
    assert bytes(f.read("half")) == bytes([0x00, 0x38])
    assert bytes(f.read("float")) == struct.pack("<f", 1.0)
    with pytest.raises(ValueError):
        H.HytFile(path, machine=1)       # converted for the other machine
    whole = bytes(f.read("重み"))
    for a in range(9):
        for b in range(a, 9):
            assert bytes(f.read("重み", a, b - a)) == whole[a:b]
    for first, n in [(8, 1), (9, 0), (1 << 63, 1)]:
        with pytest.raises(ValueError):
            f.read("重み", first, n)
    with pytest.raises(ValueError):
        f.read("half", 1, 2)                       # bytes behind an entry are not readable through it
    with pytest.raises(KeyError):
        f.read("absent")


@pytest.mark.parametrize("at,fmt,value", [
    (0, "<I", 0), (4, "<I", 1), (8, "<I", 2), (12, "<I", 2 ** 32 - 1), (16, "<Q", 4080), (24, "<Q", 16384),
    (106, "<Q", 12288), (106, "<Q", 2 ** 64 - 4096), (146, "<Q", 0), (114, "<Q", 9)])
def test_reference_golden_mutations_are_rejected(tmp_path, at, fmt, value):
    raw = bytearray(reference_golden())
    struct.pack_into(fmt, raw, at, value)
    p = tmp_path / "bad.hyt"
    p.write_bytes(raw)
    with pytest.raises((ValueError, UnicodeDecodeError)):
        hyt().HytFile(p)


def test_truncated_files_are_rejected(tmp_path):
    raw = reference_golden()
    for n in (0, 63, 4095, len(raw) - 1):
        p = tmp_path / f"t{n}.hyt"
        p.write_bytes(raw[:n])
        with pytest.raises(ValueError):
            hyt().HytFile(p)


def test_storage_bytes():
    H = hyt()
    assert H.storage_bytes((2, 1, 16), (H.TAG_NVFP4, 0, 0)) == 1048                  # hyt.rs:692
    assert H.storage_bytes((129, 80), (H.TAG_NVFP4, 0, 0)) == F.nvfp4_tiled_bytes(129, 80)
    assert H.storage_bytes((2048, 4096), (H.TAG_EXL3, 5, 2)) == 2048 * 4096 * 5 // 16 + 2 * 6144
    assert H.storage_bytes((2, 64), (H.TAG_MXFP8, 0, 0)) == 128 + 128 * 4
    assert H.storage_bytes((2, 64), (H.TAG_Q4_BF16, 0, 32)) == 64 + 2 * 2 * 2
    assert H.storage_bytes((2, 64), (H.TAG_INT8_ROW, 0, 256)) == 128 + 8
    assert H.storage_bytes((2, 64), (H.TAG_PER_TENSOR, 8, 0)) == 64 + 4              # int4
    assert H.storage_bytes((), (H.TAG_PLAIN, 0, 0)) == 4
    for shape, quant in [((17,), (H.TAG_NVFP4, 0, 0)), ((2, 64), (H.TAG_PLAIN, 9, 0)), ((2, 64), (H.TAG_PLAIN, 0, 1)),
                         ((2, 64), (H.TAG_Q4_BF16, 0, 0)), ((0,), (H.TAG_PLAIN, 0, 0)), ((1,) * 7, (H.TAG_PLAIN, 0, 0)),
                         ((2, 64), (8, 0, 0)), ((100, 128), (H.TAG_EXL3, 4, 0))]:
        with pytest.raises(ValueError):
            H.storage_bytes(shape, quant)


def test_write_read_round_trip_and_empty_file(tmp_path):
    H = hyt()
    rng = np.random.default_rng(3)
    tensors = [(f"重み{i}", (2, 64), q, rng.integers(0, 255, H.storage_bytes((2, 64), q), dtype=np.uint8))
               for i, q in enumerate([(H.TAG_NVFP4, 0, 0), (H.TAG_MXFP8, 0, 0), (H.TAG_Q4_BF16, 0, 32), (H.TAG_INT8_ROW, 0, 0),
                                      (H.TAG_PLAIN, 1, 0), (H.TAG_PER_TENSOR, 3, 0)])]
    tensors.append(("scalar", (), (H.TAG_PLAIN, 0, 0), np.float32([2.5])))
    H.write(tmp_path / "a.hyt", tensors, machine=1, source_hash=bytes(range(16)))
    f = H.HytFile(tmp_path / "a.hyt", machine=1)
    assert f.source_hash == bytes(range(16)) and [e.name for e in f.entries] == [t[0] for t in tensors]
    for name, shape, quant, raw in tensors:
        e = f.by_name[name]
        assert (e.shape, e.quant) == (tuple(shape), quant) and e.offset % 4096 == 0
        assert np.array_equal(f.read(name), np.ascontiguousarray(raw).view(np.uint8).reshape(-1))
    H.write(tmp_path / "empty.hyt", [])
    assert H.HytFile(tmp_path / "empty.hyt").entries == []
    H.write(tmp_path / "dup.hyt", [("a", (1,), (H.TAG_PLAIN, 0, 0), np.float32([1])), ("a", (1,), (H.TAG_PLAIN, 0, 0), np.float32([1]))])
    with pytest.raises(ValueError):
        H.HytFile(tmp_path / "dup.hyt")


def test_layer_images_from_reference_written_file():
    H = hyt()
    want = np.load(os.path.join(GOLD, "hyt_layer_expected.npz"))
    f = H.HytFile(os.path.join(GOLD, "hyt_layer.hyt"))
    assert [e.name for e in f.entries] == list(want["names"])
    assert [e.offset for e in f.entries] == list(want["offsets"]) and [e.nbytes for e in f.entries] == list(want["sizes"])
    assert [list(e.quant) for e in f.entries] == want["tags"].tolist() and f.source_hash == want["source_hash"].tobytes()
    images = H.layer_images(f, 2)
    assert images.dtype == np.uint8 and np.array_equal(images, want["images"])
    # the image is what the oracle's layout functions expect: stride, and a decode that agrees with the tensor decoded alone
    hidden, inter = 64, 32
    stride = F.hayate_expert_stride(hidden, inter)
    assert images.shape == (2, 3 * stride)
    for e in range(2):
        for i, (stem, n, k) in enumerate((("gate", inter, hidden), ("up", inter, hidden), ("down", hidden, inter))):
            alone = np.array(f.read(f"mlp.experts.{e}.{stem}_proj.weight"))
            part = images[e, i * stride:(i + 1) * stride]
            assert np.array_equal(F.nvfp4_tiled_decode(part[:alone.size], n, k), F.nvfp4_tiled_decode(alone, n, k))
            assert not part[alone.size:].any()
            w = F.nvfp4_tiled_decode(alone, n, k)
            assert np.isfinite(w).all() and 0.01 < np.abs(w).max() < 1.0          # weights were drawn with std 0.05
    with pytest.raises(KeyError):
        H.expert_image(f, 2)
    assert np.array_equal(H.layer_images(f, 1, first=1), want["images"][1:])          # one rank's block of experts
    assert np.array_equal(H.mlp_image(f, "mlp.shared_experts"), want["shared"])
    router = H.plain_tensor(f, "mlp.gate.weight")
    assert router.shape == (2, 64) and router.dtype == np.float32 and 0 < np.abs(router).max() < 1
    assert not H.plain_tensor(f, "mlp.gate.e_score_correction_bias").any()
    with pytest.raises(ValueError):
        H.plain_tensor(f, "self_attn.o_proj.weight")


def test_plain_tensor_decodes_bf16_and_f16(tmp_path):
    H = hyt()
    v = np.float32([1.0, -2.5, 0.15625, 30720.0])
    bf = (v.view(np.uint32) >> 16).astype(np.uint16)
    H.write(tmp_path / "p.hyt", [("b", (2, 2), (H.TAG_PLAIN, 1, 0), bf), ("h", (4,), (H.TAG_PLAIN, 2, 0), v.astype(np.float16))])
    f = H.HytFile(tmp_path / "p.hyt")
    assert np.array_equal(H.plain_tensor(f, "b"), v.reshape(2, 2)) and np.array_equal(H.plain_tensor(f, "h"), v.astype(np.float16).astype(np.float32))


def test_invalid_nvfp4_images_are_rejected(tmp_path):
    H = hyt()
    src = H.HytFile(os.path.join(GOLD, "hyt_layer.hyt"))
    n, k = 32, 64
    for case in ("nan_scale", "zero_global", "inf_global", "ok"):
        tensors = []
        for stem, shape in (("gate", (n, k)), ("up", (n, k)), ("down", (k, n))):
            raw = np.array(src.read(f"mlp.experts.0.{stem}_proj.weight"))
            if stem == "up":
                if case == "nan_scale":
                    raw[n * k // 2 + 5] = 0xFF
                elif case == "zero_global":
                    raw[-4:] = 0
                elif case == "inf_global":
                    raw[-4:] = np.frombuffer(struct.pack("<f", float("inf")), np.uint8)
            tensors.append((f"mlp.experts.0.{stem}_proj.weight", shape, (H.TAG_NVFP4, 0, 0), raw))
        H.write(tmp_path / f"{case}.hyt", tensors)
        f = H.HytFile(tmp_path / f"{case}.hyt")
        if case == "ok":
            assert H.expert_image(f, 0).size == 3 * F.hayate_expert_stride(k, n)
        else:
            with pytest.raises(ValueError):
                H.expert_image(f, 0)


def test_load_layer_hands_the_file_to_the_layer(monkeypatch):
    """`load_layer` without a GPU: the layer class is replaced by a recorder; the tensors it receives are the file's."""
    import torch

    import darask_inference_engine_b200.hayate as hayate_mod
    H = hyt()
    want = np.load(os.path.join(GOLD, "hyt_layer_expected.npz"))
    seen = {}

    class Recorder:
        def __init__(self, hidden, inter, experts, topk, scale, max_tokens, device):
            seen["shape"] = (hidden, inter, experts, topk, scale, max_tokens, device)

        def load(self, router, bias, images, shared):
            seen.update(router=router, bias=bias, images=images, shared=shared)

    monkeypatch.setattr(hayate_mod, "HayateMoeLayer", Recorder)
    m = H.load_layer(os.path.join(GOLD, "hyt_layer.hyt"), topk=1, max_tokens=4, device="cpu")
    assert isinstance(m, Recorder) and seen["shape"] == (64, 32, 2, 1, 2.5, 4, "cpu")
    assert seen["router"].shape == (2, 64) and seen["bias"].dtype == torch.float32
    assert np.array_equal(seen["images"].numpy(), want["images"]) and np.array_equal(seen["shared"].numpy(), want["shared"])
