"""Generates tests/golden/hyt_layer.hyt and hyt_layer_expected.npz with the reference engine's own Python tools:
the table entries come from hayate_tools.hyt.encode_entry, the header from its HEADER struct (composed as
hayate_tools/glm53_convert.py composes a file) and the NVFP4 / FP8 tensor bytes from hayate_tools.quant.quantize.
The expected expert images are put together here tensor by tensor (gate, up, down, each at the next multiple of
256 bytes) so that the test has them independently of the library's assembly.

The header and tensor table of the reference's own golden file for the container (engines/hayate/python-tools/tests/
golden.hyt, the one its Rust and Python tests share) are recorded as `golden_head`; everything else in that file is
zero padding and the three tensors whose bytes the reference's Rust test states, so the test rebuilds the file.

Run where a reference checkout exists:  python tests/golden/make_hyt_layer_golden.py [ref]
"""
import hashlib
import os
import sys
import types

import numpy as np
import torch

os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
sys.dont_write_bytecode = True
here = os.path.dirname(os.path.abspath(__file__))
ref = sys.argv[1] if len(sys.argv) > 1 else os.path.join(here, "..", "..", "..", "reference")
pkg = types.ModuleType("hayate_tools")
pkg.__path__ = [os.path.join(ref, "engines/hayate/python-tools/hayate_tools")]
sys.modules["hayate_tools"] = pkg
from hayate_tools import quant  # noqa: E402
from hayate_tools.hyt import (E4M3, F32, FORMAT_VERSION, HEADER, NVFP4, PER_TENSOR, PLAIN, align, encode_entry,  # noqa: E402
                              storage_bytes)

EXPERTS, HIDDEN, INTER = 2, 64, 32
rng = np.random.Generator(np.random.PCG64(77))
tensors, weights = [], {}


def add(name, w, spec):
    raw = quant.quantize(torch.from_numpy(w), spec).numpy() if spec[0] != PLAIN else w.view(np.uint8).reshape(-1)
    assert raw.size == storage_bytes(list(w.shape), spec)
    tensors.append((name, list(w.shape), spec, raw))
    weights[name] = raw


add("mlp.gate.weight", (rng.standard_normal((EXPERTS, HIDDEN)) * 0.1).astype(np.float32), (PLAIN, F32, 0))
add("mlp.gate.e_score_correction_bias", np.zeros(EXPERTS, np.float32), (PLAIN, F32, 0))
for e in range(EXPERTS):                       # written down, up, gate: the reader must go by name, not by order
    for stem, shape in (("down", (HIDDEN, INTER)), ("up", (INTER, HIDDEN)), ("gate", (INTER, HIDDEN))):
        add(f"mlp.experts.{e}.{stem}_proj.weight", (rng.standard_normal(shape) * 0.05).astype(np.float32), (NVFP4, 0, 0))
for stem, shape in (("gate", (INTER, HIDDEN)), ("up", (INTER, HIDDEN)), ("down", (HIDDEN, INTER))):
    add(f"mlp.shared_experts.{stem}_proj.weight", (rng.standard_normal(shape) * 0.05).astype(np.float32), (NVFP4, 0, 0))
add("self_attn.o_proj.weight", (rng.standard_normal((8, 64)) * 0.3).astype(np.float32), (PER_TENSOR, E4M3, 0))

offset, entries = 0, []
for name, shape, spec, raw in tensors:
    entries.append((name, shape, spec, offset, raw.size))
    offset = align(offset + raw.size)
table = b"".join(encode_entry(*e) for e in entries)
base = align(64 + len(table))
digest = hashlib.sha256(b"hyt layer fixture").digest()
path = os.path.join(here, "hyt_layer.hyt")
with open(path, "wb") as out:
    out.write(HEADER.pack(b"HYT0", FORMAT_VERSION, 0, len(entries), 64, base, digest[:16]))
    out.write(table)
    for (name, shape, spec, rel, size), (_, _, _, raw) in zip(entries, tensors):
        out.seek(base + rel)
        out.write(raw.tobytes())
    out.truncate(base + entries[-1][3] + entries[-1][4])

images = []
for e in range(EXPERTS):
    img = b""
    for stem in ("gate", "up", "down"):
        raw = weights[f"mlp.experts.{e}.{stem}_proj.weight"].tobytes()
        img += raw + b"\0" * (-len(raw) % 256)
    images.append(np.frombuffer(img, np.uint8))
shared = b"".join(weights[f"mlp.shared_experts.{stem}_proj.weight"].tobytes().ljust(1792, b"\0") for stem in ("gate", "up", "down"))
gold = open(os.path.join(ref, "engines/hayate/python-tools/tests/golden.hyt"), "rb").read()
head_len = max(i for i in range(4096) if gold[i]) + 1
data = {4096: bytes([0x00, 0x38, 0xB8, 0x7E, 0, 0, 0x80, 0x3F]), 8192: bytes([0x00, 0x38]), 12288: bytes([0, 0, 0x80, 0x3F])}
rebuilt = bytearray(len(gold))
rebuilt[:head_len] = gold[:head_len]
for at, raw in data.items():
    rebuilt[at:at + len(raw)] = raw
assert bytes(rebuilt) == gold and len(gold) == 12292
np.savez_compressed(os.path.join(here, "hyt_layer_expected.npz"), golden_head=np.frombuffer(gold[:head_len], np.uint8), images=np.stack(images), shared=np.frombuffer(shared, np.uint8),
                    names=np.array([e[0] for e in entries]), offsets=np.array([base + e[3] for e in entries]),
                    sizes=np.array([e[4] for e in entries]), tags=np.array([e[2] for e in entries]),
                    source_hash=np.frombuffer(digest[:16], np.uint8))
print(os.path.getsize(path), np.stack(images).shape)
