"""Seeded synthetic MoE layers with the shapes and value distributions of the benchmark
configurations (activations bf16 ~N(0,1), weights ~N(0,0.02) quantized, Zipf or uniform
routing skew). Weights are quantized with the oracle's quantizers; distinct experts are
drawn from a small pool (expert e uses pool entry e % pool) so that full-size layers build
in seconds - every expert the router can pick still holds properly quantized data.
"""
from __future__ import annotations

import numpy as np

from oracle import formats as F
from oracle import layers as L


def rng_for(seed):
    return np.random.Generator(np.random.PCG64(seed))


def zipf_bias(rng, experts, s=1.1):
    """log of a Zipf(s) pmf over a random permutation of the experts (logit offset)."""
    pmf = 1.0 / np.arange(1, experts + 1) ** s
    pmf /= pmf.sum()
    return np.log(pmf[rng.permutation(experts)]).astype(np.float32)


def normal(rng, shape, std):
    return (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)


def kogarashi_layer(seed, hidden, inter, experts, topk, tokens, shared=True, zipf=None, pool=8,
                    gate_ty=F.GGML_Q4_K, down_ty=F.GGML_Q6_K):
    """-> (oracle KogarashiLayer, dict(n, x, bias)). Draw order: activations, router, bias,
    per pool entry gate/up/down, shared expert."""
    rng = rng_for(seed)
    n = F.bf16_round(normal(rng, (tokens, hidden), 1.0))
    x = normal(rng, (tokens, hidden), 1.0)
    router = normal(rng, (experts, hidden), 0.02)
    bias = zipf_bias(rng, experts, zipf) if zipf else None
    pool = min(pool, experts)
    g = [F.ggml_quantize(normal(rng, (inter, hidden), 0.02), gate_ty) for _ in range(pool)]
    u = [F.ggml_quantize(normal(rng, (inter, hidden), 0.02), gate_ty) for _ in range(pool)]
    d = [F.ggml_quantize(normal(rng, (hidden, inter), 0.02), down_ty) for _ in range(pool)]
    idx = np.arange(experts) % pool
    layer = L.KogarashiLayer(hidden, inter, experts, topk, router,
                             np.stack(g)[idx], np.stack(u)[idx], np.stack(d)[idx], gate_ty, gate_ty, down_ty)
    if shared:
        layer.sh_gate = F.ggml_quantize(normal(rng, (inter, hidden), 0.02), gate_ty)
        layer.sh_up = F.ggml_quantize(normal(rng, (inter, hidden), 0.02), gate_ty)
        layer.sh_down = F.ggml_quantize(normal(rng, (hidden, inter), 0.02), down_ty)
        layer.sh_inp = normal(rng, (hidden,), 0.02)
    return layer, dict(n=n, x=x, bias=bias)


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def check_output(got, ref, rel=1e-3, max_abs=2e-3):
    """The layer tolerance: relative L2 <= 1e-3 and max abs error <= 2e-3 * max|ref|."""
    r = rel_l2(got, ref)
    m = float(np.abs(np.asarray(got, np.float64) - np.asarray(ref, np.float64)).max())
    bound = max_abs * float(np.abs(ref).max())
    assert r <= rel, f"relative L2 {r:.3e} > {rel}"
    assert m <= bound, f"max abs {m:.3e} > {bound:.3e}"
    return r, m


def tsumuji_layer(seed, hidden, inter, experts, topk, tokens, pool=8, uniform_logits=False):
    """-> (oracle TsumujiLayer, dict(x, logits)). NVFP4 routed experts in the linear layout, dense bf16
    shared expert, bf16 router with the shared-gate row. `uniform_logits`: logits drawn i.i.d. uniform
    (near-balanced load) instead of coming from the router projection."""
    rng = rng_for(seed)
    x = F.bf16_round(normal(rng, (tokens, hidden), 1.0))
    router = F.bf16_round(normal(rng, (experts + 1, hidden), 0.02))
    pool = min(pool, experts)
    blocks, gs = [], []
    for _ in range(pool):
        b, g = F.tsumuji_expert_block(normal(rng, (inter, hidden), 0.02), normal(rng, (inter, hidden), 0.02),
                                      normal(rng, (hidden, inter), 0.02))
        blocks.append(b)
        gs.append(g)
    idx = np.arange(experts) % pool
    shared_gu = F.bf16_round(normal(rng, (2 * inter, hidden), 0.02))
    shared_down = F.bf16_round(normal(rng, (hidden, inter), 0.02))
    layer = L.TsumujiLayer(hidden, inter, experts, topk, router, np.stack(blocks)[idx], np.stack(gs)[idx], shared_gu, shared_down)
    logits = rng.uniform(-1, 1, (tokens, experts + 1)).astype(np.float32) if uniform_logits else None
    return layer, dict(x=x, logits=logits)


def hayate_layer(seed, hidden, inter, experts, topk, tokens, scale=2.5, pool=8):
    """-> (oracle HayateLayer, dict(x)). bf16 activations and router, float32 bias ~N(0, 0.1), NVFP4 images
    in the tiled-scale layout (gate | up | down at the 256-byte aligned stride), one shared expert image."""
    rng = rng_for(seed)
    x = F.bf16_round(normal(rng, (tokens, hidden), 1.0))
    router = F.bf16_round(normal(rng, (experts, hidden), 0.02))
    bias = normal(rng, (experts,), 0.1)
    pool = min(pool, experts)
    imgs = [F.hayate_expert_image(normal(rng, (inter, hidden), 0.02), normal(rng, (inter, hidden), 0.02),
                                  normal(rng, (hidden, inter), 0.02)) for _ in range(pool)]
    shared = F.hayate_expert_image(normal(rng, (inter, hidden), 0.02), normal(rng, (inter, hidden), 0.02),
                                   normal(rng, (hidden, inter), 0.02))
    stride = F.hayate_expert_stride(hidden, inter)
    layer = L.HayateLayer(hidden, inter, experts, topk, scale, router, bias, np.stack(imgs)[np.arange(experts) % pool], stride, shared)
    return layer, dict(x=x)


def fp8_layer(seed, hidden, inter, experts, topk, tokens, pool=4, zipf=None):
    """Block-FP8 experts (a pool of distinct experts repeated), bf16-valued activations, router logits."""
    rng = rng_for(seed)
    pool = min(pool, experts)
    mats = []
    for _ in range(pool):
        mats.append(tuple(F.fp8_block_quantize(normal(rng, shp, std)) for shp, std in
                          (((inter, hidden), hidden ** -0.5), ((inter, hidden), hidden ** -0.5), ((hidden, inter), inter ** -0.5))))
    layer = L.Fp8Layer(hidden, inter, experts, topk)
    for e in range(experts):
        g, u, d = mats[e % pool]
        layer.gate.append(g), layer.up.append(u), layer.down.append(d)
    x = F.bf16_round(normal(rng, (tokens, hidden), 1.0))
    logits = normal(rng, (tokens, experts), 1.0)
    if zipf:
        logits = (logits + zipf_bias(rng, experts, zipf)[None, :]).astype(np.float32)
    return layer, dict(x=x, logits=logits)
