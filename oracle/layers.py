"""Whole MoE FFN layers of the three executors, restated on the CPU (numpy, float64 sums).

Test infrastructure only.  Weights are decoded exactly as the reference kernels decode
them (``formats``), products are summed in float64 and rounded to the storage type at the
points where the reference rounds (bf16 in Hayate, float32 elsewhere).  The result is the
"fp32-accumulated reference" up to float32 summation noise (~1e-6 relative), far inside
the 1e-3 relative-L2 tolerance the layers are compared under.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from . import formats as F
from . import routing as R


def _silu64(g):
    return g / (1.0 + np.exp(-g))


# ----------------------------------------------------------------------------
# Kogarashi (qwen3.5-moe; kernels/native.cu, engine.rs:530-632)
# ----------------------------------------------------------------------------

@dataclass
class KogarashiLayer:
    hidden: int
    inter: int
    experts: int
    topk: int
    router: np.ndarray            # float32 [E,H]
    gate: np.ndarray              # bytes [E, F, rowbytes(H)]
    up: np.ndarray
    down: np.ndarray              # bytes [E, H, rowbytes(F)]
    gate_ty: int = F.GGML_Q4_K
    up_ty: int = F.GGML_Q4_K
    down_ty: int = F.GGML_Q6_K
    sh_gate: np.ndarray | None = None     # bytes [F, rowbytes(H)]
    sh_up: np.ndarray | None = None
    sh_down: np.ndarray | None = None     # bytes [H, rowbytes(F)]
    sh_inp: np.ndarray | None = None      # float32 [H]: shared-expert gate projection


def kogarashi_logits(layer: KogarashiLayer, n: np.ndarray) -> np.ndarray:
    """router GEMV, float32 weights x float32 activations (engine.rs:530-538)."""
    return (layer.router.astype(np.float64) @ n.astype(np.float64).T).T.astype(np.float32)


def kogarashi_entry(x: np.ndarray, attn_out, norm_w: np.ndarray, eps: float):
    """The two launches in front of the MoE block: `residual` (x += out) and `rms_native`
    (n = x * rsqrt(sum(x^2) / h + eps) * w), engines/kogarashi/kernels/native.cu:89-96, called at engine.rs:507-526.
    float32 x and n as the kernels produce them, except that the sum of squares is taken in float64 here (the kernel adds
    in float32 in a fixed thread order; the difference stays below 1e-6 relative)."""
    x = np.asarray(x, np.float32)
    if attn_out is not None:
        x = (x + np.asarray(attn_out, np.float32)).astype(np.float32)
    h = x.shape[-1]
    mean = (x.astype(np.float64) ** 2).sum(-1, keepdims=True) / h
    scale = (1.0 / np.sqrt(mean.astype(np.float32) + np.float32(eps))).astype(np.float32)
    n = ((x * scale).astype(np.float32) * np.asarray(norm_w, np.float32)).astype(np.float32)
    return x, n


def kogarashi_forward(layer: KogarashiLayer, x: np.ndarray, n: np.ndarray, logits=None):
    """x float32 [T,H] residual stream, n float32 [T,H] normalised input.
    -> dict(logits, ids, prob, out) with out = x + sum_s p_s down_s + sigmoid(sg) shared
    (native.cu:113-117)."""
    t_n = n.shape[0]
    if logits is None:
        logits = kogarashi_logits(layer, n)
    ids, prob = R.route_kogarashi(logits, layer.topk)
    out = x.astype(np.float64).copy()
    cache = {}
    for t in range(t_n):
        xt = n[t].astype(np.float64)
        for s in range(layer.topk):
            e = int(ids[t, s])
            if e not in cache:
                cache[e] = (F.ggml_decode(layer.gate[e], layer.gate_ty, layer.hidden).astype(np.float64),
                            F.ggml_decode(layer.up[e], layer.up_ty, layer.hidden).astype(np.float64),
                            F.ggml_decode(layer.down[e], layer.down_ty, layer.inter).astype(np.float64))
            g, u, d = cache[e]
            ff = (_silu64(g @ xt) * (u @ xt)).astype(np.float32).astype(np.float64)
            out[t] += float(prob[t, s]) * (d @ ff)
    if layer.sh_gate is not None:
        g = F.ggml_decode(layer.sh_gate, layer.gate_ty, layer.hidden).astype(np.float64)
        u = F.ggml_decode(layer.sh_up, layer.up_ty, layer.hidden).astype(np.float64)
        d = F.ggml_decode(layer.sh_down, layer.down_ty, layer.inter).astype(np.float64)
        nt = n.astype(np.float64)
        ff = (_silu64(nt @ g.T) * (nt @ u.T)).astype(np.float32).astype(np.float64)
        sg = nt @ layer.sh_inp.astype(np.float64)
        out += (1.0 / (1.0 + np.exp(-sg)))[:, None] * (ff @ d.T)
    return dict(logits=logits, ids=ids, prob=prob, out=out.astype(np.float32))


# ----------------------------------------------------------------------------
# Tsumuji (qwen-next; decode/ops.cu:148-230, decode/gemv.cu:64-158)
# ----------------------------------------------------------------------------

@dataclass
class TsumujiLayer:
    hidden: int
    inter: int
    experts: int
    topk: int
    router: np.ndarray            # bf16-valued float32 [E+1,H]; row E = shared gate
    blocks: np.ndarray            # bytes [E, 27/16*F*H]
    gs: np.ndarray                # float32 [E,3]
    shared_gu: np.ndarray         # bf16-valued float32 [2F,H] (gate rows, then up rows)
    shared_down: np.ndarray       # bf16-valued float32 [H,F]


def tsumuji_logits(layer: TsumujiLayer, x: np.ndarray) -> np.ndarray:
    return (x.astype(np.float64) @ layer.router.astype(np.float64).T).astype(np.float32)


def tsumuji_forward(layer: TsumujiLayer, x: np.ndarray, logits=None, ids=None):
    """x float32 [N,H] -> dict(logits, ids, w, shared_gate, out float32 [N,H]);
    out = sum_s w_s y_s + shared_gate * y_shared (ops.cu:217-223, without the residual
    stream write-back)."""
    h, f, k = layer.hidden, layer.inter, layer.topk
    if logits is None:
        logits = tsumuji_logits(layer, x)
    sel, w, sgate = R.route_tsumuji(logits, layer.experts, k)
    if ids is None:
        ids = sel
    else:                                   # a given selection (near-tie resolved differently): its own weights
        ids = np.asarray(ids, np.int32)
        w = R.weights_for_ids(R.TSUMUJI, logits, ids, layer.experts)
    out = np.zeros((x.shape[0], h), np.float64)
    cache = {}
    for t in range(x.shape[0]):
        xt = x[t].astype(np.float64)
        for s in range(k):
            e = int(ids[t, s])
            if e not in cache:
                cache[e] = [m.astype(np.float64) for m in F.tsumuji_block_decode(layer.blocks[e], layer.gs[e], h, f)]
            g, u, d = cache[e]
            gs = layer.gs[e].astype(np.float64)
            hh = (_silu64((g @ xt) * gs[0]) * ((u @ xt) * gs[1])).astype(np.float32).astype(np.float64)
            out[t] += float(w[t, s]) * ((d @ hh) * gs[2])
    xs = x.astype(np.float64)
    g = xs @ layer.shared_gu[:f].astype(np.float64).T
    u = xs @ layer.shared_gu[f:].astype(np.float64).T
    hh = (_silu64(g) * u).astype(np.float32).astype(np.float64)
    out += sgate.astype(np.float64)[:, None] * (hh @ layer.shared_down.astype(np.float64).T)
    return dict(logits=logits, ids=ids, w=w, shared_gate=sgate, out=out.astype(np.float32))


# ----------------------------------------------------------------------------
# Hayate (GLM; cu/glm53/decode.cu:18-59, math.cuh:31-39, dense.cuh)
# ----------------------------------------------------------------------------

def hayate_swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """bf16(bf16(g' * sigmoid(g')) * u'), g' = min(g,10), u' = clamp(u,-10,10) (math.cuh:31-34)."""
    g = np.minimum(np.asarray(gate, np.float32), np.float32(10))
    u = np.clip(np.asarray(up, np.float32), np.float32(-10), np.float32(10))
    sig = (1.0 / (1.0 + np.exp(-g.astype(np.float64)))).astype(np.float32)
    return F.bf16_round((F.bf16_round((g * sig).astype(np.float32)) * u).astype(np.float32))


@dataclass
class HayateLayer:
    hidden: int
    inter: int
    experts: int
    topk: int
    scale: float
    router: np.ndarray            # bf16-valued float32 [E,H]
    bias: np.ndarray              # float32 [E]
    images: np.ndarray            # bytes [E, 3*stride] NVFP4 tiled gate | up | down
    stride: int
    shared: np.ndarray            # bytes [3*stride] same layout (rounded weights)


def hayate_logits(layer: HayateLayer, x: np.ndarray) -> np.ndarray:
    return (x.astype(np.float64) @ layer.router.astype(np.float64).T).astype(np.float32)


def _hayate_mats(img, stride, h, f, rounded):
    return (F.nvfp4_tiled_decode(img[0:], f, h, rounded=rounded).astype(np.float64),
            F.nvfp4_tiled_decode(img[stride:], f, h, rounded=rounded).astype(np.float64),
            F.nvfp4_tiled_decode(img[2 * stride:], h, f, rounded=rounded).astype(np.float64))


def hayate_forward(layer: HayateLayer, x: np.ndarray, logits=None, ids=None):
    """x bf16-valued float32 [T,H] -> dict(logits, ids, weights, out bf16-valued [T,H]).
    Routed experts: unrounded NVFP4 weights; shared expert: bf16-rounded weights
    (decode.cu:44-45,52). Products and expert outputs are rounded to bf16, experts are
    added in ascending expert id with a bf16 rounding after every add, the shared expert
    last and ungated (decode.cu:55-59)."""
    h, f, k = layer.hidden, layer.inter, layer.topk
    if logits is None:
        logits = hayate_logits(layer, x)
    sel, w = R.route_hayate(logits, layer.bias, k, layer.scale)
    if ids is None:
        ids = sel
    else:
        ids = np.asarray(ids, np.int32)
        w = R.weights_for_ids(R.HAYATE, logits, ids, layer.experts, layer.bias, layer.scale)
    out = np.zeros((x.shape[0], h), np.float32)
    cache = {}
    sg, su, sd = _hayate_mats(layer.shared, layer.stride, h, f, True)
    for t in range(x.shape[0]):
        xt = x[t].astype(np.float64)
        ys = []
        for s in range(k):
            e = int(ids[t, s])
            if e not in cache:
                cache[e] = _hayate_mats(layer.images[e], layer.stride, h, f, False)
            g, u, d = cache[e]
            p = hayate_swiglu(F.bf16_round((g @ xt).astype(np.float32)), F.bf16_round((u @ xt).astype(np.float32)))
            ys.append(F.bf16_round((d @ p.astype(np.float64)).astype(np.float32)))
        p = hayate_swiglu(F.bf16_round((sg @ xt).astype(np.float32)), F.bf16_round((su @ xt).astype(np.float32)))
        ysh = F.bf16_round((sd @ p.astype(np.float64)).astype(np.float32))
        acc = np.zeros(h, np.float32)
        for a in R.route_order(ids[t]):
            acc = F.bf16_round(acc + F.bf16_round((ys[a] * w[t, a]).astype(np.float32)))
        out[t] = F.bf16_round((acc + ysh).astype(np.float32))
    return dict(logits=logits, ids=ids, weights=w, out=out)


# ----------------------------------------------------------------------------
# FP8 prefill layer (block-FP8 weights, per token x 128 FP8 activations)
# ----------------------------------------------------------------------------

@dataclass
class Fp8Layer:
    hidden: int
    inter: int
    experts: int
    topk: int
    gate: list = field(default_factory=list)   # per expert (payload [F,H], scale [F/128,H/128])
    up: list = field(default_factory=list)
    down: list = field(default_factory=list)   # per expert (payload [H,F], scale [H/128,F/128])


def fp8_dequant_gemm(aq, a_scale, wq, w_scale):
    """sum over 128-wide K blocks of (A_blk @ W_blk^T) * a_scale[t,kb] * w_scale[nb,kb],
    e4m3 products summed in float64. aq [M,K] codes, wq [N,K] codes."""
    a = F.e4m3_decode(aq).astype(np.float64)
    w = F.e4m3_decode(wq).astype(np.float64)
    m, k = a.shape
    n = w.shape[0]
    out = np.zeros((m, n), np.float64)
    ws = np.repeat(w_scale.astype(np.float64), 128, 0)[:n]          # [N, K/128]
    for kb in range(k // 128):
        part = a[:, kb * 128:(kb + 1) * 128] @ w[:, kb * 128:(kb + 1) * 128].T
        out += part * a_scale[:, kb].astype(np.float64)[:, None] * ws[:, kb][None, :]
    return out


def fp8_forward(layer: Fp8Layer, x: np.ndarray, logits: np.ndarray):
    """x bf16-valued float32 [T,H], logits float32 [T,E] (softmax top-k, renormalised, as
    Kogarashi). Activations and the SwiGLU product (stored as bf16 between the two grouped
    products) are quantized to e4m3 with one float32 scale per token and 128 channels.
    -> dict(ids, prob, out float32 [T,H])."""
    ids, prob = R.route_kogarashi(logits, layer.topk)
    xq, xs = F.fp8_act_quantize(x)
    out = np.zeros((x.shape[0], layer.hidden), np.float64)
    assign, counts, offsets = R.permutation(ids, layer.experts, layer.topk)
    for e in range(layer.experts):
        if not counts[e]:
            continue
        a = assign[offsets[e]:offsets[e] + counts[e]]
        tok = a // layer.topk
        g = fp8_dequant_gemm(xq[tok], xs[tok], *layer.gate[e])
        u = fp8_dequant_gemm(xq[tok], xs[tok], *layer.up[e])
        hq, hs = F.fp8_act_quantize(F.bf16_round((_silu64(g) * u).astype(np.float32)))
        y = fp8_dequant_gemm(hq, hs, *layer.down[e]).astype(np.float32)
        np.add.at(out, tok, y.astype(np.float64) * prob.reshape(-1)[a].astype(np.float64)[:, None])
    return dict(ids=ids, prob=prob, out=out.astype(np.float32))
