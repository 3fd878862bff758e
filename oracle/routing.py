"""Router definitions of the three executors and the dispatch permutation (numpy).

Test infrastructure only.  Selection (ids and their order) is computed with the same
float32 keys and the same tie rule as the reference kernels so that it can be compared
bit for bit; gate weights are float32 values that fall under the output tolerance.
"""
from __future__ import annotations

import numpy as np

KOGARASHI, TSUMUJI, HAYATE = 0, 1, 2


def _f32(x):
    return np.asarray(x, np.float32)


def _exp32(x):
    return np.exp(_f32(x).astype(np.float64)).astype(np.float32)


def _sigmoid32(x):
    """1/(1+exp(-x)) in float32 steps (kogarashi native.cu:18, tsumuji decode.cuh:23,
    hayate math.cuh:13)."""
    e = _exp32(-_f32(x))
    return (np.float32(1) / (np.float32(1) + e)).astype(np.float32)


def _argmax_rounds(key: np.ndarray, k: int):
    """k rounds of arg-max, value descending, ties to the lower index."""
    key = key.astype(np.float32).copy()
    ids = np.empty(k, np.int32)
    vals = np.empty(k, np.float32)
    for s in range(k):
        i = int(np.argmax(key))            # numpy returns the first maximum
        ids[s], vals[s] = i, key[i]
        key[i] = -np.inf
    return ids, vals


def route_kogarashi(logits: np.ndarray, k: int = 8):
    """top-k by raw logit, then softmax over the k selected (native.cu:100-112).
    logits float32 [T,E] -> ids int32 [T,k] (selection order), prob float32 [T,k]."""
    logits = np.atleast_2d(_f32(logits))
    ids = np.empty((logits.shape[0], k), np.int32)
    prob = np.empty((logits.shape[0], k), np.float32)
    for t, row in enumerate(logits):
        i, v = _argmax_rounds(row, k)
        z = _exp32(v - v[0])
        ids[t], prob[t] = i, (z / z.astype(np.float64).sum().astype(np.float32)).astype(np.float32)
    return ids, prob


def route_tsumuji(logits: np.ndarray, experts: int, k: int):
    """softmax over E, top-k keyed on exp(logit - max) in float32, w = p / sum of selected p;
    shared gate = sigmoid(logits[E]) (tsumuji decode/ops.cu:148-200).
    logits float32 [T,E+1] -> ids [T,k], w [T,k], shared_gate [T]."""
    logits = np.atleast_2d(_f32(logits))
    t_n = logits.shape[0]
    ids = np.empty((t_n, k), np.int32)
    w = np.empty((t_n, k), np.float32)
    for t in range(t_n):
        row = logits[t, :experts]
        key = _exp32(row - row.max())
        s = np.float32(key.astype(np.float64).sum())
        i, v = _argmax_rounds(key, k)
        p = (v / s).astype(np.float32)
        ids[t], w[t] = i, (p / np.float32(p.astype(np.float64).sum())).astype(np.float32)
    return ids, w, _sigmoid32(logits[:, experts])


def route_hayate(logits: np.ndarray, bias: np.ndarray, k: int = 8, scale: float = 2.5):
    """score = sigmoid(logit); select by score + bias (strict >, lowest id on ties);
    w = score / (sum + 1e-20) * scale (hayate cu/glm53/ops.cu:100-114, decode.cu:23-31)."""
    logits = np.atleast_2d(_f32(logits))
    score = _sigmoid32(logits)
    choice = (score + _f32(bias)[None, :]).astype(np.float32)
    ids = np.empty((logits.shape[0], k), np.int32)
    w = np.empty((logits.shape[0], k), np.float32)
    for t in range(logits.shape[0]):
        i, _ = _argmax_rounds(choice[t], k)
        sel = score[t, i]
        total = np.float32(0)
        for v in sel:                       # the kernel sums in selection order
            total = np.float32(total + v)
        ids[t] = i
        w[t] = ((sel / np.float32(total + np.float32(1e-20))).astype(np.float32) * np.float32(scale)).astype(np.float32)
    return ids, w


def weights_for_ids(mode: int, logits: np.ndarray, ids: np.ndarray, experts: int, bias=None, scale: float = 1.0):
    """Gate weights of a GIVEN selection (ids [T,k], selection order), formed as each router forms them. Used when a
    device resolved a near-tie of two selection keys differently from numpy: the outputs are then compared on the
    device's own selection."""
    logits = np.atleast_2d(_f32(logits))
    ids = np.atleast_2d(np.asarray(ids, np.int64))
    w = np.empty(ids.shape, np.float32)
    for t in range(ids.shape[0]):
        row = logits[t, :experts]
        if mode == KOGARASHI:
            v = row[ids[t]]
            z = _exp32(v - v[0])
            w[t] = (z / z.astype(np.float64).sum().astype(np.float32)).astype(np.float32)
        elif mode == TSUMUJI:
            key = _exp32(row - row.max())
            p = (key[ids[t]] / np.float32(key.astype(np.float64).sum())).astype(np.float32)
            w[t] = (p / np.float32(p.astype(np.float64).sum())).astype(np.float32)
        else:
            sel = _sigmoid32(row)[ids[t]]
            total = np.float32(0)
            for v in sel:
                total = np.float32(total + v)
            w[t] = ((sel / np.float32(total + np.float32(1e-20))).astype(np.float32) * np.float32(scale)).astype(np.float32)
    return w


def selection_keys(mode: int, logits: np.ndarray, experts: int, bias=None) -> np.ndarray:
    """The float32 keys each router sorts by, as the oracle forms them."""
    logits = np.atleast_2d(_f32(logits))[:, :experts]
    if mode == KOGARASHI:
        return logits
    if mode == TSUMUJI:
        return _exp32(logits - logits.max(-1, keepdims=True))
    return (_sigmoid32(logits) + _f32(bias)[None, :]).astype(np.float32)


def groups(ids: np.ndarray, experts: int, k: int):
    """Dispatch permutation (hayate models/src/glm53/prefill.rs:12-26): assignment index
    a = token*k + slot; groups[e] lists every a whose expert is e, ascending.
    Rejects an empty or ragged id list, ids >= experts and duplicates within a token."""
    flat = np.asarray(ids).reshape(-1)
    if flat.size == 0 or flat.size % k:
        raise ValueError("route count")
    out = [[] for _ in range(experts)]
    for token, row in enumerate(flat.reshape(-1, k)):
        for j, e in enumerate(row):
            if e < 0 or e >= experts or e in row[:j]:
                raise ValueError("invalid/duplicate expert route")
            out[int(e)].append(token * k + j)
    return out


def permutation(ids: np.ndarray, experts: int, k: int):
    """-> (assignments uint32 [T*k] = concatenation of groups in ascending expert id,
    counts uint32 [E], offsets uint32 [E] (exclusive prefix sum)). gpu.rs:29-80,2300-2305."""
    g = groups(ids, experts, k)
    counts = np.array([len(x) for x in g], np.uint32)
    offsets = np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.uint32)
    assignments = np.array([a for x in g for a in x], np.uint32)
    return assignments, counts, offsets


def route_order(ids) -> np.ndarray:
    """Stable insertion sort of slot indices by expert id (hayate math.cuh:35-38)."""
    ids = list(ids)
    order = list(range(len(ids)))
    for i in range(1, len(ids)):
        v, j = order[i], i
        while j and ids[order[j - 1]] > ids[v]:
            order[j] = order[j - 1]
            j -= 1
        order[j] = v
    return np.array(order, np.int32)
