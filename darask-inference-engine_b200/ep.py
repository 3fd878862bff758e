"""Expert-parallel FP8 prefill MoE layer: one process per GPU, experts sharded in contiguous blocks, tokens
data-parallel, two all-to-all-v exchanges per layer over `torch.distributed` (NCCL on GPUs).

Rank g of G holds experts [g*E/G, (g+1)*E/G).  Every rank routes its own tokens, sorts the routed rows by expert (which
also groups them by destination rank), exchanges the per-expert row counts, sends the FP8 rows and their scales,
runs the grouped products over what it received, sends the float32 rows back and combines them with the routing
weights.  The reference engines have no multi-GPU path; their single-GPU orchestration is `prefill_experts`,
engines/hayate/crates/models/src/glm53/gpu.rs:2068-2566.

`ep_forward` is the device-agnostic orchestration (split sizes, exchanges); the kernels sit behind a backend object.
`CudaFp8Backend` is the product backend (C ABI calls); the tests drive `ep_forward` with a CPU backend under gloo.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib


def exchange_counts(counts: torch.Tensor, group=None):
    """counts int32 [G, E/G] (rows this rank sends to each rank's experts) -> (recv_counts [G, E/G], send_splits,
    recv_splits).  One all-to-all of G*E/G integers and one device->host copy."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        recv = counts.clone()
    else:
        recv = torch.empty_like(counts)
        dist.all_to_all_single(recv, counts.contiguous(), group=group)
    both = torch.stack([counts.sum(1), recv.sum(1)]).cpu()
    return recv, [int(v) for v in both[0]], [int(v) for v in both[1]]


def all_to_all_rows(send: torch.Tensor, send_splits, recv_splits, group=None, pad_rows: int = 0, out=None) -> torch.Tensor:
    """Rows of `send` (first sum(send_splits) rows) to the ranks as split; returns sum(recv_splits) (+ pad_rows) rows
    (the pad rows are uninitialised: the grouped GEMM loads them as part of its last tile and discards the result).
    `out`: optional preallocated buffer with at least that many rows."""
    n_recv = sum(recv_splits)
    if out is None or out.shape[0] < n_recv + pad_rows:
        out = torch.empty((n_recv + pad_rows,) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
    else:
        out = out[:n_recv + pad_rows]
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    n_send = sum(send_splits)
    if world == 1:
        out[:n_recv] = send[:n_send]
    else:
        dist.all_to_all_single(out[:n_recv], send[:n_send], recv_splits, send_splits, group=group)
    return out


def ep_forward(backend, *inputs, group=None, marks=None):
    """One expert-parallel layer call on this rank's tokens; returns (out, info).

    backend.dispatch(*inputs) -> dict with `send` (list of row tensors in ascending expert order), `ranges` [E, 2];
    backend.run_experts(recv_counts, received list, n_recv) -> rows [n_recv, H] in received order;
    backend.combine(rows back in dispatch order, dispatch dict) -> out."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    mark = (lambda name: marks.append((name, _event()))) if marks is not None else (lambda name: None)
    mark("start")
    d = backend.dispatch(*inputs)                                     # rows in ascending expert order
    mark("dispatch")
    counts = d["ranges"][:, 0].to(torch.int32).reshape(world, -1)
    recv_counts, send_splits, recv_splits = exchange_counts(counts, group)
    mark("counts")
    bufs = getattr(backend, "buffers", {})
    received = [all_to_all_rows(t, send_splits, recv_splits, group, pad_rows=backend.pad_rows, out=bufs.get(f"recv{i}"))
                for i, t in enumerate(d["send"])]
    mark("a2a_out")
    n_recv = sum(recv_splits)
    y_recv = backend.run_experts(recv_counts, received, n_recv)       # [n_recv, H] in received order
    mark("experts")
    y_home = all_to_all_rows(y_recv, recv_splits, send_splits, group, out=bufs.get("y_home"))
    mark("a2a_back")
    out = backend.combine(y_home, d)
    mark("combine")
    return out, dict(ids=d["ids"], prob=d["prob"], send_rows=sum(send_splits), recv_rows=n_recv,
                     cross_rows=sum(send_splits) - send_splits[dist.get_rank(group) if world > 1 else 0])


def all_to_all_equal(send: torch.Tensor, group=None, out=None) -> torch.Tensor:
    """Equal-split all-to-all: `send` is [G, ...], slice r goes to rank r; returns [G, ...] with slice r from rank r."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return send
    out = torch.empty_like(send) if out is None else out
    dist.all_to_all_single(out, send.contiguous(), group=group)
    return out


def ep_forward_packed(backend, *inputs, group=None, marks=None):
    """One expert-parallel layer call whose exchanges need no sizes on the host: fixed-capacity slabs of packed rows out,
    rows pre-reduced per (token, expert rank) back, no device->host copy between the launches.

    backend.dispatch_packed(*inputs) -> dict with `send` [G, cap, row bytes], `counts` int32 [G, E/G];
    backend.run_experts_packed(recv_counts [G, E/G], recv [G, cap, row bytes]) -> z [G, tcap, H] (slice s: partial rows for
    rank s's tokens); backend.sum_packed(zr [G, tcap, H], dispatch dict) -> out."""
    mark = (lambda name: marks.append((name, _event()))) if marks is not None else (lambda name: None)
    bufs = getattr(backend, "buffers", {})
    mark("start")
    d = backend.dispatch_packed(*inputs)
    mark("dispatch")
    recv_counts = all_to_all_equal(d["counts"], group, out=bufs.get("recv_counts"))
    mark("counts")
    recv = all_to_all_equal(d["send"], group, out=bufs.get("recv_slabs"))
    mark("a2a_out")
    z = backend.run_experts_packed(recv_counts, recv)
    mark("experts")
    zr = all_to_all_equal(z, group, out=bufs.get("zr"))
    mark("a2a_back")
    out = backend.sum_packed(zr, d)
    mark("combine")
    return out, dict(ids=d["ids"], prob=d["prob"], recv_counts=recv_counts, send_counts=d["counts"])


def _event():
    e = torch.cuda.Event(enable_timing=True)
    e.record()
    return e


def stage_times(forward, group=None, calls: int = 5):
    """Microseconds per stage of `ep_forward` on the device (CUDA events on the launching stream, mean over `calls`,
    then the maximum over the ranks), plus the host wall time of a whole call. `forward(marks)` makes one layer call."""
    import time
    forward(None)
    torch.cuda.synchronize()
    acc, wall = {}, 0.0
    for _ in range(calls):
        marks = []
        t0 = time.perf_counter()
        forward(marks)
        torch.cuda.synchronize()
        wall += time.perf_counter() - t0
        for (_, a), (name, b) in zip(marks[:-1], marks[1:]):
            acc[name] = acc.get(name, 0.0) + a.elapsed_time(b) * 1e3
    names = list(acc)
    vals = torch.tensor([acc[n] / calls for n in names] + [wall / calls * 1e6], dtype=torch.float64, device="cuda")
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX, group=group)
    out = {n: round(float(v), 1) for n, v in zip(names, vals[:-1])}
    out["host_wall"] = round(float(vals[-1]), 1)
    return out


class CudaFp8Backend:
    """Kernels of one rank: block-FP8 weights of its E/G experts resident on the GPU."""
    pad_rows = 128          # the grouped GEMM loads whole 128-row tiles

    def __init__(self, hidden, inter, experts, topk, world, max_tokens, device="cuda", capacity_factor=None):
        if experts % world:
            raise ValueError("experts must divide evenly over the ranks")
        self.hidden, self.inter, self.experts, self.topk, self.world = hidden, inter, experts, topk, world
        self.capacity_factor = capacity_factor
        self.local = experts // world
        self.max_tokens, self.device = max_tokens, torch.device(device)
        lib = _lib.lib()
        self.scratch = torch.zeros(lib.darask_fp8_ep_dispatch_scratch_bytes(hidden, experts, topk, max_tokens), dtype=torch.uint8,
                                   device=self.device)
        rows = max_tokens * topk + self.pad_rows
        self.send_codes = torch.zeros(rows, hidden, dtype=torch.uint8, device=self.device)
        self.send_scales = torch.zeros(rows, hidden // 128, dtype=torch.float32, device=self.device)
        self.ranges = torch.zeros(experts, 2, dtype=torch.int32, device=self.device)
        self.position = torch.zeros(max_tokens * topk, dtype=torch.int32, device=self.device)
        self.ids = torch.zeros(max_tokens, topk, dtype=torch.int32, device=self.device)
        self.prob = torch.zeros(max_tokens, topk, dtype=torch.float32, device=self.device)
        self.seg = torch.zeros(world * self.local * 2, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.w = {}
        # receive-side buffers, kept between calls; `capacity` rows (default: twice the mean load) grow on demand
        self.capacity = 0
        self.buffers = {}
        self._reserve(2 * max_tokens * topk)
        self.buffers["y_home"] = torch.empty(max_tokens * topk, hidden, dtype=torch.float32, device=self.device)
        self.packed_ready = False

    def _reserve_packed(self):
        """Buffers of the exchange without host-side sizes: a slab holds a rank's worst case, max_tokens * topk rows."""
        if self.packed_ready:
            return
        dev, g = self.device, self.world
        # rows per (source, destination) slab: the worst case, or capacity_factor x the mean load (rows beyond it are
        # dropped and reported in the status word)
        worst = self.max_tokens * self.topk
        self.cap = worst if self.capacity_factor is None else max(1, min(worst, int(-(-worst * self.capacity_factor // g))))
        self.row_bytes = _lib.lib().darask_fp8_ep_packed_row_bytes(self.hidden)
        rows = g * self.cap
        self._reserve(rows)
        self.send_slabs = torch.zeros(g, self.cap, self.row_bytes, dtype=torch.uint8, device=dev)
        self.send_counts = torch.zeros(g, self.local, dtype=torch.int32, device=dev)
        self.buffers["recv_slabs"] = torch.zeros(g, self.cap, self.row_bytes, dtype=torch.uint8, device=dev)
        self.buffers["recv_counts"] = torch.zeros(g, self.local, dtype=torch.int32, device=dev)
        self.buffers["zr"] = torch.empty(g, self.max_tokens, self.hidden, dtype=torch.float32, device=dev)
        self.z = torch.empty(g, self.max_tokens, self.hidden, dtype=torch.float32, device=dev)
        self.meta_src = torch.zeros(rows, dtype=torch.int32, device=dev)
        self.meta_tok = torch.zeros(rows, dtype=torch.int32, device=dev)
        self.meta_prob = torch.zeros(rows, dtype=torch.float32, device=dev)
        self.count = torch.zeros(g * self.max_tokens, dtype=torch.int32, device=dev)
        self.list = torch.zeros(g * self.max_tokens * self.topk, dtype=torch.int32, device=dev)
        self.packed_ready = True

    def dispatch_packed(self, x, logits):
        t = x.shape[0]
        if t > self.max_tokens or x.dtype != torch.bfloat16 or logits.dtype != torch.float32 or not x.is_contiguous() or not logits.is_contiguous():
            raise ValueError("x must be contiguous bf16 [T<=max_tokens,H], logits contiguous float32 [T,E]")
        self._reserve_packed()
        _lib.check(_lib.lib().darask_fp8_ep_dispatch_packed(
            x.data_ptr(), logits.data_ptr(), self.hidden, self.experts, self.topk, t, self.world, self.cap, self.ids.data_ptr(),
            self.prob.data_ptr(), self.send_slabs.data_ptr(), self.send_counts.data_ptr(), self.ranges.data_ptr(), self.position.data_ptr(),
            self.status.data_ptr(), self.scratch.data_ptr(), self.scratch.numel(), self._stream()), "darask_fp8_ep_dispatch_packed")
        return dict(send=self.send_slabs, counts=self.send_counts, ids=self.ids[:t], prob=self.prob[:t], tokens=t)

    def run_experts_packed(self, recv_counts, recv):
        lib = _lib.lib()
        (gw, gs), (uw, us), (dw, ds) = self.w["gate"], self.w["up"], self.w["down"]
        rows = self.world * self.cap
        _lib.check(lib.darask_fp8_ep_regroup_packed(
            recv_counts.data_ptr(), self.world, self.local, recv.data_ptr(), self.cap, self.hidden, self.codes.data_ptr(),
            self.scales.data_ptr(), self.local_ranges.data_ptr(), self.row_map.data_ptr(), self.meta_src.data_ptr(), self.meta_tok.data_ptr(),
            self.meta_prob.data_ptr(), self.seg.data_ptr(), self.seg.numel() * 4, self._stream()), "darask_fp8_ep_regroup_packed")
        _lib.check(lib.darask_fp8_ep_experts(
            self.codes.data_ptr(), self.scales.data_ptr(), rows + self.pad_rows, self.local_ranges.data_ptr(), self.local, self.hidden,
            self.inter, gw.data_ptr(), uw.data_ptr(), dw.data_ptr(), gs.data_ptr(), us.data_ptr(), ds.data_ptr(), None, self.y.data_ptr(),
            self.prod.data_ptr(), self.prod_s.data_ptr(), self.status.data_ptr(), self._stream()), "darask_fp8_ep_experts")
        _lib.check(lib.darask_fp8_ep_reduce(
            self.y.data_ptr(), self.local_ranges.data_ptr(), self.local, self.meta_src.data_ptr(), self.meta_tok.data_ptr(),
            self.meta_prob.data_ptr(), self.world, self.cap, self.max_tokens, self.topk, self.hidden, self.z.data_ptr(), self.count.data_ptr(),
            self.list.data_ptr(), self.status.data_ptr(), self._stream()), "darask_fp8_ep_reduce")
        return self.z

    def sum_packed(self, zr, d):
        t = d["tokens"]
        out = torch.empty(t, self.hidden, dtype=torch.float32, device=self.device)
        _lib.check(_lib.lib().darask_fp8_ep_sum(out.data_ptr(), zr.data_ptr(), self.world, t, self.max_tokens, self.hidden, self._stream()),
                   "darask_fp8_ep_sum")
        return out

    def _reserve(self, rows):
        if rows <= self.capacity:
            return
        dev, alloc = self.device, rows + self.pad_rows
        self.capacity = rows
        self.buffers["recv0"] = torch.empty(alloc, self.hidden, dtype=torch.uint8, device=dev)
        self.buffers["recv1"] = torch.empty(alloc, self.hidden // 128, dtype=torch.float32, device=dev)
        self.codes = torch.empty(alloc, self.hidden, dtype=torch.uint8, device=dev)
        self.scales = torch.empty(alloc, self.hidden // 128, dtype=torch.float32, device=dev)
        self.prod = torch.empty(alloc, self.inter, dtype=torch.uint8, device=dev)
        self.prod_s = torch.empty(alloc, self.inter // 128, dtype=torch.float32, device=dev)
        self.y = torch.empty(rows, self.hidden, dtype=torch.float32, device=dev)
        self.row_map = torch.empty(rows, dtype=torch.int32, device=dev)
        self.local_ranges = torch.empty(self.local, 2, dtype=torch.int32, device=dev)

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def load(self, name: str, payload: torch.Tensor, scales: torch.Tensor) -> None:
        """This rank's experts: payload uint8 [E/G, n, k], scales float32 [E/G, n/128, k/128]; name in gate|up|down."""
        n, k = (self.hidden, self.inter) if name == "down" else (self.inter, self.hidden)
        if tuple(payload.shape) != (self.local, n, k) or tuple(scales.shape) != (self.local, n // 128, k // 128):
            raise ValueError(f"{name}: expected payload [{self.local},{n},{k}] and scales [{self.local},{n // 128},{k // 128}]")
        self.w[name] = (payload.to(self.device, torch.uint8).contiguous(), scales.to(self.device, torch.float32).contiguous())

    def dispatch(self, x, logits):
        t = x.shape[0]
        if t > self.max_tokens or x.dtype != torch.bfloat16 or logits.dtype != torch.float32 or not x.is_contiguous() or not logits.is_contiguous():
            raise ValueError("x must be contiguous bf16 [T<=max_tokens,H], logits contiguous float32 [T,E]")
        _lib.check(_lib.lib().darask_fp8_ep_dispatch(
            x.data_ptr(), logits.data_ptr(), self.hidden, self.experts, self.topk, t, self.ids.data_ptr(), self.prob.data_ptr(),
            self.send_codes.data_ptr(), self.send_scales.data_ptr(), self.ranges.data_ptr(), self.position.data_ptr(),
            self.scratch.data_ptr(), self.scratch.numel(), self._stream()), "darask_fp8_ep_dispatch")
        return dict(send=[self.send_codes, self.send_scales], ranges=self.ranges, position=self.position, ids=self.ids[:t],
                    prob=self.prob[:t], tokens=t)

    def run_experts(self, recv_counts, received, n_recv):
        recv_codes, recv_scales = received
        lib = _lib.lib()
        if n_recv == 0:
            return self.y[:0]
        self._reserve(n_recv)            # no-op unless this call received more rows than any before
        rows = n_recv + self.pad_rows
        (gw, gs), (uw, us), (dw, ds) = self.w["gate"], self.w["up"], self.w["down"]
        ranges, y = self.local_ranges, self.y[:n_recv]
        if self.world == 1:
            # one rank: the received order already is the expert order
            codes, scales = recv_codes, recv_scales
            ranges.copy_(self._ranges_from_counts(recv_counts))
            row_map_ptr = None
        else:
            codes, scales = self.codes, self.scales
            _lib.check(lib.darask_fp8_ep_regroup(
                recv_counts.data_ptr(), self.world, self.local, recv_codes.data_ptr(), recv_scales.data_ptr(), self.hidden, n_recv,
                codes.data_ptr(), scales.data_ptr(), ranges.data_ptr(), self.row_map.data_ptr(), self.seg.data_ptr(), self.seg.numel() * 4,
                self._stream()), "darask_fp8_ep_regroup")
            row_map_ptr = self.row_map.data_ptr()
        _lib.check(lib.darask_fp8_ep_experts(
            codes.data_ptr(), scales.data_ptr(), rows, ranges.data_ptr(), self.local, self.hidden, self.inter, gw.data_ptr(),
            uw.data_ptr(), dw.data_ptr(), gs.data_ptr(), us.data_ptr(), ds.data_ptr(), row_map_ptr, y.data_ptr(), self.prod.data_ptr(),
            self.prod_s.data_ptr(), self.status.data_ptr(), self._stream()), "darask_fp8_ep_experts")
        return y

    @staticmethod
    def _ranges_from_counts(counts):
        c = counts.reshape(-1).to(torch.int32)
        off = torch.cumsum(c, 0, dtype=torch.int32) - c
        return torch.stack([c, off], 1)

    def combine(self, y_home, d):
        t = d["tokens"]
        out = torch.empty(t, self.hidden, dtype=torch.float32, device=self.device)
        _lib.check(_lib.lib().darask_fp8_ep_combine(out.data_ptr(), y_home.data_ptr(), d["prob"].data_ptr(), d["position"].data_ptr(), t,
                                                    self.hidden, self.topk, self._stream()), "darask_fp8_ep_combine")
        return out

    def device_status(self) -> int:
        return int(self.status.item())


class Fp8ExpertParallelMoe:
    """The call a user makes: `forward(x, logits)` on every rank with that rank's tokens."""

    def __init__(self, hidden, inter, experts, topk, max_tokens, group=None, device="cuda", exchange="packed", capacity_factor=None):
        """exchange = "packed": fixed-capacity slabs out, rows pre-reduced per (token, expert rank) back, no host
        synchronisation inside a call (every rank passes the same max_tokens); "exact": all-to-all-v of exactly the
        routed rows with the split sizes read on the host, float32 rows back, combined in slot order.
        capacity_factor (packed): rows a (source, destination) slab holds, as a multiple of the mean load tokens*topk/G;
        None = the worst case tokens*topk. Rows that do not fit are dropped and `backend.device_status()` has bit 16."""
        if exchange not in ("packed", "exact"):
            raise ValueError("exchange")
        self.group, self.exchange = group, exchange
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.backend = CudaFp8Backend(hidden, inter, experts, topk, world, max_tokens, device, capacity_factor)
        self.first_expert = self.rank * self.backend.local

    def load(self, name, payload, scales):
        self.backend.load(name, payload, scales)

    def _call(self, x, logits, marks=None):
        fn = ep_forward_packed if self.exchange == "packed" else ep_forward
        return fn(self.backend, x, logits, group=self.group, marks=marks)

    def forward(self, x, logits):
        out, self.info = self._call(x, logits)
        return out

    def rows(self):
        """(rows sent, rows received, rows sent to other ranks) of the last call; reads device counters (synchronizes)."""
        if "send_rows" in self.info:
            return self.info["send_rows"], self.info["recv_rows"], self.info["cross_rows"]
        sent = self.info["send_counts"].sum(1).cpu()
        return int(sent.sum()), int(self.info["recv_counts"].sum().item()), int(sent.sum() - sent[self.rank])

    def stage_times(self, x, logits):
        return stage_times(lambda marks: self._call(x, logits, marks), self.group)


class CudaTsumujiBackend:
    """Kernels of one rank of the Tsumuji (NVFP4, Qwen-Next-shaped) layer: its E/G packed expert blocks, the router and
    the shared expert replicated.  Reference single-GPU call site: tsumuji-engine/src/engine.rs:1586-1683."""
    pad_rows = 0

    def __init__(self, hidden, inter, experts, topk, world, max_tokens, device="cuda"):
        if experts % world:
            raise ValueError("experts must divide evenly over the ranks")
        self.hidden, self.inter, self.experts, self.topk, self.world = hidden, inter, experts, topk, world
        self.local, self.max_tokens, self.device = experts // world, max_tokens, torch.device(device)
        lib, dev = _lib.lib(), self.device
        self.workspace = torch.zeros(lib.tsumuji_moe_workspace_bytes(hidden, inter, experts, topk, max_tokens), dtype=torch.uint8, device=dev)
        self.rlogits = torch.zeros(max_tokens, experts + 1, dtype=torch.float32, device=dev)
        self.sel = torch.zeros(max_tokens, topk, dtype=torch.int32, device=dev)
        self.rw = torch.zeros(max_tokens, topk, dtype=torch.float32, device=dev)
        self.sgate = torch.zeros(max_tokens, dtype=torch.float32, device=dev)
        self.send_x = torch.empty(max_tokens * topk, hidden, dtype=torch.float32, device=dev)
        self.ranges = torch.zeros(experts, 2, dtype=torch.int32, device=dev)
        self.position = torch.zeros(max_tokens * topk, dtype=torch.int32, device=dev)
        self.y_shared = torch.empty(max_tokens, hidden, dtype=torch.float32, device=dev)
        self.buffers = {"y_home": torch.empty(max_tokens * topk, hidden, dtype=torch.float32, device=dev)}
        self.capacity = 0
        self._reserve(2 * max_tokens * topk)

    def _reserve(self, rows):
        if rows <= self.capacity:
            return
        self.capacity = rows
        self.buffers["recv0"] = torch.empty(rows, self.hidden, dtype=torch.float32, device=self.device)
        self.y = torch.empty(rows, self.hidden, dtype=torch.float32, device=self.device)
        nbytes = _lib.lib().tsumuji_ep_experts_workspace_bytes(self.hidden, self.inter, self.local, rows)
        self.expert_ws = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def load(self, router, blocks, gs, shared_gu, shared_down):
        """router bf16 [E+1,H] (replicated), blocks uint8 [E/G * 27/16 F H] and gs float32 [E/G,3] (this rank's experts),
        shared_gu bf16 [2F,H], shared_down bf16 [H,F] (replicated)."""
        dev = self.device
        self.router = router.to(dev, torch.bfloat16).contiguous()
        self.blocks = blocks.to(dev, torch.uint8).contiguous()
        self.gs = gs.to(dev, torch.float32).contiguous()
        self.shared_gu = shared_gu.to(dev, torch.bfloat16).contiguous()
        self.shared_down = shared_down.to(dev, torch.bfloat16).contiguous()
        if self.blocks.numel() != self.local * self.hidden * self.inter * 27 // 16 or tuple(self.gs.shape) != (self.local, 3):
            raise ValueError("blocks / gs: expected this rank's E/G experts")

    def dispatch(self, x):
        n = x.shape[0]
        if n > self.max_tokens or x.dtype != torch.float32 or not x.is_contiguous():
            raise ValueError("x must be contiguous float32 [N<=max_tokens,H]")
        d = _lib.TsumujiMoe()
        d.hidden, d.inter, d.experts, d.topk, d.tokens = self.hidden, self.inter, self.experts, self.topk, n
        d.router_w, d.shared_gu, d.shared_down = self.router.data_ptr(), self.shared_gu.data_ptr(), self.shared_down.data_ptr()
        d.x, d.rlogits, d.sel, d.rw, d.shared_gate = x.data_ptr(), self.rlogits.data_ptr(), self.sel.data_ptr(), self.rw.data_ptr(), self.sgate.data_ptr()
        d.workspace, d.workspace_bytes = self.workspace.data_ptr(), self.workspace.numel()
        _lib.check(_lib.lib().tsumuji_ep_dispatch(ctypes.byref(d), self.send_x.data_ptr(), self.ranges.data_ptr(), self.position.data_ptr(),
                                                  self.y_shared.data_ptr(), self._stream()), "tsumuji_ep_dispatch")
        return dict(send=[self.send_x], ranges=self.ranges, position=self.position, ids=self.sel[:n], prob=self.rw[:n], tokens=n)

    def run_experts(self, recv_counts, received, n_recv):
        if n_recv == 0:
            return self.y[:0]
        self._reserve(n_recv)
        x_rows, y = received[0], self.y[:n_recv]
        _lib.check(_lib.lib().tsumuji_ep_experts(
            self.blocks.data_ptr(), self.gs.data_ptr(), self.hidden, self.inter, self.local, self.world, recv_counts.data_ptr(),
            x_rows.data_ptr(), n_recv, y.data_ptr(), self.expert_ws.data_ptr(), self.expert_ws.numel(), self._stream()),
            "tsumuji_ep_experts")
        return y

    def combine(self, y_home, d):
        n = d["tokens"]
        out = torch.empty(n, self.hidden, dtype=torch.float32, device=self.device)
        _lib.check(_lib.lib().tsumuji_ep_combine(out.data_ptr(), y_home.data_ptr(), self.rw.data_ptr(), self.position.data_ptr(),
                                                 self.sgate.data_ptr(), self.y_shared.data_ptr(), n, self.hidden, self.topk, 0,
                                                 self._stream()), "tsumuji_ep_combine")
        return out


class TsumujiExpertParallelMoe:
    """`forward(x)` on every rank with that rank's float32 token rows."""

    def __init__(self, hidden, inter, experts, topk, max_tokens, group=None, device="cuda"):
        self.group = group
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.backend = CudaTsumujiBackend(hidden, inter, experts, topk, world, max_tokens, device)

    def load(self, *weights):
        self.backend.load(*weights)

    def forward(self, x):
        out, self.info = ep_forward(self.backend, x, group=self.group)
        return out
