"""Host-side mirror of the Tsumuji MoE half-layer call.

Reference: `Engine::mlp_half`, engines/tsumuji/crates/tsumuji-engine/src/engine.rs:1534-1685, with the
expert weights packed as `pack_experts` packs them (weights.rs:448-509: one block of 27/16*F*H bytes per
routed expert, `gs` [E][3]) and the buffers of engine.rs:382-387 (`rlogits`, `sel`, `rw`, `sgate`).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .formats import nvfp4_linear_expert_bytes


class TsumujiMoeLayer:
    def __init__(self, hidden: int, inter: int, experts: int, topk: int, max_tokens: int = 8, device="cuda"):
        self.hidden, self.inter, self.experts, self.topk, self.max_tokens = hidden, inter, experts, topk, max_tokens
        self.device = torch.device(device)
        lib = _lib.lib()
        nbytes = lib.tsumuji_moe_workspace_bytes(hidden, inter, experts, topk, max_tokens)
        self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        _lib.check(lib.tsumuji_moe_workspace_init(self.workspace.data_ptr(), nbytes, self._stream()), "workspace_init")
        self.rlogits = torch.empty(max_tokens, experts + 1, dtype=torch.float32, device=self.device)
        self.sel = torch.empty(max_tokens, topk, dtype=torch.int32, device=self.device)
        self.rw = torch.empty(max_tokens, topk, dtype=torch.float32, device=self.device)
        self.sgate = torch.empty(max_tokens, dtype=torch.float32, device=self.device)
        self.router = self.experts_w = self.gs = self.shared_gu = self.shared_down = None

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def load(self, router, experts_w, gs, shared_gu, shared_down) -> None:
        """router bf16 [E+1,H] (or None: logits come from the caller), experts_w uint8 [E, 27/16 F H],
        gs float32 [E,3], shared_gu bf16 [2F,H], shared_down bf16 [H,F]."""
        e, f, h = self.experts, self.inter, self.hidden
        if experts_w.dtype != torch.uint8 or experts_w.numel() != e * nvfp4_linear_expert_bytes(h, f):
            raise ValueError("experts_w: expected [E, 27/16*F*H] bytes")
        if tuple(gs.shape) != (e, 3) or tuple(shared_gu.shape) != (2 * f, h) or tuple(shared_down.shape) != (h, f):
            raise ValueError("gs / shared expert shapes")
        to = lambda t, dt: t.to(self.device, dt).contiguous()
        self.router = to(router, torch.bfloat16) if router is not None else None
        self.experts_w, self.gs = to(experts_w, torch.uint8), to(gs, torch.float32)
        self.shared_gu, self.shared_down = to(shared_gu, torch.bfloat16), to(shared_down, torch.bfloat16)

    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False, writeback=None) -> torch.Tensor:
        """x float32 [N,H] -> out float32 [N,H] = sum_s w_s y_s + shared_gate y_shared.
        writeback: optional dict(R float32 [N,HC,H] updated in place, di float32 [Sd,N,ld], rank int, ss float32
        [N, ceil(H/256), HC] written) -- the residual-stream part of the reference's `moe_combine`."""
        n = x.shape[0]
        if n > self.max_tokens or x.shape[1] != self.hidden or x.dtype != torch.float32 or not x.is_contiguous():
            raise ValueError("x must be contiguous float32 [N<=max_tokens, hidden]")
        if out is None:
            out = torch.empty_like(x)
        d = _lib.TsumujiMoe()
        d.hidden, d.inter, d.experts, d.topk, d.tokens = self.hidden, self.inter, self.experts, self.topk, n
        d.router_w = self.router.data_ptr() if self.router is not None else None
        d.experts_w, d.gs = self.experts_w.data_ptr(), self.gs.data_ptr()
        d.shared_gu, d.shared_down = self.shared_gu.data_ptr(), self.shared_down.data_ptr()
        d.x, d.out = x.data_ptr(), out.data_ptr()
        d.rlogits, d.sel, d.rw, d.shared_gate = (self.rlogits.data_ptr(), self.sel.data_ptr(), self.rw.data_ptr(),
                                                 self.sgate.data_ptr())
        d.accumulate = 1 if accumulate else 0
        if writeback is not None:
            r, di, ss = writeback["R"], writeback["di"], writeback["ss"]
            hc = r.shape[1]
            if r.dtype != torch.float32 or tuple(r.shape) != (n, hc, self.hidden) or not r.is_contiguous() or di.dtype != torch.float32 \
                    or di.shape[1] != n or not di.is_contiguous() or tuple(ss.shape) != (n, (self.hidden + 255) // 256, hc):
                raise ValueError("writeback: R [N,HC,H], di [Sd,N,ld], ss [N,ceil(H/256),HC], all float32")
            d.R, d.di, d.ss = r.data_ptr(), di.data_ptr(), ss.data_ptr()
            d.Sd, d.ld, d.rank, d.HC = di.shape[0], di.shape[2], int(writeback["rank"]), hc
        d.workspace, d.workspace_bytes = self.workspace.data_ptr(), self.workspace.numel()
        _lib.check(_lib.lib().tsumuji_moe_layer(ctypes.byref(d), self._stream()), "tsumuji_moe_layer")
        return out
