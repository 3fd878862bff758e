"""Host-side mirror of the Kogarashi MoE layer call.

Reference: `Engine::record`, engines/kogarashi/crates/kogarashi-engine/src/engine.rs:530-632,
with weights held as in `struct Weight {data, ty, k, rows, ne}` (engine.rs:13-19, upload at
:73-107) and the activation buffers of engine.rs:128-139 ("n", "x", "router", "ids", "prob").
The twelve launches of the reference become one call of `kogarashi_moe_layer`.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib
from .formats import GGML_Q6_K, ggml_tensor_bytes

TENSORS = ("ffn_gate_inp.weight", "ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight",
           "ffn_gate_shexp.weight", "ffn_up_shexp.weight", "ffn_down_shexp.weight", "ffn_gate_inp_shexp.weight")


@dataclass
class Weight:
    data: torch.Tensor      # uint8, device
    ty: int
    k: int
    rows: int
    ne: tuple


class KogarashiMoeLayer:
    """One layer's MoE FFN: weights resident on one GPU, buffers sized for `max_tokens`."""

    def __init__(self, hidden: int, inter: int, experts: int, topk: int, max_tokens: int = 1, device="cuda"):
        self.hidden, self.inter, self.experts, self.topk, self.max_tokens = hidden, inter, experts, topk, max_tokens
        self.device = torch.device(device)
        self.weights: dict[str, Weight] = {}
        self.router_bias = None   # optional float32 [experts] logit offset (not in the reference model)
        lib = _lib.lib()
        nbytes = lib.kogarashi_moe_workspace_bytes(hidden, inter, experts, topk, max_tokens)
        self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        _lib.check(lib.kogarashi_moe_workspace_init(self.workspace.data_ptr(), nbytes, self._stream()), "workspace_init")
        self.logits = torch.empty(max_tokens, experts, dtype=torch.float32, device=self.device)
        self.ids = torch.empty(max_tokens, topk, dtype=torch.int32, device=self.device)
        self.prob = torch.empty(max_tokens, topk, dtype=torch.float32, device=self.device)

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def load(self, name: str, raw: torch.Tensor, ty: int, ne) -> None:
        """Takes the bytes of a GGUF tensor (GGML order ne = [k, rows(, experts)]). Q6_K tensors are
        regrouped once into the 16-byte aligned device layout (lossless)."""
        if name not in TENSORS:
            raise KeyError(name)
        ne = tuple(int(d) for d in ne)
        if raw.dtype != torch.uint8 or raw.numel() != ggml_tensor_bytes(ty, ne):
            raise ValueError(f"{name}: expected {ggml_tensor_bytes(ty, ne)} bytes of GGML type {ty}")
        raw = raw.to(self.device).contiguous()
        k, rows = ne[0], ne[1] if len(ne) > 1 else 1
        if ty == GGML_Q6_K:
            lib = _lib.lib()
            total_rows = raw.numel() // (k // 256 * 210)
            packed = torch.empty(lib.darask_q6k_repacked_bytes(total_rows, k), dtype=torch.uint8, device=self.device)
            _lib.check(lib.darask_q6k_repack(packed.data_ptr(), raw.data_ptr(), total_rows, k, 0, self._stream()), "q6k_repack")
            raw = packed
        self.weights[name] = Weight(raw, ty, k, rows, ne)

    def _w(self, name):
        w = self.weights.get(name)
        return (w.data.data_ptr(), w.ty) if w is not None else (None, 0)

    def forward(self, x: torch.Tensor, n: torch.Tensor, attn_out: torch.Tensor | None = None, norm_w: torch.Tensor | None = None,
                eps: float = 1e-6) -> torch.Tensor:
        """x [T,H] float32 residual stream (updated in place), n [T,H] float32 normalised input.
        With `norm_w` (post_attention_norm.weight) the layer entry of engine.rs:507-526 is part of the call: x += attn_out
        (when given), n = rms_norm(x) * norm_w is computed by the layer and written to `n`."""
        t = n.shape[0]
        if t > self.max_tokens or n.shape != x.shape or n.shape[1] != self.hidden:
            raise ValueError("token count / shape")
        if x.dtype != torch.float32 or n.dtype != torch.float32 or not x.is_contiguous() or not n.is_contiguous():
            raise ValueError("x and n must be contiguous float32")
        d = _lib.KogarashiMoe()
        d.hidden, d.inter, d.experts, d.topk, d.tokens = self.hidden, self.inter, self.experts, self.topk, t
        d.router_w, d.router_ty = self._w("ffn_gate_inp.weight")
        d.router_bias = self.router_bias.data_ptr() if self.router_bias is not None else None
        d.gate_w, d.gate_ty = self._w("ffn_gate_exps.weight")
        d.up_w, d.up_ty = self._w("ffn_up_exps.weight")
        d.down_w, d.down_ty = self._w("ffn_down_exps.weight")
        d.sh_gate_w = self._w("ffn_gate_shexp.weight")[0]
        d.sh_up_w = self._w("ffn_up_shexp.weight")[0]
        d.sh_down_w = self._w("ffn_down_shexp.weight")[0]
        d.sh_inp_w = self._w("ffn_gate_inp_shexp.weight")[0]
        d.n, d.x = n.data_ptr(), x.data_ptr()
        if norm_w is not None:
            if norm_w.dtype != torch.float32 or norm_w.numel() != self.hidden or (attn_out is not None and (attn_out.shape != x.shape or attn_out.dtype != torch.float32)):
                raise ValueError("norm_w / attn_out")
            d.norm_w, d.norm_eps = norm_w.data_ptr(), eps
            d.attn_out = attn_out.data_ptr() if attn_out is not None else None
        elif attn_out is not None:
            raise ValueError("attn_out needs norm_w")
        d.logits, d.ids, d.prob = self.logits.data_ptr(), self.ids.data_ptr(), self.prob.data_ptr()
        d.workspace, d.workspace_bytes = self.workspace.data_ptr(), self.workspace.numel()
        _lib.check(_lib.lib().kogarashi_moe_layer(ctypes.byref(d), self._stream()), "kogarashi_moe_layer")
        return x

    def forward_host(self, x_host: torch.Tensor, n_host: torch.Tensor, out_host: torch.Tensor | None = None) -> torch.Tensor:
        """The layer for activations that live in host memory: x [T,H] and n [T,H] float32 on the CPU in, the updated
        x on the CPU out (a pinned buffer owned by the layer unless `out_host` is given).

        The two host->device copies, the layer call and the device->host copy are recorded once per token count as one
        CUDA graph over pinned staging buffers; a call copies the inputs into the staging buffers, replays the graph
        and waits for it. (The copies and the launch then cost one graph launch instead of four asynchronous calls.)"""
        t = n_host.shape[0]
        if x_host.shape != n_host.shape or n_host.shape[1] != self.hidden or t > self.max_tokens:
            raise ValueError("token count / shape")
        if x_host.dtype != torch.float32 or n_host.dtype != torch.float32 or x_host.is_cuda or n_host.is_cuda:
            raise ValueError("x_host and n_host must be float32 CPU tensors")
        plan = self._host_plans.get(t) if hasattr(self, "_host_plans") else None
        if plan is None:
            if not hasattr(self, "_host_plans"):
                self._host_plans = {}
            pin = lambda: torch.empty((t, self.hidden), dtype=torch.float32).pin_memory()
            plan = dict(pin_x=pin(), pin_n=pin(), pin_out=pin(), dx=torch.empty((t, self.hidden), device=self.device),
                        dn=torch.empty((t, self.hidden), device=self.device), graph=torch.cuda.CUDAGraph())
            plan["pin_x"].copy_(x_host)
            plan["pin_n"].copy_(n_host)

            def record():
                plan["dn"].copy_(plan["pin_n"], non_blocking=True)
                plan["dx"].copy_(plan["pin_x"], non_blocking=True)
                self.forward(plan["dx"], plan["dn"])
                plan["pin_out"].copy_(plan["dx"], non_blocking=True)

            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                record()                                   # once outside the capture: function attributes, lazy state
                side.synchronize()
                with torch.cuda.graph(plan["graph"], stream=side):
                    record()
            torch.cuda.current_stream(self.device).wait_stream(side)
            self._host_plans[t] = plan
        plan["pin_x"].copy_(x_host)
        plan["pin_n"].copy_(n_host)
        plan["graph"].replay()
        torch.cuda.current_stream(self.device).synchronize()
        if out_host is not None:
            out_host.copy_(plan["pin_out"])
            return out_host
        return plan["pin_out"]

    def status(self) -> int:
        out = ctypes.c_uint(0)
        _lib.check(_lib.lib().kogarashi_moe_status(self.workspace.data_ptr(), ctypes.byref(out), self._stream()), "status")
        return out.value
