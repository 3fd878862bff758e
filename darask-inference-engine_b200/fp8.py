"""Host-side mirror of the FP8 prefill MoE path: block-scaled e4m3 expert weights, e4m3 activations, grouped
products on the tcgen05 tensor cores.

Reference: `prefill_experts`, engines/hayate/crates/models/src/glm53/gpu.rs:2068-2566 (route, group the routes by
expert, gather rows, grouped gate/up product, SwiGLU, grouped down product, scatter with the routing weights); weight
format `Fp8Block`, engines/hayate/crates/kernels/src/cpu/glm53.rs:23-24.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def grouped_gemm(a_codes, a_scales, ranges, w0, sw0, w1=None, sw1=None, quantize=False, row_map=None):
    """Ragged grouped product. a_codes uint8 [rows(+pad), k], a_scales float32 [rows(+pad), k/128], ranges uint32
    [E, 2] = {rows, offset}, w uint8 [E, n, k], sw float32 [E, n/128, k/128].  Without w1: float32 a w0^T (dispatch
    row i written to row row_map[i] when a map is given).  With w1: bf16 silu(a w0^T) * (a w1^T), or with `quantize`
    its e4m3 codes and float32 scales per row and 128 columns.  Rows outside every range are left untouched."""
    experts, n, k = w0.shape
    rows = a_codes.shape[0]
    dev = a_codes.device
    mode = 0 if w1 is None else (2 if quantize else 1)
    out = torch.zeros(rows, n, dtype=(torch.float32, torch.bfloat16, torch.uint8)[mode], device=dev)
    scales = torch.zeros(rows, n // 128, dtype=torch.float32, device=dev) if mode == 2 else None
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream(dev).cuda_stream
    _lib.check(_lib.lib().darask_fp8_grouped_gemm(
        a_codes.data_ptr(), a_scales.data_ptr(), rows, w0.data_ptr(), w1.data_ptr() if mode else None, sw0.data_ptr(),
        sw1.data_ptr() if mode else None, experts, n, k, mode, ranges.data_ptr(), out.data_ptr(),
        scales.data_ptr() if mode == 2 else None, row_map.data_ptr() if row_map is not None else None, status.data_ptr(), st),
        "darask_fp8_grouped_gemm")
    if int(status.item()):
        raise RuntimeError(f"darask_fp8_grouped_gemm: device status {int(status.item()):#x}")
    return (out, scales) if mode == 2 else out


class Fp8MoeLayer:
    def __init__(self, hidden: int, inter: int, experts: int, topk: int, max_tokens: int, device="cuda"):
        self.hidden, self.inter, self.experts, self.topk, self.max_tokens = hidden, inter, experts, topk, max_tokens
        self.device = torch.device(device)
        nbytes = _lib.lib().darask_fp8_moe_workspace_bytes(hidden, inter, experts, topk, max_tokens)
        self.workspace = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        self.ids = torch.empty(max_tokens, topk, dtype=torch.int32, device=self.device)
        self.prob = torch.empty(max_tokens, topk, dtype=torch.float32, device=self.device)
        self.w = {}

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def load(self, name: str, payload: torch.Tensor, scales: torch.Tensor) -> None:
        """name in gate|up|down; payload uint8 [E, n, k]; scales float32 [E, n/128, k/128]."""
        n, k = (self.hidden, self.inter) if name == "down" else (self.inter, self.hidden)
        if tuple(payload.shape) != (self.experts, n, k) or tuple(scales.shape) != (self.experts, n // 128, k // 128):
            raise ValueError(f"{name}: expected payload [E,{n},{k}] and scales [E,{n // 128},{k // 128}]")
        self.w[name] = (payload.to(self.device, torch.uint8).contiguous(), scales.to(self.device, torch.float32).contiguous())

    def forward(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        """x bf16 [T,H], logits float32 [T,E] -> float32 [T,H] (the routed experts' weighted sum)."""
        t = x.shape[0]
        if t > self.max_tokens or x.dtype != torch.bfloat16 or logits.dtype != torch.float32 or not x.is_contiguous() or not logits.is_contiguous():
            raise ValueError("x must be contiguous bf16 [T<=max_tokens,H], logits contiguous float32 [T,E]")
        out = torch.empty(t, self.hidden, dtype=torch.float32, device=self.device)
        d = _lib.DaraskFp8Moe()
        d.hidden, d.inter, d.experts, d.topk, d.tokens = self.hidden, self.inter, self.experts, self.topk, t
        d.x, d.logits = x.data_ptr(), logits.data_ptr()
        (gw, gs), (uw, us), (dw, ds) = self.w["gate"], self.w["up"], self.w["down"]
        d.gate_w, d.up_w, d.down_w = gw.data_ptr(), uw.data_ptr(), dw.data_ptr()
        d.gate_s, d.up_s, d.down_s = gs.data_ptr(), us.data_ptr(), ds.data_ptr()
        d.out, d.ids, d.prob = out.data_ptr(), self.ids.data_ptr(), self.prob.data_ptr()
        d.workspace, d.workspace_bytes = self.workspace.data_ptr(), self.workspace.numel()
        _lib.check(_lib.lib().darask_fp8_moe_layer(ctypes.byref(d), self._stream()), "darask_fp8_moe_layer")
        return out

    def status(self) -> int:
        s = ctypes.c_uint(0)
        _lib.check(_lib.lib().darask_fp8_moe_status(self.workspace.data_ptr(), ctypes.byref(s), self._stream()), "darask_fp8_moe_status")
        return s.value
