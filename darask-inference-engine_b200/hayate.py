"""Host-side mirror of the Hayate MoE layer calls.

Reference: `Layer::decode` / `decode_moe` / `decode_moe_reduce`, engines/hayate/crates/models/src/glm53/gpu.rs:
1582-1905, with expert images laid out as engines/hayate/crates/models/src/glm53/experts.rs:68-74 (gate | up |
down at a 256-byte aligned stride, NVFP4 matrices with 128x4-tiled scales).  All images are resident on the
GPU; the reference's CPU slots and placement tables have no counterpart here.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .formats import nvfp4_expert_stride


class HayateMoeLayer:
    def __init__(self, hidden: int, inter: int, experts: int, topk: int, scale: float = 2.5, max_tokens: int = 1, device="cuda"):
        self.hidden, self.inter, self.experts, self.topk, self.scale = hidden, inter, experts, topk, scale
        self.max_tokens, self.device = max_tokens, torch.device(device)
        self.stride = nvfp4_expert_stride(hidden, inter)
        lib = _lib.lib()
        nbytes = lib.hayate_moe_workspace_bytes(hidden, inter, experts, topk, max_tokens)
        self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        _lib.check(lib.hayate_moe_workspace_init(self.workspace.data_ptr(), nbytes, self._stream()), "workspace_init")
        self.logits = torch.empty(max_tokens, experts, dtype=torch.float32, device=self.device)
        self.ids = torch.empty(max_tokens, topk, dtype=torch.int32, device=self.device)
        self.weights = torch.empty(max_tokens, topk, dtype=torch.float32, device=self.device)
        self.router = self.bias = self.images = self.shared = None

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def load(self, router, bias, images, shared_image) -> None:
        """router bf16 [E,H], bias float32 [E], images uint8 [E, 3*stride], shared_image uint8 [3*stride]."""
        if images.dtype != torch.uint8 or images.numel() != self.experts * 3 * self.stride or shared_image.numel() != 3 * self.stride:
            raise ValueError("images: expected [E, 3*stride] bytes and a shared image of 3*stride bytes")
        self.router = router.to(self.device, torch.bfloat16).contiguous()
        self.bias = bias.to(self.device, torch.float32).contiguous()
        self.images = images.to(self.device).contiguous()
        self.shared = shared_image.to(self.device).contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x bf16 [T,H] -> bf16 [T,H]."""
        t = x.shape[0]
        if t > self.max_tokens or x.shape[1] != self.hidden or x.dtype != torch.bfloat16 or not x.is_contiguous():
            raise ValueError("x must be contiguous bf16 [T<=max_tokens, hidden]")
        out = torch.empty_like(x)
        d = _lib.HayateMoe()
        d.hidden, d.inter, d.experts, d.topk, d.tokens, d.scale = self.hidden, self.inter, self.experts, self.topk, t, self.scale
        d.router_w, d.bias = self.router.data_ptr(), self.bias.data_ptr()
        d.images, d.stride, d.shared_image = self.images.data_ptr(), self.stride, self.shared.data_ptr()
        d.x, d.out = x.data_ptr(), out.data_ptr()
        d.logits, d.ids, d.weights = self.logits.data_ptr(), self.ids.data_ptr(), self.weights.data_ptr()
        d.workspace, d.workspace_bytes = self.workspace.data_ptr(), self.workspace.numel()
        _lib.check(_lib.lib().hayate_moe_layer(ctypes.byref(d), self._stream()), "hayate_moe_layer")
        return out
