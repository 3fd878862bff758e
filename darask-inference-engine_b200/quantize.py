"""Load-time quantizers (device kernels behind the C ABI): float32 tensors on the GPU -> the byte
layouts of the expert kernels. Mirrors the reference's load-time conversion steps
(engines/tsumuji/kernels/decode/quant.cu:77-114, engines/hayate/python-tools/hayate_tools/quant.py)."""
from __future__ import annotations

import torch

from . import _lib
from .formats import (GGML_Q4_K, GGML_Q6_K, fp8_block_bytes, ggml_tensor_bytes, nvfp4_linear_expert_bytes,
                      nvfp4_tiled_bytes)


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def ggml(w: torch.Tensor, ty: int) -> torch.Tensor:
    """float32 [..., k] (k % 256 == 0) -> uint8 GGUF Q4_K / Q6_K blocks, row-major."""
    if ty not in (GGML_Q4_K, GGML_Q6_K) or w.dtype != torch.float32 or w.shape[-1] % 256:
        raise ValueError("ggml quantizer: float32 input with k % 256 == 0, type 12 or 14")
    w = w.contiguous()
    out = torch.empty(ggml_tensor_bytes(ty, [w.numel()]), dtype=torch.uint8, device=w.device)
    _lib.check(_lib.lib().darask_quantize_ggml(out.data_ptr(), w.data_ptr(), ty, w.numel(), _stream(w)), "quantize_ggml")
    return out


def nvfp4_tiled(w: torch.Tensor) -> torch.Tensor:
    """float32 [n, k] -> Hayate NVFP4 matrix image."""
    n, k = w.shape
    w = w.contiguous()
    out = torch.empty(nvfp4_tiled_bytes(n, k), dtype=torch.uint8, device=w.device)
    scratch = torch.zeros(1, dtype=torch.int32, device=w.device)
    _lib.check(_lib.lib().darask_quantize_nvfp4_tiled(out.data_ptr(), w.data_ptr(), n, k, scratch.data_ptr(), _stream(w)),
               "quantize_nvfp4_tiled")
    return out


def nvfp4_linear_expert(gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor):
    """Three float32 matrices ([F,H], [F,H], [H,F]) -> (Tsumuji expert block uint8 [27/16 F H], gs float32 [3])."""
    f, h = gate.shape
    fh = f * h
    block = torch.empty(nvfp4_linear_expert_bytes(h, f), dtype=torch.uint8, device=gate.device)
    gs = torch.empty(3, dtype=torch.float32, device=gate.device)
    scratch = torch.zeros(1, dtype=torch.int32, device=gate.device)
    lib = _lib.lib()
    for i, (m, rows, cols) in enumerate(((gate, f, h), (up, f, h), (down, h, f))):
        m = m.contiguous()
        _lib.check(lib.darask_quantize_nvfp4_linear(block.data_ptr(), 0, i * fh // 2, fh * 3 // 2 + i * fh // 16,
                                                    gs.data_ptr() + 4 * i, 1, m.data_ptr(), 0, 1, rows, cols,
                                                    scratch.data_ptr(), _stream(m)), "quantize_nvfp4_linear")
    return block, gs


def fp8_block(w: torch.Tensor):
    """float32 [n, k] -> (e4m3 payload uint8 [n, k], float32 scales [ceil(n/128), ceil(k/128)])."""
    n, k = w.shape
    w = w.contiguous()
    payload = torch.empty((n, k), dtype=torch.uint8, device=w.device)
    scales = torch.empty(((n + 127) // 128, (k + 127) // 128), dtype=torch.float32, device=w.device)
    _lib.check(_lib.lib().darask_quantize_fp8_block(payload.data_ptr(), scales.data_ptr(), w.data_ptr(), n, k, _stream(w)),
               "quantize_fp8_block")
    return payload, scales


def fp8_act(x: torch.Tensor):
    """[rows, k] float32 or bf16 -> (e4m3 codes uint8 [rows, k], float32 scales [rows, k/128])."""
    rows, k = x.shape
    x = x.contiguous()
    codes = torch.empty((rows, k), dtype=torch.uint8, device=x.device)
    scales = torch.empty((rows, k // 128), dtype=torch.float32, device=x.device)
    _lib.check(_lib.lib().darask_quantize_fp8_act(codes.data_ptr(), scales.data_ptr(), x.data_ptr(),
                                                  1 if x.dtype == torch.bfloat16 else 0, rows, k, _stream(x)),
               "quantize_fp8_act")
    return codes, scales


__all__ = ["ggml", "nvfp4_tiled", "nvfp4_linear_expert", "fp8_block", "fp8_act", "fp8_block_bytes"]
