"""ctypes binding of libdarask_moe_b200.so. There is no fallback: a missing library is an error."""
from __future__ import annotations

import ctypes
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libdarask_moe_b200.so"
_lib = None

c_void_p, c_int, c_float, c_size_t, c_uint, c_longlong = (ctypes.c_void_p, ctypes.c_int, ctypes.c_float,
                                                           ctypes.c_size_t, ctypes.c_uint, ctypes.c_longlong)


class KogarashiMoe(ctypes.Structure):
    """Mirror of `KogarashiMoe` in include/darask_moe_b200.h."""
    _fields_ = [
        ("hidden", c_int), ("inter", c_int), ("experts", c_int), ("topk", c_int), ("tokens", c_int),
        ("router_w", c_void_p), ("router_ty", c_int), ("router_bias", c_void_p),
        ("gate_w", c_void_p), ("gate_ty", c_int),
        ("up_w", c_void_p), ("up_ty", c_int),
        ("down_w", c_void_p), ("down_ty", c_int),
        ("sh_gate_w", c_void_p), ("sh_up_w", c_void_p), ("sh_down_w", c_void_p), ("sh_inp_w", c_void_p),
        ("n", c_void_p), ("x", c_void_p), ("logits", c_void_p), ("ids", c_void_p), ("prob", c_void_p),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("attn_out", c_void_p), ("norm_w", c_void_p), ("norm_eps", c_float), ("reserved", c_int),
    ]


class TsumujiMoe(ctypes.Structure):
    """Mirror of `TsumujiMoe` in include/darask_moe_b200.h."""
    _fields_ = [
        ("hidden", c_int), ("inter", c_int), ("experts", c_int), ("topk", c_int), ("tokens", c_int),
        ("router_w", c_void_p), ("experts_w", c_void_p), ("gs", c_void_p),
        ("shared_gu", c_void_p), ("shared_down", c_void_p),
        ("x", c_void_p), ("out", c_void_p), ("rlogits", c_void_p), ("sel", c_void_p), ("rw", c_void_p),
        ("shared_gate", c_void_p), ("accumulate", c_int),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("R", c_void_p), ("di", c_void_p), ("Sd", c_int), ("ld", c_int), ("rank", c_int), ("HC", c_int), ("ss", c_void_p),
    ]


class HayateDenseWeight(ctypes.Structure):
    _fields_ = [("data", c_void_p), ("scale", c_void_p), ("format", c_uint)]


class HayateMoe(ctypes.Structure):
    """Mirror of `HayateMoe` in include/darask_moe_b200.h."""
    _fields_ = [
        ("hidden", c_int), ("inter", c_int), ("experts", c_int), ("topk", c_int), ("tokens", c_int), ("scale", c_float),
        ("router_w", c_void_p), ("bias", c_void_p), ("images", c_void_p), ("stride", c_size_t), ("shared_image", c_void_p),
        ("x", c_void_p), ("out", c_void_p), ("logits", c_void_p), ("ids", c_void_p), ("weights", c_void_p),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
    ]


class DaraskFp8Moe(ctypes.Structure):
    """Mirror of `DaraskFp8Moe` in include/darask_moe_b200.h."""
    _fields_ = [
        ("hidden", c_int), ("inter", c_int), ("experts", c_int), ("topk", c_int), ("tokens", c_int),
        ("x", c_void_p), ("logits", c_void_p), ("gate_w", c_void_p), ("up_w", c_void_p), ("down_w", c_void_p),
        ("gate_s", c_void_p), ("up_s", c_void_p), ("down_s", c_void_p), ("out", c_void_p), ("ids", c_void_p), ("prob", c_void_p),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
    ]


_SIGNATURES = {
    "darask_route_topk": (c_int, [c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p,
                                  c_void_p, c_void_p]),
    "darask_route_topk_hayate": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p,
                                         c_void_p]),
    "darask_moe_permute": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p]),
    "darask_q6k_repacked_bytes": (c_size_t, [c_longlong, c_int]),
    "darask_q6k_repack": (c_int, [c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p]),
    "darask_quantize_ggml": (c_int, [c_void_p, c_void_p, c_int, c_longlong, c_void_p]),
    "darask_quantize_nvfp4_linear": (c_int, [c_void_p, c_longlong, c_longlong, c_longlong, c_void_p, c_int, c_void_p,
                                             c_longlong, c_int, c_int, c_int, c_void_p, c_void_p]),
    "darask_quantize_nvfp4_tiled": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "darask_quantize_fp8_block": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "darask_quantize_fp8_act": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_int, c_void_p]),
    "darask_moe_permute_scratch_bytes": (c_size_t, [c_int, c_int, c_int]),
    "darask_moe_permute_large": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_size_t, c_void_p]),
    "darask_fp8_grouped_gemm": (c_int, [c_void_p, c_void_p, ctypes.c_ulonglong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                        c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "tsumuji_ep_dispatch": (c_int, [ctypes.POINTER(TsumujiMoe), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "tsumuji_ep_experts_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "tsumuji_ep_experts": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_size_t,
                                   c_void_p]),
    "tsumuji_ep_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "hayate_glm_grouped": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_uint, c_uint, c_uint, c_void_p, c_void_p]),
    "hayate_glm_grouped_nvfp4": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_uint, c_uint, c_uint, c_void_p, c_void_p,
                                         c_uint, c_void_p]),
    "hayate_glm_restore": (c_int, [c_void_p, c_void_p, c_void_p, c_uint, c_uint, c_void_p]),
    "hayate_glm_nvfp4_restore": (c_int, [c_void_p, c_void_p, c_uint, c_uint, c_void_p]),
    "hayate_glm_nvfp4_restore_unscaled": (c_int, [c_void_p, c_void_p, c_void_p, c_uint, c_uint, c_void_p]),
    "hayate_glm_gather": (c_int, [c_void_p, c_void_p, c_void_p, c_uint, c_uint, c_void_p]),
    "hayate_glm_scatter": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_uint, c_uint, c_void_p]),
    "hayate_glm_copy": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "hayate_glm_grouped_packed_set_config": (c_int, [c_uint]),
    "hayate_glm_grouped_packed_gate_up": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_uint, c_uint, c_uint, c_void_p]),
    "hayate_glm_grouped_packed_down": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_uint, c_uint, c_uint, c_void_p]),
    "hayate_glm_grouped_packed_status": (c_int, [c_void_p, c_void_p]),
    "darask_fp8_ep_dispatch_scratch_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "darask_fp8_ep_dispatch": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_size_t, c_void_p]),
    "darask_fp8_ep_regroup": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, ctypes.c_longlong, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_size_t, c_void_p]),
    "darask_fp8_ep_experts": (c_int, [c_void_p, c_void_p, ctypes.c_ulonglong, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "darask_fp8_ep_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "darask_fp8_ep_packed_row_bytes": (c_size_t, [c_int]),
    "darask_fp8_ep_dispatch_packed": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "darask_fp8_ep_regroup_packed": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "darask_fp8_ep_reduce": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p]),
    "darask_fp8_ep_sum": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "darask_fp8_moe_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "darask_fp8_moe_layer": (c_int, [ctypes.POINTER(DaraskFp8Moe), c_void_p]),
    "darask_fp8_moe_status": (c_int, [c_void_p, ctypes.POINTER(c_uint), c_void_p]),
    "hayate_glm_moe_set_shape": (c_int, [c_uint, c_uint, c_uint, c_uint, c_float]),
    "hayate_glm_moe_workspace_bytes": (c_size_t, [c_uint, c_uint, c_uint, c_uint, c_uint]),
    "hayate_glm_moe_set_workspace": (c_int, [c_void_p, c_size_t, c_void_p]),
    "hayate_glm_route_decode": (c_int, [c_void_p] * 6 + [c_void_p]),
    "hayate_glm_route": (c_int, [c_void_p] * 6 + [c_uint, c_uint, c_uint, c_uint, c_void_p]),
    "hayate_glm_route_batch": (c_int, [c_void_p] * 6 + [c_uint, c_void_p]),
    "hayate_glm_moe_gate_up": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, HayateDenseWeight, HayateDenseWeight, c_int,
                                       c_int, c_size_t, c_void_p]),
    "hayate_glm_moe_down": (c_int, [c_void_p, c_void_p, c_void_p, HayateDenseWeight, c_int, c_int, c_size_t, c_void_p]),
    "hayate_glm_moe_reduce": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "hayate_moe_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "hayate_moe_workspace_init": (c_int, [c_void_p, c_size_t, c_void_p]),
    "hayate_moe_layer": (c_int, [ctypes.POINTER(HayateMoe), c_void_p]),
    "tsumuji_moe_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "tsumuji_moe_workspace_init": (c_int, [c_void_p, c_size_t, c_void_p]),
    "tsumuji_moe_layer": (c_int, [ctypes.POINTER(TsumujiMoe), c_void_p]),
    "kogarashi_moe_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "kogarashi_moe_workspace_init": (c_int, [c_void_p, c_size_t, c_void_p]),
    "kogarashi_moe_layer": (c_int, [ctypes.POINTER(KogarashiMoe), c_void_p]),
    "kogarashi_moe_set_single_launch": (c_int, [c_int]),
    "kogarashi_moe_static_scratch_bytes": (c_size_t, []),
    "kogarashi_moe_layer_static": (c_int, [ctypes.POINTER(KogarashiMoe), c_void_p]),
    "kogarashi_moe_static_status": (c_int, [ctypes.POINTER(c_uint), c_void_p]),
    "kogarashi_moe_status": (c_int, [c_void_p, ctypes.POINTER(c_uint), c_void_p]),
}


def exported_symbols():
    return sorted(_SIGNATURES)


def lib() -> ctypes.CDLL:
    """Loads the shared library (built by build.py). Raises if it is missing."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: run `python {HERE / 'build.py'}` (needs nvcc). "
                               "There is no CPU fallback for the MoE kernels.")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


class CudaError(RuntimeError):
    pass


def check(code: int, what: str) -> None:
    if code != 0:
        raise CudaError(f"{what} failed with cudaError {code}")
