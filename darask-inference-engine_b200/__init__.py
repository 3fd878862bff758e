"""B200-native MoE FFN layer for the Darask inference engines (Kogarashi, Tsumuji, Hayate).

The product is the CUDA library ``libdarask_moe_b200.so`` (C ABI in ``include/darask_moe_b200.h``);
the modules here are the host-side mirror of the reference engines' MoE layer calls on top of it.
PyTorch is used for device memory and streams only.
"""
from . import _lib  # noqa: F401
from .formats import (GGML_BF16, GGML_F16, GGML_F32, GGML_Q4_K, GGML_Q6_K, ggml_tensor_bytes,  # noqa: F401
                      nvfp4_tiled_bytes)
from . import quantize  # noqa: F401
from .kogarashi import KogarashiMoeLayer  # noqa: F401
from .tsumuji import TsumujiMoeLayer  # noqa: F401
from .hayate import HayateMoeLayer  # noqa: F401
from .fp8 import Fp8MoeLayer  # noqa: F401
from . import fp8  # noqa: F401
from . import ep  # noqa: F401
from . import gguf  # noqa: F401
from . import tsumuji_loader  # noqa: F401
from . import hyt  # noqa: F401
from .ep import Fp8ExpertParallelMoe, TsumujiExpertParallelMoe  # noqa: F401

__all__ = ["KogarashiMoeLayer", "ggml_tensor_bytes", "nvfp4_tiled_bytes"]
