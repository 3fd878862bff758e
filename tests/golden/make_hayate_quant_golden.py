"""Generates tests/golden/hayate_quant.npz by running the reference engine's own Python
quantizer (engines/hayate/python-tools/hayate_tools/quant.py) on seeded inputs.

Run where a reference checkout exists:  python tests/golden/make_hayate_quant_golden.py [ref]
The package __init__ of hayate_tools probes for a CUDA driver, so the module is imported
through a stub package that only sets the search path.
"""
import os
import sys
import types

import numpy as np
import torch

os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
sys.dont_write_bytecode = True
# the reference checkout: first argument, else a directory named "reference" beside this repository
ref = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "..", "reference")
pkg = types.ModuleType("hayate_tools")
pkg.__path__ = [os.path.join(ref, "engines/hayate/python-tools/hayate_tools")]
sys.modules["hayate_tools"] = pkg
from hayate_tools import quant  # noqa: E402
from hayate_tools.hyt import E4M3, NVFP4, PER_TENSOR  # noqa: E402

out = {}
rng = np.random.Generator(np.random.PCG64(1234))
for name, shape, std in [("a", (129, 80), 0.02), ("b", (256, 256), 0.02), ("c", (32, 512), 1.0)]:
    w = (rng.standard_normal(shape) * std).astype(np.float32)
    if name == "c":
        w[0, :16] = 0.0                       # an all-zero block
        w[1, :16] = [0., .25, .5, .75, 1., 1.25, 1.5, 1.75, 2., 2.5, 3., 3.5, 4., 5., 6., -0.]
    img = quant.quantize(torch.from_numpy(w), (NVFP4, 0, 0)).numpy()
    deq = quant.dequantize_nvfp4(torch.from_numpy(img), w.shape).numpy()
    out[f"nvfp4_{name}_w"], out[f"nvfp4_{name}_img"], out[f"nvfp4_{name}_deq"] = w, img, deq
w = (rng.standard_normal((4, 64)) * 3).astype(np.float32)
out["fp8_w"] = w
out["fp8_img"] = quant.quantize(torch.from_numpy(w), (PER_TENSOR, E4M3, 0)).numpy()
# e4m3 rounding of a dense sweep, through torch (the conversion quant.py relies on)
sweep = np.concatenate([np.linspace(-448, 448, 20001), rng.standard_normal(20000) * 0.01,
                        np.array([0, -0.0, 2 ** -10, 2 ** -9 * 1.5, 2 ** -9 * 2.5, 0.001953125 * 0.5])]).astype(np.float32)
out["e4m3_in"] = sweep
out["e4m3_code"] = torch.from_numpy(sweep).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "hayate_quant.npz"), **out)
print({k: v.shape for k, v in out.items()})
