"""CPU restatement of the reference MoE FFN arithmetic. TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this directory.  It exists so that the
CUDA path can be checked against the reference engine's own formulas:

* ``formats``  - weight formats (GGUF Q4_K / Q6_K, NVFP4 linear and tiled,
  block FP8) : byte layouts, decoders, quantizers.
* ``routing``  - the three router definitions and the dispatch permutation.
* ``layers``   - whole MoE layers per engine (Kogarashi, Tsumuji, Hayate) and
  the FP8 prefill layer, accumulated in float64 from exactly decoded weights.
* ``cpu_moe.c`` - a multithreaded C restatement of the expert products, used
  for large parity cases and as the timed CPU baseline.

Pinning: decoders, code tables, scale tiling, SwiGLU/bf16 rounding, reduction
order and the dispatch permutation are pinned by the reference's own known
answer tests (restated in ``tests/test_oracle_golden.py``), by fixtures that
the reference's Python quantizer produced (``tests/golden``) and by the
reference's host-compilable C++ headers built into ``oracle/_ref``.  The GGUF
Q4_K / Q6_K *quantizers* are written fresh from the block layout that the
reference decoder defines (the reference ships no quantizer for them):
their parity is unpinned; only the decode formulas are pinned.
"""
