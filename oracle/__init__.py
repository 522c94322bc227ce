"""CPU oracle for the DecDEC decode hot path.

TEST INFRASTRUCTURE ONLY.  This package restates, in numpy / CPU torch, the arithmetic of the
reference implementation (SNU-ARC/DecDEC) for the quantized-weight GEMV with dynamic error
compensation.  It exists to check the CUDA library; nothing in the shipped package imports it.
Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may use it.

Pinning status: the reference ships no golden vectors and no assertions for this path
(its `decdec_extension/tests/*.py` only print values).  The pins used instead are
  * fixtures under `tests/golden/` produced by importing the reference's own Python functions
    (`decdec_setup/cheatsheet.py:_process_layer`, `llm-awq/quantize/quantizer.py:pseudo_quantize_tensor`,
    `evaluation/evaltools.py:lutgemm_dequant/sqllm_dequant`) in a CPU container, and
  * a numpy emulation of the reference CUDA bit manipulation for the any-precision layout
    (`decdec_extension/anyprec.cu:11-66,261-331`).
The bucket selection of `decdec_extension/dec.cu:78-182` has no CPU counterpart in the reference;
it is restated here with a reproducible choice inside the bucket that overflows the quota (lowest
channel indices first) and a fixed output order, because the reference leaves both to atomic arrival
order.
"""

from . import formats, residual, selection, forward  # noqa: F401
