"""CPU oracle for the sparse-DiT hot path (TEST INFRASTRUCTURE ONLY).

This package restates, in numpy / fp32 torch on the CPU, what the reference computes for
mask packing, block-sparse attention, GEMM-Q and GEMM-O, plus the canonical outputs of the
mask-compaction step. It exists to check the CUDA path; nothing in the product package may
import it. Only the tests, the smoke entry and the benchmark's CPU-baseline leg use it.

Pinning: the reference holds no stored golden outputs for this path. The only known-answer
vectors it has are the two docstring examples of bit packing (flashomni/quantization.py:90-93
and :133-138); `oracle.masks` is checked against both. For the floating-point functions the
reference's own check is an on-the-fly comparison with dense masked torch attention
(benchmark/test_flashomni_attention.py:197-231) and `nn.Linear` (benchmark/test_flashomni_gemm_q.py:29-78,
benchmark/test_flashomni_gemm_o.py:73-87); `oracle.attention` / `oracle.gemm` restate exactly those
constructions and are cross-checked against a dense masked-softmax formula in the CPU tests.
"""

from . import masks, attention, gemm  # noqa: F401
