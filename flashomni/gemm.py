"""`flashomni.gemm` of the reference (flashomni/gemm.py:156-216), served by flashomni_b200.gemm."""

from flashomni_b200.gemm import flashomni_gemm, flashomni_gemm_reduction

__all__ = ["flashomni_gemm", "flashomni_gemm_reduction"]
