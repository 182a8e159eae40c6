"""`flashomni.quantization` of the reference (flashomni/quantization.py:68-159), served by flashomni_b200.quantization."""

from flashomni_b200.quantization import packbits, segment_packbits

__all__ = ["packbits", "segment_packbits"]
