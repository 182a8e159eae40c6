"""flashomni_b200: the FlashOmni sparse-DiT hot path re-built for NVIDIA B200 (sm_100a).

Same public names as the reference package `flashomni` (flashomni/__init__.py:17-28):
`BatchFlashOmniFAWithRaggedKVWrapper`, `flashomni_gemm`, `flashomni_gemm_reduction`, `packbits`,
`segment_packbits`. Python host code -> C ABI (include/flashomni_b200.h) -> hand-written CUDA.
"""

__version__ = "0.1.0"

from . import attention as attention  # noqa: F401
from .attention import (BatchFlashOmniFAWithRaggedKVWrapper, _compute_sparse_info_indptr,  # noqa: F401
                        _compute_sparse_kv_info_indptr)
from .gemm import flashomni_gemm as flashomni_gemm  # noqa: F401
from .gemm import flashomni_gemm_reduction as flashomni_gemm_reduction  # noqa: F401
from .quantization import packbits as packbits  # noqa: F401
from .quantization import segment_packbits as segment_packbits  # noqa: F401
from .selection import select_blocks as select_blocks  # noqa: F401
