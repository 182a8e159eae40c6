"""`flashomni.attention` of the reference (flashomni/attention.py:165-869), served by flashomni_b200.attention."""

from flashomni_b200.attention import (BatchFlashOmniFAWithRaggedKVWrapper, _compute_sparse_info_indptr,
                                      _compute_sparse_kv_info_indptr)

__all__ = ["BatchFlashOmniFAWithRaggedKVWrapper"]
