"""`flashomni.utils` of the reference (flashomni/utils.py:30-44,86-94,179-206,369-387): the enums and argument
checks that callers of the wrapper use, served by flashomni_b200.utils."""

from flashomni_b200.utils import (MaskMode, PosEncodingMode, TensorLayout, _check_cached_qkv_data_type,
                                  _check_kv_layout, _check_pos_encoding_mode, _check_shape_dtype_device,
                                  canonicalize_torch_dtype)

__all__ = ["MaskMode", "PosEncodingMode", "TensorLayout", "canonicalize_torch_dtype"]
