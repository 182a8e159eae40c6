"""ctypes binding of libflashomni_b200.so (the C ABI declared in include/flashomni_b200.h).

The library is built in-tree by `python -m flashomni_b200.build`. There is no fallback of any kind:
if the library is missing, or no CUDA device is present when an op is called, the call raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int32, c_int64, c_size_t, c_void_p

_LIB_ENV = "FLASHOMNI_B200_LIB"
_HERE = os.path.dirname(os.path.abspath(__file__))
_DEFAULT = os.path.join(_HERE, "lib", "libflashomni_b200.so")

FO_OK, FO_ERR_INVALID_ARG, FO_ERR_UNSUPPORTED, FO_ERR_CUDA, FO_ERR_WORKSPACE = 0, 1, 2, 3, 4
FO_DTYPE_F16, FO_DTYPE_BF16 = 0, 1
FO_DEV_OK, FO_DEV_WAIT_TIMEOUT, FO_DEV_BAD_INDEX = 0, 1, 2

# name -> (restype, argtypes); mirrors include/flashomni_b200.h one to one
_P = c_void_p
SIGNATURES = {
    "fo_last_error": (c_char_p, []),
    "fo_strided_gather": (c_int32, [c_int32, _P, _P, _P, _P, _P, c_int64, _P]),
    "fo_gemm_q_prepared": (c_int32, [_P, _P, _P, _P, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, _P, c_size_t, _P]),
    "fo_gemm_o_prepared": (c_int32, [_P, _P, _P, _P, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                                     _P, c_size_t, _P]),
    "fo_select_blocks_scratch_bytes": (c_size_t, [c_int32, c_int32]),
    "fo_select_blocks": (c_int32, [_P, c_int32, c_int32, c_int32, c_int32, _P, _P, c_int32, _P, c_int64, _P, c_int64,
                                   _P, _P, _P, c_size_t, _P]),
    "fo_abi_version": (c_int32, []),
    "fo_launch_count": (ctypes.c_longlong, []),
    "fo_reduce_rows": (c_int32, [c_int32, _P, c_int64, _P, c_int64, _P, c_int64, c_int64, c_int64, c_int32, _P]),
    "fo_peer_barrier": (c_int32, [c_int32, c_int32, _P, c_int32, c_int32, _P, _P, c_int64, _P]),
    "fo_packbits": (c_int32, [_P, c_int64, c_int32, _P, _P]),
    "fo_segment_packbits": (c_int32, [_P, _P, _P, c_int32, c_int64, c_int32, _P, _P]),
    "fo_mask_compact_scratch_bytes": (c_size_t, [c_int64, c_int32]),
    "fo_mask_compact": (c_int32, [_P, c_int64, _P, c_int64, _P, _P, _P, _P,
                                  c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                                  c_int64, c_int32, c_int64, c_int64,
                                  _P, _P, _P, _P, _P, _P, c_size_t, _P]),
    "fo_attn_units": (c_int32, [_P, _P, _P, _P, _P, _P, _P, c_int64, c_int32, c_int32, c_int32, c_int32, c_int32,
                                c_int32, c_int64, c_int64, _P, _P, _P, _P]),
    "fo_attn_partial_bytes": (c_size_t, [c_int64]),
    "fo_cast_fp8": (c_int32, [_P, c_int64, c_int32, c_int32, _P, _P]),
    "fo_sparse_attn_fwd": (c_int32, [_P, _P, _P, _P, _P, c_int32,
                                     c_int64, c_int64, c_int32, c_int32, c_int32,
                                     c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                     c_int32, c_int32, _P, _P, _P,
                                     c_int64, _P, _P, c_int64, c_int32, c_float, _P, _P]),
    "fo_sparse_attn_fwd_softcap": (c_int32, [_P, _P, _P, _P, _P, c_int32,
                                             c_int64, c_int64, c_int32, c_int32, c_int32,
                                             c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                             c_int32, c_int32, _P, _P, _P,
                                             c_int64, _P, _P, c_int64, c_int32, c_float, c_float, _P, _P]),
    "fo_sparse_attn_fwd_causal": (c_int32, [_P, _P, _P, _P, _P, c_int32,
                                            c_int64, c_int64, c_int32, c_int32, c_int32,
                                            c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                            c_int32, c_int32, _P, _P, _P,
                                            c_int64, c_int32, c_float, c_float, _P, _P]),
    "fo_sparse_attn_fwd_custom_mask": (c_int32, [_P, _P, _P, _P, _P, c_int32,
                                                 c_int64, c_int64, c_int32, c_int32, c_int32,
                                                 c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                                 c_int32, c_int32, _P, _P, _P,
                                                 c_int64, c_int32, c_float, c_float, _P, c_int64, _P, _P, _P, _P, _P]),
    "fo_gemm_workspace_bytes": (c_size_t, [c_int32, c_int32, c_int32, c_int32, c_int32]),
    "fo_gemm_dense_tile_rows": (c_int32, [c_int32, c_int32, c_int32, c_int32, c_int32, c_int32]),
    "fo_gemm_dense_tile_cols": (c_int32, [c_int32, c_int32, c_int32, c_int32, c_int32, c_int32]),
    "fo_gemm_q": (c_int32, [_P, _P, _P, _P, c_int32, c_int32, c_int32, c_int32, c_int32,
                            c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                            _P, c_int64, _P, _P, c_size_t, _P]),
    "fo_gemm_o": (c_int32, [_P, _P, _P, _P, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                            c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                            _P, c_int64, _P, _P, c_size_t, _P]),
    "fo_gemm_q_static_max_bytes": (c_size_t, []),
    "fo_gemm_q_static_last_error": (c_char_p, []),
    "fo_gemm_q_static": (c_int32, [_P, _P, _P, _P, c_int32, c_int32, c_int32, c_int32, c_int32,
                                   c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                                   _P, c_int64, _P, _P]),
    "fo_gemm_q_worklist": (c_int32, [c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                                     c_int32, _P, c_int64, _P, _P, c_size_t, _P]),
    "fo_gemm_o_worklist": (c_int32, [c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                                     c_int32, _P, c_int64, _P, _P, c_size_t, _P]),
}

_lib = None


def lib_path() -> str:
    return os.environ.get(_LIB_ENV, _DEFAULT)


def load():
    """Loads the shared library once and sets the prototypes. Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"flashomni_b200: native library not found at {path}; build it with "
            "`python -m flashomni_b200.build` (there is no non-CUDA fallback)")
    import torch  # noqa: F401  (loads the CUDA runtime the library links against)
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if lib.fo_abi_version() != 2:
        raise RuntimeError("flashomni_b200: ABI version mismatch")
    _lib = lib
    return lib


def last_error() -> str:
    return load().fo_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    """Maps a C-ABI return code to the exceptions the reference raises for the same condition:
    argument / shape problems -> ValueError / RuntimeError (TORCH_CHECK), CUDA failures -> RuntimeError."""
    if rc == FO_OK:
        return
    msg = f"{what}: {last_error()}"
    if rc == FO_ERR_INVALID_ARG:
        raise ValueError(msg)
    if rc == FO_ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(msg)


def ptr(t) -> int | None:
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("flashomni_b200: tensors must live on a CUDA device (no CPU path exists)")


def current_stream(device) -> int:
    import torch
    return torch.cuda.current_stream(device).cuda_stream


def debug_checks() -> bool:
    """FLASHOMNI_B200_CHECK=1 makes every op synchronise and verify its device status word."""
    return os.environ.get("FLASHOMNI_B200_CHECK", "0") not in ("0", "")
