"""Enums and argument checks used by plan()/run() (reference: flashomni/utils.py:30-44,196-206,369-387)."""

from __future__ import annotations

from enum import Enum
from typing import Union

import torch


class PosEncodingMode(Enum):
    NONE = 0
    ROPE_LLAMA = 1
    ALIBI = 2


class MaskMode(Enum):
    NON_CAUSAL = 0
    CAUSAL = 1
    CUSTOM = 2


class TensorLayout(Enum):
    NHD = 0
    HND = 1


def _check_kv_layout(kv_layout: str) -> None:
    if not hasattr(TensorLayout, kv_layout):
        raise KeyError("Invalid kv_layout {}".format(kv_layout))


def _check_pos_encoding_mode(pos_encoding_mode: str) -> None:
    if not hasattr(PosEncodingMode, pos_encoding_mode):
        raise KeyError("Invalid pos_encoding_mode {}".format(pos_encoding_mode))


def canonicalize_torch_dtype(dtype: Union[torch.dtype, str]) -> torch.dtype:
    if isinstance(dtype, str):
        return getattr(torch, dtype)
    if isinstance(dtype, torch.dtype):
        return dtype
    raise TypeError("dtype must be a string or torch.dtype, got {}".format(type(dtype)))


def _check_cached_qkv_data_type(q, k, dtype_q, dtype_kv) -> None:
    if q.dtype != dtype_q:
        raise ValueError(
            f"The dtype of q {q.dtype} does not match the q_data_type {dtype_q} specified in plan function.")
    if k.dtype != dtype_kv:
        raise ValueError(
            f"The dtype of k {k.dtype} does not match the kv_data_type {dtype_kv} specified in plan function.")


def _check_shape_dtype_device(x, expected_shape, expected_dtype, expected_device, name) -> None:
    if tuple(x.shape) != tuple(expected_shape):
        raise ValueError(f"Invalid shape of {name}: expected {tuple(expected_shape)}, got {tuple(x.shape)}")
    if x.dtype != expected_dtype:
        raise ValueError(f"Invalid dtype of {name}: expected {expected_dtype}, got {x.dtype}")
    if x.device != expected_device:
        raise ValueError(f"Invalid device of {name}: expected {expected_device}, got {x.device}")


def native_dtype(dtype: torch.dtype) -> int:
    """torch dtype -> FO_DTYPE_* (the kernels compute in fp32 from fp16 / bf16 inputs)."""
    if dtype == torch.bfloat16:
        return 1
    if dtype == torch.float16:
        return 0
    raise NotImplementedError(f"flashomni_b200 implements float16 and bfloat16, got {dtype}")
