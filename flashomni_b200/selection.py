"""Block selection: pooled attention scores -> the packed masks the hot path consumes.

The reference builds its masks with torch ops and Triton fill kernels on an unpacked `[B, H, nq, nkv]` layout
(`benchmark/test_attn_score.py:93-133`) that callers transpose to `[B, nq, H, nkv]` and bit-pack
(`benchmark/utils.py:83-84`). `select_blocks` does the whole step in CUDA and returns the four tensors that
`BatchFlashOmniFAWithRaggedKVWrapper.run`, `flashomni_gemm` and `flashomni_gemm_reduction` take."""

from __future__ import annotations

from typing import Tuple, Union

import torch

from . import _native

Threshold = Union[float, torch.Tensor]


def _threshold(t: Threshold, n: int, device, what: str) -> torch.Tensor:
    if isinstance(t, torch.Tensor):
        if t.numel() not in (1, n):
            raise ValueError(f"{what} must be a scalar or have {n} entries")
        return t.to(device=device, dtype=torch.float32).reshape(-1).expand(n).contiguous()
    return torch.full((n,), float(t), dtype=torch.float32, device=device)


def select_blocks(pooled_score: torch.Tensor, num_text_blocks: int, q_threshold: Threshold,
                  kv_threshold: Threshold, zero_inactive: bool = True
                  ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """pooled_score: fp32 CUDA tensor [B, H, n, n] (n q-blocks = n kv-blocks, the first `num_text_blocks` text).
    q_threshold: scalar or [B]; kv_threshold: scalar or [H] (cumulative softmax mass that may be switched off).
    Returns (sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr): uint8 bit streams
    (little-endian, one segment per request) and int32 byte indptrs."""
    if pooled_score.dim() != 4 or pooled_score.shape[2] != pooled_score.shape[3]:
        raise ValueError("pooled_score must be [B, H, n, n]")
    if pooled_score.dtype != torch.float32:
        raise ValueError("pooled_score must be float32")
    _native.require_cuda(pooled_score)
    s = pooled_score.contiguous()
    B, H, n, _ = s.shape
    if not 0 <= num_text_blocks <= n:
        raise ValueError("num_text_blocks out of range")
    dev = s.device
    lib = _native.load()
    qthr = _threshold(q_threshold, B, dev, "q_threshold")
    kthr = _threshold(kv_threshold, H, dev, "kv_threshold")
    info_seg = (n * H + 7) // 8
    kv_seg = (n * H * n + 7) // 8
    kv_alloc = (B * kv_seg + 3) // 4 * 4
    sparse_info = torch.empty(B * info_seg, dtype=torch.uint8, device=dev)
    sparse_kv = torch.empty(kv_alloc, dtype=torch.uint8, device=dev)
    ip = torch.empty(B + 1, dtype=torch.int32, device=dev)
    kp = torch.empty(B + 1, dtype=torch.int32, device=dev)
    scratch = torch.empty(lib.fo_select_blocks_scratch_bytes(B, n), dtype=torch.uint8, device=dev)
    rc = lib.fo_select_blocks(_native.ptr(s), B, H, n, int(num_text_blocks), _native.ptr(qthr), _native.ptr(kthr),
                              int(bool(zero_inactive)), _native.ptr(sparse_info), sparse_info.numel(),
                              _native.ptr(sparse_kv), sparse_kv.numel(), _native.ptr(ip), _native.ptr(kp),
                              _native.ptr(scratch), scratch.numel(), _native.current_stream(dev))
    _native.check(rc, "select_blocks")
    return sparse_info, sparse_kv[:B * kv_seg], ip, kp
