"""Bit packing of the block masks (drop-in for flashomni/quantization.py:68-159)."""

from __future__ import annotations

from typing import Tuple

import torch

from . import _native


def _little(bitorder: str) -> int:
    if bitorder not in ("big", "little"):
        raise ValueError(f"bitorder must be 'big' or 'little', got {bitorder!r}")
    return 1 if bitorder == "little" else 0


def _as_bytes(x: torch.Tensor) -> torch.Tensor:
    x = x.contiguous().view(-1)
    if x.dtype == torch.bool:
        return x.view(torch.uint8)
    if x.dtype in (torch.uint8, torch.int8):
        return x.view(torch.uint8)
    return (x != 0).view(torch.uint8)


def packbits(x: torch.Tensor, bitorder: str = "big") -> torch.Tensor:
    """Packs a 1-D binary-valued tensor into bits, same semantics as numpy.packbits
    (reference: flashomni/quantization.py:68-99)."""
    little = _little(bitorder)
    _native.require_cuda(x)
    xb = _as_bytes(x)
    n = xb.numel()
    y = torch.empty((n + 7) // 8, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        rc = _native.load().fo_packbits(_native.ptr(xb), n, little, _native.ptr(y),
                                        _native.current_stream(x.device))
    _native.check(rc, "packbits")
    return y


def segment_packbits(x: torch.Tensor, indptr: torch.Tensor, bitorder: str = "big") -> Tuple[torch.Tensor, torch.Tensor]:
    """Packs each segment x[indptr[i]:indptr[i+1]] separately; returns (y, new_indptr) with
    new_indptr[i+1]-new_indptr[i] == ceil(len_i/8) (reference: flashomni/quantization.py:102-159,
    including its one host synchronisation to size the output)."""
    little = _little(bitorder)
    _native.require_cuda(x)
    seglen = indptr[1:] - indptr[:-1]
    packed_len = (seglen + 7) // 8
    indptr_new = torch.zeros(len(indptr), dtype=indptr.dtype, device=indptr.device)
    indptr_new[1:] = torch.cumsum(packed_len, 0)
    output_nnzs = int(indptr_new[-1].item())
    device = x.device
    indptr32 = indptr.to(device=device, dtype=torch.int32).contiguous()
    indptr_new = indptr_new.to(device=device, dtype=torch.int32).contiguous()
    xb = _as_bytes(x)
    y = torch.empty(output_nnzs, dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        rc = _native.load().fo_segment_packbits(_native.ptr(xb), _native.ptr(indptr32), _native.ptr(indptr_new),
                                                len(indptr) - 1, output_nnzs, little, _native.ptr(y),
                                                _native.current_stream(device))
    _native.check(rc, "segment_packbits")
    return y, indptr_new
