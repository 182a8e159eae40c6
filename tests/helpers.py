"""Shared helpers of the test-suite."""

from __future__ import annotations

import numpy as np
import torch

MAX_ABS = 2e-2   # bf16 outputs vs the fp32 oracle: max-abs bound of the benchmark contract
MEAN_ABS = 2e-3  # and mean-abs bound


def dev(x, device, dtype=None):
    if isinstance(x, np.ndarray):
        x = torch.from_numpy(x)
    return x.to(device=device, dtype=dtype) if dtype is not None else x.to(device)


def masks_to_device(m, device):
    return (dev(m.sparse_info, device), dev(m.sparse_kv_info, device), dev(m.info_indptr, device),
            dev(m.kv_info_indptr, device))


def bf16_ulp(x: torch.Tensor) -> torch.Tensor:
    """Size of one bf16 unit in the last place at |x| (8 significant bits)."""
    ax = x.abs().float().clamp_min(1e-30)
    return torch.exp2(torch.floor(torch.log2(ax)) - 7)


def assert_close_bf16(got: torch.Tensor, ref: torch.Tensor, what: str, max_abs=MAX_ABS, mean_abs=MEAN_ABS,
                      allow_ulp: float = 0.0):
    """max-abs <= 2e-2 and mean-abs <= 2e-3 against the fp32 oracle. `allow_ulp` widens the max-abs
    bound to that many bf16 ulps of the reference value where that is larger (outputs of magnitude > 4,
    whose rounding step alone exceeds 2e-2)."""
    got = got.float().cpu()
    ref = ref.float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    diff = (got - ref).abs()
    bound = torch.full_like(diff, max_abs)
    if allow_ulp > 0:
        bound = torch.maximum(bound, allow_ulp * bf16_ulp(ref))
    worst = (diff - bound).max().item()
    assert worst <= 0, f"{what}: max-abs {diff.max().item():.4g} exceeds bound by {worst:.4g}"
    assert diff.mean().item() <= mean_abs, f"{what}: mean-abs {diff.mean().item():.4g} > {mean_abs}"
