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


def load_selection_golden():
    """Cases of tests/golden/reference_selection.npz (masks made by the reference's own torch + Triton selection
    path on a GPU, see tests/golden/make_selection_golden.py): list of dicts."""
    import json
    import os
    import numpy as np
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_selection.npz")
    z = np.load(path)
    names = json.loads(bytes(z["names"]).decode())
    cases = []
    for nm in names:
        seed, B, H, n, t2t = (int(v) for v in z[f"{nm}.meta"])
        cases.append(dict(name=nm, B=B, H=H, n=n, t2t=t2t, score=z[f"{nm}.score"], q_threshold=z[f"{nm}.q_threshold"],
                          kv_threshold=z[f"{nm}.kv_threshold"], sparse_info=z[f"{nm}.sparse_info"],
                          sparse_kv_info=z[f"{nm}.sparse_kv_info"], q_margin=z[f"{nm}.q_margin"],
                          kv_margin=z[f"{nm}.kv_margin"]))
    return cases, json.loads(bytes(z["timing_us"]).decode())


# A cumulative softmax mass this close to the threshold may fall on either side of it under another summation
# order (the reference sums in fp32 on the GPU; the restatement accumulates exact integers): such rows are
# allowed to differ from the golden masks by the blocks at the boundary, every other row must be identical.
SELECTION_MARGIN = 2e-6


def check_selection_against_golden(case, q_active, kv_kept):
    """q_active [B, n, H], kv_kept [B, n, H, n] (zero_inactive=False) against one golden case, which stores the
    reference's layouts [B, H, n] and [B, H, n, n]. Returns the number of rows that differ under the margin rule."""
    import numpy as np
    B, H, n, t2t = case["B"], case["H"], case["n"], case["t2t"]
    gq = case["sparse_info"].transpose(0, 2, 1)            # -> [B, n, H]
    gk = case["sparse_kv_info"].transpose(0, 2, 1, 3)      # -> [B, n, H, n]
    exempt = 0
    for b in range(B):
        if not np.array_equal(q_active[b], gq[b]):
            assert case["q_margin"][b] < SELECTION_MARGIN, f"{case['name']}: q-blocks of request {b}"
            assert np.abs(q_active[b].astype(int).sum(0) - gq[b].astype(int).sum(0)).max() <= 1
            exempt += 1
        assert np.array_equal(kv_kept[b, :t2t], gk[b, :t2t])
        for h in range(H):
            for i in range(n - t2t):
                got, ref = kv_kept[b, t2t + i, h], gk[b, t2t + i, h]
                if not np.array_equal(got, ref):
                    assert case["kv_margin"][b, h, i] < SELECTION_MARGIN, f"{case['name']}: kv row b{b} h{h} q{t2t + i}"
                    assert abs(int(got.sum()) - int(ref.sum())) <= 1
                    exempt += 1
    return exempt
