"""Block selection on the GPU: bit-exact against the CPU statement, and usable by the hot path as is."""

import numpy as np
import pytest
import torch

import flashomni_b200 as fo
from oracle import select as osel

pytestmark = pytest.mark.gpu


def _run(s, t2t, qthr, kthr, zero_inactive, device):
    out = fo.select_blocks(torch.from_numpy(s).to(device), t2t, qthr, kthr, zero_inactive=zero_inactive)
    torch.cuda.synchronize()
    return [t.cpu().numpy() for t in out]


@pytest.mark.parametrize("B,H,n,t2t", [(1, 2, 5, 2), (2, 3, 36, 4), (1, 4, 77, 3), (2, 24, 36, 4), (1, 2, 604, 4),
                                       (3, 1, 33, 0), (1, 3, 40, 40)])
@pytest.mark.parametrize("zero_inactive", [True, False])
def test_bit_exact(cuda_device, B, H, n, t2t, zero_inactive):
    rng = np.random.default_rng(1000 * n + H)
    s = (rng.standard_normal((B, H, n, n)) * 1.5).astype(np.float32)
    qthr = rng.uniform(0.05, 0.5, B).astype(np.float32)
    kthr = rng.uniform(0.05, 0.6, H).astype(np.float32)
    info, kv, ip, kp = _run(s, t2t, torch.from_numpy(qthr), torch.from_numpy(kthr), zero_inactive, cuda_device)
    qa, kk = osel.select_blocks(s, t2t, qthr, kthr, zero_inactive=zero_inactive)
    rinfo, rkv, rip, rkp = osel.pack_selection(qa, kk)
    assert np.array_equal(ip, rip) and np.array_equal(kp, rkp)
    assert np.array_equal(info, rinfo)
    assert np.array_equal(kv, rkv)


def test_ties_and_extremes(cuda_device):
    n = 64
    s = np.zeros((1, 2, n, n), dtype=np.float32)          # all scores equal: ties broken by block index
    s[0, 1, :, ::2] = -200.0                                # masses that round to zero are switched off first
    for thr in (0.0, 0.25, 1.0):
        info, kv, ip, kp = _run(s, 2, thr, thr, False, cuda_device)
        qa, kk = osel.select_blocks(s, 2, thr, thr, zero_inactive=False)
        rinfo, rkv, _, _ = osel.pack_selection(qa, kk)
        assert np.array_equal(info, rinfo) and np.array_equal(kv, rkv)


def test_feeds_the_hot_path(cuda_device):
    """The emitted tensors go straight into the attention wrapper; the result equals the run on masks packed
    from the CPU statement."""
    from flashomni_b200 import workloads as wl
    from helpers import dev
    B, H, n, D = 1, 4, 8, 128
    S = n * 128
    rng = np.random.default_rng(7)
    s = rng.standard_normal((B, H, n, n)).astype(np.float32)
    masks = fo.select_blocks(torch.from_numpy(s).to(cuda_device), 1, 0.3, 0.4)
    qa, kk = osel.select_blocks(s, 1, 0.3, 0.4)
    ref_masks = [torch.from_numpy(a).to(cuda_device) for a in osel.pack_selection(qa, kk)]
    q, k, v = (dev(wl.randn_bf16((S, H, D), 20 + i), cuda_device) for i in range(3))
    indptr = torch.tensor([0, S], dtype=torch.int32, device=cuda_device)
    w = fo.BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1 << 20, dtype=torch.uint8, device=cuda_device))
    w.plan(indptr, indptr, H, H, D, q_data_type=torch.bfloat16)
    a = w.run(q, k, v, *masks).clone()
    b = w.run(q, k, v, *ref_masks)
    w.check_status()
    assert torch.equal(a, b)


def test_matches_the_reference_masks(cuda_device):
    """fo_select_blocks against the masks the reference's own torch + Triton path produced
    (tests/golden/reference_selection.npz), same rule for rows at the threshold as the CPU statement's test."""
    from helpers import check_selection_against_golden, load_selection_golden
    from oracle.masks import unpack_segment
    cases, _ = load_selection_golden()
    for c in cases:
        B, H, n = c["B"], c["H"], c["n"]
        info, kv, ip, kp = _run(c["score"], c["t2t"], torch.from_numpy(c["q_threshold"]),
                                torch.from_numpy(c["kv_threshold"]), False, cuda_device)
        qa = np.stack([unpack_segment(info, int(ip[b]), n * H).reshape(n, H) for b in range(B)])
        kk = np.stack([unpack_segment(kv, int(kp[b]), n * H * n).reshape(n, H, n) for b in range(B)])
        check_selection_against_golden(c, qa, kk)
