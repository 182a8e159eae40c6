"""CPU: the floating-point oracles against independent dense formulas (small cases)."""

import math

import numpy as np
import torch

from oracle import attention as oa
from oracle import gemm as og
from flashomni_b200 import workloads as wl


def _inputs(lens_q, lens_kv, H, D, seed, density=0.6):
    qo = np.concatenate([[0], np.cumsum(lens_q)]); kv = np.concatenate([[0], np.cumsum(lens_kv)])
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(int(qo[-1]), H, D, generator=g)
    k = torch.randn(int(kv[-1]), H, D, generator=g)
    v = torch.randn(int(kv[-1]), H, D, generator=g)
    rng = np.random.default_rng(seed)
    qa, kk = [], []
    for lq, lk in zip(lens_q, lens_kv):
        nq, nkv = -(-lq // 128), -(-lk // 128)
        qa.append((rng.random((nq, H)) < density).astype(np.uint8))
        kk.append((rng.random((nq, H, nkv)) < density).astype(np.uint8))
    return q, k, v, qo, kv, wl.pack_masks(qa, kk)


def test_blockwise_equals_dense_masked_softmax():
    q, k, v, qo, kv, m = _inputs([256, 200], [384, 130], 2, 16, seed=1)
    prior = torch.randn(q.shape[0], 2, 16)
    a = oa.sparse_attention(q, k, v, qo, kv, m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr,
                            out_prior=prior, dtype=torch.float64)
    b = oa.dense_masked_attention(q, k, v, qo, kv, m.q_active, m.kv_kept, out_prior=prior)
    assert torch.allclose(a, b, atol=1e-10)


def test_skipped_rows_keep_prior_and_empty_rows_are_zero():
    q, k, v, qo, kv, _ = _inputs([256], [256], 1, 8, seed=2)
    qa = [np.array([[1], [0]], dtype=np.uint8)]
    kk = [np.zeros((2, 1, 2), dtype=np.uint8)]
    m = wl.pack_masks(qa, kk)
    prior = torch.full((256, 1, 8), 7.0)
    o, lse = oa.sparse_attention(q, k, v, qo, kv, m.sparse_info, m.sparse_kv_info, m.info_indptr,
                                 m.kv_info_indptr, out_prior=prior, return_lse=True)
    assert torch.all(o[:128] == 0) and torch.all(o[128:] == 7.0)
    assert torch.all(lse[:128] == -5e4)


def test_is_full_equals_plain_softmax_and_lse_is_base2():
    q, k, v, qo, kv, _ = _inputs([130], [300], 2, 8, seed=3)
    o, lse = oa.sparse_attention(q, k, v, qo, kv, is_full=True, return_lse=True, dtype=torch.float64)
    s = torch.einsum("qhd,khd->hqk", q.double(), k.double()) / math.sqrt(8)
    ref = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v.double())
    assert torch.allclose(o, ref, atol=1e-10)
    assert torch.allclose(lse, (torch.logsumexp(s, -1) / math.log(2)).T, atol=1e-9)


def test_soft_cap_matches_the_formula_and_zero_disables_it():
    """logits = cap * tanh(q.k * sm_scale / cap) before the softmax (reference: variants.cuh:47-50,72-74)."""
    q, k, v, qo, kv, _ = _inputs([130], [300], 2, 8, seed=5)
    cap = 0.8
    o, lse = oa.sparse_attention(q, k, v, qo, kv, is_full=True, return_lse=True, dtype=torch.float64, logits_soft_cap=cap)
    s = torch.einsum("qhd,khd->hqk", q.double(), k.double()) / math.sqrt(8)
    s = cap * torch.tanh(s / cap)
    ref = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v.double())
    assert torch.allclose(o, ref, atol=1e-10)
    assert torch.allclose(lse, (torch.logsumexp(s, -1) / math.log(2)).T, atol=1e-9)
    o0 = oa.sparse_attention(q, k, v, qo, kv, is_full=True, dtype=torch.float64, logits_soft_cap=0.0)
    assert torch.equal(o0, oa.sparse_attention(q, k, v, qo, kv, is_full=True, dtype=torch.float64))


def test_gemm_q_inactive_tiles_keep_prior():
    m = wl.flux_masks(1, 2, 3, 3, 0.5, seed=4, text_blocks=1)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, 384, 64, generator=g); w = torch.randn(256, 64, generator=g)
    prior = torch.randn(1, 384, 256, generator=g); bias = torch.randn(256, generator=g)
    y = og.gemm_q(x, w, 2, m.sparse_info, m.info_indptr, 0, bias, prior)
    dense = x @ w.T + bias
    for iy in range(3):
        for h in range(2):
            blk = (slice(0, 1), slice(iy * 128, iy * 128 + 128), slice(h * 128, h * 128 + 128))
            exp = dense[blk] if m.q_active[0][iy, h] else prior[blk]
            assert torch.allclose(y[blk], exp, atol=1e-5)


def test_gemm_o_cache_plus_active_is_dense():
    # the reference's own check: benchmark/test_flashomni_gemm_o.py:73-87
    m = wl.flux_masks(2, 4, 3, 3, 0.5, seed=6, text_blocks=1)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 384, 4 * 64, generator=g); w = torch.randn(256, 4 * 64, generator=g)
    bias = torch.randn(256, generator=g)
    cache = og.gemm_o(x, w, 4, m.sparse_info, m.info_indptr, 0, bias, is_for_cache=True)
    y = og.gemm_o(x, w, 4, m.sparse_info, m.info_indptr, 0, cache, is_for_cache=False)
    assert torch.allclose(y, x @ w.T + bias, atol=1e-4)
