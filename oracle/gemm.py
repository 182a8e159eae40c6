"""CPU oracle (test infrastructure): GEMM-Q and GEMM-O in fp32 torch.

GEMM-Q (include/flashomni/gemm/w16a16/gemm.cuh:27-228, csrc/gemm.cu:24-59): for every 128x128 output
tile whose (q-block, head) bit is 1, Y = bias + X W^T; other tiles keep their prior contents. The
reference's own check builds the same value from nn.Linear with inactive tiles masked
(benchmark/test_flashomni_gemm_q.py:29-36,78).

GEMM-O (include/flashomni/gemm/w16a16/gemm_reduction.cuh:27-276): every output tile is written,
Y = init + sum over selected heads of X[:, hD:(h+1)D] W[:, hD:(h+1)D]^T with selected = bit 1
(`is_for_cache=False`) or bit 0 (`True`); init = cache [B,M,N] / 1-D bias / 0 (:77-95). The reference's
check is cache pass + active pass == dense linear (benchmark/test_flashomni_gemm_o.py:73-87).
"""

from __future__ import annotations

import numpy as np
import torch

from . import masks as _masks


def gemm_q(x, w, num_heads, sparse_info=None, info_indptr=None, num_text_tokens=0, bias=None,
           out_prior=None, sparse_q_size=128, is_full=False, head_begin=0, head_dim=None,
           dtype=torch.float32):
    """x [B, M, K], w [N, K]; returns fp32 [B, M, N]. Inactive tiles = `out_prior` (zeros if None)."""
    B, M, K = x.shape
    N = w.shape[0]
    if head_dim is None:
        head_dim = N // num_heads
    y_full = x.to(dtype) @ w.to(dtype).T
    if bias is not None:
        y_full = y_full + bias.to(dtype)[None, None, :]
    if is_full:
        return y_full
    out = torch.zeros(B, M, N, dtype=dtype) if out_prior is None else out_prior.to(dtype).clone()
    tiles = _masks.gemm_q_tiles(np.asarray(sparse_info, dtype=np.uint8), info_indptr, B, M, N, num_heads,
                                sparse_q_size, num_text_tokens, False, head_begin, head_dim)
    for b, iy, ix in tiles:
        out[b, iy * 128:(iy + 1) * 128, ix * 128:(ix + 1) * 128] = \
            y_full[b, iy * 128:(iy + 1) * 128, ix * 128:(ix + 1) * 128]
    return out


def gemm_o(x, w, num_heads, sparse_info, info_indptr, num_text_tokens=0, bias=None, is_for_cache=False,
           sparse_q_size=128, head_begin=0, head_dim=None, dtype=torch.float32):
    """x [B, M, K], w [N, K]; returns fp32 [B, M, N]."""
    B, M, K = x.shape
    N = w.shape[0]
    if head_dim is None:
        head_dim = K // num_heads
    xf, wf = x.to(dtype), w.to(dtype)
    if bias is None:
        out = torch.zeros(B, M, N, dtype=dtype)
    elif is_for_cache:
        out = bias.to(dtype).reshape(1, 1, N).expand(B, M, N).clone()
    else:
        out = bias.to(dtype).reshape(B, M, N).clone()
    indptr, heads, _ = _masks.gemm_o_rows(np.asarray(sparse_info, dtype=np.uint8), info_indptr, B, M, K,
                                          num_heads, sparse_q_size, num_text_tokens, is_for_cache,
                                          head_begin, head_dim)
    r = 0
    for b in range(B):
        for iy in range(M // 128):
            for h in heads[indptr[r]:indptr[r + 1]]:
                h = int(h)
                out[b, iy * 128:(iy + 1) * 128] += \
                    xf[b, iy * 128:(iy + 1) * 128, h * head_dim:(h + 1) * head_dim] @ \
                    wf[:, h * head_dim:(h + 1) * head_dim].T
            r += 1
    return out
