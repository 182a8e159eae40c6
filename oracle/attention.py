"""CPU oracle (test infrastructure): block-sparse attention in fp32 torch.

Restates what `BatchFlashOmniFAWithRaggedKVKernel` computes
(include/flashomni/attention/prefill.cuh:1203-1531) the way the reference's own check builds its
comparison value: dense softmax attention with the masked blocks excluded
(benchmark/test_flashomni_attention.py:197-199,231). Two forms are given: a blockwise gather per
(head, q-block) (fast; used for parity and as the timed CPU baseline) and a dense boolean-mask
softmax (slow; used to validate the blockwise form on small cases).

Semantics kept from the kernel:
  * q-block bit 0  -> the rows of `out` (and `lse`) keep their prior contents (prefill.cuh:1291-1293)
  * active q-block with no kept kv-block -> zeros, lse = -5e4 (math.cuh:32, prefill.cuh:944-946)
  * ragged tail: kv columns >= kv_len are excluded (prefill.cuh:715-757)
  * `is_full` ignores both masks (prefill.cuh:1284,1383,1434)
  * lse is base-2: log2(sum exp2(s*log2e - m)) + m with s = q.k*sm_scale (prefill.cuh:1517-1520)
"""

from __future__ import annotations

import math

import numpy as np
import torch

from . import masks as _masks

NEG_INF_LSE = -5e4


def sparse_attention(q, k, v, qo_indptr, kv_indptr, sparse_info=None, sparse_kv_info=None,
                     info_indptr=None, kv_info_indptr=None, sbq: int = 128, sbkv: int = 128,
                     is_full: bool = False, sm_scale: float | None = None, out_prior=None,
                     lse_prior=None, return_lse: bool = False, head_begin: int = 0, num_mask_heads=None,
                     dtype=torch.float32, logits_soft_cap: float = 0.0, causal: bool = False, custom_mask=None):
    """q [Tq, H, D], k/v [Tkv, Hkv, D] (any float dtype, computed in `dtype`). Returns fp32 `out`
    (and base-2 `lse`). With `logits_soft_cap` > 0 the logits are cap * tanh(q.k * sm_scale / cap)
    (include/flashomni/attention/variants.cuh:47-50,72-74). `out_prior` supplies the rows of skipped q-blocks (zeros if None, as
    flashomni/attention.py:778-781 allocates). With `causal`, kv position j of a request is visible to q token i only if
    j <= i + kv_len - q_len (prefill.cuh:746-751); a row without any visible kept position gives zeros and lse = -5e4
    (the reference fills masked logits with -5e4, not -inf, and would average V there: a degenerate case that the
    golden cases avoid). `custom_mask`: per request a boolean [q_len, kv_len] array; position (i, j) is visible iff it
    is set (MaskMode::kCustom, variants.cuh:76-87); it takes the place of `causal`. kv head `hk` reads mask head `head_begin + hk` (of `num_mask_heads`)."""
    Tq, H, D = q.shape
    Hkv = k.shape[1]
    group = H // Hkv
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    qf, kf, vf = q.to(dtype), k.to(dtype), v.to(dtype)
    out = torch.zeros(Tq, H, v.shape[-1], dtype=dtype) if out_prior is None else out_prior.to(dtype).clone()
    lse = None
    if return_lse:
        lse = torch.zeros(Tq, H, dtype=dtype) if lse_prior is None else lse_prior.to(dtype).clone()
    qo = np.asarray(qo_indptr, dtype=np.int64)
    kv = np.asarray(kv_indptr, dtype=np.int64)
    if not is_full:
        sparse_info = np.asarray(sparse_info, dtype=np.uint8)
        sparse_kv_info = np.asarray(sparse_kv_info, dtype=np.uint8)
    # Grouped heads (H > Hkv): the reference's kernel works on packed rows, a packed row being a (token, q head of
    # the group) pair in token-major order; a q tile is 128 packed rows of ONE kv head and the masks hold one bit per
    # (packed block, kv head) (prefill.cuh:1283-1291: `qo_tile_idx * CTA_TILE_Q / sbq * num_kv_heads + kv_head_idx`).
    # A mask q-block therefore covers sbq / group tokens of all `group` q heads of a kv head. group = 1 is the plain
    # (sbq tokens, head) layout.
    if sbq % group != 0:
        raise ValueError("sbq must be a multiple of num_qo_heads / num_kv_heads")
    qtok = sbq // group
    if num_mask_heads is None:
        num_mask_heads = Hkv
    for b in range(len(qo) - 1):
        q0, q1, k0, k1 = int(qo[b]), int(qo[b + 1]), int(kv[b]), int(kv[b + 1])
        nq = -(-(q1 - q0) // qtok)
        nkv = -(-(k1 - k0) // sbkv)
        if not is_full:
            qa = _masks.unpack_segment(sparse_info, int(info_indptr[b]),
                                       nq * num_mask_heads).reshape(nq, num_mask_heads)
            kk = _masks.unpack_segment(sparse_kv_info, int(kv_info_indptr[b]),
                                       nq * num_mask_heads * nkv).reshape(nq, num_mask_heads, nkv)
        for hk in range(Hkv):
            mh = head_begin + hk
            for qb in range(nq):
                if not is_full and not qa[qb, mh]:
                    continue
                r0, r1 = q0 + qb * qtok, min(q0 + (qb + 1) * qtok, q1)
                kept = np.arange(nkv) if is_full else np.nonzero(kk[qb, mh])[0]
                for h in range(hk * group, (hk + 1) * group):
                    if len(kept) == 0:
                        out[r0:r1, h] = 0
                        if return_lse:
                            lse[r0:r1, h] = NEG_INF_LSE
                        continue
                    cols = np.concatenate([np.arange(k0 + j * sbkv, min(k0 + (j + 1) * sbkv, k1)) for j in kept])
                    cols_t = torch.from_numpy(cols)
                    s = (qf[r0:r1, h] @ kf[cols_t, hk].T) * sm_scale
                    if logits_soft_cap > 0:
                        s = torch.tanh(s / logits_soft_cap) * logits_soft_cap
                    if custom_mask is not None:
                        cm = torch.from_numpy(np.asarray(custom_mask[b], dtype=bool)[r0 - q0:r1 - q0][:, cols - k0])
                        s = s.masked_fill(~cm, float("-inf"))
                    elif causal:
                        qi = torch.arange(r0 - q0, r1 - q0).view(-1, 1)
                        kj = torch.from_numpy(cols - k0).view(1, -1)
                        s = s.masked_fill(kj > qi + ((k1 - k0) - (q1 - q0)), float("-inf"))
                    p = torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0)   # a row with nothing visible: zeros
                    out[r0:r1, h] = p @ vf[cols_t, hk]
                    if return_lse:
                        l2 = torch.logsumexp(s, dim=-1) * math.log2(math.e)
                        lse[r0:r1, h] = torch.where(torch.isinf(l2), torch.full_like(l2, NEG_INF_LSE), l2)
    return (out, lse) if return_lse else out


def dense_masked_attention(q, k, v, qo_indptr, kv_indptr, q_active, kv_kept, sbq=128, sbkv=128,
                           sm_scale=None, out_prior=None):
    """Dense boolean-mask formulation (benchmark/test_flashomni_attention.py:197-199,231) on the
    unpacked masks: `q_active[b]` is [nq, H], `kv_kept[b]` is [nq, H, nkv]. fp64, small cases only."""
    Tq, H, D = q.shape
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    out = torch.zeros(Tq, H, v.shape[-1], dtype=torch.float64) if out_prior is None \
        else out_prior.to(torch.float64).clone()
    qd, kd, vd = q.double(), k.double(), v.double()
    for b in range(len(qo_indptr) - 1):
        q0, q1, k0, k1 = int(qo_indptr[b]), int(qo_indptr[b + 1]), int(kv_indptr[b]), int(kv_indptr[b + 1])
        lq, lk = q1 - q0, k1 - k0
        for h in range(H):
            kept = torch.from_numpy(np.asarray(kv_kept[b][:, h, :], dtype=bool))
            elem = kept.repeat_interleave(sbq, 0).repeat_interleave(sbkv, 1)[:lq, :lk]
            act = torch.from_numpy(np.asarray(q_active[b][:, h], dtype=bool)).repeat_interleave(sbq)[:lq]
            s = (qd[q0:q1, h] @ kd[k0:k1, h].T) * sm_scale
            s = s.masked_fill(~elem, float("-inf"))
            p = torch.softmax(s, dim=-1)
            p = torch.nan_to_num(p, nan=0.0)  # rows with nothing kept -> zeros
            o = p @ vd[k0:k1, h]
            rows = torch.nonzero(act).flatten() + q0
            out[rows, h] = o[act]
    return out
