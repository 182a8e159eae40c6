"""CPU restatement of the block-selection step that produces the masks of the hot path (test infrastructure:
only tests/ and the smoke / baseline legs may import this package).

The reference generates its masks in `benchmark/test_attn_score.py:93-161`: from a pooled score tensor
`[B, H, nq, nkv]` (nq == nkv, the first T2T blocks are text)

* q-blocks: the text-to-image scores summed over heads and text rows, softmax over the image blocks, ascending
  sort, cumulative sum, `searchsorted(threshold, right=True)` lowest blocks are switched off for every head
  (`test_attn_score.py:100-110`, fill kernel `:52-61`);
* kv-blocks: per (b, h, image q-block) the row softmax over all kv blocks, the same sort / cumsum / searchsorted
  with a per-head threshold, the lowest blocks switched off (`:122-133`, fill kernel `:71-81`); text q rows keep
  everything;
* callers then transpose `[B, H, nq, nkv] -> [B, nq, H, nkv]` and bit-pack per batch (`benchmark/utils.py:83-84`).

`select_blocks` below states the same algorithm with arithmetic that a GPU can reproduce bit for bit:
exponentials by a fixed polynomial evaluated with separately rounded fp32 multiplies and adds (`det_exp2`),
masses accumulated as integers (exact and order-free), ties between equal masses broken by the block index. The
selection can differ from a float evaluation only where a cumulative mass falls within float rounding of the
threshold; `select_blocks_float` is the float evaluation in the reference's own operation order, used by the
tests to pin the restatement.
"""

from __future__ import annotations

import numpy as np

from .masks import packbits

_F = np.float32
_LOG2E = _F(1.4426950408889634)
_C = [_F(1.0), _F(0.6931471806), _F(0.2402265070), _F(0.0555041087), _F(0.0096181291), _F(0.0013333558)]
MASS_SHIFT = 31  # masses are floor(e * 2^31): e = 1 (the row maximum) is 2^31


def det_exp2_mass(x: np.ndarray) -> np.ndarray:
    """uint32 mass of every entry of a score row: floor(2^31 * exp(x - max(x))) with the exponential evaluated
    as 2^(n + f), n = rint(t), f = t - n, t = (x - max) * log2(e), 2^f by a degree-5 Horner polynomial whose
    multiplies and adds are rounded separately (no fused multiply-add), 2^n exact. Entries with t < -64 are 0."""
    x = np.asarray(x, dtype=_F)
    d = (x - x.max(axis=-1, keepdims=True)).astype(_F)
    t = (d * _LOG2E).astype(_F)
    small = t < _F(-64.0)
    t = np.where(small, _F(-64.0), t).astype(_F)
    n = np.rint(t).astype(_F)
    f = (t - n).astype(_F)
    p = np.full_like(f, _C[5])
    for c in (_C[4], _C[3], _C[2], _C[1], _C[0]):
        p = ((p * f).astype(_F) + c).astype(_F)
    e = np.ldexp(p, n.astype(np.int32)).astype(_F)
    m = np.minimum(np.floor(e.astype(np.float64) * float(1 << MASS_SHIFT)), float(1 << MASS_SHIFT)).astype(np.uint64)
    m = np.where(small, np.uint64(0), m)
    return m.astype(np.uint32)


def drop_lowest(mass: np.ndarray, threshold: float) -> np.ndarray:
    """For one row of masses: boolean array, True where the block is switched off. Blocks are taken in ascending
    (mass, index) order while the cumulative mass stays <= floor(threshold * total) (threshold as fp32, product
    in fp64): the integer form of `searchsorted(cumsum(sorted softmax), threshold, right=True)`."""
    mass = np.asarray(mass, dtype=np.uint64)
    n = mass.shape[0]
    total = int(mass.sum())
    limit = int(np.floor(np.float64(np.float32(threshold)) * np.float64(total)))
    order = np.lexsort((np.arange(n), mass))
    cum = np.cumsum(mass[order].astype(np.uint64))
    num = int(np.count_nonzero(cum <= np.uint64(max(limit, 0)))) if limit >= 0 else 0
    off = np.zeros(n, dtype=bool)
    off[order[:num]] = True
    return off


def text_to_image_scores(score_b: np.ndarray, t2t: int) -> np.ndarray:
    """[n_img] fp32: sum over heads (outer) and text q rows (inner) of score[h, q, t2t + j], accumulated
    sequentially in that order in fp32 (`test_attn_score.py:98-99` sums the same entries)."""
    H, nq, nkv = score_b.shape
    acc = np.zeros(nkv - t2t, dtype=_F)
    for h in range(H):
        for q in range(t2t):
            acc = (acc + score_b[h, q, t2t:].astype(_F)).astype(_F)
    return acc


def select_blocks(pooled_score: np.ndarray, num_text_blocks: int, q_threshold, kv_threshold,
                  zero_inactive: bool = True):
    """pooled_score [B, H, n, n] fp32. q_threshold: scalar or [B]; kv_threshold: scalar or [H].
    Returns (q_active uint8 [B, n, H], kv_kept uint8 [B, n, H, n]) in the hot path's index order.
    With `zero_inactive` the kv rows of switched-off q-blocks are zero (the reference's callers do that,
    `benchmark/test_flashomni_attention.py:201`)."""
    s = np.asarray(pooled_score, dtype=_F)
    B, H, nq, nkv = s.shape
    if nq != nkv:
        raise ValueError("block selection needs as many q-blocks as kv-blocks")
    t2t = int(num_text_blocks)
    qthr = np.broadcast_to(np.asarray(q_threshold, dtype=_F), (B,))
    kthr = np.broadcast_to(np.asarray(kv_threshold, dtype=_F), (H,))
    q_active = np.ones((B, nq, H), dtype=np.uint8)
    kv_kept = np.ones((B, nq, H, nkv), dtype=np.uint8)
    for b in range(B):
        if nkv > t2t and t2t > 0:
            off = drop_lowest(det_exp2_mass(text_to_image_scores(s[b], t2t)), float(qthr[b]))
            q_active[b, t2t:, :][off] = 0
        for h in range(H):
            mass = det_exp2_mass(s[b, h, t2t:, :])
            for i in range(nq - t2t):
                kv_kept[b, t2t + i, h, drop_lowest(mass[i], float(kthr[h]))] = 0
        if zero_inactive:
            kv_kept[b] *= q_active[b][:, :, None]
    return q_active, kv_kept


def pack_selection(q_active: np.ndarray, kv_kept: np.ndarray):
    """Packed byte streams and byte indptrs of the hot path (little-endian bits, one segment per request)."""
    B = q_active.shape[0]
    info, kv, ip, kp = [], [], [0], [0]
    for b in range(B):
        a = packbits(q_active[b].reshape(-1), "little")
        k = packbits(kv_kept[b].reshape(-1), "little")
        info.append(a); kv.append(k)
        ip.append(ip[-1] + len(a)); kp.append(kp[-1] + len(k))
    return (np.concatenate(info), np.concatenate(kv), np.asarray(ip, dtype=np.int32), np.asarray(kp, dtype=np.int32))


def select_blocks_float(pooled_score, num_text_blocks: int, q_threshold, kv_threshold, zero_inactive: bool = True):
    """The float evaluation in the reference's operation order (torch CPU, fp32): sum, softmax, ascending sort,
    cumsum, searchsorted(right=True), scatter of zeros (`test_attn_score.py:93-133`). Same outputs as
    `select_blocks`."""
    import torch
    s = torch.as_tensor(np.asarray(pooled_score, dtype=np.float32))
    B, H, nq, nkv = s.shape
    t2t = int(num_text_blocks)
    qthr = torch.as_tensor(np.broadcast_to(np.asarray(q_threshold, dtype=np.float32), (B,)).copy())
    kthr = torch.as_tensor(np.broadcast_to(np.asarray(kv_threshold, dtype=np.float32), (H,)).copy())
    q_active = torch.ones((B, H, nq), dtype=torch.uint8)
    kv_kept = torch.ones((B, H, nq, nkv), dtype=torch.uint8)
    if nkv > t2t and t2t > 0:
        t2i = s[:, :, :t2t, t2t:].sum(dim=[1, 2]).softmax(-1)
        srt = torch.sort(t2i, dim=-1, descending=False, stable=True)
        num = torch.searchsorted(torch.cumsum(srt.values, -1), qthr.view(B, 1).contiguous(), right=True).squeeze(-1)
        for b in range(B):
            q_active[b, :, t2t + srt.indices[b, :int(num[b])]] = 0
    img = s[:, :, t2t:, :].softmax(-1)
    srt = torch.sort(img, dim=-1, descending=False, stable=True)
    thr = kthr.view(1, H, 1, 1).expand(B, -1, nq - t2t, 1).contiguous()
    num = torch.searchsorted(torch.cumsum(srt.values, -1), thr, right=True).squeeze(-1)
    for b in range(B):
        for h in range(H):
            for i in range(nq - t2t):
                kv_kept[b, h, t2t + i, srt.indices[b, h, i, :int(num[b, h, i])]] = 0
    qa = q_active.permute(0, 2, 1).contiguous().numpy()
    kk = kv_kept.permute(0, 2, 1, 3).contiguous().numpy()
    if zero_inactive:
        kk = kk * qa[:, :, :, None]
    return qa, kk
