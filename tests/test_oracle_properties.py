"""Property checks of the CPU statements of the mask step (hypothesis, CPU only): whatever the ragged shapes,
densities and head windows, the work lists hold every kept block exactly once and in the documented order."""

import numpy as np
from hypothesis import given, settings, strategies as st

from flashomni_b200 import workloads as wl
from oracle import masks as om


@st.composite
def ragged_masks(draw):
    B = draw(st.integers(1, 3))
    H = draw(st.integers(1, 5))
    lens_q = [draw(st.integers(1, 700)) for _ in range(B)]
    lens_kv = [draw(st.integers(1, 700)) for _ in range(B)]
    seed = draw(st.integers(0, 2 ** 16))
    dq = draw(st.sampled_from([0.0, 0.3, 0.7, 1.0]))
    dk = draw(st.sampled_from([0.0, 0.4, 1.0]))
    rng = np.random.default_rng(seed)
    qa = [(rng.random((-(-a // 128), H)) < dq).astype(np.uint8) for a in lens_q]
    kk = [(rng.random((-(-a // 128), H, -(-b // 128))) < dk).astype(np.uint8) for a, b in zip(lens_q, lens_kv)]
    hb = draw(st.integers(0, H - 1))
    hc = draw(st.integers(1, H - hb))
    return lens_q, lens_kv, H, qa, kk, hb, hc


@settings(max_examples=60, deadline=None)
@given(ragged_masks())
def test_compaction_lists_cover_the_masks_exactly(case):
    lens_q, lens_kv, H, qa, kk, hb, hc = case
    qo = np.concatenate([[0], np.cumsum(lens_q)])
    kv = np.concatenate([[0], np.cumsum(lens_kv)])
    m = wl.pack_masks(qa, kk)
    out = om.compact(m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr, qo, kv, H, 128, 128, hb, hc)
    items, ptr, idx, order = out["items"], out["kv_indptr"], out["kv_idx"], out["order"]
    # one item per active (b, qb, h) of the head window, ascending in (b, qb, h)
    want = [(b, h, qb) for b in range(len(lens_q)) for qb in range(qa[b].shape[0]) for h in range(hb, hb + hc)
            if qa[b][qb, h]]
    assert [tuple(r[:3]) for r in items.tolist()] == want
    # each item's list is exactly its kept kv-blocks, ascending
    for i, (b, h, qb, n) in enumerate(items.tolist()):
        kept = np.nonzero(kk[b][qb, h])[0]
        assert n == len(kept) and np.array_equal(idx[ptr[i]:ptr[i + 1]], kept)
    assert ptr[-1] == len(idx) == sum(int(kk[b][qb, h].sum()) for b, h, qb in want)
    # the processing order is a permutation, grouped by (b, group of heads) ascending; inside a group the longest
    # lists come first (these small cases are all below the bucket limit), ties in list order
    assert sorted(order.tolist()) == list(range(len(items)))
    max_nkv = max(-(-int(x) // 128) for x in lens_kv)
    hpg, by_length = om.order_groups(len(lens_q), hc, max_nkv)
    assert by_length
    keys = [(items[i][0], (items[i][1] - hb) // hpg, -items[i][3], i) for i in order.tolist()]
    assert keys == sorted(keys)


@settings(max_examples=60, deadline=None)
@given(st.integers(1, 3), st.integers(1, 6), st.integers(1, 6), st.integers(0, 2 ** 16),
       st.sampled_from([0.0, 0.5, 1.0]))
def test_gemm_q_records_pair_the_active_tiles(B, mt, H, seed, density):
    rng = np.random.default_rng(seed)
    qa = [(rng.random((mt, H)) < density).astype(np.uint8) for _ in range(B)]
    kk = [np.ones((mt, H, mt), np.uint8) for _ in range(B)]
    m = wl.pack_masks(qa, kk)
    tiles = om.gemm_q_tiles(m.sparse_info, m.info_indptr, B, mt * 128, H * 128, H)
    recs = om.gemm_q_tile_pairs(m.sparse_info, m.info_indptr, B, mt * 128, H * 128, H)
    assert [tuple(t) for t in tiles.tolist()] == [(b, iy, h) for b in range(B) for iy in range(mt) for h in range(H)
                                                   if qa[b][iy, h]]
    covered = []
    seen_single = False
    for b, iy, ix0, ix1 in recs.tolist():
        if ix1 < 0:
            seen_single = True
            covered.append((b, iy, ix0))
        else:
            assert not seen_single and ix0 < ix1      # two-block records come first
            covered += [(b, iy, ix0), (b, iy, ix1)]
    assert sorted(covered) == [tuple(t) for t in tiles.tolist()]
    # at most one single-block record per row block
    singles = [(b, iy) for b, iy, _, ix1 in recs.tolist() if ix1 < 0]
    assert len(singles) == len(set(singles))
