"""CPU: the mask oracle against the reference's known-answer vectors and against numpy."""

import numpy as np
import pytest

from oracle import masks as om
from flashomni_b200 import workloads as wl


def test_packbits_kat_from_reference_docstring():
    # flashomni/quantization.py:90-93
    x = np.array([1, 0, 1, 1, 0, 0, 1, 1], dtype=np.uint8)
    assert om.packbits(x, "big").tolist() == [0b10110011]
    assert om.packbits(x, "little").tolist() == [0b11001101]


def test_segment_packbits_kat_from_reference_docstring():
    # flashomni/quantization.py:133-138
    x = np.array([1, 0, 1, 1, 0, 0, 1, 1, 1, 0, 1], dtype=np.uint8)
    y, ip = om.segment_packbits(x, np.array([0, 4, 7, 11]), "big")
    assert y.tolist() == [0b10110000, 0b100000, 0b11010000]
    assert ip.tolist() == [0, 1, 2, 3]


@pytest.mark.parametrize("order", ["big", "little"])
def test_segment_packbits_matches_numpy(order):
    rng = np.random.default_rng(0)
    lens = [0, 1, 7, 8, 9, 63, 64, 65, 1000]
    indptr = np.concatenate([[0], np.cumsum(lens)])
    x = rng.integers(0, 2, indptr[-1]).astype(np.uint8)
    y, ip = om.segment_packbits(x, indptr, order)
    for i, n in enumerate(lens):
        ref = np.packbits(x[indptr[i]:indptr[i + 1]].astype(bool), bitorder=order)
        assert np.array_equal(y[ip[i]:ip[i + 1]], ref)
        assert ip[i + 1] - ip[i] == (n + 7) // 8


def test_bad_bitorder():
    with pytest.raises(ValueError):
        om.packbits(np.zeros(8, np.uint8), "middle")


def test_indptr_formulas_match_reference_convention():
    qo = np.array([0, 300, 300 + 129])
    kv = np.array([0, 256, 256 + 1000])
    assert om.sparse_info_indptr(qo, 3, 128).tolist() == [0, 9, 15]
    assert om.sparse_kv_info_indptr(qo, kv, 3, 128, 128).tolist() == [0, 18, 18 + 2 * 8 * 3]


def test_compact_handmade():
    # one request, 2 q-blocks, 2 heads, 3 kv-blocks
    qa = np.array([[1, 0], [1, 1]], dtype=np.uint8)
    kk = np.zeros((2, 2, 3), dtype=np.uint8)
    kk[0, 0] = [1, 0, 1]
    kk[1, 0] = [0, 0, 0]
    kk[1, 1] = [1, 1, 1]
    m = wl.pack_masks([qa], [kk])
    qo = kv = np.array([0, 256]); kv = np.array([0, 384])
    c = om.compact(m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr, qo, kv, 2, 128, 128)
    assert c["items"].tolist() == [[0, 0, 0, 2], [0, 0, 1, 0], [0, 1, 1, 3]]
    assert c["kv_indptr"].tolist() == [0, 2, 2, 5]
    assert c["kv_idx"].tolist() == [0, 2, 0, 1, 2]
    assert c["order"].tolist() == [2, 0, 1]  # one group of both heads, longest list first: n_kept = 3, 2, 0
    # head window and is_full
    c1 = om.compact(m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr, qo, kv, 2, 128, 128,
                    head_begin=1, head_count=1)
    assert c1["items"].tolist() == [[0, 1, 1, 3]]
    cf = om.compact(None, None, None, None, qo, kv, 2, 128, 128, is_full=True)
    assert len(cf["items"]) == 4 and cf["kv_idx"].tolist() == [0, 1, 2] * 4


def test_compact_counts_match_unpacked_masks():
    m = wl.flux_masks(2, 5, 7, 9, 0.5, seed=3, text_blocks=2)
    qo = np.array([0, 7 * 128, 14 * 128]); kv = np.array([0, 9 * 128, 18 * 128])
    c = om.compact(m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr, qo, kv, 5, 128, 128)
    assert len(c["items"]) == sum(int(q.sum()) for q in m.q_active)
    assert len(c["kv_idx"]) == wl.executed_attention_tiles(m)
    assert sorted(c["order"].tolist()) == list(range(len(c["items"])))
    # one group of all five heads per request: longest lists first, ties in list order
    assert om.order_groups(2, 5, 9) == (5, True)
    keys = [(int(c["items"][i][0]), -int(c["items"][i][3]), int(i)) for i in c["order"].tolist()]
    assert keys == sorted(keys)
    # with more (request, group, length) buckets than the kernel sorts by: single heads, q-blocks ascending
    mb = wl.flux_masks(1, 40, 2, 604, 0.5, seed=4, text_blocks=1)
    qo = np.array([0, 2 * 128]); kv = np.array([0, 604 * 128])
    assert om.order_groups(1, 40, 604) == (1, False)
    cb = om.compact(mb.sparse_info, mb.sparse_kv_info, mb.info_indptr, mb.kv_info_indptr, qo, kv, 40, 128, 128)
    keys = [(int(b), int(h), int(qb)) for b, h, qb, _ in cb["items"][cb["order"]].tolist()]
    assert keys == sorted(keys)
    # groups of heads: 24 heads of 36 kv blocks (2.25 MiB of K + V each) -> two groups of 12
    assert om.order_groups(2, 24, 36) == (12, True)
    assert om.order_groups(1, 3, 36) == (3, True)


def test_attention_units_cut_long_lists_only_when_items_are_few():
    m = wl.flux_masks(1, 6, 20, 20, 0.7, seed=9, text_blocks=2)
    qo = kv = np.array([0, 20 * 128 - 50])           # ragged last q and kv block
    c = om.compact(m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr, qo, kv, 6, 128, 128)
    n = len(c["items"])
    # more items than the unit count aimed at: one unit per item, in processing order, no partial slots
    u, slots, chunk = om.attn_units(c, qo, kv, num_streams=n - 1)
    assert slots == 0 and chunk == 0x7fffffff and len(u) == n
    for r, it in zip(u.tolist(), c["order"].tolist()):
        b, h, qb, nk = c["items"][it].tolist()
        assert r[0] == nk and r[1] == c["kv_indptr"][it] and r[2] == h and r[3] == qb * 128
        assert (r[4] & 0xffff) == (128 if qb < 19 else 128 - 50) and r[5] == 0
        last_is_partial = nk > 0 and c["kv_idx"][c["kv_indptr"][it] + nk - 1] == 19
        assert (r[4] >> 16) == (128 - 50 if last_is_partial else 0) and (r[7] & 0xffffffff) == 0xffff0001
        assert r[6] == qb * 128        # causal base: q and kv of the request have the same length
    # few items per stream: lists longer than chunk_max are cut into parts that tile the list without gaps
    u, slots, chunk = om.attn_units(c, qo, kv, num_streams=2 * n, min_chunk=6)
    assert chunk == max(6, -(-int(c["items"][:, 3].sum()) // (2 * n)))
    assert om.attn_units(c, qo, kv, num_streams=n, min_chunk=6)[1] > 0     # exactly as many items: still cut
    lens_u = u[:, 0].tolist()
    assert lens_u == sorted(lens_u, reverse=True)            # cut lists: units in descending order of length
    by_off = {int(r[1]): r for r in u.tolist() if r[0] > 0}  # non-empty units by their first kv_idx entry
    used, seen = 0, 0
    for it in c["order"].tolist():
        nk = int(c["items"][it][3])
        if nk == 0:
            continue
        n_parts = -(-nk // chunk) if nk > chunk else 1
        off = int(c["kv_indptr"][it])
        for p in range(n_parts):
            r = by_off[off]
            assert r[0] > 0
            off += r[0]
            w = r[7] & 0xffffffff
            if n_parts > 1:
                assert (w & 0xff) == n_parts and ((w >> 8) & 0xff) == p and (w >> 16) == used + p
            else:
                assert w == 0xffff0001
            assert (r[4] >> 16) == 0 or p == n_parts - 1   # only the last part can end with the partial block
            seen += 1
        assert off == int(c["kv_indptr"][it]) + nk           # the parts tile the list without gaps
        used += n_parts if n_parts > 1 else 0
    n_empty = int((c["items"][:, 3] == 0).sum())
    assert seen + n_empty == len(u) and int((u[:, 0] == 0).sum()) == n_empty
    assert used == slots and slots > 0


def test_gemm_lists():
    m = wl.flux_masks(2, 4, 6, 6, 0.5, seed=5, text_blocks=1)
    tiles = om.gemm_q_tiles(m.sparse_info, m.info_indptr, 2, 6 * 128, 4 * 128, 4)
    exp = [(b, iy, ix) for b in range(2) for iy in range(6) for ix in range(4) if m.q_active[b][iy, ix]]
    assert tiles.tolist() == [list(t) for t in exp]
    pairs = om.gemm_q_tile_pairs(m.sparse_info, m.info_indptr, 2, 6 * 128, 4 * 128, 4)
    flat = [(b, iy, ix) for b, iy, i0, i1 in pairs.tolist() for ix in (i0, i1) if ix >= 0]
    assert sorted(flat) == [tuple(t) for t in tiles.tolist()]
    assert all(i1 == -1 or i1 > i0 for _, _, i0, i1 in pairs.tolist())
    # two-block records first, single-block records last, each part in ascending (b, iy) order
    kinds = [i1 < 0 for _, _, _, i1 in pairs.tolist()]
    assert kinds == sorted(kinds)
    for part in ([r for r in pairs.tolist() if r[3] >= 0], [r for r in pairs.tolist() if r[3] < 0]):
        assert part == sorted(part)
    # a row offset (num_text_tokens) shifts the q-block a row tile maps to
    tiles2 = om.gemm_q_tiles(m.sparse_info, m.info_indptr, 2, 4 * 128, 4 * 128, 4, num_text_tokens=256)
    exp2 = [(b, iy, ix) for b in range(2) for iy in range(4) for ix in range(4) if m.q_active[b][iy + 2, ix]]
    assert tiles2.tolist() == [list(t) for t in exp2]
    ip, heads, order = om.gemm_o_rows(m.sparse_info, m.info_indptr, 2, 6 * 128, 4 * 128, 4)
    ipc, headsc, _ = om.gemm_o_rows(m.sparse_info, m.info_indptr, 2, 6 * 128, 4 * 128, 4, is_for_cache=True)
    r = 0
    for b in range(2):
        for iy in range(6):
            a = set(heads[ip[r]:ip[r + 1]].tolist()); c = set(headsc[ipc[r]:ipc[r + 1]].tolist())
            assert a == {h for h in range(4) if m.q_active[b][iy, h]}
            assert a | c == set(range(4)) and not (a & c)
            r += 1
    cnt = (ip[1:] - ip[:-1])[order]
    assert np.all(cnt[:-1] >= cnt[1:])


def test_gemm_q_split_rule():
    # 463 two-block and 32 single-block tiles on 148 CTAs: three full rounds of two-block tiles (444), the other
    # 19 cut into 38 singles, so the launch ends after 3 * 20 + 13 instead of 4 * 20 time units
    assert om.gemm_q_makespan(463, 32, 148) == 80
    assert om.gemm_q_split_rule(463, 32, 148, 10 ** 6) == 19
    assert om.gemm_q_makespan(444, 70, 148) == 73
    # one round with room to spare: nothing to gain below one two-block tile unless every tile is cut
    assert om.gemm_q_split_rule(101, 38, 148, 10 ** 6) == 0
    assert om.gemm_q_split_rule(37, 41, 148, 10 ** 6) == 37 and om.gemm_q_makespan(0, 115, 148) == 13
    # capacity: records may not exceed max_records
    assert om.gemm_q_split_rule(37, 41, 148, 80) == 0
    assert om.gemm_q_split_rule(0, 5, 148, 100) == 0
    # the list with a cut: same tiles, two-block records first, cut records between them and the leftover singles
    m = wl.flux_masks(2, 4, 6, 6, 0.5, seed=5, text_blocks=1)
    plain = om.gemm_q_tile_pairs(m.sparse_info, m.info_indptr, 2, 6 * 128, 4 * 128, 4)
    P, S = int((plain[:, 3] >= 0).sum()), int((plain[:, 3] < 0).sum())
    cut = om.gemm_q_tile_pairs(m.sparse_info, m.info_indptr, 2, 6 * 128, 4 * 128, 4, num_ctas=11)
    k = om.gemm_q_split_rule(P, S, 11, 2 * 6 * 4)
    assert k > 0 and len(cut) == P + S + k
    assert np.array_equal(cut[:P - k], plain[:P - k]) and np.array_equal(cut[P + k:], plain[P:])
    for j in range(k):
        b, iy, i0, i1 = plain[P - k + j]
        assert cut[P - k + 2 * j].tolist() == [b, iy, i0, -1] and cut[P - k + 2 * j + 1].tolist() == [b, iy, i1, -1]
