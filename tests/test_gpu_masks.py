"""GPU: packbits / segment_packbits / mask compaction / GEMM work lists, bit-exact against the oracle."""

import numpy as np
import pytest
import torch

import flashomni_b200 as fo
from flashomni_b200 import _native, workloads as wl
from oracle import masks as om
from helpers import dev, masks_to_device

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("order", ["big", "little"])
@pytest.mark.parametrize("n", [1, 7, 8, 9, 64, 1000, 4097, 1 << 20])
def test_packbits_matches_numpy(cuda_device, order, n):
    rng = np.random.default_rng(n)
    x = rng.integers(0, 2, n).astype(np.uint8)
    y = fo.packbits(dev(x, cuda_device).bool(), bitorder=order)
    assert np.array_equal(y.cpu().numpy(), om.packbits(x, order))


def test_packbits_reference_docstring_kat(cuda_device):
    x = torch.tensor([1, 0, 1, 1, 0, 0, 1, 1], dtype=torch.bool, device=cuda_device)
    assert fo.packbits(x).tolist() == [0b10110011]
    xs = torch.tensor([1, 0, 1, 1, 0, 0, 1, 1, 1, 0, 1], dtype=torch.bool, device=cuda_device)
    y, ip = fo.segment_packbits(xs, torch.tensor([0, 4, 7, 11], device=cuda_device), bitorder="big")
    assert y.tolist() == [0b10110000, 0b100000, 0b11010000]
    assert ip.tolist() == [0, 1, 2, 3]


@pytest.mark.parametrize("order", ["big", "little"])
def test_segment_packbits_ragged(cuda_device, order):
    rng = np.random.default_rng(1)
    lens = [0, 1, 7, 8, 9, 63, 64, 65, 1000, 0, 31104, 5]
    indptr = np.concatenate([[0], np.cumsum(lens)])
    x = rng.integers(0, 2, int(indptr[-1])).astype(np.uint8)
    y, ip = fo.segment_packbits(dev(x, cuda_device), dev(indptr, cuda_device), bitorder=order)
    ry, rip = om.segment_packbits(x, indptr, order)
    assert np.array_equal(ip.cpu().numpy(), rip)
    assert np.array_equal(y.cpu().numpy(), ry)
    # uint8 input whose non-zero values are not 1, and int32 indptr
    x2 = x * 200
    y2, _ = fo.segment_packbits(dev(x2, cuda_device), dev(indptr.astype(np.int32), cuda_device), bitorder=order)
    assert np.array_equal(y2.cpu().numpy(), ry)


def _compact_gpu(device, m, qo, kv, H, head_begin=0, head_count=None, is_full=False):
    hc = H - head_begin if head_count is None else head_count
    w = fo.BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1024, dtype=torch.uint8, device=device))
    w.plan(dev(qo.astype(np.int32), device), dev(kv.astype(np.int32), device), hc, hc, 128, q_data_type=torch.bfloat16,
           mask_num_heads=H, mask_head_begin=head_begin)
    lib = _native.load()
    si, skv, ip, kp = masks_to_device(m, device)
    ws = w._ws
    rc = lib.fo_mask_compact(_native.ptr(si), si.numel(), _native.ptr(skv), skv.numel(), _native.ptr(ip), _native.ptr(kp),
                             _native.ptr(w._qo_indptr_buf), _native.ptr(w._kv_indptr_buf), len(qo) - 1, H, head_begin, hc,
                             128, 128, 1 if is_full else 0, w._n_cand, w._max_nkv, max(w._n_cand, 1), max(w._max_kept, 1),
                             _native.ptr(ws["items"]), _native.ptr(ws["kv_ptr"]), _native.ptr(ws["kv_idx"]),
                             _native.ptr(ws["order"]), _native.ptr(ws["counters"]), _native.ptr(ws["scratch"]),
                             w._scratch_bytes, torch.cuda.current_stream(device).cuda_stream)
    _native.check(rc, "fo_mask_compact")
    torch.cuda.synchronize()
    return w.work_lists()


def _assert_lists_equal(got, ref):
    assert got["status"] == 0
    assert got["n_items"] == len(ref["items"])
    assert got["total_kept"] == len(ref["kv_idx"])
    for k in ("items", "kv_indptr", "kv_idx", "order"):
        assert np.array_equal(got[k], ref[k]), k


@pytest.mark.parametrize("case", ["flux_b1", "flux_b2", "ragged", "window", "full", "sparse_extreme"])
def test_attention_compaction_bit_exact(cuda_device, case):
    H = 24
    if case == "flux_b1":
        m = wl.flux_masks(1, H, 36, 36, 0.5, seed=11); qo = kv = np.array([0, 4608])
        args = {}
    elif case == "flux_b2":
        m = wl.flux_masks(2, H, 36, 36, 0.5, seed=12); qo = kv = np.array([0, 4608, 9216])
        args = {}
    elif case == "ragged":
        H = 5
        lens_q, lens_kv = [300, 128, 1000, 77], [256, 700, 1300, 129]
        qo = np.concatenate([[0], np.cumsum(lens_q)]); kv = np.concatenate([[0], np.cumsum(lens_kv)])
        rng = np.random.default_rng(2)
        qa = [(rng.random((-(-a // 128), H)) < 0.6).astype(np.uint8) for a in lens_q]
        kk = [(rng.random((-(-a // 128), H, -(-b // 128))) < 0.5).astype(np.uint8) for a, b in zip(lens_q, lens_kv)]
        m = wl.pack_masks(qa, kk); args = {}
    elif case == "window":
        m = wl.flux_masks(2, H, 36, 36, 0.5, seed=13); qo = kv = np.array([0, 4608, 9216])
        args = {"head_begin": 6, "head_count": 3}
    elif case == "full":
        m = wl.flux_masks(1, H, 9, 11, 0.5, seed=14); qo = np.array([0, 9 * 128]); kv = np.array([0, 11 * 128])
        args = {"is_full": True}
    else:  # nothing active in most rows, long kv rows (more than 32 words per row)
        H = 3
        rng = np.random.default_rng(3)
        qa = [(rng.random((7, H)) < 0.2).astype(np.uint8)]
        kk = [(rng.random((7, H, 1100)) < 0.03).astype(np.uint8)]
        m = wl.pack_masks(qa, kk); qo = np.array([0, 7 * 128]); kv = np.array([0, 1100 * 128]); args = {}
    got = _compact_gpu(cuda_device, m, qo, kv, H, **args)
    ref = om.compact(m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr, qo, kv, H, 128, 128, **args)
    _assert_lists_equal(got, ref)


def test_attention_compaction_random_ragged_cases(cuda_device):
    """Forty seeded cases: ragged request lengths, densities from empty to full, head windows."""
    rng = np.random.default_rng(2025)
    for _ in range(40):
        B, H = int(rng.integers(1, 5)), int(rng.integers(1, 7))
        lens_q = [int(rng.integers(1, 1500)) for _ in range(B)]
        lens_kv = [int(rng.integers(1, 6000)) for _ in range(B)]
        dq, dk = float(rng.choice([0.0, 0.3, 0.8, 1.0])), float(rng.choice([0.0, 0.05, 0.5, 1.0]))
        qa = [(rng.random((-(-a // 128), H)) < dq).astype(np.uint8) for a in lens_q]
        kk = [(rng.random((-(-a // 128), H, -(-b // 128))) < dk).astype(np.uint8) for a, b in zip(lens_q, lens_kv)]
        hb = int(rng.integers(0, H))
        hc = int(rng.integers(1, H - hb + 1))
        qo = np.concatenate([[0], np.cumsum(lens_q)]); kv = np.concatenate([[0], np.cumsum(lens_kv)])
        m = wl.pack_masks(qa, kk)
        got = _compact_gpu(cuda_device, m, qo, kv, H, head_begin=hb, head_count=hc)
        ref = om.compact(m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr, qo, kv, H, 128, 128, hb, hc)
        _assert_lists_equal(got, ref)


def test_gemm_worklists_bit_exact(cuda_device):
    lib = _native.load()
    B, H, nq = 2, 24, 36
    m = wl.flux_masks(B, H, nq, nq, 0.5, seed=21)
    si, _, ip, _ = masks_to_device(m, cuda_device)
    M, N, K = nq * 128, H * 128, H * 128
    nbytes = lib.fo_gemm_workspace_bytes(B, M, N, K, 128)
    ws = torch.zeros(nbytes, dtype=torch.uint8, device=cuda_device)
    st = torch.cuda.current_stream(cuda_device).cuda_stream
    sms = torch.cuda.get_device_properties(cuda_device).multi_processor_count
    for ntt, m_rows in ((0, M), (512, M - 512)):
        # all heads, and head windows as a rank of 2 / 8 has them (few records: the rule cuts more of them)
        for hb, hc in ((0, H), (12, 12), (21, 3)):
            rc = lib.fo_gemm_q_worklist(B, m_rows, hc * 128, H, hb, 128, 128, ntt, 0, _native.ptr(si), si.numel(),
                                        _native.ptr(ip), _native.ptr(ws), ws.numel(), st)
            _native.check(rc, "fo_gemm_q_worklist")
            w = ws.view(torch.int32).cpu().numpy()
            ref = om.gemm_q_tile_pairs(m.sparse_info, m.info_indptr, B, m_rows, hc * 128, H, 128, ntt, head_begin=hb,
                                       head_dim=128, num_ctas=sms)
            assert w[0] == len(ref) and w[2] == 0
            assert w[1] == len(om.gemm_q_tiles(m.sparse_info, m.info_indptr, B, m_rows, hc * 128, H, 128, ntt,
                                               head_begin=hb, head_dim=128))
            assert w[3] == int((ref[:, 3] >= 0).sum())
            assert np.array_equal(w[8:8 + 4 * len(ref)].reshape(-1, 4), ref)
        for cache in (0, 1):
            rc = lib.fo_gemm_o_worklist(B, m_rows, K, H, 0, 128, 128, ntt, cache, _native.ptr(si), si.numel(),
                                        _native.ptr(ip), _native.ptr(ws), ws.numel(), st)
            _native.check(rc, "fo_gemm_o_worklist")
            w = ws.view(torch.int32).cpu().numpy()
            rip, rheads, rorder = om.gemm_o_rows(m.sparse_info, m.info_indptr, B, m_rows, K, H, 128, ntt, bool(cache))
            R = B * m_rows // 128
            assert w[0] == R and w[1] == len(rheads)
            assert np.array_equal(w[8:8 + R + 1], rip)
            assert np.array_equal(w[8 + R + 1:8 + R + 1 + len(rheads)], rheads)
            o0 = 8 + R + 1 + R * H
            assert np.array_equal(w[o0:o0 + R], rorder)


def test_strided_gather_matches_torch(cuda_device):
    """fo_strided_gather on local buffers: the two layouts of the sequence-parallel exchange."""
    from flashomni_b200.parallel import PeerExchange
    g = torch.Generator().manual_seed(5)
    H, D, hc = 8, 128, 2
    srcs = [torch.randn(n, H, D, generator=g).to(torch.bfloat16).to(cuda_device) for n in (256, 128, 384)]
    out = torch.zeros(sum(t.shape[0] for t in srcs), hc, D, dtype=torch.bfloat16, device=cuda_device)
    row = hc * D * 2
    offs = [0, 256, 384]
    PeerExchange.gather([t.data_ptr() + 3 * row for t in srcs], [H * D * 2] * 3, [t.shape[0] for t in srcs],
                        [out.data_ptr() + o * row for o in offs], [row] * 3, row)
    torch.cuda.synchronize()
    assert torch.equal(out, torch.cat([t[:, 6:8] for t in srcs]))
    # the way back: contiguous source rows into a column block of a wider destination
    back = torch.zeros(128, H, D, dtype=torch.bfloat16, device=cuda_device)
    PeerExchange.gather([out.data_ptr() + 256 * row], [row], [128], [back.data_ptr() + 3 * row], [H * D * 2], row)
    torch.cuda.synchronize()
    assert torch.equal(back[:, 6:8], srcs[1][:, 6:8]) and int(back[:, :6].abs().sum()) == 0
    with pytest.raises(ValueError):
        PeerExchange.gather([out.data_ptr() + 2], [row], [1], [back.data_ptr()], [row], row)   # misaligned


@pytest.mark.parametrize("case", ["few_items_cut", "many_items_whole", "ragged"])
def test_attention_work_units_bit_exact(cuda_device, case, monkeypatch):
    """The unit list the attention kernel walks (fo_attn_units) against the oracle's statement: long kv lists are
    cut into parts when the launch has few items per stream, never otherwise."""
    monkeypatch.setattr(fo.BatchFlashOmniFAWithRaggedKVWrapper, "UNITS_PER_SM", 2)   # list cutting on
    if case == "few_items_cut":
        H, lens = 6, [36 * 128]                      # about 195 items: between one and two per SM
        m = wl.flux_masks(1, H, 36, 36, 0.9, seed=21)
    elif case == "many_items_whole":
        H, lens = 24, [36 * 128, 36 * 128]
        m = wl.flux_masks(2, H, 36, 36, 0.9, seed=22)
    else:
        H, lens = 3, [700, 128 * 9 + 5, 40]
        rng = np.random.default_rng(23)
        qa = [(rng.random((-(-n // 128), H)) < 0.8).astype(np.uint8) for n in lens]
        kk = [(rng.random((-(-n // 128), H, -(-n // 128))) < 0.7).astype(np.uint8) * a[:, :, None] for n, a in zip(lens, qa)]
        m = wl.pack_masks(qa, kk)
    qo = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    w = fo.BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1024, dtype=torch.uint8, device=cuda_device))
    w.plan(dev(qo, cuda_device), dev(qo, cuda_device), H, H, 128, q_data_type=torch.bfloat16)
    w.build_work_lists(*masks_to_device(m, cuda_device))
    torch.cuda.synchronize()
    got = w.work_lists()
    ref = om.compact(m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr, qo, qo, H, 128, 128)
    _assert_lists_equal(got, ref)
    units, slots, chunk = om.attn_units(ref, qo, qo, w._num_streams, w.MIN_CHUNK, max_slots=w._partial_slots,
                                        min_items=w._min_items)
    assert got["unit_status"] == 0 and got["chunk_max"] == chunk and got["partial_slots_used"] == slots
    assert got["n_units"] == len(units) and np.array_equal(got["units"], units)
    if case == "many_items_whole":
        assert slots == 0 and len(units) == len(ref["items"])
    if case == "few_items_cut":
        assert slots > 0
    assert got["n_units"] <= w._max_units and slots <= w._partial_slots
