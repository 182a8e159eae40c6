"""GPU: block-sparse attention through the wrapper against the fp32 oracle."""

import math

import numpy as np
import pytest
import torch

import flashomni_b200 as fo
from flashomni_b200 import workloads as wl
from oracle import attention as oa
from helpers import assert_close_bf16, dev, masks_to_device

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["default", "split"])
def attention_kernel_choice(request, monkeypatch):
    """Every test of this file runs twice: with the wrapper's own rule for cutting kv lists into parts, and with
    every list of more than two blocks cut (small cases only), so that each case also goes through the partial
    results and their merge. The wrapper's own rule is tested separately."""
    monkeypatch.setattr(fo.BatchFlashOmniFAWithRaggedKVWrapper, "FORCE_SPLIT", request.param == "split")
    return request.param


def _wrapper(device, qo, kv, H, dtype=torch.bfloat16, layout="NHD", **kw):
    w = fo.BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1 << 20, dtype=torch.uint8, device=device), layout)
    w.plan(dev(np.asarray(qo, np.int32), device), dev(np.asarray(kv, np.int32), device), H, H, 128,
           q_data_type=dtype, **kw)
    return w


def _run(device, w, q, k, v, m, **kw):
    si, skv, ip, kp = masks_to_device(m, device)
    r = w.run(dev(q, device), dev(k, device), dev(v, device), si, skv, ip, kp, **kw)
    w.check_status()
    return r


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("seq,H,density", [(128, 1, 1.0), (256, 2, 1.0), (512, 2, 0.6), (1024, 4, 0.5)])
def test_small_uniform(cuda_device, dtype, seq, H, density):
    inp = wl.attention_inputs(1, H, seq, 128, density, seed=40 + seq, dtype=dtype)
    w = _wrapper(cuda_device, inp.qo_indptr, inp.kv_indptr, H, dtype)
    prior = wl.randn_bf16(inp.q.shape, 99, dtype=dtype)
    out = dev(prior, cuda_device).clone()
    o = _run(cuda_device, w, inp.q, inp.k, inp.v, inp.masks, out=out)
    m = inp.masks
    ref = oa.sparse_attention(inp.q, inp.k, inp.v, inp.qo_indptr.numpy(), inp.kv_indptr.numpy(), m.sparse_info,
                              m.sparse_kv_info, m.info_indptr, m.kv_info_indptr, out_prior=prior)
    assert_close_bf16(o, ref, f"attention S={seq} H={H} {dtype}")
    # skipped q-blocks are never written
    oc = o.cpu()
    for qb in range(seq // 128):
        for h in range(H):
            if not m.q_active[0][qb, h]:
                assert torch.equal(oc[qb * 128:(qb + 1) * 128, h], prior[qb * 128:(qb + 1) * 128, h])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_logits_soft_cap(cuda_device, dtype):
    """logits = cap * tanh(q.k * sm_scale / cap) (reference: variants.cuh:47-50,72-74); the cap is small enough
    for the tanh to bend most logits (q.k * sm_scale ~ N(0, 1) here). Ragged kv tail included."""
    H, cap = 2, 1.5
    lens_q, lens_kv = [384, 200], [640, 300]
    qo = np.concatenate([[0], np.cumsum(lens_q)]); kv = np.concatenate([[0], np.cumsum(lens_kv)])
    rng = np.random.default_rng(15)
    qa = [np.ones((-(-a // 128), H), np.uint8) for a in lens_q]
    kk = [(rng.random((-(-a // 128), H, -(-b // 128))) < 0.7).astype(np.uint8) for a, b in zip(lens_q, lens_kv)]
    for x in kk:
        x[:, :, -1] = 1   # the ragged last kv-block is kept everywhere
    m = wl.pack_masks(qa, kk)
    q = wl.randn_bf16((int(qo[-1]), H, 128), 11, dtype=dtype)
    k = wl.randn_bf16((int(kv[-1]), H, 128), 12, dtype=dtype)
    v = wl.randn_bf16((int(kv[-1]), H, 128), 13, dtype=dtype)
    w = _wrapper(cuda_device, qo, kv, H, dtype, logits_soft_cap=cap)
    o, lse = _run(cuda_device, w, q, k, v, m, return_lse=True)
    ref, ref_lse = oa.sparse_attention(q, k, v, qo, kv, m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr,
                                       return_lse=True, logits_soft_cap=cap)
    assert_close_bf16(o, ref, f"soft-capped attention {dtype}")
    assert torch.allclose(lse.cpu(), ref_lse, atol=2e-2, rtol=1e-4)
    # and it differs from the uncapped result (the cap is really applied)
    plain = oa.sparse_attention(q, k, v, qo, kv, m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr)
    assert (plain - ref).abs().max() > 5e-2


def test_ragged_batch_with_empty_rows_and_lse(cuda_device):
    H = 3
    lens_q, lens_kv = [300, 128, 1000, 77], [256, 700, 1300, 129]
    qo = np.concatenate([[0], np.cumsum(lens_q)]); kv = np.concatenate([[0], np.cumsum(lens_kv)])
    rng = np.random.default_rng(5)
    qa = [(rng.random((-(-a // 128), H)) < 0.7).astype(np.uint8) for a in lens_q]
    kk = [(rng.random((-(-a // 128), H, -(-b // 128))) < 0.5).astype(np.uint8) for a, b in zip(lens_q, lens_kv)]
    qa[0][0, 0] = 1; kk[0][0, 0, :] = 0       # an active q-block that keeps nothing -> zeros, lse = -5e4
    qa[2][7, 1] = 1; kk[2][7, 1, :] = 0; kk[2][7, 1, 10] = 1   # only the ragged last kv-block kept
    m = wl.pack_masks(qa, kk)
    q = wl.randn_bf16((int(qo[-1]), H, 128), 1); k = wl.randn_bf16((int(kv[-1]), H, 128), 2); v = wl.randn_bf16((int(kv[-1]), H, 128), 3)
    w = _wrapper(cuda_device, qo, kv, H)
    prior = wl.randn_bf16(q.shape, 4)
    lse_prior = torch.full((q.shape[0], H), 3.0)
    o, lse = _run(cuda_device, w, q, k, v, m, out=dev(prior, cuda_device).clone(), lse=dev(lse_prior, cuda_device).clone(),
                  return_lse=True)
    ref, ref_lse = oa.sparse_attention(q, k, v, qo, kv, m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr,
                                       out_prior=prior, lse_prior=lse_prior, return_lse=True)
    assert_close_bf16(o, ref, "ragged attention")
    assert torch.all(o[:128, 0] == 0)
    assert torch.allclose(lse.cpu(), ref_lse, atol=2e-2, rtol=1e-4)


def test_is_full_matches_dense_sdpa_and_default_zero_out(cuda_device):
    H, S = 2, 640
    q = wl.randn_bf16((S, H, 128), 1); k = wl.randn_bf16((S, H, 128), 2); v = wl.randn_bf16((S, H, 128), 3)
    w = _wrapper(cuda_device, [0, S], [0, S], H)
    o = w.run(dev(q, cuda_device), dev(k, cuda_device), dev(v, cuda_device), is_full=True)
    w.check_status()
    ref = torch.nn.functional.scaled_dot_product_attention(q.float().transpose(0, 1), k.float().transpose(0, 1),
                                                           v.float().transpose(0, 1)).transpose(0, 1)
    assert_close_bf16(o, ref, "is_full attention")
    with pytest.raises(ValueError):
        w.run(dev(q, cuda_device), dev(k, cuda_device), dev(v, cuda_device))  # masks missing, is_full False


def test_hnd_layout_sm_scale_and_head_window(cuda_device):
    Htot, hb, hc, S = 6, 2, 3, 512
    inp = wl.attention_inputs(1, Htot, S, 128, 0.6, seed=7)
    q, k, v = inp.q[:, hb:hb + hc].contiguous(), inp.k[:, hb:hb + hc].contiguous(), inp.v[:, hb:hb + hc].contiguous()
    w = _wrapper(cuda_device, inp.qo_indptr, inp.kv_indptr, hc, layout="HND", sm_scale=0.05, mask_num_heads=Htot,
                 mask_head_begin=hb)
    si, skv, ip, kp = masks_to_device(inp.masks, cuda_device)
    o = w.run(dev(q, cuda_device), dev(k, cuda_device).transpose(0, 1).contiguous(),
              dev(v, cuda_device).transpose(0, 1).contiguous(), si, skv, ip, kp)
    w.check_status()
    m = inp.masks
    ref = oa.sparse_attention(q, k, v, inp.qo_indptr.numpy(), inp.kv_indptr.numpy(), m.sparse_info, m.sparse_kv_info,
                              m.info_indptr, m.kv_info_indptr, sm_scale=0.05, head_begin=hb, num_mask_heads=Htot)
    assert_close_bf16(o, ref, "HND + window attention")


def test_flux_layer_size_sampled_heads(cuda_device):
    """Config-1 size (B=1, H=24, S=4608, D=128, density 0.5). The whole layer runs on the GPU; three heads
    are compared with the CPU oracle (bounded CPU time) and every head with an fp32 blockwise
    computation on the GPU."""
    H, S = 24, 4608
    inp = wl.attention_inputs(1, H, S, 128, 0.5, seed=8)
    w = _wrapper(cuda_device, inp.qo_indptr, inp.kv_indptr, H)
    prior = wl.randn_bf16(inp.q.shape, 9)
    o = _run(cuda_device, w, inp.q, inp.k, inp.v, inp.masks, out=dev(prior, cuda_device).clone())
    lists = w.work_lists()
    assert lists["total_kept"] == wl.executed_attention_tiles(inp.masks)
    m = inp.masks
    for h in (0, 11, 23):
        mh = wl.pack_masks([m.q_active[0][:, h:h + 1]], [m.kv_kept[0][:, h:h + 1]])
        ref = oa.sparse_attention(inp.q[:, h:h + 1], inp.k[:, h:h + 1], inp.v[:, h:h + 1], [0, S], [0, S], mh.sparse_info,
                                  mh.sparse_kv_info, mh.info_indptr, mh.kv_info_indptr, out_prior=prior[:, h:h + 1])
        assert_close_bf16(o[:, h:h + 1], ref, f"flux layer head {h}")
    # all heads, fp32 on the GPU with a dense element mask
    qd, kd, vd = (dev(t, cuda_device).float().transpose(0, 1) for t in (inp.q, inp.k, inp.v))
    kept = torch.from_numpy(m.kv_kept[0]).to(cuda_device).bool().permute(1, 0, 2)  # [H, nq, nkv]
    act = torch.from_numpy(m.q_active[0]).to(cuda_device).bool().T                 # [H, nq]
    worst = 0.0
    for h in range(H):
        s = (qd[h] @ kd[h].T) / math.sqrt(128)
        el = kept[h].repeat_interleave(128, 0).repeat_interleave(128, 1)
        p = torch.softmax(s.masked_fill(~el, float("-inf")), -1).nan_to_num(0.0)
        ref = p @ vd[h]
        rows = act[h].repeat_interleave(128)
        ref = torch.where(rows[:, None], ref, dev(prior, cuda_device)[:, h].float())
        assert_close_bf16(o[:, h], ref, f"flux layer head {h} (gpu fp32)")


def test_prepare_masks_on_side_stream_gives_identical_result(cuda_device):
    H, S = 4, 1024
    inp = wl.attention_inputs(1, H, S, 128, 0.5, seed=91)
    w = _wrapper(cuda_device, inp.qo_indptr, inp.kv_indptr, H)
    si, skv, ip, kp = masks_to_device(inp.masks, cuda_device)
    q, k, v = (dev(t, cuda_device) for t in (inp.q, inp.k, inp.v))
    a = w.run(q, k, v, si, skv, ip, kp).clone()
    w.prepare_masks(si, skv, ip, kp)
    b = w.run(q, k, v, si, skv, ip, kp).clone()
    w.check_status()
    assert torch.equal(a, b)
    # a mask changed in place after prepare_masks() must not re-use the prepared lists
    w.prepare_masks(si, skv, ip, kp)
    si.fill_(255)
    c = w.run(q, k, v, si, skv, ip, kp).clone()
    w.check_status()
    assert w.work_lists()["n_items"] == H * (S // 128)   # every q-block active now: the lists were rebuilt
    assert torch.equal(c, w.run(q, k, v, si, skv, ip, kp))
    # the compaction alone, on the caller's stream or on a stream of the caller's choice after an event
    w.build_work_lists(si, skv, ip, kp)
    assert w.work_lists()["n_items"] == H * (S // 128)
    side, ev = torch.cuda.Stream(cuda_device), torch.cuda.Event()
    ev.record()
    w.prepare_masks(si, skv, ip, kp, stream=side, after=ev)
    assert torch.equal(c, w.run(q, k, v, si, skv, ip, kp))
    w.check_status()


def test_block_forward_is_cuda_graph_capturable(cuda_device, monkeypatch):
    monkeypatch.delenv("FLASHOMNI_B200_CHECK", raising=False)  # the debug checks synchronise: not capturable
    _block_graph_capture(cuda_device)


def _block_graph_capture(cuda_device):
    """The whole block (projections, side-stream mask compaction, attention, GEMM-O) captured in one CUDA graph
    and replayed gives the eager result (the reference supports graph capture of run(), attention.py:353-377)."""
    from flashomni_b200.layer import BlockWeights, SparseDiTAttentionBlock
    B, H, S, hid = 1, 4, 1024, 512
    m = wl.flux_masks(B, H, S // 128, S // 128, 0.5, seed=93, text_blocks=1)
    si, skv, ip, kp = masks_to_device(m, cuda_device)
    ws = [dev(wl.randn_bf16((hid, hid), 94 + i, std=hid ** -0.5), cuda_device) for i in range(4)]
    blk = SparseDiTAttentionBlock(BlockWeights(*ws), H, 128, B, S, device=cuda_device)
    blk.cache.copy_(dev(wl.randn_bf16((B, S, hid), 99), cuda_device))
    x = dev(wl.randn_bf16((B, S, hid), 98), cuda_device)
    for _ in range(2):
        eager = blk.forward(x, si, skv, ip, kp).clone()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(cuda_device)
    side.wait_stream(torch.cuda.current_stream(cuda_device))
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            y = blk.forward(x, si, skv, ip, kp)
    blk.y.zero_()
    g.replay()
    torch.cuda.synchronize()
    blk.wrapper.check_status()
    assert torch.equal(y, eager)
    # new input, same graph
    x.copy_(dev(wl.randn_bf16((B, S, hid), 97), cuda_device))
    g.replay()
    torch.cuda.synchronize()
    replayed = y.clone()
    assert torch.equal(replayed, blk.forward(x, si, skv, ip, kp))


def test_block_schedule_kv_first_matches(cuda_device, monkeypatch):
    """The kv_first schedule (all list kernels on a side stream beside the dense projections, prepared GEMM
    work lists) gives bit-identical results to the default schedule, eagerly and from a CUDA graph."""
    monkeypatch.delenv("FLASHOMNI_B200_CHECK", raising=False)
    from flashomni_b200.layer import BlockWeights, SparseDiTAttentionBlock
    B, H, S, hid = 2, 4, 1024, 512
    m = wl.flux_masks(B, H, S // 128, S // 128, 0.5, seed=193, text_blocks=1)
    si, skv, ip, kp = masks_to_device(m, cuda_device)
    ws = [dev(wl.randn_bf16((hid, hid), 194 + i, std=hid ** -0.5), cuda_device) for i in range(4)]
    cache = dev(wl.randn_bf16((B, S, hid), 199), cuda_device)
    x = dev(wl.randn_bf16((B, S, hid), 198), cuda_device)
    outs = {}
    for sched in ("q_first", "kv_first"):
        blk = SparseDiTAttentionBlock(BlockWeights(*ws), H, 128, B, S, device=cuda_device, schedule=sched)
        blk.cache.copy_(cache)
        for _ in range(3):
            y = blk.forward(x, si, skv, ip, kp)
        torch.cuda.synchronize()
        blk.wrapper.check_status()
        outs[sched] = y.clone()
    assert torch.equal(outs["q_first"], outs["kv_first"])
    g = torch.cuda.CUDAGraph()
    cs = torch.cuda.Stream(cuda_device)
    cs.wait_stream(torch.cuda.current_stream(cuda_device))
    with torch.cuda.stream(cs):
        with torch.cuda.graph(g, stream=cs):
            y = blk.forward(x, si, skv, ip, kp)
    blk.y.zero_()
    for _ in range(2):
        g.replay()
    torch.cuda.synchronize()
    blk.wrapper.check_status()
    assert torch.equal(y, outs["q_first"])


def test_video_layer_size_sampled_rows(cuda_device):
    """Config-5 size (77 312 tokens = 604 blocks, spatiotemporal-local mask at density ~0.25), four heads. The
    whole attention runs on the GPU; sampled (head, q-block) rows are compared with an fp32 blockwise computation
    on the GPU over the row's kept kv-blocks (a CPU oracle of this size would take minutes)."""
    H, frames, bpf = 4, 20, 30
    nblk = 4 + frames * bpf
    S = nblk * 128
    m = wl.video_masks(H, frames, bpf, seed=77)
    q, k, v = (dev(wl.randn_bf16((S, H, 128), 80 + i), cuda_device) for i in range(3))
    si, skv, ip, kp = masks_to_device(m, cuda_device)
    indptr = torch.tensor([0, S], dtype=torch.int32, device=cuda_device)
    w = fo.BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1 << 20, dtype=torch.uint8, device=cuda_device))
    w.plan(indptr, indptr, H, H, 128, q_data_type=torch.bfloat16)
    o = w.run(q, k, v, si, skv, ip, kp)
    w.check_status()
    lists = w.work_lists()
    assert lists["n_items"] == H * nblk and lists["total_kept"] == wl.executed_attention_tiles(m)
    # the lists of this size, entry by entry, against the oracle's statement (items, offsets, kept indices, order)
    from oracle import masks as om
    ref_lists = om.compact(m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr, np.array([0, S]),
                           np.array([0, S]), H, 128, 128)
    for key in ("items", "kv_indptr", "kv_idx", "order"):
        assert np.array_equal(lists[key], ref_lists[key]), key
    rng = np.random.default_rng(5)
    rows = [(0, 0), (1, 3), (2, 4), (3, nblk - 1), (0, 33), (1, 34)] + [(int(rng.integers(H)), int(rng.integers(nblk)))
                                                                          for _ in range(10)]
    for h, qb in rows:
        kept = np.nonzero(m.kv_kept[0][qb, h])[0]
        cols = torch.from_numpy(np.concatenate([np.arange(b * 128, b * 128 + 128) for b in kept])).to(cuda_device)
        qf = q[qb * 128:(qb + 1) * 128, h].float()
        s = (qf @ k[cols, h].float().T) / math.sqrt(128)
        ref = torch.softmax(s, -1) @ v[cols, h].float()
        assert_close_bf16(o[qb * 128:(qb + 1) * 128, h].cpu(), ref.cpu(), f"video layer head {h} q-block {qb}")


@pytest.mark.parametrize("H,Hkv", [(8, 2), (4, 2), (16, 1), (6, 3)])
def test_grouped_query_attention(cuda_device, H, Hkv):
    """Several q heads per kv head: the masks are indexed the way the reference's kernel indexes them
    (prefill.cuh:1283-1291), one bit per (128 packed rows, kv head), a packed row being a (token, q head of the
    group) pair: a mask q-block covers 128 / group tokens. Ragged requests, lse, rows of switched-off blocks kept."""
    g = H // Hkv
    qt = 128 // g
    lens_q, lens_kv = [200, 75], [300, 128]
    qo = np.concatenate([[0], np.cumsum(lens_q)]).astype(np.int32)
    kv = np.concatenate([[0], np.cumsum(lens_kv)]).astype(np.int32)
    rng = np.random.default_rng(3 + H)
    qa = [(rng.random((-(-a // qt), Hkv)) < 0.7).astype(np.uint8) for a in lens_q]
    kk = [(rng.random((-(-a // qt), Hkv, -(-b // 128))) < 0.6).astype(np.uint8) for a, b in zip(lens_q, lens_kv)]
    kk[0][0, 0, :] = 0            # an active q-block that keeps nothing: zeros, lse -5e4
    qa[0][0, 0] = 1
    m = wl.pack_masks(qa, kk)
    q = wl.randn_bf16((int(qo[-1]), H, 128), 32)
    k = wl.randn_bf16((int(kv[-1]), Hkv, 128), 33)
    v = wl.randn_bf16((int(kv[-1]), Hkv, 128), 34)
    prior = wl.randn_bf16((int(qo[-1]), H, 128), 35)
    si, skv, ip, kp = masks_to_device(m, cuda_device)
    w = fo.BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1 << 20, dtype=torch.uint8, device=cuda_device))
    w.plan(dev(qo, cuda_device), dev(kv, cuda_device), H, Hkv, 128, q_data_type=torch.bfloat16)
    o, lse = w.run(dev(q, cuda_device), dev(k, cuda_device), dev(v, cuda_device), si, skv, ip, kp,
                   out=dev(prior, cuda_device).clone(), return_lse=True)
    w.check_status()
    ref, ref_lse = oa.sparse_attention(q, k, v, qo, kv, m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr,
                                       out_prior=prior, return_lse=True)
    assert_close_bf16(o.cpu(), ref, "gqa")
    act = torch.zeros(int(qo[-1]), H, dtype=torch.bool)
    for b in range(2):
        for qb in range(qa[b].shape[0]):
            r0 = int(qo[b]) + qb * qt
            r1 = min(r0 + qt, int(qo[b + 1]))
            for hk in range(Hkv):
                if qa[b][qb, hk]:
                    act[r0:r1, hk * g:(hk + 1) * g] = True
                else:
                    assert torch.equal(o[r0:r1, hk * g:(hk + 1) * g].cpu(), prior[r0:r1, hk * g:(hk + 1) * g])
    assert torch.allclose(lse.cpu()[act], ref_lse[act], atol=2e-2, rtol=1e-4)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("soft_cap", [0.0, 30.0])
@pytest.mark.parametrize("D", [64, 256])
def test_head_dim_64_and_256(cuda_device, dtype, soft_cap, D):
    """Head dimension 64 (half tiles, four Q K^T MMAs, 64 columns of O) and 256 (four-half tiles in single slots,
    sixteen Q K^T MMAs, 256 columns of O, P written over S): ragged requests, an active q-block that keeps nothing,
    lse, rows of switched-off blocks kept, with and without the cap."""
    H = 3
    lens_q, lens_kv = [300, 205, 128], [256, 333, 70]
    qo = np.concatenate([[0], np.cumsum(lens_q)]).astype(np.int32)
    kv = np.concatenate([[0], np.cumsum(lens_kv)]).astype(np.int32)
    rng = np.random.default_rng(64)
    qa = [(rng.random((-(-a // 128), H)) < 0.7).astype(np.uint8) for a in lens_q]
    kk = [(rng.random((-(-a // 128), H, -(-b // 128))) < 0.6).astype(np.uint8) for a, b in zip(lens_q, lens_kv)]
    qa[0][1, 2] = 1; kk[0][1, 2, :] = 0
    m = wl.pack_masks(qa, kk)
    q = wl.randn_bf16((int(qo[-1]), H, D), 65, dtype=dtype)
    k = wl.randn_bf16((int(kv[-1]), H, D), 66, dtype=dtype)
    v = wl.randn_bf16((int(kv[-1]), H, D), 67, dtype=dtype)
    prior = wl.randn_bf16((int(qo[-1]), H, D), 68, dtype=dtype)
    w = fo.BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1 << 20, dtype=torch.uint8, device=cuda_device))
    w.plan(dev(qo, cuda_device), dev(kv, cuda_device), H, H, D, q_data_type=dtype,
           logits_soft_cap=soft_cap if soft_cap > 0 else None)
    si, skv, ip, kp = masks_to_device(m, cuda_device)
    o, lse = w.run(dev(q, cuda_device), dev(k, cuda_device), dev(v, cuda_device), si, skv, ip, kp,
                   out=dev(prior, cuda_device).clone(), return_lse=True)
    w.check_status()
    ref, ref_lse = oa.sparse_attention(q, k, v, qo, kv, m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr,
                                       out_prior=prior, return_lse=True, logits_soft_cap=soft_cap)
    assert_close_bf16(o.cpu(), ref, f"head_dim {D} {dtype} cap {soft_cap}")
    act = torch.zeros(int(qo[-1]), H, dtype=torch.bool)
    for b in range(len(lens_q)):
        for qb in range(qa[b].shape[0]):
            r0 = int(qo[b]) + qb * 128
            r1 = min(r0 + 128, int(qo[b + 1]))
            for h in range(H):
                if qa[b][qb, h]:
                    act[r0:r1, h] = True
                else:
                    assert torch.equal(o[r0:r1, h].cpu(), prior[r0:r1, h])
    assert torch.allclose(lse.cpu()[act], ref_lse[act], atol=2e-2, rtol=1e-3)


@pytest.mark.parametrize("H,D", [(24, 64), (12, 256)])
def test_head_dim_64_and_256_flux_size(cuda_device, H, D):
    """24 heads of dimension 64 / 12 of dimension 256 over 4608 tokens at density 0.5 (several items per CTA, lists of
    about 18 blocks) against the fp32 computation on sampled (head, q-block) rows."""
    S = 4608
    inp = wl.attention_inputs(1, H, S, D, 0.5, seed=97)
    w = fo.BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1 << 20, dtype=torch.uint8, device=cuda_device))
    ind = inp.qo_indptr.to(cuda_device)
    w.plan(ind, ind, H, H, D, q_data_type=torch.bfloat16)
    si, skv, ip, kp = masks_to_device(inp.masks, cuda_device)
    q, k, v = (dev(t, cuda_device) for t in (inp.q, inp.k, inp.v))
    o = w.run(q, k, v, si, skv, ip, kp)
    w.check_status()
    m = inp.masks
    rng = np.random.default_rng(5)
    done = 0
    while done < 8:
        h, qb = int(rng.integers(H)), int(rng.integers(S // 128))
        if not m.q_active[0][qb, h]:
            continue
        kept = np.nonzero(m.kv_kept[0][qb, h])[0]
        cols = torch.from_numpy(np.concatenate([np.arange(b * 128, b * 128 + 128) for b in kept]))
        s_ = (inp.q[qb * 128:(qb + 1) * 128, h].float() @ inp.k[cols, h].float().T) / math.sqrt(D)
        ref = torch.softmax(s_, -1) @ inp.v[cols, h].float()
        assert_close_bf16(o[qb * 128:(qb + 1) * 128, h].cpu(), ref, f"head_dim {D} head {h} q-block {qb}")
        done += 1


@pytest.mark.parametrize("H,Hkv,D,dtype,soft_cap", [(3, 3, 128, torch.bfloat16, 0.0), (4, 2, 128, torch.float16, 0.0),
                                                    (3, 3, 64, torch.bfloat16, 0.0), (2, 2, 128, torch.bfloat16, 25.0)])
def test_causal_mask(cuda_device, H, Hkv, D, dtype, soft_cap):
    """plan(causal=True): inside the kept blocks kv position j is visible to q token i only if j <= i + kv_len - q_len
    (the reference's MaskMode::kCausal). Requests with kv longer than q, equal, and SHORTER than q (their first
    tokens then see nothing: zeros, lse -5e4), ragged tails, grouped heads, head_dim 64, soft cap."""
    g = H // Hkv
    qt = 128 // g
    lens_q, lens_kv = [300, 205, 260], [428, 205, 200]
    qo = np.concatenate([[0], np.cumsum(lens_q)]).astype(np.int32)
    kv = np.concatenate([[0], np.cumsum(lens_kv)]).astype(np.int32)
    rng = np.random.default_rng(70 + H + D)
    qa = [(rng.random((-(-a // qt), Hkv)) < 0.8).astype(np.uint8) for a in lens_q]
    kk = [(rng.random((-(-a // qt), Hkv, -(-b // 128))) < 0.7).astype(np.uint8) for a, b in zip(lens_q, lens_kv)]
    m = wl.pack_masks(qa, kk)
    q = wl.randn_bf16((int(qo[-1]), H, D), 71, dtype=dtype)
    k = wl.randn_bf16((int(kv[-1]), Hkv, D), 72, dtype=dtype)
    v = wl.randn_bf16((int(kv[-1]), Hkv, D), 73, dtype=dtype)
    prior = wl.randn_bf16((int(qo[-1]), H, D), 74, dtype=dtype)
    w = fo.BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1 << 20, dtype=torch.uint8, device=cuda_device))
    w.plan(dev(qo, cuda_device), dev(kv, cuda_device), H, Hkv, D, causal=True, q_data_type=dtype,
           logits_soft_cap=soft_cap if soft_cap > 0 else None)
    si, skv, ip, kp = masks_to_device(m, cuda_device)
    for _ in range(2):
        o, lse = w.run(dev(q, cuda_device), dev(k, cuda_device), dev(v, cuda_device), si, skv, ip, kp,
                       out=dev(prior, cuda_device).clone(), return_lse=True)
    w.check_status()
    ref, ref_lse = oa.sparse_attention(q, k, v, qo, kv, m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr,
                                       out_prior=prior, return_lse=True, logits_soft_cap=soft_cap, causal=True)
    assert_close_bf16(o.cpu(), ref, f"causal H={H}/{Hkv} D={D} {dtype}")
    act = torch.zeros(int(qo[-1]), H, dtype=torch.bool)
    for b in range(len(lens_q)):
        for qb in range(qa[b].shape[0]):
            r0 = int(qo[b]) + qb * qt
            r1 = min(r0 + qt, int(qo[b + 1]))
            for hk in range(Hkv):
                if qa[b][qb, hk]:
                    act[r0:r1, hk * g:(hk + 1) * g] = True
                else:
                    assert torch.equal(o[r0:r1, hk * g:(hk + 1) * g].cpu(), prior[r0:r1, hk * g:(hk + 1) * g])
    assert torch.allclose(lse.cpu()[act], ref_lse[act], atol=2e-2, rtol=1e-3)
    assert (ref_lse[act] == -5e4).any()          # the case does hold rows that see nothing
    # and it differs from the unmasked result
    full = oa.sparse_attention(q, k, v, qo, kv, m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr,
                               out_prior=prior)
    assert (full - ref).abs().max() > 0.1


@pytest.mark.parametrize("H,Hkv,D,dtype,packed", [(3, 3, 128, torch.bfloat16, False), (4, 2, 128, torch.float16, True),
                                                  (2, 2, 64, torch.bfloat16, False)])
def test_custom_mask(cuda_device, H, Hkv, D, dtype, packed):
    """plan(custom_mask=...) / plan(packed_custom_mask=...): inside the kept blocks position (i, j) of a request is
    visible iff its flag is set (the reference's MaskMode::kCustom). Random flags with whole rows and whole blocks
    switched off (rows that see nothing: zeros, lse -5e4), kv lengths that are no multiple of 8 (rows of the bit
    matrix start at odd bit offsets), ragged tails, grouped heads, head_dim 64."""
    g = H // Hkv
    qt = 128 // g
    lens_q, lens_kv = [300, 205, 77], [427, 205, 333]
    qo = np.concatenate([[0], np.cumsum(lens_q)]).astype(np.int32)
    kv = np.concatenate([[0], np.cumsum(lens_kv)]).astype(np.int32)
    rng = np.random.default_rng(90 + H + D)
    qa = [(rng.random((-(-a // qt), Hkv)) < 0.8).astype(np.uint8) for a in lens_q]
    kk = [(rng.random((-(-a // qt), Hkv, -(-b // 128))) < 0.7).astype(np.uint8) for a, b in zip(lens_q, lens_kv)]
    m = wl.pack_masks(qa, kk)
    cms = [rng.random((a, b)) < 0.5 for a, b in zip(lens_q, lens_kv)]
    cms[0][5:9, :] = False                 # rows that see nothing
    cms[0][:, 128:256] = False             # a whole kv block hidden
    cms[1][:, :] = True                    # a request without restriction
    flat = torch.from_numpy(np.concatenate([c.reshape(-1) for c in cms]))
    q = wl.randn_bf16((int(qo[-1]), H, D), 91, dtype=dtype)
    k = wl.randn_bf16((int(kv[-1]), Hkv, D), 92, dtype=dtype)
    v = wl.randn_bf16((int(kv[-1]), Hkv, D), 93, dtype=dtype)
    prior = wl.randn_bf16((int(qo[-1]), H, D), 94, dtype=dtype)
    w = fo.BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1 << 20, dtype=torch.uint8, device=cuda_device))
    if packed:   # packed by the caller, every request's matrix on its own byte boundary
        elems = np.asarray([c.size for c in cms], dtype=np.int64)
        ind = torch.from_numpy(np.concatenate([[0], np.cumsum(elems)]).astype(np.int32)).to(cuda_device)
        pm, _ = fo.segment_packbits(flat.to(cuda_device), ind, bitorder="little")
        w.plan(dev(qo, cuda_device), dev(kv, cuda_device), H, Hkv, D, packed_custom_mask=pm, q_data_type=dtype)
    else:
        w.plan(dev(qo, cuda_device), dev(kv, cuda_device), H, Hkv, D, custom_mask=flat.to(cuda_device), q_data_type=dtype)
    si, skv, ip, kp = masks_to_device(m, cuda_device)
    for _ in range(2):
        o, lse = w.run(dev(q, cuda_device), dev(k, cuda_device), dev(v, cuda_device), si, skv, ip, kp,
                       out=dev(prior, cuda_device).clone(), return_lse=True)
    w.check_status()
    ref, ref_lse = oa.sparse_attention(q, k, v, qo, kv, m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr,
                                       out_prior=prior, return_lse=True, custom_mask=cms)
    assert_close_bf16(o.cpu(), ref, f"custom mask H={H}/{Hkv} D={D} {dtype}")
    act = torch.zeros(int(qo[-1]), H, dtype=torch.bool)
    for b in range(len(lens_q)):
        for qb in range(qa[b].shape[0]):
            r0 = int(qo[b]) + qb * qt
            r1 = min(r0 + qt, int(qo[b + 1]))
            for hk in range(Hkv):
                if qa[b][qb, hk]:
                    act[r0:r1, hk * g:(hk + 1) * g] = True
                else:
                    assert torch.equal(o[r0:r1, hk * g:(hk + 1) * g].cpu(), prior[r0:r1, hk * g:(hk + 1) * g])
    assert torch.allclose(lse.cpu()[act], ref_lse[act], atol=2e-2, rtol=1e-3)
    assert (ref_lse[act] == -5e4).any()


@pytest.mark.parametrize("seed", range(24))
def test_random_configurations_against_the_oracle(cuda_device, seed):
    """Seeded random draws over everything the wrapper takes at once: heads and grouping, head dimension, dtype, kv
    layout, causal mask, soft cap, lse, batch, ragged q and kv lengths (empty requests included), mask densities
    (rows that keep nothing included), prior contents of the output."""
    rng = np.random.default_rng(1000 + seed)
    g = int(rng.choice([1, 1, 2, 4]))
    Hkv = int(rng.integers(1, 4))
    H, D = Hkv * g, int(rng.choice([128, 128, 64]))
    if seed >= 16:   # the last eight draws run head dimension 256
        D = 256
    dtype = torch.bfloat16 if rng.random() < 0.6 else torch.float16
    causal = bool(rng.random() < 0.35)
    soft_cap = float(rng.choice([0.0, 0.0, 20.0]))
    layout = "HND" if rng.random() < 0.3 else "NHD"
    B = int(rng.integers(1, 4))
    lens_q = [int(rng.integers(0, 420)) for _ in range(B)]
    lens_kv = [int(rng.integers(1, 520)) if lq > 0 else int(rng.integers(0, 200)) for lq in lens_q]
    if sum(lens_q) == 0:
        lens_q[0], lens_kv[0] = 130, 257
    qt = 128 // g
    qo = np.concatenate([[0], np.cumsum(lens_q)]).astype(np.int32)
    kv = np.concatenate([[0], np.cumsum(lens_kv)]).astype(np.int32)
    dq, dk = float(rng.uniform(0.3, 1.0)), float(rng.uniform(0.1, 1.0))
    qa = [(rng.random((-(-a // qt), Hkv)) < dq).astype(np.uint8) for a in lens_q]
    kk = [(rng.random((-(-a // qt), Hkv, -(-b // 128))) < dk).astype(np.uint8) for a, b in zip(lens_q, lens_kv)]
    m = wl.pack_masks(qa, kk)
    Tq, Tkv = int(qo[-1]), max(int(kv[-1]), 1)
    q = wl.randn_bf16((Tq, H, D), 2000 + seed, dtype=dtype)
    k = wl.randn_bf16((Tkv, Hkv, D), 3000 + seed, dtype=dtype)
    v = wl.randn_bf16((Tkv, Hkv, D), 4000 + seed, dtype=dtype)
    prior = wl.randn_bf16((Tq, H, D), 5000 + seed, dtype=dtype)
    w = fo.BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1 << 20, dtype=torch.uint8, device=cuda_device), layout)
    cms, flat = None, None
    if seed % 4 == 3:   # every fourth draw: a custom element mask (it takes the place of `causal`)
        cms = [rng.random((a, b)) < 0.6 for a, b in zip(lens_q, lens_kv)]
        flat = torch.from_numpy(np.concatenate([c.reshape(-1) for c in cms] + [np.zeros(0, dtype=bool)])).to(cuda_device)
        causal = False
    w.plan(dev(qo, cuda_device), dev(kv, cuda_device), H, Hkv, D, causal=causal, q_data_type=dtype, custom_mask=flat,
           logits_soft_cap=soft_cap if soft_cap > 0 else None)
    si, skv, ip, kp = masks_to_device(m, cuda_device)
    kd, vd = dev(k, cuda_device), dev(v, cuda_device)
    if layout == "HND":
        kd, vd = kd.transpose(0, 1).contiguous(), vd.transpose(0, 1).contiguous()
    o, lse = w.run(dev(q, cuda_device), kd, vd, si, skv, ip, kp, out=dev(prior, cuda_device).clone(), return_lse=True)
    w.check_status()
    ref, ref_lse = oa.sparse_attention(q, k, v, qo, kv, m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr,
                                       out_prior=prior, return_lse=True, logits_soft_cap=soft_cap, causal=causal,
                                       custom_mask=cms)
    what = f"seed {seed}: H={H}/{Hkv} D={D} {dtype} causal={causal} cap={soft_cap} {layout} q={lens_q} kv={lens_kv}"
    assert_close_bf16(o.cpu(), ref, what)
    act = torch.zeros(Tq, H, dtype=torch.bool)
    for b in range(B):
        for qb in range(qa[b].shape[0]):
            r0 = int(qo[b]) + qb * qt
            r1 = min(r0 + qt, int(qo[b + 1]))
            for hk in range(Hkv):
                if qa[b][qb, hk]:
                    act[r0:r1, hk * g:(hk + 1) * g] = True
    assert torch.equal(o.cpu()[~act], prior[~act]), what
    assert torch.allclose(lse.cpu()[act], ref_lse[act], atol=2e-2, rtol=1e-3), what


@pytest.mark.parametrize("fp8", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("dtype,layout", [(torch.bfloat16, "NHD"), (torch.float16, "HND")])
def test_fp8_kv_is_cast_to_the_type_of_q(cuda_device, fp8, dtype, layout):
    """K / V stored as 8-bit floats: the cast is exact (every value of both formats, bit for bit against torch, with
    a ragged tail), and the attention equals the oracle on the same values in fp32."""
    codes = torch.arange(256, dtype=torch.uint8).repeat(3)[:256 * 3 - 5].to(cuda_device)
    nan = codes.view(fp8).float().isnan()
    got = fo.attention._cast_fp8(codes.view(fp8), dtype)
    want = codes.view(fp8).to(dtype)
    assert torch.equal(got[~nan].view(torch.int16), want[~nan].view(torch.int16))
    assert bool(got[nan].isnan().all())

    H, seq = 2, 512
    inp = wl.attention_inputs(1, H, seq, 128, 0.6, seed=77, dtype=dtype)
    k8, v8 = inp.k.to(fp8), inp.v.to(fp8)
    w = fo.BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1 << 20, dtype=torch.uint8, device=cuda_device), layout)
    w.plan(dev(inp.qo_indptr.numpy(), cuda_device), dev(inp.kv_indptr.numpy(), cuda_device), H, H, 128,
           q_data_type=dtype, kv_data_type=fp8)
    kd, vd = dev(k8, cuda_device), dev(v8, cuda_device)
    if layout == "HND":
        kd, vd = kd.transpose(0, 1).contiguous(), vd.transpose(0, 1).contiguous()
    si, skv, ip, kp = masks_to_device(inp.masks, cuda_device)
    o = w.run(dev(inp.q, cuda_device), kd, vd, si, skv, ip, kp)
    w.check_status()
    m = inp.masks
    ref = oa.sparse_attention(inp.q, k8.float(), v8.float(), inp.qo_indptr.numpy(), inp.kv_indptr.numpy(),
                              m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr)
    assert_close_bf16(o, ref, f"fp8 kv {fp8} {dtype} {layout}")
    with pytest.raises(ValueError):
        w.run(dev(inp.q, cuda_device), kd.to(dtype), vd.to(dtype), si, skv, ip, kp)


def test_undersized_kept_list_is_reported_not_walked(cuda_device):
    """A C-ABI caller that compacts with a kv_idx capacity below the kept count: the compaction records it, and
    the attention launch that follows touches neither the lists nor the output and reports FO_DEV_BAD_INDEX."""
    from flashomni_b200 import _native
    H, S = 2, 512
    inp = wl.attention_inputs(1, H, S, 128, 1.0, seed=77)
    w = _wrapper(cuda_device, inp.qo_indptr, inp.kv_indptr, H)
    lib = _native.load()
    si, skv, ip, kp = masks_to_device(inp.masks, cuda_device)
    ws = w._ws
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    small = 3   # 2 heads x 4 q-blocks x 4 kept blocks = 32 entries are needed
    rc = lib.fo_mask_compact(_native.ptr(si), si.numel(), _native.ptr(skv), skv.numel(), _native.ptr(ip), _native.ptr(kp),
                             _native.ptr(w._qo_indptr_buf), _native.ptr(w._kv_indptr_buf), 1, H, 0, H, 128, 128, 0,
                             w._n_cand, w._max_nkv, w._n_cand, small, _native.ptr(ws["items"]), _native.ptr(ws["kv_ptr"]),
                             _native.ptr(ws["kv_idx"]), _native.ptr(ws["order"]), _native.ptr(ws["counters"]),
                             _native.ptr(ws["scratch"]), w._scratch_bytes, stream)
    _native.check(rc, "fo_mask_compact")
    rc = lib.fo_attn_units(_native.ptr(ws["items"]), _native.ptr(ws["kv_ptr"]), _native.ptr(ws["kv_idx"]),
                           _native.ptr(ws["order"]), _native.ptr(ws["counters"]), _native.ptr(w._qo_indptr_buf),
                           _native.ptr(w._kv_indptr_buf), w._n_cand, w._max_nkv, 128, 128, w._min_items, w._num_streams, w.MIN_CHUNK,
                           w._max_units, w._partial_slots, _native.ptr(ws["units"]), _native.ptr(ws["unit_counters"]),
                           _native.ptr(ws["arrive"]), stream)
    _native.check(rc, "fo_attn_units")
    q, k, v = (dev(t, cuda_device) for t in (inp.q, inp.k, inp.v))
    prior = dev(wl.randn_bf16(inp.q.shape, 5), cuda_device)
    out = prior.clone()
    rc = lib.fo_sparse_attn_fwd(_native.ptr(q), _native.ptr(k), _native.ptr(v), _native.ptr(out), None, _native.FO_DTYPE_BF16,
                                S, S, H, H, 128, q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1),
                                out.stride(0), out.stride(1), 128, 128, _native.ptr(ws["kv_idx"]),
                                _native.ptr(ws["units"]), _native.ptr(ws["unit_counters"]), w._max_units,
                                _native.ptr(ws["arrive"]), _native.ptr(w._partials), w._partial_slots, 0, 128 ** -0.5,
                                _native.ptr(ws["status"]), stream)
    _native.check(rc, "fo_sparse_attn_fwd")
    torch.cuda.synchronize()
    words = w._ws_words[:12].cpu().tolist()
    assert words[2] == _native.FO_DEV_BAD_INDEX          # the compaction's own status
    assert words[11] == _native.FO_DEV_BAD_INDEX         # the unit builder passes it on
    assert words[4] == _native.FO_DEV_BAD_INDEX          # the attention launch's status word
    assert words[5] == 0 and words[6] == 0               # cursor and arrival count are back at zero
    assert torch.equal(out, prior)
    # the same wrapper is usable again once the lists fit
    w._ws_words[4:8].zero_()
    o = w.run(q, k, v, si, skv, ip, kp)
    w.check_status()
    ref = oa.sparse_attention(inp.q, inp.k, inp.v, [0, S], [0, S], inp.masks.sparse_info, inp.masks.sparse_kv_info,
                              inp.masks.info_indptr, inp.masks.kv_info_indptr)
    assert_close_bf16(o, ref, "attention after an undersized list")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_split_kv_lists_merge_to_the_oracle(cuda_device, dtype, attention_kernel_choice, monkeypatch):
    """Few items with long kv lists: the lists are cut into parts that run on different streams, and the part that
    delivers last merges the partial results (maxima, sums, fp32 O). Against the fp32 oracle, with the log-sum-exp,
    prior contents for skipped q-blocks, an empty item and a ragged last block; twice in a row on the same wrapper
    (the per-item arrival counters must be back at zero)."""
    monkeypatch.setattr(fo.BatchFlashOmniFAWithRaggedKVWrapper, "UNITS_PER_SM", 2)
    H, lens = 4, [40 * 128, 17 * 128 + 40]       # about 185 items: more than one per SM, fewer than two
    rng = np.random.default_rng(61)
    qa = [(rng.random((-(-n // 128), H)) < 0.8).astype(np.uint8) for n in lens]
    kk = [(rng.random((-(-n // 128), H, -(-n // 128))) < 0.8).astype(np.uint8) * a[:, :, None] for n, a in zip(lens, qa)]
    qa[0][3, 1] = 1; kk[0][3, 1, :] = 0            # an active q-block that keeps nothing
    qa[1][17, 2] = 1; kk[1][17, 2, :] = 1          # the ragged last q-block against every kv block (ragged last one too)
    m = wl.pack_masks(qa, kk)
    T = sum(lens)
    q, k, v = (wl.randn_bf16((T, H, 128), 62 + i, dtype=dtype) for i in range(3))
    qo = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    w = _wrapper(cuda_device, qo, qo, H, dtype)
    prior = wl.randn_bf16(q.shape, 70, dtype=dtype)
    ref, ref_lse = oa.sparse_attention(q, k, v, qo, qo, m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr,
                                       out_prior=prior, return_lse=True)
    for _ in range(2):
        o, lse = _run(cuda_device, w, q, k, v, m, out=dev(prior, cuda_device).clone(), return_lse=True)
        lists = w.work_lists()
        assert lists["partial_slots_used"] > 0 and lists["n_units"] > lists["n_items"]
        assert_close_bf16(o, ref, f"split attention {dtype}")
        act = torch.zeros(T, H, dtype=torch.bool)
        for b, n in enumerate(lens):
            for qb in range(-(-n // 128)):
                for h in range(H):
                    if qa[b][qb, h]:
                        act[qo[b] + qb * 128: min(qo[b] + (qb + 1) * 128, qo[b + 1]), h] = True
        assert torch.allclose(lse.cpu()[act], ref_lse[act], atol=2e-2, rtol=1e-3)
        assert torch.equal(o.cpu()[~act], prior[~act])


@pytest.mark.parametrize("heads", [6, 3])
def test_split_kv_a_share_of_the_heads_of_the_4608_token_layer(cuda_device, heads, monkeypatch):
    """A rank's share of the 4608-token layer, two requests, with list cutting switched on (up to four units per SM).
    Six heads (24 heads over 4 GPUs): about 240 items for 148 SMs, so the lists are cut; three heads (over 8 GPUs):
    about 120 items, at most one per SM, nothing is cut."""
    monkeypatch.setattr(fo.BatchFlashOmniFAWithRaggedKVWrapper, "UNITS_PER_SM", 4)
    inp = wl.attention_inputs(2, heads, 4608, 128, 0.5, seed=91)
    w = _wrapper(cuda_device, inp.qo_indptr, inp.kv_indptr, heads)
    o = _run(cuda_device, w, inp.q, inp.k, inp.v, inp.masks)
    lists = w.work_lists()
    sms = torch.cuda.get_device_properties(cuda_device).multi_processor_count
    assert (lists["partial_slots_used"] > 0) == (sms < lists["n_items"] <= 4 * sms)
    assert (lists["partial_slots_used"] > 0) == (heads == 6) or sms != 148
    m = inp.masks
    ref = oa.sparse_attention(inp.q, inp.k, inp.v, [0, 4608, 9216], [0, 4608, 9216], m.sparse_info, m.sparse_kv_info,
                              m.info_indptr, m.kv_info_indptr)
    assert_close_bf16(o, ref, f"{heads} heads of the 4608-token layer")


def test_split_rule_follows_the_planned_shape(cuda_device, monkeypatch):
    """By default no list is ever cut and no scratch is set aside. With cutting switched on: room for partial
    results when the launch has between one and UNITS_PER_SM candidate items per SM."""
    monkeypatch.setattr(fo.BatchFlashOmniFAWithRaggedKVWrapper, "FORCE_SPLIT", False)
    few = _wrapper(cuda_device, [0, 4608, 9216], [0, 4608, 9216], 3)      # 216 candidates
    assert few._partial_slots == 0 and few._max_units == few._n_cand and few._partials is None
    monkeypatch.setattr(fo.BatchFlashOmniFAWithRaggedKVWrapper, "UNITS_PER_SM", 2)
    streams = 2 * torch.cuda.get_device_properties(cuda_device).multi_processor_count
    few = _wrapper(cuda_device, [0, 4608, 9216], [0, 4608, 9216], 3)
    many = _wrapper(cuda_device, [0, 4608, 9216], [0, 4608, 9216], 24)    # 1728 candidates
    one_per_sm = _wrapper(cuda_device, [0, 4608], [0, 4608], 3)           # 108 candidates
    assert streams // 2 < few._n_cand <= streams < many._n_cand
    assert few._partial_slots > 0 and few._max_units == few._n_cand + streams
    assert many._partial_slots == 0 and many._max_units == many._n_cand and many._partials is None
    assert one_per_sm._partial_slots == 0
