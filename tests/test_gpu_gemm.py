"""GPU: GEMM-Q and GEMM-O through the public API against the fp32 oracle."""

import pytest
import torch

import flashomni_b200 as fo
from flashomni_b200 import workloads as wl
from oracle import gemm as og
from helpers import assert_close_bf16, dev, masks_to_device

pytestmark = pytest.mark.gpu


def _status_ok():
    from flashomni_b200 import gemm as g
    for ws in g._workspaces.values():
        w = ws[:32].view(torch.int32).cpu()
        assert int(w[2]) == 0 and int(w[4]) == 0, f"device status {w.tolist()}"


@pytest.mark.parametrize("shape", [(1, 128, 128, 64), (1, 256, 384, 256), (2, 512, 512, 1024), (1, 128, 256, 3072),
                                   (1, 384, 512, 192), (3, 640, 256, 320), (2, 128, 768, 64),
                                   (1, 256, 256, 96), (2, 128, 384, 32), (1, 512, 512, 288),    # K = 32 mod 64 too
                                   (2, 512, 768, 256), (1, 256, 1152, 128), (2, 1280, 1536, 192)])  # 192-column tiles
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_dense_gemm_is_full(cuda_device, shape, dtype):
    B, M, N, K = shape
    x = wl.randn_bf16((B, M, K), 1, dtype=dtype); w = wl.randn_bf16((N, K), 2, std=K ** -0.5, dtype=dtype)
    bias = wl.randn_bf16((N,), 3, dtype=dtype)
    y = fo.flashomni_gemm(dev(x, cuda_device), dev(w, cuda_device), N // 128, bias=dev(bias, cuda_device), is_full=True)
    ref = og.gemm_q(x, w, N // 128, bias=bias, is_full=True)
    _status_ok()
    assert_close_bf16(y, ref, f"dense gemm {shape} {dtype}", allow_ulp=1.0)


@pytest.mark.parametrize("density", [0.25, 0.5, 0.75])
def test_gemm_q_sparse_small(cuda_device, density):
    B, H, nq, K = 2, 4, 6, 512
    m = wl.flux_masks(B, H, nq, nq, density, seed=31, text_blocks=1)
    si, _, ip, _ = masks_to_device(m, cuda_device)
    x = wl.randn_bf16((B, nq * 128, K), 4); w = wl.randn_bf16((H * 128, K), 5, std=K ** -0.5)
    prior = wl.randn_bf16((B, nq * 128, H * 128), 6); bias = wl.randn_bf16((H * 128,), 7)
    out = dev(prior, cuda_device).clone()
    y = fo.flashomni_gemm(dev(x, cuda_device), dev(w, cuda_device), H, si, ip, 0, dev(bias, cuda_device), out=out)
    assert y.data_ptr() == out.data_ptr()
    ref = og.gemm_q(x, w, H, m.sparse_info, m.info_indptr, 0, bias, prior)
    _status_ok()
    assert_close_bf16(y, ref, "gemm_q", allow_ulp=1.0)
    # inactive tiles are never written: bit-identical to the prior contents
    yc = y.cpu()
    for b in range(B):
        for iy in range(nq):
            for h in range(H):
                if not m.q_active[b][iy, h]:
                    blk = (b, slice(iy * 128, iy * 128 + 128), slice(h * 128, h * 128 + 128))
                    assert torch.equal(yc[blk], prior[blk])


def test_gemm_q_row_offset_and_head_window(cuda_device):
    B, H, nq, K = 1, 6, 8, 256
    m = wl.flux_masks(B, H, nq, nq, 0.5, seed=32, text_blocks=2)
    si, _, ip, _ = masks_to_device(m, cuda_device)
    rows = (nq - 2) * 128
    x = wl.randn_bf16((B, rows, K), 8); w = wl.randn_bf16((2 * 128, K), 9, std=K ** -0.5)
    prior = wl.randn_bf16((B, rows, 256), 10)
    y = fo.flashomni_gemm(dev(x, cuda_device), dev(w, cuda_device), H, si, ip, 256, out=dev(prior, cuda_device).clone(),
                          head_begin=3, head_dim=128)
    ref = og.gemm_q(x, w, H, m.sparse_info, m.info_indptr, 256, None, prior, head_begin=3, head_dim=128)
    _status_ok()
    assert_close_bf16(y, ref, "gemm_q window", allow_ulp=1.0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_o_both_polarities_and_identity(cuda_device, dtype):
    B, H, nq, N = 2, 6, 5, 384
    K = H * 128
    m = wl.flux_masks(B, H, nq, nq, 0.5, seed=33, text_blocks=1)
    m.q_active[0][2, :] = 0  # a row block with no active head
    m.q_active[1][3, :] = 1  # and one with every head active
    m = wl.pack_masks(m.q_active, m.kv_kept)
    si, _, ip, _ = masks_to_device(m, cuda_device)
    x = wl.randn_bf16((B, nq * 128, K), 11, dtype=dtype); w = wl.randn_bf16((N, K), 12, std=K ** -0.5, dtype=dtype)
    bias = wl.randn_bf16((N,), 13, dtype=dtype)
    xd, wd = dev(x, cuda_device), dev(w, cuda_device)
    cache = fo.flashomni_gemm_reduction(xd, wd, H, si, ip, 0, dev(bias, cuda_device), is_for_cache=True, head_dim=128)
    ref_cache = og.gemm_o(x, w, H, m.sparse_info, m.info_indptr, 0, bias, True, head_dim=128)
    _status_ok()
    assert_close_bf16(cache, ref_cache, "gemm_o cache pass", allow_ulp=1.0)
    y = fo.flashomni_gemm_reduction(xd, wd, H, si, ip, 0, cache, is_for_cache=False, head_dim=128)
    ref_y = og.gemm_o(x, w, H, m.sparse_info, m.info_indptr, 0, cache.cpu(), False, head_dim=128)
    _status_ok()
    assert_close_bf16(y, ref_y, "gemm_o active pass", allow_ulp=1.0)
    # the reference's own check (benchmark/test_flashomni_gemm_o.py:73-87): cache pass + active pass == dense
    dense = x.float() @ w.float().T + bias.float()
    assert_close_bf16(y, dense, "gemm_o identity", max_abs=4e-2, mean_abs=4e-3, allow_ulp=2.0)
    # no bias at all
    y0 = fo.flashomni_gemm_reduction(xd, wd, H, si, ip, 0, None, is_for_cache=False, head_dim=128)
    assert_close_bf16(y0, og.gemm_o(x, w, H, m.sparse_info, m.info_indptr, 0, None, False, head_dim=128), "gemm_o no init",
                      allow_ulp=1.0)


def test_gemm_full_size_config(cuda_device):
    """Config-2/3 sizes: X [1,4608,3072], W [3072,3072], density 0.5; compared against torch fp32 on the
    GPU (the CPU oracle at this size takes too long for the suite; it covers the small cases above)."""
    B, H, nq = 1, 24, 36
    m = wl.flux_masks(B, H, nq, nq, 0.5, seed=34)
    si, _, ip, _ = masks_to_device(m, cuda_device)
    x = dev(wl.randn_bf16((B, 4608, 3072), 14), cuda_device); w = dev(wl.randn_bf16((3072, 3072), 15, std=3072 ** -0.5), cuda_device)
    prior = dev(wl.randn_bf16((B, 4608, 3072), 16), cuda_device)
    y = fo.flashomni_gemm(x, w, H, si, ip, 0, out=prior.clone())
    dense = (x.float() @ w.float().T)
    qa = torch.from_numpy(m.q_active[0]).to(cuda_device).bool()  # [nq, H]
    tile_mask = qa.repeat_interleave(128, 0).repeat_interleave(128, 1)[None]
    ref = torch.where(tile_mask, dense, prior.float())
    _status_ok()
    assert torch.equal(y[~tile_mask.expand_as(y)], prior[~tile_mask.expand_as(y)])
    assert_close_bf16(y, ref, "gemm_q 4608x3072x3072", allow_ulp=1.0)
    # GEMM-O: linearity property  cache pass + active pass == dense
    cache = fo.flashomni_gemm_reduction(x, w, H, si, ip, 0, None, is_for_cache=True)
    yo = fo.flashomni_gemm_reduction(x, w, H, si, ip, 0, cache, is_for_cache=False)
    _status_ok()
    assert_close_bf16(yo, dense, "gemm_o identity 4608", max_abs=4e-2, mean_abs=4e-3, allow_ulp=2.0)
    heads_active = qa.repeat_interleave(128, 0).float()  # [M, H]
    xs = x.float().view(4608, H, 128) * heads_active[:, :, None]
    ref_active = xs.view(1, 4608, 3072) @ w.float().T
    y_act = fo.flashomni_gemm_reduction(x, w, H, si, ip, 0, None, is_for_cache=False)
    assert_close_bf16(y_act, ref_active, "gemm_o active heads 4608", allow_ulp=1.0)


def test_prepared_worklists_give_the_same_result(cuda_device):
    """flashomni_gemm / flashomni_gemm_reduction over lists built earlier on a side stream (extension)."""
    from flashomni_b200.gemm import prepare_gemm_o_list, prepare_gemm_q_list
    B, H, S, hid = 2, 6, 1024, 768
    m = wl.flux_masks(B, H, S // 128, S // 128, 0.5, seed=61, text_blocks=1)
    si, _, ip, _ = masks_to_device(m, cuda_device)
    x = dev(wl.randn_bf16((B, S, hid), 62), cuda_device)
    w = dev(wl.randn_bf16((hid, hid), 63, std=hid ** -0.5), cuda_device)
    cache = dev(wl.randn_bf16((B, S, hid), 64), cuda_device)
    prior = dev(wl.randn_bf16((B, S, hid), 65), cuda_device)
    side = torch.cuda.Stream(cuda_device)
    side.wait_stream(torch.cuda.current_stream(cuda_device))
    ql = prepare_gemm_q_list(B, S, hid, H, si, ip, 0, stream=side)
    ol = prepare_gemm_o_list(B, S, hid, H, si, ip, 0, stream=side)
    for _ in range(2):  # the second round re-uses the lists
        a = fo.flashomni_gemm(x, w, H, si, ip, 0, out=prior.clone())
        b = fo.flashomni_gemm(x, w, H, None, None, 0, out=prior.clone(), worklist=ql)
        assert torch.equal(a, b)
        c = fo.flashomni_gemm_reduction(x, w, H, si, ip, 0, cache)
        d = fo.flashomni_gemm_reduction(x, w, H, None, None, 0, cache, worklist=ol)
        assert torch.equal(c, d)
    ql2 = prepare_gemm_q_list(B, S, hid, H, si, ip, 0, into=ql)
    assert ql2 is ql
    with pytest.raises(ValueError):
        fo.flashomni_gemm_reduction(x, w, H, None, None, 0, cache, worklist=ql)
