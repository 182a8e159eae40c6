"""Multi-GPU paths. Two GPUs (skipped on a box with fewer; each rank is a child process that only leaves between
steps, with none of its kernels or collectives in flight): the sequence-parallel (Ulysses) block and the
head-partitioned block with its cross-rank sum, both against the CPU oracle. One GPU: the row reduction with all
sources local, and the peer barrier's bounded wait (a peer that never arrives gives an error status, not a hang)."""

import os
import socket

import pytest
import torch

from flashomni_b200 import workloads as wl
from helpers import assert_close_bf16

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _case():
    H, S, hid = 4, 12 * 128, 512
    m = wl.flux_masks(1, H, S // 128, S // 128, 0.5, seed=41, text_blocks=1)
    ws = [wl.randn_bf16((hid, hid), 50 + i, std=hid ** -0.5) for i in range(4)]
    x = wl.randn_bf16((1, S, hid), 60)
    cache = wl.randn_bf16((1, S, hid), 61)
    return H, S, hid, m, ws, x, cache


def _oracle_block(H, S, hid, m, ws, x, cache):
    """The block on the CPU oracle, every intermediate rounded to bf16 as the kernels store it."""
    from oracle import attention as oa
    from oracle import gemm as og
    wq, wk, wv, wo = ws
    bf = torch.bfloat16
    q = og.gemm_q(x, wq, H, m.sparse_info, m.info_indptr, 0).to(bf)
    k = og.gemm_q(x, wk, H, is_full=True).to(bf)
    v = og.gemm_q(x, wv, H, is_full=True).to(bf)
    o = oa.sparse_attention(q.view(S, H, 128), k.view(S, H, 128), v.view(S, H, 128), [0, S], [0, S], m.sparse_info,
                            m.sparse_kv_info, m.info_indptr, m.kv_info_indptr).to(bf)
    return og.gemm_o(o.view(1, S, H * 128), wo, H, m.sparse_info, m.info_indptr, 0, cache, False)


def _worker(rank, world, port, out_dict, exchange):
    import torch.distributed as dist
    from flashomni_b200.layer import BlockWeights, UlyssesSparseDiTAttentionBlock
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        H, S, hid, m, ws, x, cache = _case()
        blk = UlyssesSparseDiTAttentionBlock(BlockWeights(*(w.to(device) for w in ws)), H, 128, S, rank, world, device,
                                             exchange=exchange)
        assert blk.exchange == exchange, getattr(blk.px, "reason", "")
        blk.cache.copy_(cache[:, blk.t0:blk.t1].to(device))
        masks = [torch.from_numpy(a).to(device) for a in (m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr)]
        xl = x[:, blk.t0:blk.t1].contiguous().to(device)
        for _ in range(2):  # the second step reuses every buffer of the first
            y = blk.forward(xl, *masks)
        torch.cuda.synchronize()
        blk.check_status()
        out_dict[rank] = (blk.t0, blk.t1, y.float().cpu())
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["p2p", "nccl"])
def test_ulysses_block_matches_single_gpu(exchange):
    """p2p: pulls over peer memory (fo_strided_gather); nccl: all_to_all_single on a side stream."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from flashomni_b200.layer import BlockWeights, SparseDiTAttentionBlock
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out, exchange), nprocs=world, join=True)
    H, S, hid, m, ws, x, cache = _case()
    device = torch.device("cuda", 0)
    blk = SparseDiTAttentionBlock(BlockWeights(*(w.to(device) for w in ws)), H, 128, 1, S, device=device)
    blk.cache.copy_(cache.to(device))
    masks = [torch.from_numpy(a).to(device) for a in (m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr)]
    ref = blk.forward(x.to(device), *masks).float().cpu()
    oracle = _oracle_block(H, S, hid, m, ws, x, cache)
    for r in range(world):
        t0, t1, y = out[r]
        # same kernels on the same rows; only the order of the kv blocks inside an item's sum may differ
        assert torch.allclose(y[0], ref[0, t0:t1], atol=2e-2, rtol=0), f"rank {r}"
        assert (y[0] - ref[0, t0:t1]).abs().mean().item() < 2e-3
        assert_close_bf16(y[0], oracle[0, t0:t1], f"rank {r} vs the oracle", allow_ulp=1.0)


def _head_worker(rank, world, port, out_dict):
    import torch.distributed as dist
    from flashomni_b200 import parallel as par
    from flashomni_b200.layer import BlockWeights, SparseDiTAttentionBlock
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        H, S, hid, m, ws, x, cache = _case()
        hb, hc = par.head_window(H, rank, world)
        sl = slice(hb * 128, (hb + hc) * 128)
        wts = BlockWeights(ws[0][sl].contiguous().to(device), ws[1][sl].contiguous().to(device),
                           ws[2][sl].contiguous().to(device), ws[3][:, sl].contiguous().to(device))
        blk = SparseDiTAttentionBlock(wts, H, 128, 1, S, hb, hc, device=device, add_cache=False)
        masks = [torch.from_numpy(a).to(device) for a in (m.sparse_info, m.sparse_kv_info, m.info_indptr, m.kv_info_indptr)]
        px = par.PeerExchange(None, device)
        assert px.available, getattr(px, "reason", "")
        part, ptrs, _h = px.alloc((S, hid), torch.bfloat16)
        rows = S // world
        mine = torch.empty((rows, hid), dtype=torch.bfloat16, device=device)
        cache_rows = cache[0, rank * rows:(rank + 1) * rows].contiguous().to(device)
        for it in range(2):   # twice: the second round re-uses the flag pads and the partial buffer
            blk.forward(x.to(device), *masks, out=part.view(1, S, hid))
            px.barrier(0)
            px.reduce_rows(ptrs, rank * rows, rows, hid, torch.bfloat16, mine, init=cache_rows)
            px.barrier(1)     # nobody overwrites its partial while a peer still reads it
        torch.cuda.synchronize()
        blk.wrapper.check_status()
        px.check_status()
        out_dict[rank] = mine.float().cpu()
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_head_partition_sum_matches_oracle():
    """Each rank runs its heads' share of the block (no cache), the partials are summed with the cache by
    fo_reduce_rows over peer memory behind fo_peer_barrier, and the rows each rank owns equal the oracle's block."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_head_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    H, S, hid, m, ws, x, cache = _case()
    oracle = _oracle_block(H, S, hid, m, ws, x, cache)
    rows = S // world
    for r in range(world):
        assert_close_bf16(out[r], oracle[0, r * rows:(r + 1) * rows], f"rank {r} rows vs the oracle", allow_ulp=1.0)


def test_reduce_rows_local_sources(cuda_device):
    """fo_reduce_rows with every source in local memory: init + sum of the sources, fp32 accumulation."""
    import ctypes
    from flashomni_b200 import _native
    lib = _native.load()
    rows, cols, n = 300, 384, 5
    srcs = [wl.randn_bf16((rows + 7, cols), 70 + i).to(cuda_device) for i in range(n)]
    init = wl.randn_bf16((rows, cols), 80).to(cuda_device)
    out = torch.empty((rows, cols), dtype=torch.bfloat16, device=cuda_device)
    ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() + 3 * cols * 2 for t in srcs])   # rows [3, 3 + rows) of every source
    rc = lib.fo_reduce_rows(n, ptrs, cols * 2, init.data_ptr(), cols * 2, out.data_ptr(), cols * 2, rows, cols * 2,
                            _native.FO_DTYPE_BF16, torch.cuda.current_stream(cuda_device).cuda_stream)
    _native.check(rc, "fo_reduce_rows")
    ref = init.float()
    for t in srcs:   # the kernel's order of additions
        ref = ref + t[3:3 + rows].float()
    assert torch.equal(out, ref.to(torch.bfloat16))
    rc = lib.fo_reduce_rows(n, ptrs, cols * 2, None, 0, out.data_ptr(), cols * 2, rows, cols * 2,
                            _native.FO_DTYPE_BF16, torch.cuda.current_stream(cuda_device).cuda_stream)
    _native.check(rc, "fo_reduce_rows")
    assert torch.equal(out, sum(t[3:3 + rows].float() for t in srcs).to(torch.bfloat16))
    assert lib.fo_reduce_rows(0, ptrs, cols * 2, None, 0, out.data_ptr(), cols * 2, rows, cols * 2, 1, None) \
        == _native.FO_ERR_INVALID_ARG


def test_peer_barrier_gives_up_with_a_status(cuda_device):
    """A barrier whose peer never arrives (a flag that nothing sets): the launch returns after its time limit with
    FO_DEV_WAIT_TIMEOUT in the status word, and the context stays usable. With the peer's arrival already in the
    pad the same launch passes."""
    import ctypes
    from flashomni_b200 import _native
    lib = _native.load()
    world, channels = 2, 4
    pads = [torch.zeros(channels * world, dtype=torch.int32, device=cuda_device) for _ in range(world)]
    epoch = torch.zeros(channels, dtype=torch.int32, device=cuda_device)
    status = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    arr = (ctypes.c_void_p * world)(*[p.data_ptr() for p in pads])
    st = torch.cuda.current_stream(cuda_device).cuda_stream
    rc = lib.fo_peer_barrier(world, 0, arr, 2, channels, epoch.data_ptr(), status.data_ptr(), 50, st)   # 50 ms
    _native.check(rc, "fo_peer_barrier")
    torch.cuda.synchronize()
    assert status[0].item() == _native.FO_DEV_WAIT_TIMEOUT
    assert epoch.tolist() == [0, 0, 1, 0]
    assert pads[1][2 * world + 0].item() == 1            # this rank's arrival was posted to the peer's pad
    # the peer "arrives": its flag for (channel 2, epoch 2) is in this rank's pad before the launch
    status.zero_()
    pads[0][2 * world + 1] = 2
    rc = lib.fo_peer_barrier(world, 0, arr, 2, channels, epoch.data_ptr(), status.data_ptr(), 50, st)
    _native.check(rc, "fo_peer_barrier")
    torch.cuda.synchronize()
    assert status[0].item() == _native.FO_DEV_OK and epoch.tolist() == [0, 0, 2, 0]
    x = torch.ones(8, device=cuda_device)
    assert x.sum().item() == 8.0
