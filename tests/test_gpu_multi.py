"""Two GPUs, NCCL: the sequence-parallel (Ulysses) block gives the rows the single-GPU block gives.

Skipped on a box with fewer than two GPUs. Each rank is a child process; a rank only leaves between
steps, with none of its kernels or collectives in flight."""

import os
import socket

import pytest
import torch

from flashomni_b200 import workloads as wl

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
        blk.wrapper.check_status()
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
    for r in range(world):
        t0, t1, y = out[r]
        # same kernels on the same rows; only the order of the kv blocks inside an item's sum may differ
        assert torch.allclose(y[0], ref[0, t0:t1], atol=2e-2, rtol=0), f"rank {r}"
        assert (y[0] - ref[0, t0:t1]).abs().mean().item() < 2e-3
