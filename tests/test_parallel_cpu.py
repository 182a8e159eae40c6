"""CPU, world_size 2 over gloo: the host-side logic of the two multi-GPU schemes."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashomni_b200 import parallel as par
from flashomni_b200 import workloads as wl
from oracle import attention as oa
from oracle import gemm as og


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_block_sharding():
    assert par.shard_blocks(604, 8) == [76] * 4 + [75] * 4
    assert par.shard_blocks(604, 2) == [302, 302]
    assert par.token_range(77312, 7, 8) == (77312 - 75 * 128, 77312)
    assert par.token_range(300, 1, 2) == (256, 300)          # ragged tail stays with the last block
    assert par.head_window(24, 3, 8) == (9, 3)
    with pytest.raises(ValueError):
        par.head_window(24, 0, 5)


def _ulysses_worker(rank, world, port, out_dict):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        S, H, D = 5 * 128 + 40, 4, 8
        g = torch.Generator().manual_seed(0)
        full = torch.randn(S, H, D, generator=g)
        a, b = par.token_range(S, rank, world)
        mine = par.tokens_to_heads(full[a:b].contiguous(), S)
        hb, hc = par.head_window(H, rank, world)
        assert torch.equal(mine, full[:, hb:hb + hc])
        back = par.heads_to_tokens(mine, S)
        assert torch.equal(back, full[a:b])
        out_dict[rank] = True
    finally:
        dist.destroy_process_group()


def test_ulysses_exchange_roundtrip_gloo():
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_ulysses_worker, args=(2, port, out), nprocs=2, join=True)
    assert out.get(0) and out.get(1)


def _head_partition_worker(rank, world, port, out_dict):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # the head-partitioned block on the oracle: partial outputs of the ranks sum to the full block
        B, H, nq, D, hid = 1, 4, 3, 16, 64
        S = nq * 128
        m = wl.flux_masks(B, H, nq, nq, 0.6, seed=5, text_blocks=1)
        g = torch.Generator().manual_seed(1)
        x = torch.randn(B, S, hid, generator=g)
        wq, wk, wv = (torch.randn(H * D, hid, generator=g) * hid ** -0.5 for _ in range(3))
        wo = torch.randn(hid, H * D, generator=g) * (H * D) ** -0.5
        indptr = [0, S]

        def block(hb, hc):
            sl = slice(hb * D, (hb + hc) * D)
            q = og.gemm_q(x, wq[sl], H, m.sparse_info, m.info_indptr, 0, head_begin=hb, head_dim=D)
            k = og.gemm_q(x, wk[sl], H, is_full=True)
            v = og.gemm_q(x, wv[sl], H, is_full=True)
            o = oa.sparse_attention(q.view(S, hc, D), k.view(S, hc, D), v.view(S, hc, D), indptr, indptr, m.sparse_info,
                                    m.sparse_kv_info, m.info_indptr, m.kv_info_indptr, head_begin=hb, num_mask_heads=H)
            return og.gemm_o(o.view(1, S, hc * D), wo[:, sl], H, m.sparse_info, m.info_indptr, 0, None, False,
                             head_begin=hb, head_dim=D)

        hb, hc = par.head_window(H, rank, world)
        part = block(hb, hc)
        dist.all_reduce(part)
        full = block(0, H)
        assert torch.allclose(part, full, atol=1e-4)
        out_dict[rank] = True
    finally:
        dist.destroy_process_group()


def test_head_partition_partials_sum_to_full_block_gloo():
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_head_partition_worker, args=(2, port, out), nprocs=2, join=True)
    assert out.get(0) and out.get(1)
