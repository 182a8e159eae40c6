"""Host-side checks of the extensions (no GPU): argument validation, CPU refusal, list bookkeeping."""

import numpy as np
import pytest
import torch

import flashomni_b200 as fo
from flashomni_b200 import parallel as par
from flashomni_b200.gemm import GemmWorklist


def test_select_blocks_rejects_cpu_and_bad_shapes():
    s = torch.zeros(1, 2, 4, 4)
    with pytest.raises(RuntimeError):
        fo.select_blocks(s, 1, 0.2, 0.2)                      # no CPU path
    with pytest.raises(ValueError):
        fo.select_blocks(torch.zeros(1, 2, 4, 5), 1, 0.2, 0.2)  # nq != nkv
    with pytest.raises(ValueError):
        fo.select_blocks(s.double(), 1, 0.2, 0.2)


def test_exchange_row_counts_of_the_video_layer():
    """The pulls of the sequence-parallel exchange are built from these per-rank token ranges."""
    sizes = [par.token_range(77312, r, 8)[1] - par.token_range(77312, r, 8)[0] for r in range(8)]
    assert sizes == [9728] * 4 + [9600] * 4 and sum(sizes) == 77312


def test_worklist_key_check():
    wl = GemmWorklist("q", (2, 256, 512, 128, False), torch.zeros(256, dtype=torch.uint8))
    wl.check("q", 2, 256, 512, 128, torch.device("cpu"))
    with pytest.raises(ValueError):
        wl.check("o", 2, 256, 512, 128, torch.device("cpu"))
    with pytest.raises(ValueError):
        wl.check("q", 2, 256, 1024, 128, torch.device("cpu"))


def test_selection_statement_is_deterministic_across_layouts():
    from oracle import select as osel
    rng = np.random.default_rng(0)
    s = rng.standard_normal((1, 2, 9, 9)).astype(np.float32)
    a = osel.select_blocks(s, 2, 0.3, 0.3)
    b = osel.select_blocks(np.ascontiguousarray(s.transpose(0, 1, 3, 2)).transpose(0, 1, 3, 2), 2, 0.3, 0.3)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_block_schedule_name_is_checked_before_anything_else():
    from flashomni_b200.layer import SparseDiTAttentionBlock
    with pytest.raises(ValueError):
        SparseDiTAttentionBlock(None, 4, 128, 1, 256, schedule="o_first")


def test_dense_gemm_tile_choice_fills_whole_waves():
    """Host-only query of the dense dispatch on a 148-SM device: the launch goes to the tile shape whose fullest SM
    ends first: 256x256 tiles, 256x192 tiles where those fill the SMs better (the heads of the flux block split over
    two GPUs: 216 tiles of 256x256 are two rounds of length 2, 288 tiles of 256x192 two rounds of length 1.5), or
    the 128-row tiles of the other kernel."""
    from flashomni_b200 import _native
    lib = _native.load()
    q = lambda b, m, n, k, full=0, sms=148: lib.fo_gemm_dense_tile_rows(b, m, n, k, full, sms)
    assert q(2, 4608, 3072, 3072) == 256          # flux block, one GPU: 432 tall tiles, 2.92 waves
    c = lambda b, m, n, k, full=0, sms=148: lib.fo_gemm_dense_tile_cols(b, m, n, k, full, sms)
    assert c(2, 4608, 3072, 3072) == 256 and c(2, 4608, 6144, 3072) == 256   # ties go to the wider tile
    assert q(2, 4608, 1536, 3072) == 256 and c(2, 4608, 1536, 3072) == 192   # heads over two GPUs
    assert q(2, 4608, 768, 3072) == 256 and c(2, 4608, 768, 3072) == 192     # over four: 144 tiles, one round
    assert q(2, 4608, 384, 3072) == 128           # over eight: one round of 128-row tiles beats one of 256x192
    assert q(1, 77312, 5120, 5120) == 256         # video layer
    assert q(1, 9728, 5120, 5120) == 256          # its token shard on eight GPUs
    assert q(1, 128, 256, 64) == 128              # a single row block
    assert q(2, 4608, 3072, 3072, full=1) == 128  # a full-tensor init is the other kernel's
    assert q(0, 4608, 3072, 3072) == 0
