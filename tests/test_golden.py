"""CPU: the oracle against golden outputs of the REFERENCE's own CUDA kernels (tests/golden/
reference_outputs.npz, produced on a B200 by tests/golden/make_golden.py). This is what pins the
oracle: its statement of attention, GEMM-Q, GEMM-O and bit packing reproduces the reference's results."""

import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import cases  # noqa: E402
from oracle import attention as oa
from oracle import gemm as og
from oracle import masks as om
from helpers import assert_close_bf16

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_outputs.npz"))


def test_packbits_bit_exact_vs_reference_kernel():
    x, indptr = cases.packbits_case()
    for order in ("big", "little"):
        y, _ = om.segment_packbits(x, indptr, order)
        assert np.array_equal(y, GOLD["packbits_" + order])


def test_attention_oracle_vs_reference_kernel():
    for name in cases.ATTENTION_CASES:
        c = cases.attention_case(name)
        m = c["masks"]
        out, lse = oa.sparse_attention(c["q"], c["k"], c["v"], c["qo"], c["kv"], m.sparse_info, m.sparse_kv_info,
                                       m.info_indptr, m.kv_info_indptr, out_prior=c["prior"], return_lse=True,
                                       causal=c["causal"], custom_mask=c["custom_mask"])
        gold = cases.from_bits(GOLD[name + "_out"])
        # the reference output is itself bf16-rounded: same tolerance as for our kernels
        assert_close_bf16(gold, out, name)
        # rows of inactive q-blocks are untouched by the reference kernel: bit-identical to the prior. A mask q-block
        # is q_block_tokens tokens of the `group` q heads that share a kv head (128 packed rows).
        g, qt = c["group"], c["q_block_tokens"]
        act = torch.zeros(out.shape[0], c["H"], dtype=torch.bool)
        for b in range(len(c["qo"]) - 1):
            for qb in range(m.q_active[b].shape[0]):
                r0 = int(c["qo"][b]) + qb * qt
                r1 = min(r0 + qt, int(c["qo"][b + 1]))
                for hk in range(c["Hkv"]):
                    heads = slice(hk * g, (hk + 1) * g)
                    if m.q_active[b][qb, hk]:
                        act[r0:r1, heads] = True
                    else:
                        assert torch.equal(gold[r0:r1, heads], c["prior"][r0:r1, heads])
        g_lse = torch.from_numpy(GOLD[name + "_lse"])
        assert torch.allclose(g_lse[act], lse[act], atol=2e-2, rtol=1e-4)


def test_gemm_oracles_vs_reference_kernels():
    c = cases.gemm_case("gemm_q")
    m = c["masks"]
    y = og.gemm_q(c["x"], c["w"], c["H"], m.sparse_info, m.info_indptr, 0, c["bias"], c["prior"])
    assert_close_bf16(cases.from_bits(GOLD["gemm_q_out"]), y, "gemm_q", allow_ulp=1.0)
    c = cases.gemm_case("gemm_o")
    m = c["masks"]
    cache = og.gemm_o(c["x"], c["w"], c["H"], m.sparse_info, m.info_indptr, 0, c["bias"], True)
    g_cache = cases.from_bits(GOLD["gemm_o_cache"])
    assert_close_bf16(g_cache, cache, "gemm_o cache", allow_ulp=1.0)
    y = og.gemm_o(c["x"], c["w"], c["H"], m.sparse_info, m.info_indptr, 0, g_cache, False)
    assert_close_bf16(cases.from_bits(GOLD["gemm_o_out"]), y, "gemm_o out", allow_ulp=1.0)
