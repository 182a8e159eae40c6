"""GPU: this project's kernels against the golden outputs of the reference's own CUDA kernels, and --
when the reference harness library is present -- against those kernels run side by side."""

import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import cases  # noqa: E402
import flashomni_b200 as fo
from flashomni_b200 import workloads as wl
from oracle import ref_cuda
from helpers import assert_close_bf16, dev, masks_to_device

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_outputs.npz"))


def test_packbits_vs_reference_kernel_output(cuda_device):
    x, indptr = cases.packbits_case()
    for order in ("big", "little"):
        y, _ = fo.segment_packbits(dev(x, cuda_device), dev(indptr, cuda_device), bitorder=order)
        assert np.array_equal(y.cpu().numpy(), GOLD["packbits_" + order])


@pytest.mark.parametrize("name", cases.ATTENTION_CASES)
def test_attention_vs_reference_kernel_output(cuda_device, name):
    c = cases.attention_case(name)
    m = c["masks"]
    w = fo.BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1 << 20, dtype=torch.uint8, device=cuda_device))
    w.plan(dev(c["qo"], cuda_device), dev(c["kv"], cuda_device), c["H"], c["Hkv"], c["D"], q_data_type=torch.bfloat16,
           causal=c["causal"],
           custom_mask=None if c["custom_mask"] is None else cases.flat_custom_mask(c).to(cuda_device))
    si, skv, ip, kp = masks_to_device(m, cuda_device)
    o, lse = w.run(dev(c["q"], cuda_device), dev(c["k"], cuda_device), dev(c["v"], cuda_device), si, skv, ip, kp,
                   out=dev(c["prior"], cuda_device).clone(), return_lse=True)
    w.check_status()
    gold = cases.from_bits(GOLD[name + "_out"])
    # two bf16-rounded results of the same value may differ by one ulp
    assert_close_bf16(o, gold.float(), name, allow_ulp=1.0)
    # rows of switched-off q-blocks: bit-identical to what the reference left there (the prior); lse on the others
    g, qt = c["group"], c["q_block_tokens"]
    act = torch.zeros(o.shape[0], c["H"], dtype=torch.bool)
    for b in range(len(c["qo"]) - 1):
        for qb in range(m.q_active[b].shape[0]):
            r0 = int(c["qo"][b]) + qb * qt
            r1 = min(r0 + qt, int(c["qo"][b + 1]))
            for hk in range(c["Hkv"]):
                heads = slice(hk * g, (hk + 1) * g)
                if m.q_active[b][qb, hk]:
                    act[r0:r1, heads] = True
                else:
                    assert torch.equal(o[r0:r1, heads].cpu(), gold[r0:r1, heads])
    assert torch.allclose(lse.cpu()[act], torch.from_numpy(GOLD[name + "_lse"])[act], atol=2e-2, rtol=1e-4)


def test_gemms_vs_reference_kernel_output(cuda_device):
    c = cases.gemm_case("gemm_q")
    m = c["masks"]
    si, _, ip, _ = masks_to_device(m, cuda_device)
    y = fo.flashomni_gemm(dev(c["x"], cuda_device), dev(c["w"], cuda_device), c["H"], si, ip, 0, dev(c["bias"], cuda_device),
                          out=dev(c["prior"], cuda_device).clone())
    assert_close_bf16(y, cases.from_bits(GOLD["gemm_q_out"]).float(), "gemm_q", allow_ulp=1.0)
    c = cases.gemm_case("gemm_o")
    m = c["masks"]
    si, _, ip, _ = masks_to_device(m, cuda_device)
    cache = fo.flashomni_gemm_reduction(dev(c["x"], cuda_device), dev(c["w"], cuda_device), c["H"], si, ip, 0,
                                        dev(c["bias"], cuda_device), is_for_cache=True)
    g_cache = cases.from_bits(GOLD["gemm_o_cache"])
    assert_close_bf16(cache, g_cache.float(), "gemm_o cache", allow_ulp=1.0)
    y = fo.flashomni_gemm_reduction(dev(c["x"], cuda_device), dev(c["w"], cuda_device), c["H"], si, ip, 0,
                                    dev(g_cache, cuda_device), is_for_cache=False)
    assert_close_bf16(y, cases.from_bits(GOLD["gemm_o_out"]).float(), "gemm_o out", allow_ulp=1.0)


@pytest.mark.skipif(not ref_cuda.available(), reason="reference harness library not built")
def test_flux_layer_side_by_side_with_reference_kernels(cuda_device):
    """Config-1 size attention, GEMM-Q and GEMM-O: our kernels and the reference's, same inputs."""
    H, S = 24, 4608
    inp = wl.attention_inputs(1, H, S, 128, 0.5, seed=77)
    m = inp.masks
    si, skv, ip, kp = masks_to_device(m, cuda_device)
    q, k, v = (dev(t, cuda_device) for t in (inp.q, inp.k, inp.v))
    qo = dev(inp.qo_indptr, cuda_device)
    prior = dev(wl.randn_bf16(inp.q.shape, 78), cuda_device)
    w = fo.BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1 << 20, dtype=torch.uint8, device=cuda_device))
    w.plan(qo, qo, H, H, 128, q_data_type=torch.bfloat16)
    ours = w.run(q, k, v, si, skv, ip, kp, out=prior.clone())
    w.check_status()
    theirs = ref_cuda.sparse_attention(q, k, v, qo, qo, si, skv, ip, kp, prior.clone())
    torch.cuda.synchronize()
    assert_close_bf16(ours, theirs.float(), "attention vs reference kernel", allow_ulp=1.0)
    x = dev(wl.randn_bf16((1, S, 3072), 79), cuda_device)
    wt = dev(wl.randn_bf16((3072, 3072), 80, std=3072 ** -0.5), cuda_device)
    pr = dev(wl.randn_bf16((1, S, 3072), 81), cuda_device)
    a = fo.flashomni_gemm(x, wt, H, si, ip, 0, out=pr.clone())
    b = ref_cuda.gemm_q(x, wt, pr.clone(), H, si, ip, 0)
    torch.cuda.synchronize()
    assert_close_bf16(a, b.float(), "gemm_q vs reference kernel", allow_ulp=1.0)
    a = fo.flashomni_gemm_reduction(x, wt, H, si, ip, 0, pr, is_for_cache=False)
    b = ref_cuda.gemm_o(x, wt, torch.empty_like(pr), H, si, ip, 0, pr, False)
    torch.cuda.synchronize()
    assert_close_bf16(a, b.float(), "gemm_o vs reference kernel", allow_ulp=1.0)
