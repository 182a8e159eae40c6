"""GPU: the allocation-free GEMM-Q entry point (fo_gemm_q_static) against fo_gemm_q.

fo_gemm_q_static exists for hosts that cannot allocate device memory when the op runs (their own
arena owns the device, or an allocation's implicit synchronisation is not acceptable): its scratch is a
fixed array inside the library instead of a caller workspace. The test drives both entry points through
the C ABI on the same inputs, twice in a row on the shared array with a different mask the second time
(so stale list contents from the first call would show), and expects the same output within the
suite's bf16 tolerance, also against the CPU oracle; around the second call (the first one may load the
library's device image) it reads the device's free memory and the torch allocator's counters to see that
the call took no device memory from either. This file sorts last on purpose, so a run that stops at the
first failure has already run everything else.
"""

import pytest
import torch

from flashomni_b200 import _native, workloads as wl
from oracle import gemm as og
from helpers import assert_close_bf16, dev, masks_to_device

pytestmark = pytest.mark.gpu


def _call(lib, static, x, w, y, bias, B, M, N, K, H, si, ip, ws, stream):
    common = (_native.ptr(x), _native.ptr(w), _native.ptr(y), _native.ptr(bias), _native.FO_DTYPE_BF16, B, M, N, K, H, 0,
              N // H, 128, 0, 0, _native.ptr(si), si.numel(), _native.ptr(ip))
    if static:
        rc = lib.fo_gemm_q_static(*common, stream)
        assert rc == _native.FO_OK, lib.fo_gemm_q_static_last_error()
    else:
        rc = lib.fo_gemm_q(*common, _native.ptr(ws), ws.numel(), stream)
        _native.check(rc, "fo_gemm_q")


def test_static_scratch_entry_matches_workspace_entry(cuda_device):
    lib = _native.load()
    B, H, nq, K = 2, 4, 6, 512
    M, N = nq * 128, H * 128
    x_h, w_h = wl.randn_bf16((B, M, K), 1), wl.randn_bf16((N, K), 2, std=K ** -0.5)
    bias_h, prior_h = wl.randn_bf16((N,), 3), wl.randn_bf16((B, M, N), 4)
    x, w, bias, prior = (dev(t, cuda_device) for t in (x_h, w_h, bias_h, prior_h))
    ws = torch.zeros(lib.fo_gemm_workspace_bytes(B, M, N, K, N // H), dtype=torch.uint8, device=cuda_device)
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    with torch.cuda.device(cuda_device):
        for call_no, (seed, density) in enumerate(((51, 0.75), (52, 0.25))):   # two calls in a row; the second list is shorter
            m = wl.flux_masks(B, H, nq, nq, density, seed=seed, text_blocks=1)
            si, _, ip, _ = masks_to_device(m, cuda_device)
            y_ref, y_static = prior.clone(), prior.clone()
            _call(lib, False, x, w, y_ref, bias, B, M, N, K, H, si, ip, ws, stream)
            torch.cuda.synchronize()
            free0 = torch.cuda.mem_get_info(cuda_device)[0]
            stats0 = torch.cuda.memory_stats(cuda_device)
            _call(lib, True, x, w, y_static, bias, B, M, N, K, H, si, ip, None, stream)
            torch.cuda.synchronize()
            if call_no == 1:   # no device memory was taken, from the driver or from torch's allocator
                assert torch.cuda.mem_get_info(cuda_device)[0] == free0
                stats1 = torch.cuda.memory_stats(cuda_device)
                for key in ("allocation.all.allocated", "segment.all.allocated", "allocated_bytes.all.current"):
                    assert stats1[key] == stats0[key], key
            assert_close_bf16(y_static, y_ref.float(), f"fo_gemm_q_static vs fo_gemm_q (density {density})")
            ref = og.gemm_q(x_h, w_h, H, m.sparse_info, m.info_indptr, 0, bias_h, prior_h)
            assert_close_bf16(y_static, ref, f"fo_gemm_q_static vs the oracle (density {density})", allow_ulp=1.0)
            assert not torch.equal(y_static, prior)


def test_static_scratch_entry_rejects_oversized_problems(cuda_device):
    lib = _native.load()
    cap = lib.fo_gemm_q_static_max_bytes()
    B, M, N, K = 64, 128 * 64, 128 * 64, 64     # 131072 list records of 16 bytes, above the 1 MiB array
    assert lib.fo_gemm_workspace_bytes(B, M, N, K, 128) > cap
    t = torch.zeros(16, dtype=torch.bfloat16, device=cuda_device)   # never dereferenced: the size check comes first
    rc = lib.fo_gemm_q_static(_native.ptr(t), _native.ptr(t), _native.ptr(t), None, _native.FO_DTYPE_BF16, B, M, N, K, 64, 0,
                              128, 128, 0, 1, None, 0, None, torch.cuda.current_stream(cuda_device).cuda_stream)
    assert rc == _native.FO_ERR_WORKSPACE
    msg = lib.fo_gemm_q_static_last_error().decode()
    assert "built-in array holds" in msg and str(cap) in msg
