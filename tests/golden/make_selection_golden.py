"""Golden masks of the block-selection step, produced by the reference's own code on a GPU.

The reference selects blocks in `benchmark/test_attn_score.py:93-133`: torch ops (sum, softmax, ascending sort,
cumsum, searchsorted(right=True)) followed by its Triton fill kernels `fill_sparse_info_triton` (`:63-69`) and
`fill_sparse_kv_info_triton` (`:83-89`). This script imports that module from a checkout of the reference
(`FLASHOMNI_REFERENCE_DIR`, the directory that holds `benchmark/`), repeats the torch calls of its `__main__`
section in the same order on CUDA tensors, calls the two fill kernels, and writes

    tests/golden/reference_selection.npz

with, per case, the scores, the thresholds, the unpacked masks `sparse_info [B, H, n]` and
`sparse_kv_info [B, H, n, n]` as the reference lays them out, and per selected row the distance of the nearest
cumulative mass from the threshold (`*_margin`): the tests exempt rows whose margin is within float rounding,
where the summation order of another implementation may move one block across the threshold.
It also times the reference's selection path at the two benchmark mask sizes (CUDA events, after warm-up) and
stores the microseconds under `timing_us`.

Needs a CUDA GPU and triton; run from the repository root:

    FLASHOMNI_REFERENCE_DIR=<checkout> python tests/golden/make_selection_golden.py
"""

from __future__ import annotations

import importlib.util
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name, seed, B, H, n, text blocks, q thresholds [B], kv thresholds [H], score scale
CASES = [
    ("tiny", 0, 1, 2, 5, 2, [0.2], [0.2, 0.2], 1.0),
    ("small", 1, 2, 3, 24, 2, [0.2, 0.35], [0.1, 0.3, 0.5], 2.0),
    ("one_text", 2, 2, 4, 17, 1, [0.5, 0.05], [0.0, 0.25, 0.6, 0.9], 3.0),
    ("flux_like", 3, 1, 24, 36, 4, [0.3], list(np.linspace(0.05, 0.6, 24).round(3)), 2.0),
    ("flat", 4, 1, 3, 16, 2, [0.4], [0.4, 0.4, 0.4], 0.05),
]
TIMED = [("flux", 1, 24, 36, 4), ("video", 1, 40, 604, 4)]


def load_reference_module():
    root = os.environ.get("FLASHOMNI_REFERENCE_DIR")
    if not root:
        sys.exit("set FLASHOMNI_REFERENCE_DIR to a checkout of the reference")
    path = os.path.join(root, "benchmark", "test_attn_score.py")
    spec = importlib.util.spec_from_file_location("reference_attn_score", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def scores(seed, B, H, n, scale):
    return (np.random.default_rng(seed).standard_normal((B, H, n, n)) * scale).astype(np.float32)


def reference_selection(ref, pooled_score, t2t, q_thr, kv_thr):
    """The torch calls of the reference's `__main__` (`test_attn_score.py:97-133`) with per-request and per-head
    thresholds, then its fill kernels. Returns the masks and the intermediate cdfs / counts."""
    B, H, n, _ = pooled_score.shape
    dev = pooled_score.device
    t2i = pooled_score[:, :, :t2t, t2t:].contiguous()
    t2i = torch.sum(t2i, dim=[1, 2]).softmax(-1)
    sparse_info = torch.ones((B, H, n), dtype=torch.uint8, device=dev)
    sorted_score = torch.sort(t2i, dim=-1, descending=False)
    cdf = torch.cumsum(sorted_score.values, dim=-1)
    thr = torch.as_tensor(q_thr, dtype=torch.float32, device=dev).view(B, 1).contiguous()
    num_q = torch.searchsorted(cdf, thr, right=True).squeeze(-1)
    # One call of the fill kernel per request: the kernel steps through `sorted_indices` with a row stride of n
    # (`test_attn_score.py:57`) while the tensor has n - T2T columns, so in a batched call request b would read
    # b * T2T entries too far (past the end for the last request). With one request per call the offset is 0 and
    # the kernel does what the script's own B = 1 example does.
    parts = [ref.fill_sparse_info_triton(sparse_info[b:b + 1], num_q[b:b + 1], sorted_score.indices[b:b + 1], T2T=t2t)
             for b in range(B)]
    sparse_info = torch.cat(parts, dim=0)

    img = pooled_score[:, :, t2t:, :].contiguous().softmax(-1)
    sparse_kv_info = torch.ones((B, H, n, n), dtype=torch.uint8, device=dev)
    sorted_kv = torch.sort(img, dim=-1, descending=False)
    cdf_kv = torch.cumsum(sorted_kv.values, dim=-1)
    kthr = torch.as_tensor(kv_thr, dtype=torch.float32, device=dev).view(1, H, 1, 1).expand(B, -1, n - t2t, 1).contiguous()
    num_kv = torch.searchsorted(cdf_kv, kthr, right=True).squeeze(-1)
    sparse_kv_info = ref.fill_sparse_kv_info_triton(sparse_kv_info, num_kv, sorted_kv.indices, T2T=t2t)
    return sparse_info, sparse_kv_info, cdf, thr, num_q, cdf_kv, kthr, num_kv


def margin(cdf, thr):
    """Per row: the smallest |cdf_k - threshold| (fp64 of the fp32 values)."""
    return (cdf.double() - thr.double()).abs().amin(dim=-1).cpu().numpy()


def main():
    if not torch.cuda.is_available():
        sys.exit("needs a CUDA GPU")
    ref = load_reference_module()
    dev = torch.device("cuda", 0)
    out = {}
    for name, seed, B, H, n, t2t, qthr, kthr, scale in CASES:
        s = scores(seed, B, H, n, scale)
        si, skv, cdf, thr, num_q, cdf_kv, kthr_t, num_kv = reference_selection(ref, torch.from_numpy(s).to(dev), t2t, qthr, kthr)
        torch.cuda.synchronize()
        out[f"{name}.score"] = s
        out[f"{name}.meta"] = np.asarray([seed, B, H, n, t2t], dtype=np.int64)
        out[f"{name}.q_threshold"] = np.asarray(qthr, dtype=np.float32)
        out[f"{name}.kv_threshold"] = np.asarray(kthr, dtype=np.float32)
        out[f"{name}.sparse_info"] = si.cpu().numpy()
        out[f"{name}.sparse_kv_info"] = skv.cpu().numpy()
        out[f"{name}.q_margin"] = margin(cdf, thr)                      # [B]
        out[f"{name}.kv_margin"] = margin(cdf_kv, kthr_t)               # [B, H, n - t2t]
        out[f"{name}.num_q"] = num_q.cpu().numpy().astype(np.int64)
        out[f"{name}.num_kv"] = num_kv.cpu().numpy().astype(np.int64)
        print(name, "q off", int(num_q.sum()), "kv off", int(num_kv.sum()), "min margins",
              float(out[f"{name}.q_margin"].min()), float(out[f"{name}.kv_margin"].min()))
    timing = {}
    for name, B, H, n, t2t in TIMED:
        s = torch.from_numpy(scores(9, B, H, n, 2.0)).to(dev)
        qthr, kthr = [0.3] * B, [0.3] * H
        for _ in range(3):
            reference_selection(ref, s, t2t, qthr, kthr)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record()
        for _ in range(reps):
            reference_selection(ref, s, t2t, qthr, kthr)
        e1.record()
        torch.cuda.synchronize()
        timing[name] = {"B": B, "H": H, "n": n, "text_blocks": t2t, "us": e0.elapsed_time(e1) * 1e3 / reps}
        print("reference selection", name, timing[name])
    out["timing_us"] = np.frombuffer(json.dumps(timing).encode(), dtype=np.uint8)
    out["names"] = np.frombuffer(json.dumps([c[0] for c in CASES]).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "reference_selection.npz"), **out)
    dst = os.environ.get("FLASHOMNI_GOLDEN_COPY")
    if dst:   # a second copy for a run whose working tree does not come back
        np.savez_compressed(dst, **out)
    print("wrote", os.path.join(HERE, "reference_selection.npz"))


if __name__ == "__main__":
    main()
