"""Generates tests/golden/reference_outputs.npz by running the REFERENCE's own CUDA kernels
(oracle/_ref/libflashomni_ref.so, built by oracle/build_ref.py from the reference headers) on the
seeded inputs of cases.py. Needs a GPU:

    python tests/golden/make_golden.py [output.npz]

The outputs are stored as raw bf16 bit patterns. They pin the CPU oracle (tests/test_golden.py) and the
CUDA kernels of this project (tests/test_gpu_golden.py) to what the reference itself computes."""

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import cases  # noqa: E402
from oracle import ref_cuda  # noqa: E402


def main(out_path):
    dev = torch.device("cuda:0")
    res = {}
    d = lambda a, dt=None: (torch.from_numpy(a) if isinstance(a, np.ndarray) else a).to(dev)
    for name in cases.ATTENTION_CASES:
        c = cases.attention_case(name)
        m = c["masks"]
        out = d(c["prior"]).clone()
        lse = torch.zeros(out.shape[0], c["H"], dtype=torch.float32, device=dev)
        extra = {}
        if c["custom_mask"] is not None:   # packed as the reference's plan() packs it (its segment_packbits kernel)
            elems = np.asarray([cm.size for cm in c["custom_mask"]], dtype=np.int64)
            ind = np.concatenate([[0], np.cumsum(elems)]).astype(np.int32)
            new_ind = np.concatenate([[0], np.cumsum((elems + 7) // 8)]).astype(np.int32)
            packed = ref_cuda.segment_packbits(d(cases.flat_custom_mask(c).to(torch.uint8)), d(ind), d(new_ind), True)
            extra = {"packed_custom_mask": packed, "mask_indptr": d(new_ind)}
        ref_cuda.sparse_attention(d(c["q"]), d(c["k"]), d(c["v"]), d(c["qo"]), d(c["kv"]), d(m.sparse_info),
                                  d(m.sparse_kv_info), d(m.info_indptr), d(m.kv_info_indptr), out, lse=lse, causal=c["causal"],
                                  **extra)
        torch.cuda.synchronize()
        res[name + "_out"] = cases.bf16_bits(out)
        res[name + "_lse"] = lse.cpu().numpy()
    c = cases.gemm_case("gemm_q")
    m = c["masks"]
    out = d(c["prior"]).clone()
    ref_cuda.gemm_q(d(c["x"]), d(c["w"]), out, c["H"], d(m.sparse_info), d(m.info_indptr), 0, d(c["bias"]))
    torch.cuda.synchronize()
    res["gemm_q_out"] = cases.bf16_bits(out)
    c = cases.gemm_case("gemm_o")
    m = c["masks"]
    cache = torch.empty_like(d(c["prior"]))
    ref_cuda.gemm_o(d(c["x"]), d(c["w"]), cache, c["H"], d(m.sparse_info), d(m.info_indptr), 0, d(c["bias"]), True)
    y = torch.empty_like(cache)
    ref_cuda.gemm_o(d(c["x"]), d(c["w"]), y, c["H"], d(m.sparse_info), d(m.info_indptr), 0, cache, False)
    torch.cuda.synchronize()
    res["gemm_o_cache"] = cases.bf16_bits(cache)
    res["gemm_o_out"] = cases.bf16_bits(y)
    x, indptr = cases.packbits_case()
    seglen = indptr[1:] - indptr[:-1]
    new_indptr = np.concatenate([[0], np.cumsum((seglen + 7) // 8)]).astype(np.int32)
    for little in (0, 1):
        y = ref_cuda.segment_packbits(d(x), d(indptr), d(new_indptr), bool(little))
        torch.cuda.synchronize()
        res["packbits_" + ("little" if little else "big")] = y.cpu().numpy()
    np.savez_compressed(out_path, **res)
    print("wrote", out_path, {k: v.shape for k, v in res.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_outputs.npz"))
