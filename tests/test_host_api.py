"""CPU: host-side behaviour of the Python surface (no device work)."""

import inspect

import pytest
import torch

import flashomni_b200 as fo


def test_public_names_match_reference_package():
    for name in ("BatchFlashOmniFAWithRaggedKVWrapper", "flashomni_gemm", "flashomni_gemm_reduction", "packbits",
                 "segment_packbits", "__version__"):
        assert hasattr(fo, name)
    w = fo.BatchFlashOmniFAWithRaggedKVWrapper
    for m in ("plan", "run", "run_return_lse", "begin_forward", "forward", "forward_return_lse", "end_forward",
              "reset_workspace_buffer", "is_cuda_graph_enabled"):
        assert hasattr(w, m)


def test_signatures_keep_reference_parameter_order():
    p = list(inspect.signature(fo.BatchFlashOmniFAWithRaggedKVWrapper.run).parameters)
    assert p[:9] == ["self", "q", "k", "v", "sparse_info", "sparse_kv_info", "sparse_info_indptr",
                     "sparse_kv_info_indptr", "is_full"]
    p = list(inspect.signature(fo.BatchFlashOmniFAWithRaggedKVWrapper.plan).parameters)
    assert p[:8] == ["self", "qo_indptr", "kv_indptr", "num_qo_heads", "num_kv_heads", "head_dim_qk",
                     "sparse_block_size_for_q", "sparse_block_size_for_kv"]
    p = list(inspect.signature(fo.flashomni_gemm).parameters)
    assert p[:10] == ["A", "B", "num_qo_heads", "sparse_info", "sparse_info_indptr", "num_text_tokens", "bias",
                      "out", "sparse_q_size", "is_full"]
    assert inspect.signature(fo.flashomni_gemm).parameters["num_text_tokens"].default == 512
    p = list(inspect.signature(fo.flashomni_gemm_reduction).parameters)
    assert p[:9] == ["A", "B", "num_qo_heads", "sparse_info", "sparse_info_indptr", "num_text_tokens", "bias",
                     "is_for_cache", "sparse_q_size"]


def test_signatures_match_the_reference_source_parameter_by_parameter():
    """Names, order and defaults of every positional parameter of the reference's public entry points (read from
    its source by tests/golden/make_reference_signatures.py); this package only adds optional keyword-only extensions."""
    import json
    import os
    with open(os.path.join(os.path.dirname(__file__), "golden", "reference_signatures.json")) as f:
        ref = json.load(f)
    assert len(ref) == 11
    for name, desc in ref.items():
        obj = fo
        for part in name.split("."):
            obj = getattr(obj, part)
        ours = [p for p in inspect.signature(obj).parameters.values() if p.kind == p.POSITIONAL_OR_KEYWORD]
        assert [p.name for p in ours] == [n for n, _ in desc["positional"]], name
        for p, (_, default) in zip(ours, desc["positional"]):
            if default is None:
                assert p.default is inspect.Parameter.empty, (name, p.name)
            else:
                assert repr(p.default) == default.replace('"', "'"), (name, p.name)
        kw = {p.name: p for p in inspect.signature(obj).parameters.values() if p.kind == p.KEYWORD_ONLY}
        for n, default in desc["keyword_only"]:   # e.g. run(..., *args, out=None, lse=None, return_lse=False)
            assert n in kw and repr(kw[n].default) == default.replace('"', "'"), (name, n)
        assert all(p.default is not inspect.Parameter.empty for p in kw.values()), name   # extensions are optional


def test_cpu_tensors_are_rejected_not_silently_computed():
    x = torch.zeros(16, dtype=torch.bool)
    with pytest.raises(RuntimeError, match="CUDA"):
        fo.packbits(x)
    with pytest.raises(RuntimeError, match="CUDA"):
        fo.flashomni_gemm(torch.zeros(1, 128, 64, dtype=torch.bfloat16), torch.zeros(128, 64, dtype=torch.bfloat16), 1,
                          is_full=True)
    with pytest.raises(RuntimeError, match="CUDA"):
        fo.BatchFlashOmniFAWithRaggedKVWrapper(torch.zeros(16, dtype=torch.uint8))


def test_bitorder_and_shape_validation():
    with pytest.raises(ValueError):
        fo.packbits(torch.zeros(8, dtype=torch.bool), bitorder="middle")
    with pytest.raises(ValueError):
        fo.flashomni_gemm(torch.zeros(1, 100, 64, dtype=torch.bfloat16), torch.zeros(128, 64, dtype=torch.bfloat16), 1,
                          is_full=True)


def test_indptr_helpers_match_oracle():
    from oracle import masks as om
    qo = torch.tensor([0, 300, 429], dtype=torch.int32)
    kv = torch.tensor([0, 256, 1256], dtype=torch.int32)
    a = fo.attention._compute_sparse_info_indptr(qo, 3, 128, device="cpu")
    b = fo.attention._compute_sparse_kv_info_indptr(qo, kv, 3, 128, 128, device="cpu")
    assert a.tolist() == om.sparse_info_indptr(qo.numpy(), 3, 128).tolist()
    assert b.tolist() == om.sparse_kv_info_indptr(qo.numpy(), kv.numpy(), 3, 128, 128).tolist()
