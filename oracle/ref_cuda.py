"""Test infrastructure: Python access to the reference's own CUDA kernels through
oracle/_ref/libflashomni_ref.so (built by oracle/build_ref.py). Used to compare this project's kernels
with the reference's on a GPU, to generate golden vectors, and to time the reference kernels beside
ours. The functions mirror the semantics of the reference ops they call:
torch.ops.flashomni_kernels.{batch_sparseFA_with_ragged_kv_run, flashomni_gemm, flashomni_gemm_reduction,
segment_packbits} (csrc/flashomni_ops.cu:20-51)."""

from __future__ import annotations

import ctypes
import math
import os

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libflashomni_ref.so")
_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(LIB_PATH)
        for n in ("ref_sparse_attn", "ref_sparse_attn_hd64", "ref_sparse_attn_hd256", "ref_sparse_attn_causal", "ref_sparse_attn_custom", "ref_gemm_q", "ref_gemm_o", "ref_segment_packbits"):
            getattr(_lib, n).restype = ctypes.c_int
    return _lib


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def plan_unsplit(qo_indptr, kv_indptr, device, group=1, cta_tile_q=128):
    """Work arrays of the reference planner for the un-split case (scheduler.cuh:67-168 with
    kv_chunk_size >= every kv length): one entry per (request, q tile of `cta_tile_q` packed rows),
    a request having qo_len * group packed rows (scheduler.cuh:82)."""
    qo = np.asarray(qo_indptr, dtype=np.int64)
    kv = np.asarray(kv_indptr, dtype=np.int64)
    req, tile = [], []
    for b in range(len(qo) - 1):
        for t in range(int(-(-((qo[b + 1] - qo[b]) * group) // cta_tile_q))):
            req.append(b)
            tile.append(t)
    mk = lambda a: torch.tensor(a, dtype=torch.int32, device=device)
    chunk = int(max(1, (kv[1:] - kv[:-1]).max()))
    return {"request": mk(req), "qo_tile": mk(tile), "kv_tile": mk([0] * len(req)), "o_indptr": mk(qo.tolist()),
            "chunk": mk([chunk]), "n": len(req)}


def sparse_attention(q, k, v, qo_indptr, kv_indptr, sparse_info, sparse_kv_info, info_indptr, kv_info_indptr,
                     out, is_full=False, sm_scale=None, lse=None, plan=None, causal=False, packed_custom_mask=None,
                     mask_indptr=None):
    """q [Tq, H, D], k/v [Tkv, Hkv, D] (NHD, D = 64, 128 or 256), `out` is written in place (only active q-blocks)."""
    dev = q.device
    if plan is None:
        plan = plan_unsplit(qo_indptr.cpu().numpy(), kv_indptr.cpu().numpy(), dev, q.shape[1] // k.shape[1],
                            cta_tile_q=64 if q.shape[-1] == 256 else 128)   # the harness runs head dimension 256 with 64-row tiles
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    u = ctypes.c_uint32
    if q.shape[-1] not in (64, 128, 256):
        raise ValueError("the harness instantiates the reference kernel for head dimensions 64, 128 and 256")
    if causal and q.shape[-1] != 128:
        raise ValueError("the harness instantiates the causal mask mode for head dimension 128 only")
    fn = load().ref_sparse_attn_causal if causal else {128: load().ref_sparse_attn, 64: load().ref_sparse_attn_hd64,
                                                       256: load().ref_sparse_attn_hd256}[q.shape[-1]]
    lead = ()
    if packed_custom_mask is not None:   # byte indptr of the per-request matrices, as segment_packbits returns it
        if q.shape[-1] != 128:
            raise ValueError("the harness instantiates the custom mask mode for head dimension 128 only")
        fn = load().ref_sparse_attn_custom
        lead = (_p(packed_custom_mask), _p(mask_indptr))
    rc = fn(
        *lead, _p(q), _p(k), _p(v), _p(out), _p(lse), _p(sparse_info), _p(sparse_kv_info), _p(info_indptr), _p(kv_info_indptr),
        _p(qo_indptr), _p(kv_indptr), _p(plan["request"]), _p(plan["qo_tile"]), _p(plan["kv_tile"]), _p(plan["o_indptr"]),
        _p(plan["chunk"]), u(plan["n"]), u(q.shape[1]), u(k.shape[1]), u(q.stride(0)), u(q.stride(1)), u(k.stride(0)),
        u(k.stride(1)), u(v.stride(0)), u(v.stride(1)), ctypes.c_float(sm_scale), ctypes.c_int(1 if is_full else 0),
        u(q.shape[0]), ctypes.c_int(1 if q.dtype == torch.bfloat16 else 0), _stream(dev))
    if rc != 0:
        raise RuntimeError(f"reference attention kernel failed: cudaError {rc}")
    return out


def gemm_q(x, w, out, num_heads, sparse_info, info_indptr, num_text_tokens=0, bias=None, sparse_q_size=128,
           is_full=False):
    B, M, K = x.shape
    N = w.shape[0]
    u = ctypes.c_uint32
    rc = load().ref_gemm_q(_p(x), _p(w), _p(out), _p(bias), u(B), u(M), u(N), u(K), u(sparse_q_size), u(num_heads),
                           u(N // num_heads), _p(sparse_info), _p(info_indptr), u(num_text_tokens),
                           ctypes.c_int(1 if is_full else 0), ctypes.c_int(1 if x.dtype == torch.bfloat16 else 0),
                           _stream(x.device))
    if rc != 0:
        raise RuntimeError(f"reference GEMM-Q kernel failed: cudaError {rc}")
    return out


def gemm_o(x, w, out, num_heads, sparse_info, info_indptr, num_text_tokens=0, bias=None, is_for_cache=False,
           sparse_q_size=128):
    B, M, K = x.shape
    N = w.shape[0]
    u = ctypes.c_uint32
    rc = load().ref_gemm_o(_p(x), _p(w), _p(out), _p(bias), u(B), u(M), u(N), u(K), u(sparse_q_size), u(num_heads),
                           u(N // num_heads), _p(sparse_info), _p(info_indptr), u(num_text_tokens),
                           ctypes.c_int(1 if is_for_cache else 0), ctypes.c_int(1 if x.dtype == torch.bfloat16 else 0),
                           _stream(x.device))
    if rc != 0:
        raise RuntimeError(f"reference GEMM-O kernel failed: cudaError {rc}")
    return out


def segment_packbits(x, indptr, new_indptr, little=True):
    y = torch.zeros(int(new_indptr[-1].item()), dtype=torch.uint8, device=x.device)
    rc = load().ref_segment_packbits(_p(x), _p(indptr), _p(new_indptr), ctypes.c_uint32(len(indptr) - 1),
                                     ctypes.c_int(1 if little else 0), _p(y), _stream(x.device))
    if rc != 0:
        raise RuntimeError(f"reference segment_packbits failed: cudaError {rc}")
    return y
