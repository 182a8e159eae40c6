"""GEMM-Q and GEMM-O (drop-in for flashomni/gemm.py:156-216).

Both ops build their work list from the packed mask on the GPU and then run one persistent tcgen05
GEMM over it. The only state kept between calls is a per-device workspace tensor (work list +
status word) that is re-used across calls on the same stream order.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import _native
from .utils import native_dtype

_workspaces = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """The work-list / status / tile-cursor words of a call: one tensor per (device, current stream), so that calls
    enqueued on different streams never share a cursor. Calls on one stream run in order and re-use it."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (device.type, index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 16), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _check_status(ws: torch.Tensor, what: str) -> None:
    words = ws[:32].view(torch.int32).cpu()
    if int(words[2]) != 0 or int(words[4]) != 0:
        raise RuntimeError(f"{what}: device status list={int(words[2])} kernel={int(words[4])}")


def _gemm_common(A: torch.Tensor, B: torch.Tensor, what: str):
    if A.dim() != 3 or B.dim() != 2:
        raise ValueError(f"{what}: expected A [batch, M, K] and B [N, K]")
    if A.shape[2] != B.shape[1]:
        raise ValueError(f"{what}: K mismatch between A {tuple(A.shape)} and B {tuple(B.shape)}")
    if A.dtype != B.dtype:
        raise ValueError(f"{what}: A and B must share a dtype")
    if not A.is_contiguous() or not B.is_contiguous():
        raise ValueError(f"{what}: A and B must be contiguous")
    # shape rule of the reference binding (csrc/gemm.cu:36): M % 128 == N % 128 == K % 32 == 0
    # (GEMM-O further needs head_dim % 64 == 0, which every head size the reference builds satisfies)
    if A.shape[1] % 128 != 0 or B.shape[0] % 128 != 0 or A.shape[2] % 32 != 0:
        raise ValueError(f"{what}: M and N must be multiples of 128 and K of 32")
    _native.require_cuda(A, B)


def flashomni_gemm(
    A: torch.Tensor,
    B: torch.Tensor,
    num_qo_heads: int,
    sparse_info: torch.Tensor = None,
    sparse_info_indptr: torch.Tensor = None,
    num_text_tokens: int = 512,
    bias: torch.Tensor = None,
    out: torch.Tensor = None,
    sparse_q_size: int = 128,
    is_full: bool = False,
    *,
    head_begin: int = 0,
    head_dim: Optional[int] = None,
    worklist: Optional["GemmWorklist"] = None,
) -> torch.Tensor:
    """GEMM-Q: out[b, rows, cols] = bias + A[b, rows, :] @ B[cols, :]^T for the 128x128 tiles whose
    (q-block, head) bit is set; other tiles of `out` keep their contents (reference:
    flashomni/gemm.py:156-186, kernel gemm.cuh:27-228). `head_begin` / `head_dim` (extensions, default =
    reference behaviour) let B hold the rows of a head window when heads are split over GPUs. `worklist`
    (extension): a list from `prepare_gemm_q_list` for the same mask and shape, built earlier (e.g. on a side
    stream); the mask arguments are then not read."""
    _gemm_common(A, B, "flashomni_gemm")
    batch, M, K = A.shape
    N = B.shape[0]
    if out is None:
        # the reference allocates with torch.empty (flashomni/gemm.py:168-173) and leaves the inactive tiles
        # uninitialised; zeros are one such value, and make its own script's comparison with the masked dense
        # result (benchmark/test_flashomni_gemm_q.py:78-89) well defined
        out = torch.zeros((batch, M, N), device=A.device, dtype=A.dtype)
    elif tuple(out.shape) != (batch, M, N) or out.dtype != A.dtype or not out.is_contiguous():
        raise ValueError("flashomni_gemm: out must be a contiguous [batch, M, N] tensor of A's dtype")
    if head_dim is None:
        head_dim = N // num_qo_heads
    lib = _native.load()
    if worklist is not None and not is_full:
        worklist.check("q", batch, M, N, head_dim, A.device)
        with torch.cuda.device(A.device):
            worklist.wait(A.device)
            rc = lib.fo_gemm_q_prepared(_native.ptr(A), _native.ptr(B), _native.ptr(out), _native.ptr(bias),
                                        native_dtype(A.dtype), batch, M, N, K, head_dim, _native.ptr(worklist.ws),
                                        worklist.ws.numel(), _native.current_stream(A.device))
        _native.check(rc, "flashomni_gemm")
        if _native.debug_checks():
            _check_status(worklist.ws, "flashomni_gemm")
        return out
    if not is_full and (sparse_info is None or sparse_info_indptr is None):
        raise ValueError("flashomni_gemm: sparse_info and sparse_info_indptr are required unless is_full=True")
    nbytes = lib.fo_gemm_workspace_bytes(batch, M, N, K, head_dim)
    ws = _workspace(A.device, nbytes)
    if sparse_info_indptr is not None and sparse_info_indptr.dtype != torch.int32:
        sparse_info_indptr = sparse_info_indptr.to(torch.int32)
    with torch.cuda.device(A.device):
        rc = lib.fo_gemm_q(_native.ptr(A), _native.ptr(B), _native.ptr(out), _native.ptr(bias),
                           native_dtype(A.dtype), batch, M, N, K, num_qo_heads, head_begin, head_dim,
                           sparse_q_size, num_text_tokens, 1 if is_full else 0, _native.ptr(sparse_info),
                           0 if sparse_info is None else sparse_info.numel(), _native.ptr(sparse_info_indptr),
                           _native.ptr(ws), ws.numel(), _native.current_stream(A.device))
    _native.check(rc, "flashomni_gemm")
    if _native.debug_checks():
        _check_status(ws, "flashomni_gemm")
    return out


def flashomni_gemm_reduction(
    A: torch.Tensor,
    B: torch.Tensor,
    num_qo_heads: int,
    sparse_info: torch.Tensor,
    sparse_info_indptr: torch.Tensor,
    num_text_tokens: int,
    bias: torch.Tensor = None,
    is_for_cache: bool = False,
    sparse_q_size: int = 128,
    *,
    head_begin: int = 0,
    head_dim: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
    worklist: Optional["GemmWorklist"] = None,
) -> torch.Tensor:
    """GEMM-O: out = init + sum over the selected heads of A[..., hD:(h+1)D] @ B[:, hD:(h+1)D]^T, selected =
    active heads (is_for_cache=False, init = the cached [batch, M, N] tensor passed as `bias`) or inactive
    heads (is_for_cache=True, init = 1-D bias) (reference: flashomni/gemm.py:188-216, kernel
    gemm_reduction.cuh:27-276). `head_begin` / `head_dim` / `out` are extensions with reference defaults."""
    _gemm_common(A, B, "flashomni_gemm_reduction")
    if worklist is None and (sparse_info is None or sparse_info_indptr is None):
        raise ValueError("flashomni_gemm_reduction: sparse_info and sparse_info_indptr are required")
    batch, M, K = A.shape
    N = B.shape[0]
    if head_dim is None:
        head_dim = N // num_qo_heads
    if out is None:
        out = torch.empty((batch, M, N), device=A.device, dtype=A.dtype)
    init_is_full = 0
    if bias is not None:
        if bias.dtype != A.dtype or not bias.is_contiguous():
            raise ValueError("flashomni_gemm_reduction: bias must be contiguous and share A's dtype")
        if is_for_cache:
            if bias.numel() != N:
                raise ValueError("flashomni_gemm_reduction: with is_for_cache=True bias must have N elements")
        else:
            if bias.numel() != batch * M * N:
                raise ValueError("flashomni_gemm_reduction: with is_for_cache=False bias must be the cached "
                                 "[batch, M, N] tensor")
            init_is_full = 1
    lib = _native.load()
    if worklist is not None:
        worklist.check("o", batch, M, K, head_dim, A.device, is_for_cache)
        with torch.cuda.device(A.device):
            worklist.wait(A.device)
            rc = lib.fo_gemm_o_prepared(_native.ptr(A), _native.ptr(B), _native.ptr(out), _native.ptr(bias), init_is_full,
                                        native_dtype(A.dtype), batch, M, N, K, head_dim, _native.ptr(worklist.ws),
                                        worklist.ws.numel(), _native.current_stream(A.device))
        _native.check(rc, "flashomni_gemm_reduction")
        if _native.debug_checks():
            _check_status(worklist.ws, "flashomni_gemm_reduction")
        return out
    nbytes = lib.fo_gemm_workspace_bytes(batch, M, N, K, head_dim)
    ws = _workspace(A.device, nbytes)
    if sparse_info_indptr.dtype != torch.int32:
        sparse_info_indptr = sparse_info_indptr.to(torch.int32)
    with torch.cuda.device(A.device):
        rc = lib.fo_gemm_o(_native.ptr(A), _native.ptr(B), _native.ptr(out), _native.ptr(bias), init_is_full,
                           native_dtype(A.dtype), batch, M, N, K, num_qo_heads, head_begin, head_dim,
                           sparse_q_size, num_text_tokens, 1 if is_for_cache else 0, _native.ptr(sparse_info),
                           sparse_info.numel(), _native.ptr(sparse_info_indptr), _native.ptr(ws), ws.numel(),
                           _native.current_stream(A.device))
    _native.check(rc, "flashomni_gemm_reduction")
    if _native.debug_checks():
        _check_status(ws, "flashomni_gemm_reduction")
    return out


class GemmWorklist:
    """A GEMM work list kept in its own workspace (extension): built from the mask by `prepare_gemm_q_list` /
    `prepare_gemm_o_list`, possibly on a side stream, and consumed by `flashomni_gemm(..., worklist=)` /
    `flashomni_gemm_reduction(..., worklist=)` on the caller's stream, which waits for the build first.
    The list depends on the mask and the shape only, not on the operands."""

    def __init__(self, kind: str, key: tuple, ws: torch.Tensor):
        self.kind, self.key, self.ws = kind, key, ws
        self.event: Optional[torch.cuda.Event] = None

    def check(self, kind: str, batch: int, M: int, n_or_k: int, head_dim: int, device, is_for_cache: bool = False):
        if (kind, (batch, M, n_or_k, head_dim, bool(is_for_cache)), device) != (self.kind, self.key, self.ws.device):
            raise ValueError("worklist was prepared for a different op, shape or device")

    def wait(self, device) -> None:
        if self.event is not None:
            torch.cuda.current_stream(device).wait_event(self.event)


def _prepare(kind: str, batch: int, M: int, N: int, K: int, num_qo_heads: int, head_dim: int, sparse_info, indptr,
             num_text_tokens: int, sparse_q_size: int, head_begin: int, is_for_cache: bool, into, stream):
    _native.require_cuda(sparse_info, indptr)
    dev = sparse_info.device
    lib = _native.load()
    # the consuming call checks the size for its full shape, which this list does not depend on (K for GEMM-Q,
    # N for GEMM-O): size for up to 256 heads / 16 384 output columns
    nbytes = lib.fo_gemm_workspace_bytes(batch, M, N if kind == "q" else 128 * 128, K if kind == "o" else 256 * head_dim,
                                         head_dim)
    key = (batch, M, N if kind == "q" else K, head_dim, bool(is_for_cache))
    if into is not None and into.kind == kind and into.key == key and into.ws.device == dev and into.ws.numel() >= nbytes:
        wl = into
    else:
        wl = GemmWorklist(kind, key, torch.zeros(max(nbytes, 256), dtype=torch.uint8, device=dev))
    if indptr.dtype != torch.int32:
        indptr = indptr.to(torch.int32)
    st = torch.cuda.current_stream(dev) if stream is None else stream
    with torch.cuda.device(dev):
        if kind == "q":
            rc = lib.fo_gemm_q_worklist(batch, M, N, num_qo_heads, head_begin, head_dim, sparse_q_size, num_text_tokens,
                                        0, _native.ptr(sparse_info), sparse_info.numel(), _native.ptr(indptr),
                                        _native.ptr(wl.ws), wl.ws.numel(), st.cuda_stream)
        else:
            rc = lib.fo_gemm_o_worklist(batch, M, K, num_qo_heads, head_begin, head_dim, sparse_q_size, num_text_tokens,
                                        1 if is_for_cache else 0, _native.ptr(sparse_info), sparse_info.numel(),
                                        _native.ptr(indptr), _native.ptr(wl.ws), wl.ws.numel(), st.cuda_stream)
        _native.check(rc, "prepare_gemm_list")
        if wl.event is None:
            wl.event = torch.cuda.Event()
        wl.event.record(st)
    return wl


def prepare_gemm_q_list(batch: int, M: int, N: int, num_qo_heads: int, sparse_info, sparse_info_indptr,
                        num_text_tokens: int = 512, sparse_q_size: int = 128, *, head_begin: int = 0,
                        head_dim: Optional[int] = None, into: Optional[GemmWorklist] = None,
                        stream: Optional[torch.cuda.Stream] = None) -> GemmWorklist:
    """Builds the GEMM-Q work list for a [batch, M, *] x [N, *] product from the mask, on `stream` (default: the
    current stream). `into` re-uses the workspace of an earlier list of the same shape."""
    hd = N // num_qo_heads if head_dim is None else head_dim
    return _prepare("q", batch, M, N, hd, num_qo_heads, hd, sparse_info, sparse_info_indptr, num_text_tokens,
                    sparse_q_size, head_begin, False, into, stream)


def prepare_gemm_o_list(batch: int, M: int, K: int, num_qo_heads: int, sparse_info, sparse_info_indptr,
                        num_text_tokens: int, is_for_cache: bool = False, sparse_q_size: int = 128, *,
                        head_begin: int = 0, head_dim: Optional[int] = None, into: Optional[GemmWorklist] = None,
                        stream: Optional[torch.cuda.Stream] = None) -> GemmWorklist:
    """Builds the GEMM-O row / head lists for a [batch, M, K] input from the mask (see prepare_gemm_q_list)."""
    hd = K // num_qo_heads if head_dim is None else head_dim
    return _prepare("o", batch, M, 128, K, num_qo_heads, hd, sparse_info, sparse_info_indptr, num_text_tokens,
                    sparse_q_size, head_begin, is_for_cache, into, stream)
