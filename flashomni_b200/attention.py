"""Block-sparse prefill attention wrapper (drop-in for flashomni/attention.py:194-869).

`plan()` does the host work once per shape (indptrs to the host, list capacities, workspace carving);
`run()` enqueues two steps on the current stream: the mask compaction (packed bits -> work lists) and
the tcgen05 attention kernel over those lists. Nothing in `run()` synchronises or allocates besides
`out` / `lse` when the caller does not pass them (as in the reference, attention.py:778-781).
"""

from __future__ import annotations

import functools
import logging
import math
from typing import Optional, Tuple, Union

import torch

from . import _native
from .utils import (MaskMode, PosEncodingMode, TensorLayout, _check_cached_qkv_data_type, _check_kv_layout,
                    _check_pos_encoding_mode, _check_shape_dtype_device, canonicalize_torch_dtype, native_dtype)


def _compute_sparse_info_indptr(qo_indptr: torch.Tensor, num_qo_heads, sparse_block_size_for_q: int,
                                device: torch.device = "cuda") -> torch.Tensor:
    """Unpacked (bit count) indptr of sparse_info (reference: flashomni/attention.py:165-176)."""
    out = torch.empty_like(qo_indptr, device=device)
    out[0] = 0
    out[1:] = torch.cumsum(
        torch.ceil((qo_indptr[1:] - qo_indptr[:-1]) / sparse_block_size_for_q) * num_qo_heads, 0)
    return out


def _compute_sparse_kv_info_indptr(qo_indptr: torch.Tensor, kv_indptr: torch.Tensor, num_qo_heads,
                                   sparse_block_size_for_q: int, sparse_block_size_for_kv: int,
                                   device: torch.device = "cuda") -> torch.Tensor:
    """Unpacked (bit count) indptr of sparse_kv_info (reference: flashomni/attention.py:178-191)."""
    out = torch.empty_like(qo_indptr, device=device)
    out[0] = 0
    out[1:] = torch.cumsum(
        torch.ceil((qo_indptr[1:] - qo_indptr[:-1]) / sparse_block_size_for_q)
        * torch.ceil((kv_indptr[1:] - kv_indptr[:-1]) / sparse_block_size_for_kv) * num_qo_heads, 0)
    return out


_FP8_KINDS = {torch.float8_e4m3fn: 0, torch.float8_e5m2: 1}


def _cast_fp8(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """An 8-bit float tensor as a new contiguous tensor of `dtype` (f16 / bf16), values unchanged."""
    if not t.is_contiguous():
        t = t.contiguous()
    out = torch.empty(t.shape, dtype=dtype, device=t.device)
    lib = _native.load()
    with torch.cuda.device(t.device):
        _native.check(lib.fo_cast_fp8(_native.ptr(t), t.numel(), _FP8_KINDS[t.dtype], native_dtype(dtype),
                                      _native.ptr(out), _native.current_stream(t.device)), "fo_cast_fp8")
    return out


class BatchFlashOmniFAWithRaggedKVWrapper:
    r"""Prefill attention over ragged q/k/v with two bit-packed block masks: `sparse_info` selects the
    (q-block, head) pairs that are computed at all, `sparse_kv_info` the kv-blocks each of them attends
    to. Same constructor / plan / run surface as the reference class (flashomni/attention.py:194-869).

    Extensions (keyword-only in `plan`, default = reference behaviour): `mask_num_heads` and
    `mask_head_begin` describe a head window when the tensors hold only heads
    [mask_head_begin, mask_head_begin + num_kv_heads) of a mask laid out for `mask_num_heads` heads
    (used when heads are partitioned over GPUs). With `num_qo_heads > num_kv_heads` the masks have one bit per
    (128 packed rows, kv head) as in the reference's kernel: a q-block is 128 / group tokens of all the q heads
    that share a kv head.
    """

    def __init__(
        self,
        float_workspace_buffer: torch.Tensor,
        kv_layout: str = "NHD",
        use_cuda_graph: bool = False,
        qo_indptr_buf: Optional[torch.Tensor] = None,
        kv_indptr_buf: Optional[torch.Tensor] = None,
        custom_mask_buf: Optional[torch.Tensor] = None,
        mask_indptr_buf: Optional[torch.Tensor] = None,
        backend: str = "auto",
    ) -> None:
        _check_kv_layout(kv_layout)
        if not float_workspace_buffer.is_cuda:
            raise RuntimeError("flashomni_b200: the workspace must live on a CUDA device (no CPU path exists)")
        self._kv_layout = kv_layout
        self._float_workspace_buffer = float_workspace_buffer
        self.device = float_workspace_buffer.device
        self._int_workspace_buffer = None  # carved in plan(); sized from the planned shapes
        self._use_cuda_graph = use_cuda_graph
        if use_cuda_graph:
            if not torch.is_tensor(qo_indptr_buf):
                raise ValueError("qo_indptr_buf should be a torch.Tensor in cuda graph mode")
            if not torch.is_tensor(kv_indptr_buf):
                raise ValueError("kv_indptr_buf should be a torch.Tensor in cuda graph mode")
            self._fixed_batch_size = len(qo_indptr_buf) - 1
            if len(kv_indptr_buf) != self._fixed_batch_size + 1:
                raise ValueError(
                    "The length of kv_indptr_buf ({}) should be the same as qo_indptr_buf ({}).".format(
                        len(kv_indptr_buf), self._fixed_batch_size))
        self._qo_indptr_buf = qo_indptr_buf
        self._kv_indptr_buf = kv_indptr_buf
        self._custom_mask_buf = custom_mask_buf
        self._mask_indptr_buf = mask_indptr_buf
        self._max_total_num_rows = None
        self._backend = backend
        self._planned = False
        self._side_stream = None
        self._prepared_event = None
        self._prepared_key = None

    @property
    def is_cuda_graph_enabled(self) -> bool:
        return self._use_cuda_graph

    def reset_workspace_buffer(self, float_workspace_buffer: torch.Tensor, int_workspace_buffer) -> None:
        """Reference: flashomni/attention.py:384-406. The int workspace, if given and large enough, is
        used for the work lists at the next plan()."""
        self._float_workspace_buffer = float_workspace_buffer
        self._int_workspace_buffer = int_workspace_buffer
        self._planned = False

    # ------------------------------------------------------------------------------------------ plan
    def plan(
        self,
        qo_indptr: torch.Tensor,
        kv_indptr: torch.Tensor,
        num_qo_heads: int,
        num_kv_heads: int,
        head_dim_qk: int,
        sparse_block_size_for_q: int = 128,
        sparse_block_size_for_kv: int = 128,
        head_dim_vo: Optional[int] = None,
        custom_mask: Optional[torch.Tensor] = None,
        packed_custom_mask: Optional[torch.Tensor] = None,
        causal: bool = False,
        pos_encoding_mode: str = "NONE",
        use_fp16_qk_reduction: bool = False,
        logits_soft_cap: Optional[float] = None,
        sm_scale: Optional[float] = None,
        rope_scale: Optional[float] = None,
        rope_theta: Optional[float] = None,
        q_data_type: Union[str, torch.dtype] = "float16",
        kv_data_type: Optional[Union[str, torch.dtype]] = None,
        *,
        mask_num_heads: Optional[int] = None,
        mask_head_begin: int = 0,
    ) -> None:
        """Reference: flashomni/attention.py:408-642. Host-only; must not be captured in a CUDA graph."""
        q_data_type = canonicalize_torch_dtype(q_data_type)
        if kv_data_type is None:
            kv_data_type = q_data_type
        kv_data_type = canonicalize_torch_dtype(kv_data_type)
        if head_dim_vo is None:
            head_dim_vo = head_dim_qk
        if logits_soft_cap is None:
            logits_soft_cap = 0.0
        _check_pos_encoding_mode(pos_encoding_mode)

        batch_size = len(qo_indptr) - 1
        if len(kv_indptr) != batch_size + 1:
            raise ValueError("The kv_indptr length should be equal to mask_indptr length.")
        # Features of the FlashInfer lineage that the DiT path never enables (the reference's AOT build
        # only instantiates mask_mode 0, setup.py:38; pos-enc and fp16-qk-reduction are forced off,
        # csrc/batch_sparseFA_config.inc:42-43):
        if PosEncodingMode[pos_encoding_mode] != PosEncodingMode.NONE:
            raise NotImplementedError("flashomni_b200: in-kernel positional encoding is not implemented")
        if logits_soft_cap < 0:
            raise ValueError("logits_soft_cap must be >= 0 (0 disables it)")
        # 8-bit float K / V: the reference casts the fragments to the type of Q before the MMA, without scales
        # (include/flashomni/attention/prefill.cuh:602-612); here run() casts the two tensors once (fo_cast_fp8)
        if q_data_type != kv_data_type and kv_data_type not in _FP8_KINDS:
            raise NotImplementedError("flashomni_b200: kv must have the dtype of q, float8_e4m3fn or float8_e5m2")
        if kv_data_type in _FP8_KINDS:   # the reference warns in the same words where it casts (attention.py:787-794)
            logging.warning("flashomni_b200: the attention kernel takes 16-bit inputs; float8 k / v are cast to the dtype "
                            "of q before every run, which costs one more pass over them")
        native_dtype(q_data_type)
        if num_kv_heads <= 0 or num_qo_heads % num_kv_heads != 0:
            raise ValueError("num_qo_heads must be a multiple of num_kv_heads")
        group = num_qo_heads // num_kv_heads
        if group not in (1, 2, 4, 8, 16):
            raise NotImplementedError("flashomni_b200: num_qo_heads / num_kv_heads must be 1, 2, 4, 8 or 16")
        if head_dim_qk != head_dim_vo or head_dim_qk not in (64, 128, 256):
            raise NotImplementedError("flashomni_b200: head_dim 64, 128 and 256 are implemented (qk and vo equal)")
        if sparse_block_size_for_q != 128 or sparse_block_size_for_kv != 128:
            raise NotImplementedError("flashomni_b200: only 128-row sparse blocks are implemented")

        qo_indptr_host = qo_indptr.to("cpu")
        kv_indptr_host = kv_indptr.to("cpu")
        total_num_rows = int(qo_indptr_host[-1])

        if self.is_cuda_graph_enabled:
            if self._max_total_num_rows is None:
                self._max_total_num_rows = total_num_rows
            elif total_num_rows > self._max_total_num_rows:
                raise ValueError(
                    "The total number of rows in qo_indptr {} in cuda graph mode cannot "
                    "exceed the number of rows set during initialization {}.".format(
                        total_num_rows, self._max_total_num_rows))
            if batch_size != self._fixed_batch_size:
                raise ValueError(
                    "The batch size should be fixed in cudagraph mode, the runtime batch size {} "
                    " mismatches the batch size set during initialization {}.".format(
                        batch_size, self._fixed_batch_size))
            self._qo_indptr_buf.copy_(qo_indptr)
            self._kv_indptr_buf.copy_(kv_indptr)
        else:
            self._qo_indptr_buf = qo_indptr.to(self.device, dtype=torch.int32)
            self._kv_indptr_buf = kv_indptr.to(self.device, dtype=torch.int32)

        self._cached_q_data_type = q_data_type
        self._cached_kv_data_type = kv_data_type

        # With grouped heads the masks are indexed as the reference's kernel indexes them
        # (include/flashomni/attention/prefill.cuh:1283-1291): one bit per (block of 128 packed rows, kv head), a
        # packed row being a (token, q head of the group) pair in token-major order, i.e. a q-block covers
        # 128 / group tokens for all the q heads of one kv head. group = 1 is the plain (128 tokens, head) layout.
        mask_heads_here = num_kv_heads
        if mask_num_heads is None:
            mask_num_heads = mask_heads_here
        if mask_head_begin < 0 or mask_head_begin + mask_heads_here > mask_num_heads:
            raise ValueError("mask head window out of range")

        ql = (qo_indptr_host[1:] - qo_indptr_host[:-1]).to(torch.int64)
        kl = (kv_indptr_host[1:] - kv_indptr_host[:-1]).to(torch.int64)
        if bool((ql < 0).any()) or bool((kl < 0).any()):
            raise ValueError("indptr arrays must be non-decreasing")
        self._q_block_tokens = sparse_block_size_for_q // group
        nq = (ql + self._q_block_tokens - 1) // self._q_block_tokens
        nkv = (kl + sparse_block_size_for_kv - 1) // sparse_block_size_for_kv
        self._n_cand = int((nq * mask_heads_here).sum())
        self._max_nkv = int(nkv.max()) if batch_size > 0 else 0
        self._max_kept = int((nq * nkv * mask_heads_here).sum())
        self._batch_size = batch_size
        self._num_qo_heads = num_qo_heads
        self._num_kv_heads = num_kv_heads
        self._head_dim = head_dim_qk
        self._mask_num_heads = mask_num_heads
        self._mask_head_begin = mask_head_begin
        self._total_q = total_num_rows
        self._total_kv = int(kv_indptr_host[-1])
        self._causal = causal
        # Custom mask (reference: flashomni/attention.py:524-533): per request a [q_len, kv_len] matrix of flags,
        # flattened and concatenated; packed here with segment_packbits exactly as the reference packs it (every
        # request's matrix starts at a byte boundary). A packed mask that the caller brings must be packed that way.
        self._packed_custom_mask = None
        self._mask_indptr = None
        if custom_mask is not None or packed_custom_mask is not None:
            elems = ql * kl
            if packed_custom_mask is None:
                from .quantization import segment_packbits
                flat = custom_mask.contiguous().view(-1).to(self.device)
                if flat.numel() != int(elems.sum()):
                    raise ValueError("custom_mask must hold sum(q_len * kv_len) flags")
                elem_indptr = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(elems, 0)]).to(
                    self.device, dtype=torch.int32)
                packed, byte_indptr = segment_packbits(flat, elem_indptr, bitorder="little")
            else:
                nbytes = (elems + 7) // 8
                byte_indptr = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(nbytes, 0)])
                packed = packed_custom_mask.to(self.device, dtype=torch.uint8).contiguous()
                if packed.numel() < int(byte_indptr[-1]):
                    raise ValueError("packed_custom_mask is shorter than sum(ceil(q_len * kv_len / 8)) bytes")
            self._packed_custom_mask = packed
            self._mask_indptr = byte_indptr.to(self.device, dtype=torch.int32)
        self._carve_workspace()

        self._sparse_block_size_for_q = sparse_block_size_for_q
        self._sparse_block_size_for_kv = sparse_block_size_for_kv
        self._causal = causal
        self._pos_encoding_mode = pos_encoding_mode
        self._use_fp16_qk_reduction = use_fp16_qk_reduction
        self._logits_soft_cap = logits_soft_cap
        self._sm_scale = sm_scale
        self._rope_scale = rope_scale
        self._rope_theta = rope_theta
        # the element indptrs of the unpacked masks (what callers feed to segment_packbits) are derived on first use:
        # a dozen small torch kernels that plan() itself does not need
        self._indptr_bases = None
        self._planned = True

    begin_forward = plan

    def _bases(self):
        if self._indptr_bases is None:
            self._indptr_bases = (
                _compute_sparse_info_indptr(self._qo_indptr_buf, self._num_qo_heads, self._sparse_block_size_for_q,
                                            device=self.device),
                _compute_sparse_kv_info_indptr(self._qo_indptr_buf, self._kv_indptr_buf, self._num_qo_heads,
                                               self._sparse_block_size_for_q, self._sparse_block_size_for_kv,
                                               device=self.device))
        return self._indptr_bases

    @property
    def _sparse_info_indptr_base(self) -> torch.Tensor:
        return self._bases()[0]

    @property
    def _sparse_kv_info_indptr_base(self) -> torch.Tensor:
        return self._bases()[1]

    # Cutting kv lists into parts (split-KV with a merge of partial results) is built and tested but OFF by default:
    # on a B200 it measured slower at every shape tried (a GPU's share of 3, 6 or 12 heads of the 4608-token layer:
    # 35 -> 43, 70 -> 79 and 113 -> 138 microseconds). The part is power-capped: SMs that end early leave their share
    # of the budget to the SMs with long lists, so an even spread of the blocks gains little, and every part pays
    # an epilogue (fp32 partial result, a CTA-wide hand-over, the merge).
    UNITS_PER_SM = 0      # > 0: kv lists are cut when the launch has more than one and at most this many items per SM
    MIN_CHUNK = 16        # shortest part (kv blocks) a kv list is cut into
    FORCE_SPLIT = False   # cut every list into parts of two blocks (tests: every case then runs the merge path)

    def _carve_workspace(self) -> None:
        """Lays the work lists out in one int32 buffer: counters[4] | status[4] | unit_counters[4] | items | kv_ptr |
        order | arrive | units | kv_idx | scratch, and sets the partial-result scratch of split items aside (in the
        caller's float workspace when that is large enough, as the reference's planner does with its own partial
        outputs, flashomni/attention.py:344-352,608-623)."""
        lib = _native.load()
        n, kept = max(self._n_cand, 1), max(self._max_kept, 1)
        scratch_bytes = lib.fo_mask_compact_scratch_bytes(n, self._max_nkv)
        # One persistent CTA per SM draws units, longest first. With UNITS_PER_SM > 0 and between one and that many
        # candidate items per SM the lists are cut into parts of about total / (UNITS_PER_SM * SMs) blocks (at least
        # MIN_CHUNK) whose partial results (fp32 O, row maxima and sums) go to scratch and are merged by the part
        # that delivers last.
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self._num_streams = max(self.UNITS_PER_SM * sms, 1)
        self._min_chunk = self.MIN_CHUNK
        self._min_items = sms
        may_split = self.UNITS_PER_SM > 0 and sms < self._n_cand <= self._num_streams
        extra_units = self._num_streams
        slots = extra_units + extra_units // 2
        if self.FORCE_SPLIT and self._max_kept <= 4096:
            may_split, self._min_chunk, self._min_items = True, 2, 0
            self._num_streams = max(self._num_streams, self._n_cand, self._max_kept)
            extra_units = slots = self._max_kept // 2 + n + 1      # parts of at least two blocks
        # those instantiations handle whole items only
        if self._causal or self._packed_custom_mask is not None or self._head_dim == 256:
            may_split = False
        self._max_units = n + (extra_units if may_split else 0)
        self._partial_slots = slots if may_split else 0

        def al(words):  # 16-byte aligned word counts
            return (words + 3) // 4 * 4

        offs, cur = {}, 0
        for name, words in (("counters", 4), ("status", 4), ("unit_counters", 4), ("items", 4 * n), ("kv_ptr", n + 1),
                            ("order", n), ("arrive", max(self._partial_slots, 1)), ("units", 8 * self._max_units), ("kv_idx", kept),
                            ("scratch", (scratch_bytes + 3) // 4)):
            offs[name] = cur
            cur += al(words)
        need = cur * 4
        buf = self._int_workspace_buffer
        if buf is None or buf.numel() * buf.element_size() < need or buf.device != self.device:
            buf = torch.zeros(need, dtype=torch.uint8, device=self.device)
            self._int_workspace_buffer = buf
        words = buf.view(torch.uint8)[: need].view(torch.int32)
        words[offs["counters"]: offs["counters"] + 12].zero_()  # counters, status / cursor words start from zero
        words[offs["arrive"]: offs["arrive"] + max(self._partial_slots, 1)].zero_()
        self._ws = {k: words[v:] for k, v in offs.items()}
        self._ws_words = words
        self._ws_offs = offs
        self._scratch_bytes = scratch_bytes
        pbytes = lib.fo_attn_partial_bytes(self._partial_slots)
        fw = self._float_workspace_buffer
        self._partials = None
        if pbytes > 0:
            if fw.device == self.device and fw.numel() * fw.element_size() >= pbytes + 16 and fw.is_contiguous():
                raw = fw.view(torch.uint8).view(-1)
                shift = (-raw.data_ptr()) % 16
                self._partials = raw[shift: shift + pbytes]
            else:
                self._partials = torch.empty(pbytes, dtype=torch.uint8, device=self.device)

    # ------------------------------------------------------------------------------------------ run
    def run(
        self,
        q: torch.Tensor,
        k: torch.Tensor,
        v: torch.Tensor,
        sparse_info: torch.Tensor = None,
        sparse_kv_info: torch.Tensor = None,
        sparse_info_indptr: torch.Tensor = None,
        sparse_kv_info_indptr: torch.Tensor = None,
        is_full: bool = False,
        *args,
        out: Optional[torch.Tensor] = None,
        lse: Optional[torch.Tensor] = None,
        return_lse: bool = False,
    ) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
        """q [qo_indptr[-1], H, D]; k, v [kv_indptr[-1], H, D] (NHD) or [H, kv_indptr[-1], D] (HND).
        `sparse_info` / `sparse_kv_info` are the packed uint8 masks and their *byte* indptrs as returned
        by `segment_packbits(..., bitorder="little")`. q-blocks whose bit is 0 keep the contents of `out`
        (zeros when `out` is allocated here). Reference: flashomni/attention.py:709-835."""
        if not self._planned:
            raise RuntimeError("plan() must be called before run()")
        _native.require_cuda(q, k, v)
        _check_cached_qkv_data_type(q, k, self._cached_q_data_type, self._cached_kv_data_type)
        if v.dtype != k.dtype:
            raise ValueError(f"v has dtype {v.dtype}, k has {k.dtype}")
        if k.dtype in _FP8_KINDS:
            k, v = _cast_fp8(k, q.dtype), _cast_fp8(v, q.dtype)
        sm_scale = self._sm_scale
        if sm_scale is None:
            sm_scale = 1.0 / math.sqrt(q.size(-1))
        if q.dim() != 3 or q.size(0) != self._total_q or q.size(1) != self._num_qo_heads or q.size(2) != self._head_dim:
            raise ValueError(f"q has shape {tuple(q.shape)}, planned [{self._total_q}, {self._num_qo_heads}, {self._head_dim}]")
        if return_lse:
            if lse is None:
                lse = torch.empty((q.size(0), q.size(1)), dtype=torch.float32, device=q.device)
            else:
                _check_shape_dtype_device(lse, (q.size(0), q.size(1)), torch.float32, q.device, "lse")
        if out is None:
            out = torch.zeros(q.shape[:-1] + v.shape[-1:], dtype=q.dtype, device=q.device)
        else:
            _check_shape_dtype_device(out, q.shape[:-1] + v.shape[-1:], q.dtype, q.device, "out")
        if not is_full:
            # the reference dereferences null masks here (csrc/batch_sparseFA.cu:123-131); raise instead
            if sparse_info is None or sparse_kv_info is None or sparse_info_indptr is None \
                    or sparse_kv_info_indptr is None:
                raise ValueError("sparse_info, sparse_kv_info and their indptrs are required unless is_full=True")
            for name, t in (("sparse_info", sparse_info), ("sparse_kv_info", sparse_kv_info)):
                if t.dtype != torch.uint8 or not t.is_cuda or not t.is_contiguous():
                    raise ValueError(f"{name} must be a contiguous uint8 CUDA tensor")
            if len(sparse_info_indptr) != self._batch_size + 1 or len(sparse_kv_info_indptr) != self._batch_size + 1:
                raise ValueError("mask indptr length must be batch_size + 1")
            if sparse_info_indptr.dtype != torch.int32:
                sparse_info_indptr = sparse_info_indptr.to(torch.int32)
            if sparse_kv_info_indptr.dtype != torch.int32:
                sparse_kv_info_indptr = sparse_kv_info_indptr.to(torch.int32)
        if self._kv_layout == "NHD":
            kn, kh, vn, vh = k.stride(0), k.stride(1), v.stride(0), v.stride(1)
            total_kv, hkv = k.size(0), k.size(1)
        else:
            kh, kn, vh, vn = k.stride(0), k.stride(1), v.stride(0), v.stride(1)
            total_kv, hkv = k.size(1), k.size(0)
        if total_kv != self._total_kv or hkv != self._num_kv_heads:
            raise ValueError("k/v shape does not match the plan")
        if q.stride(2) != 1 or k.stride(2) != 1 or v.stride(2) != 1 or out.stride(2) != 1:
            raise ValueError("the head dimension of q/k/v/out must be contiguous")
        if out.stride(1) % 8 != 0 or out.stride(0) % 8 != 0:
            raise ValueError("out strides must be multiples of 8 elements")

        lib = _native.load()
        ws = self._ws
        stream = _native.current_stream(self.device)
        with torch.cuda.device(self.device):
            key = self._mask_key(sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr, is_full)
            if self._prepared_key is not None and self._prepared_key == key:
                # the lists were built by prepare_masks() on the side stream: just order after it
                torch.cuda.current_stream(self.device).wait_event(self._prepared_event)
            else:
                self._compact(sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr, is_full, stream)
            self._prepared_key = None
            head = (_native.ptr(q), _native.ptr(k), _native.ptr(v), _native.ptr(out), _native.ptr(lse),
                    native_dtype(q.dtype), self._total_q, self._total_kv, self._num_qo_heads, self._num_kv_heads,
                    self._head_dim, q.stride(0), q.stride(1), kn, kh, vn, vh, out.stride(0), out.stride(1),
                    self._sparse_block_size_for_q, self._sparse_block_size_for_kv, _native.ptr(ws["kv_idx"]),
                    _native.ptr(ws["units"]), _native.ptr(ws["unit_counters"]), self._max_units,
                    _native.ptr(ws["arrive"]), _native.ptr(self._partials), self._partial_slots,
                    self._mask_head_begin, float(sm_scale))
            cap = float(self._logits_soft_cap or 0.0)
            if self._packed_custom_mask is not None:  # the custom mask takes precedence over `causal`, as in the reference
                rc = lib.fo_sparse_attn_fwd_custom_mask(
                    *head[:25], self._mask_head_begin, float(sm_scale), cap, _native.ptr(self._packed_custom_mask),
                    self._packed_custom_mask.numel(), _native.ptr(self._mask_indptr), _native.ptr(self._qo_indptr_buf),
                    _native.ptr(self._kv_indptr_buf), _native.ptr(ws["status"]), stream)
            elif self._causal:  # whole items only: no partial-result scratch on this path
                rc = lib.fo_sparse_attn_fwd_causal(*head[:25], self._mask_head_begin, float(sm_scale), cap,
                                                   _native.ptr(ws["status"]), stream)
            elif cap > 0:  # logits = cap * tanh(q.k * sm_scale / cap), as the reference's variant does
                rc = lib.fo_sparse_attn_fwd_softcap(*head, cap, _native.ptr(ws["status"]), stream)
            else:
                rc = lib.fo_sparse_attn_fwd(*head, _native.ptr(ws["status"]), stream)
            _native.check(rc, "BatchFlashOmniFAWithRaggedKVWrapper.run")
        if _native.debug_checks():
            self.check_status()
        return (out, lse) if return_lse else out

    run_return_lse = functools.partialmethod(run, return_lse=True)

    # ------------------------------------------------------------------------------------------ mask step
    @staticmethod
    def _mask_key(sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr, is_full):
        if is_full:
            return ("full",)
        return tuple((t.data_ptr(), t._version) for t in (sparse_info, sparse_kv_info, sparse_info_indptr,
                                                          sparse_kv_info_indptr))

    def _compact(self, sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr, is_full, stream):
        ws = self._ws
        rc = _native.load().fo_mask_compact(
            _native.ptr(sparse_info), 0 if sparse_info is None else sparse_info.numel(),
            _native.ptr(sparse_kv_info), 0 if sparse_kv_info is None else sparse_kv_info.numel(),
            _native.ptr(sparse_info_indptr), _native.ptr(sparse_kv_info_indptr),
            _native.ptr(self._qo_indptr_buf), _native.ptr(self._kv_indptr_buf),
            self._batch_size, self._mask_num_heads, self._mask_head_begin, self._num_kv_heads,
            self._q_block_tokens, self._sparse_block_size_for_kv, 1 if is_full else 0,
            self._n_cand, self._max_nkv, max(self._n_cand, 1), max(self._max_kept, 1),
            _native.ptr(ws["items"]), _native.ptr(ws["kv_ptr"]), _native.ptr(ws["kv_idx"]),
            _native.ptr(ws["order"]), _native.ptr(ws["counters"]), _native.ptr(ws["scratch"]),
            self._scratch_bytes, stream)
        _native.check(rc, "BatchFlashOmniFAWithRaggedKVWrapper (mask compaction)")
        rc = _native.load().fo_attn_units(
            _native.ptr(ws["items"]), _native.ptr(ws["kv_ptr"]), _native.ptr(ws["kv_idx"]), _native.ptr(ws["order"]),
            _native.ptr(ws["counters"]), _native.ptr(self._qo_indptr_buf), _native.ptr(self._kv_indptr_buf),
            max(self._n_cand, 1), self._max_nkv, self._q_block_tokens, self._sparse_block_size_for_kv,
            self._min_items, self._num_streams, self._min_chunk, self._max_units, self._partial_slots,
            _native.ptr(ws["units"]),
            _native.ptr(ws["unit_counters"]), _native.ptr(ws["arrive"]), stream)
        _native.check(rc, "BatchFlashOmniFAWithRaggedKVWrapper (work units)")

    def build_work_lists(self, sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr,
                         is_full: bool = False) -> None:
        """Extension: the mask compaction alone, on the current stream (what `run()` does first when the lists
        were not prepared). For callers that time or inspect the step; see `work_lists()`."""
        if not self._planned:
            raise RuntimeError("plan() must be called before build_work_lists()")
        with torch.cuda.device(self.device):
            self._compact(sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr, is_full,
                          _native.current_stream(self.device))
        self._prepared_key = None

    def prepare_masks(self, sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr,
                      is_full: bool = False, *, stream: Optional[torch.cuda.Stream] = None,
                      after: Optional[torch.cuda.Event] = None) -> None:
        """Optional (extension): builds the work lists for these mask tensors now, on a side stream that is
        ordered after the current stream, so that the step overlaps whatever the caller enqueues next (the
        Q/K/V projections). The following `run()` with the same, unmodified mask tensors re-uses the lists;
        any other `run()` compacts as usual. Masks only depend on the block selection, not on q/k/v.
        `stream` replaces the wrapper's own side stream; with `after` the side stream is ordered after that
        event instead of after everything enqueued on the current stream so far (the caller guarantees that
        the previous `run()` of this wrapper precedes the event)."""
        if not self._planned:
            raise RuntimeError("plan() must be called before prepare_masks()")
        if not is_full:
            if sparse_info_indptr.dtype != torch.int32 or sparse_kv_info_indptr.dtype != torch.int32:
                return  # run() will convert and compact itself
        with torch.cuda.device(self.device):
            if self._prepared_event is None:
                self._prepared_event = torch.cuda.Event()
            side = stream
            if side is None:
                if self._side_stream is None:
                    self._side_stream = torch.cuda.Stream(self.device)
                side = self._side_stream
            if after is not None:
                side.wait_event(after)
            else:
                side.wait_stream(torch.cuda.current_stream(self.device))
            self._compact(sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr, is_full,
                          side.cuda_stream)
            self._prepared_event.record(side)
        self._prepared_key = self._mask_key(sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr,
                                            is_full)

    # ------------------------------------------------------------------------------------------ extras
    def check_status(self) -> None:
        """Synchronises and raises if the last run() recorded a device-side problem."""
        w = self._ws_words[:12].cpu()
        if int(w[2]) != 0 or int(w[4]) != 0 or int(w[11]) != 0:
            raise RuntimeError(f"flashomni_b200 attention: device status compaction={int(w[2])} units={int(w[11])} "
                               f"kernel={int(w[4])}")

    def work_lists(self) -> dict:
        """Host copies of the lists of the last run() (synchronises; for tests and FLOP accounting)."""
        w = self._ws
        c = w["counters"][:4].cpu()
        n, kept = int(c[0]), int(c[1])
        uc = w["unit_counters"][:4].cpu()
        nu = int(uc[0])
        return {
            "n_units": nu, "partial_slots_used": int(uc[1]), "chunk_max": int(uc[2]), "unit_status": int(uc[3]),
            "units": w["units"][: 8 * nu].cpu().view(-1, 8).numpy(),
            "n_items": n, "total_kept": kept, "status": int(c[2]),
            "items": w["items"][: 4 * n].cpu().view(-1, 4).numpy(),
            "kv_indptr": w["kv_ptr"][: n + 1].cpu().numpy(),
            "kv_idx": w["kv_idx"][: kept].cpu().numpy(),
            "order": w["order"][: n].cpu().numpy(),
        }

    def forward(self, q, k, v, sparse_info=None, sparse_kv_info=None, sparse_info_indptr=None,
                sparse_kv_info_indptr=None, is_full: bool = False, causal: bool = False,
                pos_encoding_mode: str = "NONE", use_fp16_qk_reduction: bool = False,
                logits_soft_cap: Optional[float] = None, sm_scale: Optional[float] = None,
                rope_scale: Optional[float] = None, rope_theta: Optional[float] = None) -> torch.Tensor:
        """Deprecated alias kept for source compatibility (reference: flashomni/attention.py:647-673)."""
        if causal or pos_encoding_mode != "NONE":
            raise NotImplementedError("flashomni_b200: causal / pos-encoding are not implemented")
        self._sm_scale = sm_scale
        self._logits_soft_cap = logits_soft_cap or 0.0
        return self.run(q, k, v, sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr, is_full)

    def forward_return_lse(self, q, k, v, sparse_info=None, sparse_kv_info=None, sparse_info_indptr=None,
                           sparse_kv_info_indptr=None, is_full: bool = False, causal: bool = False,
                           pos_encoding_mode: str = "NONE", use_fp16_qk_reduction: bool = False,
                           logits_soft_cap: Optional[float] = None, sm_scale: Optional[float] = None,
                           rope_scale: Optional[float] = None, rope_theta: Optional[float] = None):
        """Deprecated alias (reference: flashomni/attention.py:839-865)."""
        if causal or pos_encoding_mode != "NONE":
            raise NotImplementedError("flashomni_b200: causal / pos-encoding are not implemented")
        self._sm_scale = sm_scale
        self._logits_soft_cap = logits_soft_cap or 0.0
        return self.run_return_lse(q, k, v, sparse_info, sparse_kv_info, sparse_info_indptr,
                                   sparse_kv_info_indptr, is_full)

    def end_forward(self) -> None:
        """Deprecated, no effect (reference: flashomni/attention.py:867-869)."""
        pass
