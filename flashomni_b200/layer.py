"""A sparse DiT attention block assembled from the public ops, the way a FlashOmni user wires them:
GEMM-Q (sparse) + GEMM-K/V (dense) -> block-sparse attention -> GEMM-O (active heads + cached rest).

Heads can be partitioned over ranks: a rank that owns heads [head_begin, head_begin + head_count) holds
the matching rows of W_q/W_k/W_v and the matching K-slice of W_o, reads the full hidden state and the
full masks, and produces a partial output [B, S, hidden] (its heads' contribution plus its share of the
cache). Nothing inside the block crosses GPUs; the sum of the partials is left to the caller.
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Optional

import torch

from .attention import BatchFlashOmniFAWithRaggedKVWrapper
from .gemm import flashomni_gemm, flashomni_gemm_reduction, prepare_gemm_o_list, prepare_gemm_q_list


@dataclass
class BlockWeights:
    wq: torch.Tensor   # [head_count*D, hidden]
    wk: torch.Tensor
    wv: torch.Tensor
    wo: torch.Tensor   # [hidden, head_count*D]


class SparseDiTAttentionBlock:
    def __init__(self, weights: BlockWeights, num_heads: int, head_dim: int, batch: int, seq: int,
                 head_begin: int = 0, head_count: Optional[int] = None, device=None, dtype=torch.bfloat16,
                 schedule: str = "kv_first", add_cache: bool = True, fuse_kv: bool = True):
        """`add_cache=False`: GEMM-O adds nothing to the active heads' sum (a rank of a head partition whose
        partial is summed with the others' later; only one rank, or the sum itself, adds the cache).
        `fuse_kv`: the dense K and V projections run as one GEMM over the stacked weights [W_k; W_v], writing
        one [B, S, 2 * local heads * D] buffer that the attention reads through strided views."""
        if schedule not in ("q_first", "kv_first"):
            raise ValueError("schedule must be 'q_first' or 'kv_first'")
        self.schedule = schedule
        self.add_cache = add_cache
        self.fuse_kv = fuse_kv
        self._side = None
        self._q_list = self._o_list = None
        self.w = weights
        self.H, self.D, self.B, self.S = num_heads, head_dim, batch, seq
        self.hb = head_begin
        self.hc = num_heads - head_begin if head_count is None else head_count
        self.device = device if device is not None else weights.wq.device
        self.dtype = dtype
        n_local = self.hc * head_dim
        hidden = weights.wq.shape[1]
        self.hidden = hidden
        mk = lambda *s: torch.zeros(*s, dtype=dtype, device=self.device)
        self.q = mk(batch, seq, n_local)      # doubles as the cached Q of earlier steps for inactive tiles
        if self.fuse_kv:
            self.wkv = torch.cat([weights.wk, weights.wv], dim=0).contiguous()
            self.kv = mk(batch, seq, 2 * n_local)
            self.k, self.v = self.kv[..., :n_local], self.kv[..., n_local:]
        else:
            self.k = mk(batch, seq, n_local)
            self.v = mk(batch, seq, n_local)
        self.attn = mk(batch, seq, n_local)   # skipped q-blocks keep their previous contents
        self.y = mk(batch, seq, weights.wo.shape[0])
        self.cache = mk(batch, seq, weights.wo.shape[0])
        self.wrapper = BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1 << 20, dtype=torch.uint8, device=self.device))
        indptr = torch.arange(batch + 1, dtype=torch.int32, device=self.device) * seq
        t0 = time.perf_counter()
        self.wrapper.plan(indptr, indptr, self.hc, self.hc, head_dim, q_data_type=dtype,
                          mask_num_heads=num_heads, mask_head_begin=head_begin)
        self.plan_host_ms = (time.perf_counter() - t0) * 1e3   # host time of plan(): once per shape, not per step

    def refresh_cache(self, x, sparse_info, sparse_info_indptr):
        """The full step of the two-call protocol: cache = contribution of the heads that the sparse steps
        will skip (computed from a dense attention output held in self.attn)."""
        flashomni_gemm_reduction(self.attn, self.w.wo, self.H, sparse_info, sparse_info_indptr, 0, None,
                                 is_for_cache=True, head_begin=self.hb, head_dim=self.D, out=self.cache)
        return self.cache

    def forward(self, x, sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr, out=None):
        """One sparse step. x [B, S, hidden]. Returns this rank's (partial) output [B, S, hidden] (written
        into `out` when given, else into the block's own buffer)."""
        y = self.y if out is None else out
        H, D, hb = self.H, self.D, self.hb
        # The attention work lists only depend on the masks: they are built on a side stream beside the
        # projections. The projection kernels fill every SM (shared memory), so that work runs in their tails;
        # GEMM-Q goes first because its tiles are handed out dynamically and tolerate an SM that starts late.
        # (Building the GEMM lists on a side stream as well -- prepare_gemm_q_list / prepare_gemm_o_list --
        # measured no gain here for the same reason.)
        T = self.B * self.S
        if self.schedule == "kv_first":
            return self._forward_kv_first(x, sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr, y)
        self.wrapper.prepare_masks(sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr)
        flashomni_gemm(x, self.w.wq, H, sparse_info, sparse_info_indptr, 0, None, out=self.q,
                       head_begin=hb, head_dim=D)
        if self.fuse_kv:
            flashomni_gemm(x, self.wkv, H, is_full=True, out=self.kv, head_dim=D)
            kv = self.kv.view(T, 2 * self.hc, D)
            k, v = kv[:, :self.hc], kv[:, self.hc:]
        else:
            flashomni_gemm(x, self.w.wk, H, is_full=True, out=self.k, head_dim=D)
            flashomni_gemm(x, self.w.wv, H, is_full=True, out=self.v, head_dim=D)
            k, v = self.k.view(T, self.hc, D), self.v.view(T, self.hc, D)
        self.wrapper.run(self.q.view(T, self.hc, D), k, v,
                         sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr,
                         out=self.attn.view(T, self.hc, D))
        flashomni_gemm_reduction(self.attn, self.w.wo, H, sparse_info, sparse_info_indptr, 0,
                                 self.cache if self.add_cache else None,
                                 is_for_cache=False, head_begin=hb, head_dim=D, out=y)
        return y

    def _forward_kv_first(self, x, sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr, y):
        """The same step with every mask-only kernel (GEMM-Q tile list, attention work lists, GEMM-O row lists)
        on a side stream beside the dense K and V projections, which go first: the dense kernel deals its tiles
        statically, some SMs finish a tile early, and the list kernels run there. K is enqueued before the side
        work so that its CTAs are placed first."""
        H, D, hb = self.H, self.D, self.hb
        T = self.B * self.S
        dev = self.device
        cur = torch.cuda.current_stream(dev)
        if self._side is None:
            self._side = torch.cuda.Stream(dev)
            self._start = torch.cuda.Event()
        self._start.record(cur)            # everything of the previous step precedes this event
        n_local = self.hc * D
        if self.fuse_kv:
            flashomni_gemm(x, self.wkv, H, is_full=True, out=self.kv, head_dim=D)
        else:
            flashomni_gemm(x, self.w.wk, H, is_full=True, out=self.k, head_dim=D)
        self._side.wait_event(self._start)
        self._q_list = prepare_gemm_q_list(self.B, self.S, n_local, H, sparse_info, sparse_info_indptr, 0,
                                           head_begin=hb, head_dim=D, into=self._q_list, stream=self._side)
        self.wrapper.prepare_masks(sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr,
                                   stream=self._side, after=self._start)
        self._o_list = prepare_gemm_o_list(self.B, self.S, n_local, H, sparse_info, sparse_info_indptr, 0,
                                           head_begin=hb, head_dim=D, into=self._o_list, stream=self._side)
        if self.fuse_kv:
            kv = self.kv.view(T, 2 * self.hc, D)
            k, v = kv[:, :self.hc], kv[:, self.hc:]
        else:
            flashomni_gemm(x, self.w.wv, H, is_full=True, out=self.v, head_dim=D)
            k, v = self.k.view(T, self.hc, D), self.v.view(T, self.hc, D)
        flashomni_gemm(x, self.w.wq, H, sparse_info, sparse_info_indptr, 0, None, out=self.q,
                       head_begin=hb, head_dim=D, worklist=self._q_list)
        self.wrapper.run(self.q.view(T, self.hc, D), k, v,
                         sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr,
                         out=self.attn.view(T, self.hc, D))
        flashomni_gemm_reduction(self.attn, self.w.wo, H, sparse_info, sparse_info_indptr, 0,
                                 self.cache if self.add_cache else None,
                                 is_for_cache=False, head_begin=hb, head_dim=D, out=y, worklist=self._o_list)
        return y


class UlyssesSparseDiTAttentionBlock:
    """The same block under Ulysses sequence parallelism (long video sequences, batch 1): this rank holds the
    tokens [tok_begin, tok_end) (whole 128-token blocks) and full weights; the projections run on the local
    tokens for all heads, an all-to-all regroups Q/K/V to [all tokens, local heads] for the attention, and a
    second one brings the attention output back to [local tokens, all heads] for GEMM-O. With one rank the
    exchanges are skipped."""

    def __init__(self, weights: BlockWeights, num_heads: int, head_dim: int, num_tokens: int, rank: int, world: int,
                 device, dtype=torch.bfloat16, group=None, exchange: str = "p2p"):
        from . import parallel as par
        self.par = par
        self.w, self.H, self.D, self.S = weights, num_heads, head_dim, num_tokens
        self.rank, self.world, self.group, self.device, self.dtype = rank, world, group, device, dtype
        self.t0, self.t1 = par.token_range(num_tokens, rank, world)
        self.s_loc = self.t1 - self.t0
        if self.s_loc % 128 != 0:
            raise ValueError("the local token count must be a multiple of 128 (GEMM row tiles)")
        self.hb, self.hc = par.head_window(num_heads, rank, world)
        hid_out = weights.wo.shape[0]
        mk = lambda *s: torch.zeros(*s, dtype=dtype, device=device)
        n = num_heads * head_dim
        self.px = par.PeerExchange(group, device) if (world > 1 and exchange == "p2p") else None
        if self.px is not None and self.px.available:
            # buffers that other ranks read: symmetric memory, the same (largest) shape on every rank
            rows_max = max(par.shard_blocks((num_tokens + 127) // 128, world)) * 128
            self.q_full, self.q_ptrs, _ = self.px.alloc((1, rows_max, n), dtype)
            self.k_full, self.k_ptrs, _ = self.px.alloc((1, rows_max, n), dtype)
            self.v_full, self.v_ptrs, _ = self.px.alloc((1, rows_max, n), dtype)
            self.q, self.k, self.v = (t[:, :self.s_loc] for t in (self.q_full, self.k_full, self.v_full))
            self.attn, self.attn_ptrs, _ = self.px.alloc((num_tokens, self.hc, head_dim), dtype)
            self.heads_in = [mk(num_tokens, self.hc, head_dim) for _ in range(3)]
            self.o_loc = mk(self.s_loc, num_heads, head_dim)
            self.exchange = "p2p"
        else:
            self.q, self.k, self.v = mk(1, self.s_loc, n), mk(1, self.s_loc, n), mk(1, self.s_loc, n)
            self.attn = mk(num_tokens, self.hc, head_dim)
            self.exchange = "nccl" if world > 1 else "none"
        if self.exchange == "nccl":
            # the exchange of Q (K) runs on a side stream beside the projection of K (V)
            self.heads_in = [mk(num_tokens, self.hc, head_dim) for _ in range(3)]
            self.send_buf = [mk(world * self.s_loc, self.hc, head_dim) for _ in range(3)]
            self.on_gpu = torch.device(device).type == "cuda"
            if self.on_gpu:
                self.comm_stream = torch.cuda.Stream(device=device)
                self.ev = [torch.cuda.Event() for _ in range(4)]
        self.y = mk(1, self.s_loc, hid_out)
        self.cache = mk(1, self.s_loc, hid_out)
        self.wrapper = BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1 << 20, dtype=torch.uint8, device=device))
        indptr = torch.tensor([0, num_tokens], dtype=torch.int32, device=device)
        self.wrapper.plan(indptr, indptr, self.hc, self.hc, head_dim, q_data_type=dtype, mask_num_heads=num_heads,
                          mask_head_begin=self.hb)

    def check_status(self) -> None:
        """Synchronises and raises if a kernel of the last steps recorded a device-side problem or a barrier gave up
        waiting for a peer."""
        self.wrapper.check_status()
        if self.px is not None and self.px.available:
            self.px.check_status()

    def forward(self, x_local, sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr, marks=None):
        """x_local [1, local tokens, hidden] -> this rank's rows of the block output [1, local tokens, hidden].
        `marks` (a list) receives CUDA events at the phase boundaries: start, projections + exchange done,
        attention done, exchange back done, end (with the peer-memory exchange also before and after each of the
        two barriers)."""
        H, D, S = self.H, self.D, self.S

        def mark():
            if marks is not None:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                marks.append(e)

        mark()
        self.wrapper.prepare_masks(sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr)
        # the row offset of the local tokens inside the sequence is what the ops call num_text_tokens
        if self.exchange == "p2p":
            flashomni_gemm(x_local, self.w.wq, H, sparse_info, sparse_info_indptr, self.t0, None, out=self.q, head_dim=D)
            flashomni_gemm(x_local, self.w.wk, H, is_full=True, out=self.k, head_dim=D)
            flashomni_gemm(x_local, self.w.wv, H, is_full=True, out=self.v, head_dim=D)
            mark()
            self.px.barrier(0)  # every rank's projections are complete (and its previous pull of attn is over)
            mark()
            isz = self.q.element_size()
            for ptrs, dst in zip((self.q_ptrs, self.k_ptrs, self.v_ptrs), self.heads_in):
                self.px.pull_heads(ptrs, S, H, D, isz, dst)
            qh, kh, vh = self.heads_in
        elif self.world > 1 and self.on_gpu:
            main = torch.cuda.current_stream()
            proj = ((self.q, self.w.wq, False), (self.k, self.w.wk, True), (self.v, self.w.wv, True))
            for i, (dst, w, dense) in enumerate(proj):
                if dense:
                    flashomni_gemm(x_local, w, H, is_full=True, out=dst, head_dim=D)
                else:
                    flashomni_gemm(x_local, w, H, sparse_info, sparse_info_indptr, self.t0, None, out=dst, head_dim=D)
                self.ev[i].record(main)
                with torch.cuda.stream(self.comm_stream):
                    self.comm_stream.wait_event(self.ev[i])
                    self.par.tokens_to_heads(dst.view(self.s_loc, H, D), S, self.group, out=self.heads_in[i],
                                             send_buf=self.send_buf[i])
            self.ev[3].record(self.comm_stream)
            main.wait_event(self.ev[3])
            qh, kh, vh = self.heads_in
        else:
            flashomni_gemm(x_local, self.w.wq, H, sparse_info, sparse_info_indptr, self.t0, None, out=self.q, head_dim=D)
            flashomni_gemm(x_local, self.w.wk, H, is_full=True, out=self.k, head_dim=D)
            flashomni_gemm(x_local, self.w.wv, H, is_full=True, out=self.v, head_dim=D)
            if self.world > 1:
                qh, kh, vh = (self.par.tokens_to_heads(t.view(self.s_loc, H, D), S, self.group, out=o, send_buf=sb)
                              for t, o, sb in zip((self.q, self.k, self.v), self.heads_in, self.send_buf))
            else:
                qh, kh, vh = (t.view(S, H, D) for t in (self.q, self.k, self.v))
        mark()
        self.wrapper.run(qh, kh, vh, sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr,
                         out=self.attn)
        mark()
        if self.exchange == "p2p":
            self.px.barrier(1)  # every rank's attention is complete (and its pulls of q / k / v are over)
            mark()
            self.px.pull_tokens(self.attn_ptrs, S, H, D, self.attn.element_size(), self.o_loc)
            o_loc = self.o_loc
        else:
            o_loc = self.par.heads_to_tokens(self.attn, S, self.group) if self.world > 1 else self.attn
        mark()
        flashomni_gemm_reduction(o_loc.view(1, self.s_loc, H * D), self.w.wo, H, sparse_info, sparse_info_indptr,
                                 self.t0, self.cache, is_for_cache=False, head_dim=D, out=self.y)
        mark()
        return self.y
