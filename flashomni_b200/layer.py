"""A sparse DiT attention block assembled from the public ops, the way a FlashOmni user wires them:
GEMM-Q (sparse) + GEMM-K/V (dense) -> block-sparse attention -> GEMM-O (active heads + cached rest).

Heads can be partitioned over ranks: a rank that owns heads [head_begin, head_begin + head_count) holds
the matching rows of W_q/W_k/W_v and the matching K-slice of W_o, reads the full hidden state and the
full masks, and produces a partial output [B, S, hidden] (its heads' contribution plus its share of the
cache). Nothing inside the block crosses GPUs; the sum of the partials is left to the caller.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .attention import BatchFlashOmniFAWithRaggedKVWrapper
from .gemm import flashomni_gemm, flashomni_gemm_reduction


@dataclass
class BlockWeights:
    wq: torch.Tensor   # [head_count*D, hidden]
    wk: torch.Tensor
    wv: torch.Tensor
    wo: torch.Tensor   # [hidden, head_count*D]


class SparseDiTAttentionBlock:
    def __init__(self, weights: BlockWeights, num_heads: int, head_dim: int, batch: int, seq: int,
                 head_begin: int = 0, head_count: Optional[int] = None, device=None, dtype=torch.bfloat16):
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
        self.k = mk(batch, seq, n_local)
        self.v = mk(batch, seq, n_local)
        self.attn = mk(batch, seq, n_local)   # skipped q-blocks keep their previous contents
        self.y = mk(batch, seq, weights.wo.shape[0])
        self.cache = mk(batch, seq, weights.wo.shape[0])
        self.wrapper = BatchFlashOmniFAWithRaggedKVWrapper(torch.empty(1 << 20, dtype=torch.uint8, device=self.device))
        indptr = torch.arange(batch + 1, dtype=torch.int32, device=self.device) * seq
        self.wrapper.plan(indptr, indptr, self.hc, self.hc, head_dim, q_data_type=dtype,
                          mask_num_heads=num_heads, mask_head_begin=head_begin)

    def refresh_cache(self, x, sparse_info, sparse_info_indptr):
        """The full step of the two-call protocol: cache = contribution of the heads that the sparse steps
        will skip (computed from a dense attention output held in self.attn)."""
        flashomni_gemm_reduction(self.attn, self.w.wo, self.H, sparse_info, sparse_info_indptr, 0, None,
                                 is_for_cache=True, head_begin=self.hb, head_dim=self.D, out=self.cache)
        return self.cache

    def forward(self, x, sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr):
        """One sparse step. x [B, S, hidden]. Returns this rank's (partial) output [B, S, hidden]."""
        H, D, hb = self.H, self.D, self.hb
        flashomni_gemm(x, self.w.wq, H, sparse_info, sparse_info_indptr, 0, None, out=self.q,
                       head_begin=hb, head_dim=D)
        flashomni_gemm(x, self.w.wk, H, is_full=True, out=self.k, head_dim=D)
        flashomni_gemm(x, self.w.wv, H, is_full=True, out=self.v, head_dim=D)
        T = self.B * self.S
        self.wrapper.run(self.q.view(T, self.hc, D), self.k.view(T, self.hc, D), self.v.view(T, self.hc, D),
                         sparse_info, sparse_kv_info, sparse_info_indptr, sparse_kv_info_indptr,
                         out=self.attn.view(T, self.hc, D))
        flashomni_gemm_reduction(self.attn, self.w.wo, H, sparse_info, sparse_info_indptr, 0, self.cache,
                                 is_for_cache=False, head_begin=hb, head_dim=D, out=self.y)
        return self.y
