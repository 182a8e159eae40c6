"""Multi-GPU partitioning of the sparse DiT attention block (one process per GPU).

Two schemes, both new with respect to the reference (which has no distributed code at all):

* head partition (`head_window`): rank r owns heads [r*H/P, (r+1)*H/P); nothing crosses GPUs inside the
  block (flashomni_b200.layer.SparseDiTAttentionBlock takes the window).
* Ulysses sequence parallelism for long sequences: tokens are sharded by whole 128-token blocks; the
  projections run on local tokens for all heads; one all-to-all turns [local tokens, all heads] into
  [all tokens, local heads] for the attention, and one turns the result back. The exchange is a plain
  `torch.distributed.all_to_all_single` (NCCL over NVLink on GPUs, gloo in the CPU tests); data always
  lands in the receiver's own memory before any kernel reads it.
"""

from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist

BLOCK = 128


def head_window(num_heads: int, rank: int, world: int) -> Tuple[int, int]:
    """(head_begin, head_count) of a rank; heads must divide evenly."""
    if num_heads % world != 0:
        raise ValueError(f"{num_heads} heads cannot be split evenly over {world} ranks")
    hc = num_heads // world
    return rank * hc, hc


def shard_blocks(num_blocks: int, world: int) -> List[int]:
    """Number of 128-token blocks per rank: as even as possible, the first ranks take the remainder
    (604 blocks over 8 ranks -> 76,76,76,76,75,75,75,75)."""
    base, rem = divmod(num_blocks, world)
    return [base + (1 if r < rem else 0) for r in range(world)]


def token_range(num_tokens: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) token range of a rank when tokens are sharded by whole 128-token blocks."""
    nblk = (num_tokens + BLOCK - 1) // BLOCK
    per = shard_blocks(nblk, world)
    b0 = sum(per[:rank]) * BLOCK
    b1 = min(num_tokens, b0 + per[rank] * BLOCK)
    return b0, b1


def tokens_to_heads(x: torch.Tensor, num_tokens: int, group=None, out: torch.Tensor | None = None,
                    send_buf: torch.Tensor | None = None) -> torch.Tensor:
    """[local tokens, H, D] (all heads of my token range) -> [all tokens, H/P, D] (my heads of all tokens).
    `out` ([num_tokens, H/P, D]) and `send_buf` ([P * local tokens, H/P, D]) let a caller reuse its buffers."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    s_loc, H, D = x.shape
    hc = H // world
    counts = [token_range(num_tokens, r, world) for r in range(world)]
    counts = [b - a for a, b in counts]
    assert counts[rank] == s_loc, "local token count does not match the block sharding"
    src = x.view(s_loc, world, hc, D).permute(1, 0, 2, 3)
    if send_buf is None:
        send = src.contiguous().view(world * s_loc, hc, D)
    else:
        send_buf.view(world, s_loc, hc, D).copy_(src)
        send = send_buf
    recv = out if out is not None else torch.empty((num_tokens, hc, D), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(recv, send, output_split_sizes=counts, input_split_sizes=[s_loc] * world, group=group)
    return recv


def heads_to_tokens(x: torch.Tensor, num_tokens: int, group=None) -> torch.Tensor:
    """[all tokens, H/P, D] (my heads) -> [local tokens, H, D] (all heads of my token range)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    S, hc, D = x.shape
    counts = [token_range(num_tokens, r, world) for r in range(world)]
    counts = [b - a for a, b in counts]
    s_loc = counts[rank]
    recv = torch.empty((world * s_loc, hc, D), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(recv, x.contiguous(), output_split_sizes=[s_loc] * world, input_split_sizes=counts, group=group)
    return recv.view(world, s_loc, hc, D).permute(1, 0, 2, 3).contiguous().view(s_loc, world * hc, D)
