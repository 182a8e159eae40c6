"""Multi-GPU partitioning of the sparse DiT attention block (one process per GPU).

Two schemes, both new with respect to the reference (which has no distributed code at all):

* head partition (`head_window`): rank r owns heads [r*H/P, (r+1)*H/P); nothing crosses GPUs inside the
  block (flashomni_b200.layer.SparseDiTAttentionBlock takes the window). The ranks' partial outputs are
  summed after the block by `PeerExchange.reduce_rows` (each rank sums the row slice it owns, reading the
  peers' partials over NVLink), or by a library reduce-scatter where peer memory is not available.
* Ulysses sequence parallelism for long sequences: tokens are sharded by whole 128-token blocks; the
  projections run on local tokens for all heads; one exchange turns [local tokens, all heads] into
  [all tokens, local heads] for the attention, and one turns the result back. `PeerExchange` does the
  exchange with this library's own kernels over peer memory: the buffers live in symmetric memory, every
  rank PULLS the slices it needs (`fo_strided_gather`, plain loads over NVLink, written in their final
  layout) and the steps are ordered by `fo_peer_barrier` (bounded waits, an error status instead of a
  trap). `tokens_to_heads` / `heads_to_tokens` keep the `torch.distributed.all_to_all_single` form of the
  same exchange (NCCL on GPUs, gloo in the CPU tests) for where symmetric memory cannot be set up.
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


class PeerExchange:
    """The exchanges over peer memory instead of library collectives: the buffers that other ranks read live
    in symmetric memory (every rank maps every rank's copy), each rank pulls (or sums) the slices it needs
    with one kernel of this library (`fo_strided_gather`, `fo_reduce_rows`: plain loads over NVLink, results
    written in their final layout), and the steps are ordered by `fo_peer_barrier`: a single-CTA kernel per
    rank that posts this rank's arrival into every peer's flag pad and waits, for at most `timeout_ms`, for
    theirs. A peer that never arrives leaves FO_DEV_WAIT_TIMEOUT in the status word (`check_status()` raises);
    nothing traps and the CUDA context stays usable.

    `available` is False when symmetric memory cannot be set up (CPU tensors, a torch build without it, a
    failed rendezvous); callers then keep the `all_to_all_single` / reduce-scatter path."""

    CHANNELS = 4

    def __init__(self, group, device, timeout_ms: int = 2000):
        self.group = group if group is not None else dist.group.WORLD
        self.device = torch.device(device)
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.timeout_ms = timeout_ms
        self.available = False
        self._sm = None
        if self.device.type != "cuda":
            return
        try:
            import ctypes
            import os
            # Only unicast peer pointers are used here: ask torch not to bind the buffers to an NVLink multicast
            # object (a rank that exits while bound to one can fault its peers). Unknown to a torch that has no such
            # switch, where it changes nothing.
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as sm
            self._sm = sm
            pad = sm.empty((self.CHANNELS * self.world,), dtype=torch.int32, device=self.device)
            pad.zero_()
            hdl = sm.rendezvous(pad, self.group)
            self._pad, self._pad_hdl = pad, hdl
            self._pads = (ctypes.c_void_p * self.world)(*[int(p) for p in hdl.buffer_ptrs])
            self._epoch = torch.zeros(self.CHANNELS, dtype=torch.int32, device=self.device)
            self._status = torch.zeros(4, dtype=torch.int32, device=self.device)
            # no rank may post an arrival before every pad has been zeroed
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
            self.available = True
        except Exception as e:  # noqa: BLE001 - any failure means "not available here"
            self.reason = f"{type(e).__name__}: {e}"

    def alloc(self, shape, dtype):
        """A zero-filled tensor in symmetric memory (same shape on every rank) and the device pointers of all
        ranks' copies as mapped into this process."""
        t = self._sm.empty(tuple(shape), dtype=dtype, device=self.device)
        t.zero_()
        hdl = self._sm.rendezvous(t, self.group)
        return t, [int(p) for p in hdl.buffer_ptrs], hdl

    def barrier(self, channel: int = 0):
        """All ranks' work queued before this point on their current streams is complete (and visible to the
        peers) when the current stream passes it. Ranks must use the channels in the same order."""
        from . import _native
        rc = _native.load().fo_peer_barrier(self.world, self.rank, self._pads, channel, self.CHANNELS,
                                            self._epoch.data_ptr(), self._status.data_ptr(), self.timeout_ms,
                                            torch.cuda.current_stream(self.device).cuda_stream)
        _native.check(rc, "fo_peer_barrier")

    def check_status(self) -> None:
        """Synchronises and raises if a barrier gave up waiting for a peer."""
        if int(self._status[0].item()) != 0:
            raise RuntimeError("flashomni_b200: a peer barrier timed out (a rank did not arrive)")

    def reduce_rows(self, peer_ptrs, row0: int, n_rows: int, row_elems: int, dtype, out: torch.Tensor,
                    init: torch.Tensor | None = None):
        """out[:n_rows] = init[:n_rows] + sum over ranks of their partial rows [row0, row0 + n_rows):
        `peer_ptrs[r]` is rank r's partial [rows, row_elems] in symmetric memory; fp32 accumulation."""
        import ctypes
        from . import _native
        from .utils import native_dtype
        isz = 2
        row_bytes = row_elems * isz
        n = len(peer_ptrs)
        srcs = (ctypes.c_void_p * n)(*[p + row0 * row_bytes for p in peer_ptrs])
        rc = _native.load().fo_reduce_rows(n, srcs, row_bytes, None if init is None else init.data_ptr(),
                                           0 if init is None else init.stride(0) * isz, out.data_ptr(),
                                           out.stride(0) * isz, n_rows, row_bytes, native_dtype(dtype),
                                           torch.cuda.current_stream(self.device).cuda_stream)
        _native.check(rc, "fo_reduce_rows")

    @staticmethod
    def gather(srcs, src_strides, n_rows, dsts, dst_strides, row_bytes: int):
        """One launch of the strided row gather on the current stream (lists of equal length, byte units)."""
        import ctypes
        from . import _native
        n = len(srcs)
        lib = _native.load()
        P = ctypes.c_void_p * n
        L = ctypes.c_int64 * n
        rc = lib.fo_strided_gather(n, P(*srcs), L(*src_strides), L(*n_rows), P(*dsts), L(*dst_strides), row_bytes,
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        _native.check(rc, "fo_strided_gather")

    def pull_heads(self, peer_ptrs, num_tokens: int, num_heads: int, head_dim: int, itemsize: int, out: torch.Tensor):
        """tokens -> heads: `peer_ptrs[r]` is rank r's [local tokens of r, H, D] buffer; fills `out`
        [num_tokens, H/P, D] with this rank's heads of every rank's tokens."""
        hc = num_heads // self.world
        row = hc * head_dim * itemsize
        srcs, sst, rows, dsts, dst_ = [], [], [], [], []
        for r in range(self.world):
            a, b = token_range(num_tokens, r, self.world)
            srcs.append(peer_ptrs[r] + self.rank * row)
            sst.append(num_heads * head_dim * itemsize)
            rows.append(b - a)
            dsts.append(out.data_ptr() + a * row)
            dst_.append(row)
        self.gather(srcs, sst, rows, dsts, dst_, row)

    def pull_tokens(self, peer_ptrs, num_tokens: int, num_heads: int, head_dim: int, itemsize: int, out: torch.Tensor):
        """heads -> tokens: `peer_ptrs[r]` is rank r's [num_tokens, H/P, D] buffer (its heads); fills `out`
        [local tokens, H, D] with all heads of this rank's tokens."""
        hc = num_heads // self.world
        row = hc * head_dim * itemsize
        a, b = token_range(num_tokens, self.rank, self.world)
        n = self.world
        self.gather([peer_ptrs[r] + a * row for r in range(n)], [row] * n, [b - a] * n,
                    [out.data_ptr() + r * row for r in range(n)], [num_heads * head_dim * itemsize] * n, row)
