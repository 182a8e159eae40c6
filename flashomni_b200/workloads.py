"""Seeded synthetic workloads with the shapes and value distributions of the five benchmark
configurations (FLUX-like 4608-token layer, GEMM-Q, GEMM-O, full DiT attention block, Wan-like
video layer). Pure host-side input generation (numpy / torch CPU); nothing here is on the hot path.

Sequence convention (as in the reference's scripts, benchmark/utils.py:7-85): text tokens come
first, 128-token blocks, so text = q/kv blocks 0..3 when there are 512 text tokens.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple

import numpy as np
import torch

BLOCK = 128


@dataclass
class PackedMasks:
    sparse_info: np.ndarray        # uint8, packed little-endian per request
    sparse_kv_info: np.ndarray     # uint8
    info_indptr: np.ndarray        # int32 [B+1], byte offsets
    kv_info_indptr: np.ndarray     # int32 [B+1], byte offsets
    q_active: List[np.ndarray]     # per request [nq, H] uint8
    kv_kept: List[np.ndarray]      # per request [nq, H, nkv] uint8


def pack_masks(q_active: List[np.ndarray], kv_kept: List[np.ndarray]) -> PackedMasks:
    """Packs per-request block masks the way callers of the reference do with
    segment_packbits(..., bitorder="little") (benchmark/test_flashomni_attention.py:254-255)."""
    si, skv, ip, kp = [], [], [0], [0]
    for qa, kk in zip(q_active, kv_kept):
        a = np.packbits(qa.reshape(-1).astype(bool), bitorder="little")
        b = np.packbits(kk.reshape(-1).astype(bool), bitorder="little")
        si.append(a)
        skv.append(b)
        ip.append(ip[-1] + len(a))
        kp.append(kp[-1] + len(b))
    return PackedMasks(np.concatenate(si), np.concatenate(skv), np.asarray(ip, np.int32),
                       np.asarray(kp, np.int32), q_active, kv_kept)


def flux_masks(batch: int, heads: int, nq: int, nkv: int, density: float, seed: int,
               text_blocks: int = 4, kv_density: float | None = None) -> PackedMasks:
    """sparse_info ~ Bernoulli(density) per (q-block, head) with text q-blocks always active;
    sparse_kv_info ~ Bernoulli(kv_density) per (active q-block, head, kv-block) with the diagonal and the
    text kv-blocks always kept, zero where the q-block is inactive."""
    if kv_density is None:
        kv_density = density
    rng = np.random.default_rng(seed)
    qa_l, kk_l = [], []
    for _ in range(batch):
        qa = (rng.random((nq, heads)) < density).astype(np.uint8)
        qa[:text_blocks] = 1
        kk = (rng.random((nq, heads, nkv)) < kv_density).astype(np.uint8)
        kk[:, :, :text_blocks] = 1
        d = np.arange(min(nq, nkv))
        kk[d, :, d] = 1
        kk *= qa[:, :, None]
        qa_l.append(qa)
        kk_l.append(kk)
    return pack_masks(qa_l, kk_l)


def video_masks(heads: int, frames: int, blocks_per_frame: int, seed: int, text_blocks: int = 4,
                random_density: float = 0.10) -> PackedMasks:
    """Spatiotemporal-local mask of the long video layer: every q-block active; a q-block keeps the
    text kv-blocks, the kv-blocks within +-1 frame of its own frame, and Bernoulli(random_density)
    others. Text q-blocks keep text + the random blocks."""
    rng = np.random.default_rng(seed)
    n = text_blocks + frames * blocks_per_frame
    frame = np.full(n, -10, dtype=np.int64)
    frame[text_blocks:] = (np.arange(n - text_blocks) // blocks_per_frame)
    qa = np.ones((n, heads), dtype=np.uint8)
    local = (np.abs(frame[:, None] - frame[None, :]) <= 1) & (frame[:, None] >= 0) & (frame[None, :] >= 0)
    kk = np.empty((n, heads, n), dtype=np.uint8)
    for h in range(heads):
        r = rng.random((n, n)) < random_density
        kk[:, h, :] = (r | local).astype(np.uint8)
    kk[:, :, :text_blocks] = 1
    return pack_masks([qa], [kk])


def randn_bf16(shape, seed: int, std: float = 1.0, dtype=torch.bfloat16) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(dtype)


@dataclass
class AttnInputs:
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    qo_indptr: torch.Tensor
    kv_indptr: torch.Tensor
    masks: PackedMasks


def attention_inputs(batch: int, heads: int, seq: int, head_dim: int, density: float, seed: int,
                     dtype=torch.bfloat16, kv_density: float | None = None) -> AttnInputs:
    """Config-1 style inputs: Q, K, V ~ N(0,1) [batch*seq, heads, head_dim]; equal-length requests."""
    nblk = (seq + BLOCK - 1) // BLOCK
    q = randn_bf16((batch * seq, heads, head_dim), seed + 1, dtype=dtype)
    k = randn_bf16((batch * seq, heads, head_dim), seed + 2, dtype=dtype)
    v = randn_bf16((batch * seq, heads, head_dim), seed + 3, dtype=dtype)
    indptr = torch.arange(0, batch + 1, dtype=torch.int32) * seq
    masks = flux_masks(batch, heads, nblk, nblk, density, seed, text_blocks=min(4, nblk), kv_density=kv_density)
    return AttnInputs(q, k, v, indptr, indptr.clone(), masks)


def executed_attention_tiles(masks: PackedMasks, head_begin: int = 0, head_count: int | None = None) -> int:
    tot = 0
    for qa, kk in zip(masks.q_active, masks.kv_kept):
        hc = qa.shape[1] - head_begin if head_count is None else head_count
        sl = slice(head_begin, head_begin + hc)
        tot += int((kk[:, sl, :] * qa[:, sl, None]).sum())
    return tot


def active_pairs(masks: PackedMasks, head_begin: int = 0, head_count: int | None = None) -> Tuple[int, int]:
    """(active, total) (q-block, head) pairs."""
    act = tot = 0
    for qa in masks.q_active:
        hc = qa.shape[1] - head_begin if head_count is None else head_count
        act += int(qa[:, head_begin:head_begin + hc].sum())
        tot += qa.shape[0] * hc
    return act, tot
