"""Definition of the golden cases: small seeded inputs (rebuilt identically wherever they are needed)
whose outputs were produced by the REFERENCE's own CUDA kernels (see make_golden.py)."""

from __future__ import annotations

import numpy as np
import torch

from flashomni_b200 import workloads as wl


def attention_case(name):
    group, D, causal = 1, 128, False
    if name == "attn_uniform":
        H, lens_q, lens_kv, density, seed = 2, [512], [512], 0.6, 101
    elif name == "attn_ragged":
        H, lens_q, lens_kv, density, seed = 3, [300, 205], [256, 333], 0.7, 102
    elif name == "attn_gqa":     # 4 q heads on 2 kv heads: mask q-blocks are 64 tokens x the 2 q heads of a kv head
        H, lens_q, lens_kv, density, seed, group = 4, [320, 205], [256, 333], 0.7, 103, 2
    elif name == "attn_gqa4":    # 8 q heads on 2 kv heads: 32 tokens x 4 q heads
        H, lens_q, lens_kv, density, seed, group = 8, [100, 256], [384, 130], 0.6, 104, 4
    elif name == "attn_hd64":    # head dimension 64, ragged
        H, lens_q, lens_kv, density, seed, D = 3, [300, 205], [256, 333], 0.7, 105, 64
    elif name == "attn_hd64_gqa":
        H, lens_q, lens_kv, density, seed, group, D = 4, [130, 256], [384, 130], 0.6, 106, 2, 64
    elif name == "attn_hd256":   # head dimension 256, ragged
        H, lens_q, lens_kv, density, seed, D = 3, [300, 205], [256, 333], 0.7, 111, 256
    elif name == "attn_hd256_gqa":
        H, lens_q, lens_kv, density, seed, group, D = 4, [130, 256], [384, 130], 0.6, 112, 2, 256
    elif name == "attn_causal":         # causal mask inside the kept blocks; kv longer than q (offset kv_len - q_len)
        H, lens_q, lens_kv, density, seed, causal = 3, [300, 205], [428, 333], 0.7, 107, True
    elif name == "attn_causal_gqa":
        H, lens_q, lens_kv, density, seed, group, causal = 4, [130, 256], [384, 300], 0.6, 108, 2, True
    elif name == "attn_custom_mask":     # a random element mask inside the kept blocks (column 0 always visible)
        H, lens_q, lens_kv, density, seed = 3, [300, 205], [428, 333], 0.7, 109
    elif name == "attn_custom_mask_gqa":
        H, lens_q, lens_kv, density, seed, group = 4, [130, 256], [384, 300], 0.6, 110, 2
    else:
        raise KeyError(name)
    custom = name.startswith("attn_custom_mask")
    Hkv = H // group
    qtok = 128 // group           # tokens per mask q-block (128 packed rows)
    qo = np.concatenate([[0], np.cumsum(lens_q)]).astype(np.int32)
    kv = np.concatenate([[0], np.cumsum(lens_kv)]).astype(np.int32)
    rng = np.random.default_rng(seed)
    qa = [(rng.random((-(-a // qtok), Hkv)) < density).astype(np.uint8) for a in lens_q]
    kk = [(rng.random((-(-a // qtok), Hkv, -(-b // 128))) < density).astype(np.uint8) for a, b in zip(lens_q, lens_kv)]
    for a, b in zip(qa, kk):
        a[0, 0] = 1
        b[0, 0, 0] = 1          # at least one non-trivial item
        b *= a[:, :, None]
        # the reference writes garbage-free output only if an active q-block keeps something; keep >= 1
        for qb in range(a.shape[0]):
            for h in range(Hkv):
                if a[qb, h] and (b[qb, h].sum() == 0 or causal or custom):
                    b[qb, h, 0] = 1     # causal: kv position 0 is visible to every token (kv_len >= q_len)
    m = wl.pack_masks(qa, kk)
    q = wl.randn_bf16((int(qo[-1]), H, D), seed + 1)
    k = wl.randn_bf16((int(kv[-1]), Hkv, D), seed + 2)
    v = wl.randn_bf16((int(kv[-1]), Hkv, D), seed + 3)
    prior = wl.randn_bf16((int(qo[-1]), H, D), seed + 4)
    custom_mask = None
    if custom:   # per request [q_len, kv_len] flags; kv position 0 stays visible so that no row is fully masked
        crng = np.random.default_rng(seed + 50)
        custom_mask = [crng.random((a, b)) < 0.6 for a, b in zip(lens_q, lens_kv)]
        for cm in custom_mask:
            cm[:, 0] = True
    return {"q": q, "k": k, "v": v, "qo": qo, "kv": kv, "masks": m, "prior": prior, "H": H, "Hkv": Hkv, "group": group,
            "q_block_tokens": qtok, "D": D, "causal": causal, "custom_mask": custom_mask}


def flat_custom_mask(case):
    """The case's custom mask as the reference's plan() takes it: all matrices flattened and concatenated (bool)."""
    return torch.from_numpy(np.concatenate([cm.reshape(-1) for cm in case["custom_mask"]]))


ATTENTION_CASES = ("attn_uniform", "attn_ragged", "attn_gqa", "attn_gqa4", "attn_hd64", "attn_hd64_gqa", "attn_hd256", "attn_hd256_gqa", "attn_causal",
                   "attn_causal_gqa", "attn_custom_mask", "attn_custom_mask_gqa")


def gemm_case(name):
    if name == "gemm_q":
        B, nq, H, K, seed = 1, 3, 2, 256, 201
    elif name == "gemm_o":
        B, nq, H, K, seed = 2, 2, 2, 256, 202
    else:
        raise KeyError(name)
    m = wl.flux_masks(B, H, nq, nq, 0.5, seed=seed, text_blocks=1)
    x = wl.randn_bf16((B, nq * 128, K), seed + 1)
    w = wl.randn_bf16((H * 128, K), seed + 2, std=K ** -0.5)
    bias = wl.randn_bf16((H * 128,), seed + 3)
    prior = wl.randn_bf16((B, nq * 128, H * 128), seed + 4)
    return {"x": x, "w": w, "bias": bias, "prior": prior, "masks": m, "H": H, "B": B}


def packbits_case():
    rng = np.random.default_rng(301)
    lens = [0, 1, 7, 8, 9, 63, 64, 65, 1000, 2047]
    indptr = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    x = rng.integers(0, 2, int(indptr[-1])).astype(np.uint8)
    return x, indptr


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).cpu().numpy().copy()


def from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.copy()).view(torch.bfloat16)
