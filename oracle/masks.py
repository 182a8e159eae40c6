"""CPU oracle (test infrastructure): bit packing, bit addressing and the canonical outputs of
the mask-compaction step. Integer work only; every comparison against it is bit-exact.

Follows:
  * packbits / segment_packbits: flashomni/quantization.py:68-159 (same semantics as numpy.packbits;
    per-segment packing, padding bits of a segment's last byte are zero, new indptr = cumsum of
    ceil(len/8) bytes, :148-152).
  * bit addressing used by all three kernels: include/flashomni/attention/prefill.cuh:1284-1294
    (q-block bit `qb*H + h`), :1385-1394 (kv-block bit `(qb*H + h)*nkv + kvb`),
    include/flashomni/gemm/w16a16/gemm.cuh:50-58 and gemm_reduction.cuh:128-145 (GEMM row block ->
    q-block `(num_text_tokens + iy*128) // sparse_q_size`). Bits are little-endian inside a byte.
  * unpacked indptrs: flashomni/attention.py:165-191.
"""

from __future__ import annotations

import numpy as np


def packbits(x: np.ndarray, bitorder: str = "big") -> np.ndarray:
    """flashomni/quantization.py:68-99."""
    if bitorder not in ("big", "little"):
        raise ValueError("bitorder must be 'big' or 'little'")
    x = np.asarray(x).reshape(-1)
    return np.packbits(x.astype(bool), bitorder=bitorder)


def segment_packbits(x: np.ndarray, indptr: np.ndarray, bitorder: str = "big"):
    """flashomni/quantization.py:102-159. Returns (packed uint8, new byte indptr int32)."""
    if bitorder not in ("big", "little"):
        raise ValueError("bitorder must be 'big' or 'little'")
    x = np.asarray(x).reshape(-1)
    indptr = np.asarray(indptr, dtype=np.int64)
    seglen = indptr[1:] - indptr[:-1]
    packed_len = (seglen + 7) // 8
    new_indptr = np.zeros(len(indptr), dtype=np.int64)
    new_indptr[1:] = np.cumsum(packed_len)
    out = np.zeros(int(new_indptr[-1]), dtype=np.uint8)
    for i in range(len(indptr) - 1):
        seg = x[indptr[i]:indptr[i + 1]].astype(bool)
        out[new_indptr[i]:new_indptr[i + 1]] = np.packbits(seg, bitorder=bitorder)
    return out, new_indptr.astype(np.int32)


def sparse_info_indptr(qo_indptr, num_heads: int, sbq: int) -> np.ndarray:
    """Unpacked (bit-count) indptr of `sparse_info`: flashomni/attention.py:165-176."""
    qo = np.asarray(qo_indptr, dtype=np.int64)
    nq = -(-(qo[1:] - qo[:-1]) // sbq)
    out = np.zeros(len(qo), dtype=np.int64)
    out[1:] = np.cumsum(nq * num_heads)
    return out


def sparse_kv_info_indptr(qo_indptr, kv_indptr, num_heads: int, sbq: int, sbkv: int) -> np.ndarray:
    """Unpacked (bit-count) indptr of `sparse_kv_info`: flashomni/attention.py:178-191."""
    qo = np.asarray(qo_indptr, dtype=np.int64)
    kv = np.asarray(kv_indptr, dtype=np.int64)
    nq = -(-(qo[1:] - qo[:-1]) // sbq)
    nkv = -(-(kv[1:] - kv[:-1]) // sbkv)
    out = np.zeros(len(qo), dtype=np.int64)
    out[1:] = np.cumsum(nq * nkv * num_heads)
    return out


def get_bit(seg: np.ndarray, i: int) -> int:
    """Little-endian bit i of a packed segment (prefill.cuh:1288-1290)."""
    return (int(seg[i >> 3]) >> (i & 7)) & 1


def unpack_segment(packed: np.ndarray, byte_off: int, nbits: int) -> np.ndarray:
    nbytes = (nbits + 7) // 8
    seg = np.asarray(packed[byte_off:byte_off + nbytes], dtype=np.uint8)
    return np.unpackbits(seg, bitorder="little")[:nbits]


def unpack_masks(sparse_info, sparse_kv_info, info_indptr, kv_info_indptr, qo_indptr, kv_indptr,
                 num_heads: int, sbq: int, sbkv: int):
    """Per request b: (q_active[nq, H], kv_kept[nq, H, nkv]) as uint8 arrays, decoded from the packed
    byte streams with the byte indptrs (the form the kernels receive)."""
    qo = np.asarray(qo_indptr, dtype=np.int64)
    kv = np.asarray(kv_indptr, dtype=np.int64)
    out = []
    for b in range(len(qo) - 1):
        nq = int(-(-(qo[b + 1] - qo[b]) // sbq))
        nkv = int(-(-(kv[b + 1] - kv[b]) // sbkv))
        qa = unpack_segment(sparse_info, int(info_indptr[b]), nq * num_heads).reshape(nq, num_heads)
        kk = unpack_segment(sparse_kv_info, int(kv_info_indptr[b]), nq * num_heads * nkv)
        out.append((qa, kk.reshape(nq, num_heads, nkv)))
    return out


def order_groups(batch: int, head_count: int, max_nkv: int):
    """(heads per group, by_length) of the processing order of `compact`: groups of heads whose K and V stay in
    L2 together -- 48 MiB / (max_nkv blocks * 64 KiB per head and tensor pair), evenly sized -- ordered by length
    inside a group while batch * groups_per_request * (max_nkv + 1) <= 8192, else single heads, q-blocks ascending."""
    hpg = min(max((48 << 20) // (max(max_nkv, 1) * 65536), 1), head_count)
    grp_per_req = -(-head_count // hpg)
    hpg = -(-head_count // grp_per_req)
    by_length = batch * grp_per_req * (max_nkv + 1) <= 8192
    return (hpg, True) if by_length else (1, False)


def compact(sparse_info, sparse_kv_info, info_indptr, kv_info_indptr, qo_indptr, kv_indptr,
            num_heads: int, sbq: int, sbkv: int, head_begin: int = 0, head_count: int | None = None,
            is_full: bool = False):
    """Canonical outputs of the attention mask-compaction step (the work lists the CUDA attention
    kernel consumes).

    Returns a dict of numpy arrays:
      items      int32 [n, 4]  (b, h, qb, n_kept) for every active (b, qb, h) with h in the head window,
                               ascending in (b, qb, h)
      kv_indptr  int32 [n+1]   offsets of each item's kept list inside kv_idx
      kv_idx     int32 [total] ascending kept kv-block indices of each item
      order      int32 [n]     the processing permutation: item indices grouped by (b, group of heads) ascending
                               (CTAs that run at the same time then share K / V tiles in L2). A group is
                               hpg consecutive heads of the window: hpg = min(head_count, max(1, 48 MiB //
                               (max_nkv * 64 KiB))), evened out over ceil(head_count / hpg) groups. Inside a
                               group: by descending list length, ties in canonical order, while
                               batch * groups_per_request * (max_nkv + 1) <= 8192 (the items drawn last are then
                               short ones); otherwise single-head groups with their q-blocks ascending
    With `is_full` every q-block is active and every kv-block kept (prefill.cuh:1284,1383,1434).
    """
    if head_count is None:
        head_count = num_heads - head_begin
    qo = np.asarray(qo_indptr, dtype=np.int64)
    kv = np.asarray(kv_indptr, dtype=np.int64)
    B = len(qo) - 1
    items, kv_ptr, kv_idx = [], [0], []
    for b in range(B):
        nq = int(-(-(qo[b + 1] - qo[b]) // sbq))
        nkv = int(-(-(kv[b + 1] - kv[b]) // sbkv))
        if is_full:
            qa = np.ones((nq, num_heads), dtype=np.uint8)
            kk = np.ones((nq, num_heads, nkv), dtype=np.uint8)
        else:
            qa = unpack_segment(sparse_info, int(info_indptr[b]), nq * num_heads).reshape(nq, num_heads)
            kk = unpack_segment(sparse_kv_info, int(kv_info_indptr[b]),
                                nq * num_heads * nkv).reshape(nq, num_heads, nkv)
        for qb in range(nq):
            for h in range(head_begin, head_begin + head_count):
                if qa[qb, h]:
                    kept = np.nonzero(kk[qb, h])[0]
                    items.append((b, h, qb, len(kept)))
                    kv_idx.extend(int(v) for v in kept)
                    kv_ptr.append(len(kv_idx))
    items_a = np.asarray(items, dtype=np.int32).reshape(-1, 4)
    max_nkv = max([int(-(-(kv[b + 1] - kv[b]) // sbkv)) for b in range(B)], default=0)
    hpg, by_length = order_groups(B, head_count, max_nkv)
    grp_per_req = -(-head_count // hpg)
    if len(items):
        key = items_a[:, 0].astype(np.int64) * grp_per_req + (items_a[:, 1].astype(np.int64) - head_begin) // hpg
        if by_length:
            key = key * (max_nkv + 1) + (max_nkv - items_a[:, 3].astype(np.int64))
        order = np.argsort(key, kind="stable").astype(np.int32)
    else:
        order = np.arange(len(items), dtype=np.int32)
    return {
        "items": items_a,
        "kv_indptr": np.asarray(kv_ptr, dtype=np.int32),
        "kv_idx": np.asarray(kv_idx, dtype=np.int32),
        "order": order,
    }


def attn_units(lists: dict, qo_indptr, kv_indptr, num_streams: int, min_chunk: int = 16, sbq: int = 128,
               sbkv: int = 128, max_slots: int = 1 << 30, min_items: int = 0):
    """Canonical work units of the attention kernel, from the outputs of `compact` (`lists`): the items in
    processing order, one self-contained record of eight int32 per unit:
      [0] n kv blocks of the unit (0: an active q-block that keeps nothing)   [1] offset of its first entry in kv_idx
      [2] mask head | request << 16   [3] first row of the q-block in q / o
      [4] existing rows of the q-block (1..sbq) | columns of the request's partial last kv block if the unit ends with it << 16
      [5] first kv row of the request   [6] qb * sbq + kv_len - q_len (last kv position the block's first token sees under a causal mask)
      [7] slot << 16 | part << 8 | n_parts   (a whole item: n_parts = 1, slot = 0xffff)
    A kv list longer than chunk_max is cut into ceil(n_kept / chunk_max) parts of (almost) equal length, part p
    covering entries [n_kept * p // n_parts, n_kept * (p + 1) // n_parts) -- only when there is room for partial
    results (max_slots > 0) and the launch has more than `min_items` and at most `num_streams` items (the unit count
    the caller aims at: a few per SM): chunk_max = max(min_chunk, ceil(total_kept / num_streams), ceil(max_nkv / 255)); otherwise
    every item is one unit. When lists were cut (and there are at most 2048 units) the units are then put in
    descending order of their length (stable), so that the CTAs, which draw units in list order, take the short
    ones last. (The reference's planner cuts kv RANGES instead, include/flashomni/attention/
    scheduler.cuh:35-64, which with block masks leaves parts without any kept block; cutting the kept LIST cannot.)
    Returns (units int32 [n_units, 8], partial slots in use, chunk_max)."""
    items, order, kvp, kv_idx = lists["items"], lists["order"], lists["kv_indptr"], lists["kv_idx"]
    qo = np.asarray(qo_indptr, dtype=np.int64)
    kv = np.asarray(kv_indptr, dtype=np.int64)
    n_items = len(items)
    total = int(items[:, 3].clip(min=0).sum()) if n_items else 0
    max_nkv = max([int(-(-(kv[b + 1] - kv[b]) // sbkv)) for b in range(len(kv) - 1)], default=0)
    chunk_max = 0x7fffffff
    if max(min_items, 0) < n_items and max_slots > 0 and n_items <= num_streams:
        chunk_max = max(min_chunk, -(-total // num_streams), -(-max_nkv // 255))
    units, slots = [], 0
    for it in order.tolist():
        b, h, qb, n = (int(x) for x in items[it])
        n = max(n, 0)
        n_parts = -(-n // chunk_max) if n > chunk_max else 1
        q0, q_len = int(qo[b]), int(qo[b + 1] - qo[b])
        k0, kv_len = int(kv[b]), int(kv[b + 1] - kv[b])
        q_valid = min(max(q_len - qb * sbq, 0), sbq)
        ragged = 0
        if kv_len % sbkv and n > 0 and int(kv_idx[kvp[it] + n - 1]) == kv_len // sbkv:
            ragged = kv_len % sbkv
        for p in range(n_parts):
            j0, j1 = n * p // n_parts, n * (p + 1) // n_parts
            word = (((slots + p) & 0xffff) << 16) | (p << 8) | n_parts if n_parts > 1 else (0xffff << 16) | 1
            word = word - (1 << 32) if word >= (1 << 31) else word
            units.append((j1 - j0, int(kvp[it]) + j0, h | (b << 16), q0 + qb * sbq, q_valid | ((ragged if p == n_parts - 1 else 0) << 16), k0,
                          qb * sbq + kv_len - q_len, word))
        if n_parts > 1:
            slots += n_parts
    if chunk_max != 0x7fffffff and len(units) <= 2048:
        units.sort(key=lambda r: -r[0])      # stable: equal lengths keep the order above
    return np.asarray(units, dtype=np.int32).reshape(-1, 8), slots, chunk_max


def gemm_q_tiles(sparse_info, info_indptr, batch: int, m: int, n: int, num_heads: int,
                 sparse_q_size: int = 128, num_text_tokens: int = 0, is_full: bool = False,
                 head_begin: int = 0, head_dim: int | None = None) -> np.ndarray:
    """Active 128x128 output tiles of GEMM-Q as int32 [n_tiles, 3] = (b, iy, ix), ascending.
    Tile (iy, ix) of batch b is active iff bit `qb*H + head_begin + (ix*128)//head_dim` of b's segment
    is 1, `qb = (num_text_tokens + iy*128)//sparse_q_size`, `head_dim = N//H` unless given
    (gemm.cuh:50-58, csrc/gemm.cu:26-30)."""
    if head_dim is None:
        head_dim = n // num_heads
    tiles = []
    for b in range(batch):
        for iy in range(m // 128):
            qb = (num_text_tokens + iy * 128) // sparse_q_size
            for ix in range(n // 128):
                if is_full:
                    tiles.append((b, iy, ix))
                    continue
                bit = qb * num_heads + head_begin + (ix * 128) // head_dim
                seg = sparse_info[int(info_indptr[b]):]
                if get_bit(seg, bit):
                    tiles.append((b, iy, ix))
    return np.asarray(tiles, dtype=np.int32).reshape(-1, 3)


GEMM_Q_PAIR_COST, GEMM_Q_SINGLE_COST = 20, 13


def gemm_q_makespan(pairs: int, singles: int, n: int) -> int:
    """End time of the last of `n` CTAs that draw `pairs` two-block tiles (cost 20) and then `singles` single-block
    tiles (cost 13) in list order, every tile going to the CTA that is free first."""
    full, r = divmod(pairs, n)
    t_a, c_a = full * GEMM_Q_PAIR_COST, n - r
    t_b, c_b = (full + 1) * GEMM_Q_PAIR_COST, r
    end = (full + (1 if r else 0)) * GEMM_Q_PAIR_COST
    m = singles
    while m > 0:
        if c_a > 0 and (c_b == 0 or t_a <= t_b):
            m -= c_a
            t_a += GEMM_Q_SINGLE_COST
            end = max(end, t_a)
        else:
            m -= c_b
            t_b += GEMM_Q_SINGLE_COST
            end = max(end, t_b)
    return end


def gemm_q_split_rule(pairs: int, singles: int, n_ctas: int, max_records: int) -> int:
    """How many of the last two-block records are cut into two single-block records: the k in
    [0, min(pairs, n_ctas, 1023)] with pairs + singles + k <= max_records that gives the smallest end time
    (clamped to 32767), the smallest such k."""
    best = None
    for k in range(0, min(pairs, n_ctas, 1023) + 1):
        if pairs + singles + k > max_records:
            break
        t = min(gemm_q_makespan(pairs - k, singles + 2 * k, max(n_ctas, 1)), 32767)
        if best is None or t < best[0]:
            best = (t, k)
    return 0 if best is None else best[1]


def gemm_q_tile_pairs(sparse_info, info_indptr, batch: int, m: int, n: int, num_heads: int,
                      sparse_q_size: int = 128, num_text_tokens: int = 0, is_full: bool = False,
                      head_begin: int = 0, head_dim: int | None = None, num_ctas: int | None = None) -> np.ndarray:
    """The work list GEMM-Q runs over: int32 [n_records, 4] = (b, iy, ix0, ix1). Per row block (b, iy),
    ascending, the active column blocks of `gemm_q_tiles` are taken two at a time in ascending order; a
    leftover single block has ix1 = -1. The list holds all two-block records first and the single-block
    records after them (both in ascending (b, iy) order): the GEMM hands tiles to its CTAs in list order,
    and the half-size tiles at the end fill the last wave. With `num_ctas` (the CTAs of the launch, one per SM)
    the last k two-block records are cut into two single-block records each (`gemm_q_split_rule`), placed between
    the remaining two-block records and the leftover singles."""
    tiles = gemm_q_tiles(sparse_info, info_indptr, batch, m, n, num_heads, sparse_q_size, num_text_tokens,
                         is_full, head_begin, head_dim)
    pairs, singles = [], []
    i = 0
    while i < len(tiles):
        b, iy, ix = (int(v) for v in tiles[i])
        if i + 1 < len(tiles) and int(tiles[i + 1][0]) == b and int(tiles[i + 1][1]) == iy:
            pairs.append((b, iy, ix, int(tiles[i + 1][2])))
            i += 2
        else:
            singles.append((b, iy, ix, -1))
            i += 1
    if num_ctas is not None:
        k = gemm_q_split_rule(len(pairs), len(singles), num_ctas, batch * (m // 128) * (n // 128))
        if k > 0:
            cut = []
            for (b, iy, i0, i1) in pairs[len(pairs) - k:]:
                cut += [(b, iy, i0, -1), (b, iy, i1, -1)]
            pairs = pairs[:len(pairs) - k] + cut
    return np.asarray(pairs + singles, dtype=np.int32).reshape(-1, 4)


def gemm_o_rows(sparse_info, info_indptr, batch: int, m: int, k: int, num_heads: int,
                sparse_q_size: int = 128, num_text_tokens: int = 0, is_for_cache: bool = False,
                head_begin: int = 0, head_dim: int | None = None):
    """Per 128-row block (b, iy) of GEMM-O: ascending list of the local heads whose K-slice is
    accumulated. Head h (local index, global = head_begin + h) is selected iff its bit equals 1
    (`is_for_cache=False`) or 0 (`is_for_cache=True`), gemm_reduction.cuh:128-145,199-218.
    Returns (row_indptr int32[R+1], row_heads int32[...], order int32[R]) with R = batch*m/128 and
    `order` = row blocks by descending list length, ties ascending."""
    if head_dim is None:
        head_dim = k // num_heads
    local_heads = k // head_dim
    indptr, heads = [0], []
    for b in range(batch):
        seg = sparse_info[int(info_indptr[b]):]
        for iy in range(m // 128):
            qb = (num_text_tokens + iy * 128) // sparse_q_size
            for h in range(local_heads):
                bit = get_bit(seg, qb * num_heads + head_begin + h)
                if bit == (0 if is_for_cache else 1):
                    heads.append(h)
            indptr.append(len(heads))
    indptr_a = np.asarray(indptr, dtype=np.int32)
    cnt = (indptr_a[1:] - indptr_a[:-1]).astype(np.int64)
    order = np.argsort(-cnt, kind="stable").astype(np.int32)
    return indptr_a, np.asarray(heads, dtype=np.int32), order
