"""Cutting a step's attention into work items for the kernels.

A segment is the run of consecutive tokens one request brings to a step.  It is
cut into tiles of at most ``tile_tokens`` query tokens; a tile attends over the
keys from the start of its window (or 0) up to its last token.  When a step has
too few tiles to fill the GPU and a tile's key range is long (decoding, or a
short portion late in a long prompt), the range is split and the splits are
combined by the reduce kernel, always in the same order.

Item layout (int32 x 8): seg, first query token (index in the step), query
tokens, position of the first query token, first key, one past the last key,
first partial row or -1 when not split, (splits << 16 | index of this split)
or 0 when not split.  The splits of a tile are consecutive items.
Reduction layout (int32 x 4): token index, first partial row, splits, stride
between the token's partial rows.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np

SPLIT_ALIGN = 64   # split boundaries fall on multiples of the kernels' key tiles (32 and 64)
# The shortest split: one tile of keys.  Measured on captured steps of the 0.6B shape (decoded tokens a second
# with 64 / 128 / 256 / 512 keys): batch 1 at context 4096: 1343 / 1266 / 1267 / 1081; batch 1 at context 512:
# 1478 / 1480 / 1450 / 1266; batch 8 at context 512: 10484 / 10490 / 9700 / 8648.  (Before the reduction's list
# was fetched ahead of its wait and the products' tiles were chosen anew, 256 was the best of these.)
MIN_SPLIT_KEYS = 64
MAX_SPLITS = 128   # the reduce kernel holds the weights of up to 256 splits in shared memory
# A tile of many query tokens is cut only where every part still has this many keys: its partial results are
# a tile of rows each, not one row (a 512-token portion behind 1024 tokens of context beside one decoded
# token, 0.6B shape: cut in four from 256 keys on, the attention took 25 us a layer and the reduction 17;
# whole, see profiles/prefill_2048_tokens.md).
MULTI_MIN_SPLIT_KEYS = 2048


def plan_attention(segments: Sequence[Tuple[int, int, int]], tile_tokens: int, window: Optional[int],
                   ctas_per_item: int, target_ctas: int,
                   min_split_keys: int = MIN_SPLIT_KEYS,
                   multi_min_split_keys: int = MULTI_MIN_SPLIT_KEYS) -> Tuple[np.ndarray, np.ndarray, int]:
    """segments: (first token index, token count, position of the first token) per
    segment, in step order.  Returns (work [n, 8], red [m, 4], partial rows used)."""
    seg_ids, q0s, qns, p0s = [], [], [], []
    if segments and all(c == 1 for _, c, _ in segments):
        # a decode step: one tile per segment, no per-segment array work
        a = np.asarray(segments, dtype=np.int64)
        seg_ids, q0s, qns, p0s = [np.arange(len(a))], [a[:, 0]], [a[:, 1]], [a[:, 2]]
        segments = ()
    for si, (tok0, count, pos0) in enumerate(segments):
        if count <= 0:
            continue
        # last tile first: it has the longest key range, and the kernels deal items to the
        # SMs in list order, so the long ones start early and the short ones fill the end
        starts = np.arange(0, count, tile_tokens, dtype=np.int64)[::-1]
        seg_ids.append(np.full(len(starts), si, dtype=np.int64))
        q0s.append(tok0 + starts)
        qns.append(np.minimum(tile_tokens, count - starts))
        p0s.append(pos0 + starts)
    if not seg_ids:
        return np.zeros((0, 8), np.int32), np.zeros((0, 4), np.int32), 0
    seg = np.concatenate(seg_ids); q0 = np.concatenate(q0s); qn = np.concatenate(qns); p0 = np.concatenate(p0s)
    kv_end = p0 + qn
    kv_begin = np.maximum(0, p0 - (window - 1)) if window else np.zeros_like(p0)
    n_tiles = len(seg)
    keys = kv_end - kv_begin

    splits = np.ones(n_tiles, dtype=np.int64)
    if n_tiles * ctas_per_item < target_ctas:
        # as many splits as keep the launch within the target (one or two full waves of
        # CTAs), rounded down so that the last wave is not a sliver.  A step of single tokens that
        # falls short of the target is cut in two at least; tiles of many tokens are not (their
        # partial results are large, and a portion that nearly fills the GPU is better left whole).
        want = target_ctas // (n_tiles * ctas_per_item)
        if want < 2:
            want = 2 if int(qn.max()) == 1 else 1
        floor = np.where(qn > 1, max(min_split_keys, multi_min_split_keys), min_split_keys)
        splits = np.clip(np.minimum(want, keys // floor), 1, MAX_SPLITS)
    if (splits == 1).all():
        work = np.stack([seg, q0, qn, p0, kv_begin, kv_end, np.full(n_tiles, -1), np.zeros(n_tiles, np.int64)], 1)
        return work.astype(np.int32), np.zeros((0, 4), np.int32), 0

    # every tile into its splits, without a Python loop over tiles
    chunk = -(-keys // splits)
    chunk = -(-chunk // SPLIT_ALIGN) * SPLIT_ALIGN
    n_split = np.where(splits > 1, -(-keys // chunk), 1)           # splits that really hold keys
    total = int(n_split.sum())
    tile_of = np.repeat(np.arange(n_tiles), n_split)
    first = np.cumsum(n_split) - n_split
    k = np.arange(total) - first[tile_of]                          # which split of its tile
    is_split = n_split > 1
    begin = kv_begin[tile_of] + k * chunk[tile_of]
    end = np.where(is_split[tile_of], np.minimum(begin + chunk[tile_of], kv_end[tile_of]), kv_end[tile_of])
    rows_of = np.where(is_split, n_split * qn, 0)                  # partial rows a tile uses
    base = np.cumsum(rows_of) - rows_of
    part = np.where(is_split[tile_of], base[tile_of] + k * qn[tile_of], -1)
    # which split of how many
    split = np.where(is_split[tile_of], (n_split[tile_of] << 16) | k, 0)
    work = np.stack([seg[tile_of], q0[tile_of], qn[tile_of], p0[tile_of], begin, end, part, split], 1)
    st = np.nonzero(is_split)[0]
    tile_r = np.repeat(st, qn[st])                                 # one reduction per token of a split tile
    t_in = np.arange(len(tile_r)) - np.repeat(np.cumsum(qn[st]) - qn[st], qn[st])
    red = np.stack([q0[tile_r] + t_in, base[tile_r] + t_in, n_split[tile_r], qn[tile_r]], 1)
    return work.astype(np.int32), red.astype(np.int32).reshape(-1, 4), int(rows_of.sum())


def plan_limits(max_step_tokens: int, tile_tokens: int, target_ctas: int, ctas_per_item: int = 1,
                max_segments: Optional[int] = None) -> Tuple[int, int, int]:
    """Upper bounds (work items, reductions, partial rows) for any step of at most
    ``max_step_tokens`` tokens (in at most ``max_segments`` segments, when given), so that
    buffers and launch grids can be sized once.  Tight, because a captured step launches the
    bound and the idle CTAs cost time (a CTA of the tcgen05 kernel holds an SM's whole shared
    memory even to find that it has nothing to do)."""
    # Unsplit: one item per tile; a segment of n tokens has at most n / tile + 1 tiles, and there
    # is at most one tile per token.  Split: tiles * ctas_per_item is below the target and each
    # tile is cut into max(2, target // (tiles * ctas_per_item)) parts, which is at most
    # 2 * target / ctas_per_item items in all.
    split_items = -(-2 * target_ctas // max(1, ctas_per_item))
    tiles = max_step_tokens
    if max_segments is not None:
        tiles = min(tiles, max_segments + max_step_tokens // max(1, tile_tokens))
    max_work = max(tiles, split_items)
    max_red = max_step_tokens
    max_parts = split_items * tile_tokens
    return max_work, max_red, max_parts


def many_splits(n_tokens: int, ctas_per_item: int, target_ctas: int) -> bool:
    """Whether a step of this many single tokens is cut into eight splits a tile or more (the
    planner's arithmetic): the reduction kernel then shares an entry's splits out over four
    groups of threads."""
    return target_ctas // max(1, n_tokens * ctas_per_item) >= 8
