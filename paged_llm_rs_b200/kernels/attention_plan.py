"""Cutting a step's attention into work items for the kernels.

A segment is the run of consecutive tokens one request brings to a step.  It is
cut into tiles of at most ``tile_tokens`` query tokens; a tile attends over the
keys from the start of its window (or 0) up to its last token.  When a step has
too few tiles to fill the GPU and a tile's key range is long (decoding, or a
short portion late in a long prompt), the range is split and the splits are
combined by the reduce kernel, always in the same order.

Item layout (int32 x 8): seg, first query token (index in the step), query
tokens, position of the first query token, first key, one past the last key,
first partial row or -1 when not split, unused.
Reduction layout (int32 x 4): token index, first partial row, splits, stride
between the token's partial rows.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np

SPLIT_ALIGN = 64   # split boundaries fall on multiples of the kernels' key tiles (32 and 64)
MIN_SPLIT_KEYS = 128
MAX_SPLITS = 128   # the reduce kernel holds the weights of up to 256 splits in shared memory


def plan_attention(segments: Sequence[Tuple[int, int, int]], tile_tokens: int, window: Optional[int],
                   ctas_per_item: int, target_ctas: int) -> Tuple[np.ndarray, np.ndarray, int]:
    """segments: (first token index, token count, position of the first token) per
    segment, in step order.  Returns (work [n, 8], red [m, 4], partial rows used)."""
    seg_ids, q0s, qns, p0s = [], [], [], []
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
        # CTAs), rounded down so that the last wave is not a sliver
        want = max(2, target_ctas // (n_tiles * ctas_per_item))
        splits = np.clip(np.minimum(want, keys // MIN_SPLIT_KEYS), 1, MAX_SPLITS)
    if (splits == 1).all():
        work = np.stack([seg, q0, qn, p0, kv_begin, kv_end, np.full(n_tiles, -1), np.zeros(n_tiles, np.int64)], 1)
        return work.astype(np.int32), np.zeros((0, 4), np.int32), 0

    work_rows: List[Tuple[int, ...]] = []
    red_rows: List[Tuple[int, ...]] = []
    parts = 0
    for i in range(n_tiles):
        s = int(splits[i])
        if s == 1:
            work_rows.append((seg[i], q0[i], qn[i], p0[i], kv_begin[i], kv_end[i], -1, 0))
            continue
        chunk = -(-int(keys[i]) // s)
        chunk = -(-chunk // SPLIT_ALIGN) * SPLIT_ALIGN
        begins = list(range(int(kv_begin[i]), int(kv_end[i]), chunk))
        base = parts
        for k, b in enumerate(begins):
            work_rows.append((seg[i], q0[i], qn[i], p0[i], b, min(b + chunk, int(kv_end[i])), base + k * int(qn[i]), 0))
        for t in range(int(qn[i])):
            red_rows.append((int(q0[i]) + t, base + t, len(begins), int(qn[i])))
        parts += len(begins) * int(qn[i])
    return (np.asarray(work_rows, dtype=np.int32).reshape(-1, 8),
            np.asarray(red_rows, dtype=np.int32).reshape(-1, 4), parts)


def plan_limits(max_step_tokens: int, tile_tokens: int, target_ctas: int, ctas_per_item: int = 1) -> Tuple[int, int, int]:
    """Upper bounds (work items, reductions, partial rows) for any step of at most
    ``max_step_tokens`` tokens, so that buffers and launch grids can be sized once.
    Tight, because a captured step launches the bound and the idle CTAs cost time."""
    # Unsplit: one item per tile, at most one tile per token.  Split: tiles * ctas_per_item
    # is below the target and each tile is cut into max(2, target // (tiles * ctas_per_item))
    # parts, which is at most 2 * target / ctas_per_item items in all.
    split_items = -(-2 * target_ctas // max(1, ctas_per_item))
    max_work = max(max_step_tokens, split_items)
    max_red = max_step_tokens
    max_parts = split_items * tile_tokens
    return max_work, max_red, max_parts
