"""The step function's input: a batch of (request, its next tokens) packed for
the device.

The reference's descriptor is ``Batch`` (crates/pagedllm/src/batch.rs:67-94): a
rectangle, or one row per token so that a portion of a prompt can ride beside
decoded tokens, with per-layer uploads of tables on the kernel path
(crates/pagedllm/src/kernels/paged_attention.rs:114-123).  Here a step is a list
of segments (the consecutive tokens one request brings), each cut anywhere, and
everything the kernels need goes to the device in ONE packed int32 buffer:
token ids, positions, wanted rows, segments, and per cache group the write
slots, the block tables and the attention work items.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager, RequestCache
from ..errors import CacheError, ConfigError
from ..kernels import attention_plan
from ..parts.base import AttentionWork, GroupStep, StepState


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens, and the places among them
    whose logits are wanted (may be empty)."""

    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class GroupPlanConfig:
    """How a cache group's attention is cut into work items (what its mixers wished: Mixer.plan_wish).
    A group whose mixers read no work items has None in its place."""

    tile_tokens: int      # query tokens per attention work item
    ctas_per_item: int    # CTAs the kernel launches per item (kv heads x group parts)
    window: Optional[int]
    heads: int = 1        # partial results of split items are [rows, heads, head_dim]
    head_dim: int = 1


@dataclass
class StepCaps:
    """Fixed capacities of a packed step (for steps replayed as CUDA graphs); None
    where the actual size is used."""

    tokens: int
    wanted: int
    segments: int
    table_width: int
    kinds: int = 1        # what the captured step's attention items may be (1: single tokens only, 3: anything)


class StepPacker:
    """Lays out and fills the packed buffer of a step."""

    def __init__(self, cache: CacheManager, plans: List[Optional[GroupPlanConfig]], target_ctas: int, vocab_size: int,
                 max_positions: int, device):
        self.cache, self.plans, self.target_ctas = cache, plans, target_ctas
        self.vocab_size, self.max_positions, self.device = vocab_size, max_positions, device
        self._scratch: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}

    def scratch(self, gi: int, parts: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Partial-result buffers of group gi for at least ``parts`` rows."""
        nh, hd = self.plans[gi].heads, self.plans[gi].head_dim
        cur = self._scratch.get(gi)
        if cur is None or cur[0].shape[0] < parts:
            rows = max(parts, 1)
            cur = (torch.empty((rows, nh, hd), dtype=torch.float32, device=self.device),
                   torch.empty((rows, nh, 2), dtype=torch.float32, device=self.device))
            self._scratch[gi] = cur
        return cur

    def pack(self, entries: Sequence[StepEntry],
             caps: Optional[StepCaps] = None, work_caps: Optional[List[Optional[Tuple[int, int, int]]]] = None,
             temperature: Optional[Sequence[float]] = None, uniform: Optional[Sequence[float]] = None):
        """Returns (host int32 array, layout dict, sizes) for the entries.  Pages
        must already be reserved for every token.  ``temperature`` / ``uniform``
        (one per wanted row) ride along for the sampling kernel.  With ``caps`` and
        ``work_caps`` (max work items, reductions, partial rows per group) the
        layout depends on them alone, so a captured graph can be fed any step
        that fits."""
        cache = self.cache
        tok_parts: List[np.ndarray] = []      # (arrays a request, joined once: a portion has thousands of tokens)
        pos_parts: List[np.ndarray] = []
        rows: List[int] = []
        segs: List[Tuple[int, int, int, int]] = []
        rcs: List[RequestCache] = []
        T = 0
        for e in entries:
            n = len(e.tokens)
            if n == 0:
                raise ConfigError(f"request {e.request_id!r} brings no tokens to the step")
            rc = cache.get(e.request_id)
            p0 = rc.tokens
            for w in e.want:
                if not 0 <= w < n:
                    raise ConfigError(f"request {e.request_id!r} wants place {w} among {n} tokens")
                rows.append(T + w)
            segs.append((T, n, p0, rc.state_slot))
            rcs.append(rc)
            tok_parts.append(np.asarray(e.tokens, dtype=np.int64))
            pos_parts.append(np.arange(p0, p0 + n, dtype=np.int64))
            T += n
        n_want, n_seg = len(rows), len(segs)
        toks = np.concatenate(tok_parts) if tok_parts else np.zeros(0, np.int64)
        pos = np.concatenate(pos_parts) if pos_parts else np.zeros(0, np.int64)
        if T and (toks.min() < 0 or toks.max() >= self.vocab_size):
            raise ConfigError(f"a token id lies outside the vocabulary of {self.vocab_size}")
        if T and int(pos.max()) >= self.max_positions:
            raise ConfigError(f"position {int(pos.max())} reaches past max_position_embeddings {self.max_positions}")

        ps = cache.page_size
        Tc = caps.tokens if caps else T
        nc = caps.wanted if caps else n_want
        sc = caps.segments if caps else n_seg
        if T > Tc or n_want > nc or n_seg > sc:
            raise ConfigError("the step does not fit the capacities it was given")

        group_parts = []
        planned = {}
        for gi, g in enumerate(cache.groups):
            slots = np.full(Tc, -1, dtype=np.int32)
            width = max((len(rc.tables[gi].blocks) for rc in rcs), default=1)
            W = caps.table_width if caps else max(width, 1)
            if width > W:
                raise ConfigError("a block table is wider than the step's capacity")
            tables = np.full((sc, W), -1, dtype=np.int32)
            for si, (rc, (t0, n, p0, _)) in enumerate(zip(rcs, segs)):
                tb = rc.tables[gi]
                if p0 + n > tb.capacity():
                    raise CacheError(f"request {rc.request_id!r}: no pages reserved for positions up to {p0 + n - 1}")
                blocks = tb.array()          # cached; rebuilt only when a page came or went
                tables[si, :len(blocks)] = blocks
                if n == 1:
                    page = int(blocks[p0 // ps])
                    if page < 0:
                        raise CacheError(f"request {rc.request_id!r} writes into a page it gave back")
                    slots[t0] = page * ps + p0 % ps
                else:
                    pp = np.arange(p0, p0 + n)
                    page = blocks[pp // ps].astype(np.int64)
                    if (page < 0).any():
                        raise CacheError(f"request {rc.request_id!r} writes into a page it gave back")
                    slots[t0:t0 + n] = page * ps + pp % ps
            plan = self.plans[gi]
            if plan is None:        # the group's mixers read tables and slots only
                group_parts.append((slots, tables, None, None, 0, 0, 0, W))
                continue
            # groups that cut their work alike (same tile, window, CTAs an item) share one plan
            key = (plan.tile_tokens, plan.window, plan.ctas_per_item)
            if key not in planned:
                planned[key] = attention_plan.plan_attention(
                    [(t0, n, p0) for (t0, n, p0, _) in segs], plan.tile_tokens, plan.window, plan.ctas_per_item,
                    self.target_ctas)
            work, red, parts = planned[key]
            mw, mr, mp = (work_caps[gi] if work_caps else (len(work), len(red), parts))
            if len(work) > mw or len(red) > mr or parts > mp:
                raise ConfigError("the step's attention work does not fit the capacities it was given")
            group_parts.append((slots, tables, work, red, mp, mw, mr, W))

        # layout: offsets in int32 units
        off = 0
        layout = {}

        def take(name, count):
            nonlocal off
            layout[name] = (off, count)
            off += count

        take("tokens", Tc); take("positions", Tc); take("logit_rows", max(nc, 1)); take("segments", max(sc, 1) * 4)
        take("temperature", max(nc, 1)); take("uniform", max(nc, 1))
        for gi, (slots, tables, work, red, parts, mw, mr, W) in enumerate(group_parts):
            take(f"g{gi}.slots", Tc); take(f"g{gi}.tables", sc * W)
            if work is not None:
                take(f"g{gi}.n_work", 1); take(f"g{gi}.n_red", 1)
                take(f"g{gi}.work", max(mw, 1) * 8); take(f"g{gi}.red", max(mr, 1) * 4)
        host = np.zeros(off, dtype=np.int32)

        def put(name, arr):
            o, _ = layout[name]
            a = np.asarray(arr, dtype=np.int32).reshape(-1)
            host[o:o + len(a)] = a

        put("tokens", toks); put("positions", pos); put("logit_rows", rows)
        if temperature is not None:
            put("temperature", np.asarray(temperature, dtype=np.float32).view(np.int32))
            put("uniform", np.asarray(uniform, dtype=np.float32).view(np.int32))
        put("segments", np.asarray(segs, dtype=np.int32).reshape(-1) if segs else [])
        for gi, (slots, tables, work, red, parts, mw, mr, W) in enumerate(group_parts):
            put(f"g{gi}.slots", slots); put(f"g{gi}.tables", tables)
            if work is not None:
                put(f"g{gi}.n_work", [len(work)]); put(f"g{gi}.n_red", [len(red)])
                put(f"g{gi}.work", work); put(f"g{gi}.red", red)
        # What the work items are: bit 0 items of one query token (decoded tokens, but also the
        # last tile of a portion of 33 tokens), bit 1 items of several.  Read off the items, not
        # the segments.  A step packed to capacities is a captured decode step: single tokens only.
        kinds = 0
        for p in group_parts:
            if p[2] is None:
                continue
            counts = p[2][:, 2] if len(p[2]) else np.zeros(0, np.int32)
            kinds |= (1 if (counts == 1).any() else 0) | (2 if (counts > 1).any() else 0)
        if caps is not None:
            kinds = caps.kinds      # a captured step launches the same kernels whatever it holds
        singles = bool(segs) and all(n == 1 for (_, n, _, _) in segs)
        sizes = dict(tokens=T, wanted=n_want, segments=n_seg, tokens_cap=Tc, wanted_cap=nc, segments_cap=sc, kinds=kinds,
                     groups=[dict(planned=p[2] is not None, parts=p[4], max_work=p[5], max_red=p[6], table_width=p[7])
                             for p in group_parts],
                     host_segments=segs,
                     # (a captured step of single tokens is cut for its capacity's worth of requests at the least)
                     plan_tokens=(caps.tokens if caps is not None and caps.kinds == 1 else n_seg) if (singles or caps) else 0)
        return host, layout, sizes

    def to_state(self, dev: torch.Tensor, layout, sizes, full: bool = False) -> StepState:
        """Views of the packed device buffer as the parts see it.  ``full``: take
        the capacities rather than the live sizes (graph capture)."""

        def view(name, count=None):
            o, c = layout[name]
            return dev[o:o + (c if count is None else count)]

        T = sizes["tokens_cap"] if full else sizes["tokens"]
        nw = sizes["wanted_cap"] if full else sizes["wanted"]
        groups = []
        for gi, gs in enumerate(sizes["groups"]):
            plan = None
            if gs["planned"]:
                part_o, part_ml = self.scratch(gi, gs["parts"])
                many = sizes["kinds"] == 1 and attention_plan.many_splits(max(1, sizes["plan_tokens"]), self.plans[gi].ctas_per_item,
                                                                           self.target_ctas)
                plan = AttentionWork(work=view(f"g{gi}.work").view(-1, 8), n_work=view(f"g{gi}.n_work"), max_work=gs["max_work"],
                                     red=view(f"g{gi}.red").view(-1, 4), n_red=view(f"g{gi}.n_red"), max_red=gs["max_red"],
                                     part_o=part_o, part_ml=part_ml, kinds=sizes["kinds"], many_splits=many)
            groups.append(GroupStep(block_tables=view(f"g{gi}.tables").view(sizes["segments_cap"], gs["table_width"]),
                                    slots=view(f"g{gi}.slots", T), plan=plan))
        state = StepState(n_tokens=T, tokens=view("tokens", T), positions=view("positions", T), groups=groups,
                          logit_rows=view("logit_rows", nw), n_wanted=nw,
                          segments=view("segments").view(-1, 4), host_segments=list(sizes["host_segments"]))
        state.temperature = view("temperature", max(nw, 1)).view(torch.float32)
        state.uniform = view("uniform", max(nw, 1)).view(torch.float32)
        return state


class _GroupPack(ctypes.Structure):
    """csrc/step_pack.cu: PllmGroupPack."""
    _fields_ = [("tables", ctypes.POINTER(ctypes.c_void_p)), ("table_len", ctypes.POINTER(ctypes.c_int)),
                ("window", ctypes.c_int), ("ctas_per_item", ctypes.c_int),
                ("max_work", ctypes.c_int), ("max_red", ctypes.c_int), ("max_parts", ctypes.c_int),
                ("plans", ctypes.c_int),
                ("off_slots", ctypes.c_int), ("off_tables", ctypes.c_int), ("off_n_work", ctypes.c_int),
                ("off_n_red", ctypes.c_int), ("off_work", ctypes.c_int), ("off_red", ctypes.c_int)]


class NativeDecodePacker:
    """The packer of the captured decode step: every request brings one token and
    wants its logits.  Same buffer as ``StepPacker.pack`` with capacities makes
    (the tests compare them word for word), written by native code
    (csrc/step_pack.cu) straight into the pinned buffer the step is copied from."""

    _ERRORS = {
        -10: (ConfigError, "a token id lies outside the vocabulary of {vocab}"),
        -11: (ConfigError, "request {rid!r}: its position reaches past max_position_embeddings {maxpos}"),
        -12: (CacheError, "request {rid!r}: no pages reserved for its next position"),
        -13: (CacheError, "request {rid!r} writes into a page it gave back"),
        -14: (ConfigError, "the step's attention work does not fit the capacities it was given"),
        -15: (ConfigError, "a block table is wider than the step's capacity"),
        -16: (ConfigError, "the step does not fit the capacities it was given"),
    }

    def __init__(self, packer: StepPacker, caps: StepCaps, work_caps: List[Tuple[int, int, int]], layout, out: np.ndarray):
        from ..kernels import ops
        self.packer, self.caps, self.out = packer, caps, out
        self.fn = ops.lib().pllm_pack_decode_step
        B = caps.tokens
        self.tokens = (ctypes.c_int * B)()
        self.positions = (ctypes.c_int * B)()
        self.state_slots = (ctypes.c_int * B)()
        self.temperature = (ctypes.c_float * B)()
        self.uniform = (ctypes.c_float * B)()
        self.err = ctypes.c_int(-1)
        n_groups = len(packer.cache.groups)
        self.groups = (_GroupPack * max(n_groups, 1))()
        self.ptrs, self.lens = [], []
        for gi in range(n_groups):
            ptrs, lens = (ctypes.c_void_p * B)(), (ctypes.c_int * B)()
            self.ptrs.append(ptrs); self.lens.append(lens)
            g, plan = self.groups[gi], packer.plans[gi]
            g.tables = ctypes.cast(ptrs, ctypes.POINTER(ctypes.c_void_p))
            g.table_len = ctypes.cast(lens, ctypes.POINTER(ctypes.c_int))
            g.plans = 0 if plan is None else 1
            if plan is not None:
                g.window, g.ctas_per_item = int(plan.window or 0), plan.ctas_per_item
                g.max_work, g.max_red, g.max_parts = work_caps[gi]
            for name in ("slots", "tables") + (("n_work", "n_red", "work", "red") if plan is not None else ()):
                setattr(g, f"off_{name}", layout[f"g{gi}.{name}"][0])
        self.n_groups = n_groups
        self.fixed = (caps.tokens, caps.wanted, caps.segments, caps.table_width, packer.cache.page_size, packer.vocab_size,
                      packer.max_positions, packer.target_ctas, attention_plan.MIN_SPLIT_KEYS,
                      layout["tokens"][0], layout["positions"][0], layout["logit_rows"][0], layout["segments"][0],
                      layout["temperature"][0], layout["uniform"][0], n_groups)
        self.out_ptr = out.ctypes.data

    def pack(self, entries: Sequence[StepEntry], temperature, uniform, ahead: int = 0,
             out: Optional[np.ndarray] = None) -> None:
        """``ahead``: the step is packed while the one before it still runs and is not yet committed: every
        request stands ``ahead`` tokens further than its committed count says (its pages are reserved).
        ``out``: a buffer of the pinned one's size to fill instead of it."""
        cache = self.packer.cache
        n = len(entries)
        if n > self.caps.tokens:
            raise ConfigError("the step does not fit the capacities it was given")
        if out is not None and (out.dtype != np.int32 or len(out) != len(self.out) or not out.flags.c_contiguous):
            raise ConfigError("the buffer to pack into does not match the step's")
        tables = []
        for i, e in enumerate(entries):
            rc = cache.get(e.request_id)
            self.tokens[i] = int(e.tokens[0])
            self.positions[i] = rc.tokens + ahead
            self.state_slots[i] = rc.state_slot
            tables.append(rc.tables)
        for gi in range(self.n_groups):
            ptrs, lens = self.ptrs[gi], self.lens[gi]
            for i, tbs in enumerate(tables):
                ptrs[i], lens[i] = tbs[gi].pointer()
        have = temperature is not None
        if have:
            self.temperature[:n] = [float(t) for t in temperature]
            self.uniform[:n] = [float(u) for u in uniform]
        code = self.fn(self.out_ptr if out is None else out.ctypes.data, len(self.out), n, self.tokens, self.positions,
                       self.state_slots,
                       self.temperature if have else None, self.uniform if have else None, *self.fixed,
                       self.groups, ctypes.byref(self.err))
        if code != 0:
            kind, msg = self._ERRORS.get(code, (ConfigError, f"the native step packer refused the step (code {code})"))
            i = self.err.value
            raise kind(msg.format(vocab=self.packer.vocab_size, maxpos=self.packer.max_positions,
                                  rid=entries[i].request_id if 0 <= i < n else None))
