"""The one step function: a batch of (request, its next tokens) -> logits at the
wanted places.

A step takes portions of prompts beside single decoded tokens, cut anywhere.
It runs only the tokens it is given, as one flat batch, from the cache that
earlier steps left (the reference's ``forward_paged`` over a packed batch,
``src/llmserve/engine.py:269-315`` and ``src/llmserve/model.py:270-309``).
Rows of one request are consecutive and in position order; every row has its
own position, and attends to the keys of its own request up to that position.
All rows write their key and value before any row attends (``model.py:114``).

The step's metadata is packed into ONE pinned int32 buffer and copied to the
device with one transfer; ``StepContext`` holds views into the device copy.

Steps in which every request brings exactly one token (decoding) are replayed
from CUDA graphs: the model's launches are captured once per (batch bucket,
block-table width) with the metadata at fixed addresses, rows beyond the batch
being padding (segment -1, cache slot -1) that every kernel skips.  Only models
whose mixers all say ``graph_safe`` are captured; others run launch by launch.
"""
from __future__ import annotations

import gc
import os
from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.manager import CacheFullError, CacheManager, LayerCache


@dataclass
class StepEntry:
    """One request's share of a step: its next ``tokens`` and ``want``, the indices
    among these tokens whose logits are asked for (may be empty)."""

    request_id: str
    tokens: list[int]
    want: list[int] = field(default_factory=list)


@dataclass
class Segment:
    request_id: str
    state_slot: int
    first_position: int
    count: int
    row_start: int


class StepContext:
    """Device-side description of a step (all int32) plus the host-side list of segments."""

    def __init__(self) -> None:
        self.num_tokens = 0
        self.num_segments = 0
        self.num_wanted = 0
        self.segments: list[Segment] = []
        self.token_ids: torch.Tensor = None          # [T]
        self.positions: torch.Tensor = None          # [T]
        self.segment_of_token: torch.Tensor = None   # [T], -1 for padding rows
        self.segment_start: torch.Tensor = None      # [S + 1] first row of each segment
        self.segment_first_position: torch.Tensor = None  # [S]
        self.segment_context: torch.Tensor = None    # [S] keys of the request after this step
        self.segment_state_slot: torch.Tensor = None  # [S]
        self.want_rows: torch.Tensor = None          # [W]
        self.max_segment_tokens = 0
        self.max_context = 0                         # None: not known on the host (a replayed graph)
        self.decode_only = False                     # every segment brings exactly one token
        self.long_context = False                    # some request holds more than LONG_CONTEXT keys (known on the host always:
                                                     # graphs of decode steps are captured for either case)


def _round4(n: int) -> int:
    return (n + 3) & ~3


LONG_CONTEXT = 8192   # keys of a request beyond which a decode step counts as one over long contexts


class _Layout:
    """Where each array of a step lies in the packed int32 buffer, for given capacities."""

    def __init__(self, tokens: int, segments: int, wanted: int, table_width: int, groups: int) -> None:
        self.tokens, self.segments, self.wanted, self.table_width = tokens, segments, wanted, table_width
        cursor = 0

        def take(n: int) -> tuple[int, int]:
            nonlocal cursor
            view = (cursor, cursor + n)
            cursor += _round4(n)
            return view

        self.tok, self.pos, self.seg = take(tokens), take(tokens), take(tokens)
        self.start, self.first, self.ctx, self.slot = take(segments + 1), take(segments), take(segments), take(segments)
        self.want = take(wanted)
        self.maps = [take(tokens) for _ in range(groups)]
        self.tables = [take(segments * table_width) for _ in range(groups)]
        self.size = cursor


class _Graph:
    """A captured decode step: fixed buffers, the graph and its output."""

    def __init__(self, layout: _Layout, device, pinned: bool) -> None:
        self.layout = layout
        self.host = torch.empty(layout.size, dtype=torch.int32, pin_memory=pinned)
        self.host_np = self.host.numpy()
        self.device = torch.empty(layout.size, dtype=torch.int32, device=device)
        self.graph: torch.cuda.CUDAGraph | None = None
        self.logits: torch.Tensor | None = None
        self.launches = 0        # launches of the engine's own kernels inside the graph


class _Ahead:
    """A decode step packed before its tokens were known: the graph it goes to, and what it assumed."""

    def __init__(self, key, request_ids: list[str], firsts: list[int]) -> None:
        self.key, self.request_ids, self.firsts = key, request_ids, firsts


class StepRunner:
    """Packs a step, runs the model on it and keeps the cache manager in step."""

    GRAPH_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)
    # size classes of steps with prompt portions: tokens (steps of a quarter to a half, so that at most a third
    # of a graph's rows is padding) and requests (few classes: every class is a capture)
    PORTION_BUCKETS = (16, 32, 48, 64, 96, 128, 160, 192, 256, 320, 384, 512, 640, 768, 1024, 1280, 1536, 2048,
                       2560, 3072, 4096, 5120, 6144, 8192)
    PORTION_REQUEST_BUCKETS = (1, 8, 32, 128, 256)

    def __init__(self, model, cache: CacheManager, max_tokens_per_step: int, max_segments: int,
                 use_graphs: bool = True) -> None:
        self.model = model
        self.cache = cache
        self.device = model.device
        self.max_tokens = int(max_tokens_per_step)
        self.max_segments = int(max_segments)
        self._groups = len(cache.groups)
        full = _Layout(self.max_tokens, self.max_segments, self.max_tokens,
                       _round4(cache.max_pages_per_request), self._groups)
        self._capacity = full.size
        pinned = self.device.type == "cuda"
        self._host = torch.empty(self._capacity, dtype=torch.int32, pin_memory=pinned)
        self._host_np = self._host.numpy()
        self._device = torch.empty(self._capacity, dtype=torch.int32, device=self.device)
        self._layer_views = [cache.layer_view(position) for position in range(len(model.spec.order))]
        self._copied = torch.cuda.Event() if pinned else None
        self._copy_pending = False
        self.use_graphs = bool(use_graphs) and pinned and getattr(model, "graph_safe", False)
        self._graphs: dict[tuple[int, int, bool], _Graph] = {}   # (batch bucket, block-table width, long contexts)
        self._graph_pool = None          # one memory pool for all graphs: only one of them runs at a time
        self._capture_stream = None
        self._arange = np.arange(max(self.GRAPH_BUCKETS), dtype=np.int32)
        self.graph_portions = os.environ.get("LSE_PORTION_GRAPHS", "1") != "0"
        self._portion_classes_seen: dict = {}
        self._portion_graphs: dict = {}
        self.portion_graph_replays = 0
        self.steps_run = 0
        self.graph_replays = 0
        self.ahead_steps = 0             # decode steps whose packing ran beside the step before
        self.flying_steps = 0            # of these, steps queued before the tokens of the step before reached the host
        self.graph_kernel_launches = 0
        self.last_h2d_bytes = 0

    # -- the step ------------------------------------------------------------------
    def run(self, entries: list[StepEntry]) -> torch.Tensor:
        """Run one step.  Returns float32 logits [total wanted, vocab] on the device, in the
        order of the entries and of each entry's ``want``.  The tensor may be a view of a
        buffer that the next step overwrites: use or copy it before the next ``run``."""
        self._validate(entries)
        logits = None
        if self.use_graphs and all(len(entry.tokens) == 1 for entry in entries):
            logits = self._run_graph(entries)
        elif self.use_graphs and self.graph_portions:
            logits = self._run_portion_graph(entries)
        if logits is None:
            step, caches = self.prepare(entries, validated=True)
            logits = self.model.forward(step, caches)
        self.finish(entries)
        return logits

    def _validate(self, entries: list[StepEntry]) -> None:
        if not entries:
            raise ValueError("a step needs at least one entry")
        if len(entries) > self.max_segments:
            raise ValueError(f"{len(entries)} requests in a step, at most {self.max_segments}")
        total = sum(len(entry.tokens) for entry in entries)
        if total > self.max_tokens:
            raise ValueError(f"{total} tokens in a step, at most {self.max_tokens}")
        vocab = self.model.vocab_size
        seen = set()
        for entry in entries:
            if entry.request_id in seen:
                raise ValueError(f"request {entry.request_id!r} appears twice in a step")
            seen.add(entry.request_id)
            if not entry.tokens:
                raise ValueError(f"request {entry.request_id!r} brings no tokens")
            if min(entry.tokens) < 0 or max(entry.tokens) >= vocab:
                raise ValueError(f"request {entry.request_id!r}: token id outside [0, {vocab})")
            for index in entry.want:
                if not 0 <= index < len(entry.tokens):
                    raise ValueError(f"request {entry.request_id!r}: wanted place {index} outside its tokens")
        if not self.cache.fits([(entry.request_id, len(entry.tokens)) for entry in entries]):
            raise CacheFullError("paged KV cache has no free blocks for this step")

    def _pages_after(self, entries: list[StepEntry]) -> int:
        cache = self.cache
        return max(1, max((cache.requests[e.request_id].length + len(e.tokens) + cache.page_size - 1)
                          // cache.page_size for e in entries))

    def _pack(self, entries: list[StepEntry], host: np.ndarray, lay: _Layout, wanted_all_rows: bool) -> StepContext:
        """Reserve cache room for every entry and write the step's arrays into ``host``.
        Capacities of ``lay`` beyond the entries are filled as padding."""
        cache = self.cache
        step = StepContext()
        host[lay.tok[0]:lay.tok[1]] = 0
        host[lay.pos[0]:lay.pos[1]] = 0
        host[lay.seg[0]:lay.seg[1]] = -1
        host[lay.first[0]:lay.first[1]] = 0
        host[lay.ctx[0]:lay.ctx[1]] = 0
        host[lay.slot[0]:lay.slot[1]] = 0
        host[lay.want[0]:lay.want[1]] = 0      # wanted places beyond the entries' point at row 0
        for lo, hi in lay.maps:
            host[lo:hi] = -1
        for lo, hi in lay.tables:
            host[lo:hi] = -1
        row = 0
        want_cursor = lay.want[0]
        for index, entry in enumerate(entries):
            count = len(entry.tokens)
            first = cache.reserve(entry.request_id, count)
            request = cache.requests[entry.request_id]
            step.segments.append(Segment(entry.request_id, request.state_slot, first, count, row))
            host[lay.tok[0] + row: lay.tok[0] + row + count] = entry.tokens
            host[lay.pos[0] + row: lay.pos[0] + row + count] = np.arange(first, first + count, dtype=np.int32)
            host[lay.seg[0] + row: lay.seg[0] + row + count] = index
            host[lay.start[0] + index] = row
            host[lay.first[0] + index] = first
            host[lay.ctx[0] + index] = first + count
            host[lay.slot[0] + index] = request.state_slot
            if not wanted_all_rows:
                for offset in entry.want:
                    host[want_cursor] = row + offset
                    want_cursor += 1
            for g in range(self._groups):
                host[lay.maps[g][0] + row: lay.maps[g][0] + row + count] = cache.slot_mapping(g, entry.request_id, first, count)
                table = cache.block_table_array(g, entry.request_id)
                base = lay.tables[g][0] + index * lay.table_width
                host[base: base + table.shape[0]] = table
            step.max_segment_tokens = max(step.max_segment_tokens, count)
            step.max_context = max(step.max_context, first + count)
            row += count
        host[lay.start[0] + len(entries): lay.start[1]] = row      # padding segments are empty
        step.long_context = step.max_context > LONG_CONTEXT
        if wanted_all_rows:
            host[lay.want[0]:lay.want[1]] = np.arange(lay.wanted, dtype=np.int32)
        step.decode_only = step.max_segment_tokens == 1
        return step

    def _pack_decode(self, entries: list[StepEntry], host: np.ndarray, lay: _Layout) -> StepContext:
        """``_pack`` for steps in which every entry brings one token and every row is wanted:
        the arrays are built as lists and written with one assignment each."""
        cache = self.cache
        page_size = cache.page_size
        count = len(entries)
        step = StepContext()
        tokens, firsts, slots_of = [], [], []
        for lo, hi in lay.tables:
            host[lo:hi] = -1
        group_slots = [[] for _ in range(self._groups)]
        for index, entry in enumerate(entries):
            first = cache.reserve(entry.request_id, 1)
            request = cache.requests[entry.request_id]
            tokens.append(entry.tokens[0])
            firsts.append(first)
            slots_of.append(request.state_slot)
            step.segments.append(Segment(entry.request_id, request.state_slot, first, 1, index))
            for g in range(self._groups):
                table = request.tables[g]
                group_slots[g].append(table[first // page_size] * page_size + first % page_size)
                mirror = request.tables_np[g]
                base = lay.tables[g][0] + index * lay.table_width
                host[base: base + len(table)] = mirror[:len(table)]
        pad = lay.tokens - count
        rows = list(range(count))
        host[lay.tok[0]:lay.tok[1]] = tokens + [0] * pad
        host[lay.pos[0]:lay.pos[1]] = firsts + [0] * pad
        host[lay.seg[0]:lay.seg[1]] = rows + [-1] * pad
        host[lay.start[0]:lay.start[1]] = rows + [count] * (lay.segments + 1 - count)
        host[lay.first[0]:lay.first[1]] = firsts + [0] * pad
        host[lay.ctx[0]:lay.ctx[1]] = [first + 1 for first in firsts] + [0] * pad
        host[lay.slot[0]:lay.slot[1]] = slots_of + [0] * pad
        host[lay.want[0]:lay.want[1]] = self._arange[:lay.wanted]
        for g in range(self._groups):
            host[lay.maps[g][0]:lay.maps[g][1]] = group_slots[g] + [-1] * pad
        step.max_segment_tokens = 1
        step.max_context = max(firsts) + 1
        step.long_context = step.max_context > LONG_CONTEXT
        step.decode_only = True
        return step

    def _views(self, step: StepContext, dev: torch.Tensor, lay: _Layout):
        step.num_tokens, step.num_segments, step.num_wanted = lay.tokens, lay.segments, lay.wanted
        step.token_ids = dev[lay.tok[0]:lay.tok[1]]
        step.positions = dev[lay.pos[0]:lay.pos[1]]
        step.segment_of_token = dev[lay.seg[0]:lay.seg[1]]
        step.segment_start = dev[lay.start[0]:lay.start[1]]
        step.segment_first_position = dev[lay.first[0]:lay.first[1]]
        step.segment_context = dev[lay.ctx[0]:lay.ctx[1]]
        step.segment_state_slot = dev[lay.slot[0]:lay.slot[1]]
        step.want_rows = dev[lay.want[0]:lay.want[1]]
        group_maps = [dev[lo:hi] for lo, hi in lay.maps]
        group_tables = [dev[lo:hi].view(lay.segments, lay.table_width) for lo, hi in lay.tables]
        caches = []
        for view in self._layer_views:
            layer_cache = LayerCache(keys=view.keys, values=view.values, state=view.state, group=view.group)
            if view.group >= 0:
                layer_cache.slot_mapping = group_maps[view.group]
                layer_cache.block_tables = group_tables[view.group]
            caches.append(layer_cache)
        return step, caches

    def prepare(self, entries: list[StepEntry], validated: bool = False):
        """Reserve, pack and upload a step; returns ``(StepContext, [LayerCache per layer run])``."""
        if not validated:
            self._validate(entries)
        if self._copy_pending:   # the pinned buffer is reused: the last copy must have left it
            self._copied.synchronize()
            self._copy_pending = False
        total = sum(len(entry.tokens) for entry in entries)
        wanted = sum(len(entry.want) for entry in entries)
        lay = _Layout(total, len(entries), wanted, _round4(self._pages_after(entries)), self._groups)
        if lay.size > self._capacity:
            raise ValueError("step metadata exceeds its buffer")
        step = self._pack(entries, self._host_np, lay, wanted_all_rows=False)
        self._device[:lay.size].copy_(self._host[:lay.size], non_blocking=True)
        self.last_h2d_bytes = lay.size * 4
        if self._copied is not None:
            self._copied.record()
            self._copy_pending = True
        return self._views(step, self._device, lay)

    # -- decode steps from CUDA graphs ---------------------------------------------
    def _run_graph(self, entries: list[StepEntry]) -> torch.Tensor:
        count = len(entries)
        bucket = next((b for b in self.GRAPH_BUCKETS if b >= count), None)
        if bucket is None:
            step, caches = self.prepare(entries, validated=True)
            return self.model.forward(step, caches)
        pages = self._pages_after(entries)
        key = (bucket, self._graph_width(pages), pages * self.cache.page_size > LONG_CONTEXT)
        slot = self._graphs.get(key)
        if slot is None:
            slot = _Graph(_Layout(bucket, bucket, bucket, key[1], self._groups), self.device, True)
            self._graphs[key] = slot
        if self._copy_pending:
            self._copied.synchronize()
            self._copy_pending = False
        step = self._pack_decode(entries, slot.host_np, slot.layout)
        step.max_context = None
        step.long_context = key[2]   # what the graph was, or is now, captured for
        slot.device.copy_(slot.host, non_blocking=True)
        self.last_h2d_bytes = slot.layout.size * 4
        self._copied.record()
        self._copy_pending = True
        if slot.graph is None:
            self._capture(slot, step)
        slot.graph.replay()
        self.graph_replays += 1
        self.graph_kernel_launches += slot.launches
        rows = [index for index, entry in enumerate(entries) for _ in entry.want]
        if rows == list(range(count)):
            return slot.logits[:count]
        if not rows:
            return slot.logits[:0]
        return slot.logits[torch.tensor(rows, device=self.device)]

    # -- steps with prompt portions from CUDA graphs --------------------------------------
    def _run_portion_graph(self, entries: list[StepEntry]) -> torch.Tensor | None:
        """A step with prompt portions (alone or beside decoding requests) replayed from a graph that was
        captured for its size class: tokens, requests and wanted places rounded up to the class, the
        rest padding (rows of segment -1 that every kernel skips, empty segments, wanted places that
        point at row 0).  A class is captured the second time a step falls into it; until then, and for
        steps beyond the largest class, None: the caller launches kernel by kernel.  Launching some 250
        kernels from the host takes longer than a small step takes on the device; a replay does not."""
        total = sum(len(entry.tokens) for entry in entries)
        wanted = sum(len(entry.want) for entry in entries)
        tokens = next((b for b in self.PORTION_BUCKETS if b >= total), None)
        segments = next((b for b in self.PORTION_REQUEST_BUCKETS if b >= len(entries)), None)
        if tokens is None or segments is None:
            return None
        segments = min(segments, self.max_segments, tokens)
        places = 0 if wanted == 0 else (segments if wanted <= segments else tokens)   # none, at most one a request, or any
        if wanted > places:
            return None
        # which kernels the parts launch may depend on how the rows are cut into portions: such steps get graphs of their own
        signature = self.model.launch_signature([len(entry.tokens) for entry in entries]) if hasattr(self.model, "launch_signature") else ()
        key = ("portions", tokens, segments, places, self._graph_width(self._pages_after(entries)), signature)
        slot = self._portion_graphs.get(key)
        if slot is None:
            seen = self._portion_classes_seen.get(key, 0) + 1
            self._portion_classes_seen[key] = seen
            if seen < 2:
                return None
            slot = _Graph(_Layout(tokens, segments, places, key[4], self._groups), self.device, True)
            self._portion_graphs[key] = slot
        if self._copy_pending:
            self._copied.synchronize()
            self._copy_pending = False
        step = self._pack(entries, slot.host_np, slot.layout, wanted_all_rows=False)
        step.max_context = None
        slot.device.copy_(slot.host, non_blocking=True)
        self.last_h2d_bytes = slot.layout.size * 4
        self._copied.record()
        self._copy_pending = True
        if slot.graph is None:
            self._capture(slot, step, first_use=False)   # the class ran launch by launch at its first sighting
        slot.graph.replay()
        self.graph_replays += 1
        self.portion_graph_replays += 1
        self.graph_kernel_launches += slot.launches
        return slot.logits[:wanted]

    # -- a decode step packed before its tokens are known ----------------------------
    def prepare_ahead(self, request_ids: list[str]) -> "_Ahead | None":
        """Pack, while the device still works on the step before, the decode step in which each of
        these requests will bring one token that is not known yet: positions, cache slots and block
        tables follow from the cache as it stands.  A request whose token opens a page takes that
        page now (it keeps it whatever happens next); no token is counted in, so the result may simply
        be dropped.  None when such a step cannot be packed ahead: no captured graph for it yet, or
        no free page."""
        count = len(request_ids)
        if not self.use_graphs or count == 0 or count > self.max_segments:
            return None
        bucket = next((b for b in self.GRAPH_BUCKETS if b >= count), None)
        if bucket is None:
            return None
        cache = self.cache
        page_size = cache.page_size
        firsts = []
        for rid in request_ids:
            request = cache.requests.get(rid)
            if request is None:
                return None
            first = request.length
            if any(first // page_size >= len(table) for table in request.tables) and not cache.grow(rid, 1):
                return None          # the token opens a page and none is free: the ordinary path decides
            firsts.append(first)
        pages = max(1, max(first // page_size + 1 for first in firsts))
        key = (bucket, self._graph_width(pages), pages * page_size > LONG_CONTEXT)
        slot = self._graphs.get(key)
        if slot is None or slot.graph is None:
            return None
        if self._copy_pending:
            self._copied.synchronize()
            self._copy_pending = False
        host, lay = slot.host_np, slot.layout
        for lo, hi in lay.tables:
            host[lo:hi] = -1
        slots_of = []
        group_slots = [[] for _ in range(self._groups)]
        for index, (rid, first) in enumerate(zip(request_ids, firsts)):
            request = cache.requests[rid]
            slots_of.append(request.state_slot)
            for g in range(self._groups):
                table = request.tables[g]
                group_slots[g].append(table[first // page_size] * page_size + first % page_size)
                base = lay.tables[g][0] + index * lay.table_width
                host[base: base + len(table)] = request.tables_np[g][:len(table)]
        pad = lay.tokens - count
        rows = list(range(count))
        host[lay.pos[0]:lay.pos[1]] = firsts + [0] * pad
        host[lay.seg[0]:lay.seg[1]] = rows + [-1] * pad
        host[lay.start[0]:lay.start[1]] = rows + [count] * (lay.segments + 1 - count)
        host[lay.first[0]:lay.first[1]] = firsts + [0] * pad
        host[lay.ctx[0]:lay.ctx[1]] = [first + 1 for first in firsts] + [0] * pad
        host[lay.slot[0]:lay.slot[1]] = slots_of + [0] * pad
        host[lay.want[0]:lay.want[1]] = self._arange[:lay.wanted]
        for g in range(self._groups):
            host[lay.maps[g][0]:lay.maps[g][1]] = group_slots[g] + [-1] * pad
        return _Ahead(key, list(request_ids), firsts)

    def run_ahead(self, ahead: "_Ahead", entries: list[StepEntry]) -> torch.Tensor | None:
        """Run the step that :meth:`prepare_ahead` packed, now that the tokens are known.  None
        (and nothing done) when the entries are not the ones it was packed for."""
        cache = self.cache
        if [entry.request_id for entry in entries] != ahead.request_ids:
            return None
        vocab = self.model.vocab_size
        for entry, first in zip(entries, ahead.firsts):
            request = cache.requests.get(entry.request_id)
            if (request is None or request.length != first or len(entry.tokens) != 1 or entry.want != [0]
                    or not 0 <= entry.tokens[0] < vocab):
                return None
        slot = self._graphs[ahead.key]
        for entry, first in zip(entries, ahead.firsts):
            if cache.reserve(entry.request_id, 1) != first:
                raise RuntimeError("the cache moved under a step that was packed ahead")
        lay = slot.layout
        count = len(entries)
        slot.host_np[lay.tok[0]:lay.tok[1]] = [entry.tokens[0] for entry in entries] + [0] * (lay.tokens - count)
        slot.device.copy_(slot.host, non_blocking=True)
        self.last_h2d_bytes = lay.size * 4
        self._copied.record()
        self._copy_pending = True
        slot.graph.replay()
        self.graph_replays += 1
        self.ahead_steps += 1
        self.graph_kernel_launches += slot.launches
        self.finish(entries)
        return slot.logits[:count]

    def launch_ahead(self, ahead: "_Ahead", device_tokens: torch.Tensor) -> torch.Tensor | None:
        """Queue the step that :meth:`prepare_ahead` packed behind the work already on the stream, with
        its token ids taken on the device (int32, one per request: the tokens that the step before is
        still sampling).  The host does not wait for them.  None (and nothing done) when the cache no
        longer is what the step was packed for."""
        cache = self.cache
        count = len(ahead.request_ids)
        if device_tokens.dtype != torch.int32 or device_tokens.shape[0] != count:
            return None
        for rid, first in zip(ahead.request_ids, ahead.firsts):
            request = cache.requests.get(rid)
            if request is None or request.length != first:
                return None
        slot = self._graphs[ahead.key]
        for rid, first in zip(ahead.request_ids, ahead.firsts):
            if cache.reserve(rid, 1) != first:
                raise RuntimeError("the cache moved under a step that was packed ahead")
        lay = slot.layout
        slot.device[lay.tok[0]:lay.tok[0] + count].copy_(device_tokens, non_blocking=True)
        slot.device[lay.tok[1]:lay.size].copy_(slot.host[lay.tok[1]:lay.size], non_blocking=True)   # all but the token ids
        self.last_h2d_bytes = (lay.size - lay.tok[1]) * 4
        self._copied.record()
        self._copy_pending = True
        slot.graph.replay()
        self.graph_replays += 1
        self.ahead_steps += 1
        self.flying_steps += 1
        self.graph_kernel_launches += slot.launches
        for rid in ahead.request_ids:
            cache.release_passed(rid)
        self.steps_run += 1
        return slot.logits[:count]

    def _graph_width(self, pages_needed: int) -> int:
        """Block-table width of a captured step: the whole table of a request when that is at most
        2,048 entries (one graph per batch bucket), else the next power of two."""
        full = _round4(self.cache.max_pages_per_request)
        if full <= 2048:
            return full
        width = 2048
        while width < pages_needed:
            width *= 2
        return width

    def _capture(self, slot: _Graph, step: StepContext, first_use: bool = True) -> None:
        """Run the step once launch by launch (first-use set-up happens here; left out when a step of the
        same class has run launch by launch before), then capture the same launches into a graph.  The
        captured step is this very step, so replaying it is harmless."""
        from ..kernels import library

        step, caches = self._views(step, slot.device, slot.layout)
        if first_use:
            self.model.forward(step, caches)
        current = torch.cuda.current_stream()
        current.synchronize()
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream()
            self._graph_pool = torch.cuda.graph_pool_handle()
        before = library.launches()
        graph = torch.cuda.CUDAGraph()
        self._capture_stream.wait_stream(current)
        # No garbage collection while the stream is capturing: the collector may destroy CUDA objects of
        # engines that are no longer used (their graphs, their events), and such a call from this thread
        # would invalidate the capture.
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.stream(self._capture_stream):
                graph.capture_begin(pool=self._graph_pool)
                try:
                    slot.logits = self.model.forward(step, caches)
                finally:
                    graph.capture_end()
        finally:
            if collecting:
                gc.enable()
        current.wait_stream(self._capture_stream)
        slot.launches = library.launches() - before
        slot.graph = graph

    def warmup(self, batch_sizes=None) -> None:
        """Capture the decode graphs of the given batch sizes (default: every bucket up to
        ``max_segments``) with temporary one-token requests, then give their pages back.  Before that, one
        step with a prompt portion as long as a step may be, beside a single token of another request: the
        library's products and the prompt kernels load and configure themselves at their first use, which
        would otherwise cost the first request a tenth of a second."""
        self._warm_prompt_path()
        if not self.use_graphs:
            return
        sizes = batch_sizes or [b for b in self.GRAPH_BUCKETS if b <= self.max_segments]
        if not batch_sizes and self.max_segments not in sizes:
            sizes.append(next((b for b in self.GRAPH_BUCKETS if b >= self.max_segments), self.max_segments))
        for size in sorted({min(int(n), self.max_segments) for n in sizes}):
            names = [f"__warmup_{index}" for index in range(size)]
            try:
                for name in names:
                    self.cache.create(name)
                self.run([StepEntry(name, [0], [0]) for name in names])
                torch.cuda.current_stream().synchronize()
            finally:
                for name in names:
                    if name in self.cache.requests:
                        self.cache.free(name)

    def _warm_prompt_path(self) -> None:
        cache = self.cache
        room = min(group.pool.free_pages for group in cache.groups) * cache.page_size if cache.groups else self.max_tokens
        tokens = min(self.max_tokens - 1, self.model.spec.max_position_embeddings - 1, room - cache.page_size)
        if tokens < 2 or self.max_segments < 2:
            return
        names = ["__warmup_portion", "__warmup_token"]
        try:
            for name in names:
                cache.create(name)
            self.run([StepEntry(names[0], [0] * tokens, [tokens - 1]), StepEntry(names[1], [0], [0])])
            torch.cuda.current_stream().synchronize()
        finally:
            for name in names:
                if name in cache.requests:
                    cache.free(name)

    def finish(self, entries: list[StepEntry]) -> None:
        """After the step: give back pages that a window has passed."""
        for entry in entries:
            self.cache.release_passed(entry.request_id)
        self.steps_run += 1
