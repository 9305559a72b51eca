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
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.manager import CacheManager, LayerCache


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
        self.segment_of_token: torch.Tensor = None   # [T]
        self.segment_start: torch.Tensor = None      # [S + 1] first row of each segment
        self.segment_first_position: torch.Tensor = None  # [S]
        self.segment_context: torch.Tensor = None    # [S] keys of the request after this step
        self.segment_state_slot: torch.Tensor = None  # [S]
        self.want_rows: torch.Tensor = None          # [W]
        self.max_segment_tokens = 0
        self.max_context = 0                         # None: not known on the host (a replayed graph)
        self.decode_only = False                     # every segment brings exactly one token


def _round4(n: int) -> int:
    return (n + 3) & ~3


class StepRunner:
    """Packs a step, runs the model on it and keeps the cache manager in step."""

    def __init__(self, model, cache: CacheManager, max_tokens_per_step: int, max_segments: int) -> None:
        self.model = model
        self.cache = cache
        self.device = model.device
        self.max_tokens = int(max_tokens_per_step)
        self.max_segments = int(max_segments)
        n_groups = len(cache.groups)
        table_width = _round4(cache.max_pages_per_request)
        capacity = (4 * _round4(self.max_tokens) + _round4(self.max_segments + 1) + 3 * _round4(self.max_segments)
                    + n_groups * (_round4(self.max_tokens) + self.max_segments * table_width))
        self._capacity = capacity
        self._host = torch.empty(capacity, dtype=torch.int32, pin_memory=self.device.type == "cuda")
        self._host_np = self._host.numpy()
        self._device = torch.empty(capacity, dtype=torch.int32, device=self.device)
        self._layer_views = [cache.layer_view(position) for position in range(len(model.spec.order))]
        self._copied = torch.cuda.Event() if self.device.type == "cuda" else None
        self._copy_pending = False
        self.steps_run = 0
        self.last_h2d_bytes = 0

    # -- the step ------------------------------------------------------------------
    def run(self, entries: list[StepEntry]) -> torch.Tensor:
        """Run one step.  Returns float32 logits [total wanted, vocab] on the device, in the
        order of the entries and of each entry's ``want``."""
        step, caches = self.prepare(entries)
        logits = self.model.forward(step, caches)
        self.finish(entries)
        return logits

    def prepare(self, entries: list[StepEntry]):
        cache = self.cache
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
        planned = [(entry.request_id, len(entry.tokens)) for entry in entries]
        if not cache.fits(planned):
            from ..cache.manager import CacheFullError
            raise CacheFullError("paged KV cache has no free blocks for this step")

        if self._copy_pending:   # the pinned buffer is reused: the last copy must have left it
            self._copied.synchronize()
            self._copy_pending = False
        step = StepContext()
        n_seg = len(entries)
        wanted = sum(len(entry.want) for entry in entries)
        table_width = _round4(max(1, max(
            (cache.requests[e.request_id].length + len(e.tokens) + cache.page_size - 1) // cache.page_size
            for e in entries)))
        host = self._host_np
        cursor = 0

        def take(n: int):
            nonlocal cursor
            view = (cursor, cursor + n)
            cursor += _round4(n)
            return view

        r_tok, r_pos, r_seg = take(total), take(total), take(total)
        r_start, r_first, r_ctx, r_slot = take(n_seg + 1), take(n_seg), take(n_seg), take(n_seg)
        r_want = take(wanted)
        r_maps = [take(total) for _ in cache.groups]
        r_tables = [take(n_seg * table_width) for _ in cache.groups]
        if cursor > self._capacity:
            raise ValueError("step metadata exceeds its buffer")
        for lo, hi in r_tables:
            host[lo:hi] = -1

        row = 0
        want_cursor = r_want[0]
        for index, entry in enumerate(entries):
            count = len(entry.tokens)
            first = cache.reserve(entry.request_id, count)
            request = cache.requests[entry.request_id]
            step.segments.append(Segment(entry.request_id, request.state_slot, first, count, row))
            host[r_tok[0] + row: r_tok[0] + row + count] = entry.tokens
            host[r_pos[0] + row: r_pos[0] + row + count] = np.arange(first, first + count, dtype=np.int32)
            host[r_seg[0] + row: r_seg[0] + row + count] = index
            host[r_start[0] + index] = row
            host[r_first[0] + index] = first
            host[r_ctx[0] + index] = first + count
            host[r_slot[0] + index] = request.state_slot
            for offset in entry.want:
                host[want_cursor] = row + offset
                want_cursor += 1
            for g in range(len(cache.groups)):
                host[r_maps[g][0] + row: r_maps[g][0] + row + count] = cache.slot_mapping(g, entry.request_id, first, count)
                table = cache.block_table(g, entry.request_id)
                base = r_tables[g][0] + index * table_width
                host[base: base + len(table)] = table
            step.max_segment_tokens = max(step.max_segment_tokens, count)
            step.max_context = max(step.max_context, first + count)
            row += count
        host[r_start[0] + n_seg] = row
        step.decode_only = step.max_segment_tokens == 1

        self._device[:cursor].copy_(self._host[:cursor], non_blocking=True)
        self.last_h2d_bytes = cursor * 4
        if self._copied is not None:
            self._copied.record()
            self._copy_pending = True
        dev = self._device
        step.num_tokens, step.num_segments, step.num_wanted = total, n_seg, wanted
        step.token_ids = dev[r_tok[0]:r_tok[1]]
        step.positions = dev[r_pos[0]:r_pos[1]]
        step.segment_of_token = dev[r_seg[0]:r_seg[1]]
        step.segment_start = dev[r_start[0]:r_start[1]]
        step.segment_first_position = dev[r_first[0]:r_first[1]]
        step.segment_context = dev[r_ctx[0]:r_ctx[1]]
        step.segment_state_slot = dev[r_slot[0]:r_slot[1]]
        step.want_rows = dev[r_want[0]:r_want[1]]

        group_maps = [dev[lo:hi] for lo, hi in r_maps]
        group_tables = [dev[lo:hi].view(n_seg, table_width) for lo, hi in r_tables]
        caches = []
        for view in self._layer_views:
            layer_cache = LayerCache(keys=view.keys, values=view.values, state=view.state, group=view.group)
            if view.group >= 0:
                layer_cache.slot_mapping = group_maps[view.group]
                layer_cache.block_tables = group_tables[view.group]
            caches.append(layer_cache)
        return step, caches

    def finish(self, entries: list[StepEntry]) -> None:
        """After the step: give back pages that a window has passed."""
        for entry in entries:
            self.cache.release_passed(entry.request_id)
        self.steps_run += 1
