"""The cache manager: pages of keys and values with a block table per request,
in groups of layers, and slots of fixed-size per-request state.

The reference keeps one pool for all layers, a FIFO free list with an owner
map, a block table per sequence and gives every page back when the sequence
ends (``src/llmserve/kv_cache.py:58-88,135-179,344-350``).  Kept here: the FIFO
free list and the owner checks, ``create / reserve / free``, the limit of pages
per sequence (``kv_cache.py:108-111``) and the statistics (``kv_cache.py:386-413``).
Beyond it:

* Layers are put into *groups* by what their mixer needs (number of key/value
  heads, head size, window).  Each group has its own pool of pages, its own free
  list and its own block table per request.  A group with a window gives a page
  back as soon as every key in it lies before the window of the next token.
* Mixers that keep a state of fixed size per request get *state slots*: one
  tensor [slots, *shape] per layer; a request takes a slot when it is created
  (the slot is zeroed) and gives it back when it ends.  The architecture served
  here has no such mixer; the slots still exist (with no tensors) and carry the
  per-request slot index.

Storage layout of a group: [layer in group, 2 (keys, values), page, kv head,
offset in page, head size]: the tokens of one page and one head are contiguous.
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass, field

import numpy as np
import torch

from ..config.runtime_config import CacheConfig
from ..parts.base import PagedKV, RequestState


class CacheFullError(RuntimeError):
    """No free page (or slot) is left, or a request outgrows what one request may hold."""


class PagePool:
    """O(1) allocator of fixed-size pages: FIFO free list and an owner map.
    Freed pages go to the tail, so a page is used again after all older free pages."""

    def __init__(self, num_pages: int) -> None:
        if num_pages <= 0:
            raise ValueError("num_pages must be positive")
        self.num_pages = num_pages
        self._free: deque[int] = deque(range(num_pages))
        self._owner: dict[int, str] = {}

    def allocate(self, owner: str) -> int:
        if not self._free:
            raise CacheFullError("paged KV cache has no free blocks")
        page = self._free.popleft()
        self._owner[page] = owner
        return page

    def free(self, page: int, owner: str) -> None:
        actual = self._owner.get(page)
        if actual != owner:
            raise ValueError(f"block {page} belongs to {actual!r}, not {owner!r}")
        del self._owner[page]
        self._free.append(page)

    def owner_of(self, page: int) -> str | None:
        return self._owner.get(page)

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def used_pages(self) -> int:
        return len(self._owner)


@dataclass
class CacheGroup:
    """Layers whose mixers need the same kind of pages."""

    need: PagedKV
    layers: list[int]
    page_size: int
    pool: PagePool
    storage: torch.Tensor | None = None           # [len(layers), 2, pages, kv heads, page_size, head size]
    layer_slot: dict[int, int] = field(default_factory=dict)


@dataclass
class StateGroup:
    """Per-layer state tensors [slots, *shape] of mixers with a fixed-size state."""

    tensors: dict[int, torch.Tensor] = field(default_factory=dict)


@dataclass
class RequestCache:
    request_id: str
    state_slot: int
    length: int = 0
    # per group: logical page -> physical page (-1 once a window has passed it)
    tables: list[list[int]] = field(default_factory=list)
    released: list[int] = field(default_factory=list)  # per group: logical pages given back so far
    tables_np: list = field(default_factory=list)      # per group: the same table as an int32 array (grown as needed)


@dataclass
class LayerCache:
    """What one layer's mixer sees during a step (filled by the step function)."""

    keys: torch.Tensor | None = None          # [pages, kv heads, page_size, head size]
    values: torch.Tensor | None = None
    block_tables: torch.Tensor | None = None  # int32 [segments, pages per request] of this layer's group
    slot_mapping: torch.Tensor | None = None  # int32 [tokens]: page * page_size + offset of each row
    state: torch.Tensor | None = None         # [slots, *shape] of a mixer with fixed-size state
    group: int = -1


class CacheManager:
    """Owns every layer's memory between steps.

    ``requirements``: one entry per layer run (a position in the model's order):
    ``PagedKV``, ``RequestState``, ``None``, or an int (the position whose cache this
    run reads).  "Layer" below means such a position.
    """

    def __init__(self, requirements: list, config: CacheConfig, dtype: torch.dtype, device,
                 max_position_embeddings: int, num_state_slots: int = 0) -> None:
        self.config = config
        self.dtype = dtype
        self.device = torch.device(device)
        self.page_size = config.block_size
        # logical pages of one request: the position limit decides (a windowed group may walk
        # through more logical pages than its pool holds, because it gives pages back on the way)
        self.max_pages_per_request = math.ceil(max_position_embeddings / config.block_size)
        self.groups: list[CacheGroup] = []
        self.layer_group: dict[int, int] = {}
        self.layer_source: dict[int, int] = {}
        self.states = StateGroup()
        self.num_state_slots = num_state_slots or config.num_state_slots or 64
        self._free_slots: deque[int] = deque(range(self.num_state_slots))
        self.requests: dict[str, RequestCache] = {}
        self._high_water = {"blocks": 0, "used_tokens": 0, "sequences": 0}

        by_need: dict[PagedKV, CacheGroup] = {}
        for layer, need in enumerate(requirements):
            if isinstance(need, PagedKV):
                group = by_need.get(need)
                if group is None:
                    group = CacheGroup(need, [], self.page_size, PagePool(config.num_blocks))
                    by_need[need] = group
                    self.groups.append(group)
                group.layer_slot[layer] = len(group.layers)
                group.layers.append(layer)
                self.layer_group[layer] = self.groups.index(group)
            elif isinstance(need, RequestState):
                state_dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[need.dtype]
                self.states.tensors[layer] = torch.zeros((self.num_state_slots, *need.shape), dtype=state_dtype,
                                                         device=self.device)
        for layer, need in enumerate(requirements):
            if isinstance(need, int) and not isinstance(need, bool):
                source = need
                if source in self.layer_group:
                    self.layer_group[layer] = self.layer_group[source]
                self.layer_source[layer] = source
        for group in self.groups:
            shape = (len(group.layers), 2, config.num_blocks, group.need.num_kv_heads, self.page_size,
                     group.need.head_dim)
            group.storage = torch.zeros(shape, dtype=dtype, device=self.device)

    # -- requests ----------------------------------------------------------------
    def create(self, request_id: str) -> RequestCache:
        if request_id in self.requests:
            raise ValueError(f"sequence {request_id!r} already exists")
        if not self._free_slots:
            raise CacheFullError("no free per-request state slot")
        slot = self._free_slots.popleft()
        for tensor in self.states.tensors.values():
            tensor[slot].zero_()
        request = RequestCache(request_id, slot, 0, [[] for _ in self.groups], [0 for _ in self.groups],
                               [np.full(16, -1, dtype=np.int32) for _ in self.groups])
        self.requests[request_id] = request
        return request

    def pages_needed(self, request_id: str, count: int) -> list[int]:
        """New pages per group that ``count`` more tokens of the request take."""
        request = self.requests[request_id]
        after = (request.length + count + self.page_size - 1) // self.page_size
        return [after - len(table) for table in request.tables]

    def free_pages(self) -> list[int]:
        return [group.pool.free_pages for group in self.groups]

    def fits(self, planned: list[tuple[str, int]]) -> bool:
        """Whether every group has the pages for all of ``planned`` (request, tokens)."""
        need = [0] * len(self.groups)
        for request_id, count in planned:
            for index, pages in enumerate(self.pages_needed(request_id, count)):
                need[index] += pages
        return all(n <= group.pool.free_pages for n, group in zip(need, self.groups))

    def grow(self, request_id: str, count: int) -> bool:
        """Take the pages that the request's next ``count`` tokens need, without counting the tokens
        in: a later ``reserve`` finds them there.  Pages taken early are the request's like any other
        and go back with it.  False, and nothing changed, when a group has too few free pages or the
        request would outgrow its table."""
        request = self.requests[request_id]
        after = (request.length + count + self.page_size - 1) // self.page_size
        if after > self.max_pages_per_request:
            return False
        for group, table in zip(self.groups, request.tables):
            if after - len(table) > group.pool.free_pages:
                return False
        self._extend(request, after)
        return True

    def _extend(self, request: RequestCache, after: int) -> None:
        request_id = request.request_id
        for index, (group, table) in enumerate(zip(self.groups, request.tables)):
            while len(table) < after:
                page = group.pool.allocate(request_id)
                mirror = request.tables_np[index]
                if len(table) >= mirror.shape[0]:
                    grown = np.full(max(2 * mirror.shape[0], after), -1, dtype=np.int32)
                    grown[:mirror.shape[0]] = mirror
                    request.tables_np[index] = mirror = grown
                mirror[len(table)] = page
                table.append(page)

    def reserve(self, request_id: str, count: int) -> int:
        """Make room for the request's next ``count`` tokens and return the position of
        the first.  Either every page is had or nothing changes."""
        if count <= 0:
            raise ValueError("count must be positive")
        request = self.requests[request_id]
        after = (request.length + count + self.page_size - 1) // self.page_size
        if after > self.max_pages_per_request:
            raise CacheFullError("sequence exceeds paged KV metadata capacity")
        for group, table in zip(self.groups, request.tables):
            if after - len(table) > group.pool.free_pages:
                raise CacheFullError("paged KV cache has no free blocks")
        self._extend(request, after)
        first = request.length
        request.length += count
        used = sum(group.pool.used_pages for group in self.groups)
        if used >= self._high_water["blocks"]:
            self._high_water = {"blocks": used,
                                "used_tokens": sum(item.length for item in self.requests.values()),
                                "sequences": len(self.requests)}
        return first

    def release_passed(self, request_id: str) -> int:
        """Give back the pages of windowed groups that no later token can read:
        a page whose last key lies before ``length - window + 1``.  Returns how many."""
        request = self.requests[request_id]
        given = 0
        for index, group in enumerate(self.groups):
            window = group.need.window
            if window <= 0:
                continue
            first_needed = request.length - window + 1   # smallest key the next token reads
            table = request.tables[index]
            page = request.released[index]
            while page < len(table) and (page + 1) * self.page_size <= first_needed:
                group.pool.free(table[page], request_id)
                table[page] = -1
                request.tables_np[index][page] = -1
                page += 1
                given += 1
            request.released[index] = page
        return given

    def free(self, request_id: str) -> None:
        request = self.requests.pop(request_id)
        for group, table in zip(self.groups, request.tables):
            for page in table:
                if page >= 0:
                    group.pool.free(page, request_id)
        self._free_slots.append(request.state_slot)

    def free_all(self) -> None:
        for request_id in list(self.requests):
            self.free(request_id)

    # -- metadata of a step -------------------------------------------------------
    def slot_mapping(self, group_index: int, request_id: str, first: int, count: int) -> np.ndarray:
        """Flat cache slot (page * page_size + offset) of positions first .. first+count-1."""
        table = self.requests[request_id].tables[group_index]
        positions = np.arange(first, first + count)
        pages = np.asarray(table, dtype=np.int64)[positions // self.page_size]
        return (pages * self.page_size + positions % self.page_size).astype(np.int32)

    def block_table(self, group_index: int, request_id: str) -> list[int]:
        return self.requests[request_id].tables[group_index]

    def block_table_array(self, group_index: int, request_id: str) -> np.ndarray:
        """The request's block table as an int32 array (a view; its first len(block_table) entries count)."""
        request = self.requests[request_id]
        return request.tables_np[group_index][:len(request.tables[group_index])]

    def layer_view(self, layer: int) -> LayerCache:
        """The storage of ``layer`` (or of the layer whose cache it reads)."""
        source = self.layer_source.get(layer, layer)
        view = LayerCache()
        if source in self.layer_group and source in self.groups[self.layer_group[source]].layer_slot:
            group_index = self.layer_group[source]
            group = self.groups[group_index]
            storage = group.storage[group.layer_slot[source]]
            view.keys, view.values, view.group = storage[0], storage[1], group_index
        if source in self.states.tensors:
            view.state = self.states.tensors[source]
        return view

    # -- statistics ------------------------------------------------------------
    def bytes_per_page(self, group: CacheGroup) -> int:
        return (len(group.layers) * 2 * self.page_size * group.need.num_kv_heads * group.need.head_dim
                * torch.empty((), dtype=self.dtype).element_size())

    def kv_bytes_per_token(self) -> int:
        return sum(self.bytes_per_page(group) // self.page_size for group in self.groups)

    def stats(self, contiguous_max_length: int | None = None) -> dict[str, float]:
        used_tokens = sum(request.length for request in self.requests.values())
        used_pages = sum(group.pool.used_pages for group in self.groups)
        free_pages = sum(group.pool.free_pages for group in self.groups)
        n_groups = max(len(self.groups), 1)
        allocated_slots = used_pages * self.page_size / n_groups
        waste = allocated_slots - used_tokens
        page_bytes = sum(self.bytes_per_page(group) for group in self.groups) / n_groups
        result = {
            "blocks_used": float(used_pages),
            "blocks_free": float(free_pages),
            "used_tokens": float(used_tokens),
            "paged_waste_tokens": float(waste),
            "paged_fragmentation_pct": 100.0 * waste / max(allocated_slots, 1),
            "paged_allocated_gb": used_pages * page_bytes / 1024**3,
            "peak_blocks_used": float(self._high_water["blocks"]),
            "peak_paged_allocated_gb": self._high_water["blocks"] * page_bytes / 1024**3,
        }
        if contiguous_max_length is not None:
            contiguous_slots = self._high_water["sequences"] * contiguous_max_length
            peak_slots = self._high_water["blocks"] * self.page_size / n_groups
            result.update(
                contiguous_waste_tokens=float(max(contiguous_slots - self._high_water["used_tokens"], 0)),
                memory_reduction_pct=100.0 * (contiguous_slots - peak_slots) / max(contiguous_slots, 1),
            )
        return result

    @property
    def capacity_tokens(self) -> int:
        return self.config.num_blocks * self.page_size
