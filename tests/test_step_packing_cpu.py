"""The step's metadata on the host (no GPU): what is packed for a mixed batch, and that the
fast path for decode steps writes the same arrays as the general one."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from llm_serving_engine_b200.cache import CacheManager
from llm_serving_engine_b200.config import CacheConfig
from llm_serving_engine_b200.engine.step import StepEntry, StepRunner, _Layout
from llm_serving_engine_b200.parts import PagedKV


def make_runner(groups=(PagedKV(2, 16), PagedKV(1, 32, window=20)), pages=64, page=4):
    model = SimpleNamespace(device=torch.device("cpu"), vocab_size=100, spec=SimpleNamespace(order=tuple(range(len(groups)))),
                            graph_safe=True)
    cache = CacheManager(list(groups), CacheConfig(page, pages), torch.float32, "cpu", 256, num_state_slots=8)
    return StepRunner(model, cache, max_tokens_per_step=64, max_segments=8), cache


def test_mixed_batch_metadata():
    runner, cache = make_runner()
    for rid in "abc":
        cache.create(rid)
    runner.prepare([StepEntry("a", [1, 2, 3, 4, 5, 6], []), StepEntry("b", [7], [])])   # earlier steps
    step, caches = runner.prepare([StepEntry("a", [9], [0]), StepEntry("c", [11, 12, 13], [0, 2]), StepEntry("b", [8, 9], [1])])
    assert (step.num_tokens, step.num_segments, step.num_wanted) == (6, 3, 4)
    assert step.token_ids.tolist() == [9, 11, 12, 13, 8, 9]
    assert step.positions.tolist() == [6, 0, 1, 2, 1, 2]
    assert step.segment_of_token.tolist() == [0, 1, 1, 1, 2, 2]
    assert step.segment_start.tolist() == [0, 1, 4, 6]
    assert step.segment_first_position.tolist() == [6, 0, 1] and step.segment_context.tolist() == [7, 3, 3]
    assert step.want_rows.tolist() == [0, 1, 3, 5]
    assert not step.decode_only and step.max_segment_tokens == 3 and step.max_context == 7
    assert [s.request_id for s in step.segments] == ["a", "c", "b"]
    table_a = cache.block_table(0, "a")
    assert caches[0].block_tables[0, :len(table_a)].tolist() == table_a
    assert caches[0].slot_mapping.tolist()[0] == table_a[1] * 4 + 2          # position 6 = page 1, offset 2
    assert caches[1].block_tables.data_ptr() != caches[0].block_tables.data_ptr()   # each group has its own tables


def test_step_validation():
    runner, cache = make_runner()
    cache.create("a")
    for entries, message in [([], "at least one"), ([StepEntry("a", [], [])], "no tokens"),
                             ([StepEntry("a", [100], [])], "token id"), ([StepEntry("a", [1], [1])], "wanted place"),
                             ([StepEntry("a", [1], []), StepEntry("a", [2], [])], "twice"),
                             ([StepEntry("a", list(range(65)), [])], "at most 64")]:
        with pytest.raises(ValueError, match=message):
            runner.prepare(entries)
    assert cache.requests["a"].length == 0          # nothing was reserved by refused steps


@pytest.mark.parametrize("lengths", [(5,), (1, 17, 40), (3, 3, 3, 3, 9, 30, 2)])
def test_decode_fast_path_packs_what_the_general_path_packs(lengths):
    general, fast = make_runner(), make_runner()
    names = [f"r{i}" for i in range(len(lengths))]
    for runner, cache in (general, fast):
        for name, length in zip(names, lengths):
            cache.create(name)
            cache.reserve(name, length)
            cache.release_passed(name)
    entries = [StepEntry(name, [10 + i], [0]) for i, name in enumerate(names)]
    bucket = 8
    layout = _Layout(bucket, bucket, bucket, 64, 2)
    host_a = np.zeros(layout.size, dtype=np.int32)
    host_b = np.full(layout.size, 7, dtype=np.int32)     # stale contents must be overwritten
    step_a = general[0]._pack(entries, host_a, layout, wanted_all_rows=True)
    step_b = fast[0]._pack_decode(entries, host_b, layout)
    regions = [layout.tok, layout.pos, layout.seg, layout.start, layout.first, layout.ctx, layout.slot, layout.want]
    for lo, hi in regions + layout.maps + layout.tables:     # (the padding between arrays is never read)
        assert np.array_equal(host_a[lo:hi], host_b[lo:hi]), (lo, hi)
    assert step_a.decode_only and step_b.decode_only and step_a.max_context == step_b.max_context
    assert [(s.request_id, s.first_position, s.row_start) for s in step_a.segments] == \
           [(s.request_id, s.first_position, s.row_start) for s in step_b.segments]
