"""The checked variant of the kernel library (``LSE_CHECK=1``: every index taken from a step's metadata is compared
with its range, a bad one is replaced by a safe one and recorded).  It is a library of its own and is chosen when the
library is first loaded, so the checks run in a child process: a replay of mixed traces must record nothing and
give the logits of the plain implementation; then a block table is damaged on the host (an entry of -1 inside the
context, which the ordinary library would turn into an address) and the record must name it, with no fault."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

CHILD = r"""
import random, sys
sys.path.insert(0, {tests!r}); sys.path.insert(0, {root!r})
import torch
import helpers
from tiny_configs import ALL
from llm_serving_engine_b200.kernels import library

for name, dtype in (("A", "float32"), ("D", "bfloat16"), ("E", "bfloat16")):
    config, page, _ = ALL[name]
    rng = random.Random(5)
    requests = {{f"m{{i}}": helpers.random_tokens(rng, config["vocab_size"], rng.randrange(20, 180)) for i in range(7)}}
    steps, peak = helpers.trace_mixed(requests, seed=6)
    got = helpers.run_trace(name, dtype, steps, peak, page)
    helpers.assert_close(name, dtype, requests, got, "checked build, mixed")
    whole = helpers.run_trace(name, dtype, helpers.trace_whole(requests), helpers.max_tokens_for(requests), page)
    helpers.assert_close(name, dtype, requests, whole, "checked build, whole")
    assert library.check_report() == [], library.check_report()
print("clean: nothing recorded")

# damage on the host: the checked library must notice, replace the index and go on
from llm_serving_engine_b200.cache import CacheManager
from llm_serving_engine_b200.config import CacheConfig
from llm_serving_engine_b200.engine import StepEntry, StepRunner
from llm_serving_engine_b200.models import cache_requirements, load_model
for name, dtype in (("A", "float32"), ("D", "bfloat16")):
    config, page, _ = ALL[name]
    model = load_model(helpers.model_folder(name), dtype=dtype, device="cuda")
    cache = CacheManager(cache_requirements(model.spec), CacheConfig(page, 32), model.dtype, model.device, 512, num_state_slots=2)
    runner = StepRunner(model, cache, 256, 2, use_graphs=False)
    tokens = helpers.random_tokens(random.Random(7), config["vocab_size"], 70)
    with torch.inference_mode():
        cache.create("r")
        runner.run([StepEntry("r", tokens[:60], [])])
        request = cache.requests["r"]
        kept = request.tables[0][1]
        request.tables[0][1] = -1
        request.tables_np[0][1] = -1          # keys 16 .. 31 (page 16) now point nowhere
        runner.run([StepEntry("r", tokens[60:62], [1])])      # a portion: the prompt kernels read the table
        runner.run([StepEntry("r", [tokens[62]], [0])])       # a single token: the decode kernels do
        torch.cuda.synchronize()
        report = library.check_report()
        assert any("block-table entry -1" in line for line in report), report
        request.tables[0][1] = kept
        request.tables_np[0][1] = kept
        cache.free("r")
    print(name, dtype, "recorded:", report)
"""


def test_checked_library_records_nothing_on_good_steps_and_names_a_bad_table_entry():
    tests = os.path.dirname(os.path.abspath(__file__))
    root = os.path.dirname(tests)
    env = dict(os.environ, LSE_CHECK="1")
    done = subprocess.run([sys.executable, "-c", CHILD.format(tests=tests, root=root)], env=env, capture_output=True,
                          text=True, timeout=900)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
    assert "clean: nothing recorded" in done.stdout and done.stdout.count("recorded:") == 2   # one per damaged model
