"""The sampling entry point that allocates nothing (csrc/sampling_noalloc.h), called through its
exported C symbol the way a foreign caller would, against the ordinary entry point.

It is for callers that cannot allocate device memory when they sample (frozen memory pools,
plugins without an allocator): the scratch it needs is an array inside the library image.
The file is named so that pytest collects it last."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_FLOATS = 2 * 1024 * 1024


def _symbol():
    from llm_serving_engine_b200.csrc import build
    lib = ctypes.CDLL(str(build.library_path(verbose=False)))
    fn = lib.lse_sample_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    return fn


def _inputs(rows, vocab, seed):
    generator = torch.Generator(device="cuda").manual_seed(seed)
    logits = torch.randn(rows, vocab, device="cuda", generator=generator) * 2
    temperature = torch.tensor([0.8, 1.3, 0.0, 0.5, 1.0][:rows] + [0.9] * max(0, rows - 5), device="cuda")
    top_p = torch.tensor([1.0, 0.9, 1.0, 0.4, 0.7][:rows] + [1.0] * max(0, rows - 5), device="cuda")
    seeds = torch.arange(rows, dtype=torch.int64, device="cuda") * 31 + seed
    counters = torch.arange(rows, dtype=torch.int64, device="cuda") + 2
    return logits, temperature, top_p, seeds, counters


def test_no_alloc_sampling_matches_the_ordinary_entry_point_twice_in_a_row():
    from llm_serving_engine_b200.kernels import ops
    fn = _symbol()
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row with different sizes: the second finds the first call's leftovers in the scratch
    for rows, vocab, seed in ((5, 151936, 1), (7, 1000, 2)):
        logits, temperature, top_p, seeds, counters = _inputs(rows, vocab, seed)
        want = torch.empty(rows, dtype=torch.int32, device="cuda")
        ops.sample(logits, temperature, top_p, seeds, counters, torch.empty(rows * vocab, device="cuda"), want)
        got = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
        before = torch.cuda.memory_allocated()
        code = fn(logits.data_ptr(), logits.stride(0), rows, vocab, temperature.data_ptr(), top_p.data_ptr(),
                  seeds.data_ptr(), counters.data_ptr(), got.data_ptr(), stream)
        torch.cuda.synchronize()
        assert code == 0
        assert torch.cuda.memory_allocated() == before
        assert got.tolist() == want.tolist()     # same kernel, same inputs: the same tokens exactly


def test_no_alloc_sampling_refuses_more_than_its_scratch_holds(capfd):
    fn = _symbol()
    rows, vocab = 17, 151936                      # 2.58 M floats > 2 Mi
    assert rows * vocab > MAX_FLOATS
    logits, temperature, top_p, seeds, counters = _inputs(rows, 8, 3)   # small tensors: nothing may be read
    out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    code = fn(logits.data_ptr(), 8, rows, vocab, temperature.data_ptr(), top_p.data_ptr(), seeds.data_ptr(),
              counters.data_ptr(), out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert code == -2 and out.tolist() == [-1] * rows
    assert "built-in scratch" in capfd.readouterr().err
