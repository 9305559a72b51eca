"""Loads the compiled CUDA library and declares its C entry points.

There is no fallback: if the library cannot be built or loaded, or a launch
reports an error, an exception is raised.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p

from ..csrc import build

_lib = None

_SIGNATURES = {
    "lse_embedding": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "lse_add_rmsnorm": [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_int,
                        c_int, c_float, c_int, c_int, c_void_p],
    "lse_rope_kv_write": [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_longlong, c_int, c_void_p],
    "lse_silu_mul": [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p],
    "lse_gemm_bf16_skinny": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "lse_gemm_bf16_skinny_pad": [c_int],
    "lse_gemm_bf16_skinny_splits": [c_int, c_int],
    "lse_gemm_bf16_skinny_test_hooks": [c_uint, c_int],
    "lse_gemm_bf16_skinny_status": [],
    "lse_gemm_bf16_skinny_status_async": [c_void_p, c_void_p],
    "lse_gemm_bf16_skinny_status_reset": [],
    "lse_attention_tc_status_async": [c_void_p, c_void_p],
    "lse_attention_tc_status_reset": [],
    "lse_gemm_f32_nt": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong,
                        c_longlong, c_longlong, c_int, c_longlong, c_void_p],
    "lse_gemm_f32_ranges": [c_int],
    "lse_gemm_f32_stack_ok": [c_void_p, c_void_p, c_int, c_int, c_longlong, c_longlong],
    "lse_paged_attention_generic": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                    c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                    c_int, c_int, c_int, c_void_p, c_int, c_void_p],
    "lse_attention_generic_chunk": [],
    "lse_paged_attention_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                   c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                                   c_void_p, c_void_p, c_void_p],
    "lse_paged_attention_prefill": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                    c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p],
    "lse_attention_mma_supported": [c_int, c_int, c_int],
    "lse_paged_attention_prefill_tc": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                       c_int, c_int, c_longlong, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
                                       c_void_p, c_longlong, c_void_p],
    "lse_attention_tc_scratch_floats": [],
    "lse_attention_tc_supported": [c_int, c_int, c_int, c_int],
    "lse_attention_tc_status": [],
    "lse_set_pdl": [c_int],
    "lse_argmax": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p],
    "lse_sample": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                   c_void_p, c_void_p, c_void_p],
}


class KernelError(RuntimeError):
    """A kernel launcher refused its arguments or CUDA reported an error."""


def load(verbose: bool = True):
    """The ctypes handle of the kernel library (built at the first call)."""
    global _lib
    if _lib is None:
        import os
        # LSE_TRACE=1: the tuning variant; LSE_CHECK=1: the checked variant (indices compared with their ranges)
        path = build.library_path(verbose=verbose, trace=os.environ.get("LSE_TRACE", "0") == "1",
                                  check=os.environ.get("LSE_CHECK", "0") == "1")
        lib = ctypes.CDLL(str(path))
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        if os.environ.get("LSE_PDL", "1") == "0":   # programmatic dependent launch off (for comparisons)
            lib.lse_set_pdl(0)
        _lib = lib
    return _lib


def register_signatures(signatures: dict) -> None:
    """Declare further entry points (used by kernel files added later)."""
    _SIGNATURES.update(signatures)
    if _lib is not None:
        for name, argtypes in signatures.items():
            fn = getattr(_lib, name)
            fn.argtypes = argtypes
            fn.restype = c_int


CHECK_READERS = ("lse_check_elementwise", "lse_check_attention_generic", "lse_check_attention_mma", "lse_check_attention_tc")
CHECK_KINDS = {1: "token id", 2: "cache slot", 3: "block-table entry", 4: "segment number", 5: "row index"}


def check_report(reset: bool = True) -> list[str]:
    """What the checked variant of the library (``LSE_CHECK=1``) has recorded: one line per source file whose
    kernels met an index outside its range (empty: none).  Synchronises the device.  Raises when the loaded
    library is not the checked variant."""
    lib = load()
    found = []
    for name in CHECK_READERS:
        try:
            reader = getattr(lib, name)
        except AttributeError:
            raise KernelError("the loaded kernel library is not the checked variant (set LSE_CHECK=1 before the first use)") from None
        reader.argtypes = [c_void_p, c_int]
        reader.restype = c_int
        words = (c_int * 4)()
        if reader(words, int(reset)) != 0:
            raise KernelError(f"{name}: the check words could not be read")
        if words[0]:
            found.append(f"{name[len('lse_check_'):]}: {CHECK_KINDS.get(words[0], words[0])} {words[1]} outside [{words[2]}, {words[3]})")
    return found


_launch_count = 0


def launches() -> int:
    """How many kernels of this library have been launched by this process."""
    return _launch_count


def check(code: int, name: str) -> None:
    global _launch_count
    _launch_count += 1
    if code == 0:
        return
    if code == -1:
        raise KernelError(f"{name}: unsupported or inconsistent arguments")
    if code == -2:
        raise KernelError(f"{name}: size beyond what this kernel was built for")
    raise KernelError(f"{name}: CUDA error {code}")
