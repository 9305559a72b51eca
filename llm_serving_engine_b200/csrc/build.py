"""Compile the engine's CUDA sources for sm_100a into one shared library.

The library is built with nvcc alone (no framework headers), in-tree under
``llm_serving_engine_b200/_build/``, the first time it is needed, and again
when a source or a flag changes (the key is a hash of both).  While nvcc runs,
a line is printed every few seconds so that a first call does not look hung.
Nothing outside the package directory is written unless that directory is
read-only, in which case a per-user temporary directory is used.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PACKAGE = CSRC.parent
LIB_NAME = "libllmserve_b200_kernels.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


class BuildError(RuntimeError):
    pass


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise BuildError("nvcc not found: the CUDA kernels cannot be built (set NVCC or add it to PATH)")


def _key(flags: list[str]) -> str:
    digest = hashlib.sha256()
    digest.update(" ".join(flags).encode())
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()[:16]


def _build_dir() -> Path:
    preferred = PACKAGE / "_build"
    try:
        preferred.mkdir(exist_ok=True)
        probe = preferred / f".write_probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return preferred
    except OSError:
        fallback = Path(tempfile.gettempdir()) / f"llmserve_b200_build_{os.getuid()}"
        fallback.mkdir(parents=True, exist_ok=True)
        return fallback


def _log(message: str, verbose: bool) -> None:
    if verbose:
        print(f"[llm_serving_engine_b200] {message}", file=sys.stderr, flush=True)


def library_path(verbose: bool = True, force: bool = False, trace: bool = False, check: bool = False) -> Path:
    """Path of the built library; compiles it first when it is missing or stale.

    ``trace``: the tuning variant (``-DLSE_TRACE``), in which block 0 of every kernel records when it
    started, when its wait for the kernels before returned and when it ended; a library of its own.
    ``check``: the checked variant (``-DLSE_CHECK``), in which every kernel compares the indices it takes
    from the step's metadata with their ranges, replaces a bad one by a safe one and records it; a
    library of its own as well."""
    build_dir = _build_dir()
    variant = "_trace" if trace else "_check" if check else ""
    flags = NVCC_FLAGS + (["-DLSE_TRACE"] if trace else ["-DLSE_CHECK"] if check else [])
    key = _key(flags)
    lib = build_dir / LIB_NAME.replace(".so", f"{variant}.so")
    stamp = build_dir / f"build{variant}.key"
    if not force and lib.exists() and stamp.exists() and stamp.read_text().strip() == key:
        return lib
    nvcc = _nvcc()
    srcs = sources()
    _log(f"compiling {len(srcs)} CUDA sources for sm_100a into {build_dir} (first call only)", verbose)
    started = time.time()
    done = threading.Event()

    def heartbeat() -> None:
        while not done.wait(10.0):
            _log(f"still compiling ... {time.time() - started:.0f} s", verbose)

    beat = threading.Thread(target=heartbeat, daemon=True)
    beat.start()
    objects: list[Path] = []
    try:
        def compile_one(src: Path) -> Path:
            obj = build_dir / (src.stem + f".{os.getpid()}.o")
            cmd = [nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            result = subprocess.run(cmd, capture_output=True, text=True)
            if result.returncode != 0:
                raise BuildError(f"nvcc failed on {src.name}:\n{result.stdout}\n{result.stderr}")
            _log(f"compiled {src.name} ({time.time() - started:.0f} s)", verbose)
            return obj

        with ThreadPoolExecutor(max_workers=min(8, len(srcs), os.cpu_count() or 1)) as pool:
            objects = list(pool.map(compile_one, srcs))
        tmp_lib = build_dir / f"{lib.name}.{os.getpid()}.tmp"
        cmd = [nvcc, "-shared", "-o", str(tmp_lib), *map(str, objects)]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if result.returncode != 0:
            raise BuildError(f"link failed:\n{result.stdout}\n{result.stderr}")
        os.replace(tmp_lib, lib)  # atomic: a concurrent process sees the old or the new file
        stamp.write_text(key)
    finally:
        done.set()
        for obj in objects:
            try:
                obj.unlink()
            except OSError:
                pass
    _log(f"built {lib.name} in {time.time() - started:.0f} s", verbose)
    return lib


if __name__ == "__main__":
    print(library_path(force="--force" in sys.argv))
