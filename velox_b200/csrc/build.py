"""Compiles the CUDA sources of this directory for sm_100a and loads them with ctypes.

There are two libraries: ``core`` (row-wise kernels, sampling, GEMMs; one build) and
``attention`` (one build per head size, ``-DVX_HEAD_DIM=<D>``), so a process compiles what its
model needs and nothing else.  A build is keyed by a hash of its sources, flags and compiler
version; it is made once and reused.  Builds go to ``velox_b200/_build`` inside the package when
that is writable, else to ``$VELOX_B200_BUILD_DIR``, else to a per-user folder under the
system's temporary directory.  nvcc cross-compiles without a GPU, so the build also runs on a
machine that has none.

The launchers are plain C functions over raw pointers (see ``common.cuh``); there is no torch
header in the build, which keeps a cold build to seconds per file.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import re
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

_SRC_DIR = os.path.dirname(os.path.abspath(__file__))

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo"]
# VELOX_B200_TRACE=1 builds (and loads) libraries whose kernels record a timeline.
if os.environ.get("VELOX_B200_TRACE") == "1":
    COMMON_FLAGS = COMMON_FLAGS + ["-DVX_TRACE"]

CORE_SOURCES = ("core.cu", "sampling.cu", "gemm_bf16.cu")
ATTENTION_SOURCES = ("attention.cu",)
HEADERS = ("common.cuh", "attention_static.h")

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _say(message: str) -> None:
    print(f"[velox_b200] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for candidate in (
        os.environ.get("VELOX_B200_NVCC"),
        shutil.which("nvcc"),
        os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ):
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise BuildError(
        "nvcc was not found (looked at $VELOX_B200_NVCC, PATH, $CUDA_HOME/bin and "
        "/usr/local/cuda/bin); the CUDA kernels of velox_b200 cannot be built"
    )


def build_dir() -> str:
    candidates = [os.path.join(os.path.dirname(_SRC_DIR), "_build")]
    if os.environ.get("VELOX_B200_BUILD_DIR"):
        candidates.insert(0, os.environ["VELOX_B200_BUILD_DIR"])
    candidates.append(os.path.join(tempfile.gettempdir(), f"velox_b200_build_{os.getuid()}"))
    for path in candidates:
        try:
            os.makedirs(path, exist_ok=True)
            probe = os.path.join(path, f".probe_{os.getpid()}")
            with open(probe, "w") as handle:
                handle.write("x")
            os.remove(probe)
            return path
        except OSError:
            continue
    raise BuildError(f"no writable build directory among {candidates}")


def _nvcc_version(nvcc: str) -> str:
    try:
        out = subprocess.run([nvcc, "--version"], capture_output=True, text=True, check=True).stdout
    except (OSError, subprocess.CalledProcessError) as exc:
        raise BuildError(f"cannot run {nvcc}: {exc}") from exc
    return out.strip().splitlines()[-1]


def _build_key(sources: Sequence[str], defines: Sequence[str], nvcc_version: str) -> str:
    digest = hashlib.sha256()
    for name in list(sources) + list(HEADERS):
        with open(os.path.join(_SRC_DIR, name), "rb") as handle:
            digest.update(name.encode())
            digest.update(handle.read())
    digest.update(" ".join(ARCH_FLAGS + COMMON_FLAGS + list(defines)).encode())
    digest.update(nvcc_version.encode())
    return digest.hexdigest()[:16]


def _run_with_progress(commands: List[Tuple[str, List[str]]], what: str) -> None:
    """Run compile commands in parallel, printing a line every few seconds while they run."""
    started = time.time()
    done: List[str] = []

    def run(item: Tuple[str, List[str]]) -> None:
        label, cmd = item
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"nvcc failed on {label}:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
        done.append(label)

    workers = max(1, min(len(commands), os.cpu_count() or 1))
    with ThreadPoolExecutor(max_workers=workers) as pool:
        futures = [pool.submit(run, item) for item in commands]
        while True:
            pending = [f for f in futures if not f.done()]
            if not pending:
                break
            time.sleep(0.5)
            elapsed = time.time() - started
            if int(elapsed * 2) % 10 == 0:
                _say(f"compiling {what}: {len(done)}/{len(commands)} files done after {elapsed:.0f} s")
        for future in futures:
            future.result()


def build_library(name: str, sources: Sequence[str], defines: Sequence[str] = ()) -> str:
    """Build (or find) the shared library and return its path."""
    nvcc = find_nvcc()
    version = _nvcc_version(nvcc)
    if "-DVX_TRACE" in COMMON_FLAGS:
        name = name + "_trace"
    key = _build_key(sources, defines, version)
    out_dir = build_dir()
    target = os.path.join(out_dir, f"libvelox_{name}_{key}.so")
    if os.path.isfile(target):
        return target

    started = time.time()
    _say(f"building {os.path.basename(target)} for sm_100a with {version} (first use; cached afterwards)")
    work = tempfile.mkdtemp(prefix=f"{name}_{os.getpid()}_", dir=out_dir)
    try:
        objects = []
        commands = []
        for src in sources:
            obj = os.path.join(work, os.path.splitext(src)[0] + ".o")
            objects.append(obj)
            cmd = (
                [nvcc]
                + ARCH_FLAGS
                + COMMON_FLAGS
                + list(defines)
                + ["-Xcompiler", "-fPIC", "-I", _SRC_DIR, "-c", os.path.join(_SRC_DIR, src), "-o", obj]
            )
            commands.append((src, cmd))
        _run_with_progress(commands, name)
        partial = os.path.join(work, "lib.so")
        link = [nvcc] + ARCH_FLAGS + ["-shared", "-o", partial] + objects
        proc = subprocess.run(link, capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"link failed:\n{' '.join(link)}\n{proc.stdout}\n{proc.stderr}")
        os.replace(partial, target)
        # Older builds of the same library (other source hashes) are of no use any more.
        pattern = re.compile(re.escape(f"libvelox_{name}_") + r"[0-9a-f]{16}\.so")
        for stale in os.listdir(out_dir):
            if pattern.fullmatch(stale) and stale != os.path.basename(target):
                try:
                    os.remove(os.path.join(out_dir, stale))
                except OSError:
                    pass
    finally:
        shutil.rmtree(work, ignore_errors=True)
    _say(f"built {os.path.basename(target)} in {time.time() - started:.1f} s")
    return target


def load_core() -> ctypes.CDLL:
    return _load("core", CORE_SOURCES, ())


def load_attention(head_dim: int) -> ctypes.CDLL:
    if head_dim % 16 != 0 or not 16 <= head_dim <= 256:
        raise ValueError(
            f"head size {head_dim} is not supported by the attention kernels: "
            "it must be a multiple of 16 between 16 and 256"
        )
    return _load(f"attention_d{head_dim}", ATTENTION_SOURCES, (f"-DVX_HEAD_DIM={head_dim}",))


def _load(name: str, sources: Sequence[str], defines: Sequence[str]) -> ctypes.CDLL:
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = build_library(name, sources, defines)
            try:
                lib = ctypes.CDLL(path)
            except OSError as exc:
                raise BuildError(f"cannot load {path}: {exc}") from exc
            _loaded[name] = lib
        return lib


def build_all(head_dims: Iterable[int] = (128,)) -> List[str]:
    """Compile every library (for the given head sizes) without loading anything."""
    paths = [build_library("core", CORE_SOURCES, ())]
    for head_dim in head_dims:
        paths.append(
            build_library(f"attention_d{head_dim}", ATTENTION_SOURCES, (f"-DVX_HEAD_DIM={head_dim}",))
        )
    return paths
