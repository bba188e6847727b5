"""Compiles the CUDA sources under ``csrc/`` for sm_100a with nvcc and loads the result.

The kernels are plain ``extern "C"`` entry points in one shared library, called through
ctypes with raw device pointers: no Python headers are involved, so a build takes
seconds per file.  A library is named after a hash of its sources and flags and kept
in ``csrc/_build`` (or, when the package folder is read-only, in a per-user folder
under the system's temporary directory), so the first call in a fresh checkout
compiles and later calls only load.  While compiling it reports progress on stderr.
There is no fallback: if nvcc or a source is missing, or a compile fails, the error
is raised.
"""

from __future__ import annotations

import ctypes
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

CSRC = Path(__file__).resolve().parent.parent / "csrc"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

#: sources of the core library; further modules (built per head size) name their own
CORE_SOURCES = ["elementwise.cu", "attention_generic.cu", "sampling.cu", "skinny_gemm.cu", "gemm_simt.cu", "gemm_tcgen05_decode.cu", "gemm_tcgen05_pair.cu"]
#: the tensor-core attention, built once per head size (-DDFI_HEAD_DIM=...)
ATTENTION_SOURCES = ["attention_mma.cu", "attention_tcgen05.cu"]
#: head sizes compiled ahead by ``all_libraries`` (others compile at first use)
PREBUILT_HEAD_DIMS = (16, 32, 64, 128)
#: host-only code (no CUDA calls, not linked against the driver): the safetensors reader
IO_SOURCES = ["safetensors_reader.cpp"]
#: host-only: the decode attention's plan by the kernels' own function, for tests without a device
PLAN_SOURCES = ["decode_plan_host.cpp"]


class BuildError(RuntimeError):
    pass


def _say(message: str) -> None:
    print(f"[dryft-flash-infer_b200] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for candidate in (os.environ.get("DFI_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).is_file():
            return candidate
    raise BuildError("nvcc not found (looked at $DFI_NVCC, PATH and /usr/local/cuda/bin): "
                     "the CUDA kernels cannot be compiled and there is no fallback")


def build_dir() -> Path:
    override = os.environ.get("DFI_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates.append(CSRC / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"dryft_flash_infer_b200_build_{os.getuid()}")
    for folder in candidates:
        try:
            folder.mkdir(parents=True, exist_ok=True)
            probe = folder / f".probe_{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return folder
        except OSError:
            continue
    raise BuildError("no writable folder for compiled kernels; set DFI_BUILD_DIR")


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))


def _host_only(sources: list[str]) -> bool:
    return all(s.endswith(".cpp") for s in sources)


def _digest(sources: list[str], defines: list[str]) -> str:
    h = hashlib.sha256()
    for path in [CSRC / s for s in sources] + (sorted(CSRC.glob("*.h")) if _host_only(sources) else _headers()):
        if not path.is_file():
            raise BuildError(f"kernel source missing: {path}")
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(ARCH_FLAGS + COMMON_FLAGS + defines).encode())
    return h.hexdigest()[:16]


def library_file(name: str, sources: list[str], defines: list[str]) -> Path:
    return build_dir() / f"{name}_{_digest(sources, defines)}.so"


def compile_library(name: str, sources: list[str], defines: list[str] | None = None) -> Path:
    """Builds (if not built yet) and returns the shared library of ``sources``."""
    defines = list(defines or [])
    target = library_file(name, sources, defines)
    if target.is_file():
        return target
    nvcc = find_nvcc()
    work = Path(tempfile.mkdtemp(prefix=f"{name}_", dir=target.parent))
    started = time.time()
    what = "C++ source files" if _host_only(sources) else "CUDA source files for sm_100a"
    _say(f"compiling {len(sources)} {what} ({name}); this happens once")
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _say(f"  ... still compiling {name} ({time.time() - started:.0f} s)")

    threading.Thread(target=ticker, daemon=True).start()

    def one(source: str) -> Path:
        obj = work / (Path(source).stem + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *COMMON_FLAGS, *defines, "-I", str(CSRC), "-c", str(CSRC / source), "-o", str(obj)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"nvcc failed on {source}:\n{proc.stdout}\n{proc.stderr}")
        _say(f"  compiled {source} ({time.time() - started:.0f} s)")
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(len(sources), os.cpu_count() or 1)) as pool:
            objects = list(pool.map(one, sources))
        partial = work / "out.so"
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(partial), *map(str, objects)]
        if not _host_only(sources):
            cmd.append("-lcuda")
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"linking {name} failed:\n{proc.stdout}\n{proc.stderr}")
        os.replace(partial, target)  # atomic: a concurrent builder ends with the same file
    finally:
        done.set()
        shutil.rmtree(work, ignore_errors=True)
    _say(f"built {target.name} in {time.time() - started:.0f} s")
    return target


def all_libraries() -> list[tuple[str, list[str], list[str]]]:
    """Every library the package can load: ``(name, sources, defines)``."""
    out = [("dfi_io", IO_SOURCES, []), ("dfi_plan", PLAN_SOURCES, []), ("dfi_core", CORE_SOURCES, [])]
    for dim in PREBUILT_HEAD_DIMS:
        out.append((f"dfi_attention_d{dim}", ATTENTION_SOURCES, [f"-DDFI_HEAD_DIM={dim}"]))
    return out


_LOADED: dict[str, ctypes.CDLL] = {}


def load_library(name: str, sources: list[str], defines: list[str] | None = None) -> ctypes.CDLL:
    key = name + "|" + " ".join(defines or [])
    if key not in _LOADED:
        _LOADED[key] = ctypes.CDLL(str(compile_library(name, sources, defines)))
    return _LOADED[key]
