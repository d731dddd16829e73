"""Compile the CUDA sources for sm_100a into one shared library, in place, on first use.

``nvcc`` builds every ``.cu`` file under ``csrc/`` into ``csrc/_build/`` (objects in
parallel, then one link).  The library's name carries a hash of the sources and flags, so
an edited kernel is rebuilt and a finished build is found again without compiling.  When the
package folder cannot be written, the build goes to ``$IE_B200_BUILD_DIR`` or a per-user
folder under the system's temporary directory.  Progress goes to stderr, a line per file.
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

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]

# Sources of the always-needed library.  Kernels specialised on a model's sizes are listed
# in SPECIALISED and built by `build_specialised` with -D flags.
CORE_SOURCES = ["elementwise.cu", "gemm_f32.cu", "gemm_tma.cu", "gemm_tc5.cu", "attention_generic.cu", "sampling.cu"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[inference_engine_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("IE_B200_NVCC"),
                 shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $IE_B200_NVCC, PATH, $CUDA_HOME, /usr/local/cuda); "
                     "the engine's kernels cannot be built")


_BUILD_DIR: Path | None = None


def build_dir() -> Path:
    global _BUILD_DIR
    if _BUILD_DIR is not None:
        return _BUILD_DIR
    env = os.environ.get("IE_B200_BUILD_DIR")
    candidates = [Path(env)] if env else []
    candidates.append(CSRC / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"inference_engine_b200-{os.getuid()}" / "_build")
    for d in candidates:
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".w{os.getpid()}-{threading.get_ident()}"
            probe.write_text("")
            probe.unlink(missing_ok=True)
            _BUILD_DIR = d
            return d
        except OSError:
            continue
    raise BuildError(f"no writable folder for the kernel build among {candidates}")


def _digest(sources: list[Path], defines: list[str]) -> str:
    h = hashlib.sha256()
    for extra in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(extra.name.encode())
        h.update(extra.read_bytes())
    for src in sources:
        h.update(src.name.encode())
        h.update(src.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + defines).encode())
    return h.hexdigest()[:16]


def _compile_one(nvcc: str, src: Path, obj: Path, defines: list[str]) -> None:
    t0 = time.time()
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *defines, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
    _say(f"compiled {src.name} ({time.time() - t0:.1f} s)")


def build_library(name: str, sources: list[str], defines: list[str] | None = None,
                  verbose: bool = True) -> Path:
    """Build (or find) ``lib<name>-<hash>.so`` from ``sources`` under ``csrc/``."""
    defines = list(defines or []) + os.environ.get("IE_B200_NVCC_FLAGS", "").split()
    srcs = [CSRC / s for s in sources]
    for s in srcs:
        if not s.exists():
            raise BuildError(f"kernel source {s} is missing")
    out_dir = build_dir()
    lib = out_dir / f"lib{name}-{_digest(srcs, defines)}.so"
    if lib.exists():
        return lib
    nvcc = find_nvcc()
    _say(f"building {lib.name} for sm_100a from {len(srcs)} file(s) with {nvcc} (first use only)")
    tag = f"{name}-{os.getpid()}-{threading.get_ident()}"
    objs = [out_dir / f"{tag}-{s.stem}.o" for s in srcs]
    try:
        with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 2)) as pool:
            list(pool.map(lambda so: _compile_one(nvcc, so[0], so[1], defines), zip(srcs, objs)))
        tmp = out_dir / f"{tag}.so.tmp"
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objs)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"linking {lib.name} failed:\n{proc.stdout}\n{proc.stderr}")
        os.replace(tmp, lib)  # atomic: a concurrent builder finds either nothing or all of it
    finally:
        for o in objs:
            o.unlink(missing_ok=True)
    _say(f"built {lib}")
    return lib


def build_core() -> Path:
    return build_library("ie_b200_core", CORE_SOURCES)


def build_selftest() -> Path:
    """The TMA-fed matrix products once more, as the tests' self-test library: waits give up
    after 256 polls instead of 200,000, and a switch (``ie_test_starve_tma/tc5``) makes a block
    expect a copy that is never asked for, so that a wait runs out, in a fraction of a
    millisecond, and the way out of it (report, give tensor memory back, return) can be
    tested.  Generation never loads this library."""
    return build_library("ie_b200_selftest", ["gemm_tma.cu", "gemm_tc5.cu"],
                         ["-DIE_SPIN_LIMIT=256", "-DIE_TEST_STARVE=1"])


ATTENTION_HEAD_DIMS = tuple(range(16, 129, 16))  # head sizes the tensor-core attention takes


def build_attention(head_dim: int) -> Path:
    """The bfloat16 tensor-core attention kernels for one head size (compiled on first use
    for the head size the loaded model has)."""
    if head_dim not in ATTENTION_HEAD_DIMS:
        raise BuildError(f"the tensor-core attention takes head sizes {ATTENTION_HEAD_DIMS}, not {head_dim}")
    return build_library(f"ie_b200_attn_hd{head_dim}", ["attention_mma.cu", "attention_tc5.cu"],
                         [f"-DIE_HD={head_dim}"])


def build_all(prune: bool = True) -> list[Path]:
    """Every library the package can load (the build check compiles them all).  With `prune`,
    libraries of this package in the build folder that belong to older sources are removed."""
    libs = [build_core(), build_selftest()]
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 2) as pool:
        libs += list(pool.map(build_attention, ATTENTION_HEAD_DIMS))
    if prune:
        keep = {lib.name for lib in libs}
        for old in build_dir().glob("libie_b200_*.so"):
            if old.name not in keep:
                try:
                    old.unlink()
                except OSError:
                    pass
    return libs
