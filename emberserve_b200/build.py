"""Builds the CUDA library of the package, in-tree, for sm_100a only.

``ensure_built()`` compiles every ``csrc/*.cu`` with nvcc into objects under
``csrc/_build/`` and links ``libemberserve_b200.so`` there.  It is called at the first
use of a kernel, so a fresh checkout compiles itself at its first call; a stamp of the
sources and flags makes later calls free.  Nothing depends on the home directory.  If
the tree is not writable the build goes to a per-user temporary folder instead.

There is no fallback: if nvcc is missing or a file does not compile, the error is
raised to the caller with the compiler's output.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
LIB_NAME = "libemberserve_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler",
              "-fvisibility=hidden", "--expt-relaxed-constexpr"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[emberserve_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("EMBERSERVE_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (set CUDA_HOME or EMBERSERVE_NVCC); the CUDA kernels "
                     "of emberserve_b200 cannot be built and there is no fallback")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stamp(nvcc: str) -> str:
    h = hashlib.sha256()
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    h.update(nvcc.encode())
    return h.hexdigest()


def _build_dir() -> Path:
    override = os.environ.get("EMBERSERVE_BUILD_DIR")
    if override:
        d = Path(override)
        d.mkdir(parents=True, exist_ok=True)
        return d
    d = CSRC / "_build"
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".w{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"emberserve_b200_build_{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _run(cmd: list[str], what: str) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"{what} failed:\n$ {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")


def ensure_built(verbose: bool = True, force: bool = False) -> Path:
    """Compile what is stale and return the path of the shared library."""
    nvcc = find_nvcc()
    out_dir = _build_dir()
    lib = out_dir / LIB_NAME
    stamp_file = out_dir / "stamp.json"
    stamp = _stamp(nvcc)
    if not force and lib.is_file() and stamp_file.is_file():
        try:
            if json.loads(stamp_file.read_text()).get("stamp") == stamp:
                return lib
        except (OSError, ValueError):
            pass
    srcs = sources()
    if not srcs:
        raise BuildError(f"no CUDA sources under {CSRC}")
    t0 = time.time()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir} ...")
    # Per-file stamps: only what changed is recompiled.
    header_hash = hashlib.sha256(b"".join(
        p.read_bytes() for p in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))))).hexdigest()
    flags_hash = hashlib.sha256(" ".join(ARCH_FLAGS + NVCC_FLAGS + [nvcc]).encode()).hexdigest()

    def compile_one(src: Path) -> Path:
        obj = out_dir / (src.stem + ".o")
        tag = out_dir / (src.stem + ".tag")
        want = hashlib.sha256(src.read_bytes()).hexdigest() + header_hash + flags_hash
        if not force and obj.is_file() and tag.is_file() and tag.read_text() == want:
            return obj
        t = time.time()
        _run([nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)],
             f"compiling {src.name}")
        tag.write_text(want)
        if verbose:
            _say(f"  {src.name} done in {time.time() - t:.1f} s")
        return obj

    workers = max(1, min(len(srcs), os.cpu_count() or 1))
    with concurrent.futures.ThreadPoolExecutor(workers) as pool:
        objs = list(pool.map(compile_one, srcs))
    tmp_lib = out_dir / (LIB_NAME + f".tmp{os.getpid()}")
    _run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp_lib), *map(str, objs)], "linking")
    os.replace(tmp_lib, lib)
    stamp_file.write_text(json.dumps({"stamp": stamp, "nvcc": nvcc}))
    if verbose:
        _say(f"built {lib.name} in {time.time() - t0:.1f} s")
    return lib


if __name__ == "__main__":
    print(ensure_built(force="--force" in sys.argv))
