"""Build the sm_100a kernel library with nvcc and find it again.

The kernels are plain CUDA with ``extern "C"`` launchers and no dependency on
torch's C++ headers, so the whole library compiles in well under a minute and
is loaded through ``ctypes``.  The shared object is kept in-tree, beside the
sources (``csrc/_build/``), stamped with a hash of the sources and flags; it is
rebuilt when the stamp does not match.  When the tree is not writable the
build goes to a per-user temporary folder instead.

Compare ``kernels/setup.py:37-68`` of davidjoyme/flashdecode-cuda, which builds
its two kernels for sm_120 through setuptools; this build targets
``arch=compute_100a,code=sm_100a`` only.
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
from pathlib import Path
from typing import List

CSRC = Path(__file__).resolve().parent
LIB_NAME = "libflashdecode_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def sources() -> List[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stamp() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError(
        "flashdecode_cuda_b200: nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin); "
        "the CUDA kernels cannot be built and there is no fallback")


def _build_dir() -> Path:
    d = CSRC / "_build"
    try:
        d.mkdir(exist_ok=True)
        probe = d / f".w{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"flashdecode_cuda_b200_build_{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[flashdecode_cuda_b200] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: Path, obj: Path, errors: list, verbose: bool) -> None:
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        errors.append(f"{src.name}:\n{r.stdout}\n{r.stderr}")
    elif verbose:
        sys.stderr.write(r.stderr)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``*.cu`` for sm_100a and link one shared library.
    Returns its path.  Prints a line every few seconds while it works."""
    out_dir = _build_dir()
    lib = out_dir / LIB_NAME
    stamp_file = out_dir / "stamp"
    stamp = _stamp()
    if not force and lib.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return lib
    nvcc = find_nvcc()
    srcs = sources()
    _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {out_dir} ...")
    t0 = time.time()
    errors: list = []
    threads = []
    objs = []
    for s in srcs:
        o = out_dir / (s.stem + ".o")
        objs.append(o)
        th = threading.Thread(target=_compile_one, args=(nvcc, s, o, errors, verbose))
        th.start()
        threads.append(th)
    while any(th.is_alive() for th in threads):
        for th in threads:
            th.join(timeout=5.0)
            if th.is_alive():
                break
        if any(th.is_alive() for th in threads):
            _say(f"  still compiling ({time.time() - t0:.0f} s)")
    if errors:
        raise RuntimeError("flashdecode_cuda_b200: nvcc failed\n" + "\n".join(errors))
    tmp = out_dir / (LIB_NAME + f".{os.getpid()}.tmp")
    cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"flashdecode_cuda_b200: link failed\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    stamp_file.write_text(stamp)
    _say(f"built {lib.name} in {time.time() - t0:.0f} s")
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
