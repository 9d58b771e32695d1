"""Builds the CUDA sources of this folder into one shared library for sm_100a.

``ensure_built()`` compiles what is missing or stale (a digest of sources and flags is kept
beside the library) with ``nvcc -gencode arch=compute_100a,code=sm_100a`` and returns the
library's path.  It is what the first use of a kernel calls, so a fresh checkout builds
itself; it prints a progress line per file to stderr.  No Python or torch headers are
involved: the library exports plain ``extern "C"`` functions loaded with ctypes.

    python -m clockwork_b200.csrc.build          # build now
    python -m clockwork_b200.csrc.build --ptxas  # also print registers / spills / shared memory
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor, as_completed
from pathlib import Path

CSRC = Path(__file__).resolve().parent
LIB_NAME = "libclockwork_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))


def find_nvcc() -> str:
    for env in ("CUDA_HOME", "CUDA_PATH"):
        root = os.environ.get(env)
        if root and (Path(root) / "bin" / "nvcc").is_file():
            return str(Path(root) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    if Path("/usr/local/cuda/bin/nvcc").is_file():
        return "/usr/local/cuda/bin/nvcc"
    raise RuntimeError("nvcc not found (set CUDA_HOME): the clockwork_b200 kernels cannot be built")


def _digest(extra: list[str]) -> str:
    h = hashlib.sha256()
    for p in sources() + _headers():
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + extra).encode())
    return h.hexdigest()


def build_dir() -> Path:
    """``csrc/_build`` when the tree is writable, else a per-user folder under the temp dir."""
    override = os.environ.get("CLOCKWORK_B200_BUILD_DIR")
    if override:
        d = Path(override)
        d.mkdir(parents=True, exist_ok=True)
        return d
    d = CSRC / "_build"
    try:
        d.mkdir(exist_ok=True)
        probe = d / f".w{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"clockwork_b200_build_{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _log(msg: str) -> None:
    print(f"[clockwork_b200 build] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: Path, obj: Path, extra: list[str]) -> tuple[Path, float, str]:
    t0 = time.time()
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return src, time.time() - t0, proc.stderr


def ensure_built(force: bool = False, ptxas_verbose: bool = False) -> Path:
    out_dir = build_dir()
    lib = out_dir / LIB_NAME
    stamp = out_dir / (LIB_NAME + ".digest")
    extra = ["-Xptxas", "-v"] if ptxas_verbose else []
    digest = _digest([])
    if not force and not ptxas_verbose and lib.is_file() and stamp.is_file() and stamp.read_text().strip() == digest:
        return lib
    nvcc = find_nvcc()
    srcs = sources()
    _log(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir} (first use; takes a minute or two)")
    t0 = time.time()
    objs = []
    workers = max(1, min(len(srcs), os.cpu_count() or 1, 8))
    with ThreadPoolExecutor(max_workers=workers) as pool:
        futures = []
        for src in srcs:
            obj = out_dir / (src.stem + ".o")
            objs.append(obj)
            futures.append(pool.submit(_compile_one, nvcc, src, obj, extra))
        done = 0
        for fut in as_completed(futures):
            src, secs, err = fut.result()
            done += 1
            _log(f"  [{done}/{len(srcs)}] {src.name} ({secs:.1f} s)")
            if ptxas_verbose and err:
                print(err, file=sys.stderr)
    tmp_lib = out_dir / f".{LIB_NAME}.{os.getpid()}"
    cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp_lib), *[str(o) for o in objs]]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"linking {LIB_NAME} failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp_lib, lib)
    stamp.write_text(digest)
    _log(f"built {lib.name} in {time.time() - t0:.1f} s")
    return lib


if __name__ == "__main__":
    path = ensure_built(force=True, ptxas_verbose="--ptxas" in sys.argv)
    print(path)
