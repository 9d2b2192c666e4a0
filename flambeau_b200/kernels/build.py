"""Compiles the CUDA sources under `csrc/` for sm_100a into one shared library.

The library is built on first use and rebuilt when a source changes (the key
is a hash of the sources and the flags).  It is written next to the package
(`flambeau_b200/_build/`); if that folder cannot be written, to a per-user
folder under the system's temporary directory.  Nothing is read from or
written to the home directory.
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

PACKAGE_DIR = Path(__file__).resolve().parent.parent
CSRC = PACKAGE_DIR / "csrc"
LIB_NAME = "libflambeau_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("FLAMBEAU_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $FLAMBEAU_NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin); "
                     "the CUDA kernels of flambeau_b200 cannot be compiled")


def sources() -> list[Path]:
    """The CUDA kernels (.cu) and the host-side C++ of the cache manager (.cpp, compiled by nvcc's host compiler)."""
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def source_key() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _writable_dir(path: Path) -> bool:
    try:
        path.mkdir(parents=True, exist_ok=True)
        probe = path / f".probe-{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    override = os.environ.get("FLAMBEAU_BUILD_DIR")
    if override:
        p = Path(override)
        if not _writable_dir(p):
            raise BuildError(f"FLAMBEAU_BUILD_DIR={override} cannot be written")
        return p
    in_tree = PACKAGE_DIR / "_build"
    if _writable_dir(in_tree):
        return in_tree
    p = Path(tempfile.gettempdir()) / f"flambeau_b200-build-{os.getuid()}"
    if not _writable_dir(p):
        raise BuildError(f"neither {in_tree} nor {p} can be written; set FLAMBEAU_BUILD_DIR")
    return p


def _say(msg: str) -> None:
    print(f"[flambeau_b200 build] {msg}", file=sys.stderr, flush=True)


def _run_with_heartbeat(cmd: list[str], what: str) -> None:
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def beat():
        t0 = time.time()
        while not done.wait(10.0):
            _say(f"still compiling {what} ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=beat, daemon=True)
    th.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {what}:\n{' '.join(cmd)}\n{out}")
    noisy = [ln for ln in out.splitlines() if ln.strip()]
    if noisy and os.environ.get("FLAMBEAU_BUILD_VERBOSE"):
        _say("\n".join(noisy))


def ensure_built(verbose: bool = True, extra_flags: list[str] | None = None) -> Path:
    """Path of an up-to-date shared library; compiles what is stale."""
    key = source_key()
    bdir = build_dir()
    lib = bdir / LIB_NAME
    stamp = bdir / (LIB_NAME + ".key")
    if lib.is_file() and stamp.is_file() and stamp.read_text().strip() == key:
        return lib
    nvcc = find_nvcc()
    srcs = sources()
    if not srcs:
        raise BuildError(f"no CUDA sources under {CSRC}")
    if verbose:
        _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {lib} (first use or sources changed)")
    obj_dir = bdir / f"obj-{key}"
    obj_dir.mkdir(parents=True, exist_ok=True)
    flags = NVCC_FLAGS + (extra_flags or [])
    t0 = time.time()

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        if not obj.is_file():
            tmp = obj_dir / f"{src.stem}.{os.getpid()}.tmp.o"
            _run_with_heartbeat([nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(tmp)], src.name)
            os.replace(tmp, obj)
            if verbose:
                _say(f"compiled {src.name} ({time.time() - t0:.0f} s)")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs), os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, srcs))
    tmp_lib = bdir / f"{LIB_NAME}.{os.getpid()}.tmp"
    _run_with_heartbeat([nvcc, "-shared", "-o", str(tmp_lib), *map(str, objs)], "link")
    os.replace(tmp_lib, lib)
    stamp.write_text(key)
    for old in bdir.glob("obj-*"):
        if old != obj_dir:
            shutil.rmtree(old, ignore_errors=True)
    if verbose:
        _say(f"built {lib.name} in {time.time() - t0:.0f} s")
    return lib


if __name__ == "__main__":
    print(ensure_built())
