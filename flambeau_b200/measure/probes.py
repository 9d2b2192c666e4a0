"""Small stand-alone device programs that measure one thing about the hardware the kernels are laid out by.

Each lives under csrc/probes as a program of its own (a main(), no library entry point), is compiled into the build
folder on demand with the flags of the kernel library, and prints a table.  `flambeau bench --only mma-issue` runs
mma_issue_rate: cycles per tcgen05.mma of one SM's tensor pipe for the instruction shapes of the attention kernel,
and what commits and mbarrier waits in the issuing thread's stream add.
"""
from __future__ import annotations

import subprocess

from ..kernels import build

PROBES = build.CSRC / "probes"


def build_probe(name: str):
    """Compiles csrc/probes/<name>.cu for sm_100a into the build folder (if its binary is older than the source or
    the shared headers) and returns the program's path."""
    src = PROBES / f"{name}.cu"
    if not src.is_file():
        raise build.BuildError(f"no probe '{name}' under {PROBES}")
    exe = build.build_dir() / name
    newest = max(p.stat().st_mtime for p in [src, *build.CSRC.glob("*.cuh")])
    if not exe.is_file() or exe.stat().st_mtime < newest:
        flags = [f for f in build.NVCC_FLAGS if f not in ("-Xcompiler", "-fPIC", "-fvisibility=hidden")]
        build._run_with_heartbeat([build.find_nvcc(), *flags, "-I", str(build.CSRC), "-o", str(exe), str(src)],
                                  src.name)
    return exe


def probe_names() -> list:
    return sorted(p.stem for p in PROBES.glob("*.cu"))


def run_probe(name: str) -> str:
    """Builds the probe if need be, runs it and returns what it prints."""
    exe = build_probe(name)
    done = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    if done.returncode != 0:
        raise RuntimeError(f"probe {name} failed: {done.stderr.strip() or done.stdout.strip()}")
    return done.stdout
