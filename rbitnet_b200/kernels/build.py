"""Builds the CUDA sources under ``rbitnet_b200/csrc`` into one shared library for sm_100a.

The library is built with nvcc at the first call that needs it and is found
again by a hash of the sources and flags.  It is placed beside the sources
(``csrc/_build``) when that folder can be written, else in a per-user folder
under the system's temporary directory, so a fresh checkout works for any user
and with an empty HOME.  While nvcc runs, a line is printed to stderr now and
then.
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
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fvisibility=hidden"]


def _flags():
    """The compile flags; RBITNET_CHECKED=1 in the environment adds -DRB_CHECKED (cache addresses are
    checked before use and a bad one is recorded instead of used), which makes another library."""
    extra = ["-DRB_CHECKED"] if os.environ.get("RBITNET_CHECKED", "") in ("1", "true", "yes") else []
    extra += os.environ.get("RBITNET_NVCC_EXTRA", "").split()       # further flags, for experiments
    return NVCC_FLAGS + extra


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("RBITNET_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise BuildError("nvcc not found (looked at $RBITNET_NVCC, PATH and /usr/local/cuda/bin): "
                     "the CUDA kernels cannot be built, and there is no other path")


def sources():
    return sorted(CSRC.glob("*.cu"))


def _key() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(ARCH_FLAGS + _flags()).encode())
    return h.hexdigest()[:16]


def _build_dirs():
    yield CSRC / "_build"
    uid = os.getuid() if hasattr(os, "getuid") else 0
    yield Path(tempfile.gettempdir()) / f"rbitnet_b200_build_{uid}"


def _writable(d: Path) -> bool:
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def _log(msg: str) -> None:
    print(f"[rbitnet_b200] {msg}", file=sys.stderr, flush=True)


def _run(cmd, what):
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise BuildError(f"nvcc failed on {what}:\n{' '.join(map(str, cmd))}\n{p.stdout}\n{p.stderr}")
    return p.stdout + p.stderr


def library_path(verbose: bool = True, ptxas_info: bool = False) -> Path:
    """Path of the built library; builds it first if no build of these sources exists."""
    key = _key()
    name = f"librbitnet_b200_{key}.so"
    for d in _build_dirs():
        if (d / name).is_file():
            try:
                os.utime(d / name)             # in use: the clean-up below removes the builds not used longest
            except OSError:
                pass
            return d / name
    out_dir = next((d for d in _build_dirs() if _writable(d)), None)
    if out_dir is None:
        raise BuildError("no writable folder for the kernel build (tried "
                         + ", ".join(str(d) for d in _build_dirs()) + ")")
    nvcc = _nvcc()
    srcs = sources()
    if verbose:
        _log(f"building {len(srcs)} CUDA sources for sm_100a into {out_dir} (first call only)")
    t0 = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _log(f"... still compiling ({time.time() - t0:.0f} s)")

    hb = threading.Thread(target=heartbeat, daemon=True)
    if verbose:
        hb.start()
    work = out_dir / f"obj_{key}_{os.getpid()}"
    work.mkdir(parents=True, exist_ok=True)
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    try:
        def compile_one(src: Path):
            obj = work / (src.stem + ".o")
            log = _run([nvcc, *ARCH_FLAGS, *_flags(), *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)],
                       src.name)
            if verbose:
                _log(f"compiled {src.name} ({time.time() - t0:.0f} s)")
            if ptxas_info:
                (out_dir / f"ptxas_{src.stem}.txt").write_text(log)
            return obj

        with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
            objs = list(ex.map(compile_one, srcs))
        tmp = out_dir / f".{name}.{os.getpid()}.tmp"
        _run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objs)], "link")
        os.replace(tmp, out_dir / name)
        keep = {name}
        for old in sorted(out_dir.glob("librbitnet_b200_*.so"), key=lambda p: p.stat().st_mtime, reverse=True):
            if old.name in keep:
                continue
            if len(keep) < 3:          # the builds used last stay: the plain and the checked library live side by side
                keep.add(old.name)
                continue
            try:
                old.unlink()
            except OSError:
                pass
    finally:
        done.set()
        shutil.rmtree(work, ignore_errors=True)
    if verbose:
        _log(f"built {name} in {time.time() - t0:.0f} s")
    return out_dir / name


if __name__ == "__main__":
    print(library_path(ptxas_info="--ptxas-info" in sys.argv))
