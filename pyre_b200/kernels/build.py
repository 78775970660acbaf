"""Builds the CUDA sources of ``pyre_b200/csrc`` for sm_100a, one shared library per
source file, on first use.

Nothing is compiled at import.  A caller names the libraries it needs
(``ensure_built(["elementwise", "gemm_f32"])``); the ones that are missing or older than
their sources are compiled in parallel with ``nvcc`` and a progress line goes to
stderr every few seconds, so a first run in a fresh checkout shows that it is alive.
The libraries are written next to the sources (``csrc/_build``); if that folder cannot
be written, to a per-user folder under the system's temporary directory.  No file
outside those two places is touched and no home directory is needed.
"""

from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"

# library name -> source file.  Each source is self-contained (plus the headers).
LIBRARIES = {
    "elementwise": "elementwise.cu",
    "sampling": "sampling.cu",
    "attention_generic": "attention_generic.cu",
    "gemm_f32": "gemm_f32.cu",
    "attention_mma": "attention_mma.cu",
    "gemm_tc": "gemm_tc.cu",
    "attention_prefill": "attention_prefill.cu",
    "attention_tc": "attention_tc.cu",
    "attention_mma_noalloc": "attention_mma_noalloc.cu",
}

HEADERS = ["common.cuh", "attention_mma_noalloc.h"]
# sources that a library's source includes (they count towards its fingerprint)
INCLUDED_SOURCES = {"attention_mma_noalloc": ["attention_mma.cu"]}

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


# PYRE_DEBUG_CHECKS=1 in the environment selects the debug build of every library: compiled with
# -DPYRE_DEBUG_CHECKS (device-side range checks of cache pages and slots, see csrc/common.cuh) into files of
# their own (libpyre_<name>_dbg.so), so both builds can lie side by side.
DEBUG_CHECKS = os.environ.get("PYRE_DEBUG_CHECKS", "") not in ("", "0")
DEBUG_FLAGS = ["-DPYRE_DEBUG_CHECKS"]


def _flags() -> list[str]:
    return NVCC_FLAGS + (DEBUG_FLAGS if DEBUG_CHECKS else [])


def _suffix() -> str:
    return "_dbg" if DEBUG_CHECKS else ""


class BuildError(RuntimeError):
    pass


def register_library(name: str, source: str, headers: "list[str] | None" = None) -> None:
    """Add a library (name -> source file under csrc) to the build table."""
    LIBRARIES[name] = source
    for h in headers or []:
        if h not in HEADERS:
            HEADERS.append(h)


def find_nvcc() -> str:
    for cand in (os.environ.get("PYRE_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $PYRE_NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin); "
                     "the CUDA kernels of pyre_b200 cannot be built and there is no fallback")


def _writable_dir(path: Path) -> bool:
    try:
        path.mkdir(parents=True, exist_ok=True)
        probe = path / f".probe_{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return True
    except OSError:
        return False


_build_dir: Path | None = None


def build_dir() -> Path:
    global _build_dir
    if _build_dir is None:
        override = os.environ.get("PYRE_BUILD_DIR")
        if override and _writable_dir(Path(override)):
            _build_dir = Path(override)
        elif _writable_dir(CSRC / "_build"):
            _build_dir = CSRC / "_build"
        else:
            tag = hashlib.sha1(str(CSRC).encode()).hexdigest()[:10]
            fallback = Path(tempfile.gettempdir()) / f"pyre_b200_build_{os.getuid()}_{tag}"
            if not _writable_dir(fallback):
                raise BuildError(f"cannot write a build folder: tried {CSRC / '_build'} and {fallback}")
            _build_dir = fallback
    return _build_dir


def _fingerprint(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(_flags()).encode())
    for rel in [LIBRARIES[name]] + INCLUDED_SOURCES.get(name, []) + sorted(HEADERS):
        p = CSRC / rel
        h.update(rel.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def library_path(name: str) -> Path:
    return build_dir() / f"libpyre_{name}{_suffix()}.so"


def is_current(name: str) -> bool:
    so, stamp = library_path(name), build_dir() / f"{name}{_suffix()}.stamp"
    try:
        return so.is_file() and stamp.read_text() == _fingerprint(name)
    except OSError:
        return False


def _say(msg: str) -> None:
    print(f"[pyre_b200] {msg}", file=sys.stderr, flush=True)


def ensure_built(names, verbose: bool = True, extra_flags: "list[str] | None" = None) -> None:
    """Compile the named libraries that are missing or stale; return when all are current."""
    names = [n for n in dict.fromkeys(names)]
    for n in names:
        if n not in LIBRARIES:
            raise BuildError(f"unknown kernel library {n!r}; known: {sorted(LIBRARIES)}")
    todo = [n for n in names if not is_current(n)]
    if not todo:
        return
    bdir = build_dir()
    with open(bdir / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)  # another process may be building the same files
        try:
            todo = [n for n in todo if not is_current(n)]
            if not todo:
                return
            nvcc = find_nvcc()
            t0 = time.time()
            if verbose:
                _say(f"compiling {len(todo)} CUDA librar{'y' if len(todo) == 1 else 'ies'} for sm_100a"
                     f"{' with debug checks' if DEBUG_CHECKS else ''} ({', '.join(todo)}) into {bdir}")
            procs = {}
            for n in todo:
                tmp = bdir / f".libpyre_{n}{_suffix()}.{os.getpid()}.so"
                cmd = [nvcc, *_flags(), *(extra_flags or []), "-I", str(CSRC), "-o", str(tmp), str(CSRC / LIBRARIES[n])]
                # the compiler's messages go to a file: a pipe that nobody reads until the exit would block a
                # compiler that says more than the pipe holds
                log = tempfile.TemporaryFile(mode="w+", dir=bdir)
                procs[n] = (subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT), tmp, log)
            pending = dict(procs)
            last = time.time()
            while pending:
                for n in list(pending):
                    proc, tmp, log = pending[n]
                    if proc.poll() is None:
                        continue
                    log.seek(0)
                    out = log.read()
                    log.close()
                    del pending[n]
                    if proc.returncode != 0:
                        for p, _t, _l in pending.values():
                            p.kill()
                        raise BuildError(f"nvcc failed on {LIBRARIES[n]} (exit {proc.returncode}):\n{out}")
                    os.replace(tmp, library_path(n))
                    (bdir / f"{n}{_suffix()}.stamp").write_text(_fingerprint(n))
                    if verbose:
                        _say(f"  built {n} ({time.time() - t0:.0f} s)")
                if pending:
                    time.sleep(0.2)
                    if verbose and time.time() - last > 10:
                        last = time.time()
                        _say(f"  still compiling {', '.join(pending)} ({time.time() - t0:.0f} s)")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def build_all(verbose: bool = True) -> None:
    ensure_built(list(LIBRARIES), verbose=verbose)
