"""Compile the CUDA sources of ``csrc/`` for sm_100a into one shared library.

The library is built the first time it is needed (or when a source changed),
with plain ``nvcc`` and no Python build system: every ``.cu`` file is a
translation unit without torch headers, so a full build takes well under a
minute.  Progress lines go to stderr while it runs.  The result lives in
``csrc/_build`` inside the package when that folder can be written, else in a
per-user folder under the system's temporary directory.
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
from typing import List, Optional

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_NAME = "libst_b200.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[swifttransformer_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    cands = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            cands.append(os.path.join(os.environ[var], "bin", "nvcc"))
    cands.append("/usr/local/cuda/bin/nvcc")
    which = shutil.which("nvcc")
    if which:
        cands.append(which)
    for c in cands:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc not found (looked at CUDA_HOME, /usr/local/cuda/bin and PATH); "
                     "the engine's kernels cannot be built and there is no other path")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _flags() -> List[str]:
    """NVCC_FLAGS plus what ST_B200_NVCC_EXTRA adds (e.g. -DTC_PROFILE for a kernel's timing stamps)."""
    return NVCC_FLAGS + os.environ.get("ST_B200_NVCC_EXTRA", "").split()


def _digest(nvcc: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(_flags()).encode())
    try:
        h.update(subprocess.run([nvcc, "--version"], capture_output=True, check=True).stdout)
    except Exception:
        pass
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()


def _build_dir() -> str:
    env = os.environ.get("ST_B200_BUILD_DIR")
    if env:
        os.makedirs(env, exist_ok=True)
        return env
    in_tree = os.path.join(CSRC, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"swifttransformer_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def ensure_built(verbose: bool = True) -> str:
    """Build the library if needed and return its path."""
    nvcc = find_nvcc()
    bdir = _build_dir()
    lib = os.path.join(bdir, LIB_NAME)
    stamp = os.path.join(bdir, "stamp.txt")
    want = _digest(nvcc)

    def fresh() -> bool:
        try:
            with open(stamp) as f:
                return os.path.isfile(lib) and f.read().strip() == want
        except OSError:
            return False

    if fresh():
        return lib
    with open(os.path.join(bdir, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if fresh():     # another process built it meanwhile
            return lib
        t0 = time.time()
        srcs = sources()
        if verbose:
            _log(f"compiling {len(srcs)} CUDA files for sm_100a into {bdir} (first use; takes about a minute)")
        jobs = []
        env = dict(os.environ)
        env.setdefault("TMPDIR", bdir)
        for src in srcs:
            obj = os.path.join(bdir, src[:-3] + ".o")
            cmd = [nvcc] + _flags() + ["-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
            jobs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)))
        pending = list(jobs)
        last = time.time()
        while pending:
            still = []
            for src, obj, p in pending:
                if p.poll() is None:
                    still.append((src, obj, p))
                    continue
                out = p.stdout.read().decode(errors="replace")
                if p.returncode != 0:
                    for _, _, q in jobs:
                        if q.poll() is None:
                            q.kill()
                    raise BuildError(f"nvcc failed on {src}:\n{out}")
                if verbose:
                    _log(f"  compiled {src} ({time.time() - t0:.0f}s)")
            pending = still
            if pending:
                if verbose and time.time() - last > 10:
                    _log(f"  still compiling: {', '.join(s for s, _, _ in pending)} ({time.time() - t0:.0f}s)")
                    last = time.time()
                time.sleep(0.2)
        tmp_lib = lib + f".{os.getpid()}.tmp"
        cmd = [nvcc, "-shared", "-o", tmp_lib] + [obj for _, obj, _ in jobs]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)
        if r.returncode != 0:
            raise BuildError(f"linking {LIB_NAME} failed:\n{r.stdout.decode(errors='replace')}")
        os.replace(tmp_lib, lib)
        with open(stamp, "w") as f:
            f.write(want + "\n")
        if verbose:
            _log(f"built {LIB_NAME} in {time.time() - t0:.0f}s")
    return lib
