"""Compile the CUDA sources of this folder into one shared library for sm_100a.

Each ``.cu`` file is compiled to an object on its own (several at a time) and
the objects are linked into ``libprelude_b200.so``.  Objects are reused while
the hash of their source and of the shared headers is unchanged.  The library
lands in ``_build/`` beside the sources; when that folder cannot be written it
lands in a per-user folder under the system's temporary directory.

No source includes a torch header: the interface is plain C (raw device
pointers, sizes, a stream), so a file compiles in seconds.

Run ``python -m prelude_b200.csrc.build`` to build ahead of time.
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
from typing import List, Optional

SRC_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libprelude_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr"]
# PRELUDE_TIMELINE=1 compiles the kernels' timeline marks in (see common.cuh): another set of objects, another library
if os.environ.get("PRELUDE_TIMELINE", "0") == "1":
    NVCC_FLAGS = NVCC_FLAGS + ["-DPB_TIMELINE"]
    LIB_NAME = "libprelude_b200_timeline.so"
OBJ_PREFIX = "tl__" if LIB_NAME != "libprelude_b200.so" else ""


def _say(msg: str) -> None:
    print(f"[prelude_b200.build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("PRELUDE_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise RuntimeError("nvcc not found: set PRELUDE_NVCC or CUDA_HOME; the CUDA kernels cannot be built without it")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(SRC_DIR) if f.endswith(".cu"))


def headers() -> List[str]:
    return sorted(f for f in os.listdir(SRC_DIR) if f.endswith((".cuh", ".h")))


def _sha(paths: List[str], extra: str = "") -> str:
    h = hashlib.sha256()
    h.update(extra.encode())
    for p in paths:
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:20]


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe_{os.getpid()}")
        with open(probe, "w") as f:
            f.write("x")
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    override = os.environ.get("PRELUDE_BUILD_DIR")
    if override:
        os.makedirs(override, exist_ok=True)
        return override
    local = os.path.join(SRC_DIR, "_build")
    if _writable_dir(local):
        return local
    fallback = os.path.join(tempfile.gettempdir(), f"prelude_b200_build_{os.getuid()}")
    if _writable_dir(fallback):
        return fallback
    raise RuntimeError(f"neither {local} nor {fallback} can be written: set PRELUDE_BUILD_DIR")


def source_hash() -> str:
    files = [os.path.join(SRC_DIR, f) for f in sources() + headers()]
    return _sha(files, " ".join(ARCH_FLAGS + NVCC_FLAGS))


def _compile_one(nvcc: str, src: str, obj: str, verbose: bool) -> float:
    t0 = time.time()
    cmd = [nvcc] + ARCH_FLAGS + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-I", SRC_DIR, "-c", src, "-o", obj]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed on {os.path.basename(src)}:\n{proc.stdout}\n{proc.stderr}")
    if verbose and proc.stderr:
        sys.stderr.write(proc.stderr)
    return time.time() - t0


def existing_library() -> Optional[str]:
    """Path of an up-to-date library, or None."""
    want = source_hash()
    for d in (os.environ.get("PRELUDE_BUILD_DIR"), os.path.join(SRC_DIR, "_build"),
              os.path.join(tempfile.gettempdir(), f"prelude_b200_build_{os.getuid()}")):
        if not d:
            continue
        stamp, lib = os.path.join(d, LIB_NAME + ".json"), os.path.join(d, LIB_NAME)
        try:
            with open(stamp) as f:
                if json.load(f).get("hash") == want and os.path.isfile(lib):
                    return lib
        except (OSError, ValueError):
            pass
    return None


def build(force: bool = False, verbose: bool = False) -> str:
    """Build the library if it is missing or stale; returns its path."""
    if not force:
        lib = existing_library()
        if lib:
            return lib
    nvcc = find_nvcc()
    out = build_dir()
    hdr_paths = [os.path.join(SRC_DIR, f) for f in headers()]
    flags_key = " ".join(ARCH_FLAGS + NVCC_FLAGS)
    jobs = []
    objs = []
    for name in sources():
        src = os.path.join(SRC_DIR, name)
        key = _sha([src] + hdr_paths, flags_key)
        obj = os.path.join(out, f"{OBJ_PREFIX}{name[:-3]}.{key}.o")
        objs.append(obj)
        if force or not os.path.isfile(obj):
            jobs.append((name, src, obj))
    if jobs:
        _say(f"compiling {len(jobs)} CUDA source file(s) for sm_100a with {nvcc} into {out}")
    t0 = time.time()
    workers = max(1, min(len(jobs), os.cpu_count() or 2, 8))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as pool:
            futs = {pool.submit(_compile_one, nvcc, src, obj + ".tmp.o", verbose): (name, obj) for name, src, obj in jobs}
            for fut in concurrent.futures.as_completed(futs):
                name, obj = futs[fut]
                secs = fut.result()
                os.replace(obj + ".tmp.o", obj)
                _say(f"  {name} done in {secs:.1f} s ({time.time() - t0:.0f} s since start)")
    lib = os.path.join(out, LIB_NAME)
    tmp = lib + f".tmp{os.getpid()}"
    cmd = [nvcc] + ARCH_FLAGS + ["-shared", "-Xcompiler", "-fPIC", "-o", tmp] + objs
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"linking {LIB_NAME} failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, lib)
    with open(os.path.join(out, LIB_NAME + ".json"), "w") as f:
        json.dump({"hash": source_hash(), "sources": sources(), "built": time.time()}, f)
    # drop objects of older source versions
    keep = {os.path.basename(o) for o in objs}
    for f in os.listdir(out):
        if f.endswith(".o") and f not in keep and f.startswith("tl__") == bool(OBJ_PREFIX):
            try:
                os.remove(os.path.join(out, f))
            except OSError:
                pass
    if jobs:
        _say(f"built {lib} in {time.time() - t0:.0f} s")
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
