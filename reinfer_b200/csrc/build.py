"""Building the kernel library: nvcc straight from the `.cu` files of this folder
into one shared library, at the first call that needs it.

The scheme is the reference's JIT cache (crates/jit/src/key.rs:31-57,
cache.rs:49-131, lock.rs:1-60, meta.rs:13-30) with one library in place of many
cubins: the key is the sha256 over the length-prefixed sources and headers, the
flags in their order, the compiler's version line and the architecture; the
artefact is written under a temporary name and renamed; a `.meta.json` written
after it is the commit point; a per-key `flock` with a second look under the lock
makes concurrent processes compile once.  The artefacts live in `_build/` beside
the sources (so a built library travels with the tree), else in
`$REINFER_B200_CACHE`, else in a per-user folder of the temporary directory.

Only sm_100a is built: `-gencode arch=compute_100a,code=sm_100a`, no fast-math
(the reference's rule, crates/jit/src/compile.rs:33-38).
"""
from __future__ import annotations

import fcntl
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH = "sm_100a"
FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
         "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
# extra compiler flags (e.g. -DRB_TIMELINE for the kernels' phase timestamps); part of the build key
FLAGS += [f for f in os.environ.get("REINFER_B200_NVCC_FLAGS", "").split() if f]
LIB_PREFIX = "libreinfer_b200_"


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[reinfer_b200.build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("REINFER_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc not found (set REINFER_B200_NVCC); the kernels cannot be built and there is no fallback")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cuh") or f.endswith(".h"))


def _nvcc_version(nvcc: str) -> str:
    out = subprocess.run([nvcc, "--version"], capture_output=True, text=True).stdout
    return out.strip().splitlines()[-1] if out.strip() else "unknown"


def build_key(nvcc: Optional[str] = None) -> str:
    nvcc = nvcc or find_nvcc()
    h = hashlib.sha256()

    def field(b: bytes) -> None:
        h.update(len(b).to_bytes(8, "little"))
        h.update(b)

    for name in sources() + headers():
        field(name.encode())
        with open(os.path.join(HERE, name), "rb") as f:
            field(f.read())
    for fl in FLAGS:
        field(fl.encode())
    field(_nvcc_version(nvcc).encode())
    field(os.path.realpath(nvcc).encode())
    field(ARCH.encode())
    return h.hexdigest()


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe.{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def cache_dirs() -> List[str]:
    """Where a built library may be found, in order; the first writable one is where a
    new one is built."""
    out = [os.path.join(HERE, "_build")]
    env = os.environ.get("REINFER_B200_CACHE")
    if env:
        out.append(env)
    out.append(os.path.join(tempfile.gettempdir(), f"reinfer_b200_cache_{os.getuid()}"))
    return out


def _committed(dirpath: str, key: str) -> Optional[str]:
    lib = os.path.join(dirpath, f"{LIB_PREFIX}{key[:16]}.so")
    meta = lib + ".meta.json"
    if not (os.path.exists(lib) and os.path.exists(meta)):
        return None
    try:
        with open(meta) as f:
            m = json.load(f)
        if m.get("key") != key or m.get("size") != os.path.getsize(lib):
            return None
    except (OSError, ValueError):
        return None
    return lib


def _compile(nvcc: str, outdir: str, key: str, verbose: bool) -> str:
    work = tempfile.mkdtemp(prefix=f"obj_{key[:8]}_", dir=outdir)
    srcs = sources()
    t0 = time.time()
    _say(f"compiling {len(srcs)} CUDA files for {ARCH} (first call only) ...")

    def one(src: str) -> str:
        obj = os.path.join(work, src[:-3] + ".o")
        cmd = [nvcc] + FLAGS + ["-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
        t = time.time()
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        _say(f"  {src} done in {time.time() - t:.1f}s")
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
            objs = list(ex.map(one, srcs))
        tmp_lib = os.path.join(work, "lib.so")
        cmd = [nvcc, "-shared", "-o", tmp_lib] + objs + ["-lcudart", "-lcuda"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"link failed:\n{r.stdout}\n{r.stderr}")
        lib = os.path.join(outdir, f"{LIB_PREFIX}{key[:16]}.so")
        os.replace(tmp_lib, lib)
        meta = {"key": key, "size": os.path.getsize(lib), "arch": ARCH, "flags": FLAGS,
                "nvcc": _nvcc_version(nvcc), "sources": srcs}
        tmp_meta = lib + f".meta.json.{os.getpid()}"
        with open(tmp_meta, "w") as f:
            json.dump(meta, f)
        os.replace(tmp_meta, lib + ".meta.json")            # the commit point
        _say(f"built {os.path.basename(lib)} in {time.time() - t0:.1f}s")
        return lib
    finally:
        shutil.rmtree(work, ignore_errors=True)


def ensure_built(verbose: bool = True) -> str:
    """Path of the library for the present sources, building it if no cache folder has it."""
    nvcc = find_nvcc()
    key = build_key(nvcc)
    dirs = cache_dirs()
    for d in dirs:
        lib = _committed(d, key)
        if lib:
            return lib
    target = next((d for d in dirs if _writable_dir(d)), None)
    if target is None:
        raise BuildError(f"no writable folder for the kernel library among {dirs}")
    lock_path = os.path.join(target, f".{key[:16]}.lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            lib = _committed(target, key)               # second look, under the lock
            if lib:
                return lib
            return _compile(nvcc, target, key, verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


if __name__ == "__main__":
    print(ensure_built())
