"""Builds libgarnet_b200.so in-tree with nvcc for sm_100a: one object per source
file (compiled in parallel, rebuilt only when the source or a header is newer),
then one link."""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
LIB_PATH = os.path.join(LIB_DIR, "libgarnet_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-DGARNET_B200_BUILD",
]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _headers() -> list[str]:
    deps = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh"))
    deps.append(os.path.join(os.path.dirname(HERE), "include", "garnet_b200.h"))
    return deps


def _object_of(src: str) -> str:
    return os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")


def _newer(path: str, than: float) -> bool:
    return os.path.getmtime(path) > than


def stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(_newer(d, t) for d in sources() + _headers())


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not stale():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: libgarnet_b200.so cannot be built")
    os.makedirs(OBJ_DIR, exist_ok=True)
    env = dict(os.environ)
    # The host compiler must be the system gcc; a compiler wrapper named in CC/CXX is not used.
    env.pop("CC", None)
    env.pop("CXX", None)
    header_time = max(os.path.getmtime(h) for h in _headers())
    todo = []
    for src in sources():
        obj = _object_of(src)
        if force or not os.path.exists(obj) or _newer(src, os.path.getmtime(obj)) or header_time > os.path.getmtime(obj):
            todo.append((src, obj))

    def compile_one(pair):
        src, obj = pair
        extra = os.environ.get("GARNET_B200_NVCC_FLAGS", "").split()   # e.g. -DGB_STREAM_TRACE for a timing build
        cmd = [nvcc, *NVCC_FLAGS, *extra, *(["-Xptxas", "-v"] if verbose else []), "-c", src, "-o", obj]
        subprocess.check_call(cmd, env=env)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(todo)))) as pool:
        list(pool.map(compile_one, todo))
    wanted = {_object_of(s) for s in sources()}
    for old in glob.glob(os.path.join(OBJ_DIR, "*.o")):
        if old not in wanted:
            os.remove(old)
    subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "--shared", "-o", LIB_PATH, *sorted(wanted), "-ldl"], env=env)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose=True))
