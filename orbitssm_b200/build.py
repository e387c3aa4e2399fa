"""Build ``liborbit_b200.so`` in-tree with nvcc for sm_100a:  ``python -m orbitssm_b200.build``.

Each ``csrc/*.cu`` is compiled to an object file under ``csrc/_obj`` (in parallel, and only when it or a header is newer
than its object), then the objects are linked into the shared library next to this file."""
from __future__ import annotations

import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
OUT = os.path.join(HERE, "liborbit_b200.so")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def headers():
    return glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        [os.path.join(os.path.dirname(HERE), "include", "orbit_b200.h")]


def _obj(src):
    return os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")


def _newer(path, deps):
    if not os.path.exists(path):
        return True
    t = os.path.getmtime(path)
    return any(os.path.getmtime(d) > t for d in deps)


def stale() -> bool:
    return _newer(OUT, sources() + headers())


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not stale():
        return OUT
    nvcc = os.environ.get("NVCC", "nvcc")
    os.makedirs(OBJ, exist_ok=True)
    hdrs = headers()
    todo = [s for s in sources() if force or _newer(_obj(s), [s] + hdrs)]

    def compile_one(src):
        cmd = [nvcc, *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", src, "-o", _obj(src)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        return src, cmd, res

    with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 1) or 1) as pool:
        for src, cmd, res in pool.map(compile_one, todo):
            if res.returncode != 0:
                raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
            if verbose:
                print(res.stderr)
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", OUT, *[_obj(s) for s in sources()]]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + " ".join(link) + "\n" + res.stdout + res.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
