"""Build libkuiops.so from the CUDA sources in this directory.

Usage: python build.py [--force] [--jobs N]

Each .cu is compiled for sm_100a only (-gencode arch=compute_100a,code=sm_100a) and linked into
``../lib/libkuiops.so``.  Objects are rebuilt when a source or header is newer than the object.
"""
import argparse
import concurrent.futures
import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
OBJ = HERE / "_obj"
LIB = HERE.parent / "lib" / "libkuiops.so"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def sources():
    return sorted(HERE.glob("*.cu"))


def headers():
    return sorted(HERE.glob("*.cuh")) + [HERE.parent.parent / "include" / "kuiops.h"]


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _compile(src: Path, verbose: bool) -> str:
    obj = OBJ / (src.stem + ".o")
    cmd = [NVCC, *FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return r.stderr


def build(force: bool = False, jobs: int = 0, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    LIB.parent.mkdir(exist_ok=True)
    hdrs = headers()
    todo = [s for s in sources() if force or _stale(OBJ / (s.stem + ".o"), [s, *hdrs])]
    if todo:
        with concurrent.futures.ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as ex:
            for log in ex.map(lambda s: _compile(s, verbose), todo):
                if verbose and log:
                    print(log)
    objs = [OBJ / (s.stem + ".o") for s in sources()]
    if todo or _stale(LIB, objs):
        cmd = [NVCC, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--jobs", type=int, default=0)
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.jobs, a.verbose))
