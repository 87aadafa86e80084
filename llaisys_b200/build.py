"""Builds libllaisys.so (C ABI + sm_100a CUDA kernels) in-tree with g++ and nvcc.

    python llaisys_b200/build.py [--force] [--verbose] [--no-cuda]

(run it as a script: importing the package loads the library, which may not exist yet)

The result is written to llaisys_b200/libllaisys/libllaisys.so, the place the ctypes loader looks
(the reference installs its library the same way: xmake.lua:112-121 copies lib/*.so into
python/llaisys/libllaisys/). xmake is the reference's build tool; `xmake.lua` and `xmake/nvidia.lua` at the
repository root describe the same targets for it, and this script is the path that is exercised where xmake
is not installed. Objects are cached under build/ and rebuilt when a source or any header is newer.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OUT = PKG / "libllaisys" / "libllaisys.so"
OBJ_DIR = ROOT / "build" / "obj"

# sm_100a only: the explicit -gencode form emits no generic compute_100 PTX, which would reject tcgen05.
GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]
CXXFLAGS = ["-std=c++17", "-O3", "-fPIC", "-Wall", "-Werror", "-fvisibility=hidden", "-fopenmp"]
NVCCFLAGS = ["-std=c++17", "-O3", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler",
             "-fPIC,-Wall,-fvisibility=hidden,-fopenmp"]


def find_nvcc() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if cand and Path(cand).exists() else None


def sources(with_cuda: bool) -> list[Path]:
    files = sorted(CSRC.rglob("*.cpp")) + sorted(CSRC.rglob("*.cc"))
    if with_cuda:
        files += sorted(CSRC.rglob("*.cu"))
    return files


def newest_header() -> float:
    hdrs = list(CSRC.rglob("*.hpp")) + list(CSRC.rglob("*.cuh")) + list((ROOT / "include").rglob("*.h"))
    return max(p.stat().st_mtime for p in hdrs)


def compile_one(src: Path, obj: Path, nvcc: str | None, with_cuda: bool, verbose: bool, ptxas_v: bool) -> str:
    inc = ["-I", str(ROOT / "include"), "-I", str(CSRC)]
    defs = ["-DENABLE_NVIDIA_API"] if with_cuda else []
    if src.suffix == ".cu":
        cmd = [nvcc, *GENCODE, *NVCCFLAGS, *(["-Xptxas", "-v"] if ptxas_v else []), *defs, *inc, "-c", str(src),
               "-o", str(obj)]
    else:
        cmd = ["g++", *CXXFLAGS, *defs, *inc, "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compiling {src.relative_to(ROOT)} failed:\n{res.stdout}\n{res.stderr}")
    return res.stderr if ptxas_v else ""


def build(force: bool = False, verbose: bool = False, with_cuda: bool = True, ptxas_v: bool = False) -> Path:
    nvcc = find_nvcc()
    if with_cuda and nvcc is None:
        raise RuntimeError("nvcc not found: the NVIDIA backend cannot be built (set NVCC or pass --no-cuda)")
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    OUT.parent.mkdir(parents=True, exist_ok=True)
    hdr_time = newest_header()
    tag = "cuda" if with_cuda else "cpu"
    jobs, objs = [], []
    for src in sources(with_cuda):
        obj = OBJ_DIR / (tag + "__" + "__".join(src.relative_to(CSRC).parts) + ".o")
        objs.append(obj)
        stale = force or ptxas_v or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time)
        if stale:
            jobs.append((src, obj))
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        logs = list(pool.map(lambda j: compile_one(j[0], j[1], nvcc, with_cuda, verbose, ptxas_v), jobs))
    if ptxas_v:
        print("\n".join(l for l in logs if l))
    marker = OUT.with_suffix(".kind")
    relink = bool(jobs) or not OUT.exists() or not marker.exists() or marker.read_text() != tag
    if relink:
        if with_cuda:
            # nvcc links the static CUDA runtime, so the library needs only the driver at run time and loads
            # (reporting zero devices) on a machine without one.
            cmd = [nvcc, *GENCODE, "-shared", "-o", str(OUT), *map(str, objs), "-Xcompiler", "-fopenmp",
                   "-Xlinker", "--no-undefined", "-ldl"]
        else:
            cmd = ["g++", "-shared", "-fopenmp", "-o", str(OUT), *map(str, objs), "-Wl,--no-undefined", "-ldl"]
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"linking failed:\n{res.stdout}\n{res.stderr}")
        marker.write_text(tag)
    return OUT


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--force", action="store_true", help="recompile everything")
    ap.add_argument("--verbose", action="store_true", help="print compiler commands")
    ap.add_argument("--no-cuda", action="store_true", help="CPU-only library (NVIDIA reports zero devices)")
    ap.add_argument("--ptxas-v", action="store_true", help="recompile .cu files with -Xptxas -v and print the log")
    args = ap.parse_args()
    out = build(args.force, args.verbose, not args.no_cuda, args.ptxas_v)
    print(out)


if __name__ == "__main__":
    sys.exit(main())
