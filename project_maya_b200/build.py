"""Build the CUDA library in-tree: project_maya_b200/libmaya_moe.so (sm_100a only).

    python -m project_maya_b200.build [--force] [--verbose]

Steps: generate the IQ codebook include from the installed gguf package, compile every csrc/*.cu with nvcc
(-gencode arch=compute_100a,code=sm_100a -lineinfo), link one shared library with the C ABI of include/maya_moe.h.
Objects are rebuilt only when a source or header is newer.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libmaya_moe.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fopenmp,-fvisibility=hidden",
    "-I", str(ROOT / "include"), "-I", str(CSRC),
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return exe


def _newest(paths) -> float:
    return max(p.stat().st_mtime for p in paths)


def generate_grids() -> Path:
    sys.path.insert(0, str(CSRC))
    try:
        import gen_iq_grids
    finally:
        sys.path.pop(0)
    dst = CSRC / "generated" / "maya_iq_grids.inc"
    dst.parent.mkdir(parents=True, exist_ok=True)
    text = gen_iq_grids.render()
    if not dst.exists() or dst.read_text() != text:
        dst.write_text(text)
    return dst


def build(force: bool = False, verbose: bool = False, extra_flags: list[str] | None = None, stamps: bool = False) -> Path:
    """stamps: a second library, libmaya_moe_stamps.so, whose grouped GEMM records clock stamps of its tiles' phases
    (-DMAYA_MMQ_STAMPS; read by mmq_tile_phases.py).  The product library is built without them."""
    generate_grids()
    global OBJ, LIB
    if stamps:
        OBJ, LIB = PKG / "build_stamps", PKG / "libmaya_moe_stamps.so"
        extra_flags = (extra_flags or []) + ["-DMAYA_MMQ_STAMPS"]
    else:
        OBJ, LIB = PKG / "build", PKG / "libmaya_moe.so"
    OBJ.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = list(CSRC.glob("*.cuh")) + list((CSRC / "generated").glob("*.inc")) + list((ROOT / "include").glob("*.h"))
    hdr_time = _newest(headers)
    flags = NVCC_FLAGS + (extra_flags or [])
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc(), *flags, "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for src, r in ex.map(compile_one, jobs):
                if verbose or r.returncode != 0:
                    sys.stderr.write(f"[nvcc] {src.name}\n{r.stdout}{r.stderr}")
                if r.returncode != 0:
                    raise RuntimeError(f"nvcc failed on {src.name}")
    objs = [OBJ / (s.stem + ".o") for s in sources]
    if force or jobs or not LIB.exists() or LIB.stat().st_mtime < _newest(objs):
        cmd = [nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-Xcompiler", "-fopenmp", "-lgomp"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-v", action="store_true", help="print registers / spills / shared memory per kernel")
    ap.add_argument("--stamps", action="store_true", help="build libmaya_moe_stamps.so (tile-phase clock stamps in the grouped GEMM)")
    a = ap.parse_args()
    extra = ["-Xptxas", "-v"] if a.ptxas_v else None
    lib = build(force=a.force or a.ptxas_v, verbose=a.verbose or a.ptxas_v, extra_flags=extra, stamps=a.stamps)
    print(lib)


if __name__ == "__main__":
    main()
