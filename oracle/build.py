"""Build the CPU checkers (TEST INFRASTRUCTURE - nothing the library ships depends on these).

    python oracle/build.py

  oracle/_build/libmaya_oracle.so  the C restatement (maya_oracle.c), always
  oracle/_ref/libmaya_ref.so       the reference's own CPU code for this path, compiled from the reference tree where it
                                   lies (only when that tree is present; outputs only under oracle/_ref/): the AVX-512 /
                                   AVX2 expert rows, the router test's host reference, the Q8_K quantizer transcription
  oracle/_ref/libmaya_ref_gpu.so   the reference's own CUDA expert kernels (router_top10.cu, iq_kernels.cu,
                                   native_mmvq.cu, glm_fast.cu) compiled for sm_100a behind the C ABI of ref_shim_gpu.cu:
                                   the live parity pin of the GPU tests and the bench's "GPU kernel to beat"

The reference tree is the directory MAYA_REFERENCE_TREE names, else a directory "reference" beside this repository.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
GRIDS = ROOT / "project_maya_b200" / "csrc" / "generated"
REFERENCE = Path(os.environ.get("MAYA_REFERENCE_TREE") or ROOT.parent / "reference")


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("oracle build failed")


def _stale(out: Path, deps: list[Path]) -> bool:
    return not out.exists() or out.stat().st_mtime < max(d.stat().st_mtime for d in deps)


def build_oracle() -> Path:
    sys.path.insert(0, str(ROOT))
    from project_maya_b200.build import generate_grids
    inc = generate_grids()
    out = HERE / "_build" / "libmaya_oracle.so"
    out.parent.mkdir(exist_ok=True)
    src = HERE / "maya_oracle.c"
    if _stale(out, [src, inc]):
        _run(["gcc", "-O2", "-std=gnu11", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-fvisibility=hidden",
              "-I", str(GRIDS), str(src), "-o", str(out), "-lm"])
    return out


def reference_present() -> bool:
    return (REFERENCE / "src" / "kernels" / "cpu" / "iq_avx512.cpp").exists()


def build_ref() -> Path | None:
    """Compile the reference's own CPU sources for this path (flags as its CMakeLists.txt:1610-1617 gives them)."""
    out = HERE / "_ref" / "libmaya_ref.so"
    if not reference_present():
        return out if out.exists() else None
    out.parent.mkdir(exist_ok=True)
    inc = ["-I", str(REFERENCE / "include"), "-I", str(REFERENCE / "third_party" / "ggml"), "-I", str(REFERENCE),
           "-I", "/usr/local/cuda/include"]
    common = ["g++", "-std=c++17", "-O2", "-fPIC", "-fvisibility=hidden", "-c"]
    avx512 = ["-mavx512f", "-mavx512bw", "-mavx512vl", "-mavx512dq", "-mf16c", "-mfma", "-ffp-contract=off"]
    avx2 = ["-mavx2", "-mfma", "-mf16c", "-ffp-contract=off"]
    units = [
        (REFERENCE / "src/kernels/cpu/iq_avx512.cpp", avx512),
        (REFERENCE / "src/kernels/cpu/iq_avx2.cpp", avx2),
        (HERE / "ref_shim_rows.cpp", []),
        (HERE / "ref_shim_router.cpp", []),
        (HERE / "ref_shim_q8k.cpp", []),
        (HERE / "ref_shim_layer.cpp", avx2 + ["-O3", "-pthread"]),
    ]
    objs = []
    for src, fl in units:
        obj = HERE / "_ref" / (src.stem + ".o")
        if _stale(obj, [src]):
            _run(common + fl + inc + [str(src), "-o", str(obj)])
        objs.append(obj)
    if _stale(out, objs):
        _run(["g++", "-shared", "-pthread", "-o", str(out), *map(str, objs)])
    return out


def build_ref_gpu() -> Path | None:
    """Compile the reference's CUDA expert kernels for sm_100a where they lie (no file of it is copied or changed).
    native_mmvq.cu takes --use_fast_math as in the reference's CMakeLists.txt:578-592.  glm_fast.cu takes over a minute."""
    out = HERE / "_ref" / "libmaya_ref_gpu.so"
    if not reference_present():
        return out if out.exists() else None
    out.parent.mkdir(exist_ok=True)
    nvcc = "/usr/local/cuda/bin/nvcc"
    inc = ["-I", str(REFERENCE / "include"), "-I", str(REFERENCE / "third_party" / "ggml"), "-I", str(REFERENCE / "src" / "kernels" / "cuda")]
    common = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-w", "-c"]
    cu = REFERENCE / "src" / "kernels" / "cuda"
    units = [
        (cu / "router_top10.cu", []),
        (cu / "iq_kernels.cu", []),
        (cu / "native_mmvq.cu", ["--use_fast_math"]),
        (cu / "glm_fast.cu", []),
        (HERE / "ref_shim_gpu.cu", ["-Xcompiler", "-fvisibility=hidden"]),
    ]
    import concurrent.futures as cf
    objs, jobs = [], []
    for src, fl in units:
        obj = HERE / "_ref" / ("gpu_" + src.stem + ".o")
        objs.append(obj)
        if _stale(obj, [src]):
            jobs.append(common + fl + inc + [str(src), "-o", str(obj)])
    with cf.ThreadPoolExecutor(max_workers=max(1, len(jobs))) as ex:
        list(ex.map(_run, jobs))
    if _stale(out, objs):
        _run([nvcc, "-shared", "-o", str(out), *map(str, objs)])
    return out


if __name__ == "__main__":
    print(build_oracle())
    print(build_ref())
    print(build_ref_gpu())
