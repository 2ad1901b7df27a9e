"""Where a tile of the prompt-path grouped GEMM spends its cycles.

    python -m project_maya_b200.build --stamps        # libmaya_moe_stamps.so: the library with -DMAYA_MMQ_STAMPS
    python -m project_maya_b200.mmq_tile_phases       # one C4 prompt-path layer (4096 tokens, 256 experts), needs a B200

The stamped library's mmq_kernel writes clock64() at its phase boundaries for the first 4096 tiles of each of its four
kinds of launch; this script runs a few layers with it and prints the mean cycles of each phase.  The product library
is built without the stamps.
"""
from __future__ import annotations

import ctypes
import os
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
PHASES = [(1, "set-up (tile scan, barriers, tensor-memory allocation)"), (2, "to the first product"), (3, "K loop"),
          (4, "drain, expanding warps meet"), (5, "tensor memory -> SwiGLU -> shared memory"),
          (6, "q8_1 rounding of the tile"), (7, "bulk stores (down: + tensor memory -> shared memory)")]
KINDS = ["Q8_0 / IQ2_S down", "Q8_0 / IQ2_S gate/up", "Q4_K / IQ3_S down", "Q4_K / IQ3_S gate/up"]


def main() -> None:
    lib_path = PKG / "libmaya_moe_stamps.so"
    if not lib_path.exists():
        sys.exit("build it first: python -m project_maya_b200.build --stamps")
    os.environ["MAYA_MOE_LIB"] = str(lib_path)
    sys.path.insert(0, str(PKG.parent))
    import numpy as np
    import torch

    import bench_prefill
    from project_maya_b200 import _lib

    line = bench_prefill.run(2, 2, 1)
    torch.cuda.synchronize()
    lib = _lib.load()
    buf = np.zeros(4 * 4096 * 16, dtype=np.int64)
    lib.maya_mmq_stamps_read.argtypes = [ctypes.c_void_p]
    assert lib.maya_mmq_stamps_read(buf.ctypes.data) == 0
    d = buf.reshape(4, 4096, 16)
    print(f"{line['config']['workload']}: {line['ms_per_step']:.3f} ms a layer with the stamped library")
    for k, name in enumerate(KINDS):
        a = d[k][d[k][:, 7] > 0]
        if len(a) == 0:
            continue
        pairs = int(a[0, 15])
        print(f"{name}: {len(a)} tiles, {a[:, 14].mean():.1f} rows, {pairs} K-step pairs, {(a[:, 7] - a[:, 0]).mean():.0f} cycles a tile")
        prev = 0
        for i, label in PHASES:
            if (a[:, i] == 0).all():
                continue
            v = a[:, i] - a[:, prev]
            extra = f"  ({v.mean() / pairs:.0f} a pair)" if i == 3 else ""
            print(f"    {label:58s} {v.mean():9.0f}   p10 {np.percentile(v, 10):8.0f}  p90 {np.percentile(v, 90):8.0f}{extra}")
            prev = i


if __name__ == "__main__":
    main()
