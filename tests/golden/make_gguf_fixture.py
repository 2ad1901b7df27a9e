#!/usr/bin/env python3
"""Regenerate tests/golden/iq_fixture.gguf: a small real-format GGUF of already-QUANTIZED routed-expert tensors (layer 0
Q4_K, 1 IQ2_S, 2 IQ3_S, 3 Q8_0; 2 experts of hidden 512 / FFN 256), written by the reference's own fixture tool
tools/iq_fixture.py (random valid blocks covering the whole code space; byte-deterministic for a given seed), with its
manifest of tensor hashes.  Run where the reference tree is mounted:

    python tests/golden/make_gguf_fixture.py

tests/test_gguf_quantized.py pushes the file through project_maya_b200/gguf_loader.py and the kernels.
"""
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
from oracle.build import REFERENCE  # noqa: E402

if __name__ == "__main__":
    tool = REFERENCE / "tools" / "iq_fixture.py"
    subprocess.run([sys.executable, str(tool), "--out", str(HERE / "iq_fixture.gguf"), "--types", "Q4_K,IQ2_S,IQ3_S,Q8_0",
                    "--n-embd", "512", "--n-ff", "256", "--n-expert", "2", "--seed", "1", "--check"], check=True)
