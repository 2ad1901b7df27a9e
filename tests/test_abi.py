"""The C-ABI library on a machine without a GPU: it loads, exports every symbol the header declares, and its
host-only helpers (sizes, layouts, argument refusals) behave like the reference's."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

import helpers as H

ROOT = Path(__file__).resolve().parent.parent


def declared_in_headers():
    names = set()
    for h in (ROOT / "include").glob("*.h"):
        names |= set(re.findall(r"MAYA_API[^;(]*?\b(maya_[a-z0-9_]+)\s*\(", h.read_text()))
    return names


def test_library_exports_every_declared_symbol(lib):
    names = declared_in_headers()
    assert len(names) >= 20
    for n in sorted(names):
        assert hasattr(lib, n), f"{n} is declared in include/ but not exported"


def test_python_signatures_cover_the_header():
    from project_maya_b200 import _lib
    assert set(_lib.declared_symbols()) == declared_in_headers()


def test_version_and_counters(lib):
    assert b"sm_100a" in lib.maya_version()
    assert lib.maya_launch_errors() >= 0


def test_row_and_buffer_sizes(lib):
    # bytes per row at the benchmark shapes (gate/up over 6144, down over 2048)
    assert lib.maya_row_bytes(H.Q4_K, 6144) == 3456 and lib.maya_row_bytes(H.Q4_K, 2048) == 1152
    assert lib.maya_row_bytes(H.Q8_0, 6144) == 6528 and lib.maya_row_bytes(H.Q8_0, 2048) == 2176
    assert lib.maya_row_bytes(H.IQ2_S, 6144) == 1968 and lib.maya_row_bytes(H.IQ2_S, 2048) == 656
    assert lib.maya_row_bytes(H.IQ3_S, 6144) == 2640 and lib.maya_row_bytes(H.IQ3_S, 2048) == 880
    assert lib.maya_row_bytes(H.Q4_K, 100) == 0 and lib.maya_row_bytes(7, 256) == 0
    assert lib.maya_q8_1_bytes(6144, 1) == 6912 and lib.maya_q8_1_bytes(6144, 8) == 8 * 6912
    assert lib.maya_q8_1_bytes(100, 1) == 0
    assert lib.maya_weight_bytes(H.IQ2_S, 6144, 2048) == 1968 * 2048
    for t in (H.Q8_0, H.Q4_K, H.IQ2_S, H.IQ3_S):
        assert lib.maya_type_supported(t) == 1
    assert lib.maya_type_supported(2) == 0


@pytest.mark.parametrize("name,blob", [("C1", 3538944), ("C2", 12091392), ("C3", 24772608), ("C5", 16220160)])
def test_expert_blob_sizes(name, blob):
    from project_maya_b200 import api
    cfg = H.CONFIGS[name]
    L = api.native_expert_layout(cfg["gu_type"], cfg["d_type"], cfg["n_embd"], cfg["n_ff"])
    assert L.bytes == blob
    assert L.up_off == cfg["n_ff"] * L.gu_row and L.down_off == 2 * L.up_off
    assert L.bytes == H.blob_bytes(cfg["gu_type"], cfg["d_type"], cfg["n_embd"], cfg["n_ff"])


def test_shared_and_prefill_blob_sizes():
    from project_maya_b200 import api
    assert api.native_expert_layout(H.Q8_0, H.Q8_0, 6144, 2048).bytes == 40108032
    assert api.native_expert_layout(H.Q4_K, H.Q4_K, 6144, 2048).bytes == 21233664


def test_layout_refusals():
    from project_maya_b200 import api
    with pytest.raises(api.MayaError) as e:
        api.native_expert_layout(7, H.Q4_K, 2048, 1024)
    assert e.value.status == -2
    with pytest.raises(api.MayaError) as e:
        api.native_expert_layout(H.Q4_K, H.Q4_K, 2000, 1024)
    assert e.value.status == -1


def test_refusals_need_no_device(lib):
    """Argument checks come before any launch: a bad call returns its status and counts as a launch error."""
    before = lib.maya_launch_errors()
    assert lib.maya_mmvq(7, 16, 16, 16, 256, 4, 1, None) == -2            # unsupported type
    assert lib.maya_mmvq(H.Q4_K, 16, 16, 16, 256, 4, 9, None) == -4       # more than 8 columns
    assert lib.maya_mmvq(H.Q4_K, 16, 16, 16, 100, 4, 1, None) == -1       # n_in not a whole number of blocks
    assert lib.maya_mmvq(H.Q4_K, None, 16, 16, 256, 4, 1, None) == -1     # null weights
    assert lib.maya_router_top10(16, 1, 64, 65, 16, 16, None) == -4       # k beyond 64
    assert lib.maya_router_top10(16, 0, 64, 8, 16, 16, None) == 0         # no tokens: nothing to do, as the reference
    assert lib.maya_quantize_q8_1(16, 16, 100, 1, None) == -1
    assert lib.maya_launch_errors() == before + 6


def test_host_quantizer_block_sizes():
    from project_maya_b200 import api
    for t in (H.Q8_0, H.Q4_K, H.IQ2_S, H.IQ3_S):
        q = api.quantize_weights_host(t, np.ones((2, 512), np.float32) * 0.01)
        assert tuple(q.shape) == (2, H.row_bytes(t, 512))
    with pytest.raises(api.MayaError):
        api.quantize_weights_host(H.Q4_K, np.ones((2, 100), np.float32))


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from project_maya_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libmaya_moe.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()
