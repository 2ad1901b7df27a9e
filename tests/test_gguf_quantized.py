"""An already-QUANTIZED GGUF through project_maya_b200/gguf_loader.py and the kernels.

tests/golden/iq_fixture.gguf was written by the reference's own fixture tool (tools/iq_fixture.py via
tests/golden/make_gguf_fixture.py): layer 0 Q4_K, 1 IQ2_S, 2 IQ3_S, 3 Q8_0 routed-expert tensors
blk.N.ffn_{gate,up,down}_exps.weight of 2 experts (hidden 512, FFN 256), random valid blocks over the whole code
space, with a manifest of the tensors' sha256.

Checked on the CPU: the loader leaves the bytes untouched (the manifest's hashes), builds the [gate | up | down] blob
per expert, and the oracle's quantized expert on that blob is the float expert evaluated from gguf-py's own
dequantization of the SAME tensors (an independent decoder) within the reference's gate (rel-L1 < 3e-2,
native_expert_parity.cpp:298-299).  On the GPU: the decode layer on those blobs against the oracle (<= 2e-4) and
against that float expert (<= 3e-2).
"""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

import helpers as H

GOLDEN = Path(__file__).resolve().parent / "golden"
GGUF = GOLDEN / "iq_fixture.gguf"
LAYER_TYPES = [H.Q4_K, H.IQ2_S, H.IQ3_S, H.Q8_0]


def _float_expert(gate, up, down, x):
    """double-precision SwiGLU expert from dequantized float matrices (rows in GGUF order)."""
    g = gate.astype(np.float64) @ x.astype(np.float64)
    u = up.astype(np.float64) @ x.astype(np.float64)
    h = g / (1.0 + np.exp(-g)) * u
    return down.astype(np.float64) @ h


def _dequantized(layer):
    import gguf
    rd = gguf.GGUFReader(str(GGUF))
    ts = {t.name: t for t in rd.tensors}
    out = {}
    for part in ("gate", "up", "down"):
        t = ts[f"blk.{layer}.ffn_{part}_exps.weight"]
        shape = [int(v) for v in reversed(t.shape.tolist())]                  # [E, rows, cols]
        out[part] = gguf.quants.dequantize(t.data, t.tensor_type).reshape(shape)
    return out


@pytest.mark.parametrize("layer", range(4))
def test_loader_keeps_bytes_and_builds_blobs(layer):
    from project_maya_b200 import gguf_loader
    manifest = json.loads((GOLDEN / "iq_fixture.gguf.json").read_text())
    L = gguf_loader.read_moe_layer(GGUF, layer)
    t = LAYER_TYPES[layer]
    assert (L.n_embd, L.n_ff, L.n_expert, L.ggml_type) == (512, 256, 2, t)
    for part in ("gate", "up", "down"):
        assert hashlib.sha256(getattr(L, part).tobytes()).hexdigest() == manifest["layers"][layer]["sha256"][part]
    blobs = gguf_loader.expert_blobs(L)
    gu = 256 * H.row_bytes(t, 512)
    assert blobs.shape == (2, H.blob_bytes(t, t, 512, 256))
    for e in range(2):
        assert np.array_equal(blobs[e, :gu], L.gate[e].reshape(-1))
        assert np.array_equal(blobs[e, gu:2 * gu], L.up[e].reshape(-1))
        assert np.array_equal(blobs[e, 2 * gu:], L.down[e].reshape(-1))


@pytest.mark.parametrize("layer", range(4))
def test_oracle_on_loaded_blobs_matches_gguf_py_float_expert(oracle, layer):
    from project_maya_b200 import gguf_loader
    L = gguf_loader.read_moe_layer(GGUF, layer)
    t = LAYER_TYPES[layer]
    blobs = gguf_loader.expert_blobs(L)
    deq = _dequantized(layer)
    x = H.rng_for("gguf-q", layer).standard_normal(512).astype(np.float32)
    for e in range(2):
        want = _float_expert(deq["gate"][e], deq["up"][e], deq["down"][e], x)
        got = oracle.expert_q8_1(t, t, blobs[e], 512, 256, H.INF, oracle.quantize_q8_1(x))
        assert np.abs(got - want).sum() / np.abs(want).sum() < 3e-2
        # the oracle's own double-precision evaluation decodes the blocks the way gguf-py does
        assert H.rel_err(oracle.expert_f64(t, t, blobs[e], 512, 256, x), want) <= 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("layer", range(4))
def test_layer_kernels_on_loaded_blobs(cuda, oracle, layer):
    import torch as T
    from project_maya_b200 import api, gguf_loader
    L = gguf_loader.read_moe_layer(GGUF, layer)
    t = LAYER_TYPES[layer]
    blobs_np = gguf_loader.expert_blobs(L)
    blobs = T.from_numpy(blobs_np).cuda()
    lc = api.MoeLayerConfig(512, 256, 2, 2, t, t)
    layer_k = api.MoeLayer(lc, blobs, None)
    deq = _dequantized(layer)
    rng = H.rng_for("gguf-q-gpu", layer)
    for tok in range(3):
        x = rng.standard_normal(512).astype(np.float32)
        logits = rng.standard_normal((1, 2)).astype(np.float32)
        ids, w, out = layer_k.forward(T.from_numpy(logits).cuda(), T.from_numpy(x[None]).cuda())
        ids_o, w_o = oracle.router_top10(logits, 2)
        assert np.array_equal(ids.cpu().numpy(), ids_o)
        xq = oracle.quantize_q8_1(x)
        parts = np.stack([oracle.expert_q8_1(t, t, blobs_np[int(e)], 512, 256, H.INF, xq) for e in ids_o[0]])
        want = oracle.combine_down(parts, w_o[0], None)
        got = out.cpu().numpy()[0]
        assert H.rel_err(got, want) <= 2e-4
        flt = sum(float(w_o[0][j]) * _float_expert(deq["gate"][e], deq["up"][e], deq["down"][e], x) for j, e in enumerate(ids_o[0]))
        assert np.abs(got - flt).sum() / np.abs(flt).sum() < 3e-2
    # the window path on the same blobs agrees with the single tokens
    xs = rng.standard_normal((4, 512)).astype(np.float32)
    ls = rng.standard_normal((4, 2)).astype(np.float32)
    _, _, win = layer_k.forward(T.from_numpy(ls).cuda(), T.from_numpy(xs).cuda())
    for i in range(4):
        assert T.equal(win[i], layer_k.forward(T.from_numpy(ls[i:i + 1]).cuda(), T.from_numpy(xs[i:i + 1]).cuda())[2][0])
