"""The CPU oracle pinned against everything the reference offers for this path (no GPU needed).

Pins: gguf-py's dequantizers (what the reference's fixture tool checks block decoding with); the reference's router
test (its four input distributions and its own host reference, committed as a fixture generated from the reference
sources); llama.cpp's captured sigmoid-router vectors the reference ships; the reference's CPU expert rows (fixture
for configuration C1, plus a live comparison when oracle/_ref is built); the float expert of the reference's expert
parity test, at that test's own gate.
"""
import hashlib
from pathlib import Path

import numpy as np
import pytest

import helpers as H

GOLDEN = Path(__file__).resolve().parent / "golden"
TYPES = [H.Q8_0, H.Q4_K, H.IQ2_S, H.IQ3_S]
ALL_TYPES = TYPES + list(H.MORE_TYPES)
GGUF_NAME = {H.Q8_0: "Q8_0", H.Q4_K: "Q4_K", H.IQ2_S: "IQ2_S", H.IQ3_S: "IQ3_S", H.Q5_K: "Q5_K", H.Q6_K: "Q6_K",
             H.IQ4_XS: "IQ4_XS", H.IQ3_XXS: "IQ3_XXS", H.IQ2_XXS: "IQ2_XXS", H.IQ1_S: "IQ1_S"}


@pytest.mark.parametrize("t", H.MORE_TYPES)
def test_q8_1_dot_of_the_further_types_against_the_float_product(oracle, t):
    """The q8_1 dots of Q5_K, Q6_K, IQ4_XS, IQ3_XXS, IQ2_XXS decode the same blocks as the dequantizer above (pinned to
    gguf-py bit for bit), so W . x from the integer path must sit within q8_1's rounding of the float product - a wrong
    field, sign or scale would show as O(1).  Also: the Python block sizes are the C ones."""
    rows, K = 32, 2048
    rng = H.rng_for("more-dot", t)
    w = H.constructed_blocks(t, rows, K, rng)
    assert w.shape[1] == oracle.row_bytes(t, K)
    x = rng.standard_normal((3, K)).astype(np.float32)
    wf = oracle.dequantize(t, w, rows * K).reshape(rows, K).astype(np.float64)
    for i in range(3):
        got = oracle.mmvq(t, w, oracle.quantize_q8_1(x[i]), K, rows)[0]
        assert H.rel_l2(got, wf @ x[i].astype(np.float64)) <= 2e-2
    # linear in the activations' block scales: doubling x doubles every dot exactly (powers of two)
    a = oracle.mmvq(t, w, oracle.quantize_q8_1(x[0]), K, rows)[0]
    b = oracle.mmvq(t, w, oracle.quantize_q8_1(2.0 * x[0]), K, rows)[0]
    assert np.array_equal(2.0 * a, b)


@pytest.mark.parametrize("t", ALL_TYPES)
def test_dequantize_matches_gguf_py(oracle, t):
    from gguf import GGMLQuantizationType, quants
    blocks = H.constructed_blocks(t, 16, 1024, H.rng_for("deq", t))
    want = quants.dequantize(blocks.reshape(-1), GGMLQuantizationType[GGUF_NAME[t]]).reshape(-1)
    got = oracle.dequantize(t, blocks, 16 * 1024)
    assert np.array_equal(got, want)      # bit-exact: same float operations in the same order


def test_generated_codebooks_match_reference_header_when_present():
    """The generated IQ2_S / IQ3_S tables are the GGUF format's: compared with the header the reference vendors."""
    import re
    import os
    from oracle.build import REFERENCE
    hdr = REFERENCE / "third_party" / "ggml" / "ggml-common.h"
    if not hdr.exists():
        pytest.skip("reference tree not on this machine")
    import sys
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "project_maya_b200" / "csrc"))
    import gen_iq_grids
    iq2, iq3 = gen_iq_grids.packed_grids()
    text = hdr.read_text()

    def table(name, n):
        m = re.search(name + r"(.*?)GGML_TABLE_END", text, re.S)
        vals = [int(v, 16) for v in re.findall(r"0x[0-9a-fA-F]+", m.group(1))]
        assert len(vals) == n
        return vals

    assert table(r"GGML_TABLE_BEGIN\(uint64_t, iq2s_grid, 1024\)", 1024) == [int(v) for v in iq2]
    assert table(r"GGML_TABLE_BEGIN\(uint32_t, iq3s_grid, 512\)", 512) == [int(v) for v in iq3]


def test_router_matches_reference_test_cases(oracle):
    g = np.load(GOLDEN / "router_reference_cases.npz")
    for c in range(4):
        ids, w = oracle.router_top10(g["logits"][c], 10)
        assert np.array_equal(ids, g["ids"][c]), str(g["names"][c])          # ids exact
        rel = np.abs(w - g["weights"][c]) / np.maximum(np.abs(g["weights"][c]), 1e-30)
        assert rel.max() <= 1e-5, str(g["names"][c])                         # the reference test's tolerance
        ids64, w64 = oracle.router_f64(g["logits"][c], 10)
        assert np.array_equal(ids64, g["ids"][c]) and np.array_equal(w64, g["weights"][c])


def test_router_live_against_reference_host_code(oracle, ref):
    for name, E, k, zipf in [("C1", 64, 8, None), ("C2", 256, 8, 1.1), ("x", 512, 10, None)]:
        logits = H.router_logits(name, 64, E, zipf)
        ids_r, w_r = ref.router_reference(logits, k)
        ids, w = oracle.router_top10(logits, k)
        assert np.array_equal(ids, ids_r)
        assert (np.abs(w - w_r) / np.abs(w_r)).max() <= 1e-5


def test_router_clamp_unreachable_for_the_configs():
    # top-k of a probability vector sums to at least k / n: 8/64 and 8/256 are far above 2^-14
    for k, n in [(8, 64), (8, 256)]:
        assert k / n > 2.0 ** -14


def test_sigmoid_router_matches_llama_cpp_dumps(oracle):
    g = np.load(GOLDEN / "glm5_synth_router.npz")
    for i in range(g["logits"].shape[0]):
        ids, w = oracle.router_sigmoid(g["logits"][i], g["bias"][i], g["ids"].shape[2], float(g["w_scale"]), True)
        assert np.array_equal(ids, g["ids"][i])
        assert (np.abs(w - g["weights"][i]) / np.abs(g["weights"][i])).max() <= 1e-6


def test_q8_1_blocks(oracle):
    x = H.rng_for("q81").standard_normal(4096).astype(np.float32)
    x[0:32] = 0.0                       # an all-zero block
    x[32:64] = 1.0e6                    # large values: scale stays finite in f16
    q = oracle.quantize_q8_1(x).reshape(-1, 36)
    d = q[:, 0:2].copy().view(np.float16).astype(np.float32).reshape(-1)
    s = q[:, 2:4].copy().view(np.float16).astype(np.float32).reshape(-1)
    qs = q[:, 4:].view(np.int8).astype(np.float32)
    assert d[0] == 0 and not qs[0].any()
    assert np.all(np.abs(qs) <= 127)
    xb = x.reshape(-1, 32)
    assert np.allclose(qs * d[:, None], xb, atol=float(np.abs(xb).max()) / 127 * 0.51 + 1e-3, rtol=2e-3)
    assert np.allclose(s[2:], xb[2:].sum(1), rtol=2e-3, atol=2e-2)
    assert np.isfinite(d).all() and np.isfinite(s).all()


def test_q8_K_matches_reference_transcription(oracle, ref):
    x = H.rng_for("q8k").standard_normal(8 * 256).astype(np.float32)
    x[256:512] = 0.0
    assert np.array_equal(oracle.quantize_q8_K(x), ref.quantize_q8_K(x))


def _quantized_expert(t, n_embd, n_ff, key):
    from project_maya_b200 import api
    rng = H.rng_for("expert", key, t)
    gu = api.quantize_weights_host(t, rng.normal(0, 0.02, size=(2 * n_ff, n_embd)).astype(np.float32)).numpy()
    dn = api.quantize_weights_host(t, rng.normal(0, 0.02, size=(n_embd, n_ff)).astype(np.float32)).numpy()
    return np.concatenate([gu.reshape(-1), dn.reshape(-1)])


@pytest.mark.parametrize("t", TYPES)
def test_own_quantizers_round_trip(oracle, t):
    from project_maya_b200 import api
    w = H.rng_for("rt", t).normal(0, 0.02, size=(8, 1024)).astype(np.float32)
    q = api.quantize_weights_host(t, w).numpy()
    assert q.shape == (8, H.row_bytes(t, 1024))
    back = oracle.dequantize(t, q, w.size).reshape(w.shape)
    rms = float(np.sqrt(((back - w) ** 2).mean()) / 0.02)
    assert rms < {H.Q8_0: 0.01, H.Q4_K: 0.12, H.IQ3_S: 0.2, H.IQ2_S: 0.35}[t]
    assert np.isfinite(back).all()
    zero = api.quantize_weights_host(t, np.zeros((1, 256), np.float32)).numpy()
    assert not oracle.dequantize(t, zero, 256).any()


@pytest.mark.parametrize("t", TYPES)
def test_quantized_expert_against_float_expert(oracle, t):
    """The reference's own gate (native_expert_parity.cpp:298-299): rel-L1 vs the double reference < 3e-2."""
    n_embd, n_ff = 512, 256
    blob = _quantized_expert(t, n_embd, n_ff, "f64")
    x = H.rng_for("f64x", t).standard_normal(n_embd).astype(np.float32)
    yq = oracle.expert_q8_1(t, t, blob, n_embd, n_ff, H.INF, oracle.quantize_q8_1(x))
    yf = oracle.expert_f64(t, t, blob, n_embd, n_ff, x)
    assert np.abs(yq - yf).sum() / np.abs(yf).sum() < 3e-2


@pytest.mark.parametrize("t", TYPES)
def test_q8_1_dot_against_the_reference_mmq_host_model(oracle, t):
    """oracle.mmq_host_model restates the reference's host model of its prompt-path GEMM
    (tests/glm_dsa/glmd_mmq_ids_test.cu:92-347; that test gates the reference's kernels at rel-L2 < 1e-4 from it).  The
    decode oracle's q8_1 dots round the activation scale to f16 where the model's d4 layout keeps a float, nothing else:
    both must agree to a few 1e-4, outlier included, and both sit ~1e-3 from the unquantized-activation product."""
    rows, K = 48, 1024
    rng = H.rng_for("mmq-model", t)
    w = H.constructed_blocks(t, rows, K, rng)
    x = rng.standard_normal((6, K)).astype(np.float32)
    x[0, 5] = 3000.0                                                      # the reference test's outlier
    x[1, 64:96] = 0.0                                                     # an all-zero group
    model = oracle.mmq_host_model(t, w, rows, K, x)
    q81 = np.stack([oracle.mmvq(t, w, oracle.quantize_q8_1(x[i]), K, rows)[0] for i in range(6)])
    assert np.isfinite(model).all()
    assert H.rel_l2(q81, model) <= 5e-4
    exact = x.astype(np.float64) @ oracle.dequantize(t, w, rows * K).reshape(rows, K).astype(np.float64).T
    assert H.rel_l2(model, exact) <= 2e-2


@pytest.mark.parametrize("t", TYPES)
def test_mixed_type_expert_is_the_plain_expert_when_the_types_agree(oracle, t):
    """oracle.expert_q8_1_mixed (the up rows' own type, iq_kernels.hpp:73-77) composes the single steps; with one type
    for gate and up it must be expert_q8_1 bit for bit, which pins the composition the mixed-type GPU test checks against."""
    n_embd, n_ff = 512, 256
    blob = H.constructed_expert(t, t, n_embd, n_ff, H.rng_for("mixed-pin", t))
    xq = oracle.quantize_q8_1(H.rng_for("mixed-pin-x", t).standard_normal(n_embd).astype(np.float32))
    for limit in (H.INF, 7.0):
        assert np.array_equal(oracle.expert_q8_1_mixed(t, t, t, blob, n_embd, n_ff, limit, xq),
                              oracle.expert_q8_1(t, t, blob, n_embd, n_ff, limit, xq))


@pytest.mark.parametrize("t", [H.Q4_K, H.IQ2_S, H.IQ3_S])
@pytest.mark.parametrize("avx512", [True, False])
def test_oracle_against_reference_cpu_rows(oracle, ref, t, avx512):
    """Row dots of the reference's CPU kernels (Q8_K activations) and of the oracle (q8_1 activations) on the same
    weights: both are the same integer block decoding, so both sit within the reference's 3e-2 of the float result
    and within 3e-2 of each other; a decoding error in either would show as O(1)."""
    n_embd, n_ff = 1024, 512
    blob = H.constructed_expert(t, t, n_embd, n_ff, H.rng_for("rows", t))
    x = H.rng_for("rowsx", t).standard_normal(n_embd).astype(np.float32)
    grb = H.row_bytes(t, n_embd)
    # plain rows: gate rows as a GEMV
    y_ref = ref.rows(t, blob, grb, n_embd, [oracle.quantize_q8_K(x)], 0, n_ff, avx512)[0]
    y_orc = oracle.mmvq(t, blob, oracle.quantize_q8_1(x), n_embd, n_ff)[0]
    w = oracle.dequantize(t, blob[: n_ff * grb], n_ff * n_embd).reshape(n_ff, n_embd).astype(np.float64)
    y_f = w @ x.astype(np.float64)
    scale = np.abs(y_f).max()
    assert np.abs(y_ref - y_f).max() / scale < 3e-2
    assert np.abs(y_orc - y_f).max() / scale < 3e-2
    assert np.abs(y_orc - y_ref).max() / scale < 3e-2


def test_c1_fixture_is_reproducible_and_close(oracle):
    """C1 in full on the CPU: the oracle (q8_1 path) against the committed outputs of the reference's CPU rows."""
    import sys
    sys.path.insert(0, str(GOLDEN))
    import make_golden
    g = np.load(GOLDEN / "c1_reference_cpu.npz")
    cfg = H.CONFIGS["C1"]
    blobs = make_golden.c1_experts()
    assert hashlib.sha256(blobs.tobytes()).hexdigest() == str(g["experts_sha256"])
    logits = H.router_logits("C1", cfg["tokens"], cfg["n_expert"], None)
    x = H.activations("C1", cfg["tokens"], cfg["n_embd"], "f32")
    ids, w, out = oracle.moe_layer(dict(cfg, limit=H.INF), logits, x, blobs)
    assert np.array_equal(ids, g["ids"])
    assert (np.abs(w - g["weights"]) / g["weights"]).max() <= 1e-5
    assert np.array_equal(out, g["out_oracle_q8_1"])
    # the reference's CPU path rounds activations to Q8_K, its GPU path (what the oracle restates) to q8_1: the two
    # differ by about 2e-2 here, inside the 3e-2 the reference allows either against the float result
    for t in range(cfg["tokens"]):
        assert H.rel_err(out[t], g["out_cpu_rows"][t]) < 3e-2


def test_mmvq_orders_agree(oracle):
    t, n_in, n_out = H.IQ3_S, 1024, 64
    w = H.constructed_blocks(t, n_out, n_in, H.rng_for("ord"))
    xq = oracle.quantize_q8_1(H.rng_for("ordx").standard_normal(n_in).astype(np.float32))
    a, b = oracle.mmvq(t, w, xq, n_in, n_out, order=0), oracle.mmvq(t, w, xq, n_in, n_out, order=1)
    assert H.rel_err(a, b) < 1e-5


def test_combine_orders(oracle):
    rng = H.rng_for("comb")
    parts = rng.standard_normal((8, 256)).astype(np.float32)
    w = rng.random(8).astype(np.float32)
    sh = rng.standard_normal(256).astype(np.float32)
    want = (parts.astype(np.float64) * w[:, None]).sum(0) + sh
    assert np.allclose(oracle.combine_down(parts, w, sh), want, rtol=1e-5, atol=1e-5)
    assert np.allclose(oracle.combine_native(parts, w, sh), want, rtol=1e-5, atol=1e-5)
    skip = np.zeros(8, np.uint8); skip[3] = 1
    want2 = want - parts[3] * w[3]
    assert np.allclose(oracle.combine_down(parts, w, sh, skip), want2, rtol=1e-5, atol=1e-5)


def test_allreduce_in_order(oracle):
    parts = np.array([[1e8, 1.0, -0.0], [-1e8, 1e-8, 0.0], [1.0, -1.0, -0.0]], np.float32)
    out = oracle.allreduce_in_order(parts)
    assert out[0] == np.float32(np.float32(np.float32(1e8) + np.float32(-1e8)) + np.float32(1.0))
    assert out[1] == np.float32(np.float32(np.float32(1.0) + np.float32(1e-8)) + np.float32(-1.0))


def test_expert_group(oracle):
    ids = np.array([[3, 1], [1, 0], [3, 3]], np.int32)
    counts, bounds, pos, row_tok = oracle.expert_group(ids, 2, 4)
    assert counts.tolist() == [1, 2, 0, 3] and bounds.tolist() == [0, 1, 3, 3, 6]
    assert pos.tolist() == [3, 1, 2, 0, 4, 5] and row_tok.tolist() == [1, 0, 1, 0, 2, 2]


def test_rms_router_against_float64(oracle):
    """glmf::rms_q8's norm and the router GEMV: the oracle against a float64 evaluation, and against llama.cpp's captured
    router logits of the synthetic GGUF layer (x = the captured FFN input, unit norm weights undone by construction)."""
    rng = H.rng_for("rms-router")
    n, E, eps = 1536, 40, 1e-5
    h, add = rng.standard_normal(n).astype(np.float32), (0.1 * rng.standard_normal(n)).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    rw = (0.05 * rng.standard_normal((E, n))).astype(np.float32)
    h_out, x, logits = oracle.rms_router(h, add, w, eps, rw)
    t = h.astype(np.float64) + add.astype(np.float64)
    x64 = t / np.sqrt((t * t).mean() + eps) * w
    assert np.array_equal(h_out, h + add)
    assert np.abs(x - x64).max() <= 2e-6 * np.abs(x64).max()
    assert np.abs(logits - rw.astype(np.float64) @ x64).max() <= 1e-5
    g = np.load(GOLDEN / "glm5_synth_moe_layer1.npz")
    xin = g["x"][3]
    # choose norm weights that undo the normalisation, so that x == the captured input and the logits must be llama.cpp's
    inv = 1.0 / np.sqrt((xin.astype(np.float64) ** 2).mean() + eps)
    _, x2, lg = oracle.rms_router(xin, None, (np.ones_like(xin) / inv).astype(np.float32), eps, g["router"])
    assert np.abs(x2 - xin).max() <= 1e-6
    assert np.abs(lg - g["logits"][3]).max() <= 1e-5
