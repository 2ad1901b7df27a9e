"""Parity of the CUDA decode path against the CPU oracle, through the C ABI (needs a B200).

Bars: router ids bit-exact, router weights rel <= 1e-5 (the reference test's tolerance); q8_1 blocks byte-exact;
FFN outputs max|got - want| / max|want| <= 1e-2 against the oracle (the stated tolerance), with a tighter 2e-4 check
beside it because only the order of FP32 additions differs from the oracle; bit-for-bit where the reference promises
it (multi-column == single-column, window == token by token).
"""
from pathlib import Path

import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).resolve().parent / "golden"
TYPES = [H.Q8_0, H.Q4_K, H.IQ2_S, H.IQ3_S]
MORE = list(H.MORE_TYPES)          # Q5_K, Q6_K, IQ4_XS, IQ3_XXS, IQ2_XXS: the staged decode paths
TOL = 1e-2      # the path's stated tolerance
TIGHT = 2e-4    # what an implementation with the oracle's integer arithmetic actually reaches


@pytest.fixture(scope="module")
def T(cuda):
    import torch
    return torch


@pytest.fixture(scope="module")
def api(cuda):
    from project_maya_b200 import api as a
    return a


def dev(T, a, dtype=None):
    t = T.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def expert_blob(t, n_embd, n_ff, key, quantized):
    if quantized:
        from project_maya_b200 import api as a
        rng = H.rng_for("gpu-expert", key, t)
        gu = a.quantize_weights_host(t, rng.normal(0, 0.02, size=(2 * n_ff, n_embd)).astype(np.float32)).numpy()
        dn = a.quantize_weights_host(t, rng.normal(0, 0.02, size=(n_embd, n_ff)).astype(np.float32)).numpy()
        return np.concatenate([gu.reshape(-1), dn.reshape(-1)])
    return H.constructed_expert(t, t, n_embd, n_ff, H.rng_for("gpu-expert-c", key, t))


# ------------------------------------------------------------------------------------------------ router
def test_router_reference_cases(T, api, oracle):
    g = np.load(GOLDEN / "router_reference_cases.npz")
    for c in range(4):
        ids, w = api.router_top10(dev(T, g["logits"][c]), 10)
        ids, w = ids.cpu().numpy(), w.cpu().numpy()
        assert np.array_equal(ids, g["ids"][c]), str(g["names"][c])
        assert (np.abs(w - g["weights"][c]) / np.abs(g["weights"][c])).max() <= 1e-5
        assert np.abs(w.sum(1) - 1).max() < 1e-5


@pytest.mark.parametrize("name,E,k,zipf,n_tok", [("C1", 64, 8, None, 16), ("C2", 256, 8, 1.1, 256), ("C3", 256, 8, 1.1, 8),
                                                 ("C4", 256, 8, None, 4096), ("C5", 256, 8, 1.1, 64),
                                                 ("wide", 2048, 64, None, 4), ("odd", 77, 5, None, 33)])
def test_router_configs_bit_exact(T, api, oracle, name, E, k, zipf, n_tok):
    logits = H.router_logits(name, n_tok, E, zipf)
    ids, w = api.router_top10(dev(T, logits), k)
    ids_o, w_o = oracle.router_top10(logits, k)
    assert np.array_equal(ids.cpu().numpy(), ids_o)
    assert (np.abs(w.cpu().numpy() - w_o) / np.abs(w_o)).max() <= 1e-5


def test_router_ties_and_extremes(T, api, oracle):
    E, k = 256, 8
    cases = [np.full((4, E), 0.5, np.float32), np.zeros((4, E), np.float32)]
    c = H.rng_for("ties").standard_normal((4, E)).astype(np.float32)
    c[:, 10:30] = 3.0                                   # a 20-way tie across the cut
    cases.append(c)
    d = np.full((4, E), -80.0, np.float32)               # exp underflows to tiny values: many equal probabilities
    d[:, 5] = 80.0
    cases.append(d)
    for logits in cases:
        ids, w = api.router_top10(dev(T, logits), k)
        ids_o, w_o = oracle.router_top10(logits, k)
        assert np.array_equal(ids.cpu().numpy(), ids_o)
        assert np.allclose(w.cpu().numpy(), w_o, rtol=1e-5, atol=1e-30)


def test_router_sigmoid_golden(T, api):
    g = np.load(GOLDEN / "glm5_synth_router.npz")
    for i in range(g["logits"].shape[0]):
        ids, w = api.router_sigmoid(dev(T, g["logits"][i]), dev(T, g["bias"][i]), g["ids"].shape[2], float(g["w_scale"]), True)
        assert np.array_equal(ids.cpu().numpy(), g["ids"][i])
        assert (np.abs(w.cpu().numpy() - g["weights"][i]) / g["weights"][i]).max() <= 1e-6


# ------------------------------------------------------------------------------------------------ q8_1
@pytest.mark.parametrize("act", ["f32", "bf16"])
def test_quantize_q8_1_bytes(T, api, oracle, act):
    x = H.activations("q81", 5, 6144, act)
    x[0, :32] = 0.0
    x[1, 32:64] *= 1.0e6
    if act == "bf16":
        x = H.to_bf16_f32(x)
    xd = dev(T, x, T.bfloat16 if act == "bf16" else None)
    got = api.native_quantize_q8_1(xd).cpu().numpy()
    want = np.stack([oracle.quantize_q8_1(x[i]) for i in range(5)])
    assert np.array_equal(got, want)


def test_swiglu_q8_1(T, api, oracle):
    rng = H.rng_for("swq")
    g, u = (rng.standard_normal(2048) * 4).astype(np.float32), (rng.standard_normal(2048) * 4).astype(np.float32)
    for limit in (H.INF, 7.0):
        got = api.swiglu_q8_1(dev(T, g), dev(T, u), limit).cpu().numpy()
        want = oracle.quantize_q8_1(oracle.swiglu(g, u, limit))
        # expf on the device may differ from libm in the last place: allow a handful of quants off by one
        diff = got.reshape(-1, 36)[:, 4:].view(np.int8).astype(int) - want.reshape(-1, 36)[:, 4:].view(np.int8).astype(int)
        assert np.abs(diff).max() <= 1 and (diff != 0).mean() < 0.01


# ------------------------------------------------------------------------------------------------ GEMV
@pytest.mark.parametrize("t", TYPES + MORE)
@pytest.mark.parametrize("n_in,n_out", [(2048, 1024), (6144, 515), (256, 7)])
def test_mmvq_matches_oracle(T, api, oracle, t, n_in, n_out):
    w = H.constructed_blocks(t, n_out, n_in, H.rng_for("mv", t, n_in))
    x = H.rng_for("mvx", t, n_in).standard_normal((1, n_in)).astype(np.float32)
    xq = api.native_quantize_q8_1(dev(T, x))
    y = api.native_mmvq(t, dev(T, w), xq, n_in, n_out).cpu().numpy()
    want = oracle.mmvq(t, w, oracle.quantize_q8_1(x), n_in, n_out)
    assert H.rel_err(y, want) <= TOL
    assert H.rel_err(y, want) <= TIGHT


@pytest.mark.parametrize("t", TYPES + MORE)
def test_mmvq_multi_column_is_single_column_bitwise(T, api, t):
    n_in, n_out = 2048, 300
    w = dev(T, H.constructed_blocks(t, n_out, n_in, H.rng_for("mc", t)))
    x = H.rng_for("mcx", t).standard_normal((8, n_in)).astype(np.float32)
    xq = api.native_quantize_q8_1(dev(T, x))
    single = T.stack([api.native_mmvq(t, w, xq[c], n_in, n_out)[0] for c in range(8)])
    for ncols in (1, 2, 3, 4, 5, 7, 8):
        y = api.native_mmvq(t, w, xq[:ncols].contiguous(), n_in, n_out, ncols)
        assert T.equal(y, single[:ncols]), f"ncols {ncols}"


def test_mmvq_refusals(T, api):
    w = T.zeros(144 * 8, dtype=T.uint8, device="cuda")
    xq = T.zeros(36 * 8, dtype=T.uint8, device="cuda")
    with pytest.raises(api.MayaError) as e:
        api.native_mmvq(H.Q4_K, w, xq, 256, 8, 9)
    assert e.value.status == -4
    with pytest.raises(api.MayaError) as e:
        api.native_mmvq(3, w, xq, 256, 8, 1)
    assert e.value.status == -2


# ------------------------------------------------------------------------------------------------ plan form
def run_plan(T, api, t, n_embd, n_ff, blobs, weights, x, limit, skip_entries=(), shared=None, cpu_part=None):
    """moe_gate_up + moe_down for one token; blobs: list of numpy blobs (one per plan entry)."""
    k = len(blobs)
    store = dev(T, np.stack(blobs))
    ptrs = [store[i].data_ptr() for i in range(k)]
    for i in skip_entries:
        ptrs[i] = 0
    plan_ptr = T.tensor(ptrs, dtype=T.int64, device="cuda")
    plan_w = dev(T, np.asarray(weights, np.float32))
    xq = api.native_quantize_q8_1(dev(T, x.reshape(1, -1)))
    hq = T.zeros(k * (n_ff // 32) * 36, dtype=T.uint8, device="cuda")
    out = T.zeros(n_embd, dtype=T.float32, device="cuda")
    flag = T.ones(1, dtype=T.int32, device="cuda") if cpu_part is not None else None
    cpu_part_d = dev(T, cpu_part) if cpu_part is not None else None      # the plan holds raw addresses: keep it alive
    plan = api.make_plan(plan_ptr, plan_w, cpu_part_d, flag)
    sh_out = None
    if shared is not None:
        sh_t, sh_ff, sh_blob = shared
        sb = dev(T, sh_blob)
        gu = api.native_mmvq(sh_t, sb, xq, n_embd, 2 * sh_ff)
        sh_hq = api.swiglu_q8_1(gu[0, :sh_ff].contiguous(), gu[0, sh_ff:].contiguous(), limit)
        sh_out = T.zeros(n_embd, dtype=T.float32, device="cuda")
        down_off = 2 * sh_ff * H.row_bytes(sh_t, n_embd)
        api.moe_gate_up(t, plan, k, n_embd, n_ff, limit, xq, hq, sb[down_off:], sh_t, sh_hq, sh_ff, sh_out)
    else:
        api.moe_gate_up(t, plan, k, n_embd, n_ff, limit, xq, hq)
    api.moe_down(t, plan, k, n_embd, n_ff, 2 * n_ff * H.row_bytes(t, n_embd), hq, sh_out, out)
    T.cuda.synchronize()
    return out.cpu().numpy(), hq.cpu().numpy()


def oracle_plan(oracle, t, n_embd, n_ff, blobs, weights, x, limit, skip_entries=(), shared=None, cpu_part=None):
    xq = oracle.quantize_q8_1(x)
    k = len(blobs)
    parts = np.zeros((k, n_embd), np.float32)
    skip = np.zeros(k, np.uint8)
    for i in range(k):
        if i in skip_entries:
            skip[i] = 1
        else:
            parts[i] = oracle.expert_q8_1(t, t, blobs[i], n_embd, n_ff, limit, xq)
    sh = None
    if shared is not None:
        sh = oracle.expert_q8_1(shared[0], shared[0], shared[2], n_embd, shared[1], limit, xq)
    out = oracle.combine_down(parts, np.asarray(weights, np.float32), None, skip)
    if cpu_part is not None:
        out = out + cpu_part
    if sh is not None:
        out = out + sh
    return out.astype(np.float32)


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("quantized", [True, False])
def test_gate_up_down_plan(T, api, oracle, t, quantized):
    n_embd, n_ff, k = 512, 256, 8
    blobs = [expert_blob(t, n_embd, n_ff, i, quantized) for i in range(k)]
    w = H.rng_for("pw", t).random(k).astype(np.float32)
    w /= w.sum()
    x = H.rng_for("px", t).standard_normal(n_embd).astype(np.float32)
    limit = 7.0 if quantized else H.INF
    got, _ = run_plan(T, api, t, n_embd, n_ff, blobs, w, x, limit)
    want = oracle_plan(oracle, t, n_embd, n_ff, blobs, w, x, limit)
    assert H.rel_err(got, want) <= TOL
    assert H.rel_err(got, want) <= TIGHT


@pytest.mark.parametrize("t", MORE)
def test_gate_up_down_plan_further_types(T, api, oracle, t):
    """The plan kernels on the rest of glmf::moe_supported's types (glm_fast.cu:5798-5801): random valid blocks, k = 8,
    clamped and plain SwiGLU, a skipped entry."""
    n_embd, n_ff, k = 1024, 512, 8
    blobs = [expert_blob(t, n_embd, n_ff, i, False) for i in range(k)]
    w = H.rng_for("pw-more", t).random(k).astype(np.float32)
    w /= w.sum()
    x = H.rng_for("px-more", t).standard_normal(n_embd).astype(np.float32)
    for limit, skip in ((H.INF, ()), (7.0, (2,))):
        got, _ = run_plan(T, api, t, n_embd, n_ff, blobs, w, x, limit, skip_entries=skip)
        want = oracle_plan(oracle, t, n_embd, n_ff, blobs, w, x, limit, skip_entries=skip)
        assert H.rel_err(got, want) <= TIGHT


def test_plan_edge_cases(T, api, oracle):
    t, n_embd, n_ff = H.IQ3_S, 512, 256
    blobs = [expert_blob(t, n_embd, n_ff, i, False) for i in range(5)]          # k = 5 < 8
    w = np.array([0.4, 0.3, 0.15, 0.1, 0.05], np.float32)
    x = H.rng_for("edge").standard_normal(n_embd).astype(np.float32)
    cpu_part = H.rng_for("edge-cpu").standard_normal(n_embd).astype(np.float32)
    shared = (H.Q8_0, 256, expert_blob(H.Q8_0, n_embd, 256, "sh", True))
    got, _ = run_plan(T, api, t, n_embd, n_ff, blobs, w, x, 7.0, skip_entries=(1, 4), shared=shared, cpu_part=cpu_part)
    want = oracle_plan(oracle, t, n_embd, n_ff, blobs, w, x, 7.0, skip_entries=(1, 4), shared=shared, cpu_part=cpu_part)
    assert H.rel_err(got, want) <= TIGHT
    # an all-zero activation gives an all-zero output
    got0, _ = run_plan(T, api, t, n_embd, n_ff, blobs, w, np.zeros(n_embd, np.float32), H.INF)
    assert not got0.any()


def test_plan_skip_flag_leaves_output_alone(T, api):
    t, n_embd, n_ff, k = H.Q4_K, 512, 256, 2
    store = dev(T, np.stack([expert_blob(t, n_embd, n_ff, i, False) for i in range(k)]))
    plan_ptr = T.tensor([store[i].data_ptr() for i in range(k)], dtype=T.int64, device="cuda")
    plan_w = T.ones(k, dtype=T.float32, device="cuda")
    skip = T.ones(1, dtype=T.int32, device="cuda")
    plan = api.make_plan(plan_ptr, plan_w, None, None, skip)
    xq = api.native_quantize_q8_1(T.ones(1, n_embd, device="cuda"))
    hq = T.full((k * (n_ff // 32) * 36,), 7, dtype=T.uint8, device="cuda")
    out = T.full((n_embd,), 3.0, dtype=T.float32, device="cuda")
    api.moe_gate_up(t, plan, k, n_embd, n_ff, H.INF, xq, hq)
    api.moe_down(t, plan, k, n_embd, n_ff, 2 * n_ff * H.row_bytes(t, n_embd), hq, None, out)
    assert bool((hq == 7).all()) and bool((out == 3.0).all())


def test_plan_refusals(T, api):
    plan = api.make_plan(T.zeros(8, dtype=T.int64, device="cuda"), T.zeros(8, device="cuda"))
    buf = T.zeros(4096, dtype=T.uint8, device="cuda")
    with pytest.raises(api.MayaError) as e:
        api.moe_gate_up(H.Q4_K, plan, 9, 512, 256, H.INF, buf, buf)       # k beyond 8
    assert e.value.status == -4
    with pytest.raises(api.MayaError) as e:
        api.moe_gate_up(H.Q4_K, plan, 8, 512, 200, H.INF, buf, buf)       # n_ff not a multiple of 32 / the block
    assert e.value.status == -1
    with pytest.raises(api.MayaError) as e:
        api.moe_down(5, plan, 8, 512, 256, 0, buf, None, buf)
    assert e.value.status == -2


# ------------------------------------------------------------------------------------------------ window form
def run_window(T, api, t, n_embd, n_ff, store, ids, w, x, limit):
    from project_maya_b200._lib import MoeWin
    n_tok, k = ids.shape
    ptr = np.zeros((n_tok, 8), np.int64)
    pw = np.zeros((n_tok, 8), np.float32)
    for i in range(n_tok):
        for j in range(k):
            ptr[i, j] = store[int(ids[i, j])].data_ptr() if ids[i, j] >= 0 else 0
            pw[i, j] = w[i, j]
    plan_ptr, plan_w = dev(T, ptr), dev(T, pw)
    xq = api.native_quantize_q8_1(dev(T, x))
    z = lambda n, dt: T.zeros(n, dtype=dt, device="cuda")
    keep = dict(hq=z(n_tok * 8 * (n_ff // 32) * 36, T.uint8), part=z(n_tok * 8 * n_embd, T.float32),
                out=z(n_tok * n_embd, T.float32), gp=z(n_tok * 8, T.int64), gs=z(n_tok * 8 + 1, T.int32),
                ge=z(n_tok * 8, T.int32), ng=z(1, T.int32))
    win = MoeWin(plan_ptr.data_ptr(), plan_w.data_ptr(), None, None, xq.data_ptr(), xq.shape[1], keep["hq"].data_ptr(),
                 keep["part"].data_ptr(), None, keep["out"].data_ptr(), n_embd, keep["gp"].data_ptr(),
                 keep["gs"].data_ptr(), keep["ge"].data_ptr(), keep["ng"].data_ptr(), n_tok, k, n_embd, n_ff, limit,
                 2 * n_ff * H.row_bytes(t, n_embd))
    api.moe_win_experts(t, t, win)
    T.cuda.synchronize()
    return keep["out"].reshape(n_tok, n_embd), plan_ptr, plan_w, xq, keep


@pytest.mark.parametrize("t,n_tok", [(t, n) for t in TYPES for n in (1, 3, 8, 16)] + [(t, n) for t in MORE for n in (3, 8)])
def test_window_equals_token_by_token_bitwise(T, api, oracle, t, n_tok):
    n_embd, n_ff, E, k = 512, 256, 12, 4
    store = dev(T, np.stack([expert_blob(t, n_embd, n_ff, e, False) for e in range(E)]))
    rng = H.rng_for("win", t, n_tok)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(n_tok)]).astype(np.int64)   # heavy overlap: 12 experts
    if n_tok > 1:
        ids[1, 2] = -1                                                               # one skipped plan slot
    w = rng.random((n_tok, k)).astype(np.float32)
    x = rng.standard_normal((n_tok, n_embd)).astype(np.float32)
    out, plan_ptr, plan_w, xq, keep = run_window(T, api, t, n_embd, n_ff, store, ids, w, x, 7.0)
    ng = int(keep["ng"].item())
    assert ng == len({int(v) for v in ids.reshape(-1) if v >= 0})
    for i in range(n_tok):
        plan = api.make_plan(plan_ptr[i], plan_w[i])
        hq = T.zeros(k * (n_ff // 32) * 36, dtype=T.uint8, device="cuda")
        one = T.zeros(n_embd, dtype=T.float32, device="cuda")
        api.moe_gate_up(t, plan, k, n_embd, n_ff, 7.0, xq[i], hq)
        api.moe_down(t, plan, k, n_embd, n_ff, 2 * n_ff * H.row_bytes(t, n_embd), hq, None, one)
        assert T.equal(out[i], one), f"token {i}"
    # and against the oracle for the first token
    blobs = [store[int(e)].cpu().numpy() for e in ids[0]]
    want = oracle_plan(oracle, t, n_embd, n_ff, blobs, w[0], x[0], 7.0)
    assert H.rel_err(out[0].cpu().numpy(), want) <= TIGHT


# ------------------------------------------------------------------------------------------------ grouped (native) form
@pytest.mark.parametrize("t", [H.Q4_K, H.IQ2_S, H.Q6_K, H.IQ4_XS, H.IQ3_XXS])
def test_expert_grouped(T, api, oracle, t):
    n_embd, n_ff, n_tok = 512, 256, 6
    blobs = [expert_blob(t, n_embd, n_ff, e, False) for e in range(3)]
    store = dev(T, np.stack(blobs))
    x = H.rng_for("grp", t).standard_normal((n_tok, n_embd)).astype(np.float32)
    # group 0: tokens 0, 3, 5, 1, 2 (five entries: more than one pass of four columns); group 1: none; group 2: token 4
    grp_ptr = T.tensor([store[0].data_ptr(), store[1].data_ptr(), store[2].data_ptr(), 0], dtype=T.int64, device="cuda")
    grp_start = T.tensor([0, 5, 5, 6, 6], dtype=T.int32, device="cuda")
    ent_tok = T.tensor([0, 3, 5, 1, 2, 4, 0, 0], dtype=T.int32, device="cuda")
    ent_dst = T.tensor([5, 4, 3, 2, 1, 0, 0, 0], dtype=T.int32, device="cuda")
    n_groups = T.tensor([3], dtype=T.int32, device="cuda")
    L = api.native_expert_layout(t, t, n_embd, n_ff)
    xq = api.native_quantize_q8_1(dev(T, x))
    scratch = T.zeros(api.native_expert_scratch_bytes(8, n_ff), dtype=T.uint8, device="cuda")
    out = T.full((8, n_embd), 9.0, dtype=T.float32, device="cuda")
    api.native_expert_grouped(L, grp_ptr, grp_start, n_groups, ent_dst, ent_tok, 4, 8, xq, scratch, out)
    got = out.cpu().numpy()
    plan = [(0, 0, 5), (0, 3, 4), (0, 5, 3), (0, 1, 2), (0, 2, 1), (2, 4, 0)]
    for g, tok, dst in plan:
        want = oracle.expert_q8_1(t, t, blobs[g], n_embd, n_ff, H.INF, oracle.quantize_q8_1(x[tok]))
        assert H.rel_err(got[dst], want) <= TIGHT
    assert (got[6:] == 9.0).all()


@pytest.mark.parametrize("tg,tu,td", [(H.IQ2_S, H.IQ3_S, H.Q4_K), (H.Q4_K, H.Q8_0, H.IQ2_S), (H.Q8_0, H.IQ2_S, H.Q8_0),
                                      (H.IQ3_S, H.Q4_K, H.IQ3_S)])
def test_expert_grouped_mixed_gate_up_types(T, api, oracle, tg, tu, td):
    """native_expert_layout(gu_type, up_type, d_type, ...) with up rows of their own type (iq_kernels.hpp:73-77)."""
    n_embd, n_ff, n_tok = 512, 256, 6
    rng = H.rng_for("grp-mixed", tg, tu, td)
    blobs = [np.concatenate([H.constructed_blocks(tg, n_ff, n_embd, rng).reshape(-1),
                             H.constructed_blocks(tu, n_ff, n_embd, rng).reshape(-1),
                             H.constructed_blocks(td, n_embd, n_ff, rng).reshape(-1)]) for _ in range(2)]
    L = api.native_expert_layout(tg, td, n_embd, n_ff, up_type=tu)
    assert L.bytes == blobs[0].size and L.up_off == n_ff * H.row_bytes(tg, n_embd)
    store = dev(T, np.stack(blobs))
    x = rng.standard_normal((n_tok, n_embd)).astype(np.float32)
    grp_ptr = T.tensor([store[0].data_ptr(), store[1].data_ptr()], dtype=T.int64, device="cuda")
    grp_start = T.tensor([0, 5, 6], dtype=T.int32, device="cuda")          # five entries (two passes of columns), then one
    ent_tok = T.tensor([0, 3, 5, 1, 2, 4], dtype=T.int32, device="cuda")
    ent_dst = T.tensor([5, 4, 3, 2, 1, 0], dtype=T.int32, device="cuda")
    n_groups = T.tensor([2], dtype=T.int32, device="cuda")
    xq = api.native_quantize_q8_1(dev(T, x))
    scratch = T.zeros(api.native_expert_scratch_bytes(6, n_ff), dtype=T.uint8, device="cuda")
    out = T.full((6, n_embd), 9.0, dtype=T.float32, device="cuda")
    api.native_expert_grouped(L, grp_ptr, grp_start, n_groups, ent_dst, ent_tok, 2, 6, xq, scratch, out)
    got = out.cpu().numpy()
    for g, tok, dst in [(0, 0, 5), (0, 3, 4), (0, 5, 3), (0, 1, 2), (0, 2, 1), (1, 4, 0)]:
        want = oracle.expert_q8_1_mixed(tg, tu, td, blobs[g], n_embd, n_ff, H.INF, oracle.quantize_q8_1(x[tok]))
        assert H.rel_err(got[dst], want) <= TIGHT
    # the static-scratch entry point runs the same launches
    out2 = T.full((6, n_embd), 9.0, dtype=T.float32, device="cuda")
    api.native_expert_grouped_static(L, grp_ptr, grp_start, n_groups, ent_dst, ent_tok, 2, 6, xq, out2)
    assert T.equal(out, out2)


def test_combine_bitwise(T, api, oracle):
    rng = H.rng_for("cmb")
    parts = rng.standard_normal((3, 8, 2048)).astype(np.float32)
    w = rng.random((3, 8)).astype(np.float32)
    sh = rng.standard_normal((3, 2048)).astype(np.float32)
    y = api.moe_combine(dev(T, parts), dev(T, w), dev(T, sh), 2048, 8, 3).cpu().numpy()
    for i in range(3):
        assert np.array_equal(y[i], oracle.combine_native(parts[i], w[i], sh[i]))
    y1 = api.moe_combine(dev(T, parts[0, :1]), dev(T, w[0, :1]), None, 2048, 1, 1).cpu().numpy()
    assert np.array_equal(y1[0], oracle.combine_native(parts[0, :1], w[0, :1]))


# ------------------------------------------------------------------------------------------------ synthetic weights
@pytest.mark.parametrize("t", TYPES)
def test_synth_weights_are_valid_blocks(T, api, oracle, t):
    n_rows, n_cols = 64, 2048
    blocks = api.synth_weights(t, 1234, 0.02, n_rows, n_cols).cpu().numpy()
    again = api.synth_weights(t, 1234, 0.02, n_rows, n_cols).cpu().numpy()
    assert np.array_equal(blocks, again)                                  # a pure function of (seed, shape)
    vals = oracle.dequantize(t, blocks, n_rows * n_cols)
    assert np.isfinite(vals).all()
    assert 0.7 < float(vals.std()) / 0.02 < 1.3                           # N(0, 0.02) rounded to the type's grid
    assert abs(float(vals.mean())) < 2e-3
    other = api.synth_weights(t, 1235, 0.02, n_rows, n_cols).cpu().numpy()
    assert not np.array_equal(blocks, other)


# ------------------------------------------------------------------------------------------------ prefill grouping
@pytest.mark.parametrize("n_tok,k,E", [(4096, 8, 256), (33, 3, 12), (1, 8, 64), (1500, 8, 2048)])
def test_expert_group_matches_oracle(T, api, oracle, n_tok, k, E):
    rng = H.rng_for("group", n_tok, E)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(n_tok)]).astype(np.int32)
    counts, bounds, pos, row_tok = api.expert_group(dev(T, ids), E)
    c_o, b_o, p_o, r_o = oracle.expert_group(ids, k, E)
    assert np.array_equal(counts.cpu().numpy(), c_o) and np.array_equal(bounds.cpu().numpy(), b_o)
    assert np.array_equal(pos.cpu().numpy(), p_o) and np.array_equal(row_tok.cpu().numpy(), r_o)
    rows = np.sort(pos.cpu().numpy())
    assert np.array_equal(rows, np.arange(n_tok * k))                    # a permutation of the sorted rows


def test_swiglu_rows_and_combine_rows(T, api, oracle):
    rng = H.rng_for("glue")
    rows, n_ff, n_embd, n_tok, k = 24, 64, 96, 3, 8
    gu = (rng.standard_normal((rows, 2 * n_ff)) * 4).astype(np.float32)
    h = api.swiglu_rows(dev(T, gu), n_ff, 7.0).cpu().numpy()
    want = np.stack([oracle.swiglu(gu[r, :n_ff], gu[r, n_ff:], 7.0) for r in range(rows)])
    assert np.allclose(h, want, rtol=2e-6, atol=1e-6)
    out = rng.standard_normal((rows, n_embd)).astype(np.float32)
    pos = rng.permutation(rows)[: n_tok * k].astype(np.int32)
    w = rng.random((n_tok, k)).astype(np.float32)
    sh = rng.standard_normal((n_tok, n_embd)).astype(np.float32)
    ffn = api.moe_combine_rows(dev(T, out), dev(T, pos), dev(T, w), dev(T, sh), n_tok, k, n_embd).cpu().numpy()
    for t in range(n_tok):
        assert np.array_equal(ffn[t], oracle.combine_down(out[pos[t * k:(t + 1) * k]], w[t], sh[t]))
