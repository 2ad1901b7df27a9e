"""The live pin: the SAME expert blobs, logits and activations through the reference's own CUDA kernels (compiled for
sm_100a from the reference tree by oracle/build.py into oracle/_ref/libmaya_ref_gpu.so: router_top10, glmf::quantize_q8_1,
native_mmvq, glmf::swiglu_q8, glmf::moe_gate_up, glmf::moe_down, glmf::moe_win_experts, native_expert_grouped) and
through this library's entry points, on one B200.  Expert ids bit-exact, routing weights to 1e-6, FFN outputs within the
stated 1e-2 (max |a - b| / max |b|; what is reached is 1e-6 .. 2e-4: both sides do the same integer dots and differ in the
order and contraction of the FP32 operations).  Configurations C1, C2, C3 and C5 at their full shapes, 64 seeded tokens each.

Skipped when the reference library is not built (the reference tree is not on the GPU box; the prebuilt file travels)."""
import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu
TOL, TIGHT = 1e-2, 1e-3


@pytest.fixture(scope="module")
def T(cuda):
    import torch
    return torch


@pytest.fixture(scope="module")
def api(cuda):
    from project_maya_b200 import api as a
    return a


@pytest.fixture(scope="module")
def refgpu(cuda):
    from oracle import ref_gpu
    if not ref_gpu.available():
        pytest.skip("oracle/_ref/libmaya_ref_gpu.so not built (python oracle/build.py with the reference tree present)")
    return ref_gpu


def dev(T, a, dtype=None):
    t = T.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def build(T, api, cfg, n_expert, seed):
    from test_gpu_layer import synth_layer
    return synth_layer(T, api, cfg, n_expert, seed)


def rel(T, got, want):
    return float((got.double() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


@pytest.mark.parametrize("name,n_tokens", [("C1", 16), ("C2", 64), ("C5", 64)])
def test_single_token_layer_matches_reference_kernels(T, api, refgpu, name, n_tokens):
    cfg = H.CONFIGS[name]
    lc, experts, shared = build(T, api, cfg, cfg["n_expert"], seed=41)
    ours = api.MoeLayer(lc, experts, shared)
    ref = refgpu.RefLayer(refgpu.RefGpu(), cfg["n_embd"], cfg["n_ff"], cfg["n_expert"], cfg["k"], cfg["gu_type"], cfg["d_type"],
                          H.row_bytes, experts, shared, cfg.get("n_ff_sh", 0), cfg.get("sh_gu_type", H.Q8_0))
    logits = dev(T, H.router_logits(name, n_tokens, cfg["n_expert"], cfg.get("zipf"), seed=3))
    x = dev(T, H.activations(name, n_tokens, cfg["n_embd"], cfg["act"], seed=3), T.bfloat16 if cfg["act"] == "bf16" else None)
    worst = 0.0
    T.cuda.synchronize()
    with T.cuda.stream(T.cuda.Stream()):                # the reference's native_* calls refuse the null stream
        for t in range(n_tokens):
            ids, w, out = ours.forward(logits[t:t + 1], x[t:t + 1])
            ids_r, w_r, out_r = ref.forward(logits[t:t + 1], x[t:t + 1])
            assert T.equal(ids, ids_r), f"token {t}: expert ids differ from the reference router"
            assert float((w - w_r).abs().max()) <= 1e-6
            e = rel(T, out[0], out_r)
            worst = max(worst, e)
            assert e <= TOL, f"token {t}: {e}"
    print(f"{name}: worst relative difference from the reference kernels over {n_tokens} tokens: {worst:.3g}")
    assert worst <= TIGHT, worst
    assert ours.error() == 0


def test_c3_window_matches_reference_window_kernel(T, api, refgpu):
    """Eight tokens at once (C3: Q4_K, hidden 7168, 256 experts, Zipf-skewed so that tokens share experts) through
    glmf::moe_win_experts and through maya_moe_layer_decode's window path."""
    cfg = H.CONFIGS["C3"]
    E, k, Hd, FF = cfg["n_expert"], cfg["k"], cfg["n_embd"], cfg["n_ff"]
    lc, experts, _ = build(T, api, cfg, E, seed=43)
    ours = api.MoeLayer(lc, experts, None)
    R = refgpu.RefGpu()
    L, s = R.lib, R._stream()
    down_off = 2 * FF * H.row_bytes(cfg["gu_type"], Hd)
    for rep in range(8):
        logits = dev(T, H.router_logits("C3", 8, E, cfg["zipf"], seed=rep))
        x = dev(T, H.activations("C3", 8, Hd, "bf16", seed=rep), T.bfloat16)
        ids, w, out = ours.forward(logits, x)
        ids_r, w_r = R.router(logits, k)
        assert T.equal(ids, ids_r)
        assert len(T.unique(ids)) < 8 * k
        xf = x.float().contiguous()
        xq = T.empty((8, Hd // 32 * 36), dtype=T.uint8, device="cuda")
        for t in range(8):
            R._ck("quantize", L.ref_quantize_q8_1(refgpu._p(xf[t]), refgpu._p(xq[t]), Hd, s))
        plan_ptr = (ids_r.to(T.int64) * experts.stride(0) + experts.data_ptr()).contiguous()
        plan_w = w_r.contiguous()
        hq = T.empty(8 * 8 * (FF // 32) * 36, dtype=T.uint8, device="cuda")
        part = T.empty((8 * 8, Hd), dtype=T.float32, device="cuda")
        out_r = T.empty((8, Hd), dtype=T.float32, device="cuda")
        grp_ptr = T.zeros(64, dtype=T.int64, device="cuda")
        grp_start = T.zeros(65, dtype=T.int32, device="cuda")
        grp_ent = T.zeros(64, dtype=T.int32, device="cuda")
        n_groups = T.zeros(1, dtype=T.int32, device="cuda")
        cpu_flag = T.zeros(8, dtype=T.int32, device="cuda")      # read unconditionally by the reference's combine kernel
        p = refgpu._p
        R._ck("moe_win_experts", L.ref_moe_win_experts(cfg["gu_type"], cfg["d_type"], p(plan_ptr), p(plan_w), None, p(cpu_flag),
                                                       p(xq), xq.stride(0),
                                                       p(hq), p(part), None, p(out_r), Hd, p(grp_ptr), p(grp_start), p(grp_ent),
                                                       p(n_groups), 8, k, Hd, FF, float("inf"), down_off, s))
        T.cuda.synchronize()
        e = rel(T, out, out_r)
        print(f"C3 window {rep}: {e:.3g}")
        assert e <= TOL and e <= TIGHT, e


@pytest.mark.parametrize("t", [H.Q4_K, H.IQ2_S, H.IQ3_S])
def test_expert_grouped_matches_reference_native_expert_grouped(T, api, refgpu, t):
    """maya_expert_grouped against native_expert_grouped (iq_kernels.cu:1120-1194) on the same groups and entries."""
    n_embd, n_ff, n_exp, n_tok = 2048, 1024, 6, 5
    cfg = dict(n_embd=n_embd, n_ff=n_ff, n_expert=n_exp, k=2, gu_type=t, d_type=t)
    lc, experts, _ = build(T, api, cfg, n_exp, seed=47)
    R = refgpu.RefGpu()
    x = dev(T, H.activations("grouped", n_tok, n_embd, "f32"))
    xq = T.empty((n_tok, n_embd // 32 * 36), dtype=T.uint8, device="cuda")
    R._ck("quantize rows", R.lib.ref_quantize_q8_1_rows(refgpu._p(x), n_tok, n_embd, refgpu._p(xq), R._stream()))
    # groups: expert 4 <- tokens 0, 3; expert 1 <- token 2; expert 5 <- tokens 1, 4, 0
    groups = [(4, [0, 3]), (1, [2]), (5, [1, 4, 0])]
    ent_tok = [tk for _, toks in groups for tk in toks]
    n_ent = len(ent_tok)
    grp_ptr = T.tensor([experts.data_ptr() + e * experts.stride(0) for e, _ in groups], dtype=T.int64, device="cuda")
    starts = np.cumsum([0] + [len(toks) for _, toks in groups]).astype(np.int32)
    grp_start = dev(T, starts)
    n_groups = dev(T, np.array([len(groups)], np.int32))
    ent_dst = dev(T, np.arange(n_ent, dtype=np.int32))
    ent_tok_d = dev(T, np.array(ent_tok, np.int32))
    p = refgpu._p
    out_r = T.zeros((n_ent, n_embd), dtype=T.float32, device="cuda")
    scr_r = T.zeros(int(R.lib.ref_native_expert_scratch_bytes(n_ent, n_ff)), dtype=T.uint8, device="cuda")
    R._ck("native_expert_grouped", R.lib.ref_native_expert_grouped(t, t, n_embd, n_ff, p(grp_ptr), p(grp_start), p(n_groups), p(ent_dst),
                                                                    p(ent_tok_d), len(groups), n_ent, p(xq), p(scr_r), p(out_r),
                                                                    R._stream(), float("inf")))
    Lo = api.native_expert_layout(t, t, n_embd, n_ff)
    scr = T.zeros(api.native_expert_scratch_bytes(n_ent, n_ff), dtype=T.uint8, device="cuda")
    out = T.zeros((n_ent, n_embd), dtype=T.float32, device="cuda")
    api.native_expert_grouped(Lo, grp_ptr, grp_start, n_groups, ent_dst, ent_tok_d, len(groups), n_ent, xq, scr, out)
    T.cuda.synchronize()
    e = rel(T, out, out_r)
    assert e <= TOL and e <= TIGHT, e
