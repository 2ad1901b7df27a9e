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


def _ref_token_mixed(T, R, refgpu, cfg, ptr_of, type_of, ids_row, w_row, x_row, bufs):
    """One token through glmf::quantize_q8_1 + moe_gate_up + moe_down, once per storage type among its experts (plan
    entries of the other types are null: the reference's kernels add nothing for them); the types' results add up."""
    Hd, FF, k = cfg["n_embd"], cfg["n_ff"], cfg["k"]
    L, s, p = R.lib, R._stream(), refgpu._p
    bufs["xf"].copy_(x_row.float().reshape(-1))
    R._ck("quantize", L.ref_quantize_q8_1(p(bufs["xf"]), p(bufs["xq"]), Hd, s))
    total = T.zeros(Hd, dtype=T.float32, device="cuda")
    ids_h = [int(v) for v in ids_row.tolist()]
    for t in sorted({type_of(e) for e in ids_h}):
        ptrs = [ptr_of(e) if type_of(e) == t else 0 for e in ids_h]
        bufs["plan_ptr"][:k] = T.tensor(ptrs, dtype=T.int64, device="cuda")
        bufs["plan_w"][:k] = w_row
        R._ck("moe_gate_up", L.ref_moe_gate_up(t, p(bufs["plan_ptr"]), p(bufs["plan_w"]), k, Hd, FF, float("inf"), p(bufs["xq"]),
                                               p(bufs["hq"]), None, 8, None, 0, None, s))
        R._ck("moe_down", L.ref_moe_down(t, p(bufs["plan_ptr"]), p(bufs["plan_w"]), None, p(bufs["cpu_flag"]), k, Hd, FF,
                                         2 * FF * H.row_bytes(t, Hd), p(bufs["hq"]), None, p(bufs["out"]), s))
        total += bufs["out"]
    return total


def _ref_bufs(T, cfg):
    Hd, FF = cfg["n_embd"], cfg["n_ff"]
    return dict(xf=T.empty(Hd, dtype=T.float32, device="cuda"), xq=T.empty(Hd // 32 * 36, dtype=T.uint8, device="cuda"),
                plan_ptr=T.zeros(8, dtype=T.int64, device="cuda"), plan_w=T.zeros(8, dtype=T.float32, device="cuda"),
                hq=T.empty(8 * (FF // 32) * 36, dtype=T.uint8, device="cuda"), out=T.empty(Hd, dtype=T.float32, device="cuda"),
                cpu_flag=T.zeros(16, dtype=T.int32, device="cuda"))


def test_prompt_path_c5_batch64_full_shape_matches_reference_decode_kernels(T, api, refgpu):
    """C5's 64-token batch at its full shape (256 IQ3_S experts, Zipf-skewed) through the prompt path (tensor-core grouped
    product over f16 operands) against the reference's decode kernels token by token: every one of the 64 tokens."""
    cfg = H.CONFIGS["C5"]
    E, k, Hd = cfg["n_expert"], cfg["k"], cfg["n_embd"]
    lc, experts, _ = build(T, api, cfg, E, seed=53)
    logits = dev(T, H.router_logits("C5", 64, E, cfg["zipf"], seed=5))
    x = dev(T, H.activations("C5", 64, Hd, "bf16", seed=5), T.bfloat16)
    pf = api.MoePrefill(lc, experts, max_tokens=64)
    ids, w, ffn = pf.forward(logits, x)
    T.cuda.synchronize()
    assert pf.error() == 0
    R = refgpu.RefGpu()
    ids_r, w_r = R.router(logits, k)
    assert T.equal(ids, ids_r) and float((w - w_r).abs().max()) <= 1e-6
    bufs = _ref_bufs(T, cfg)
    worst = 0.0
    with T.cuda.stream(T.cuda.Stream()):
        for t in range(64):
            want = _ref_token_mixed(T, R, refgpu, cfg, lambda e: experts.data_ptr() + e * experts.stride(0),
                                    lambda e: cfg["gu_type"], ids_r[t], w_r[t], x[t], bufs)
            T.cuda.current_stream().synchronize()
            worst = max(worst, rel(T, ffn[t], want))
    print(f"C5 batch 64, prompt path vs reference decode kernels: worst {worst:.3g}")
    assert worst <= TOL, worst


def test_prompt_path_c4_full_shape_matches_reference_decode_kernels(T, api, refgpu):
    """C4 at its full shape (4096 tokens, 256 experts, half Q8_0 and half Q4_K) through the prompt path; 64 tokens spread
    over the chunk against the reference's DECODE kernels (one pass per storage type of a token's experts).  All 4096
    tokens' ids and routing weights must agree.  The outputs are bounded at 5e-2 only: for Q4_K the reference's decode
    dot multiplies a group's constant term -dmin * m by the sum of the ROUNDED activations (native_mmvq.cu:170,
    glm_fast.cu:238), while its prompt path - llama.cpp's MMQ, which this path follows and tests/test_gpu_prefill.py pins
    to the reference's host model of it at 1e-3 per product - multiplies it by the stored sum of the unquantized ones;
    the reference's two paths are 1e-2 .. 3e-2 apart on an expert of such weights."""
    from test_gpu_prefill import build_pools
    c = H.CONFIGS["C4"]
    cfg = dict(n_embd=c["n_embd"], n_ff=c["n_ff"], n_expert=c["n_expert"], k=c["k"])
    n_tok, E = c["T"], c["n_expert"]
    types = H.expert_types("C4", E, c["types"])
    pools, where = build_pools(T, api, cfg, types, 5000)
    lc = api.MoeLayerConfig(cfg["n_embd"], cfg["n_ff"], E, cfg["k"], H.Q8_0, H.Q8_0)
    logits = dev(T, H.router_logits("c4", n_tok, E, None))
    x = dev(T, H.activations("c4", n_tok, cfg["n_embd"], "bf16"), T.bfloat16)
    pf = api.MoePrefill(lc, None, max_tokens=n_tok, pools=pools)
    ids, w, ffn = pf.forward(logits, x)
    T.cuda.synchronize()
    assert pf.error() == 0
    R = refgpu.RefGpu()
    ids_r, w_r = R.router(logits, cfg["k"])
    assert T.equal(ids, ids_r) and float((w - w_r).abs().max()) <= 1e-6          # all 4096 tokens
    bufs = _ref_bufs(T, cfg)

    def ptr_of(e):
        t, blobs, i = where[e]
        return blobs.data_ptr() + i * blobs.stride(0)

    worst = 0.0
    with T.cuda.stream(T.cuda.Stream()):
        for t in range(0, n_tok, n_tok // 64):
            want = _ref_token_mixed(T, R, refgpu, cfg, ptr_of, lambda e: int(where[e][0]), ids_r[t], w_r[t], x[t], bufs)
            T.cuda.current_stream().synchronize()
            worst = max(worst, rel(T, ffn[t], want))
    print(f"C4, prompt path vs reference decode kernels on 64 of 4096 tokens: worst {worst:.3g}")
    assert worst <= 5e-2, worst


@pytest.mark.parametrize("t", list(H.MORE_TYPES))
def test_further_block_types_match_reference_kernels(T, api, refgpu, t):
    """Q5_K, Q6_K, IQ4_XS, IQ3_XXS, IQ2_XXS experts (random valid blocks) through glmf::moe_gate_up / moe_down and through
    maya_moe_layer_decode's staged kernels, 16 tokens; and the 8-token window against glmf::moe_win_experts."""
    n_embd, n_ff, E, k = 2048, 1024, 16, 8
    rng = H.rng_for("ref-more", t)
    experts = dev(T, np.stack([H.constructed_expert(t, t, n_embd, n_ff, rng) for _ in range(E)]))
    lc = api.MoeLayerConfig(n_embd, n_ff, E, k, t, t)
    ours = api.MoeLayer(lc, experts, None)
    ref = refgpu.RefLayer(refgpu.RefGpu(), n_embd, n_ff, E, k, t, t, H.row_bytes, experts)
    logits = dev(T, rng.standard_normal((16, E)).astype(np.float32))
    x = dev(T, rng.standard_normal((16, n_embd)).astype(np.float32))
    worst = 0.0
    with T.cuda.stream(T.cuda.Stream()):
        for i in range(16):
            ids, w, out = ours.forward(logits[i:i + 1], x[i:i + 1])
            ids_r, w_r, out_r = ref.forward(logits[i:i + 1], x[i:i + 1])
            assert T.equal(ids, ids_r)
            worst = max(worst, rel(T, out[0], out_r))
    print(f"type {t}: worst relative difference from the reference kernels over 16 tokens: {worst:.3g}")
    assert worst <= TIGHT, worst
