"""A layer of a real GGUF against llama.cpp's own activations.

tests/golden/glm5_synth_moe_layer1.npz holds layer 1 of the synthetic GLM-5 GGUF the reference ships
(data/glm5-synth.gguf: F32 tensors, 12 experts of 128 x 64, top-3 sigmoid routing with selection bias and weight
scale 2.5, SwiGLU clamp 10, one shared expert) as read by project_maya_b200.gguf_loader, and llama.cpp's captured
tensors of that layer's MoE block for 8 tokens (data/glm5-synth-dumps): its input, the routing, the routed output,
the shared expert's output.  That pins the data path end to end - GGUF tensor order -> per-expert blobs, the router's
semantics, clamped SwiGLU, weighted combine, the shared expert's plain add - against outputs nobody here computed.

The tensors are F32, the kernels take quantized blocks: the experts are quantized to Q8_0 with the library's quantizer
first, so the comparison carries Q8_0's and q8_1's rounding (measured: 1.4e-2 to 1.7e-2 of the output's largest value); the
bound asserted is 3e-2, the reference's own gate for a quantized expert against the float one
(native_expert_parity.cpp:298-299).  The float64 evaluation of the same tensors matches the dumps to 1e-6, which is what
shows that the semantics are read correctly.
"""
from pathlib import Path

import numpy as np
import pytest

import helpers as H

GOLD = Path(__file__).resolve().parent / "golden" / "glm5_synth_moe_layer1.npz"
QUANT_TOL = 3e-2


@pytest.fixture(scope="module")
def g():
    return np.load(GOLD)


def swiglu64(gt, up, lim):
    gt = np.minimum(gt, lim)
    up = np.clip(up, -lim, lim)
    return gt / (1.0 + np.exp(-gt)) * up


def layer_tensors(g):
    from project_maya_b200.gguf_loader import MoeLayerTensors
    E, FF, Hd = g["gate"].shape
    return MoeLayerTensors(Hd, FF, E, g["gate"], g["up"], g["down"], None, g["router"], g["router_bias"], g["sh_gate"],
                           g["sh_up"], g["sh_down"])


def test_float_evaluation_reproduces_llama_cpp(g):
    """The dumps are what these tensors give in float: logits = ffn_gate_inp . x; routed output = sum of the captured
    weights times down(SwiGLU_clamped(gate x, up x)); shared output = the same with the shared tensors; out = their sum."""
    x = g["x"].astype(np.float64)
    assert np.abs(x @ g["router"].astype(np.float64).T - g["logits"]).max() <= 1e-5
    lim, lim_sh = float(g["clamp"]), float(g["clamp_sh"])
    moe = np.zeros_like(x)
    for t in range(x.shape[0]):
        for j, e in enumerate(g["ids"][t]):
            h = swiglu64(g["gate"][e].astype(np.float64) @ x[t], g["up"][e].astype(np.float64) @ x[t], lim)
            moe[t] += float(g["weights"][t, j]) * (g["down"][e].astype(np.float64) @ h)
    sh = np.stack([g["sh_down"].astype(np.float64) @ swiglu64(g["sh_gate"].astype(np.float64) @ x[t],
                                                              g["sh_up"].astype(np.float64) @ x[t], lim_sh) for t in range(x.shape[0])])
    assert H.rel_err(moe, g["moe_out"]) <= 1e-5
    assert H.rel_err(sh, g["shexp"]) <= 1e-5
    assert np.array_equal(g["moe_out"] + g["shexp"], g["out"])


def test_oracle_router_matches_llama_cpp(g, oracle):
    ids, w = oracle.router_sigmoid(g["logits"], g["router_bias"], g["ids"].shape[1], float(g["w_scale"]), True)
    assert np.array_equal(ids, g["ids"])
    assert np.abs(w - g["weights"]).max() <= 1e-6


def test_blobs_from_gguf_tensors(g, oracle):
    """The loader's blob of expert e is [gate rows | up rows | down rows]: dequantizing it gives the GGUF rows back to
    Q8_0's rounding."""
    from project_maya_b200 import gguf_loader
    L = layer_tensors(g)
    blobs = gguf_loader.expert_blobs(L, H.Q8_0)
    assert blobs.shape == (L.n_expert, H.blob_bytes(H.Q8_0, H.Q8_0, L.n_embd, L.n_ff))
    gu = L.n_ff * H.row_bytes(H.Q8_0, L.n_embd)
    for e in (0, 5, 11):
        gate = oracle.dequantize(H.Q8_0, blobs[e, :gu], L.n_ff * L.n_embd).reshape(L.n_ff, L.n_embd)
        up = oracle.dequantize(H.Q8_0, blobs[e, gu:2 * gu], L.n_ff * L.n_embd).reshape(L.n_ff, L.n_embd)
        down = oracle.dequantize(H.Q8_0, blobs[e, 2 * gu:], L.n_embd * L.n_ff).reshape(L.n_embd, L.n_ff)
        for got, want in ((gate, g["gate"][e]), (up, g["up"][e]), (down, g["down"][e])):
            assert np.abs(got - want).max() <= np.abs(want).max() / 127.0 * 0.51


def test_oracle_layer_matches_llama_cpp(g, oracle):
    """The CPU oracle (q8_1 activations x Q8_0 blocks, the reference GPU path's arithmetic) on the GGUF layer."""
    from project_maya_b200 import gguf_loader
    L = layer_tensors(g)
    blobs, sh = gguf_loader.expert_blobs(L, H.Q8_0), gguf_loader.shared_blob(L, H.Q8_0)
    lim = float(g["clamp"])
    moe, shx = np.zeros_like(g["moe_out"]), np.zeros_like(g["shexp"])
    for t in range(g["x"].shape[0]):
        xq = oracle.quantize_q8_1(g["x"][t])
        parts = np.stack([oracle.expert_q8_1(H.Q8_0, H.Q8_0, blobs[e], L.n_embd, L.n_ff, lim, xq) for e in g["ids"][t]])
        moe[t] = oracle.combine_down(parts, g["weights"][t])
        shx[t] = oracle.expert_q8_1(H.Q8_0, H.Q8_0, sh, L.n_embd, L.sh_gate.shape[0], float(g["clamp_sh"]), xq)
    assert H.rel_err(moe, g["moe_out"]) <= QUANT_TOL
    assert H.rel_err(shx, g["shexp"]) <= QUANT_TOL
    assert H.rel_err(moe + shx, g["out"]) <= QUANT_TOL


def hc_inputs(g, t):
    """Token t's hyper-connection inputs in the kernels' convention: comb dst-major (llama.cpp stores [src][dst])."""
    return g["hc_R_old"][t], g["hc_post"][t], np.ascontiguousarray(g["hc_comb_src_major"][t].T)


def test_oracle_hc_post_matches_llama_cpp(g, oracle):
    """What follows the MoE block: llama.cpp's residual stack after the layer (l_out) is the hyper-connection write of
    its ffn_out into the stack before it - the oracle's hc_post on the captured tensors, to float rounding (llama.cpp
    sums in another order)."""
    for t in range(g["x"].shape[0]):
        R_old, post, comb = hc_inputs(g, t)
        got = oracle.hc_post(g["out"][t], R_old, post, comb)
        assert np.abs(got - g["hc_R_new"][t]).max() <= 1e-6
        wrong = oracle.hc_post(g["out"][t], R_old, post, comb.T.copy())      # the dst/src mix-up must show
        assert np.abs(wrong - g["hc_R_new"][t]).max() > 1e-2


@pytest.mark.gpu
def test_hc_post_kernel_and_fused_epilogue(g, oracle, cuda):
    """maya_hc_post is the oracle bit for bit (same product and multiply-add chain), on llama.cpp's captured tensors
    and on a wide random case; the layer kernel's epilogue (maya_moe_layer_decode_hc) writes the same bits as the layer
    followed by the stand-alone launch, for one token (fused) and a window (staged)."""
    import torch as T
    from project_maya_b200 import api
    for t in range(g["x"].shape[0]):
        R_old, post, comb = hc_inputs(g, t)
        got = api.hc_post(*[T.from_numpy(np.ascontiguousarray(a)).cuda() for a in (g["out"][t], R_old, post, comb)])
        assert got.cpu().numpy().tobytes() == oracle.hc_post(g["out"][t], R_old, post, comb).tobytes()
        assert np.abs(got.cpu().numpy() - g["hc_R_new"][t]).max() <= 1e-6
    rng = np.random.default_rng(3)
    n = 6144
    b, R = rng.standard_normal(n).astype(np.float32), rng.standard_normal((4, n)).astype(np.float32)
    post, comb = rng.standard_normal(4).astype(np.float32), rng.standard_normal((4, 4)).astype(np.float32)
    got = api.hc_post(*[T.from_numpy(a).cuda() for a in (b, R, post, comb)])
    assert got.cpu().numpy().tobytes() == oracle.hc_post(b, R, post, comb).tobytes()
    with pytest.raises(api.MayaError):
        Rd = T.from_numpy(R).cuda()
        api.hc_post(T.from_numpy(b).cuda(), Rd, T.from_numpy(post).cuda(), T.from_numpy(comb).cuda(), R_new=Rd)

    cfg = api.MoeLayerConfig(1024, 512, 8, 2, H.Q8_0, H.Q8_0)
    experts = T.empty((8, cfg.blob_bytes), dtype=T.uint8, device="cuda")
    gu = 2 * 512 * H.row_bytes(H.Q8_0, 1024)
    for e in range(8):
        api.synth_weights(H.Q8_0, 2 * e, 0.02, 2 * 512, 1024, experts[e, :gu])
        api.synth_weights(H.Q8_0, 2 * e + 1, 0.02, 1024, 512, experts[e, gu:])
    layer = api.MoeLayer(cfg, experts, None)
    ld = T.from_numpy(H.router_logits("hc", 5, 8, 1.1)).cuda()
    xd = T.from_numpy(H.activations("hc", 5, 1024, "bf16")).to(T.bfloat16).cuda()
    for sl in (slice(0, 1), slice(1, 5)):                      # one token: the fused kernel; four: the staged kernels
        nt = sl.stop - sl.start
        R_old = T.from_numpy(rng.standard_normal((nt, 4, 1024)).astype(np.float32)).cuda()
        post_d = T.from_numpy(rng.standard_normal((nt, 4)).astype(np.float32)).cuda()
        comb_d = T.from_numpy(rng.standard_normal((nt, 4, 4)).astype(np.float32)).cuda()
        R_new = T.zeros((nt, 4, 1024), dtype=T.float32, device="cuda")
        plain = layer.forward(ld[sl], xd[sl])[2].clone()
        out = layer.forward(ld[sl], xd[sl], hc=(R_old, post_d, comb_d, R_new))[2]
        assert T.equal(out, plain)
        for t in range(nt):
            assert T.equal(R_new[t], api.hc_post(plain[t], R_old[t], post_d[t], comb_d[t]))


@pytest.mark.gpu
def test_kernels_on_gguf_layer_match_llama_cpp(g, oracle, cuda):
    """The CUDA path on the same layer: sigmoid router (ids exact), plan-form gate/up + down with the shared expert's
    down rows in the gate/up launch; against llama.cpp's dumps at the quantization bound and against the oracle tightly."""
    import torch as T
    from project_maya_b200 import api, gguf_loader
    L = layer_tensors(g)
    k, lim = g["ids"].shape[1], float(g["clamp"])
    blobs = T.from_numpy(gguf_loader.expert_blobs(L, H.Q8_0)).cuda()
    sh = T.from_numpy(gguf_loader.shared_blob(L, H.Q8_0)).cuda()
    n_ff_sh = L.sh_gate.shape[0]
    logits = T.from_numpy(g["logits"]).cuda()
    ids, w = api.router_sigmoid(logits, T.from_numpy(g["router_bias"]).cuda(), k, float(g["w_scale"]), True)
    assert np.array_equal(ids.cpu().numpy(), g["ids"])
    assert np.abs(w.cpu().numpy() - g["weights"]).max() <= 1e-6
    got = np.zeros_like(g["out"])
    want_oracle = np.zeros_like(g["out"])
    sh_down_off = 2 * n_ff_sh * H.row_bytes(H.Q8_0, L.n_embd)
    for t in range(g["x"].shape[0]):
        x = T.from_numpy(g["x"][t:t + 1]).cuda()
        xq = api.native_quantize_q8_1(x)
        plan_ptr = T.tensor([blobs[int(e)].data_ptr() for e in g["ids"][t]], dtype=T.int64, device="cuda")
        plan = api.make_plan(plan_ptr, w[t].contiguous())
        hq = T.zeros(k * (L.n_ff // 32) * 36, dtype=T.uint8, device="cuda")
        gu = api.native_mmvq(H.Q8_0, sh, xq, L.n_embd, 2 * n_ff_sh)
        sh_hq = api.swiglu_q8_1(gu[0, :n_ff_sh].contiguous(), gu[0, n_ff_sh:].contiguous(), float(g["clamp_sh"]))
        sh_out = T.zeros(L.n_embd, dtype=T.float32, device="cuda")
        out = T.zeros(L.n_embd, dtype=T.float32, device="cuda")
        api.moe_gate_up(H.Q8_0, plan, k, L.n_embd, L.n_ff, lim, xq, hq, sh[sh_down_off:], H.Q8_0, sh_hq, n_ff_sh, sh_out)
        api.moe_down(H.Q8_0, plan, k, L.n_embd, L.n_ff, 2 * L.n_ff * H.row_bytes(H.Q8_0, L.n_embd), hq, sh_out, out)
        T.cuda.synchronize()
        got[t] = out.cpu().numpy()
        xo = oracle.quantize_q8_1(g["x"][t])
        parts = np.stack([oracle.expert_q8_1(H.Q8_0, H.Q8_0, blobs[int(e)].cpu().numpy(), L.n_embd, L.n_ff, lim, xo)
                          for e in g["ids"][t]])
        sho = oracle.expert_q8_1(H.Q8_0, H.Q8_0, sh.cpu().numpy(), L.n_embd, n_ff_sh, float(g["clamp_sh"]), xo)
        want_oracle[t] = oracle.combine_down(parts, g["weights"][t], sho)
    assert H.rel_err(got, want_oracle) <= 2e-4
    assert H.rel_err(got, g["out"]) <= QUANT_TOL
    # the same layer through ONE call: maya_moe_layer_decode with its sigmoid-router option (selection bias, weight scale,
    # normalised weights) - the fused single-token kernel and the window path - gives the staged sequence's bits
    if float(g["clamp"]) == float(g["clamp_sh"]):
        lc = api.MoeLayerConfig(L.n_embd, L.n_ff, blobs.shape[0], k, H.Q8_0, H.Q8_0, n_ff_sh, H.Q8_0, H.Q8_0, lim)
        bias = T.from_numpy(g["router_bias"]).cuda()
        layer = api.MoeLayer(lc, blobs, sh, sigmoid=(bias, float(g["w_scale"]), True))
        xs = T.from_numpy(g["x"]).cuda()
        for t in range(g["x"].shape[0]):
            ids1, w1, out1 = layer.forward(logits[t:t + 1], xs[t:t + 1])
            assert np.array_equal(ids1.cpu().numpy()[0], g["ids"][t])
            assert out1.cpu().numpy()[0].tobytes() == got[t].tobytes()
        nwin = min(g["x"].shape[0], 16)
        ids_w, _, out_w = layer.forward(logits[:nwin], xs[:nwin])
        assert np.array_equal(ids_w.cpu().numpy(), g["ids"][:nwin])
        assert out_w.cpu().numpy().tobytes() == got[:nwin].tobytes()
