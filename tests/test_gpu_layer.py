"""The whole decode layer (route -> experts -> combine, shared expert alongside) through maya_moe_layer_decode, on
the benchmark configurations: C1 in full against the committed fixtures; C2 / C3 / C5 at their full shapes on
synthetic device-generated experts, checked against the oracle on the experts each token actually routed, and
through size-independent properties (window == token by token bit for bit; the expert-parallel partition's partial
outputs sum to the unpartitioned output)."""
import hashlib
import sys
from pathlib import Path

import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
TOL, TIGHT = 1e-2, 2e-4


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


def layer_cfg(api, cfg, with_shared=True):
    return api.MoeLayerConfig(cfg["n_embd"], cfg["n_ff"], cfg["n_expert"], cfg["k"], cfg["gu_type"], cfg["d_type"],
                              cfg.get("n_ff_sh", 0) if with_shared else 0, cfg.get("sh_gu_type", H.Q8_0),
                              cfg.get("sh_d_type", H.Q8_0), cfg.get("limit", H.INF))


def synth_layer(T, api, cfg, n_expert, seed):
    """n_expert synthetic experts (N(0, 0.02) quantized on the device) + the shared expert when the config has one."""
    lc = layer_cfg(api, dict(cfg, n_expert=n_expert))
    experts = T.empty((n_expert, lc.blob_bytes), dtype=T.uint8, device="cuda")
    H_, FF = cfg["n_embd"], cfg["n_ff"]
    gu_bytes = 2 * FF * H.row_bytes(cfg["gu_type"], H_)
    for e in range(n_expert):
        api.synth_weights(cfg["gu_type"], seed * 100003 + 2 * e, 0.02, 2 * FF, H_, experts[e, :gu_bytes])
        api.synth_weights(cfg["d_type"], seed * 100003 + 2 * e + 1, 0.02, H_, FF, experts[e, gu_bytes:])
    shared = None
    if cfg.get("n_ff_sh"):
        shared = T.empty(lc.shared_bytes, dtype=T.uint8, device="cuda")
        sgu = 2 * cfg["n_ff_sh"] * H.row_bytes(cfg["sh_gu_type"], H_)
        api.synth_weights(cfg["sh_gu_type"], seed * 7 + 1, 0.02, 2 * cfg["n_ff_sh"], H_, shared[:sgu])
        api.synth_weights(cfg["sh_d_type"], seed * 7 + 2, 0.02, H_, cfg["n_ff_sh"], shared[sgu:])
    T.cuda.synchronize()
    return lc, experts, shared


def oracle_token(oracle, cfg, experts, shared, ids, w, x, limit=H.INF):
    """The oracle on one token, given the routing: only the routed experts' blobs are brought to the host."""
    H_, FF, k = cfg["n_embd"], cfg["n_ff"], cfg["k"]
    xq = oracle.quantize_q8_1(x)
    parts = np.stack([oracle.expert_q8_1(cfg["gu_type"], cfg["d_type"], experts[int(e)].cpu().numpy(), H_, FF, limit, xq)
                      for e in ids])
    sh = None
    if shared is not None:
        sh = oracle.expert_q8_1(cfg["sh_gu_type"], cfg["sh_d_type"], shared.cpu().numpy(), H_, cfg["n_ff_sh"], limit, xq)
    return oracle.combine_down(parts, w, sh)


def test_c1_full_against_fixtures(T, api, oracle):
    sys.path.insert(0, str(GOLDEN))
    import make_golden
    g = np.load(GOLDEN / "c1_reference_cpu.npz")
    cfg = H.CONFIGS["C1"]
    blobs = make_golden.c1_experts()
    assert hashlib.sha256(blobs.tobytes()).hexdigest() == str(g["experts_sha256"])
    layer = api.MoeLayer(layer_cfg(api, cfg), dev(T, blobs))
    logits = H.router_logits("C1", cfg["tokens"], cfg["n_expert"], None)
    x = H.activations("C1", cfg["tokens"], cfg["n_embd"], "f32")
    for t in range(cfg["tokens"]):                      # batch 1, 16 seeded tokens
        ids, w, out = layer.forward(dev(T, logits[t:t + 1]), dev(T, x[t:t + 1]))
        assert np.array_equal(ids.cpu().numpy()[0], g["ids"][t])                       # routing bit-exact
        assert (np.abs(w.cpu().numpy()[0] - g["weights"][t]) / g["weights"][t]).max() <= 1e-5
        o = out.cpu().numpy()[0]
        assert H.rel_err(o, g["out_oracle_q8_1"][t]) <= TOL
        assert H.rel_err(o, g["out_oracle_q8_1"][t]) <= TIGHT
        # against the reference's CPU rows (Q8_K activations): the gate the reference holds its own two paths to
        assert H.rel_err(o, g["out_cpu_rows"][t]) <= 3e-2
    # the same 16 tokens as one window: the same bits
    ids16, w16, out16 = layer.forward(dev(T, logits), dev(T, x))
    for t in range(cfg["tokens"]):
        _, _, one = layer.forward(dev(T, logits[t:t + 1]), dev(T, x[t:t + 1]))
        assert T.equal(out16[t], one[0])


@pytest.mark.parametrize("name,n_tok_check", [("C2", 3), ("C5", 2)])
def test_full_shape_single_token(T, api, oracle, name, n_tok_check):
    cfg = H.CONFIGS[name]
    lc, experts, shared = synth_layer(T, api, cfg, cfg["n_expert"], seed=11)
    layer = api.MoeLayer(lc, experts, shared)
    logits = H.router_logits(name, 8, cfg["n_expert"], cfg.get("zipf"))
    x = H.activations(name, 8, cfg["n_embd"], cfg["act"])
    ids_o, w_o = oracle.router_top10(logits, cfg["k"])
    for t in range(n_tok_check):
        xd = dev(T, x[t:t + 1], T.bfloat16)
        ids, w, out = layer.forward(dev(T, logits[t:t + 1]), xd)
        assert np.array_equal(ids.cpu().numpy()[0], ids_o[t])
        want = oracle_token(oracle, cfg, experts, shared, ids_o[t], w_o[t], x[t])
        got = out.cpu().numpy()[0]
        assert H.rel_err(got, want) <= TOL
        assert H.rel_err(got, want) <= TIGHT


def test_c3_window_of_eight(T, api, oracle):
    cfg = H.CONFIGS["C3"]
    n_expert = 64                                       # reduced expert count, full hidden / FFN widths
    lc, experts, _ = synth_layer(T, api, cfg, n_expert, seed=5)
    layer = api.MoeLayer(lc, experts)
    logits = H.router_logits("C3", 8, n_expert, cfg["zipf"])
    x = H.activations("C3", 8, cfg["n_embd"], "bf16")
    ids, w, out = layer.forward(dev(T, logits), dev(T, x, T.bfloat16))
    ids_o, w_o = oracle.router_top10(logits, cfg["k"])
    assert np.array_equal(ids.cpu().numpy(), ids_o)
    assert len(np.unique(ids_o)) < 8 * cfg["k"]         # the skew makes tokens share experts
    for t in range(8):
        _, _, one = layer.forward(dev(T, logits[t:t + 1]), dev(T, x[t:t + 1], T.bfloat16))
        assert T.equal(out[t], one[0])                  # window == token by token, bit for bit
    want = oracle_token(oracle, dict(cfg, n_expert=n_expert), experts, None, ids_o[0], w_o[0], x[0])
    assert H.rel_err(out[0].cpu().numpy(), want) <= TIGHT


def test_expert_parallel_partition_sums_to_whole(T, api, oracle):
    cfg = dict(H.CONFIGS["C5"], n_expert=32)
    lc, experts, _ = synth_layer(T, api, cfg, 32, seed=9)
    logits = H.router_logits("C5", 4, 32, 1.1)
    x = H.activations("C5", 4, cfg["n_embd"], "bf16")
    ld, xd = dev(T, logits), dev(T, x, T.bfloat16)
    _, _, whole = api.MoeLayer(lc, experts).forward(ld, xd)
    parts = []
    for n_ranks in (2, 8):
        per = 32 // n_ranks
        partial = [api.MoeLayer(lc, experts, expert_range=(r * per, (r + 1) * per)).forward(ld, xd)[2].cpu().numpy()
                   for r in range(n_ranks)]
        summed = np.stack([oracle.allreduce_in_order(np.stack([p[t] for p in partial])) for t in range(4)])
        parts.append(summed)
        assert H.rel_err(summed, whole.cpu().numpy()) <= 1e-5
    # a rank with none of a token's experts contributes exact zeros
    empty = api.MoeLayer(lc, experts, expert_range=(0, 0)).forward(ld, xd)[2]
    assert not bool(empty.any())


@pytest.mark.parametrize("n_ranks", [2, 8])
def test_width_sliced_shared_expert_sums_to_whole(T, api, oracle, n_ranks):
    """Expert-parallel ranks that each hold 1/n of the shared expert's FFN width (its gate/up rows and the same
    columns of the down rows): the rank-ordered sum of the partial outputs is the one-rank output up to the order of
    the shared expert's down sums; a slice that the staged kernels would have to run is refused."""
    cfg = dict(H.CONFIGS["C2"], n_expert=16)
    lc, experts, shared = synth_layer(T, api, cfg, 16, seed=21)
    logits = H.router_logits("C2", 3, 16, 1.1)
    x = H.activations("C2", 3, cfg["n_embd"], "bf16")
    ld, xd = dev(T, logits), dev(T, x, T.bfloat16)
    per, wid = 16 // n_ranks, cfg["n_ff_sh"] // n_ranks
    for t in range(3):
        whole = api.MoeLayer(lc, experts, shared).forward(ld[t:t + 1], xd[t:t + 1])[2].cpu().numpy()[0]
        partial = [api.MoeLayer(lc, experts, shared, expert_range=(r * per, (r + 1) * per),
                                shared_range=(r * wid, (r + 1) * wid)).forward(ld[t:t + 1], xd[t:t + 1])[2].cpu().numpy()[0]
                   for r in range(n_ranks)]
        summed = oracle.allreduce_in_order(np.stack(partial))
        assert H.rel_err(summed, whole) <= 1e-5
        assert np.abs(partial[-1]).max() > 0            # every rank carries a share
    sliced = api.MoeLayer(lc, experts, shared, shared_range=(0, wid))
    with pytest.raises(api.MayaError):
        sliced.forward(ld[:2], xd[:2])                   # two tokens: the staged kernels do not slice
    with pytest.raises(api.MayaError):
        api.MoeLayer(lc, experts, shared, shared_range=(16, wid)).forward(ld[:1], xd[:1])     # not a multiple of 32


@pytest.mark.parametrize("n_ranks", [2, 4, 8])
def test_width_sliced_experts_sum_to_whole(T, api, oracle, n_ranks):
    """Tensor-parallel ranks: every rank holds FFN rows [r * n_ff / N, (r + 1) * n_ff / N) of EVERY expert as blobs of
    their own (api.width_slice) and runs the same layer kernel on them; routing is replicated (same ids on every rank),
    the rank-ordered sum of the partial outputs is the one-rank output up to the order of the down sums.  At N = 8 a
    slice is one 256-value block wide."""
    cfg = dict(H.CONFIGS["C2"], n_expert=16)
    lc, experts, shared = synth_layer(T, api, cfg, 16, seed=23)
    logits = H.router_logits("C2", 3, 16, 1.1)
    x = H.activations("C2", 3, cfg["n_embd"], "bf16")
    ld, xd = dev(T, logits), dev(T, x, T.bfloat16)
    wid = cfg["n_ff"] // n_ranks
    ranks = []
    for r in range(n_ranks):
        c, ex, sh = api.width_slice(lc, experts, shared, r * wid, (r + 1) * wid)
        assert c.n_ff == wid and ex.shape == (16, c.blob_bytes) and sh.numel() == c.shared_bytes
        ranks.append(api.MoeLayer(c, ex, sh))
    whole_layer = api.MoeLayer(lc, experts, shared)
    for t in range(3):
        ids0, w0, whole = whole_layer.forward(ld[t:t + 1], xd[t:t + 1])
        parts = []
        for L in ranks:
            ids, w, out = L.forward(ld[t:t + 1], xd[t:t + 1])
            assert T.equal(ids, ids0) and T.equal(w, w0)
            parts.append(out.cpu().numpy()[0])
        assert H.rel_err(oracle.allreduce_in_order(np.stack(parts)), whole.cpu().numpy()[0]) <= 1e-5
        assert min(np.abs(p).max() for p in parts) > 0
    with pytest.raises(ValueError):
        api.width_slice(lc, experts, shared, 0, 100)       # not whole blocks


@pytest.mark.parametrize("t,shared", [(H.Q4_K, False), (H.Q8_0, False), (H.IQ2_S, True), (H.IQ3_S, True), (H.IQ3_S, False)])
@pytest.mark.parametrize("n_ff", [768, 256])
def test_fused_token_kernel_equals_staged_kernels_bitwise(T, api, oracle, t, shared, n_ff):
    """One token through the single fused kernel and through the separate launches: the same bits, and the oracle's
    values.  Odd sizes on purpose: the FFN and output rows do not divide evenly over the blocks.  FFN width 256 leaves
    fewer 32-row units than half the grid: the kernel then cuts every unit in two for two blocks."""
    n_embd, n_expert, k = 1024, 20, 6
    cfg = dict(n_embd=n_embd, n_ff=n_ff, n_expert=n_expert, k=k, gu_type=t, d_type=t, limit=7.0)
    if shared:
        cfg.update(n_ff_sh=512, sh_gu_type=H.Q8_0, sh_d_type=H.Q8_0)
    lc, experts, sh = synth_layer(T, api, cfg, n_expert, seed=21)
    lc.limit = 7.0
    fused = api.MoeLayer(lc, experts, sh, expert_range=(0, 17))
    staged = api.MoeLayer(lc, experts, sh, expert_range=(0, 17), staged=True)
    logits = H.router_logits("fused", 6, n_expert, 1.1)
    x = H.activations("fused", 6, n_embd, "bf16")
    ids_o, w_o = oracle.router_top10(logits, k)
    for i in range(6):
        ld, xd = dev(T, logits[i:i + 1]), dev(T, x[i:i + 1], T.bfloat16)
        ids_f, w_f, out_f = fused.forward(ld, xd)
        ids_s, w_s, out_s = staged.forward(ld, xd)
        assert T.equal(ids_f, ids_s) and T.equal(w_f, w_s)
        assert np.array_equal(ids_f.cpu().numpy()[0], ids_o[i])
        assert T.equal(out_f, out_s), f"token {i}"
    assert fused.error() == 0
    # f32 activations and the oracle, experts 17..19 left to "another rank"
    xf = H.activations("fused32", 1, n_embd, "f32")
    _, _, out = fused.forward(dev(T, logits[:1]), dev(T, xf))
    xq = oracle.quantize_q8_1(xf[0])
    parts = np.zeros((k, n_embd), np.float32)
    skip = np.zeros(k, np.uint8)
    for j, e in enumerate(ids_o[0]):
        if e < 17:
            parts[j] = oracle.expert_q8_1(t, t, experts[int(e)].cpu().numpy(), n_embd, n_ff, 7.0, xq)
        else:
            skip[j] = 1
    shv = oracle.expert_q8_1(H.Q8_0, H.Q8_0, sh.cpu().numpy(), n_embd, 512, 7.0, xq) if shared else None
    want = oracle.combine_down(parts, w_o[0], shv, skip)
    assert H.rel_err(out.cpu().numpy()[0], want) <= TIGHT


def test_fused_kernel_many_calls_one_scratch(T, api):
    """The grid barrier's counter lives in the scratch: hundreds of calls, single tokens and windows interleaved."""
    cfg = dict(n_embd=512, n_ff=256, n_expert=8, k=4, gu_type=H.Q4_K, d_type=H.Q4_K)
    lc, experts, _ = synth_layer(T, api, cfg, 8, seed=3)
    layer = api.MoeLayer(lc, experts)
    logits = dev(T, H.router_logits("many", 16, 8, None))
    x = dev(T, H.activations("many", 16, 512, "f32"))
    first = layer.forward(logits[:1], x[:1])[2].clone()
    for i in range(300):
        if i % 50 == 7:
            layer.forward(logits, x)              # a 16-token window through the staged kernels, same scratch
        out = layer.forward(logits[:1], x[:1])[2]
    T.cuda.synchronize()
    assert T.equal(out, first)
    assert layer.error() == 0


@pytest.mark.parametrize("t", [H.IQ2_S, H.Q4_K])
def test_layer_sigmoid_router_and_host_lane_hooks(T, api, oracle, t):
    """maya_moe_layer's options: sigmoid routing (selection bias, weight scale, normalisation: router_sigmoid's
    arithmetic) and the tier hooks cpu_part / cpu_flag (MoeDev's, glm_fast.hpp:299-300).  The fused single-token kernel,
    the staged kernels and the window path agree bit for bit; the ids are the oracle's sigmoid router's; the host lane's
    vector enters after the routed terms and before the shared expert (moe_down's order), only when its flag is set."""
    n_embd, n_ff, E, k = 1024, 512, 24, 4
    cfg = dict(n_embd=n_embd, n_ff=n_ff, n_expert=E, k=k, gu_type=t, d_type=t, n_ff_sh=256, sh_gu_type=H.Q8_0, sh_d_type=H.Q8_0)
    lc, experts, sh = synth_layer(T, api, cfg, E, seed=17)
    rng = H.rng_for("sigmoid-layer", t)
    bias = (0.3 * rng.standard_normal(E)).astype(np.float32)
    logits = H.router_logits("sigmoid-layer", 6, E, None)
    x = H.activations("sigmoid-layer", 6, n_embd, "bf16")
    cpu_part = rng.standard_normal((6, n_embd)).astype(np.float32)
    flags = np.array([1, 0, 1, 1, 0, 1], np.int32)
    ld, xd, bd = dev(T, logits), dev(T, x, T.bfloat16), dev(T, bias)
    cp, cf = dev(T, cpu_part), dev(T, flags)
    ids_o, w_o = oracle.router_sigmoid(logits, bias, k, 2.5, True)
    plain = api.MoeLayer(lc, experts, sh, sigmoid=(bd, 2.5, True))
    staged_plain = api.MoeLayer(lc, experts, sh, sigmoid=(bd, 2.5, True), staged=True)
    for i in range(6):
        hooked = api.MoeLayer(lc, experts, sh, sigmoid=(bd, 2.5, True), cpu_part=cp[i:i + 1], cpu_flag=cf[i:i + 1])
        hooked_staged = api.MoeLayer(lc, experts, sh, sigmoid=(bd, 2.5, True), cpu_part=cp[i:i + 1], cpu_flag=cf[i:i + 1], staged=True)
        ids_f, w_f, out_f = hooked.forward(ld[i:i + 1], xd[i:i + 1])
        ids_s, w_s, out_s = hooked_staged.forward(ld[i:i + 1], xd[i:i + 1])
        assert np.array_equal(ids_f.cpu().numpy()[0], ids_o[i]) and T.equal(ids_f, ids_s)
        assert np.abs(w_f.cpu().numpy()[0] - w_o[i]).max() <= 1e-6 and T.equal(w_f, w_s)
        assert T.equal(out_f, out_s), f"token {i}: fused and staged kernels differ"
        base = plain.forward(ld[i:i + 1], xd[i:i + 1])[2]
        assert T.equal(base, staged_plain.forward(ld[i:i + 1], xd[i:i + 1])[2])
        if flags[i]:
            assert not T.equal(out_f, base)
            assert H.rel_err((out_f - base).cpu().numpy()[0], cpu_part[i]) <= 1e-5
        else:
            assert T.equal(out_f, base)
    win = api.MoeLayer(lc, experts, sh, sigmoid=(bd, 2.5, True), cpu_part=cp, cpu_flag=cf)
    ids_w, _, out_w = win.forward(ld, xd)
    assert np.array_equal(ids_w.cpu().numpy(), ids_o)
    for i in range(6):
        one = api.MoeLayer(lc, experts, sh, sigmoid=(bd, 2.5, True), cpu_part=cp[i:i + 1], cpu_flag=cf[i:i + 1])
        assert T.equal(out_w[i], one.forward(ld[i:i + 1], xd[i:i + 1])[2][0]), f"window row {i}"
    with pytest.raises(api.MayaError):
        api.MoeLayer(lc, experts, sh, cpu_flag=cf[:1]).forward(ld[:1], xd[:1])        # a flag without the vector


def test_window_combine_carries_the_cross_rank_sum(T, api, oracle):
    """2..16 tokens on an expert-parallel rank: the rank-ordered sum of out[T][n_embd] runs inside the window's combine
    launch.  Three ranks on this GPU, one after another; what the ranks still to run would push is placed beforehand."""
    from project_maya_b200.peer import PeerGroup
    from test_gpu_allreduce import place_peer_pushes
    n_embd, n_ff, n_expert, k, nm, n_tok = 1024, 512, 12, 4, 3, 5
    cfg = dict(n_embd=n_embd, n_ff=n_ff, n_expert=n_expert, k=k, gu_type=H.Q4_K, d_type=H.Q4_K, n_ff_sh=256,
               sh_gu_type=H.Q8_0, sh_d_type=H.Q8_0)
    lc, experts, sh = synth_layer(T, api, cfg, n_expert, seed=9)
    logits = dev(T, H.router_logits("winar", n_tok, n_expert, 1.1))
    x = dev(T, H.activations("winar", n_tok, n_embd, "bf16"), T.bfloat16)
    per = n_expert // nm
    layers = [api.MoeLayer(lc, experts, sh, expert_range=(r * per, (r + 1) * per), shared_here=(r == 0)) for r in range(nm)]
    partial = [l.forward(logits, x)[2].clone() for l in layers]                     # each rank's own terms
    want = np.stack([oracle.allreduce_in_order(np.stack([p[t].cpu().numpy() for p in partial])) for t in range(n_tok)])
    ranks = PeerGroup.on_one_device(nm, stride=16 * n_embd, timeout_ms=200.0)
    for r in ranks:
        r.device_seq = False
    vecs = [p.reshape(-1) for p in partial]
    for mi in range(nm):
        place_peer_pushes(T, ranks, mi, 1, vecs, later_only=True)
    for r in range(nm):
        out = layers[r].forward(logits, x, peer=ranks[r])[2]
        T.cuda.synchronize()
        assert not ranks[r].poisoned()
        assert out.cpu().numpy().tobytes() == want.tobytes(), f"rank {r}"


def test_fused_layer_barrier_times_out_and_reports(T, api):
    """The fused kernel's one wait on other blocks is bounded: with the scratch's epoch word set ahead of its arrival
    counter (a state no launch leaves behind) the grid barrier can never be satisfied; the call still returns after the
    time limit, every block having skipped the second phase, and the sticky error word says so."""
    cfg = dict(n_embd=512, n_ff=256, n_expert=8, k=4, gu_type=H.Q4_K, d_type=H.Q4_K)
    lc, experts, _ = synth_layer(T, api, cfg, 8, seed=3)
    layer = api.MoeLayer(lc, experts)
    logits = dev(T, H.router_logits("timeout", 1, 8, None))
    x = dev(T, H.activations("timeout", 1, 512, "f32"))
    layer.forward(logits, x)
    T.cuda.synchronize()
    assert layer.error() == 0
    words = layer.scratch[:16].view(T.int32)
    words[1] += 7                                  # the epoch word: the barrier now waits for arrivals that never come
    layer.forward(logits, x)
    T.cuda.synchronize()                           # returns: the wait gave up after its second
    assert layer.error() != 0


def test_layer_refusals(T, api):
    cfg = H.CONFIGS["C1"]
    lc = layer_cfg(api, cfg)
    experts = T.zeros((2, lc.blob_bytes), dtype=T.uint8, device="cuda")
    layer = api.MoeLayer(api.MoeLayerConfig(cfg["n_embd"], cfg["n_ff"], 2, 2, H.Q4_K, H.Q4_K), experts)
    with pytest.raises(api.MayaError) as e:
        layer.forward(T.zeros((17, 2), device="cuda"), T.zeros((17, cfg["n_embd"]), device="cuda"))
    assert e.value.status == -4
    with pytest.raises(api.MayaError):
        api.MoeLayer(api.MoeLayerConfig(cfg["n_embd"], cfg["n_ff"], 2, 9, H.Q4_K, H.Q4_K), experts)


@pytest.mark.parametrize("router_dtype", ["f32", "bf16"])
def test_rms_router_and_two_launch_layer(T, api, oracle, router_dtype):
    """maya_rms_router (residual add + RMS norm + router logits, one launch) against the oracle, and a decode layer
    as two launches: that kernel, then the fused layer kernel on its x and logits - the routing and the output are the
    oracle's on the same numbers."""
    cfg = dict(H.CONFIGS["C2"], n_expert=32)
    lc, experts, shared = synth_layer(T, api, cfg, 32, seed=33)
    Hd, E = cfg["n_embd"], 32
    rng = H.rng_for("rms-router-gpu", router_dtype)
    h = rng.standard_normal(Hd).astype(np.float32)
    add = (0.2 * rng.standard_normal(Hd)).astype(np.float32)
    nw = (1.0 + 0.1 * rng.standard_normal(Hd)).astype(np.float32)
    rw = (0.08 * rng.standard_normal((E, Hd))).astype(np.float32)
    if router_dtype == "bf16":
        rw = H.to_bf16_f32(rw)
    rw_d = dev(T, rw, T.bfloat16 if router_dtype == "bf16" else None)
    h_out = T.empty(Hd, dtype=T.float32, device="cuda")
    x, logits = api.rms_router(dev(T, h), dev(T, add), dev(T, nw), 1e-5, rw_d, h_out=h_out)
    T.cuda.synchronize()
    ho, xo, lo = oracle.rms_router(h, add, nw, 1e-5, rw)
    assert np.array_equal(h_out.cpu().numpy(), ho)
    assert H.rel_err(x.cpu().numpy(), xo) <= 2e-6
    assert np.abs(logits.cpu().numpy() - lo).max() <= 2e-5
    with pytest.raises(api.MayaError):                       # in place with an add: other blocks would read the sum
        hd = dev(T, h)
        api.rms_router(hd, dev(T, add), dev(T, nw), 1e-5, rw_d, h_out=hd)
    # launch 2: the layer on the first launch's outputs
    ids, w, out = api.MoeLayer(lc, experts, shared).forward(logits.reshape(1, E), x.reshape(1, Hd))
    T.cuda.synchronize()
    lg, xg = logits.cpu().numpy().reshape(1, E), x.cpu().numpy()
    ids_o, w_o = oracle.router_top10(lg, cfg["k"])
    assert np.array_equal(ids.cpu().numpy(), ids_o)
    want = oracle_token(oracle, cfg, experts, shared, ids_o[0], w_o[0], xg)
    assert H.rel_err(out.cpu().numpy()[0], want) <= TIGHT


def _word_area(T, r):
    """The {seq, value} words of rank r's receive buffer: they follow its 2 x nm x stride floats of rows."""
    return r.keep[0][r.mi][2 * r.nm * r.stride * 4:].view(T.int64).view(2, r.nm, r.stride)


def _words(seq, v):
    return ((np.uint64(seq) << np.uint64(32)) | v.view(np.uint32).astype(np.uint64)).view(np.int64)


def test_fused_layer_exchanges_flagged_words(T, api, oracle):
    """The cross-rank sum in the fused kernel's epilogue, on one GPU: rank 1 of 3 runs alone with the other ranks'
    {seq, value} words placed in its receive area beforehand.  Its output is rank 0's + its own + rank 2's vector, added
    in that order (bit for bit), and its own words land in both peers' areas with the call's sequence number."""
    from project_maya_b200.peer import PeerGroup
    cfg = dict(n_embd=1024, n_ff=512, n_expert=8, k=2, gu_type=H.Q8_0, d_type=H.Q8_0)
    lc, experts, _ = synth_layer(T, api, cfg, 8, seed=31)
    layer = api.MoeLayer(lc, experts, None)
    n = cfg["n_embd"]
    ranks = PeerGroup.on_one_device(3, stride=n, timeout_ms=50.0)
    logits = H.router_logits("words", 3, 8, 1.1)
    x = H.activations("words", 3, n, "bf16")
    ld, xd = dev(T, logits), dev(T, x, T.bfloat16)
    rng = np.random.default_rng(5)
    for t, seq in enumerate((1, 2, 3)):
        local = layer.forward(ld[t:t + 1], xd[t:t + 1])[2].cpu().numpy()[0]
        others = {m: rng.standard_normal(n).astype(np.float32) for m in (0, 2)}
        others[0][:4] = [0.0, -0.0, np.float32(1e-38), np.float32(3e38)]
        area = _word_area(T, ranks[1])
        for m, v in others.items():
            area[seq & 1, m, :n] = T.from_numpy(_words(seq, v)).cuda()
        got = layer.forward(ld[t:t + 1], xd[t:t + 1], peer=ranks[1])[2].cpu().numpy()[0]
        want = oracle.allreduce_in_order(np.stack([others[0], local, others[2]]))
        assert got.tobytes() == want.tobytes()
        for m in (0, 2):
            pushed = _word_area(T, ranks[m])[seq & 1, 1, :n].cpu().numpy()
            assert np.array_equal(pushed, _words(seq, local))
    assert not ranks[1].poisoned()


def test_fused_layer_word_exchange_sequence_wraps(T, api, oracle):
    """The device-side sequence count across 2^32 (the reference's own transport test starts at 0xffffffe0,
    tests/ds4_peer_allreduce_test.cu:143): preset to 0xfffffff8, 24 single-token calls on rank 1 of 2 with rank 0's words
    placed beforehand under the number each call will use.  The count never takes the value 0 (a zeroed word would
    match it): 0xffffffff is followed by 2, which also keeps the two receive slots alternating."""
    from project_maya_b200.peer import PeerGroup
    cfg = dict(n_embd=1024, n_ff=512, n_expert=8, k=2, gu_type=H.Q8_0, d_type=H.Q8_0)
    lc, experts, _ = synth_layer(T, api, cfg, 8, seed=31)
    layer = api.MoeLayer(lc, experts, None)
    n = cfg["n_embd"]
    ranks = PeerGroup.on_one_device(2, stride=n, timeout_ms=50.0)
    r = ranks[1]
    r.seq = 0xFFFFFFF8
    r.set_device_seq(True)
    ld, xd = dev(T, H.router_logits("wrap", 1, 8, 1.1)), dev(T, H.activations("wrap", 1, n, "bf16"), T.bfloat16)
    local = layer.forward(ld, xd)[2].cpu().numpy()[0]
    rng = np.random.default_rng(9)
    seq, seen = 0xFFFFFFF8, []
    for _ in range(24):
        seq = 2 if seq == 0xFFFFFFFF else seq + 1
        seen.append(seq)
        other = rng.standard_normal(n).astype(np.float32)
        _word_area(T, r)[seq & 1, 0, :n] = T.from_numpy(_words(seq, other)).cuda()
        got = layer.forward(ld, xd, peer=r)[2].cpu().numpy()[0]
        assert got.tobytes() == oracle.allreduce_in_order(np.stack([other, local])).tobytes(), hex(seq)
        pushed = _word_area(T, ranks[0])[seq & 1, 1, :n].cpu().numpy()
        assert np.array_equal(pushed, _words(seq, local))
    assert 0 not in seen and 0xFFFFFFFF in seen and 2 in seen
    assert all((a & 1) != (b & 1) for a, b in zip(seen, seen[1:]))         # the slots alternate across the wrap too
    r.set_device_seq(False)
    assert r.seq == seen[-1] and not r.poisoned()


def test_fused_layer_exchange_times_out_and_poisons(T, api):
    """A peer that never sends: the wait in the fused kernel's epilogue gives up after the time-out, records who it
    waited for and poisons the transport; later calls return at once and the device still answers."""
    import time
    from project_maya_b200.peer import PeerGroup
    cfg = dict(n_embd=1024, n_ff=512, n_expert=8, k=2, gu_type=H.Q8_0, d_type=H.Q8_0)
    lc, experts, _ = synth_layer(T, api, cfg, 8, seed=31)
    layer = api.MoeLayer(lc, experts, None)
    r = PeerGroup.on_one_device(2, stride=cfg["n_embd"], timeout_ms=20.0)[0]
    ld, xd = dev(T, H.router_logits("words", 1, 8, 1.1)), dev(T, H.activations("words", 1, cfg["n_embd"], "bf16"), T.bfloat16)
    t0 = time.time()
    layer.forward(ld, xd, peer=r)
    T.cuda.synchronize()
    assert time.time() - t0 < 2.0
    assert r.poisoned()
    f = r.failure_record()
    assert f.captured == 1 and f.sequence == 1 and f.rank == 0 and f.waited_for == 1 and f.elapsed_ns >= f.timeout_ns
    t0 = time.time()
    for _ in range(32):
        layer.forward(ld, xd, peer=r)
    T.cuda.synchronize()
    assert time.time() - t0 < 1.0
    assert layer.error() == 0                                   # the layer's own barrier is not affected
    assert bool((T.ones(4, device="cuda") * 2 == 2).all())


@pytest.mark.parametrize("t", list(H.MORE_TYPES))
def test_layer_with_further_block_types(T, api, oracle, t):
    """maya_moe_layer_decode on routed experts stored as Q5_K, Q6_K, IQ4_XS, IQ3_XXS or IQ2_XXS (the rest of
    glmf::moe_supported's table): the staged kernels run, with a Q8_0 shared expert beside them; single tokens against the
    oracle, and a 5-token window equal to its tokens bit for bit."""
    n_embd, n_ff, E, k, n_sh = 1024, 512, 12, 4, 256
    cfg = dict(n_embd=n_embd, n_ff=n_ff, n_expert=E, k=k, gu_type=t, d_type=t, n_ff_sh=n_sh, sh_gu_type=H.Q8_0, sh_d_type=H.Q8_0)
    rng = H.rng_for("layer-more", t)
    experts_np = np.stack([H.constructed_expert(t, t, n_embd, n_ff, rng) for _ in range(E)])
    shared_np = H.constructed_expert(H.Q8_0, H.Q8_0, n_embd, n_sh, rng)
    experts, shared = dev(T, experts_np), dev(T, shared_np)
    lc = api.MoeLayerConfig(n_embd, n_ff, E, k, t, t, n_sh, H.Q8_0, H.Q8_0, 7.0)
    layer = api.MoeLayer(lc, experts, shared)
    logits = rng.standard_normal((5, E)).astype(np.float32)
    x = rng.standard_normal((5, n_embd)).astype(np.float32)
    ids_o, w_o = oracle.router_top10(logits, k)
    singles = []
    for i in range(5):
        ids, w, out = layer.forward(dev(T, logits[i:i + 1]), dev(T, x[i:i + 1]))
        assert np.array_equal(ids.cpu().numpy()[0], ids_o[i])
        want = oracle_token(oracle, cfg, experts, shared, ids_o[i], w_o[i], x[i], 7.0)
        assert H.rel_err(out.cpu().numpy()[0], want) <= 2e-4
        singles.append(out[0].clone())
    _, _, win = layer.forward(dev(T, logits), dev(T, x))
    for i in range(5):
        assert T.equal(win[i], singles[i])
    assert layer.error() == 0
