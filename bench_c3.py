"""Configuration C3 for `bench.py` (its `extra.c3` object, or `--workload c3`): concurrent decode at batch 8 - hidden
7168, 256 routed experts of FFN 2048 stored as Q4_K, top-8 with Zipf(1.1)-skewed routing so that the 8 tokens of a step
share experts (about 40 of the 64 picks are distinct).  A step is one 8-token window through maya_moe_layer_decode: the
window kernels read each distinct expert's rows once for all the tokens that routed to it.

Roofline: HBM; algorithmic bytes of a step = distinct experts x 24,772,608 B (the bytes a perfect row reuse reads).
16 seeded windows are captured in one CUDA graph and replayed; CUDA events, median of 5 replays.  Beside it the
reference's own window kernel (glmf::moe_win_experts, compiled for sm_100a from the reference tree into oracle/_ref) on
the same expert table and tokens, its router and q8_1 launches included, captured the same way.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

from project_maya_b200 import synthetic as S

ROOT = Path(__file__).resolve().parent
CFG = S.CONFIGS["C3"]
N_WIN = 16


def _peak():
    p = ROOT / "MEASURED_PEAKS.json"
    return (float(json.loads(p.read_text())["hbm_gbs"]), "measured") if p.exists() else (6650.0, "fallback")


def _median_ms(torch, stream, fn, runs=5):
    out = []
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        for _ in range(runs):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            fn()
            e1.record(stream)
            stream.synchronize()
            out.append(e0.elapsed_time(e1))
    return float(np.median(out))


def run(torch, api) -> dict:
    cfg = CFG
    Hd, FF, E, k, T = cfg["n_embd"], cfg["n_ff"], cfg["n_expert"], cfg["k"], cfg["T"]
    t = cfg["gu_type"]
    lc = api.MoeLayerConfig(Hd, FF, E, k, t, t)
    experts = torch.empty((E, lc.blob_bytes), dtype=torch.uint8, device="cuda")
    gu = 2 * FF * S.row_bytes(t, Hd)
    for e in range(E):
        api.synth_weights(t, 300000 + 2 * e, 0.02, 2 * FF, Hd, experts[e, :gu])
        api.synth_weights(t, 300001 + 2 * e, 0.02, Hd, FF, experts[e, gu:])
    torch.cuda.synchronize()
    layer = api.MoeLayer(lc, experts, None, max_tokens=T)
    logits_np = np.concatenate([S.router_logits("C3", T, E, cfg["zipf"], seed=w) for w in range(N_WIN)])
    logits = torch.from_numpy(logits_np).cuda()
    x = torch.from_numpy(S.bf16_bits(np.concatenate([S.activations("C3", T, Hd, "bf16", seed=w) for w in range(N_WIN)]))
                         .view(np.int16)).view(torch.bfloat16).cuda()
    top = np.argsort(-logits_np, axis=1, kind="stable")[:, :k].reshape(N_WIN, T * k)
    distinct = [len(np.unique(r)) for r in top]
    bytes_step = float(np.mean(distinct)) * lc.blob_bytes
    out = torch.empty((N_WIN * T, Hd), dtype=torch.float32, device="cuda")
    ids = torch.empty((N_WIN * T, k), dtype=torch.int32, device="cuda")
    w = torch.empty((N_WIN * T, k), dtype=torch.float32, device="cuda")
    stream = torch.cuda.Stream()

    def ours():
        for i in range(N_WIN):
            sl = slice(i * T, (i + 1) * T)
            layer.forward(logits[sl], x[sl], ids[sl], w[sl], out[sl])

    with torch.cuda.stream(stream):
        ours()
    stream.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        ours()
    ms = _median_ms(torch, stream, g.replay)
    us = ms * 1e3 / N_WIN
    peak, kind = _peak()
    res = {"workload": f"C3: H{Hd} E{E} FF{FF} top{k} Q4_K, bf16 acts, batch {T}, Zipf(1.1), {N_WIN} seeded windows",
           "distinct_experts_per_step_mean": float(np.mean(distinct)), "picks_per_step": T * k,
           "us_per_step": us, "tok_s_layer": T * 1e6 / us, "launch": f"CUDA graph of {N_WIN} windows",
           "roofline": {"bound": "hbm", "algorithmic_bytes_per_step": bytes_step, "achieved": bytes_step / us / 1e3, "peak": peak,
                        "peak_kind": kind, "unit": "GB/s", "frac": bytes_step / us / 1e3 / peak,
                        "kernels": "win_group + gate_up_kernel + down_groups_kernel + win_combine_kernel per window"},
           "error": layer.error()}

    # ---- the same windows through the prompt path (tensor-core grouped product over f16 operands: within 1e-2 of the
    #      window kernels, not bit-identical to them) - where the crossover between the two paths lies at this batch
    pf = api.MoePrefill(lc, experts, max_tokens=T)
    pf_out = torch.empty((N_WIN * T, Hd), dtype=torch.float32, device="cuda")

    def prompt_path():
        for i in range(N_WIN):
            sl = slice(i * T, (i + 1) * T)
            pf_out[sl].copy_(pf.forward(logits[sl], x[sl])[2])

    with torch.cuda.stream(stream):
        prompt_path()
    stream.synchronize()
    g1 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g1, stream=stream):
        prompt_path()
    us_pf = _median_ms(torch, stream, g1.replay) * 1e3 / N_WIN
    res["prompt_path"] = {"us_per_step": us_pf, "tok_s_layer": T * 1e6 / us_pf, "hbm_gbs": bytes_step / us_pf / 1e3,
                          "frac": bytes_step / us_pf / 1e3 / peak, "launch": f"CUDA graph of {N_WIN} x api.MoePrefill.forward",
                          "max_rel_diff_from_window_kernels": float((pf_out.double() - out.double()).abs().max() / out.double().abs().max()),
                          "error": pf.error()}

    # ---- the reference's window kernel on the same table and tokens
    from oracle import ref_gpu
    if not ref_gpu.available():
        res["gpu_baseline"] = {"unavailable": "oracle/_ref/libmaya_ref_gpu.so is not built"}
        return res
    R = ref_gpu.RefGpu()
    L, p = R.lib, ref_gpu._p
    xf = x.float().contiguous()
    xq = torch.empty((N_WIN * T, Hd // 32 * 36), dtype=torch.uint8, device="cuda")
    ids_r = torch.empty((N_WIN * T, k), dtype=torch.int32, device="cuda")
    w_r = torch.empty((N_WIN * T, k), dtype=torch.float32, device="cuda")
    plan_ptr = torch.zeros((N_WIN * T, 8), dtype=torch.int64, device="cuda")
    hq = torch.empty(T * 8 * (FF // 32) * 36, dtype=torch.uint8, device="cuda")
    part = torch.empty((T * 8, Hd), dtype=torch.float32, device="cuda")
    out_r = torch.empty((N_WIN * T, Hd), dtype=torch.float32, device="cuda")
    grp_ptr = torch.zeros(T * 8, dtype=torch.int64, device="cuda")
    grp_start = torch.zeros(T * 8 + 1, dtype=torch.int32, device="cuda")
    grp_ent = torch.zeros(T * 8, dtype=torch.int32, device="cuda")
    n_groups = torch.zeros(1, dtype=torch.int32, device="cuda")
    cpu_flag = torch.zeros(T, dtype=torch.int32, device="cuda")
    down_off = 2 * FF * S.row_bytes(t, Hd)

    def theirs():
        s_ = R._stream()
        for i in range(N_WIN):
            sl = slice(i * T, (i + 1) * T)
            R._ck("router", L.ref_router_top10(p(logits[sl]), T, E, k, p(ids_r[sl]), p(w_r[sl]), s_))
            for j in range(T):
                R._ck("quantize", L.ref_quantize_q8_1(p(xf[i * T + j]), p(xq[i * T + j]), Hd, s_))
            plan_ptr[sl, :k] = ids_r[sl].to(torch.int64) * experts.stride(0) + experts.data_ptr()
            R._ck("moe_win_experts", L.ref_moe_win_experts(t, t, p(plan_ptr[sl]), p(w_r[sl]), None, p(cpu_flag), p(xq[sl]),
                                                           xq.stride(0), p(hq), p(part), None, p(out_r[sl]), Hd, p(grp_ptr),
                                                           p(grp_start), p(grp_ent), p(n_groups), T, k, Hd, FF, float("inf"),
                                                           down_off, s_))

    with torch.cuda.stream(stream):
        theirs()
    stream.synchronize()
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g2, stream=stream):
        theirs()
    ms_r = _median_ms(torch, stream, g2.replay)
    us_r = ms_r * 1e3 / N_WIN
    diff = float((out.double() - out_r.double()).abs().max() / out_r.double().abs().max())
    res["gpu_baseline"] = {"kernels": "router_top10 + 8 x glmf::quantize_q8_1 + glmf::moe_win_experts (the reference's CUDA kernels "
                                      "built for sm_100a), same table and tokens, CUDA graph", "us_per_step": us_r,
                           "tok_s_layer": T * 1e6 / us_r, "hbm_gbs": bytes_step / us_r / 1e3,
                           "max_rel_diff_of_outputs": diff, "ids_equal": bool(torch.equal(ids, ids_r))}
    return res
