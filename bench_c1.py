"""Configuration C1 for `bench.py` (its `extra.c1` object): the reference's own CPU-runnable case on the GPU - hidden 2048,
64 routed experts of FFN 1024 stored as Q4_K, top-8, no shared expert, f32 activations, one token a step.

A token reads 8 x 3,538,944 B = 28.3 MB: 4.3 us of HBM time, so the step is bound by what does not scale with bytes
(routing, the grid barrier, the launch).  Four layer copies (226 MB each: more than L2) and 16 seeded tokens rotate
through a CUDA graph of 64 steps; CUDA events, median of 5 replays.  Beside it the reference's own CUDA kernels
(oracle/_ref) on the same layers and tokens, captured the same way.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

from project_maya_b200 import synthetic as S

ROOT = Path(__file__).resolve().parent
CFG = S.CONFIGS["C1"]
N_STEPS, N_LAYERS = 64, 4


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
    Hd, FF, E, k, t = cfg["n_embd"], cfg["n_ff"], cfg["n_expert"], cfg["k"], cfg["gu_type"]
    lc = api.MoeLayerConfig(Hd, FF, E, k, t, t)
    gu = 2 * FF * S.row_bytes(t, Hd)
    experts0 = torch.empty((E, lc.blob_bytes), dtype=torch.uint8, device="cuda")
    for e in range(E):
        api.synth_weights(t, 700000 + 2 * e, 0.02, 2 * FF, Hd, experts0[e, :gu])
        api.synth_weights(t, 700001 + 2 * e, 0.02, Hd, FF, experts0[e, gu:])
    tables = [experts0] + [experts0.clone() for _ in range(N_LAYERS - 1)]
    layers = [api.MoeLayer(lc, ex, None, max_tokens=1) for ex in tables]
    n_tok = cfg["tokens"]
    logits = torch.from_numpy(S.router_logits("C1", n_tok, E, None)).cuda()
    x = torch.from_numpy(S.activations("C1", n_tok, Hd, "f32")).cuda()
    ids = torch.empty((1, k), dtype=torch.int32, device="cuda")
    w = torch.empty((1, k), dtype=torch.float32, device="cuda")
    out = torch.empty((N_STEPS, Hd), dtype=torch.float32, device="cuda")
    stream = torch.cuda.Stream()

    def ours():
        for s in range(N_STEPS):
            i = s % n_tok
            layers[s % N_LAYERS].forward(logits[i:i + 1], x[i:i + 1], ids, w, out[s:s + 1])

    with torch.cuda.stream(stream):
        ours()
    stream.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        ours()
    us = _median_ms(torch, stream, g.replay) * 1e3 / N_STEPS
    peak, kind = _peak()
    nbytes = float(k * lc.blob_bytes)
    res = {"workload": f"C1: H{Hd} E{E} FF{FF} top{k} Q4_K, f32 acts, batch 1, {n_tok} seeded tokens, {N_LAYERS} resident layers",
           "us_per_token": us, "tok_s_layer": 1e6 / us, "launch": f"CUDA graph of {N_STEPS} steps",
           "roofline": {"bound": "hbm", "algorithmic_bytes_per_step": nbytes, "achieved": nbytes / us / 1e3, "peak": peak,
                        "peak_kind": kind, "unit": "GB/s", "frac": nbytes / us / 1e3 / peak,
                        "kernel": "moe_layer_t1_kernel<Q4_K, none> (one launch a step)"},
           "error": max(l.error() for l in layers)}

    from oracle import ref_gpu
    if not ref_gpu.available():
        res["gpu_baseline"] = {"unavailable": "oracle/_ref/libmaya_ref_gpu.so is not built"}
        return res
    R = ref_gpu.RefGpu()
    refs = [ref_gpu.RefLayer(R, Hd, FF, E, k, t, t, S.row_bytes, ex) for ex in tables]
    out_r = torch.empty((N_STEPS, Hd), dtype=torch.float32, device="cuda")

    def theirs():
        for s in range(N_STEPS):
            i = s % n_tok
            refs[s % N_LAYERS].forward(logits[i:i + 1], x[i:i + 1], out_r[s])

    with torch.cuda.stream(stream):
        theirs()
    stream.synchronize()
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g2, stream=stream):
        theirs()
    us_r = _median_ms(torch, stream, g2.replay) * 1e3 / N_STEPS
    res["gpu_baseline"] = {"kernels": "router_top10 + glmf::quantize_q8_1 + glmf::moe_gate_up + glmf::moe_down (the reference's CUDA "
                                      "kernels built for sm_100a), same layers and tokens, CUDA graph",
                           "us_per_token": us_r, "tok_s_layer": 1e6 / us_r, "hbm_gbs": nbytes / us_r / 1e3,
                           "max_rel_diff_of_outputs": float((out.double() - out_r.double()).abs().max() / out_r.double().abs().max())}
    return res
