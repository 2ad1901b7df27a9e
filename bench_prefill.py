"""Benchmark of the prompt path on configuration C4 (4096 tokens x top-8 over 256 experts of hidden 6144 / FFN 2048,
half of the experts stored as Q8_0 and half as Q4_K, bf16 activations).  `python bench.py --workload prefill` calls
`run`; one JSON line comes back.

A step is one whole prompt-path layer over one 4096-token chunk (route, group, quantize, gate/up + SwiGLU product that
writes h already quantized, down product, combine).  Steps rotate over `layers` layer copies (2 x 7.3 GB of expert blobs by default), so no
step finds its weights in L2.  The dominant kernel is the grouped GEMM; it is timed by itself with CUDA events and
reported against the measured dense bf16 peak: its algorithmic work is 2 * rows * (3 * n_embd * n_ff) flops per layer
(rows = tokens * k), whatever padding its 128-row groups carry.
"""
from __future__ import annotations

import contextlib
import json
from pathlib import Path

import numpy as np

from project_maya_b200 import synthetic as S

ROOT = Path(__file__).resolve().parent
CFG = S.CONFIGS["C4"]


def tensor_peak(sustained: bool = False) -> tuple[float, str]:
    """The pool's measured cuBLAS bf16 rate: the burst figure (a kernel timed alone for a few ms) or the sustained one
    (seconds at the board's power limit)."""
    p = ROOT / "MEASURED_PEAKS.json"
    fallback = 1400.0 if sustained else 1590.0
    if p.exists():
        try:
            v = json.loads(p.read_text()).get("bf16_tflops_sustained" if sustained else "bf16_tflops")
            if v:
                return float(v), "measured"
        except (ValueError, OSError):
            pass
    return fallback, "fallback"


def build_pools(torch, api, seed: int, E: int):
    Hd, FF = CFG["n_embd"], CFG["n_ff"]
    types = S.expert_types("C4", E, CFG["types"])
    pools = []
    for t in sorted(set(int(v) for v in types)):
        members = [e for e in range(E) if int(types[e]) == t]
        gu = 2 * FF * S.row_bytes(t, Hd)
        blobs = torch.empty((len(members), gu + Hd * S.row_bytes(t, FF)), dtype=torch.uint8, device="cuda")
        for i, e in enumerate(members):
            api.synth_weights(t, seed + 2 * e, 0.02, 2 * FF, Hd, blobs[i, :gu])
            api.synth_weights(t, seed + 2 * e + 1, 0.02, Hd, FF, blobs[i, gu:])
        pools.append((t, blobs, members))
    torch.cuda.synchronize()
    return pools


def run(steps: int, warmup: int, layers: int, clock_sampler=None, scale: int = 1, sustained_steps: int = 0,
        sustained_sampler=None) -> dict:
    """scale > 1 divides both the number of experts and the number of tokens (the rows per expert stay the same): a
    reduced case of the same kernels for profiler captures; the headline configuration is scale = 1."""
    import torch

    from project_maya_b200 import _lib, api

    lib = _lib.load()
    Hd, FF, E, k, T = CFG["n_embd"], CFG["n_ff"], CFG["n_expert"] // scale, CFG["k"], CFG["T"] // scale
    lc = api.MoeLayerConfig(Hd, FF, E, k, S.Q8_0, S.Q8_0)
    pf = [api.MoePrefill(lc, None, max_tokens=T, pools=build_pools(torch, api, 7000 + 100000 * i, E)) for i in range(layers)]
    logits_h = torch.from_numpy(S.router_logits("C4", T, E, None)).pin_memory()
    x_h = torch.from_numpy(S.bf16_bits(S.activations("C4", T, Hd, "bf16")).view(np.int16)).view(torch.bfloat16).pin_memory()
    logits_d, x_d = logits_h.cuda(), x_h.cuda()
    stage_l, stage_x = torch.empty_like(logits_d), torch.empty_like(x_d)
    out_h = torch.empty((T, Hd), dtype=torch.float32).pin_memory()
    stream = torch.cuda.Stream()
    W = max(warmup, 3)

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            e0.record(stream)
            for s in range(n):
                fn(s)
            stream.wait_stream(s_in)                      # the side streams' copies belong to the timed region
            stream.wait_stream(s_out)
            e1.record(stream)
        stream.synchronize()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3

    def step_dev(s):
        pf[s % layers].forward(logits_d, x_d, stream=stream)

    # end to end: a step's inputs come from pinned host memory and its result goes back, inside the timed region; the
    # copies run on their own streams (two staging slots each way), so chunk s + 1 arrives while chunk s is computed
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    stage = [(torch.empty_like(logits_d), torch.empty_like(x_d)) for _ in range(2)]
    outs = [torch.empty((T, Hd), dtype=torch.float32, device="cuda") for _ in range(2)]
    e2e_state = {"done": [], "copied": []}

    def step_e2e(s):
        sl, sx = stage[s % 2]
        done, copied = e2e_state["done"], e2e_state["copied"]
        with torch.cuda.stream(s_in):
            if len(done) >= 2:
                s_in.wait_event(done[-2])                 # the step that last read this staging slot
            sl.copy_(logits_h, non_blocking=True)
            sx.copy_(x_h, non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(s_in)
        stream.wait_event(ready)
        if len(copied) >= 2:
            stream.wait_event(copied[-2])                 # the output slot has left for the host
        _, _, ffn = pf[s % layers].forward(sl, sx, stream=stream)
        outs[s % 2].copy_(ffn, non_blocking=True)         # on `stream`: frees the layer's own buffer for step s + layers
        ev = torch.cuda.Event()
        ev.record(stream)
        done.append(ev)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev)
            out_h.copy_(outs[s % 2], non_blocking=True)
            cp = torch.cuda.Event()
            cp.record(s_out)
            copied.append(cp)

    timed(step_dev, W)
    timed(step_e2e, W)
    l0 = lib.maya_launch_count()
    with (clock_sampler if clock_sampler is not None else contextlib.nullcontext()):
        dt = timed(step_dev, steps)
    launches = int(lib.maya_launch_count() - l0)
    dt_e2e = timed(step_e2e, steps)
    assert all(p.error() == 0 for p in pf), "a bounded wait inside a grouped GEMM ran out"

    # the dominant kernel by itself: the gate/up + SwiGLU product of one pool sequence (both pools), CUDA events
    rows = T * k
    flops_layer = 2.0 * rows * 3 * Hd * FF
    p0 = pf[0]

    def products_only(s):
        p = pf[s % layers]
        for gt, dt_, blobs, stride, down_off, n_p, emap in p.pools:
            api.mmq_run_glu(api.mmq_product(blobs, gt, 2 * FF, Hd, stride, n_p, p.xq, p.bounds, None, rows, None, FF,
                                            expert_map=emap, error=p.err, xq_out=p.hq), lc.limit, stream=stream)
        for gt, dt_, blobs, stride, down_off, n_p, emap in p.pools:
            api.mmq_run(api.mmq_product(blobs.data_ptr() + down_off, dt_, Hd, FF, stride, n_p, p.hq, p.bounds, None, rows,
                                        p.out, Hd, expert_map=emap, error=p.err), stream=stream)

    timed(products_only, 2)
    n_prod = max(4, min(steps, 16))
    dt_prod = timed(products_only, n_prod) / n_prod
    peak, src = tensor_peak()
    achieved = flops_layer / dt_prod / 1e12
    weight_bytes = sum(int(q[2].numel()) for q in p0.pools)
    sustained = None
    if sustained_steps > 0:
        # The prompt path runs at the board's power limit: a few steps are a burst, hundreds settle ~ 12 % slower at
        # ~ 1.4 GHz.  The same device-resident step, back to back, with the clocks sampled.
        with (sustained_sampler if sustained_sampler is not None else contextlib.nullcontext()):
            dt_s = timed(step_dev, sustained_steps)
        dt_ps = timed(products_only, max(16, sustained_steps // 4)) / max(16, sustained_steps // 4)
        peak_s, src_s = tensor_peak(True)
        sustained = {"steps": sustained_steps, "ms_per_step": dt_s / sustained_steps * 1e3, "tok_s_layer": sustained_steps * T / dt_s,
                     "products_us_per_layer": dt_ps * 1e6, "products_tflops": flops_layer / dt_ps / 1e12,
                     "frac_of_sustained_peak": flops_layer / dt_ps / 1e12 / peak_s, "sustained_peak": peak_s,
                     "peak_source": f"{src_s} dense bf16, sustained"}
    line = {
        "metric": "MoE expert-FFN prefill tokens/s per layer", "value": steps * T / dt, "unit": "tok/s/layer",
        "n_gpus": 1, "steps": steps, "warmup": W, "ms_per_step": dt / steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 operands from q8_1 x GGUF blocks, f32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"C4 prefill: {T} tokens, hidden 6144, {E} experts of FFN 2048 (half Q8_0, half Q4_K), top-8"
                               + ("" if scale == 1 else f" [reduced 1/{scale} case]"),
                   "layers_rotated": layers, "l2": f"inputs larger than L2: {weight_bytes / 1e9:.1f} GB of expert blobs per layer"},
        "e2e": {"value": steps * T / dt_e2e, "unit": "tok/s/layer",
                "h2d_bytes_per_step": int(logits_h.numel() * 4 + x_h.numel() * 2), "d2h_bytes_per_step": int(out_h.numel() * 4)},
        "gpu_launches": launches,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": f"{src} dense bf16", "kernel": "mmq_kernel (4 launches: 2 pools x gate/up+SwiGLU, down)",
                     "us_per_layer": dt_prod * 1e6, "flops_per_layer": flops_layer,
                     "weight_stream_gbs": weight_bytes / dt_prod / 1e9},
    }
    if sustained is not None:
        line["sustained"] = sustained
    return line
