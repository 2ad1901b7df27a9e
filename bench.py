#!/usr/bin/env python3
"""Benchmark of the routed-MoE expert-FFN decode layer (route -> experts -> combine, shared expert alongside).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

Workload (N = 1): the decode layer of the headline configuration - hidden 6144, 256 routed experts of FFN 2048 stored
as IQ2_S plus one always-on shared expert of FFN 2048 stored as Q8_0, top-8 softmax routing, bf16 activations, batch 1,
256 seeded tokens whose router logits are N(0,1) plus a Zipf(1.1) per-expert bias.  Expert weights are N(0, 0.02)
quantized on the device by the library's own quantizers (synthetic data; no checkpoint is involved).  One step = one
token through one layer.  `--layers` copies of the layer are resident and steps rotate through them, so every step's
136.8 MB of expert blocks come from HBM, not from L2 (working set >> 126 MB).

One JSON line on stdout (rank 0): `value` = tokens/s through one layer with inputs resident in HBM (CUDA-graph replay
of the K steps, CUDA-event timed); `e2e` = the same with each step's logits and activations copied from pinned host
memory and the output copied back, inside the timed region; `roofline` = the dominant kernel's algorithmic bytes over
its CUDA-event duration against the measured HBM peak; `cpu_baseline` = the reference's CPU expert rows on this box's
host cores over a bounded sample of the same tokens.

`--impl reference` times the reference's own CPU implementation of the path (oracle/_ref when it was built from the
reference tree, else the CPU restatement) with all host threads; under torchrun only rank 0 works.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from project_maya_b200 import synthetic as S  # noqa: E402

CFG = dict(S.CONFIGS["C2"], limit=S.INF)
WORKLOAD = "C2 decode: H6144 E256 FF2048 top8 IQ2_S + shared Q8_0 FF2048, bf16 acts, batch 1, 256 seeded tokens, Zipf(1.1)"
N_TOKENS = 256
MIN_TIMED_S, MIN_REPLAYS, MAX_REPLAYS = 0.2, 5, 200     # the timed graph of K steps is replayed for at least this long


def algorithmic_bytes_per_token(cfg=CFG) -> int:
    routed = cfg["k"] * S.blob_bytes(cfg["gu_type"], cfg["d_type"], cfg["n_embd"], cfg["n_ff"])
    shared = S.blob_bytes(cfg["sh_gu_type"], cfg["sh_d_type"], cfg["n_embd"], cfg["n_ff_sh"]) if cfg.get("n_ff_sh") else 0
    return routed + shared


def measured_peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": nv.nvmlClocksThrottleReasonHwSlowdown,
                 "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown,
                 "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.reasons |= {k for k, bit in names.items() if r & bit}
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_layer_tokens(tokens: list[int], threads: int, repeats: int = 5):
    """The reference's CPU expert path on `tokens` of the workload, in native code on a persistent thread pool
    (oracle/ref_shim_layer.cpp): Q8_K activations, the routed experts through the reference's AVX-512 / AVX2 rows with
    every expert's rows split across all threads (as its pool does), the Q8_0 shared expert through an AVX2 dot (the
    reference hands Q8_0 to ggml-cpu, which is not in its tree), plain weighted sum; router in double on the host.
    The tokens run `repeats` times and the best pass counts.  Returns (seconds per token, kind, note)."""
    from oracle.oracle import Oracle, Ref
    orc = Oracle()
    ref = Ref() if Ref.available() else None
    cfg = CFG
    Hd, FF, E, k = cfg["n_embd"], cfg["n_ff"], cfg["n_expert"], cfg["k"]
    logits = S.router_logits("C2", N_TOKENS, E, cfg["zipf"])
    x = S.activations("C2", N_TOKENS, Hd, "bf16")
    t, d = cfg["gu_type"], cfg["d_type"]
    # constructed (random valid) blocks: on the CPU the byte values do not change the work; a token's 8 experts are drawn
    # from a pool (290 MB) larger than the last-level cache, so the rows stream from DRAM as in production
    pool_n = 24
    rng = S.rng_for("cpu-pool")
    pool = [S.constructed_expert(t, d, Hd, FF, rng) for _ in range(pool_n)]
    shared = S.constructed_expert(cfg["sh_gu_type"], cfg["sh_d_type"], Hd, cfg["n_ff_sh"], rng)
    ids, w = orc.router_f64(logits, k)
    if ref is not None:
        ref.pool_threads(threads)
        blobs = [pool[(int(ids[ti, j]) + ti) % pool_n] for ti in tokens for j in range(k)]
        xs, ws = x[tokens], w[tokens]
        ref.layer_tokens(t, d, S.row_bytes(t, Hd), S.row_bytes(d, FF), Hd, FF, k, blobs[:k], ws[:1], xs[:1], shared, cfg["n_ff_sh"])
        best = min(ref.layer_tokens(t, d, S.row_bytes(t, Hd), S.row_bytes(d, FF), Hd, FF, k, blobs, ws, xs, shared,
                                    cfg["n_ff_sh"])[1] for _ in range(repeats))
        return best / len(tokens), "reference", (
            "routed IQ2_S experts: the reference's AVX-512 CPU rows (oracle/_ref) over Q8_K activations, every expert's rows "
            "split over the threads of a persistent native pool; shared Q8_0 expert: AVX2 int8 dot over q8_1 activations; "
            f"router in double; best of {repeats} passes; random valid blocks from a 24-expert pool (290 MB)")
    t0 = time.perf_counter()
    for ti in tokens:
        xq = orc.quantize_q8_1(x[ti])
        parts = np.stack([orc.expert_q8_1(t, d, pool[(int(ids[ti, j]) + ti) % pool_n], Hd, FF, S.INF, xq) for j in range(k)])
        sh = orc.expert_q8_1(cfg["sh_gu_type"], cfg["sh_d_type"], shared, Hd, cfg["n_ff_sh"], S.INF, xq)
        orc.combine_native(parts, w[ti], sh)
    dt = time.perf_counter() - t0
    return dt / len(tokens), "port", "CPU restatement of the q8_1 path (OpenMP); router in double; random valid blocks"


def reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    os.environ.setdefault("OMP_NUM_THREADS", str(threads))
    sample = 16
    times = []
    kind = note = None
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_layer_tokens(list(range(sample)), threads, repeats=1)
    for s in range(args.steps):
        toks = [(s * sample + i) % N_TOKENS for i in range(sample)]
        per_tok, kind, note = cpu_layer_tokens(toks, threads, repeats=5)
        times.append(per_tok)
        if sum(times) * sample * 5 > 150.0:      # keep the whole run within a few minutes whatever the host
            break
    per_tok = float(np.median(times))
    value = 1.0 / per_tok
    line = {"impl": "reference", "metric": "MoE expert-FFN decode tokens/s per layer", "value": value, "unit": "tok/s/layer",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_tok * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8 x int8 -> f32",
            "data": "synthetic", "config": {"workload": WORKLOAD, "sample": f"{sample} tokens per step, best of 5 passes"},
            "cpu_baseline": {"value": value, "unit": "tok/s/layer", "cores": threads, "kind": kind,
                             "effective_gbs": algorithmic_bytes_per_token() / per_tok / 1e9,
                             "sample": f"{sample} tokens per step, median over {len(times)} steps; {note}"},
            "e2e": {"value": value, "unit": "tok/s/layer", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ GPU arm
def build_layers(torch, api, n_layers: int, rank: int, world: int, partition: str):
    """The resident layers of this rank.  N > 1, partition "width": FFN rows [rank * n_ff / N, (rank + 1) * n_ff / N) of
    every expert (the reference's tensor-parallel split; every rank carries 1 / N of every token); "expert": experts
    [rank * E / N, (rank + 1) * E / N) whole, the shared expert width-sliced."""
    cfg = CFG
    lc = api.MoeLayerConfig(cfg["n_embd"], cfg["n_ff"], cfg["n_expert"], cfg["k"], cfg["gu_type"], cfg["d_type"],
                            cfg["n_ff_sh"], cfg["sh_gu_type"], cfg["sh_d_type"], cfg["limit"])
    Hd, FF, E = cfg["n_embd"], cfg["n_ff"], cfg["n_expert"]
    gu = 2 * FF * S.row_bytes(cfg["gu_type"], Hd)
    experts0 = torch.empty((E, lc.blob_bytes), dtype=torch.uint8, device="cuda")
    for e in range(E):
        api.synth_weights(cfg["gu_type"], 2 * e, 0.02, 2 * FF, Hd, experts0[e, :gu])
        api.synth_weights(cfg["d_type"], 2 * e + 1, 0.02, Hd, FF, experts0[e, gu:])
    shared0 = torch.empty(lc.shared_bytes, dtype=torch.uint8, device="cuda")
    sgu = 2 * cfg["n_ff_sh"] * S.row_bytes(cfg["sh_gu_type"], Hd)
    api.synth_weights(cfg["sh_gu_type"], 100001, 0.02, 2 * cfg["n_ff_sh"], Hd, shared0[:sgu])
    api.synth_weights(cfg["sh_d_type"], 100002, 0.02, Hd, cfg["n_ff_sh"], shared0[sgu:])
    expert_range = shared_range = None
    if world > 1 and partition == "width":
        wid, wid_sh = FF // world, cfg["n_ff_sh"] // world
        lc, experts0, shared0 = api.width_slice(lc, experts0, shared0, rank * wid, (rank + 1) * wid, rank * wid_sh, (rank + 1) * wid_sh)
        torch.cuda.empty_cache()
    elif world > 1:
        per, wid_sh = E // world, cfg["n_ff_sh"] // world
        expert_range, shared_range = (rank * per, (rank + 1) * per), (rank * wid_sh, (rank + 1) * wid_sh)
    layers = []
    for i in range(n_layers):
        # further layers are byte copies in their own memory: the values do not change the work, the addresses do
        ex = experts0 if i == 0 else experts0.clone()
        sh = shared0 if i == 0 else shared0.clone()
        layers.append(api.MoeLayer(lc, ex, sh, expert_range=expert_range, shared_range=shared_range, max_tokens=1))
    torch.cuda.synchronize()
    return lc, layers


def gpu_arm(args) -> None:
    import torch
    import torch.distributed as dist

    from project_maya_b200 import _lib, api

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this path has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    lib = _lib.load()
    if lib.maya_device_ok() != 0:
        raise SystemExit("the library is built for sm_100a only")
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    cfg = CFG
    Hd, E, k = cfg["n_embd"], cfg["n_expert"], cfg["k"]
    per = E // world
    lc, layers = build_layers(torch, api, args.layers, rank, world, args.partition)

    logits_h = torch.from_numpy(S.router_logits("C2", N_TOKENS, E, cfg["zipf"])).pin_memory()
    x_h = torch.from_numpy(S.bf16_bits(S.activations("C2", N_TOKENS, Hd, "bf16")).view(np.int16)).view(torch.bfloat16).pin_memory()
    logits_d, x_d = logits_h.cuda(), x_h.cuda()
    # a step's inputs as one pinned record [logits f32 | x bf16], the way an engine hands a token over: one copy a step
    IN_L, IN_BYTES = E * 4, E * 4 + Hd * 2
    in_h = torch.empty((N_TOKENS, IN_BYTES), dtype=torch.uint8).pin_memory()
    in_h[:, :IN_L] = logits_h.view(torch.uint8).view(N_TOKENS, IN_L)
    in_h[:, IN_L:] = x_h.view(torch.uint8).view(N_TOKENS, Hd * 2)
    K, W = args.steps, args.warmup
    out_d = torch.empty((K, Hd), dtype=torch.float32, device="cuda")
    ids_d = torch.empty((K, k), dtype=torch.int32, device="cuda")
    w_d = torch.empty((K, k), dtype=torch.float32, device="cuda")
    out_h = torch.empty((K, Hd), dtype=torch.float32).pin_memory()
    stage = torch.empty((K, IN_BYTES), dtype=torch.uint8, device="cuda")
    stage_l = [None] * K
    stage_x = [None] * K
    for s_ in range(K):
        stage_l[s_] = stage[s_, :IN_L].view(torch.float32).view(1, E)
        stage_x[s_] = stage[s_, IN_L:].view(torch.bfloat16).view(1, Hd)

    peer = None
    if world > 1 and args.ar == "peer":
        from project_maya_b200.peer import PeerGroup
        peer = PeerGroup.over_processes(rank, world, Hd, timeout_ms=5000.0)
        peer.set_device_seq(True)   # sequence numbers counted on the device: the K steps can be captured in a graph

    def step(s: int, l_row, x_row):
        layers[s % len(layers)].forward(l_row, x_row, ids_d[s:s + 1], w_d[s:s + 1], out_d[s:s + 1], peer=peer)
        if world > 1 and peer is None:
            dist.all_reduce(out_d[s:s + 1])

    def step_dev(s: int):
        tok = s % N_TOKENS
        step(s, logits_d[tok:tok + 1], x_d[tok:tok + 1])

    # End to end: every step copies its inputs from pinned host memory and its output back, inside the timed region.
    # The copies run on their own streams, as a serving engine would issue them: step s's inputs may be up to
    # E2E_DEPTH steps ahead of the layer kernel (a ring of staging slots), its output leaves while step s + 1 computes.
    E2E_DEPTH = 4
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def run_e2e_steps():
        cur = torch.cuda.current_stream()
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        done = []
        for s in range(K):
            tok = s % N_TOKENS
            with torch.cuda.stream(s_in):
                if s >= E2E_DEPTH:
                    s_in.wait_event(done[s - E2E_DEPTH])
                stage[s].copy_(in_h[tok], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(s_in)
            cur.wait_event(ready)
            step(s, stage_l[s], stage_x[s])
            ev = torch.cuda.Event()
            ev.record(cur)
            done.append(ev)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev)
                out_h[s:s + 1].copy_(out_d[s:s + 1], non_blocking=True)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)

    def step_e2e(s: int):                      # the unpipelined form, for the eager warm-up only
        tok = s % N_TOKENS
        stage[s].copy_(in_h[tok], non_blocking=True)
        step(s, stage_l[s], stage_x[s])
        out_h[s:s + 1].copy_(out_d[s:s + 1], non_blocking=True)

    stream = torch.cuda.Stream()
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        for s in range(max(W, 3)):              # eager warm-up: loads every kernel, sets shared-memory attributes
            step_dev(s)
            step_e2e(s)
    stream.synchronize()

    use_graph = world == 1 or peer is not None
    launches0 = lib.maya_launch_count()
    if use_graph:
        g_dev, g_e2e = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_dev, stream=stream):
            for s in range(K):
                step_dev(s)
        launches_per_run = lib.maya_launch_count() - launches0
        with torch.cuda.graph(g_e2e, stream=stream):
            run_e2e_steps()
        run_dev, run_e2e = g_dev.replay, g_e2e.replay
    else:
        def run_dev():
            for s in range(K):
                step_dev(s)

        run_e2e = run_e2e_steps
        run_dev()
        launches_per_run = lib.maya_launch_count() - launches0

    def timed(fn) -> list[float]:
        """The K steps, replayed until at least MIN_TIMED_S have gone by (5 replays or more), one CUDA-event pair per
        replay on the launching stream, barrier + synchronize on both sides of every replay; the max over ranks of each
        replay's time.  The reported step time is the median replay's."""
        out = []
        with torch.cuda.stream(stream):
            fn()                                 # one untimed pass of the same K steps
            stream.synchronize()
            t_begin = time.perf_counter()
            while len(out) < MIN_REPLAYS or (time.perf_counter() - t_begin < MIN_TIMED_S and len(out) < MAX_REPLAYS):
                if world > 1:
                    dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                fn()
                e1.record(stream)
                stream.synchronize()
                torch.cuda.synchronize()
                ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
                if world > 1:
                    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
                out.append(float(ms.item()))
        return out

    with ClockSampler(local_rank) as clocks:
        runs_dev = timed(run_dev)
        # block 0's stamps of the timed run's last step (with the cross-rank sum in the kernel when N > 1)
        step_phases = layers[(K - 1) % len(layers)].phase_ns(stream)
        runs_e2e = timed(run_e2e)
    ms_dev, ms_e2e = float(np.median(runs_dev)), float(np.median(runs_e2e))

    # ---- the dominant kernel alone: gate/up of the routed experts (+ the shared expert's down rows in the same launch)
    roof = None
    if rank == 0:
        roof = dominant_kernel_roofline(torch, api, lc, layers, logits_d, x_d, min(K, 64), stream, world,
                                        ms_dev * 1e3 / K, use_graph)
        if world > 1:
            names = ["route+quantize", "gate_up", "grid_barrier", "down+combine", "cross_rank_sum"]
            roof["block0_phase_end_us_last_timed_step"] = {n: step_phases[i + 1] / 1e3 for i, n in enumerate(names)}

    # ---- configuration C5 (IQ3_S, experts partitioned by id, batch 1 and 64; peer exchange against NCCL) on every rank
    c5 = None
    if not args.no_c5:
        import bench_c5
        peer1 = peer64 = None
        if world > 1:
            from project_maya_b200.peer import PeerGroup
            peer1 = PeerGroup.over_processes(rank, world, Hd, timeout_ms=5000.0)
            peer64 = PeerGroup.over_processes(rank, world, 64 * Hd, timeout_ms=5000.0)
        c5 = bench_c5.run(torch, api, dist if world > 1 else None, rank, world, peer1, peer64)

    if rank == 0:
        bytes_tok = algorithmic_bytes_per_token()
        value = K / (ms_dev * 1e-3)
        e2e = K / (ms_e2e * 1e-3)
        peak, peak_kind = measured_peaks()
        line = {
            "metric": "MoE expert-FFN decode tokens/s per layer", "value": value, "unit": "tok/s/layer", "n_gpus": world,
            "steps": K, "warmup": max(W, 3), "ms_per_step": ms_dev / K, "higher_is_better": True,
            "scaling": "strong",     # the token stream is the same at every N: the experts (the work) are divided among the ranks
            "vs_baseline": None, "dtype": "int8 x int8 -> f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "layers_resident": len(layers),
                       "l2": "inputs larger than L2: steps rotate over %d resident layers and 256 tokens" % len(layers),
                       "launch": ("CUDA graph of the K steps" + (", partial outputs summed over peer HBM in the layer kernel's epilogue" if peer is not None else "")),
                       "e2e_pipeline": f"input copies up to {E2E_DEPTH} steps ahead on a copy stream, output copy on a third stream"
                       if use_graph else "eager launches + NCCL all-reduce of the partial outputs (comparison baseline)",
                       "parallelism": "1 GPU" if world == 1 else
                       (f"width-sliced experts (tensor parallel): every rank holds FFN rows {cfg['n_ff'] // world} of {cfg['n_ff']} of all {E} experts and of the shared one"
                        if args.partition == "width" else
                        f"expert-parallel {world} x {per} experts, shared expert width-sliced {world} x {cfg['n_ff_sh'] // world}")},
            # per GPU: at N > 1 every rank streams 1 / N of a token's bytes
            "hbm_gbs_per_gpu": bytes_tok * value / 1e9 / world,
            "hbm_frac_of_%s_peak_per_gpu" % peak_kind: bytes_tok * value / 1e9 / world / peak,
            "hbm_frac_of_nominal_8TBs_per_gpu": bytes_tok * value / 8e12 / world,
            "e2e": {"value": e2e, "unit": "tok/s/layer", "h2d_bytes_per_step": E * 4 + Hd * 2, "d2h_bytes_per_step": Hd * 4,
                    "ms_per_step": ms_e2e / K},
            "gpu_launches": int(launches_per_run),
            "clocks": clocks.summary(),
            "timing": {"replays_of_the_K_steps": len(runs_dev), "ms_per_step_median": ms_dev / K,
                       "ms_per_step_min": min(runs_dev) / K, "ms_per_step_max": max(runs_dev) / K,
                       "e2e_replays": len(runs_e2e), "e2e_ms_per_step_min": min(runs_e2e) / K,
                       "e2e_ms_per_step_max": max(runs_e2e) / K,
                       "us_per_step_x_median_sm_mhz": (ms_dev / K * 1e3) * (clocks.summary()["sm_mhz"] or 0.0)},
            "roofline": roof,
        }
        extra = {}
        if c5 is not None:
            extra["c5"] = c5
        if world == 1 and not args.no_extra:
            del layers[1:]                      # the other workloads bring their own expert tables: make room
            torch.cuda.empty_cache()
            import bench_c1
            import bench_c3
            import bench_prefill
            extra["c1"] = bench_c1.run(torch, api)
            torch.cuda.empty_cache()
            extra["c3"] = bench_c3.run(torch, api)
            torch.cuda.empty_cache()
            pf_clk = ClockSampler(local_rank)
            pf = bench_prefill.run(4, 3, 1, sustained_steps=200, sustained_sampler=pf_clk)   # 4 steps = a burst; 200 = 0.8 s at the power limit
            pf["sustained"]["clocks"] = pf_clk.summary()
            extra["prefill_c4"] = {"workload": pf["config"]["workload"], "tok_s_layer": pf["value"], "ms_per_4096_token_chunk": pf["ms_per_step"],
                                   "e2e_tok_s_layer": pf["e2e"]["value"], "roofline": pf["roofline"], "gpu_launches": pf["gpu_launches"],
                                   "note": "value and roofline: a burst of 4 steps against the burst bf16 peak; sustained: 200 steps back "
                                           "to back at the board's power limit against the sustained bf16 peak",
                                   "sustained": pf["sustained"]}
        if extra:
            line["extra"] = extra
        if world == 1:
            line["gpu_baseline"] = reference_gpu_leg(torch, layers, logits_d, x_d, K)
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            os.environ.setdefault("OMP_NUM_THREADS", str(threads))
            samples = [cpu_layer_tokens(list(range(16)), threads, repeats=5) for _ in range(3)]
            per_tok, kind, note = sorted(samples, key=lambda r: r[0])[1]          # the median of three samples
            line["cpu_baseline"] = {"value": 1.0 / per_tok, "unit": "tok/s/layer", "cores": threads, "kind": kind,
                                    "effective_gbs": bytes_tok / per_tok / 1e9,
                                    "sample": "tokens 0..15 of the 256 after a warm-up token; " + note}
        print(json.dumps(line), flush=True)
    if world > 1:
        if peer is not None and peer.poisoned():
            raise SystemExit("the peer all-reduce timed out: results invalid")
        dist.barrier()
        dist.destroy_process_group()


def reference_gpu_leg(torch, layers, logits_d, x_d, K: int) -> dict:
    """The GPU kernels to beat: the reference's own CUDA kernels for this layer, compiled for sm_100a from the reference
    tree (oracle/_ref/libmaya_ref_gpu.so), on the same resident layers and tokens: router_top10, glmf::quantize_q8_1,
    native_mmvq + glmf::swiglu_q8 (shared gate/up), glmf::moe_gate_up, glmf::moe_down - its launches per token captured
    in one CUDA graph of K steps like this library's arm, CUDA-event timed, median of 5 replays."""
    from oracle import ref_gpu
    if not ref_gpu.available():
        return {"unavailable": "oracle/_ref/libmaya_ref_gpu.so is not built (the reference tree was not present at build time)"}
    cfg = CFG
    R = ref_gpu.RefGpu()
    k = min(K, 256)
    refs = [ref_gpu.RefLayer(R, cfg["n_embd"], cfg["n_ff"], cfg["n_expert"], cfg["k"], cfg["gu_type"], cfg["d_type"], S.row_bytes,
                             L.experts, L.shared, cfg["n_ff_sh"], cfg["sh_gu_type"]) for L in layers]
    xf = x_d.float()
    st = torch.cuda.Stream()
    torch.cuda.synchronize()
    with torch.cuda.stream(st):
        for s_ in range(3):
            refs[s_ % len(refs)].forward(logits_d[s_:s_ + 1], xf[s_:s_ + 1])
    st.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=st):
        for s_ in range(k):
            tok = s_ % N_TOKENS
            refs[s_ % len(refs)].forward(logits_d[tok:tok + 1], xf[tok:tok + 1])
    times = []
    with torch.cuda.stream(st):
        g.replay()
        st.synchronize()
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            g.replay()
            e1.record(st)
            st.synchronize()
            times.append(e0.elapsed_time(e1))
    us = float(np.median(times)) * 1e3 / k
    return {"kernels": "router_top10 + glmf::quantize_q8_1 + native_mmvq/glmf::swiglu_q8 (shared gate/up) + glmf::moe_gate_up + "
                       "glmf::moe_down: the reference's CUDA kernels built for sm_100a, same layers and tokens, CUDA graph",
            "us_per_token": us, "value": 1e6 / us, "unit": "tok/s/layer", "steps": k, "replays": len(times),
            "hbm_gbs": algorithmic_bytes_per_token() / us / 1e3}


# dram__bytes_read.sum + dram__bytes_write.sum of one moe_layer_t1_kernel launch of this workload on one GPU, from the ncu
# capture summarised in profiles/moe_layer_t1_kernel_C2.md (the algorithmic bytes are 136.8 MB: no re-reads)
NCU_TRAFFIC_BYTES_PER_LAUNCH = 141.9e6


def dominant_kernel_roofline(torch, api, lc, layers, logits_d, x_d, steps: int, stream, world: int, us_step: float,
                             in_graph: bool) -> dict:
    """The fused layer kernel against the HBM roofline.  A step of the timed loop IS one launch of this kernel (with the
    cross-rank sum in its epilogue at N > 1), so its average launch duration is the timed region's CUDA-event time over
    its K launches (us_step; it includes the gap between two launches of the graph).  A second leg times launches one
    by one, eagerly, with an event pair each - same rotating layers and tokens - for block 0's phase stamps and as a
    cross-check (event records and eager launch overhead make it the larger number)."""
    cfg = CFG
    Hd, k = cfg["n_embd"], cfg["k"]
    ids = torch.empty((1, k), dtype=torch.int32, device="cuda")
    w = torch.empty((1, k), dtype=torch.float32, device="cuda")
    out = torch.empty((1, Hd), dtype=torch.float32, device="cuda")
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    with torch.cuda.stream(stream):
        for rep in range(2):                     # the first pass is a warm-up
            for s in range(steps):
                tok = s % N_TOKENS
                evs[s][0].record(stream)
                layers[s % len(layers)].forward(logits_d[tok:tok + 1], x_d[tok:tok + 1], ids, w, out)
                evs[s][1].record(stream)
            stream.synchronize()
    us_eager = float(np.mean([a.elapsed_time(b) for a, b in evs])) * 1e3
    us = us_step if in_graph else us_eager
    phases = layers[(steps - 1) % len(layers)].phase_ns(stream)
    peak, kind = measured_peaks()
    alg = algorithmic_bytes_per_token() // world        # N > 1: this rank's mean share (its experts, its slice of the shared one)
    achieved = alg / (us * 1e-6) / 1e9
    return {"bound": "hbm", "kernel": "moe_layer_t1_kernel<IQ2_S, Q8_0> (the whole layer: route, q8_1, gate/up + SwiGLU, down, combine)",
            "achieved": achieved, "peak": peak, "peak_kind": kind, "unit": "GB/s", "frac": achieved / peak,
            "algorithmic_bytes_per_launch": alg, "us_per_launch": us,
            "us_per_launch_from": "the timed region: CUDA events around the graph of K launches, / K" if in_graph else "one CUDA-event pair per eager launch",
            "us_per_launch_eager_event_pairs": us_eager, "eager_launches_timed": steps,
            "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH if world == 1 else None,
            "block0_phase_end_us": {"route+quantize": phases[1] / 1e3, "gate_up": phases[2] / 1e3, "grid_barrier": phases[3] / 1e3,
                                    "down+combine": phases[4] / 1e3}}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1024)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip extra.c1, extra.c3 and extra.prefill_c4 (1 GPU)")
    ap.add_argument("--no-c5", action="store_true", help="skip the extra.c5 leg (IQ3_S expert-parallel layer, batch 1 and 64)")
    ap.add_argument("--ar", default="peer", choices=["peer", "nccl"], help="N > 1: how the ranks' partial outputs are summed")
    ap.add_argument("--partition", default="width", choices=["width", "expert"],
                    help="N > 1: every rank holds a width slice of every expert (default), or whole experts by id")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "c3"],
                    help="decode: the headline single-token layer (C2); prefill: the 4096-token prompt chunk (C4), 1 GPU; "
                         "c3: the 8-token decode window (C3), 1 GPU")
    ap.add_argument("--prefill-scale", type=int, default=1,
                    help="prefill only: divide experts and tokens by this (a reduced case for profiler captures)")
    args = ap.parse_args()
    if args.workload == "prefill" and args.impl == "ours":
        import bench_prefill
        steps = args.steps if args.steps != 256 else 8
        sampler = ClockSampler(0)
        line = bench_prefill.run(steps, args.warmup if args.warmup != 8 else 3, min(args.layers, 2), sampler, args.prefill_scale)
        line["clocks"] = sampler.summary()
        print(json.dumps(line))
        return
    if args.workload == "c3" and args.impl == "ours":
        import torch
        import bench_c3
        from project_maya_b200 import api
        print(json.dumps(bench_c3.run(torch, api)))
        return
    if args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
