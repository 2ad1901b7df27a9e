"""Configuration C5 for `bench.py` (its `extra.c5` object): the expert-parallel decode layer - hidden 6144, 256 routed
experts of FFN 2048 stored as IQ3_S, top-8 with Zipf(1.1)-skewed routing, no shared expert - at batch 1 and batch 64,
with experts [rank * E / N, (rank + 1) * E / N) on rank `rank` and the ranks' partial outputs summed

  * "peer": inside this library's kernels (batch 1: the fused layer kernel's epilogue, {seq, value} words into every
    peer's HBM; batch 64: the prompt path, the rows + flags exchange inside its combine launch), or
  * "nccl": by ncclAllReduce after the layer (the comparison baseline).

Batch 1 replays a CUDA graph of 64 tokens, batch 64 a CUDA graph of 4 prompt-path steps (the NCCL arm launches eagerly).  Times are CUDA events on
the launching stream, the maximum over the ranks, the median of 5 runs.  Also reported: the load imbalance the skewed
routing leaves (bytes of distinct local experts per rank: max / mean over ranks, averaged over the steps).
"""
from __future__ import annotations

import numpy as np

from project_maya_b200 import synthetic as S

CFG = S.CONFIGS["C5"]
N_T1, N_T64_STEPS = 64, 4


def _timed(torch, dist, world, stream, fn, runs=5):
    out = []
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        for _ in range(runs):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            fn()
            e1.record(stream)
            stream.synchronize()
            ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            out.append(float(ms.item()))
    return float(np.median(out))


def run(torch, api, dist, rank: int, world: int, peer1, peer64) -> dict:
    """peer1 / peer64: peer.PeerRank transports sized for n_embd and 64 * n_embd floats (None at one GPU)."""
    cfg = CFG
    Hd, FF, E, k = cfg["n_embd"], cfg["n_ff"], cfg["n_expert"], cfg["k"]
    t = cfg["gu_type"]
    lc = api.MoeLayerConfig(Hd, FF, E, k, t, t)
    per = E // world
    lo, hi = rank * per, (rank + 1) * per
    # every rank allocates the whole table but fills (and reads) only its own experts
    experts = torch.empty((E, lc.blob_bytes), dtype=torch.uint8, device="cuda")
    gu = 2 * FF * S.row_bytes(t, Hd)
    for e in range(lo, hi):
        api.synth_weights(t, 500000 + 2 * e, 0.02, 2 * FF, Hd, experts[e, :gu])
        api.synth_weights(t, 500001 + 2 * e, 0.02, Hd, FF, experts[e, gu:])
    torch.cuda.synchronize()
    rng = (lo, hi) if world > 1 else None
    layer = api.MoeLayer(lc, experts, None, expert_range=rng, max_tokens=1)
    prefill = api.MoePrefill(lc, experts, max_tokens=64, expert_range=rng)
    logits_np = S.router_logits("C5", 64 * N_T64_STEPS, E, cfg["zipf"])
    logits = torch.from_numpy(logits_np).cuda()
    x = torch.from_numpy(S.bf16_bits(S.activations("C5", 64 * N_T64_STEPS, Hd, "bf16")).view(np.int16)).view(torch.bfloat16).cuda()
    out1 = torch.empty((N_T1, Hd), dtype=torch.float32, device="cuda")
    ids1 = torch.empty((N_T1, k), dtype=torch.int32, device="cuda")
    w1 = torch.empty((N_T1, k), dtype=torch.float32, device="cuda")
    stream = torch.cuda.Stream()
    res = {"workload": "C5: H6144 E256 FF2048 top8 IQ3_S, bf16 acts, Zipf(1.1), experts partitioned by id over the ranks",
           "n_gpus": world}

    # ---- load balance of the partition on these tokens (host arithmetic on the routing)
    order = np.argsort(-logits_np, axis=1, kind="stable")[:, :k]
    blob = lc.blob_bytes
    def imbalance(groups):
        ratios = []
        for g in groups:
            per_rank = [len({int(e) for e in np.unique(order[g]) if r * per <= e < (r + 1) * per}) * blob for r in range(world)]
            ratios.append(max(per_rank) / max(np.mean(per_rank), 1.0))
        return float(np.mean(ratios))
    res["expert_bytes_max_over_mean"] = {"batch_1": imbalance([[i] for i in range(N_T1)]),
                                         "batch_64": imbalance([list(range(64 * s, 64 * s + 64)) for s in range(N_T64_STEPS)])}

    # ---- batch 1
    def t1_steps(peer):
        for s in range(N_T1):
            layer.forward(logits[s:s + 1], x[s:s + 1], ids1[s:s + 1], w1[s:s + 1], out1[s:s + 1], peer=peer)
            if world > 1 and peer is None:
                dist.all_reduce(out1[s:s + 1])
    modes = [("peer", peer1)] if world > 1 else [("single", None)]
    if world > 1:
        modes.append(("nccl", None))
    b1 = {}
    for name, peer in modes:
        with torch.cuda.stream(stream):
            for s in range(3):
                layer.forward(logits[s:s + 1], x[s:s + 1], ids1[s:s + 1], w1[s:s + 1], out1[s:s + 1], peer=peer)
        stream.synchronize()
        if name == "nccl":
            fn = lambda: t1_steps(None)                          # eager launches + ncclAllReduce per token
        else:
            if peer is not None:
                peer.set_device_seq(True)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                t1_steps(peer)
            fn = g.replay
        ms = _timed(torch, dist, world, stream, fn)
        b1[name] = {"us_per_token": ms * 1e3 / N_T1, "tok_s_layer": N_T1 / (ms * 1e-3),
                    "launch": "eager + ncclAllReduce" if name == "nccl" else "CUDA graph of 64 tokens"}
        if peer is not None:
            peer.set_device_seq(False)
    res["batch_1"] = b1

    # ---- batch 64: the prompt path
    def t64_steps(peer):
        for s in range(N_T64_STEPS):
            ffn = prefill.forward(logits[64 * s:64 * s + 64], x[64 * s:64 * s + 64], peer=peer)[2]
            if world > 1 and peer is None:
                dist.all_reduce(ffn)
    b64 = {}
    for name, peer in ([("peer", peer64), ("nccl", None)] if world > 1 else [("single", None)]):
        with torch.cuda.stream(stream):
            t64_steps(peer)
        stream.synchronize()
        if name == "nccl":
            fn = lambda: t64_steps(None)
        else:
            if peer is not None:
                peer.set_device_seq(True)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                t64_steps(peer)
            fn = g.replay
        ms = _timed(torch, dist, world, stream, fn)
        b64[name] = {"us_per_64_tokens": ms * 1e3 / N_T64_STEPS, "tok_s_layer": 64 * N_T64_STEPS / (ms * 1e-3),
                     "launch": "eager launches of the prompt path + ncclAllReduce" if name == "nccl"
                     else f"CUDA graph of {N_T64_STEPS} prompt-path steps"}
        if peer is not None:
            peer.set_device_seq(False)
    res["batch_64"] = b64
    res["errors"] = {"layer": layer.error(), "prefill": prefill.error(),
                     "peer": bool(peer1.poisoned() or peer64.poisoned()) if world > 1 else False}
    return res
