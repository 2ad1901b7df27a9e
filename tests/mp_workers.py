"""Worker functions for the multi-process tests (one process per rank)."""
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

SPECIAL = np.array([0.0, -0.0, 3.4028234663852886e38, -3.4028234663852886e38, 1.401298464324817e-45,
                    -1.401298464324817e-45, 1.1754942106924411e-38, 1.0, -1.0, 16777216.0, 1e-20, 0.33333334], np.float32)


def rank_vector(rank: int, call: int, n: int) -> np.ndarray:
    """Deterministic per-(rank, call) data every rank can regenerate: normal values with special values mixed in."""
    rng = np.random.Generator(np.random.Philox(key=[rank * 1000003 + call, 77]))
    v = rng.standard_normal(n).astype(np.float32)
    idx = rng.integers(0, n, size=max(4, n // 64))
    v[idx] = SPECIAL[rng.integers(0, SPECIAL.size, size=idx.size)]
    return v


def _init(rank: int, world: int, port: int, gpu: bool):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    if gpu:
        torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    return torch, dist


def peer_allreduce_worker(rank: int, world: int, port: int, n: int, calls: int, first_seq: int, q):
    """`calls` un-barriered all-reduces; every result must equal the rank-ordered sum bit for bit on every rank."""
    try:
        torch, dist = _init(rank, world, port, True)
        from oracle.oracle import Oracle
        from project_maya_b200.peer import PeerGroup
        orc = Oracle()
        peer = PeerGroup.over_processes(rank, world, n, timeout_ms=5000.0)
        if first_seq != 1:      # flags start at first_seq - 1 on every rank (sequence numbers wrap modulo 2^32)
            raise NotImplementedError
        bad = 0
        outs = []
        for c in range(calls):
            x = torch.from_numpy(rank_vector(rank, c, n)).cuda()
            peer.allreduce(x)
            outs.append(x)
        torch.cuda.synchronize()
        for c in range(calls):
            want = orc.allreduce_in_order(np.stack([rank_vector(m, c, n) for m in range(world)]))
            got = outs[c].cpu().numpy()
            if got.tobytes() != want.tobytes():
                bad += 1
        poisoned = peer.poisoned()
        dist.barrier()
        q.put((rank, bad, poisoned, None))
    except Exception as e:   # noqa: BLE001
        q.put((rank, -1, True, repr(e)))


def layer_ep_worker(rank: int, world: int, port: int, q):
    """Expert-parallel layer: every rank holds all experts' bytes (same seeds) but owns a slice; the fused kernel's
    epilogue sums the partial outputs across ranks.  Checks: same bits on every rank, and equal to the rank-ordered sum of
    the partials computed without the exchange."""
    try:
        torch, dist = _init(rank, world, port, True)
        import helpers as H
        from oracle.oracle import Oracle
        from project_maya_b200 import api
        from project_maya_b200.peer import PeerGroup
        orc = Oracle()
        n_embd, n_ff, E, k = 2048, 2048, 16, 8
        lc = api.MoeLayerConfig(n_embd, n_ff, E, k, api.IQ3_S, api.IQ3_S, n_ff_sh=512)
        experts = torch.empty((E, lc.blob_bytes), dtype=torch.uint8, device="cuda")
        gu = 2 * n_ff * api.row_bytes(api.IQ3_S, n_embd)
        for e in range(E):
            api.synth_weights(api.IQ3_S, 2 * e, 0.02, 2 * n_ff, n_embd, experts[e, :gu])
            api.synth_weights(api.IQ3_S, 2 * e + 1, 0.02, n_embd, n_ff, experts[e, gu:])
        shared = torch.empty(lc.shared_bytes, dtype=torch.uint8, device="cuda")
        sgu = 2 * 512 * api.row_bytes(api.Q8_0, n_embd)
        api.synth_weights(api.Q8_0, 901, 0.02, 2 * 512, n_embd, shared[:sgu])
        api.synth_weights(api.Q8_0, 902, 0.02, n_embd, 512, shared[sgu:])
        per = E // world
        layer = api.MoeLayer(lc, experts, shared, expert_range=(rank * per, (rank + 1) * per), shared_here=(rank == 0))
        partial_layers = [api.MoeLayer(lc, experts, shared, expert_range=(m * per, (m + 1) * per), shared_here=(m == 0))
                          for m in range(world)]
        peer = PeerGroup.over_processes(rank, world, 16 * n_embd, timeout_ms=5000.0)
        logits = H.router_logits("ep", 24, E, 1.1)
        x = H.activations("ep", 24, n_embd, "bf16")
        ld, xd = torch.from_numpy(logits).cuda(), torch.from_numpy(x).to(torch.bfloat16).cuda()
        bad = 0
        results = []
        for t in range(8):                                   # single tokens: the fused kernel's epilogue
            results.append(layer.forward(ld[t:t + 1], xd[t:t + 1], peer=peer)[2].clone())
        results.append(layer.forward(ld[8:24], xd[8:24], peer=peer)[2].clone())   # a 16-token window: staged + allreduce
        torch.cuda.synchronize()
        for i, got in enumerate(results):
            sl = slice(i, i + 1) if i < 8 else slice(8, 24)
            parts = [pl.forward(ld[sl], xd[sl])[2].cpu().numpy() for pl in partial_layers]
            want = np.stack([orc.allreduce_in_order(np.stack([p[r] for p in parts])) for r in range(parts[0].shape[0])])
            if got.cpu().numpy().tobytes() != want.tobytes():
                bad += 1
        # sequence numbers counted on the device: three single-token calls captured in a CUDA graph, replayed twice
        peer.set_device_seq(True)
        ids_g = torch.empty((3, 1, k), dtype=torch.int32, device="cuda")
        w_g = torch.empty((3, 1, k), dtype=torch.float32, device="cuda")
        out_g = torch.zeros((3, 1, n_embd), dtype=torch.float32, device="cuda")
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for t in range(3):
                layer.forward(ld[t:t + 1], xd[t:t + 1], ids_g[t], w_g[t], out_g[t], peer=peer)
        for _ in range(2):
            out_g.zero_()
            graph.replay()
            torch.cuda.synchronize()
            for t in range(3):
                if out_g[t].cpu().numpy().tobytes() != results[t].cpu().numpy().tobytes():
                    bad += 1
        # every rank holds the same bits
        mine = np.concatenate([r.cpu().numpy().reshape(-1) for r in results])
        gathered = [None] * world
        dist.all_gather_object(gathered, mine.tobytes())
        same = all(g == gathered[0] for g in gathered)
        dist.barrier()
        q.put((rank, bad + (0 if same else 100), peer.poisoned(), None))
    except Exception as e:   # noqa: BLE001
        import traceback
        q.put((rank, -1, True, traceback.format_exc()))


def gloo_partition_worker(rank: int, world: int, port: int, q):
    """CPU only: the expert-parallel partition's host logic with gloo - each rank computes its experts' partial with the
    oracle, the partials are gathered and summed in rank order."""
    try:
        torch, dist = _init(rank, world, port, False)
        import helpers as H
        from oracle.oracle import Oracle
        orc = Oracle()
        cfg = dict(n_embd=512, n_ff=256, n_expert=8, k=4, gu_type=H.Q4_K, d_type=H.Q4_K, limit=H.INF)
        rng = H.rng_for("gloo-ep")
        experts = np.stack([H.constructed_expert(H.Q4_K, H.Q4_K, 512, 256, rng) for _ in range(8)])
        logits = H.router_logits("gloo", 3, 8, None)
        x = H.activations("gloo", 3, 512, "f32")
        per = 8 // world
        ids, w, part = orc.moe_layer(cfg, logits, x, experts, expert_range=(rank * per, (rank + 1) * per))
        gathered = [None] * world
        dist.all_gather_object(gathered, part.tobytes())
        parts = [np.frombuffer(g, np.float32).reshape(part.shape) for g in gathered]
        total = np.stack([orc.allreduce_in_order(np.stack([p[t] for p in parts])) for t in range(3)])
        _, _, whole = orc.moe_layer(cfg, logits, x, experts)
        err = float(np.abs(total - whole).max() / np.abs(whole).max())
        ids_all = [None] * world
        dist.all_gather_object(ids_all, ids.tobytes())
        q.put((rank, 0 if (err < 1e-5 and all(i == ids_all[0] for i in ids_all)) else 1, False, None))
    except Exception as e:   # noqa: BLE001
        import traceback
        q.put((rank, -1, True, traceback.format_exc()))
