"""More than one rank: the partition's host logic on CPU with gloo (always), the peer-memory all-reduce and the
expert-parallel layer on real GPUs (when the machine has at least two)."""
import socket

import numpy as np
import pytest

import helpers as H


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(worker, world, *args, timeout=300):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, *args, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    try:
        for _ in range(world):
            results.append(q.get(timeout=timeout))
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.terminate()
    for rank, bad, poisoned, err in sorted(results):
        assert err is None, f"rank {rank}: {err}"
        assert bad == 0 and not poisoned, f"rank {rank}: {bad} mismatches, poisoned={poisoned}"


def test_partition_host_logic_gloo_world2():
    import mp_workers
    _run(mp_workers.gloo_partition_worker, 2)


def _gpus() -> int:
    import torch
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_allreduce_bit_equal_over_unbarriered_calls(world):
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    import mp_workers
    _run(mp_workers.peer_allreduce_worker, world, 6144, 128, 1)


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_layer_fused_allreduce(world):
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    import mp_workers
    _run(mp_workers.layer_ep_worker, world)
