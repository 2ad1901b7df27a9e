"""The peer-memory all-reduce on one GPU: every "rank" of a group lives on the same device and runs alone, with the
other ranks' rows and flags placed in its receive buffers beforehand (what their pushes would have left there).
Checks the rank-ordered sum bit for bit on special values, the pushes a rank makes, sequence wrap, argument refusals,
and the bounded wait: a flag nobody sets makes the call give up, record the failure and poison the transport."""
import ctypes as C
import time

import numpy as np
import pytest

import helpers as H
from mp_workers import SPECIAL, rank_vector

pytestmark = pytest.mark.gpu

BLOCKS, FSTRIDE = 256, 32


@pytest.fixture(scope="module")
def T(cuda):
    import torch
    return torch


def buffers(T, r):
    recv = r.keep[0][r.mi][: 2 * r.nm * r.stride * 4].view(T.float32).view(2, r.nm, r.stride)
    flags = r.keep[1][r.mi].view(T.int32).view(2, r.nm, BLOCKS, FSTRIDE)
    return recv, flags


def place_peer_pushes(T, ranks, mi, seq, vectors, later_only=False):
    """What ranks != mi would have stored into rank mi's buffers for call `seq`.  later_only: only the ranks that run
    after mi in a test that runs the ranks in order - the earlier ranks' rows and flags then come from their real pushes."""
    recv, flags = buffers(T, ranks[mi])
    slot = seq & 1
    for m, v in enumerate(vectors):
        if m != mi and (m > mi or not later_only):
            recv[slot, m, : v.numel()] = v
            flags[slot, m, :, 0] = int(np.array(seq, np.uint32).view(np.int32))


@pytest.mark.parametrize("nm", [2, 3, 8])
@pytest.mark.parametrize("n", [6144, 64 * 6144, 4])
def test_rank_ordered_sum_and_pushes(T, oracle, nm, n):
    from project_maya_b200.peer import PeerGroup
    ranks = PeerGroup.on_one_device(nm, stride=max(n, 8), timeout_ms=50.0)
    for seq in (1, 2, 3):
        vecs_np = [rank_vector(m, seq, n) for m in range(nm)]
        vecs_np[0][:SPECIAL.size if n >= SPECIAL.size else n] = SPECIAL[: min(n, SPECIAL.size)]
        want = oracle.allreduce_in_order(np.stack(vecs_np))
        vecs = [T.from_numpy(v).cuda() for v in vecs_np]
        for mi in range(nm):
            place_peer_pushes(T, ranks, mi, seq, vecs, later_only=True)
        outs = []
        for mi in range(nm):
            x = vecs[mi].clone()
            ranks[mi].allreduce(x, seq=seq)
            outs.append(x)
        T.cuda.synchronize()
        for mi in range(nm):
            assert outs[mi].cpu().numpy().tobytes() == want.tobytes(), f"rank {mi} seq {seq}"   # same bits on every rank
            assert not ranks[mi].poisoned()
        # every rank pushed its own row and flag into every peer
        for mi in range(nm):
            recv, flags = buffers(T, ranks[mi])
            for m in range(nm):
                if m != mi:
                    assert T.equal(recv[seq & 1, m, :n], vecs[m])
                    assert int(flags[seq & 1, m, 0, 0].item()) == seq


def test_sequence_wraps(T, oracle):
    from project_maya_b200.peer import PeerGroup
    nm, n = 2, 1024
    ranks = PeerGroup.on_one_device(nm, stride=n, timeout_ms=50.0)
    first = 0xFFFFFFF0
    for r in ranks:                                     # flags start at first_seq - 1
        buffers(T, r)[1].fill_(int(np.array(first - 1, np.uint32).view(np.int32)))
    for i in range(40):                                 # crosses 2^32
        seq = (first + i) & 0xFFFFFFFF
        vecs_np = [rank_vector(m, i, n) for m in range(nm)]
        vecs = [T.from_numpy(v).cuda() for v in vecs_np]
        for mi in range(nm):
            place_peer_pushes(T, ranks, mi, seq, vecs)
        x = vecs[1].clone()
        ranks[1].allreduce(x, seq=seq)
        assert x.cpu().numpy().tobytes() == oracle.allreduce_in_order(np.stack(vecs_np)).tobytes()
    assert not ranks[1].poisoned()


def test_missing_rank_times_out_and_poisons(T):
    from project_maya_b200.peer import PeerGroup
    nm, n = 4, 6144
    ranks = PeerGroup.on_one_device(nm, stride=n, timeout_ms=20.0)
    vecs = [T.from_numpy(rank_vector(m, 0, n)).cuda() for m in range(nm)]
    place_peer_pushes(T, ranks, 0, 1, vecs)
    buffers(T, ranks[0])[1][1, 2].zero_()               # rank 2 never arrives: its flags stay behind
    x = vecs[0].clone()
    t0 = time.time()
    ranks[0].allreduce(x, seq=1)
    T.cuda.synchronize()
    assert time.time() - t0 < 2.0                       # bounded: gave up after ~20 ms, the context is still usable
    assert ranks[0].poisoned()
    f = ranks[0].failure_record()
    assert f.captured == 1 and f.sequence == 1 and f.rank == 0 and f.waited_for == 2 and f.elapsed_ns >= f.timeout_ns
    assert T.equal(x, vecs[0])                          # left as the local partial
    t0 = time.time()
    for seq in range(2, 34):                            # a poisoned transport drains later calls at once
        ranks[0].allreduce(x, seq=seq)
    T.cuda.synchronize()
    assert time.time() - t0 < 1.0
    assert T.equal(x, vecs[0])
    assert bool((T.ones(4, device="cuda") * 2 == 2).all())   # the device still answers


def test_refusals(T):
    from project_maya_b200 import api
    from project_maya_b200.peer import PeerGroup
    r = PeerGroup.on_one_device(2, stride=1024)[0]
    x = T.zeros(1024, device="cuda")
    with pytest.raises(api.MayaError):
        r.allreduce(x[:1022], seq=1)                    # n % 4 != 0
    big = T.zeros(2048, device="cuda")
    with pytest.raises(api.MayaError):
        r.allreduce(big, seq=1)                         # n beyond the slots' stride
    with pytest.raises(api.MayaError):
        r.allreduce(T.zeros(1028, device="cuda")[1:1025], seq=1)   # not 16-byte aligned
    assert not r.poisoned()
