"""The entry point for callers that cannot allocate: maya_expert_grouped_static keeps its scratch inside the library.

Checked through the C ABI against maya_expert_grouped (caller-provided scratch) on the same inputs: same bits, on two
calls in a row with different inputs (the built-in array still holds the first call's h when the second starts), and
the size limit is refused with a status rather than overrun.  Runs last by name so a failure here cannot hide others.
"""
import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu


def _case(T, api, t, n_embd, n_ff, n_tok, seed):
    rng = H.rng_for("no-alloc", seed, t)
    blobs = np.stack([H.constructed_expert(t, t, n_embd, n_ff, rng) for _ in range(3)])
    store = T.from_numpy(blobs).cuda()
    x = T.from_numpy(rng.standard_normal((n_tok, n_embd)).astype(np.float32)).cuda()
    xq = api.native_quantize_q8_1(x)
    order = rng.permutation(n_tok)
    cut = int(rng.integers(1, n_tok))
    grp_ptr = T.tensor([store[0].data_ptr(), store[1].data_ptr(), store[2].data_ptr()], dtype=T.int64, device="cuda")
    grp_start = T.tensor([0, cut, cut, n_tok], dtype=T.int32, device="cuda")      # the middle group is empty
    ent_tok = T.from_numpy(order.astype(np.int32)).cuda()
    ent_dst = T.from_numpy(rng.permutation(n_tok).astype(np.int32)).cuda()
    n_groups = T.tensor([3], dtype=T.int32, device="cuda")
    return dict(store=store, xq=xq, grp_ptr=grp_ptr, grp_start=grp_start, ent_tok=ent_tok, ent_dst=ent_dst,
                n_groups=n_groups, n_tok=n_tok)


def test_static_scratch_variant_matches_caller_scratch_variant(cuda):
    import torch as T
    from project_maya_b200 import _lib, api
    lib = _lib.load()
    assert lib.maya_expert_static_scratch_bytes() == 2 << 20
    n_embd, n_ff = 512, 256
    for call, (t, n_tok) in enumerate([(H.IQ2_S, 7), (H.Q4_K, 5)]):              # two calls in a row, different inputs
        c = _case(T, api, t, n_embd, n_ff, n_tok, call)
        L = api.native_expert_layout(t, t, n_embd, n_ff)
        want = T.full((n_tok, n_embd), 5.0, dtype=T.float32, device="cuda")
        scratch = T.zeros(api.native_expert_scratch_bytes(n_tok, n_ff), dtype=T.uint8, device="cuda")
        api.native_expert_grouped(L, c["grp_ptr"], c["grp_start"], c["n_groups"], c["ent_dst"], c["ent_tok"], 3, n_tok,
                                  c["xq"], scratch, want, 7.0)
        got = T.full((n_tok, n_embd), 5.0, dtype=T.float32, device="cuda")
        api.native_expert_grouped_static(L, c["grp_ptr"], c["grp_start"], c["n_groups"], c["ent_dst"], c["ent_tok"], 3,
                                         n_tok, c["xq"], got, 7.0)
        T.cuda.synchronize()
        assert T.equal(got, want), f"call {call}"
        assert bool(T.isfinite(got).all()) and bool((got != 5.0).any())


def test_static_scratch_limit_is_refused(cuda):
    import torch as T
    from project_maya_b200 import api
    L = api.native_expert_layout(H.Q4_K, H.Q4_K, 512, 2048)
    too_many = (2 << 20) // (2048 // 32 * 36) + 1
    dummy = T.zeros(64, dtype=T.int32, device="cuda")
    with pytest.raises(api.MayaError) as e:
        api.native_expert_grouped_static(L, dummy, dummy, dummy, dummy, dummy, 1, too_many, dummy, dummy.float())
    assert e.value.status == -4


def test_entry_cap_holds_on_the_device(cuda):
    """A start table that claims more entries than cap_entries (inconsistent device data) must not make the kernels
    write past the scratch - here the library's own array - or past `out`: entries at and beyond the cap are left alone."""
    import torch as T
    from project_maya_b200 import api
    t, n_embd, n_ff, cap, claimed = H.Q4_K, 512, 256, 4, 9
    rng = H.rng_for("cap")
    blob = T.from_numpy(H.constructed_expert(t, t, n_embd, n_ff, rng)).cuda()
    x = T.from_numpy(rng.standard_normal((claimed, n_embd)).astype(np.float32)).cuda()
    xq = api.native_quantize_q8_1(x)
    grp_ptr = T.tensor([blob.data_ptr()], dtype=T.int64, device="cuda")
    ent = T.arange(claimed, dtype=T.int32, device="cuda")
    n_groups = T.tensor([1], dtype=T.int32, device="cuda")
    L = api.native_expert_layout(t, t, n_embd, n_ff)
    outs = []
    for n_claim in (cap, claimed):
        grp_start = T.tensor([0, n_claim], dtype=T.int32, device="cuda")
        out = T.full((claimed, n_embd), 5.0, dtype=T.float32, device="cuda")
        api.native_expert_grouped_static(L, grp_ptr, grp_start, n_groups, ent, ent, 1, cap, xq, out, 7.0)
        T.cuda.synchronize()
        assert bool((out[cap:] == 5.0).all()), "rows beyond cap_entries were written"
        outs.append(out)
    assert T.equal(outs[0], outs[1])
    assert bool((outs[0][:cap] != 5.0).any())

