"""Seeded synthetic inputs: the five benchmark configurations' shapes and value distributions (tests and bench)."""
from __future__ import annotations

import numpy as np

Q8_0, Q4_K, IQ3_S, IQ2_S = 8, 12, 21, 22
Q5_K, Q6_K, IQ2_XXS, IQ3_XXS, IQ1_S, IQ4_XS = 13, 14, 16, 18, 19, 23   # staged decode paths only
BLOCK = {Q8_0: (32, 34), Q4_K: (256, 144), IQ3_S: (256, 110), IQ2_S: (256, 82),
         Q5_K: (256, 176), Q6_K: (256, 210), IQ2_XXS: (256, 66), IQ3_XXS: (256, 98), IQ4_XS: (256, 136), IQ1_S: (256, 50)}
CORE_TYPES = (Q8_0, Q4_K, IQ2_S, IQ3_S)
MORE_TYPES = (Q5_K, Q6_K, IQ4_XS, IQ3_XXS, IQ2_XXS, IQ1_S)
INF = float("inf")

# name -> (n_embd, n_ff, n_expert, k, gu/d type, shared (n_ff_sh, type) or None, activation dtype, tokens per step)
CONFIGS = {
    "C1": dict(n_embd=2048, n_ff=1024, n_expert=64, k=8, gu_type=Q4_K, d_type=Q4_K, act="f32", T=1, tokens=16),
    "C2": dict(n_embd=6144, n_ff=2048, n_expert=256, k=8, gu_type=IQ2_S, d_type=IQ2_S, n_ff_sh=2048, sh_gu_type=Q8_0,
               sh_d_type=Q8_0, act="bf16", T=1, tokens=256, zipf=1.1),
    "C3": dict(n_embd=7168, n_ff=2048, n_expert=256, k=8, gu_type=Q4_K, d_type=Q4_K, act="bf16", T=8, zipf=1.1),
    "C4": dict(n_embd=6144, n_ff=2048, n_expert=256, k=8, types=(Q8_0, Q4_K), act="bf16", T=4096),
    "C5": dict(n_embd=6144, n_ff=2048, n_expert=256, k=8, gu_type=IQ3_S, d_type=IQ3_S, act="bf16", T=64, zipf=1.1),
}


def rng_for(*key) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[hash_key(key), 0x6d617961]))


def hash_key(key) -> int:
    h = 1469598103934665603
    for part in key:
        for b in str(part).encode():
            h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


def row_bytes(t: int, n: int) -> int:
    qk, bb = BLOCK[t]
    return n // qk * bb


def blob_bytes(gu_type: int, d_type: int, n_embd: int, n_ff: int) -> int:
    return 2 * n_ff * row_bytes(gu_type, n_embd) + n_embd * row_bytes(d_type, n_ff)


def expert_types(cfg_name: str, n_expert: int, types) -> np.ndarray:
    """Seeded assignment of storage types to experts, the same number of experts for every type (C4: half Q8_0, half
    Q4_K)."""
    perm = rng_for(cfg_name, "types").permutation(n_expert)
    out = np.empty(n_expert, dtype=np.int32)
    for i, t in enumerate(types):
        out[perm[i * n_expert // len(types):(i + 1) * n_expert // len(types)]] = t
    return out


def to_bf16_f32(x: np.ndarray) -> np.ndarray:
    """Round f32 to bf16 (nearest even) and widen back: what a bf16 activation holds."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def bf16_bits(x_f32_rounded: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(x_f32_rounded, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


def zipf_bias(n_expert: int, s: float, rng: np.random.Generator) -> np.ndarray:
    """Additive router bias log(zipf pmf) over a seeded permutation of the experts."""
    ranks = np.arange(1, n_expert + 1, dtype=np.float64)
    pmf = ranks ** (-s)
    pmf /= pmf.sum()
    bias = np.log(pmf) - np.log(pmf).mean()
    return bias[rng.permutation(n_expert)].astype(np.float32)


def router_logits(cfg_name: str, n_tokens: int, n_expert: int, zipf: float | None, seed=0) -> np.ndarray:
    rng = rng_for(cfg_name, "logits", seed)
    l = rng.standard_normal((n_tokens, n_expert)).astype(np.float32)
    if zipf:
        l = l + zipf_bias(n_expert, zipf, rng_for(cfg_name, "zipf", seed))[None, :]
    return l.astype(np.float32)


def activations(cfg_name: str, n_tokens: int, n_embd: int, act: str, seed=0) -> np.ndarray:
    x = rng_for(cfg_name, "x", seed).standard_normal((n_tokens, n_embd)).astype(np.float32)
    return to_bf16_f32(x) if act == "bf16" else x


def constructed_blocks(t: int, n_rows: int, n_cols: int, rng: np.random.Generator) -> np.ndarray:
    """Random valid blocks (every bit pattern of the index / sign / scale fields is a valid encoding) with finite
    positive f16 super-scales, the construction the reference's fixture tool uses for its K- and i-quant tensors."""
    qk, bb = BLOCK[t]
    nb = n_rows * (n_cols // qk)
    b = rng.integers(0, 256, size=(nb, bb), dtype=np.uint8)
    lo, hi = {Q8_0: (2e-4, 6e-4), Q4_K: (1e-4, 4e-4), IQ2_S: (2e-3, 6e-3), IQ3_S: (2e-3, 6e-3), Q5_K: (5e-5, 2e-4),
              Q6_K: (1e-5, 3e-5), IQ4_XS: (1e-5, 3e-5), IQ3_XXS: (2e-4, 6e-4), IQ2_XXS: (2e-4, 6e-4), IQ1_S: (2e-3, 6e-3)}[t]
    d_at = 208 if t == Q6_K else 0                        # Q6_K keeps its super-scale at the end of the block
    b[:, d_at:d_at + 2] = rng.uniform(lo, hi, size=nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    if t in (Q4_K, Q5_K):
        b[:, 2:4] = rng.uniform(lo, hi, size=nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    if t == Q8_0:   # keep -128 out of the weights, as a quantizer would
        q = b[:, 2:].view(np.int8)
        np.clip(q, -127, 127, out=q)
    return b.reshape(n_rows, n_cols // qk * bb)


def constructed_expert(gu_type: int, d_type: int, n_embd: int, n_ff: int, rng: np.random.Generator) -> np.ndarray:
    gu = constructed_blocks(gu_type, 2 * n_ff, n_embd, rng).reshape(-1)
    dn = constructed_blocks(d_type, n_embd, n_ff, rng).reshape(-1)
    return np.concatenate([gu, dn])


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    """max |got - want| / max |want|: the tolerance metric of the output parity tests."""
    want = np.asarray(want, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def rel_l2(got: np.ndarray, want: np.ndarray) -> float:
    want = np.asarray(want, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
