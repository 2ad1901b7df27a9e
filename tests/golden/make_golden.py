#!/usr/bin/env python3
"""Generate the committed golden fixtures of tests/golden/ (run where the reference tree is mounted).

    python tests/golden/make_golden.py

Needs oracle/_ref/libmaya_ref.so (python oracle/build.py), i.e. the reference's own CPU code compiled from its tree,
and the reference's data directory.  Writes:

  router_reference_cases.npz  the four input distributions of the reference's router test (its generator and seed;
                              first 16 of the 64 tokens, 512 experts, k = 10) with the ids / weights its own host
                              reference gives
  glm5_synth_moe_layer1.npz   layer 1 of data/glm5-synth.gguf (expert, shared-expert and router tensors, F32) with llama.cpp's
                              captured inputs and outputs of its MoE block for 8 tokens (data/glm5-synth-dumps/ffn_*-1.f32)
  glm5_synth_router.npz       the sigmoid router's golden vectors captured from llama.cpp that the reference ships
                              (data/glm5-synth-dumps/ffn_moe_{logits,topk,weights}-{1..5}.f32) with the selection bias
                              and weight scale read from data/glm5-synth.gguf
  c1_reference_cpu.npz        configuration C1 (hidden 2048, 64 experts of FFN 1024, top-8, Q4_K, f32 activations,
                              16 seeded tokens): ids / weights / outputs from the reference's AVX-512 CPU expert rows
                              (Q8_K activations) and the sha256 of the synthetic expert bytes they were computed on
"""
from __future__ import annotations

import hashlib
import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import helpers as H  # noqa: E402
from oracle.oracle import Oracle, Ref  # noqa: E402

from oracle.build import REFERENCE  # noqa: E402  (MAYA_REFERENCE_TREE, else a "reference" directory beside this repository)


def router_cases(ref: Ref) -> None:
    inp = ref.router_test_inputs()[:, :16, :].copy()
    ids = np.empty((4, 16, 10), np.int32)
    w = np.empty((4, 16, 10), np.float32)
    for c in range(4):
        ids[c], w[c] = ref.router_reference(inp[c], 10)
    np.savez_compressed(HERE / "router_reference_cases.npz", logits=inp, ids=ids, weights=w,
                        names=np.array(["random normal", "all equal", "12-way tie", "dominant expert"]))


def glm5_router() -> None:
    import gguf
    rd = gguf.GGUFReader(str(REFERENCE / "data" / "glm5-synth.gguf"))
    tensors = {t.name: t for t in rd.tensors}
    fields = rd.fields
    scale = None
    for name, f in fields.items():
        if name.endswith("expert_weights_scale"):
            scale = float(f.parts[-1][0])
    assert scale is not None
    dumps = REFERENCE / "data" / "glm5-synth-dumps"
    logits, bias, topk, weights, layers = [], [], [], [], []
    for il in range(1, 6):
        l = np.fromfile(dumps / f"ffn_moe_logits-{il}.f32", dtype=np.float32)
        b = np.asarray(tensors[f"blk.{il}.exp_probs_b.bias"].data, dtype=np.float32).reshape(-1)
        n_expert = b.size
        t = np.fromfile(dumps / f"ffn_moe_topk-{il}.f32", dtype=np.int32)
        w = np.fromfile(dumps / f"ffn_moe_weights-{il}.f32", dtype=np.float32)
        n_tok = l.size // n_expert
        k = t.size // n_tok
        logits.append(l.reshape(n_tok, n_expert))
        bias.append(b)
        topk.append(t.reshape(n_tok, k))
        weights.append(w.reshape(n_tok, k))
        layers.append(il)
    np.savez_compressed(HERE / "glm5_synth_router.npz", logits=np.stack(logits), bias=np.stack(bias),
                        ids=np.stack(topk), weights=np.stack(weights), w_scale=np.float32(scale), layers=np.array(layers))


def glm5_moe_layer(layer: int = 1) -> None:
    """Layer `layer` of data/glm5-synth.gguf (F32 tensors: 12 experts of 128 x 64, top-3 sigmoid routing, one shared
    expert) read through the package's own loader, with llama.cpp's captured activations of that layer for 8 tokens:
    the normed hidden state that enters the MoE block, the routing, the routed output, the shared expert's output; and
    what follows the block: the residual stack before it (hc_attn_post), the hyper-connection gains (hc_post_ffn,
    hc_comb_ffn - stored src-major, [src][dst]) and the residual stack after it (l_out)."""
    import gguf
    from project_maya_b200 import gguf_loader
    path = REFERENCE / "data" / "glm5-synth.gguf"
    L = gguf_loader.read_moe_layer(path, layer)
    rd = gguf.GGUFReader(str(path))
    meta = {}
    for name, f in rd.fields.items():
        for key in ("expert_weights_scale", "expert_used_count", "swiglu_clamp_exp", "swiglu_clamp_shexp"):
            if name.endswith(key):
                meta[key] = float(np.asarray(f.parts[f.data[min(layer, len(f.data) - 1)]]).reshape(-1)[0])
    dumps = REFERENCE / "data" / "glm5-synth-dumps"
    d = lambda n, dt=np.float32: np.fromfile(dumps / f"{n}-{layer}.f32", dtype=dt)
    n_tok = d("ffn_norm").size // L.n_embd
    k = int(meta["expert_used_count"])
    np.savez_compressed(
        HERE / "glm5_synth_moe_layer1.npz", layer=np.int32(layer), gate=L.gate, up=L.up, down=L.down, router=L.router,
        router_bias=L.router_bias, sh_gate=L.sh_gate, sh_up=L.sh_up, sh_down=L.sh_down,
        x=d("ffn_norm").reshape(n_tok, L.n_embd), logits=d("ffn_moe_logits").reshape(n_tok, L.n_expert),
        ids=d("ffn_moe_topk", np.int32).reshape(n_tok, k), weights=d("ffn_moe_weights").reshape(n_tok, k),
        moe_out=d("ffn_moe_out").reshape(n_tok, L.n_embd), shexp=d("ffn_shexp").reshape(n_tok, L.n_embd),
        out=d("ffn_out").reshape(n_tok, L.n_embd), w_scale=np.float32(meta["expert_weights_scale"]),
        clamp=np.float32(meta["swiglu_clamp_exp"]), clamp_sh=np.float32(meta["swiglu_clamp_shexp"]),
        hc_R_old=d("hc_attn_post").reshape(n_tok, 4, L.n_embd), hc_post=d("hc_post_ffn").reshape(n_tok, 4),
        hc_comb_src_major=d("hc_comb_ffn").reshape(n_tok, 4, 4), hc_R_new=d("l_out").reshape(n_tok, 4, L.n_embd))


def c1_experts():
    """The C1 layer's synthetic experts: N(0, 0.02) weights quantized to Q4_K by the library's host quantizer."""
    from project_maya_b200 import api
    cfg = H.CONFIGS["C1"]
    Hd, FF, E = cfg["n_embd"], cfg["n_ff"], cfg["n_expert"]
    blobs = np.empty((E, H.blob_bytes(H.Q4_K, H.Q4_K, Hd, FF)), np.uint8)
    for e in range(E):
        rng = H.rng_for("C1", "expert", e)
        gu = api.quantize_weights_host(H.Q4_K, rng.normal(0.0, 0.02, size=(2 * FF, Hd)).astype(np.float32)).numpy()
        dn = api.quantize_weights_host(H.Q4_K, rng.normal(0.0, 0.02, size=(Hd, FF)).astype(np.float32)).numpy()
        blobs[e] = np.concatenate([gu.reshape(-1), dn.reshape(-1)])
    return blobs


def c1_reference(ref: Ref, orc: Oracle) -> None:
    cfg = H.CONFIGS["C1"]
    Hd, FF, E, k, T = cfg["n_embd"], cfg["n_ff"], cfg["n_expert"], cfg["k"], cfg["tokens"]
    blobs = c1_experts()
    logits = H.router_logits("C1", T, E, None)
    x = H.activations("C1", T, Hd, "f32")
    grb, drb = H.row_bytes(H.Q4_K, Hd), H.row_bytes(H.Q4_K, FF)
    ids, w = ref.router_reference(logits, k)
    out = np.zeros((T, Hd), np.float32)
    for t in range(T):
        a = orc.quantize_q8_K(x[t])
        acc = np.zeros(Hd, np.float32)
        parts = np.zeros((k, Hd), np.float32)
        for j in range(k):
            blob = blobs[ids[t, j]]
            h = ref.gu_rows(H.Q4_K, blob, grb, FF * grb, Hd, [a], 0, FF, avx512=True)[0]
            hq = orc.quantize_q8_K(h)
            parts[j] = ref.rows(H.Q4_K, blob[2 * FF * grb:], drb, FF, [hq], 0, Hd, avx512=True)[0]
        out[t] = orc.combine_native(parts, w[t])
        del acc
    _, _, out_q81 = orc.moe_layer(dict(cfg, limit=H.INF), logits, x, blobs)
    np.savez_compressed(HERE / "c1_reference_cpu.npz", ids=ids, weights=w, out_cpu_rows=out, out_oracle_q8_1=out_q81,
                        experts_sha256=np.array(hashlib.sha256(blobs.tobytes()).hexdigest()))


def main() -> None:
    ref, orc = Ref(), Oracle()
    router_cases(ref)
    glm5_router()
    glm5_moe_layer(1)
    c1_reference(ref, orc)
    for p in sorted(HERE.glob("*.npz")):
        print(p.name, p.stat().st_size)


if __name__ == "__main__":
    main()
