"""GGUF expert tensors -> the per-expert blobs the kernels read.

A Maya / llama.cpp GGUF stores a layer's routed experts as three stacked tensors, `blk.N.ffn_{gate,up,down}_exps.weight`
with GGUF dimensions [n_embd, n_ff, n_expert] (gate, up) and [n_ff, n_embd, n_expert] (down): expert e's gate matrix is
n_ff rows of n_embd values.  The kernels read one blob per expert, [gate rows | up rows | down rows], raw GGUF blocks
(NativeExpertLayout, include/strata/kernels/iq_kernels.hpp:63-72; mmq::gather_native, src/prefill/moe_mmq.cu:230-245,
builds the same thing on the device).  This module does that regrouping on the host with the `gguf` package:
quantized tensors keep their bytes untouched, F32 / F16 tensors (test models) are quantized with the library's own host
quantizer.  Nothing here is on a timed path.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import synthetic as S

GGML_NAMES = {"Q8_0": S.Q8_0, "Q4_K": S.Q4_K, "IQ3_S": S.IQ3_S, "IQ2_S": S.IQ2_S}


@dataclass
class MoeLayerTensors:
    """One layer's expert-FFN tensors, expert-major, rows in GGUF order."""
    n_embd: int
    n_ff: int
    n_expert: int
    gate: np.ndarray            # [E, n_ff, n_embd] f32, or raw uint8 [E, n_ff * row_bytes] when quantized
    up: np.ndarray
    down: np.ndarray            # [E, n_embd, n_ff] f32 or raw
    ggml_type: int | None       # None: float tensors
    router: np.ndarray | None = None        # ffn_gate_inp [E, n_embd]
    router_bias: np.ndarray | None = None   # exp_probs_b [E]
    sh_gate: np.ndarray | None = None       # shared expert [n_ff_sh, n_embd]
    sh_up: np.ndarray | None = None
    sh_down: np.ndarray | None = None       # [n_embd, n_ff_sh]


def _tensor(t):
    """(array, ggml type id or None).  Float tensors come back as f32 [.., rows, cols]; quantized ones as raw bytes with
    the GGUF shape's slowest dimension first."""
    shape = [int(x) for x in reversed(t.shape.tolist())]
    name = t.tensor_type.name
    if name in ("F32", "F16", "BF16"):
        return np.asarray(t.data, dtype=np.float32).reshape(shape), None
    if name not in GGML_NAMES:
        raise ValueError(f"{t.name}: ggml type {name} has no kernel here")
    return np.ascontiguousarray(t.data).view(np.uint8).reshape(shape[0], -1), GGML_NAMES[name]


def read_moe_layer(path, layer: int) -> MoeLayerTensors:
    import gguf
    rd = gguf.GGUFReader(str(path))
    ts = {t.name: t for t in rd.tensors}
    pre = f"blk.{layer}."
    gate, tg = _tensor(ts[pre + "ffn_gate_exps.weight"])
    up, tu = _tensor(ts[pre + "ffn_up_exps.weight"])
    down, td = _tensor(ts[pre + "ffn_down_exps.weight"])
    if not (tg == tu == td):
        raise ValueError("mixed expert tensor types in one layer are not handled by this loader")
    dims = [int(x) for x in ts[pre + "ffn_gate_exps.weight"].shape.tolist()]          # [n_embd, n_ff, E]
    out = MoeLayerTensors(dims[0], dims[1], dims[2], gate, up, down, tg)
    opt = {"router": "ffn_gate_inp.weight", "router_bias": "exp_probs_b.bias", "sh_gate": "ffn_gate_shexp.weight",
           "sh_up": "ffn_up_shexp.weight", "sh_down": "ffn_down_shexp.weight"}
    for field, name in opt.items():
        if pre + name in ts:
            a, ty = _tensor(ts[pre + name])
            if ty is not None:
                raise ValueError(f"{pre + name}: quantized side tensors are not handled by this loader")
            setattr(out, field, a.reshape(-1) if field == "router_bias" else a)
    return out


def quantize_rows(ggml_type: int, w: np.ndarray) -> np.ndarray:
    """f32 [rows, cols] -> raw blocks uint8 [rows * row_bytes], through the library's host quantizer."""
    from . import api
    return api.quantize_weights_host(ggml_type, np.ascontiguousarray(w, dtype=np.float32)).numpy().reshape(-1)


def expert_blobs(L: MoeLayerTensors, ggml_type: int | None = None) -> np.ndarray:
    """uint8 [E, blob_bytes]: expert e = its gate rows, its up rows, its down rows (mmq::gather_native's layout).
    Quantized tensors keep their bytes; float tensors are quantized to `ggml_type`."""
    t = L.ggml_type if L.ggml_type is not None else ggml_type
    if t is None:
        raise ValueError("float tensors need a target ggml type")
    blob = S.blob_bytes(t, t, L.n_embd, L.n_ff)
    out = np.empty((L.n_expert, blob), np.uint8)
    gu = L.n_ff * S.row_bytes(t, L.n_embd)
    for e in range(L.n_expert):
        if L.ggml_type is not None:
            parts = [L.gate[e].reshape(-1), L.up[e].reshape(-1), L.down[e].reshape(-1)]
        else:
            parts = [quantize_rows(t, L.gate[e]), quantize_rows(t, L.up[e]), quantize_rows(t, L.down[e])]
        assert parts[0].size == gu and parts[2].size == L.n_embd * S.row_bytes(t, L.n_ff)
        out[e] = np.concatenate(parts)
    return out


def shared_blob(L: MoeLayerTensors, ggml_type: int) -> np.ndarray | None:
    if L.sh_gate is None:
        return None
    return np.concatenate([quantize_rows(ggml_type, L.sh_gate), quantize_rows(ggml_type, L.sh_up), quantize_rows(ggml_type, L.sh_down)])
