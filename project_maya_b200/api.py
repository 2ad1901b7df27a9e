"""Host-side mirror of the reference's per-layer expert-FFN entry points, over the C ABI (include/maya_moe.h).

Names, argument meaning and error behaviour follow the reference's C++ free functions (namespace strata::kernels,
strata::kernels::glmf): device buffers in, device buffers out, an explicit stream, nothing allocated by the callee.
torch is used only for device memory and streams: every function takes torch CUDA tensors (or raw integer device
addresses) and launches this library's own CUDA kernels.  A negative status raises MayaError, as the reference's
`native_*` family throws std::invalid_argument / std::runtime_error (native_mmvq.cu:1080-1099).
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import ExpertLayout, HcPostArgs, MmqProduct, MoeLayerDesc, MoePlan, MoeWin

Q8_0, Q4_K, IQ3_S, IQ2_S = 8, 12, 21, 22
Q5_K, Q6_K, IQ2_XXS, IQ3_XXS, IQ1_S, IQ4_XS = 13, 14, 16, 18, 19, 23      # staged decode paths only (see maya_ggml_type in the header)
_BLOCK = {Q8_0: 32, Q4_K: 256, IQ3_S: 256, IQ2_S: 256, Q5_K: 256, Q6_K: 256, IQ2_XXS: 256, IQ3_XXS: 256, IQ4_XS: 256, IQ1_S: 256}   # values per GGUF block
TYPE_NAMES = {Q8_0: "Q8_0", Q4_K: "Q4_K", IQ3_S: "IQ3_S", IQ2_S: "IQ2_S", Q5_K: "Q5_K", Q6_K: "Q6_K", IQ2_XXS: "IQ2_XXS",
              IQ3_XXS: "IQ3_XXS", IQ4_XS: "IQ4_XS", IQ1_S: "IQ1_S"}
STATUS = {0: "ok", -1: "bad argument", -2: "unsupported ggml type", -3: "CUDA launch failed", -4: "beyond a limit",
          -5: "no sm_100 device"}
INF = float("inf")


class MayaError(RuntimeError):
    def __init__(self, what: str, status: int):
        super().__init__(f"{what}: {STATUS.get(status, status)} (status {status})")
        self.status = status


def _check(what: str, status: int) -> None:
    if status != 0:
        raise MayaError(what, status)


def _ptr(t) -> int | None:
    if t is None:
        return None
    if isinstance(t, int):
        return t
    assert t.is_cuda and t.is_contiguous(), "device-contiguous tensor expected"
    return t.data_ptr()


def _stream(stream=None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream if hasattr(s, "cuda_stream") else int(s)


# ---------------------------------------------------------------- formats (host only: usable without a GPU)
def row_bytes(ggml_type: int, n: int) -> int:
    return int(_lib.load().maya_row_bytes(ggml_type, n))


def q8_1_bytes(n_in: int, ncols: int = 1) -> int:
    return int(_lib.load().maya_q8_1_bytes(n_in, ncols))


def native_expert_layout(gu_type: int, d_type: int, n_embd: int, n_ff: int, up_type: int | None = None) -> ExpertLayout:
    L = ExpertLayout()
    _check("native_expert_layout", _lib.load().maya_expert_layout_make(gu_type, gu_type if up_type is None else up_type,
                                                                       d_type, n_embd, n_ff, C.byref(L)))
    return L


def quantize_weights_host(ggml_type: int, w) -> "torch.Tensor":
    """Host f32 rows [n_rows, n_cols] -> uint8 [n_rows, row_bytes] of GGUF blocks (this library's own quantizers)."""
    w = torch.as_tensor(w, dtype=torch.float32).contiguous().cpu()
    n_rows, n_cols = w.shape
    out = torch.empty((n_rows, row_bytes(ggml_type, n_cols)), dtype=torch.uint8)
    _check("quantize_weights_host",
           _lib.load().maya_quantize_weights_host(ggml_type, w.data_ptr(), n_rows, n_cols, out.data_ptr()))
    return out


def synth_weights(ggml_type: int, seed: int, sigma: float, n_rows: int, n_cols: int, out=None, stream=None):
    """Device: n_rows x n_cols N(0, sigma) weights quantized to ggml_type, written as blocks into `out` (uint8)."""
    nbytes = n_rows * row_bytes(ggml_type, n_cols)
    if out is None:
        out = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    _check("synth_weights", _lib.load().maya_synth_weights(ggml_type, seed, sigma, n_rows, n_cols, _ptr(out), _stream(stream)))
    return out


# ---------------------------------------------------------------- router
def router_top10(logits, k: int, ids=None, weights=None, stream=None):
    """router_top10 (router_top10.hpp:17).  logits [n_tokens, n_expert] f32 -> ids i32, weights f32 [n_tokens, k]."""
    T, E = logits.shape
    ids = ids if ids is not None else torch.empty((T, k), dtype=torch.int32, device=logits.device)
    weights = weights if weights is not None else torch.empty((T, k), dtype=torch.float32, device=logits.device)
    _check("router_top10", _lib.load().maya_router_top10(_ptr(logits), T, E, k, _ptr(ids), _ptr(weights), _stream(stream)))
    return ids, weights


def router_sigmoid(logits, bias, k: int, w_scale: float = 1.0, norm_w: bool = True, stream=None):
    T, E = logits.shape
    ids = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    weights = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    _check("router_sigmoid", _lib.load().maya_router_sigmoid(_ptr(logits), _ptr(bias), T, E, k, w_scale, int(norm_w),
                                                             _ptr(ids), _ptr(weights), _stream(stream)))
    return ids, weights


# ---------------------------------------------------------------- activations
def native_quantize_q8_1(x, out=None, stream=None):
    """native_quantize_q8_1 (native_mmvq.hpp:38).  x [ncols, n_in] f32 or bf16 -> uint8 [ncols, n_in/32*36]."""
    x2 = x.reshape(-1, x.shape[-1])
    ncols, n_in = x2.shape
    out = out if out is not None else torch.empty((ncols, n_in // 32 * 36), dtype=torch.uint8, device=x.device)
    lib = _lib.load()
    if x.dtype == torch.bfloat16:
        _check("quantize_q8_1", lib.maya_quantize_q8_1_bf16(_ptr(x2), _ptr(out), n_in, ncols, _stream(stream)))
    else:
        assert x.dtype == torch.float32
        _check("quantize_q8_1", lib.maya_quantize_q8_1(_ptr(x2), _ptr(out), n_in, ncols, _stream(stream)))
    return out


def swiglu_q8_1(gate, up, limit: float = INF, out=None, stream=None):
    n = gate.numel()
    out = out if out is not None else torch.empty(n // 32 * 36, dtype=torch.uint8, device=gate.device)
    _check("swiglu_q8_1", _lib.load().maya_swiglu_q8_1(_ptr(gate), _ptr(up), limit, n, _ptr(out), _stream(stream)))
    return out


# ---------------------------------------------------------------- GEMV
def native_mmvq(ggml_type: int, weights, x_q8_1, n_in: int, n_out: int, ncols: int = 1, y=None, stream=None):
    """native_mmvq (native_mmvq.hpp:109) / iq_mmvq (iq_kernels.hpp:24): y [ncols, n_out] f32."""
    y = y if y is not None else torch.empty((ncols, n_out), dtype=torch.float32, device="cuda")
    _check("native_mmvq", _lib.load().maya_mmvq(ggml_type, _ptr(weights), _ptr(x_q8_1), _ptr(y), n_in, n_out, ncols,
                                               _stream(stream)))
    return y


# ---------------------------------------------------------------- decode experts
def make_plan(plan_ptr, plan_w, cpu_part=None, cpu_flag=None, skip=None) -> MoePlan:
    return MoePlan(_ptr(plan_ptr), _ptr(plan_w), _ptr(cpu_part), _ptr(cpu_flag), _ptr(skip))


def moe_gate_up(gu_type: int, plan: MoePlan, k: int, n_embd: int, n_ff: int, limit: float, xq, hq, sh_down=None,
                sh_type: int = 0, sh_hq=None, n_ff_sh: int = 0, sh_out=None, stream=None) -> None:
    """glmf::moe_gate_up (glm_fast.hpp:496)."""
    _check("moe_gate_up", _lib.load().maya_moe_gate_up(gu_type, C.byref(plan), k, n_embd, n_ff, limit, _ptr(xq), _ptr(hq),
                                                      _ptr(sh_down), sh_type, _ptr(sh_hq), n_ff_sh, _ptr(sh_out),
                                                      _stream(stream)))


def moe_down(d_type: int, plan: MoePlan, k: int, n_embd: int, n_ff: int, down_off: int, hq, sh_out, out, stream=None) -> None:
    """glmf::moe_down (glm_fast.hpp:499)."""
    _check("moe_down", _lib.load().maya_moe_down(d_type, C.byref(plan), k, n_embd, n_ff, down_off, _ptr(hq), _ptr(sh_out),
                                                _ptr(out), _stream(stream)))


def moe_win_experts(gu_type: int, d_type: int, win: MoeWin, stream=None) -> None:
    """glmf::moe_win_experts (glm_fast.hpp:465)."""
    _check("moe_win_experts", _lib.load().maya_moe_win_experts(gu_type, d_type, C.byref(win), _stream(stream)))


def native_expert_scratch_bytes(cap_entries: int, n_ff: int) -> int:
    return int(_lib.load().maya_expert_scratch_bytes(cap_entries, n_ff))


def native_expert_grouped(L: ExpertLayout, grp_ptr, grp_start, n_groups, ent_dst, ent_tok, cap_groups: int,
                          cap_entries: int, x_q8_1, scratch, out, swiglu_limit: float = INF, stream=None) -> None:
    """native_expert_grouped (iq_kernels.hpp:89)."""
    _check("native_expert_grouped",
           _lib.load().maya_expert_grouped(C.byref(L), _ptr(grp_ptr), _ptr(grp_start), _ptr(n_groups), _ptr(ent_dst),
                                           _ptr(ent_tok), cap_groups, cap_entries, _ptr(x_q8_1), _ptr(scratch), _ptr(out),
                                           _stream(stream), swiglu_limit))


def native_expert_grouped_static(L: ExpertLayout, grp_ptr, grp_start, n_groups, ent_dst, ent_tok, cap_groups: int,
                                 cap_entries: int, x_q8_1, out, swiglu_limit: float = INF, stream=None) -> None:
    """native_expert_grouped without a scratch argument: for callers that cannot allocate or pass device scratch.
    The q8_1 image of h lives in a 2 MiB array built into the library (see maya_expert_grouped_static in the header:
    size limit, first call outside stream capture, calls on one GPU must not overlap)."""
    _check("native_expert_grouped_static",
           _lib.load().maya_expert_grouped_static(C.byref(L), _ptr(grp_ptr), _ptr(grp_start), _ptr(n_groups), _ptr(ent_dst),
                                                  _ptr(ent_tok), cap_groups, cap_entries, _ptr(x_q8_1), _ptr(out),
                                                  _stream(stream), swiglu_limit))


def moe_combine(parts, weights, shared, n_embd: int, k: int, n_tok: int = 1, y=None, stream=None):
    """native_moe_combine[_multi] (native_moe.hpp:16-20) / moe_combine (shared_expert.hpp:98)."""
    y = y if y is not None else torch.empty((n_tok, n_embd), dtype=torch.float32, device="cuda")
    _check("moe_combine", _lib.load().maya_moe_combine(_ptr(parts), _ptr(weights), _ptr(shared), _ptr(y), n_embd, k, n_tok,
                                                      _stream(stream)))
    return y


# ---------------------------------------------------------------- prefill grouping
def expert_group(ids, n_expert: int, stream=None):
    """glmb::expert_count + the device-side bounds scan + glmb::expert_scatter.  ids [T, k] i32 ->
    (counts [E], bounds [E + 1], pos [T * k], row_tok [T * k]) with no host round trip."""
    T, k = ids.shape
    n = T * k
    dev = ids.device
    counts = torch.empty(n_expert, dtype=torch.int32, device=dev)
    rank = torch.empty(n, dtype=torch.int32, device=dev)
    bounds = torch.empty(n_expert + 1, dtype=torch.int32, device=dev)
    pos = torch.empty(n, dtype=torch.int32, device=dev)
    row_tok = torch.empty(n, dtype=torch.int32, device=dev)
    lib, s = _lib.load(), _stream(stream)
    _check("expert_count", lib.maya_expert_count(_ptr(ids), n, n_expert, _ptr(counts), _ptr(rank), s))
    _check("expert_bounds", lib.maya_expert_bounds(_ptr(counts), n_expert, _ptr(bounds), s))
    _check("expert_scatter", lib.maya_expert_scatter(_ptr(ids), _ptr(rank), _ptr(bounds), n, k, _ptr(row_tok), _ptr(pos), s))
    return counts, bounds, pos, row_tok


def swiglu_rows(gu, n_ff: int, limit: float = INF, stream=None):
    rows = gu.shape[0]
    h = torch.empty((rows, n_ff), dtype=torch.float32, device=gu.device)
    _check("swiglu_rows", _lib.load().maya_swiglu_rows(_ptr(gu), _ptr(h), rows, n_ff, limit, 0, _stream(stream)))
    return h


def moe_combine_rows(out, pos, w, sh, T: int, k: int, n_embd: int, stream=None):
    ffn = torch.empty((T, n_embd), dtype=torch.float32, device=out.device)
    _check("moe_combine_rows", _lib.load().maya_moe_combine_rows(_ptr(out), _ptr(pos), _ptr(w), _ptr(sh), T, k, n_embd,
                                                                _ptr(ffn), _stream(stream)))
    return ffn


# ---------------------------------------------------------------- the producer in front of the layer
def rms_router(h, add, norm_w, eps: float, router_w, h_out=None, stream=None):
    """glmf::rms_q8 (glm_fast.hpp:534) + the router GEMV (glm_fast_path.cu:6925) in one launch: returns (x f32 [n_embd],
    logits f32 [n_expert]); h_out receives h + add when given.  router_w: [n_expert, n_embd] f32 or bf16."""
    n_embd, n_expert = h.numel(), router_w.shape[0]
    assert router_w.dtype in (torch.float32, torch.bfloat16) and router_w.shape[1] == n_embd
    x = torch.empty(n_embd, dtype=torch.float32, device=h.device)
    logits = torch.empty(n_expert, dtype=torch.float32, device=h.device)
    _check("rms_router", _lib.load().maya_rms_router(_ptr(h), _ptr(add), _ptr(norm_w), eps, n_embd, _ptr(router_w),
                                                    int(router_w.dtype == torch.bfloat16), n_expert, _ptr(h_out), _ptr(x),
                                                    _ptr(logits), _stream(stream)))
    return x, logits


# ---------------------------------------------------------------- prompt-path grouped GEMM (tensor cores)
def hc_post(block_out, R_old, post, comb, R_new=None, stream=None):
    """glmf::hc_post: R_new [4, n_embd] = block_out * post[d] + comb[d, :] . R_old[:, e] (comb dst-major)."""
    n = block_out.numel()
    R_new = R_new if R_new is not None else torch.empty((4, n), dtype=torch.float32, device=block_out.device)
    _check("hc_post", _lib.load().maya_hc_post(_ptr(block_out), _ptr(R_old), _ptr(post), _ptr(comb), n, _ptr(R_new), _stream(stream)))
    return R_new


def mmq_supported(ggml_type: int) -> bool:
    """mmq::supported (include/strata/prefill/moe_mmq.hpp:16)."""
    return bool(_lib.load().maya_mmq_supported(ggml_type))


def mmq_q8_bytes(rows: int, cols: int) -> int:
    """mmq::q8_bytes (moe_mmq.hpp:20)."""
    return int(_lib.load().maya_mmq_q8_bytes(rows, cols))


def mmq_quantize(x, ids, ggml_type: int, rows: int | None = None, xq=None, stream=None):
    """mmq::quantize (moe_mmq.hpp:34): row i of the result = q8_1 of x[ids[i]] (x[i] when ids is None)."""
    cols, ld = x.shape[1], x.stride(0)
    rows = rows if rows is not None else (ids.numel() if ids is not None else x.shape[0])
    xq = xq if xq is not None else torch.empty(max(mmq_q8_bytes(rows, cols), 16), dtype=torch.uint8, device=x.device)
    assert x.dtype in (torch.float32, torch.bfloat16)
    fn = _lib.load().maya_mmq_quantize_bf16 if x.dtype == torch.bfloat16 else _lib.load().maya_mmq_quantize
    _check("mmq_quantize", fn(_ptr(x), _ptr(ids), _ptr(xq), ggml_type, cols, ld, rows, _stream(stream)))
    return xq


def mmq_quantize_routed(x, pos, k: int, ggml_type: int, xq=None, stream=None):
    """No counterpart in the reference: every row of x rounded once, its q8_1 image stored to the k rows pos[t * k + j]
    (pos from expert_groups) - the bytes mmq_quantize(x, row_tok, ...) writes."""
    assert x.dtype in (torch.float32, torch.bfloat16)
    T, cols, ld = x.shape[0], x.shape[1], x.stride(0)
    xq = xq if xq is not None else torch.empty(max(mmq_q8_bytes(T * k, cols), 16), dtype=torch.uint8, device=x.device)
    fn = _lib.load().maya_mmq_quantize_routed_bf16 if x.dtype == torch.bfloat16 else _lib.load().maya_mmq_quantize_routed
    _check("mmq_quantize_routed", fn(_ptr(x), _ptr(pos), k, _ptr(xq), ggml_type, cols, ld, T, _stream(stream)))
    return xq


def mmq_product(w, ggml_type: int, w_rows: int, w_cols: int, expert_bytes: int, n: int, xq, bounds, ids,
                total_rows: int, dst, ld_dst: int, max_rows: int = 0, expert_map=None, error=None, xq_out=None) -> MmqProduct:
    """mmq::Product (moe_mmq.hpp:41-53).  The tensors must outlive the launch: the struct holds raw addresses."""
    return MmqProduct(_ptr(w), ggml_type, w_rows, w_cols, expert_bytes, n, _ptr(xq), _ptr(bounds), _ptr(ids), total_rows,
                      max_rows, _ptr(dst), ld_dst, _ptr(expert_map), _ptr(error), _ptr(xq_out))


def mmq_run(p: MmqProduct, stream=None) -> None:
    """mmq::Context::run (moe_mmq.hpp:74)."""
    _check("mmq_run", _lib.load().maya_mmq_run(C.byref(p), _stream(stream)))


def mmq_run_glu(p: MmqProduct, limit: float = INF, stream=None) -> None:
    """mmq::Context::run_glu (moe_mmq.hpp:81)."""
    _check("mmq_run_glu", _lib.load().maya_mmq_run_glu(C.byref(p), limit, _stream(stream)))


# ---------------------------------------------------------------- whole layer
@dataclass
class MoeLayerConfig:
    n_embd: int
    n_ff: int
    n_expert: int
    k: int
    gu_type: int
    d_type: int
    n_ff_sh: int = 0
    sh_gu_type: int = Q8_0
    sh_d_type: int = Q8_0
    limit: float = INF

    @property
    def blob_bytes(self) -> int:
        return 2 * self.n_ff * row_bytes(self.gu_type, self.n_embd) + self.n_embd * row_bytes(self.d_type, self.n_ff)

    @property
    def shared_bytes(self) -> int:
        if not self.n_ff_sh:
            return 0
        return 2 * self.n_ff_sh * row_bytes(self.sh_gu_type, self.n_embd) + self.n_embd * row_bytes(self.sh_d_type, self.n_ff_sh)


def width_slice(cfg: MoeLayerConfig, experts, shared, lo: int, hi: int, sh_lo: int | None = None, sh_hi: int | None = None):
    """(cfg', experts', shared'): FFN rows lo..hi-1 of every routed expert (sh_lo..sh_hi-1 of the shared one) as blobs
    of their own - each expert's gate and up rows of that range and the same COLUMNS of its down rows.

    A width slice of an expert is an expert of FFN width hi - lo, and the slices' outputs add up to the whole expert's:
    out = sum over slices of down[:, slice] . SwiGLU(gate[slice] x, up[slice] x).  This is how the reference splits
    experts under tensor parallelism (its experts are width-sliced, never partitioned by id): every rank then carries
    1 / N of EVERY token's work whatever the routing, where a partition by expert id gives a rank whatever share of
    the token's experts it happens to hold.  The partial outputs are summed by the same all-reduce.  lo, hi must be
    multiples of the down type's block size (256 for the k- and i-quants) so that the column slice is whole blocks; the
    result is this rank's resident copy (nothing refers to the full blobs afterwards)."""
    H = cfg.n_embd

    def cut(blob, gu_t, d_t, n_ff, a, b):          # blob: [..., blob_bytes]
        rb, drb = row_bytes(gu_t, H), row_bytes(d_t, n_ff)
        gu = n_ff * rb
        lead = blob.shape[:-1]
        gate = blob[..., :gu].reshape(*lead, n_ff, rb)[..., a:b, :].reshape(*lead, -1)
        up = blob[..., gu:2 * gu].reshape(*lead, n_ff, rb)[..., a:b, :].reshape(*lead, -1)
        down = blob[..., 2 * gu:].reshape(*lead, H, drb)[..., row_bytes(d_t, a):row_bytes(d_t, b)].reshape(*lead, -1)
        return torch.cat([gate, up, down], dim=-1).contiguous()

    def whole_blocks(t, *vals):
        for v in vals:
            if v % _BLOCK[t] != 0:
                raise ValueError(f"width slice bound {v} is not a multiple of the block size {_BLOCK[t]}")

    whole_blocks(cfg.d_type, lo, hi)
    ex = cut(experts, cfg.gu_type, cfg.d_type, cfg.n_ff, lo, hi)
    sh, n_ff_sh = None, 0
    if shared is not None and cfg.n_ff_sh:
        sh_lo = lo if sh_lo is None else sh_lo
        sh_hi = hi if sh_hi is None else sh_hi
        whole_blocks(cfg.sh_d_type, sh_lo, sh_hi)
        sh = cut(shared, cfg.sh_gu_type, cfg.sh_d_type, cfg.n_ff_sh, sh_lo, sh_hi)
        n_ff_sh = sh_hi - sh_lo
    out = MoeLayerConfig(cfg.n_embd, hi - lo, cfg.n_expert, cfg.k, cfg.gu_type, cfg.d_type, n_ff_sh, cfg.sh_gu_type,
                         cfg.sh_d_type, cfg.limit)
    return out, ex, sh


class MoeLayer:
    """One resident MoE layer: `experts` uint8 [n_expert, blob_bytes] on the device, optional `shared` blob.

    forward(logits, x) runs route -> experts -> combine for up to 16 tokens and returns (ids, weights, out).
    expert_range = (lo, hi) restricts this rank to experts lo..hi-1 (expert-parallel partition); the others' terms are
    left out of `out` (another rank adds them).  shared_range = (lo, hi) gives this rank a slice of the shared expert's
    FFN width instead of all of it (single-token calls only).  sigmoid = (bias [n_expert] or None, w_scale, norm_w):
    sigmoid routing with a selection bias instead of softmax.  cpu_part [T, n_embd] f32 / cpu_flag [T] i32: a host lane's
    contribution, added to token t's output when cpu_flag[t] != 0 (the tier hooks of the reference's MoeDev)."""

    def __init__(self, cfg: MoeLayerConfig, experts, shared=None, expert_range=None, shared_here=True, max_tokens: int = 16,
                 staged: bool = False, shared_range=None, sigmoid=None, cpu_part=None, cpu_flag=None):
        self.cfg = cfg
        self.experts = experts
        self.shared = shared
        lo, hi = expert_range if expert_range is not None else (0, cfg.n_expert)
        self.desc = MoeLayerDesc(cfg.n_embd, cfg.n_ff, cfg.n_expert, cfg.k, cfg.gu_type, cfg.d_type, _ptr(experts),
                                 cfg.blob_bytes, cfg.n_ff_sh if shared is not None else 0, cfg.sh_gu_type,
                                 cfg.sh_d_type, _ptr(shared), cfg.limit, lo, hi, int(bool(shared_here)), int(bool(staged)),
                                 *(shared_range if shared_range is not None else (0, 0)),
                                 *((1, _ptr(sigmoid[0]), float(sigmoid[1]), int(bool(sigmoid[2]))) if sigmoid is not None else (0, None, 1.0, 0)),
                                 _ptr(cpu_part), _ptr(cpu_flag))
        self._keep = (sigmoid, cpu_part, cpu_flag)
        self.max_tokens = max_tokens
        nbytes = int(_lib.load().maya_moe_layer_scratch_bytes(C.byref(self.desc), max_tokens))
        if nbytes == 0:
            raise MayaError("moe_layer_scratch_bytes", -1)
        self.scratch = torch.zeros(nbytes, dtype=torch.uint8, device=experts.device)   # zeroed: holds a barrier counter

    def forward(self, logits, x, ids=None, weights=None, out=None, stream=None, peer=None, hc=None):
        """hc = (R_old [T, 4, n_embd], post [T, 4], comb [T, 4, 4], R_new [T, 4, n_embd]): also write the block's output
        into the residual stack (glmf::hc_post) - in the layer kernel's epilogue for one token."""
        T = logits.shape[0]
        dev = logits.device
        ids = ids if ids is not None else torch.empty((T, self.cfg.k), dtype=torch.int32, device=dev)
        weights = weights if weights is not None else torch.empty((T, self.cfg.k), dtype=torch.float32, device=dev)
        out = out if out is not None else torch.empty((T, self.cfg.n_embd), dtype=torch.float32, device=dev)
        assert x.dtype in (torch.float32, torch.bfloat16)
        if hc is not None:
            args = HcPostArgs(*[_ptr(t) for t in hc])
            seq = 0
            if peer is not None:
                seq = 0 if peer.device_seq else peer.next_seq()
            _check("moe_layer_decode_hc",
                   _lib.load().maya_moe_layer_decode_hc(C.byref(self.desc), _ptr(logits), _ptr(x), int(x.dtype == torch.bfloat16),
                                                        T, _ptr(ids), _ptr(weights), _ptr(out), _ptr(self.scratch),
                                                        self.scratch.numel(), C.byref(peer.desc) if peer is not None else None,
                                                        peer.mi if peer is not None else 0, seq, C.byref(args), _stream(stream)))
            return ids, weights, out
        if peer is not None:     # expert-parallel: `out` becomes the rank-ordered sum over the group (peer.PeerRank)
            _check("moe_layer_decode_ar",
                   _lib.load().maya_moe_layer_decode_ar(C.byref(self.desc), _ptr(logits), _ptr(x), int(x.dtype == torch.bfloat16),
                                                        T, _ptr(ids), _ptr(weights), _ptr(out), _ptr(self.scratch),
                                                        self.scratch.numel(), C.byref(peer.desc), peer.mi,
                                                        0 if peer.device_seq else peer.next_seq(),
                                                        _stream(stream)))
            return ids, weights, out
        _check("moe_layer_decode",
               _lib.load().maya_moe_layer_decode(C.byref(self.desc), _ptr(logits), _ptr(x), int(x.dtype == torch.bfloat16), T,
                                                 _ptr(ids), _ptr(weights), _ptr(out), _ptr(self.scratch),
                                                 self.scratch.numel(), _stream(stream)))
        return ids, weights, out

    def phase_ns(self, stream=None):
        """Block 0's phase stamps of the last fused single-token launch, as offsets in ns from its start."""
        buf = (C.c_ulonglong * 6)()
        _check("moe_layer_phase_ns", _lib.load().maya_moe_layer_phase_ns(C.byref(self.desc), _ptr(self.scratch), _stream(stream), buf))
        return [int(buf[i]) - int(buf[0]) for i in range(6)]

    def error(self, stream=None) -> int:
        """The scratch's sticky device-side error word (0 = none); synchronises the stream."""
        return int(_lib.load().maya_moe_layer_error(C.byref(self.desc), self.max_tokens, _ptr(self.scratch), _stream(stream)))


class MoePrefill:
    """The prompt path of one resident layer for a chunk of up to `max_tokens` tokens, with no host round trip:
    route -> group rows by expert -> q8_1 of the gathered rows -> gate/up grouped GEMM with SwiGLU in its write-back ->
    q8_1 of h -> down grouped GEMM -> weighted combine (+ the shared expert as one more product over all rows).

    Follows the reference's prefill_run expert sequence (src/core/glm_prefill.cu:3230-3420: expert_count, bases,
    expert_scatter, mmq::quantize, Context::run_glu, mmq::quantize, Context::run, moe_combine), except that the bases
    are scanned on the device.  Every buffer is allocated once, here.

    expert_range = (lo, hi) makes this an expert-parallel rank: only experts lo..hi-1 are multiplied and combined, and
    the returned ffn is this rank's partial sum (the ranks' results add up; pass `shared` on one rank only).

    `experts` is uint8 [n_expert, blob_bytes] of one type (cfg.gu_type == cfg.d_type is not required), or None with
    `pools` = [(ggml_type, blobs uint8 [n_i, blob_bytes of that type], expert ids of the n_i blobs), ...] for a layer whose
    experts are stored in different types: one product per pool, each matrix finding its rows through the pool's
    expert map (the reference's staged groups, moe_mmq.hpp:41-53 with bounds per group)."""

    def __init__(self, cfg: MoeLayerConfig, experts, shared=None, max_tokens: int = 4096, pools=None, expert_range=None):
        H, FF = cfg.n_embd, cfg.n_ff
        self.expert_range = expert_range         # (lo, hi): an expert-parallel rank's experts; ffn is then its partial sum
        if pools is None:
            if expert_range is None:
                pools = [((cfg.gu_type, cfg.d_type), experts, None)]
            else:                                # this rank's blobs only (a view), found through an expert map
                lo, hi = expert_range
                pools = [((cfg.gu_type, cfg.d_type), experts[lo:hi], list(range(lo, hi)))] if hi > lo else []
        elif expert_range is not None:
            lo, hi = expert_range
            kept = []
            for types, blobs, expert_ids in pools:
                sel = [i for i, e in enumerate(expert_ids) if lo <= e < hi]
                if sel:
                    kept.append((types, blobs[sel[0]:sel[-1] + 1] if sel == list(range(sel[0], sel[-1] + 1)) else blobs[sel].contiguous(),
                                 [expert_ids[i] for i in sel]))
            pools = kept
        self.pools = []
        for types, blobs, expert_ids in pools:
            gt, dt = types if isinstance(types, tuple) else (types, types)
            if not (mmq_supported(gt) and mmq_supported(dt)):
                raise MayaError("MoePrefill: type without a grouped GEMM", -2)
            stride = 2 * FF * row_bytes(gt, H) + H * row_bytes(dt, FF)
            assert blobs.shape[1] == stride, "a pool's blobs must be [gate | up | down] of its own type"
            emap = None if expert_ids is None else torch.as_tensor(expert_ids, dtype=torch.int32).to(blobs.device)
            self.pools.append((gt, dt, blobs, stride, 2 * FF * row_bytes(gt, H), blobs.shape[0], emap))
        if shared is not None and not (mmq_supported(cfg.sh_gu_type) and mmq_supported(cfg.sh_d_type)):
            raise MayaError("MoePrefill: shared expert's type without a grouped GEMM", -2)
        self.cfg, self.shared, self.max_tokens = cfg, shared, max_tokens
        dev, T, k, E = (self.pools[0][2].device if self.pools else experts.device), max_tokens, cfg.k, cfg.n_expert
        i32 = dict(dtype=torch.int32, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        u8 = dict(dtype=torch.uint8, device=dev)
        n = T * k
        self.ids, self.weights = torch.empty((T, k), **i32), torch.empty((T, k), **f32)
        self.counts, self.rank, self.bounds = torch.empty(E, **i32), torch.empty(n, **i32), torch.empty(E + 1, **i32)
        self.pos, self.row_tok = torch.empty(n, **i32), torch.empty(n, **i32)
        self.xq = torch.empty(mmq_q8_bytes(n, H), **u8)
        self.hq = torch.empty(mmq_q8_bytes(n, FF), **u8)
        self.out, self.ffn = torch.empty((n, H), **f32), torch.empty((T, H), **f32)
        self.err = torch.zeros(1, dtype=torch.int32, device=dev)
        if shared is not None:
            FS = cfg.n_ff_sh
            self.sh_bounds, self._sh_T = torch.zeros(2, **i32), -1
            self.sh_xq = torch.empty(mmq_q8_bytes(T, H), **u8)
            self.sh_hq = torch.empty(mmq_q8_bytes(T, FS), **u8)
            self.sh_out = torch.empty((T, H), **f32)
            self.sh_down_off = 2 * FS * row_bytes(cfg.sh_gu_type, H)

    def forward(self, logits, x, stream=None, peer=None):
        """peer (a peer.PeerRank whose stride holds T * n_embd floats), on an expert-parallel rank: the returned ffn is the
        rank-ordered sum over the group, exchanged inside the combine launch."""
        cfg, lib, s = self.cfg, _lib.load(), _stream(stream)
        T, k, H, FF, E = logits.shape[0], cfg.k, cfg.n_embd, cfg.n_ff, cfg.n_expert
        assert T <= self.max_tokens and x.shape == (T, H) and x.dtype in (torch.float32, torch.bfloat16)
        n = T * k
        quant = lib.maya_mmq_quantize_bf16 if x.dtype == torch.bfloat16 else lib.maya_mmq_quantize
        quant_routed = lib.maya_mmq_quantize_routed_bf16 if x.dtype == torch.bfloat16 else lib.maya_mmq_quantize_routed
        ids, w = self.ids[:T], self.weights[:T]
        _check("router_top10", lib.maya_router_top10(_ptr(logits), T, E, k, _ptr(ids), _ptr(w), s))
        _check("expert_count", lib.maya_expert_count(_ptr(ids), n, E, _ptr(self.counts), _ptr(self.rank), s))
        _check("expert_bounds", lib.maya_expert_bounds(_ptr(self.counts), E, _ptr(self.bounds), s))
        _check("expert_scatter", lib.maya_expert_scatter(_ptr(ids), _ptr(self.rank), _ptr(self.bounds), n, k,
                                                         _ptr(self.row_tok), _ptr(self.pos), s))
        qtype = self.pools[0][0] if self.pools else cfg.gu_type
        # each token rounded once, its image stored to its k sorted rows (the bytes quant(x, row_tok, ...) would write)
        _check("mmq_quantize_routed", quant_routed(_ptr(x), _ptr(self.pos), k, _ptr(self.xq), qtype, H, x.stride(0), T, s))
        for gt, dt, blobs, stride, down_off, n_p, emap in self.pools:
            gu = mmq_product(blobs, gt, 2 * FF, H, stride, n_p, self.xq, self.bounds, None, n, None, FF, expert_map=emap,
                             error=self.err, xq_out=self.hq)        # h leaves the product already quantized
            _check("mmq_run_glu", lib.maya_mmq_run_glu(C.byref(gu), cfg.limit, s))
        for gt, dt, blobs, stride, down_off, n_p, emap in self.pools:
            dn = mmq_product(blobs.data_ptr() + down_off, dt, H, FF, stride, n_p, self.hq, self.bounds, None, n, self.out, H,
                             expert_map=emap, error=self.err)
            _check("mmq_run", lib.maya_mmq_run(C.byref(dn), s))
        sh_out = None
        if self.shared is not None:
            FS = cfg.n_ff_sh
            if self._sh_T != T:      # the shared expert is one more "expert" that owns every row
                self.sh_bounds[1], self._sh_T = T, T
            _check("mmq_quantize", quant(_ptr(x), None, _ptr(self.sh_xq), cfg.sh_gu_type, H, x.stride(0), T, s))
            sgu = mmq_product(self.shared, cfg.sh_gu_type, 2 * FS, H, cfg.shared_bytes, 1, self.sh_xq, self.sh_bounds, None, T,
                              None, FS, error=self.err, xq_out=self.sh_hq)
            _check("mmq_run_glu", lib.maya_mmq_run_glu(C.byref(sgu), cfg.limit, s))
            sdn = mmq_product(self.shared.data_ptr() + self.sh_down_off, cfg.sh_d_type, H, FS, cfg.shared_bytes, 1, self.sh_hq,
                              self.sh_bounds, None, T, self.sh_out, H, error=self.err)
            _check("mmq_run", lib.maya_mmq_run(C.byref(sdn), s))
            sh_out = self.sh_out
        ffn = self.ffn[:T]
        if self.expert_range is None:
            _check("moe_combine_rows", lib.maya_moe_combine_rows(_ptr(self.out), _ptr(self.pos), _ptr(w), _ptr(sh_out), T, k, H,
                                                                _ptr(ffn), s))
        elif peer is not None:
            _check("moe_combine_rows_local_ar",
                   lib.maya_moe_combine_rows_local_ar(_ptr(self.out), _ptr(self.pos), _ptr(w), _ptr(ids), self.expert_range[0],
                                                      self.expert_range[1], _ptr(sh_out), T, k, H, _ptr(ffn), C.byref(peer.desc),
                                                      peer.mi, 0 if peer.device_seq else peer.next_seq(), s))
        else:
            _check("moe_combine_rows_local",
                   lib.maya_moe_combine_rows_local(_ptr(self.out), _ptr(self.pos), _ptr(w), _ptr(ids), self.expert_range[0],
                                                   self.expert_range[1], _ptr(sh_out), T, k, H, _ptr(ffn), s))
        return ids, w, ffn

    def error(self) -> int:
        """1 when a bounded wait inside a grouped-GEMM launch ran out (synchronises)."""
        return int(self.err.item())
