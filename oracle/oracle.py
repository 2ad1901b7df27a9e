"""ctypes + numpy front end of the CPU checkers.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm import this module.  The shipped
library (project_maya_b200) never does: its CUDA path has no CPU fallback.

  Oracle   the C restatement of the reference's arithmetic (oracle/maya_oracle.c -> oracle/_build/libmaya_oracle.so)
  Ref      the reference's own CPU sources for this path compiled where they lie (oracle/_ref/libmaya_ref.so), when built
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
Q8_0, Q4_K, IQ3_S, IQ2_S = 8, 12, 21, 22

_u8p = C.POINTER(C.c_uint8)
_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int32)


def _p(a: np.ndarray, ty):
    return a.ctypes.data_as(ty)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    return a.view(np.uint8).reshape(-1)


class Oracle:
    def __init__(self, path: Path | None = None):
        path = path or HERE / "_build" / "libmaya_oracle.so"
        if not path.exists() or path.stat().st_mtime < (HERE / "maya_oracle.c").stat().st_mtime:   # missing or stale
            import importlib.util
            spec = importlib.util.spec_from_file_location("maya_oracle_build", HERE / "build.py")
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.build_oracle()
        self.lib = C.CDLL(str(path))
        L = self.lib
        L.orc_row_bytes.restype = C.c_size_t
        L.orc_row_bytes.argtypes = [C.c_int, C.c_int64]

    # ---- formats
    def row_bytes(self, t: int, n: int) -> int:
        return int(self.lib.orc_row_bytes(t, n))

    def blob_bytes(self, gu_type: int, d_type: int, n_embd: int, n_ff: int) -> int:
        return 2 * n_ff * self.row_bytes(gu_type, n_embd) + n_embd * self.row_bytes(d_type, n_ff)

    def quantize_q8_1(self, x) -> np.ndarray:
        x = _f32(x).reshape(-1)
        y = np.empty(x.size // 32 * 36, np.uint8)
        self.lib.orc_quantize_q8_1(_p(x, _f32p), _p(y, _u8p), C.c_int64(x.size))
        return y

    def quantize_q8_K(self, x) -> np.ndarray:
        x = _f32(x).reshape(-1)
        y = np.empty(x.size // 256 * 292, np.uint8)
        self.lib.orc_quantize_q8_K(_p(x, _f32p), _p(y, _u8p), C.c_int64(x.size))
        return y

    def dequantize(self, t: int, w, n: int) -> np.ndarray:
        w = _u8(w)
        y = np.empty(n, np.float32)
        rc = self.lib.orc_dequantize(t, _p(w, _u8p), C.c_int64(n), _p(y, _f32p))
        assert rc == 0
        return y

    # ---- GEMV
    def mmvq(self, t: int, w, xq, n_in: int, n_out: int, ncols: int = 1, order: int = 0) -> np.ndarray:
        w, xq = _u8(w), _u8(xq)
        y = np.empty((ncols, n_out), np.float32)
        rc = self.lib.orc_mmvq(t, _p(w, _u8p), _p(xq, _u8p), _p(y, _f32p), n_in, n_out, ncols, order)
        assert rc == 0
        return y

    def swiglu(self, g, u, limit: float) -> np.ndarray:
        g, u = _f32(g).reshape(-1), _f32(u).reshape(-1)
        h = np.empty_like(g)
        self.lib.orc_swiglu(_p(g, _f32p), _p(u, _f32p), C.c_float(limit), C.c_int64(g.size), _p(h, _f32p))
        return h

    # ---- experts
    def expert_q8_1(self, gu_type, d_type, blob, n_embd, n_ff, limit, xq, want_hq=False):
        blob, xq = _u8(blob), _u8(xq)
        part = np.empty(n_embd, np.float32)
        hq = np.empty(n_ff // 32 * 36, np.uint8)
        rc = self.lib.orc_expert_q8_1(gu_type, d_type, _p(blob, _u8p), n_embd, n_ff, C.c_float(limit), _p(xq, _u8p),
                                      _p(part, _f32p), _p(hq, _u8p))
        assert rc == 0
        return (part, hq) if want_hq else part

    def expert_q8_1_mixed(self, g_type, u_type, d_type, blob, n_embd, n_ff, limit, xq) -> np.ndarray:
        """A layer whose up rows have their own type (native_expert_layout(gu_type, up_type, d_type, ...),
        iq_kernels.hpp:73-77): gate rows, then up rows, then down rows in the blob; the same three GEMVs, SwiGLU and
        q8_1 image of h as expert_q8_1, composed from the single steps.  With g_type == u_type it is expert_q8_1."""
        blob = _u8(blob)
        up_off = n_ff * self.row_bytes(g_type, n_embd)
        down_off = up_off + n_ff * self.row_bytes(u_type, n_embd)
        g = self.mmvq(g_type, blob[:up_off], xq, n_embd, n_ff)[0]
        u = self.mmvq(u_type, blob[up_off:down_off], xq, n_embd, n_ff)[0]
        hq = self.quantize_q8_1(self.swiglu(g, u, limit))
        return self.mmvq(d_type, blob[down_off:], hq, n_ff, n_embd)[0]

    # ---- the prompt path's arithmetic as the reference models it on the host
    def mmq_host_model(self, t: int, w, n_rows: int, K: int, x) -> np.ndarray:
        """The reference's host model of what its prompt-path GEMM (llama.cpp's MMQ behind mmq::Context::run) computes,
        restated from tests/glm_dsa/glmd_mmq_ids_test.cu:92-244,288-347 (the dp4a form its CUDA builds keep):
          activations per 32 values: d_inv = 127 / amax, u = round(x d_inv) (half away from zero), d = 1 / d_inv in float,
            kept as float for the "d4" layout (Q8_0, IQ2_S, IQ3_S) and rounded to f16 for "ds4" (Q4_K); xr = u d;
          weights: to_float's values;
          "plain" (d4 types): y = sum_k w_k xr_k;
          "offset" (Q4_K): y = sum over 32-value groups b of [sum_{k in b} w_k xr_k + c_b (S_b - sum_{k in b} xr_k)] with
            c_b = -(dmin m_b), the group's constant term, and S_b the f16-rounded sum of the UNQUANTIZED values, added in
            the order of quantize_mmq_q8_1 (4 values per thread left to right, then a shuffle tree);
          every sum in double, in k order.  w: n_rows rows of K quantized values; x [n, K] f32.  Returns [n, n_rows] f64."""
        x = _f32(x).reshape(-1, K)
        n = x.shape[0]
        wf = self.dequantize(t, w, n_rows * K).reshape(n_rows, K).astype(np.float64)
        xb = x.reshape(n, K // 32, 32)
        am = np.abs(xb).max(axis=2, keepdims=True).astype(np.float32)
        with np.errstate(divide="ignore", invalid="ignore"):
            d_inv = (np.float32(127.0) / am).astype(np.float32)
            d = (np.float32(1.0) / d_inv).astype(np.float32)
            v = (xb * d_inv).astype(np.float32)
        u = np.where(am > 0, np.sign(v) * np.floor(np.abs(v).astype(np.float64) + 0.5), 0.0).astype(np.float32)   # roundf
        offset = t == 12                                                   # Q4_K: the ds4 layout
        ds = d.astype(np.float16).astype(np.float32) if offset else d
        xr = np.where(am > 0, u * ds, 0.0).astype(np.float32).reshape(n, K).astype(np.float64)
        y = xr @ wf.T
        if offset:
            blk = _u8(w).reshape(n_rows, K // 256, 144)
            dmin = blk[:, :, 2:4].copy().view(np.float16).astype(np.float32)[:, :, 0]
            sc8 = blk[:, :, 4:16].astype(np.int32)
            mn = np.stack([(sc8[:, :, sb + 4] & 63) if sb < 4 else ((sc8[:, :, sb + 4] >> 4) | ((sc8[:, :, sb] >> 6) << 4))
                           for sb in range(8)], axis=-1)                   # [rows, nb, 8]
            c = -(dmin[:, :, None] * mn.astype(np.float32)).astype(np.float32).reshape(n_rows, K // 32).astype(np.float64)
            pt = xb.reshape(n, K // 32, 8, 4)
            part = ((pt[..., 0] + pt[..., 1]).astype(np.float32) + pt[..., 2]).astype(np.float32)
            part = (part + pt[..., 3]).astype(np.float32)                  # each thread: its 4 values left to right
            for off in (4, 2, 1):
                part = (part[..., :off] + part[..., off:2 * off]).astype(np.float32)
            S = part[..., 0].astype(np.float16).astype(np.float64)         # [n, K / 32]
            xa = S - xr.reshape(n, K // 32, 32).sum(axis=2)
            y = y + xa @ c.T
        return y

    def expert_mmq(self, gu_type, d_type, blob, n_embd, n_ff, limit, x) -> np.ndarray:
        """One expert as the reference's PROMPT path computes it (src/core/glm_prefill.cu:3230-3420: mmq::quantize,
        run_glu, mmq::quantize of h, run): both products by mmq_host_model, SwiGLU on f32 values between them.  Differs
        from expert_q8_1 (the decode kernels) where a type has a constant term per group: Q4_K's decode dot multiplies
        -dmin * m by the sum of the ROUNDED activations (dp4a with 0x01010101, native_mmvq.cu:170), MMQ by the stored
        sum of the unquantized ones - about 1e-2 apart in rel-L2 on N(0, 0.02) weights."""
        blob = _u8(blob)
        gu = 2 * n_ff * self.row_bytes(gu_type, n_embd)
        y = self.mmq_host_model(gu_type, blob[:gu], 2 * n_ff, n_embd, x)[0]
        h = self.swiglu(y[:n_ff].astype(np.float32), y[n_ff:].astype(np.float32), limit)
        return self.mmq_host_model(d_type, blob[gu:], n_embd, n_ff, h)[0].astype(np.float32)

    def expert_f64(self, gu_type, d_type, blob, n_embd, n_ff, x) -> np.ndarray:
        blob, x = _u8(blob), _f32(x).reshape(-1)
        out = np.empty(n_embd, np.float32)
        rc = self.lib.orc_expert_f64(gu_type, d_type, _p(blob, _u8p), n_embd, n_ff, _p(x, _f32p), _p(out, _f32p))
        assert rc == 0
        return out

    def combine_down(self, parts, w, shared=None, skip=None) -> np.ndarray:
        parts, w = _f32(parts), _f32(w).reshape(-1)
        k, n = parts.shape
        out = np.empty(n, np.float32)
        sh = _f32(shared).reshape(-1) if shared is not None else None
        sk = np.ascontiguousarray(skip, dtype=np.uint8) if skip is not None else None
        self.lib.orc_combine_down(_p(parts, _f32p), _p(w, _f32p), _p(sk, _u8p) if sk is not None else None, k,
                                  _p(sh, _f32p) if sh is not None else None, C.c_int64(n), _p(out, _f32p))
        return out

    def combine_native(self, parts, w, shared=None) -> np.ndarray:
        parts, w = _f32(parts), _f32(w).reshape(-1)
        k, n = parts.shape
        out = np.empty(n, np.float32)
        sh = _f32(shared).reshape(-1) if shared is not None else None
        self.lib.orc_combine_native(_p(parts, _f32p), _p(w, _f32p), k, _p(sh, _f32p) if sh is not None else None,
                                    C.c_int64(n), _p(out, _f32p))
        return out

    # ---- routers
    def _route_out(self, logits, k):
        logits = _f32(logits)
        T, E = logits.shape
        return logits, T, E, np.empty((T, k), np.int32), np.empty((T, k), np.float32)

    def router_top10(self, logits, k):
        logits, T, E, ids, w = self._route_out(logits, k)
        assert self.lib.orc_router_top10(_p(logits, _f32p), T, E, k, _p(ids, _i32p), _p(w, _f32p)) == 0
        return ids, w

    def router_f64(self, logits, k):
        logits, T, E, ids, w = self._route_out(logits, k)
        assert self.lib.orc_router_f64(_p(logits, _f32p), T, E, k, _p(ids, _i32p), _p(w, _f32p)) == 0
        return ids, w

    def router_sigmoid(self, logits, bias, k, w_scale=1.0, norm_w=True):
        logits, T, E, ids, w = self._route_out(logits, k)
        b = _f32(bias).reshape(-1) if bias is not None else None
        rc = self.lib.orc_router_sigmoid(_p(logits, _f32p), _p(b, _f32p) if b is not None else None, T, E, k,
                                         C.c_float(w_scale), int(norm_w), _p(ids, _i32p), _p(w, _f32p))
        assert rc == 0
        return ids, w

    def rms_router(self, h, add, w, eps, router_w):
        """(h + add, x = rms(h + add) * w, logits = router_w . x)"""
        h, w, router_w = _f32(h).reshape(-1), _f32(w).reshape(-1), _f32(router_w)
        a = _f32(add).reshape(-1) if add is not None else None
        n, E = h.size, router_w.shape[0]
        h_out, x, logits = np.empty(n, np.float32), np.empty(n, np.float32), np.empty(E, np.float32)
        self.lib.orc_rms_router(_p(h, _f32p), _p(a, _f32p) if a is not None else None, _p(w, _f32p), C.c_float(eps), n,
                                _p(router_w, _f32p), E, _p(h_out, _f32p), _p(x, _f32p), _p(logits, _f32p))
        return h_out, x, logits

    def hc_post(self, block_out, R_old, post, comb):
        """R_new [4, n_embd] = block_out * post[d] + comb[d, :] . R_old[:, e]"""
        b, R, po, co = _f32(block_out).reshape(-1), _f32(R_old), _f32(post).reshape(-1), _f32(comb).reshape(-1)
        n = b.size
        assert R.shape == (4, n) and po.size == 4 and co.size == 16
        out = np.empty((4, n), np.float32)
        self.lib.orc_hc_post(_p(b, _f32p), _p(R, _f32p), _p(po, _f32p), _p(co, _f32p), n, _p(out, _f32p))
        return out

    # ---- misc
    def allreduce_in_order(self, parts) -> np.ndarray:
        parts = _f32(parts)
        nm, n = parts.shape
        out = np.empty(n, np.float32)
        self.lib.orc_allreduce_in_order(_p(parts, _f32p), nm, C.c_int64(n), _p(out, _f32p))
        return out

    def expert_group(self, ids, k, n_expert):
        ids = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
        n = ids.size
        counts = np.empty(n_expert, np.int32)
        bounds = np.empty(n_expert + 1, np.int32)
        pos = np.empty(n, np.int32)
        row_tok = np.empty(n, np.int32)
        self.lib.orc_expert_group(_p(ids, _i32p), n, k, n_expert, _p(counts, _i32p), _p(bounds, _i32p), _p(pos, _i32p),
                                  _p(row_tok, _i32p))
        return counts, bounds, pos, row_tok

    # ---- whole layer (route -> experts -> combine [+ shared]) through the quantized path, token by token
    def moe_layer(self, cfg, logits, x, experts, shared=None, expert_range=None):
        """cfg: dict(n_embd, n_ff, n_expert, k, gu_type, d_type, limit[, n_ff_sh, sh_gu_type, sh_d_type]).
        experts: uint8 [n_expert, blob_bytes]; x: f32 [T, n_embd] (already rounded if the input was bf16).
        Returns ids, weights, out."""
        H, FF, k = cfg["n_embd"], cfg["n_ff"], cfg["k"]
        limit = cfg.get("limit", float("inf"))
        logits, x = _f32(logits), _f32(x)
        T = x.shape[0]
        ids, w = self.router_top10(logits, k)
        out = np.zeros((T, H), np.float32)
        lo, hi = expert_range if expert_range is not None else (0, cfg["n_expert"])
        for t in range(T):
            xq = self.quantize_q8_1(x[t])
            parts = np.zeros((k, H), np.float32)
            skip = np.zeros(k, np.uint8)
            for j in range(k):
                e = int(ids[t, j])
                if lo <= e < hi:
                    parts[j] = self.expert_q8_1(cfg["gu_type"], cfg["d_type"], experts[e], H, FF, limit, xq)
                else:
                    skip[j] = 1
            sh = None
            if shared is not None:
                sh = self.expert_q8_1(cfg["sh_gu_type"], cfg["sh_d_type"], shared, H, cfg["n_ff_sh"], limit, xq)
            out[t] = self.combine_down(parts, w[t], sh, skip)
        return ids, w, out


class Ref:
    """The reference's own CPU code (present only where oracle/_ref/libmaya_ref.so was built)."""

    def __init__(self, path: Path | None = None):
        path = path or HERE / "_ref" / "libmaya_ref.so"
        if not path.exists():
            raise FileNotFoundError(str(path))
        self.lib = C.CDLL(str(path))

    @staticmethod
    def available() -> bool:
        return (HERE / "_ref" / "libmaya_ref.so").exists()

    def router_reference(self, logits, k):
        logits = _f32(logits)
        T, E = logits.shape
        ids = np.empty((T, k), np.int32)
        w = np.empty((T, k), np.float32)
        self.lib.ref_router_reference(_p(logits, _f32p), T, E, k, _p(ids, _i32p), _p(w, _f32p))
        return ids, w

    def router_test_inputs(self) -> np.ndarray:
        out = np.empty((4, 64, 512), np.float32)
        self.lib.ref_router_test_inputs(_p(out, _f32p))
        return out

    def quantize_q8_K(self, x) -> np.ndarray:
        x = _f32(x).reshape(-1)
        y = np.zeros(x.size // 256 * 292, np.uint8)
        self.lib.ref_quantize_q8_K(_p(x, _f32p), C.c_longlong(x.size), _p(y, _u8p))
        return y

    def _acts(self, acts):
        acts = [np.ascontiguousarray(a, dtype=np.uint8) for a in acts]
        arr = (C.c_void_p * len(acts))(*[a.ctypes.data for a in acts])
        return acts, arr

    def gu_rows(self, t, blob, gu_row, up_off, n, acts_q8k, r0, r1, avx512=True) -> np.ndarray:
        blob = _u8(blob)
        keep, arr = self._acts(acts_q8k)
        nt = len(keep)
        ff = np.zeros((nt, r1), np.float32)
        outs = (C.c_void_p * nt)(*[ff[i].ctypes.data for i in range(nt)])
        self.lib.ref_gu_rows(int(avx512), t, _p(blob, _u8p), C.c_size_t(gu_row), C.c_size_t(up_off), n, arr, nt, outs,
                             r0, r1)
        return ff

    def rows(self, t, w, row_bytes, n, acts_q8k, r0, r1, avx512=True) -> np.ndarray:
        w = _u8(w)
        keep, arr = self._acts(acts_q8k)
        nt = len(keep)
        out = np.zeros((nt, r1), np.float32)
        outs = (C.c_void_p * nt)(*[out[i].ctypes.data for i in range(nt)])
        self.lib.ref_rows(int(avx512), t, _p(w, _u8p), C.c_size_t(row_bytes), n, arr, nt, outs, r0, r1)
        return out

    def pool_threads(self, threads: int) -> int:
        return int(self.lib.ref_pool_threads(int(threads)))

    def layer_tokens(self, gu_type, d_type, gu_row, d_row, n_embd, n_ff, k, blobs, weights, x, shared, n_ff_sh, avx512=True):
        """n_tok decode tokens of a layer on the host pool (ref_shim_layer.cpp): blobs = n_tok * k uint8 arrays (token t's
        j-th routed expert), weights [n_tok, k], x [n_tok, n_embd] f32, shared = the Q8_0 shared expert's blob or None.
        Returns (out [n_tok, n_embd], seconds)."""
        x = _f32(x)
        n_tok = x.shape[0]
        weights = _f32(weights)
        keep = [_u8(b) for b in blobs]
        arr = (C.c_void_p * len(keep))(*[b.ctypes.data for b in keep])
        sh = _u8(shared) if shared is not None else None
        out = np.zeros((n_tok, n_embd), np.float32)
        self.lib.ref_layer_tokens.restype = C.c_double
        dt = self.lib.ref_layer_tokens(int(avx512), gu_type, d_type, C.c_size_t(gu_row), C.c_size_t(d_row), n_embd, n_ff, k, arr,
                                       _p(weights, _f32p), _p(x, _f32p), _p(sh, _u8p) if sh is not None else None,
                                       n_ff_sh if sh is not None else 0, n_tok, _p(out, _f32p))
        return out, float(dt)
