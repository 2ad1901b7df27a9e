"""TEST INFRASTRUCTURE: the reference's own CUDA expert kernels on this GPU (oracle/_ref/libmaya_ref_gpu.so, built by
oracle/build.py from the reference tree where it lies).  Only tests/ and bench.py's `gpu_baseline` leg load it; nothing
under project_maya_b200/ does.

RefGpu.layer_token runs the sequence the reference's decode path drives for one token of a MoE layer
(Glm5Model::fast_moe, src/core/glm_fast_path.cu:6917-7100, all experts resident):
router_top10 -> glmf::quantize_q8_1 -> [shared expert: native_mmvq of its gate|up rows + glmf::swiglu_q8] ->
glmf::moe_gate_up -> glmf::moe_down, every step the reference's unmodified kernel.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

LIB = Path(__file__).resolve().parent / "_ref" / "libmaya_ref_gpu.so"
Q81 = 36


def available() -> bool:
    return LIB.exists()


def _p(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


class RefGpu:
    def __init__(self):
        if not LIB.exists():
            raise RuntimeError(f"{LIB} is not built (python oracle/build.py, with the reference tree present)")
        self.lib = C.CDLL(str(LIB))
        L = self.lib
        vp, i, f, sz, i64 = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_int64
        L.ref_router_top10.argtypes = [vp, i, i, i, vp, vp, vp]
        L.ref_quantize_q8_1.argtypes = [vp, vp, i, vp]
        L.ref_quantize_q8_1_rows.argtypes = [vp, i64, i64, vp, vp]
        L.ref_iq_mmvq.argtypes = [i, vp, vp, vp, i, i, i, vp]
        L.ref_native_mmvq.argtypes = [i, vp, vp, vp, i, i, i, vp]
        L.ref_swiglu_q8.argtypes = [vp, vp, f, i, vp, vp]
        L.ref_native_expert_scratch_bytes.argtypes = [i64, i64]
        L.ref_native_expert_scratch_bytes.restype = sz
        L.ref_native_expert_grouped.argtypes = [i, i, i64, i64, vp, vp, vp, vp, vp, i64, i64, vp, vp, vp, vp, f]
        L.ref_moe_gate_up.argtypes = [i, vp, vp, i, i, i, f, vp, vp, vp, i, vp, i, vp, vp]
        L.ref_moe_down.argtypes = [i, vp, vp, vp, vp, i, i, i, sz, vp, vp, vp, vp]
        L.ref_moe_win_experts.argtypes = [i, i, vp, vp, vp, vp, vp, sz, vp, vp, vp, vp, sz, vp, vp, vp, vp, i, i, i, i, f, sz, vp]
        for name in ("ref_router_top10", "ref_quantize_q8_1", "ref_quantize_q8_1_rows", "ref_iq_mmvq", "ref_native_mmvq",
                     "ref_swiglu_q8", "ref_native_expert_grouped", "ref_moe_gate_up", "ref_moe_down", "ref_moe_win_experts",
                     "ref_launch_errors", "ref_moe_supported", "ref_iq_supported", "ref_native_mmvq_supported"):
            getattr(L, name).restype = C.c_int
        L.ref_moe_supported.argtypes = [i]
        L.ref_iq_supported.argtypes = [i]
        L.ref_native_mmvq_supported.argtypes = [i]

    @staticmethod
    def _stream():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def _ck(self, what, st):
        if st != 0:
            raise RuntimeError(f"reference {what} failed ({st})")

    def router(self, logits, k):
        T, E = logits.shape
        ids = torch.empty((T, k), dtype=torch.int32, device=logits.device)
        w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
        self._ck("router_top10", self.lib.ref_router_top10(_p(logits), T, E, k, _p(ids), _p(w), self._stream()))
        return ids, w

    def quantize(self, xf):
        n = xf.numel()
        xq = torch.empty(n // 32 * Q81, dtype=torch.uint8, device=xf.device)
        self._ck("quantize_q8_1", self.lib.ref_quantize_q8_1(_p(xf), _p(xq), n, self._stream()))
        return xq


class RefLayer:
    """One resident layer for the reference's single-token sequence; every buffer allocated once, so that forward()
    only enqueues launches (it can be captured in a CUDA graph)."""

    def __init__(self, ref: RefGpu, n_embd, n_ff, n_expert, k, gu_type, d_type, row_bytes, experts, shared=None, n_ff_sh=0,
                 sh_type=8, limit=float("inf")):
        self.ref, self.k, self.n_embd, self.n_ff, self.n_expert = ref, k, n_embd, n_ff, n_expert
        self.gu_type, self.d_type, self.sh_type, self.limit = gu_type, d_type, sh_type, limit
        self.experts, self.shared, self.n_ff_sh = experts, shared, n_ff_sh if shared is not None else 0
        self.stride = experts.stride(0)
        self.down_off = 2 * n_ff * row_bytes(gu_type, n_embd)
        dev = experts.device
        self.xf = torch.empty(n_embd, dtype=torch.float32, device=dev)
        self.xq = torch.empty(n_embd // 32 * Q81, dtype=torch.uint8, device=dev)
        self.plan_ptr = torch.zeros(8, dtype=torch.int64, device=dev)
        self.plan_w = torch.zeros(8, dtype=torch.float32, device=dev)
        self.hq = torch.empty(8 * (n_ff // 32) * Q81, dtype=torch.uint8, device=dev)
        self.ids = torch.empty((1, k), dtype=torch.int32, device=dev)
        self.w = torch.empty((1, k), dtype=torch.float32, device=dev)
        self.out = torch.empty(n_embd, dtype=torch.float32, device=dev)
        self.cpu_flag = torch.zeros(16, dtype=torch.int32, device=dev)   # read unconditionally by the reference's down kernel
        if self.n_ff_sh:
            self.sh_gu = torch.empty(2 * n_ff_sh, dtype=torch.float32, device=dev)
            self.sh_hq = torch.empty(n_ff_sh // 32 * Q81, dtype=torch.uint8, device=dev)
            self.sh_out = torch.empty(n_embd, dtype=torch.float32, device=dev)
            self.sh_down = shared[2 * n_ff_sh * row_bytes(sh_type, n_embd):]

    def forward(self, logits, x, out=None):
        """logits [1, n_expert] f32, x [1, n_embd] f32 or bf16 -> (ids [1, k], weights [1, k], out [n_embd])."""
        L, s = self.ref.lib, self.ref._stream()
        ck = self.ref._ck
        out = self.out if out is None else out
        ck("router_top10", L.ref_router_top10(_p(logits), 1, self.n_expert, self.k, _p(self.ids), _p(self.w), s))
        self.xf.copy_(x.reshape(-1))
        ck("quantize_q8_1", L.ref_quantize_q8_1(_p(self.xf), _p(self.xq), self.n_embd, s))
        self.plan_ptr[: self.k] = self.ids[0].to(torch.int64) * self.stride + self.experts.data_ptr()
        self.plan_w[: self.k] = self.w[0]
        sh = self.n_ff_sh > 0
        if sh:
            ck("native_mmvq", L.ref_native_mmvq(self.sh_type, _p(self.shared), _p(self.xq), _p(self.sh_gu), self.n_embd,
                                                2 * self.n_ff_sh, 1, s))
            ck("swiglu_q8", L.ref_swiglu_q8(_p(self.sh_gu), _p(self.sh_gu[self.n_ff_sh:]), self.limit, self.n_ff_sh,
                                            _p(self.sh_hq), s))
        ck("moe_gate_up", L.ref_moe_gate_up(self.gu_type, _p(self.plan_ptr), _p(self.plan_w), self.k, self.n_embd, self.n_ff,
                                            self.limit, _p(self.xq), _p(self.hq), _p(self.sh_down) if sh else None, self.sh_type,
                                            _p(self.sh_hq) if sh else None, self.n_ff_sh, _p(self.sh_out) if sh else None, s))
        ck("moe_down", L.ref_moe_down(self.d_type, _p(self.plan_ptr), _p(self.plan_w), None, _p(self.cpu_flag), self.k, self.n_embd,
                                      self.n_ff, self.down_off, _p(self.hq), _p(self.sh_out) if sh else None, _p(out), s))
        return self.ids, self.w, out
