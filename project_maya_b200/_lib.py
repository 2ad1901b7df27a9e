"""Loader of the C-ABI library (libmaya_moe.so) and its ctypes signatures.

There is no fallback: if the library has not been built, importing the compute entry points raises.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

PKG = Path(__file__).resolve().parent
# MAYA_MOE_LIB: another build of the same library (comparing two builds on one machine); it must export the same ABI
LIB_PATH = Path(os.environ.get("MAYA_MOE_LIB") or PKG / "libmaya_moe.so")

c_void_p, c_int, c_float, c_size_t, c_int64, c_uint64 = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_int64, C.c_uint64


class ExpertLayout(C.Structure):
    _fields_ = [("gu_type", c_int), ("d_type", c_int), ("n_embd", c_int64), ("n_ff", c_int64),
                ("gu_row", c_size_t), ("d_row", c_size_t), ("up_off", c_size_t), ("down_off", c_size_t),
                ("bytes", c_size_t), ("u_type", c_int), ("u_row", c_size_t)]


class MoePlan(C.Structure):
    _fields_ = [("plan_ptr", c_void_p), ("plan_w", c_void_p), ("cpu_part", c_void_p), ("cpu_flag", c_void_p),
                ("skip", c_void_p)]


class MoeWin(C.Structure):
    _fields_ = [("plan_ptr", c_void_p), ("plan_w", c_void_p), ("cpu_part", c_void_p), ("cpu_flag", c_void_p),
                ("xq", c_void_p), ("xq_stride", c_size_t), ("hq", c_void_p), ("part", c_void_p), ("sh_out", c_void_p),
                ("out", c_void_p), ("out_stride", c_size_t), ("grp_ptr", c_void_p), ("grp_start", c_void_p),
                ("grp_ent", c_void_p), ("n_groups", c_void_p), ("T", c_int), ("k", c_int), ("n_embd", c_int),
                ("n_ff", c_int), ("limit", c_float), ("down_off", c_size_t)]


class MoeLayerDesc(C.Structure):
    _fields_ = [("n_embd", c_int), ("n_ff", c_int), ("n_expert", c_int), ("k", c_int), ("gu_type", c_int),
                ("d_type", c_int), ("experts", c_void_p), ("expert_stride", c_size_t), ("n_ff_sh", c_int),
                ("sh_gu_type", c_int), ("sh_d_type", c_int), ("shared", c_void_p), ("limit", c_float),
                ("expert_lo", c_int), ("expert_hi", c_int), ("shared_here", c_int), ("staged", c_int), ("sh_lo", c_int),
                ("sh_hi", c_int), ("router", c_int), ("router_bias", c_void_p), ("router_w_scale", c_float),
                ("router_norm_w", c_int), ("cpu_part", c_void_p), ("cpu_flag", c_void_p)]


class MmqProduct(C.Structure):
    _fields_ = [("w", c_void_p), ("type", c_int), ("w_rows", c_int64), ("w_cols", c_int64), ("expert_bytes", c_size_t),
                ("n", c_int), ("xq", c_void_p), ("bounds", c_void_p), ("ids", c_void_p), ("total_rows", c_int64),
                ("max_rows", c_int64), ("dst", c_void_p), ("ld_dst", c_int64), ("expert_map", c_void_p),
                ("error", c_void_p), ("xq_out", c_void_p)]


class PeerArFailure(C.Structure):
    _fields_ = [("captured", C.c_uint), ("sequence", C.c_uint), ("observed", C.c_uint), ("block", C.c_uint),
                ("n4", C.c_uint), ("rank", C.c_uint), ("waited_for", C.c_uint), ("pad", C.c_uint),
                ("elapsed_ns", C.c_ulonglong), ("timeout_ns", C.c_ulonglong)]


class PeerArDesc(C.Structure):
    _fields_ = [("recv", c_void_p), ("peer_recv", c_void_p), ("flags", c_void_p), ("peer_flags", c_void_p),
                ("error", c_void_p), ("failure", c_void_p), ("stride", c_size_t), ("timeout_ns", C.c_ulonglong),
                ("nm", c_int), ("seq_counter", c_void_p)]


class HcPostArgs(C.Structure):
    _fields_ = [("R_old", c_void_p), ("post", c_void_p), ("comb", c_void_p), ("R_new", c_void_p)]


_SIGNATURES = {
    "maya_version": (C.c_char_p, []),
    "maya_last_cuda_error": (c_int, []),
    "maya_launch_errors": (c_int, []),
    "maya_launch_count": (C.c_longlong, []),
    "maya_device_ok": (c_int, []),
    "maya_type_supported": (c_int, [c_int]),
    "maya_row_bytes": (c_size_t, [c_int, c_int64]),
    "maya_weight_bytes": (c_size_t, [c_int, c_int, c_int]),
    "maya_q8_1_bytes": (c_size_t, [c_int, c_int]),
    "maya_expert_layout_make": (c_int, [c_int, c_int, c_int, c_int64, c_int64, C.POINTER(ExpertLayout)]),
    "maya_router_top10": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "maya_router_sigmoid": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p]),
    "maya_quantize_q8_1": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "maya_quantize_q8_1_bf16": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "maya_swiglu_q8_1": (c_int, [c_void_p, c_void_p, c_float, c_int64, c_void_p, c_void_p]),
    "maya_mmvq": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "maya_moe_gate_up": (c_int, [c_int, C.POINTER(MoePlan), c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p,
                                 c_int, c_void_p, c_int, c_void_p, c_void_p]),
    "maya_moe_down": (c_int, [c_int, C.POINTER(MoePlan), c_int, c_int, c_int, c_size_t, c_void_p, c_void_p, c_void_p,
                              c_void_p]),
    "maya_moe_win_experts": (c_int, [c_int, c_int, C.POINTER(MoeWin), c_void_p]),
    "maya_moe_win_group": (c_int, [C.POINTER(MoeWin), c_void_p]),
    "maya_expert_scratch_bytes": (c_size_t, [c_int64, c_int64]),
    "maya_expert_grouped": (c_int, [C.POINTER(ExpertLayout), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                    c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_float]),
    "maya_expert_static_scratch_bytes": (c_size_t, []),
    "maya_expert_grouped_static": (c_int, [C.POINTER(ExpertLayout), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                           c_int64, c_void_p, c_void_p, c_void_p, c_float]),
    "maya_moe_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "maya_expert_count": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "maya_expert_bounds": (c_int, [c_void_p, c_int, c_void_p, c_void_p]),
    "maya_expert_scatter": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "maya_swiglu_rows": (c_int, [c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p]),
    "maya_moe_combine_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "maya_rms_router": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                c_void_p]),
    "maya_mmq_supported": (c_int, [c_int]),
    "maya_mmq_q8_bytes": (c_size_t, [c_int64, c_int64]),
    "maya_mmq_quantize": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p]),
    "maya_mmq_quantize_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p]),
    "maya_mmq_quantize_routed": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p]),
    "maya_mmq_quantize_routed_bf16": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p]),
    "maya_mmq_run": (c_int, [C.POINTER(MmqProduct), c_void_p]),
    "maya_mmq_run_glu": (c_int, [C.POINTER(MmqProduct), c_float, c_void_p]),
    "maya_moe_combine_rows_local": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int,
                                            c_void_p, c_void_p]),
    "maya_moe_combine_rows_local_ar": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int,
                                               c_void_p, c_void_p, c_int, C.c_uint, c_void_p]),
    "maya_moe_combine_add": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "maya_moe_layer_scratch_bytes": (c_size_t, [C.POINTER(MoeLayerDesc), c_int]),
    "maya_moe_layer_error": (c_int, [C.POINTER(MoeLayerDesc), c_int, c_void_p, c_void_p]),
    "maya_moe_layer_phase_ns": (c_int, [C.POINTER(MoeLayerDesc), c_void_p, c_void_p, C.POINTER(C.c_ulonglong)]),
    "maya_moe_layer_decode": (c_int, [C.POINTER(MoeLayerDesc), c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_size_t, c_void_p]),
    "maya_peer_ar_recv_bytes": (c_size_t, [c_int, c_size_t]),
    "maya_peer_ar_flag_bytes": (c_size_t, [c_int]),
    "maya_peer_ar_preload": (c_int, [c_void_p]),
    "maya_allreduce_peer": (c_int, [c_void_p, c_int, C.POINTER(PeerArDesc), c_int, C.c_uint, c_void_p]),
    "maya_moe_layer_decode_ar": (c_int, [C.POINTER(MoeLayerDesc), c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_size_t, C.POINTER(PeerArDesc), c_int, C.c_uint, c_void_p]),
    "maya_hc_post": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "maya_moe_layer_decode_hc": (c_int, [C.POINTER(MoeLayerDesc), c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_size_t, C.POINTER(PeerArDesc), c_int, C.c_uint,
                                         C.POINTER(HcPostArgs), c_void_p]),
    "maya_peer_buffer_create": (c_int, [c_size_t, C.POINTER(c_void_p), C.c_char_p]),
    "maya_peer_buffer_open": (c_int, [C.c_char_p, C.POINTER(c_void_p)]),
    "maya_peer_buffer_close": (c_int, [c_void_p]),
    "maya_peer_buffer_destroy": (c_int, [c_void_p]),
    "maya_quantize_weights_host": (c_int, [c_int, c_void_p, c_int64, c_int64, c_void_p]),
    "maya_synth_weights": (c_int, [c_int, c_uint64, c_float, c_int64, c_int64, c_void_p, c_void_p]),
}

_lib = None


def load() -> C.CDLL:
    """The loaded library; raises if it has not been built (python -m project_maya_b200.build)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m project_maya_b200.build` "
                               "(there is no CPU or PyTorch fallback for this path)")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def declared_symbols() -> list[str]:
    return sorted(_SIGNATURES)
