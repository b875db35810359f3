"""ctypes binding of libglorcq_b200.so (the C ABI declared in include/glorcq_b200.h).

There is no fallback: if the library is missing, or a call returns a non-zero status, a
RuntimeError is raised -- the same exception type the reference's native modules raise through
TORCH_CHECK (inference/kernels/turbo_matmul.cu:250-283).
"""

from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# GLQ_LIB selects another build of the same ABI (e.g. one compiled with -DGLQ_CHECKED)
LIB_PATH = os.environ.get("GLQ_LIB") or os.path.join(HERE, "libglorcq_b200.so")

FMT_Q2, FMT_Q4, FMT_T2, FMT_F16 = 0, 1, 2, 3
EPI_LINEAR, EPI_SWIGLU = 0, 1

vp = C.c_void_p


class Weight(C.Structure):
    """glq_weight_t"""
    _fields_ = [("codes", vp), ("reserved0", vp), ("norms", vp), ("centroids", vp), ("sv", vp), ("bias", vp),
                ("N", C.c_int32), ("K", C.c_int32), ("rank", C.c_int32), ("reserved", C.c_int32)]


class MMArgs(C.Structure):
    """glq_mm_args_t"""
    _fields_ = [("fmt", C.c_int32), ("group_size", C.c_int32), ("epilogue", C.c_int32), ("n_problems", C.c_int32),
                ("max_rows", C.c_int32), ("rows_stride", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
                ("rank", C.c_int32), ("total_rows", C.c_int32),
                ("w", Weight), ("w_table", vp),
                ("slot_index", vp), ("n_slots", vp), ("slot_count", vp), ("slot_offset", vp), ("entry_row", vp),
                ("entry_scale", vp),
                ("x", vp), ("ldx", C.c_int64), ("a0", vp), ("a1", vp), ("lda", C.c_int64),
                ("y", vp), ("ldy", C.c_int64), ("workspace", vp), ("workspace_bytes", C.c_size_t),
                ("counters", vp), ("n_counters", C.c_size_t), ("flags", C.c_int32), ("reserved", C.c_int32)]


class MoeDesc(C.Structure):
    """glq_moe_desc_t"""
    _fields_ = [("H", C.c_int32), ("I", C.c_int32), ("E", C.c_int32), ("top_k", C.c_int32),
                ("I_shared", C.c_int32), ("rank", C.c_int32), ("fmt", C.c_int32), ("group_size", C.c_int32),
                ("norm_topk_prob", C.c_int32), ("router_rows", C.c_int32), ("slot_order_max_tokens", C.c_int32),
                ("reserved", C.c_int32),
                ("router_t", vp), ("gate_up", vp), ("down", vp), ("ut_gate_up", vp), ("ut_down", vp),
                ("dense0_rows", C.c_int32), ("sh_a_row", C.c_int32),
                ("sh_gate_up", Weight), ("sh_down", Weight),
                ("sh_ut_gate", vp), ("sh_ut_up", vp), ("sh_ut_down", vp),
                ("rot_in", vp), ("rot_mid", vp), ("sh_rot_mid", vp),
                ("rht_in", vp), ("rht_mid", vp), ("sh_rht_mid", vp),
                ("router_rm", vp), ("ut_rm_gate_up", vp), ("ut_rm_down", vp), ("sh_ut_rm_down", vp)]


class EpPeers(C.Structure):
    """glq_ep_peers_t"""
    _fields_ = [("entry_bufs", vp), ("flags", vp), ("epoch", vp), ("error", vp), ("half_elems", C.c_size_t),
                ("wait_limit_ns", C.c_uint64)]


class MoeEp(C.Structure):
    """glq_moe_ep_t"""
    _fields_ = [("rank", C.c_int32), ("world", C.c_int32), ("phase", C.c_int32), ("flags", C.c_int32),
                ("entry_out", vp), ("sel_in", vp), ("weight_in", vp),
                ("residual", vp), ("norm_weight", vp), ("normed_out", vp), ("norm_eps", C.c_float), ("reserved2", C.c_int32),
                ("peers", C.POINTER(EpPeers))]


MOE_PHASE_ALL, MOE_PHASE_EXPERTS, MOE_PHASE_COMBINE, MOE_PHASE_EXCHANGE = 0, 1, 2, 3
MOE_EP_NO_ZERO_FILL = 1

_SIGS = {
    "glq_version": (C.c_int, []),
    "glq_status_string": (C.c_char_p, [C.c_int]),
    "glq_last_cuda_error": (C.c_int, []),
    "glq_turbo_dequant_matmul": (C.c_int, [vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, vp]),
    "glq_static_scratch_bytes": (C.c_size_t, []),
    "glq_static_scratch_needed": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "glq_turbo_dequant_matmul_static": (C.c_int, [vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, vp]),
    "glq_turbo_dequant_grouped_gemv": (C.c_int, [vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, vp]),
    "glq_gptq_dequant_matmul": (C.c_int, [vp, vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                          C.c_int, vp]),
    "glq_tiled_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "glq_sv_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "glq_rows_f32_count": (C.c_size_t, [C.c_int, C.c_int]),
    "glq_tiled_f16_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "glq_pack_gptq": (C.c_int, [vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, vp, C.c_int, C.c_int, vp]),
    "glq_pack_turbo": (C.c_int, [vp, C.c_int, C.c_int, vp, C.c_int, C.c_int, vp]),
    "glq_pack_rows_f32": (C.c_int, [vp, C.c_int, vp, C.c_int, C.c_int, vp]),
    "glq_pack_sv": (C.c_int, [vp, C.c_int, C.c_int, vp, C.c_int, C.c_int, vp]),
    "glq_pack_f16": (C.c_int, [vp, C.c_long, C.c_long, C.c_int, C.c_int, vp, vp]),
    "glq_dequant_tiled": (C.c_int, [C.c_int, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, vp, vp]),
    "glq_debug_error": (C.c_int, [vp, C.c_int]),
    "glq_add_rmsnorm": (C.c_int, [vp, vp, vp, C.c_float, C.c_int, C.c_int, vp, vp, vp]),
    "glq_attn_decode_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "glq_rope_prefill": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp, vp,
                         C.c_float, vp]),
    "glq_attn_prefill": (C.c_int, [vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp]),
    "glq_attn_decode": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp, vp,
                                  C.c_float, vp, C.c_size_t, vp, C.c_size_t, vp]),
    "glq_lm_head_workspace_bytes": (C.c_size_t, []),
    "glq_lm_head": (C.c_int, [vp, C.c_int64, vp, C.c_int, C.c_int, C.c_int, vp, C.c_int64, vp, vp, C.c_size_t, vp, vp]),
    "glq_rht_forward": (C.c_int, [vp, C.c_int, C.c_int64, vp, C.c_int, C.c_int, C.c_float, vp, C.c_int, C.c_int64, vp]),
    "glq_mm_workspace_bytes": (C.c_size_t, [C.POINTER(MMArgs)]),
    "glq_mm_counters": (C.c_size_t, [C.POINTER(MMArgs)]),
    "glq_grouped_matmul": (C.c_int, [C.POINTER(MMArgs), vp]),
    "glq_linear_counters": (C.c_size_t, [C.c_int, C.c_int, C.POINTER(Weight), C.c_int]),
    "glq_linear_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int, C.POINTER(Weight), C.c_int]),
    "glq_linear_forward": (C.c_int, [C.c_int, C.c_int, C.POINTER(Weight), vp, vp, C.c_int64, vp, vp, C.c_int64,
                                     C.c_int, vp, C.c_size_t, vp, C.c_size_t, vp]),
    "glq_moe_fused_trace": (C.c_int, [vp, C.c_int]),
    "glq_moe_uses_fused_kernel": (C.c_int, [C.POINTER(MoeDesc), C.c_int]),
    "glq_moe_workspace_bytes": (C.c_size_t, [C.POINTER(MoeDesc), C.c_int]),
    "glq_moe_counters": (C.c_size_t, [C.POINTER(MoeDesc), C.c_int]),
    "glq_moe_forward": (C.c_int, [C.POINTER(MoeDesc), vp, C.c_int, vp, vp, vp, vp, vp, C.c_size_t, vp, C.c_size_t, vp,
                                  vp, vp, vp]),
    "glq_moe_forward_ep": (C.c_int, [C.POINTER(MoeDesc), vp, C.c_int, vp, vp, vp, vp, vp, C.c_size_t, vp, C.c_size_t,
                                     vp, vp, vp, vp, C.POINTER(MoeEp)]),
}

_lib = None


def lib():
    """The loaded library; raises RuntimeError when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m glorcq_b200._build` (nvcc, sm_100a). "
                "glorcq_b200 has no CPU or PyTorch fallback.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGS.items():
            if not hasattr(L, name):
                continue
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def exported_symbols():
    return list(_SIGS.keys())


def check(status: int, what: str = "glorcq_b200"):
    if status != 0:
        L = lib()
        msg = L.glq_status_string(status).decode()
        extra = f" (cudaError {L.glq_last_cuda_error()})" if status == -4 else ""
        raise RuntimeError(f"{what}: {msg}{extra}")
