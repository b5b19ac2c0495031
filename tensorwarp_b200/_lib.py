"""ctypes view of the C ABI declared in ``include/twmarlin.h``.

Loading fails loudly: there is no Python or CPU stand-in for any entry point.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
# TWMARLIN_LIB points at another build of the same library (e.g. one compiled with other tuning macros)
LIB_PATH = os.environ.get("TWMARLIN_LIB", os.path.join(PKG, "libtwmarlin.so"))

TWM_OK, TWM_EINVAL, TWM_EALIGN, TWM_EWORKSPACE, TWM_ELAUNCH, TWM_EARCH, TWM_ETIMEOUT = 0, -1, -2, -3, -4, -5, -6
TWM_F32, TWM_F16 = 0, 1
TWM_KERNEL_AUTO, TWM_KERNEL_SIMT, TWM_KERNEL_TC, TWM_KERNEL_MMA, TWM_KERNEL_TCW, TWM_KERNEL_TCR = 0, 1, 2, 3, 4, 5
TWM_FLAG_PDL, TWM_FLAG_ACCUMULATE, TWM_FLAG_INDEPENDENT = 1, 2, 4
TWM_A_PLAIN, TWM_A_SILU_MUL, TWM_A_GEGLU = 0, 1, 2


class GemmArgs(C.Structure):
    """``twm_gemm_args``."""
    _fields_ = [
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
        ("group_size", C.c_int),
        ("a_dtype", C.c_int), ("c_dtype", C.c_int),
        ("a", C.c_void_p), ("lda", C.c_long),
        ("packed", C.c_void_p), ("scales", C.c_void_p),
        ("c", C.c_void_p), ("ldc", C.c_long),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("splits_override", C.c_int), ("kernel_override", C.c_int), ("flags", C.c_int),
        ("packed_offsets", C.c_void_p), ("scales_offsets", C.c_void_p), ("expert_idx", C.c_int),
        ("comm", C.c_void_p),
        ("a_prologue", C.c_int),
        ("next", C.c_void_p),
    ]


class Comm(C.Structure):
    """``twm_comm``."""
    _fields_ = [("n_ranks", C.c_int), ("rank", C.c_int), ("slot_elems", C.c_long),
                ("data", C.c_void_p * 8), ("flags", C.c_void_p * 8), ("state", C.c_void_p),
                ("wait_ns", C.c_ulonglong)]


class MoeArgs(C.Structure):
    """``twm_moe_args``."""
    _fields_ = [("top_k", C.c_int), ("N", C.c_int), ("K", C.c_int), ("group_size", C.c_int),
                ("a", C.c_void_p), ("a_slot_stride", C.c_long), ("a_prologue", C.c_int),
                ("packed_base", C.c_void_p), ("scales_base", C.c_void_p),
                ("packed_bytes_per_expert", C.c_size_t), ("scales_per_expert", C.c_size_t),
                ("topk_ids", C.c_void_p), ("topk_weights", C.c_void_p),
                ("c", C.c_void_p), ("c_dtype", C.c_int), ("c_slot_stride", C.c_long),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("flags", C.c_int)]


class ChainOp(C.Structure):
    """``twm_chain_op``."""
    _fields_ = [("gemm", GemmArgs)]


class ChainInfo(C.Structure):
    """``twm_chain_info_t``."""
    _fields_ = [("count", C.c_int), ("grid", C.c_int), ("rows", C.c_int), ("device_bytes", C.c_size_t),
                ("split_tiles", C.c_int), ("max_pieces", C.c_int)]


class Plan(C.Structure):
    """``twm_plan_t``."""
    _fields_ = [
        ("kernel", C.c_int), ("n_tile", C.c_int), ("splits", C.c_int), ("blocks_per_split", C.c_int),
        ("grid_x", C.c_int), ("grid_y", C.c_int), ("workspace_bytes", C.c_size_t), ("cluster_reduce", C.c_int),
    ]


# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "twm_plan": (C.c_int, [C.c_int] * 7 + [C.POINTER(Plan)]),
    "twm_workspace_bytes": (C.c_size_t, [C.c_int] * 4),
    "twm_gemm_w4a16": (C.c_int, [C.POINTER(GemmArgs), C.c_void_p]),
    "twm_gemm_w4a16_static_ws": (C.c_int, [C.POINTER(GemmArgs), C.c_void_p]),
    "twm_static_ws_capacity": (C.c_size_t, []),
    "twm_moe_workspace_bytes": (C.c_size_t, [C.c_int] * 4),
    "twm_moe_gate_up": (C.c_int, [C.POINTER(MoeArgs), C.c_void_p]),
    "twm_moe_down_axpy": (C.c_int, [C.POINTER(MoeArgs), C.c_void_p]),
    "twm_chain_create": (C.c_int, [C.POINTER(ChainOp), C.c_int, C.POINTER(C.c_void_p)]),
    "twm_chain_launch": (C.c_int, [C.c_void_p, C.c_void_p]),
    "twm_chain_info": (C.c_int, [C.c_void_p, C.POINTER(ChainInfo)]),
    "twm_chain_destroy": (C.c_int, [C.c_void_p]),
    "twm_chain_partition": (C.c_int, [C.c_int] * 5 + [C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "twm_dequant": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "twm_quantize_pack": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "twm_reorder_to_tw_marlin": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "twm_fuse_n": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.c_int, C.c_int,
                             C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "twm_slice_n": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                              C.c_void_p, C.c_void_p]),
    "twm_slice_k_offsets": (C.c_int, [C.c_int] * 5 + [C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "twm_device_error": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint)]),
    "twm_comm_bytes": (C.c_size_t, [C.c_int, C.c_long]),
    "twm_comm_layout": (C.c_int, [C.c_void_p, C.c_int, C.c_long, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                  C.POINTER(C.c_void_p)]),
    "twm_allreduce_add_rmsnorm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float,
                                            C.c_int, C.c_void_p]),
    "twm_ipc_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "twm_ipc_free": (C.c_int, [C.c_void_p]),
    "twm_ipc_get_handle": (C.c_int, [C.c_void_p, C.c_char_p]),
    "twm_ipc_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "twm_ipc_close": (C.c_int, [C.c_void_p]),
    # include/twm_decode.h
    "twm_embed": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "twm_rmsnorm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p]),
    "twm_add_rmsnorm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_int,
                                  C.c_void_p]),
    "twm_rope_append": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                  C.c_int, C.c_void_p, C.c_int, C.c_float, C.c_int, C.c_void_p]),
    "twm_attn_scratch_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "twm_attn_decode": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                  C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]),
    "twm_rope_table": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_int, C.c_void_p]),
    "twm_attn_decode_rope": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                       C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.c_int,
                                       C.c_void_p]),
    "twm_silu_mul": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "twm_lm_head": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "twm_argmax_scratch_bytes": (C.c_size_t, []),
    "twm_argmax_advance": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                     C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]),
    "twm_status_string": (C.c_char_p, [C.c_int]),
    "twm_last_error": (C.c_char_p, []),
    "twm_version": (C.c_char_p, []),
}

_lib = None


def lib() -> C.CDLL:
    """Load ``libtwmarlin.so`` (built by ``tensorwarp_b200.build``) and bind every entry point."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: run `python -m tensorwarp_b200.build` (needs nvcc). "
                "There is no fallback path.")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)   # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


class TwmError(RuntimeError):
    """A non-zero ``twm_status``; mirrors ``DeviceError`` on the reference's side."""

    def __init__(self, status: int, where: str):
        self.status = status
        l = lib()
        detail = l.twm_last_error().decode() if status == TWM_ELAUNCH else ""
        super().__init__(f"{where}: {l.twm_status_string(status).decode()}" + (f" [{detail}]" if detail else ""))


def check(status: int, where: str) -> None:
    if status != TWM_OK:
        raise TwmError(status, where)
