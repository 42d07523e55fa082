"""ctypes binding of libmoe_b200.so (the C ABI declared in include/moe_b200.h).

The library is the product: there is no Python or CPU fallback behind it. If it is missing and
cannot be built, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint8, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
# MOE_B200_LIB points at another build of the same library (A/B comparisons of kernel variants)
LIB_PATH = os.environ.get("MOE_B200_LIB") or os.path.join(_HERE, "libmoe_b200.so")

STATUS_NAMES = {
    0: "OK", 1: "INVALID_ARGUMENT", 2: "CUDA_ERROR", 3: "WORKSPACE_TOO_SMALL", 4: "DEVICE_TIMEOUT",
    5: "NOT_REGISTERED", 6: "DRIVER_ENTRY_POINT", 7: "TOO_LARGE",
}
ACT_CODES = {"silu": 0, "swigluoai": 1}


class MoeB200Error(RuntimeError):
    """A libmoe_b200 entry point returned a non-zero status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"libmoe_b200: {STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        try:
            from . import build as _build
            _build.build()
        except Exception as e:  # noqa: BLE001
            raise RuntimeError(
                f"{LIB_PATH} is missing and could not be built ({e}). "
                "Run `python layered-prefill_b200/build.py` on a machine with nvcc 12.8+."
            ) from e
    return ctypes.CDLL(LIB_PATH)


lib = _load()

# name -> (restype, argtypes); every symbol of include/moe_b200.h
SIGNATURES = {
    "moe_b200_last_error": (c_char_p, []),
    "moe_b200_abi_version": (c_int, []),
    "moe_b200_block_m": (c_int, []),
    "moe_b200_launch_count": (ctypes.c_uint64, []),
    "moe_b200_grouped_gemm_gate_up": (c_int, [c_void_p] * 7 + [c_int] * 7 + [c_void_p, c_void_p]),
    "moe_b200_grouped_gemm_down": (c_int, [c_void_p, c_int] + [c_void_p] * 7 + [c_int] * 5 + [c_void_p, c_void_p]),
    "moe_b200_rms_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p]),
    "moe_b200_add_rms_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p]),
    "moe_b200_pre_moe_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "moe_b200_add_rms_norm_router": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 5 + [c_void_p, c_size_t, c_void_p, c_void_p]),
    "moe_b200_topk_softmax": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "moe_b200_align_workspace_bytes": (c_size_t, [c_int, c_int]),
    "moe_b200_moe_align_block_size": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_size_t, c_void_p]),
    "moe_b200_moe_align_static_scratch_bytes": (c_size_t, []),
    "moe_b200_moe_align_block_size_static": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p]),
    "moe_b200_silu_and_mul": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "moe_b200_swigluoai_and_mul": (c_int, [c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_void_p]),
    "moe_b200_moe_sum": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "moe_b200_fused_experts_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "moe_b200_fused_experts": (c_int, [c_void_p] * 8 + [c_int] * 6 + [c_void_p, c_size_t, c_void_p, c_void_p]),
    "moe_b200_fused_experts_fp8_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "moe_b200_fused_experts_fp8": (c_int, [c_void_p, c_void_p, POINTER(c_float), c_void_p, POINTER(c_float), c_void_p, c_void_p, c_void_p] + [c_int] * 5 + [c_void_p, c_size_t, c_void_p, c_void_p]),
    "moe_b200_fused_experts_fp8_tp": (c_int, [c_void_p, c_void_p, POINTER(c_float), c_void_p, POINTER(c_float), c_void_p, c_void_p, c_void_p] + [c_int] * 7 + [c_void_p, c_size_t, c_void_p, c_void_p]),
    "moe_b200_fused_experts_fp8_tp_reduce": (c_int, [c_void_p, c_void_p, POINTER(c_float), c_void_p, POINTER(c_float), c_void_p, c_void_p, c_void_p] + [c_int] * 7 + [c_void_p, c_size_t, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "moe_b200_quant_fp8_per_token_group": (c_int, [c_void_p, c_int, c_int, c_void_p, POINTER(c_float), c_void_p]),
    "moe_b200_fused_moe_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "moe_b200_fused_moe_forward": (c_int, [c_void_p, c_void_p, c_int] + [c_void_p] * 7 + [c_int] * 7 + [c_void_p, c_size_t, c_void_p, c_void_p]),
    "moe_b200_read_status": (c_int, [c_void_p, POINTER(c_int32), c_void_p]),
    "moe_b200_ar_meta_size": (c_int64, []),
    "moe_b200_ar_allocate_shared_buffer": (c_int, [c_int64, POINTER(c_int64), POINTER(c_uint8)]),
    "moe_b200_ar_open_mem_handle": (c_int, [POINTER(c_uint8), POINTER(c_int64)]),
    "moe_b200_ar_close_mem_handle": (c_int, [c_int64]),
    "moe_b200_ar_free_shared_buffer": (c_int, [c_int64]),
    "moe_b200_ar_init": (c_int, [POINTER(c_int64), c_int, c_void_p, c_int64, c_int, c_int, POINTER(c_int64)]),
    "moe_b200_ar_dispose": (c_int, [c_int64]),
    "moe_b200_ar_register_buffer": (c_int, [c_int64, POINTER(c_int64)]),
    "moe_b200_ar_register_fused_buffer": (c_int, [c_int64, POINTER(c_int64), c_int64]),
    "moe_b200_ar_register_ll_buffer": (c_int, [c_int64, POINTER(c_int64), c_int64]),
    "moe_b200_ar_all_reduce": (c_int, [c_int64, c_void_p, c_void_p, c_int64, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "moe_b200_ar_moe_sum_all_reduce": (c_int, [c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "moe_b200_ar_all_reduce_add_rms_norm": (c_int, [c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "moe_b200_ar_moe_sum_all_reduce_add_rms_norm": (c_int, [c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "moe_b200_fused_moe_forward_tp_add_rms_norm": (c_int, [c_void_p, c_void_p, c_int] + [c_void_p] * 6 + [c_float, c_void_p, c_void_p] + [c_int] * 7 + [c_void_p, c_size_t, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "moe_b200_ar_set_wait_limit_ns": (c_int, [c_int64, ctypes.c_uint64]),
    "moe_b200_ar_wait_probe": (c_int, [c_int64, ctypes.c_uint64, c_void_p, c_void_p]),
    "moe_b200_ar_graph_buffer_count": (c_int, [c_int64, POINTER(c_int)]),
    "moe_b200_ar_get_graph_buffer_ipc_meta": (c_int, [c_int64, POINTER(c_uint8), POINTER(c_int64), c_int]),
    "moe_b200_ar_register_graph_buffers": (c_int, [c_int64, POINTER(c_uint8), POINTER(c_int64), c_int]),
    "moe_b200_fused_moe_forward_tp": (c_int, [c_void_p, c_void_p, c_int] + [c_void_p] * 5 + [c_int] * 7 + [c_void_p, c_size_t, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    return lib.moe_b200_last_error().decode()


def check(status: int) -> None:
    if status != 0:
        raise MoeB200Error(status, last_error())
