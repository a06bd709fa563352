"""ctypes binding of ``liblmoe.so`` (declared in ``include/lmoe.h``).

Only plain pointers and sizes cross the boundary; tensors are passed as
``data_ptr()``.  Every wrapper raises ``LmoeError`` on a non-zero return code.
There is no fallback: if the library is missing, loading raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liblmoe.so")

BF16, F32, E4M3 = 0, 1, 2
ROW_PAD = 128


class LmoeError(RuntimeError):
    pass


class Shape(Structure):
    _fields_ = [(n, c_int32) for n in ("T", "D", "L", "E", "K", "F", "Fs", "n_shared")]


class Route(Structure):
    _fields_ = [(n, c_void_p) for n in ("counts", "offsets", "perm", "pad_offsets", "pos", "row_src", "tile_expert",
                                        "n_tiles")]


# name -> (restype, argtypes); must list every symbol include/lmoe.h declares
P = c_void_p
SP = POINTER(Shape)
RP = POINTER(Route)
SIGNATURES = {
    "lmoe_version": (c_int, []),
    "lmoe_status_string": (c_char_p, [c_int]),
    "lmoe_launch_count": (c_int64, []),
    "lmoe_profile_enable": (c_int, [c_int]),
    "lmoe_profile_collect": (c_int, [P, P]),
    "lmoe_padded_rows": (c_int64, [SP]),
    "lmoe_route_workspace_bytes": (c_size_t, [SP]),
    "lmoe_pair_gemm_enable": (c_int, [c_int]),
    "lmoe_chain_enable": (c_int, [c_int]),
    "lmoe_chain_applies": (c_int, [c_int, c_int]),
    "lmoe_gemm_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "lmoe_gemm_bf16": (c_int, [c_int, c_int, c_int, P, c_int64, c_int, P, c_int64, c_int, P, c_int64, c_int, c_int, P,
                               c_size_t, P, P]),
    "lmoe_wgrad_workspace_bytes": (c_size_t, [SP]),
    "lmoe_xproj_fwd": (c_int, [SP, P, P, P, P, P, P, P]),
    "lmoe_gate_topk_fwd": (c_int, [SP, P, P, c_float, P, P, P, P, P, P]),
    "lmoe_route_permute": (c_int, [SP, P, RP, P, c_size_t, P]),
    "lmoe_route_permute_static": (c_int, [SP, P, RP, P]),
    "lmoe_experts_fwd": (c_int, [SP, P, P, P, RP, P, P, P, P, P, P]),
    "lmoe_shared_gateup_fwd": (c_int, [SP, P, P, P, P, P, P]),
    "lmoe_combine_out_fwd": (c_int, [SP, P, RP, P, P, P, P, P, P, P]),
    "lmoe_combine_out_bwd_dgrad": (c_int, [SP, P, P, P, P, P, P, P, P, P]),
    "lmoe_combine_out_bwd_wgrad": (c_int, [SP, P, P, P, P, c_int, P, c_size_t, P, P]),
    "lmoe_combine_bwd": (c_int, [SP, P, P, P, RP, P, P, P]),
    "lmoe_swiglu_bwd": (c_int, [c_int64, c_int, P, P, P, c_int64, P, P]),
    "lmoe_experts_bwd_dgrad": (c_int, [SP, P, P, P, P, RP, P, P, P, P, P]),
    "lmoe_experts_bwd_wgrad": (c_int, [SP, P, P, P, P, RP, P, P, P, P]),
    "lmoe_unpermute_sum_bwd": (c_int, [SP, P, RP, P, P]),
    "lmoe_gate_topk_bwd": (c_int, [SP, P, P, P, P, P, P, c_float, P, P]),
    "lmoe_xside_bwd": (c_int, [SP, P, P, P, P, P, P, P, P, P, c_int, P, c_size_t, P, P]),
    "lmoe_grouped_fwd": (c_int, [c_int64, c_int, c_int, c_int, P, P, P, P, P, P, P, P, P, P, P]),
    "lmoe_grouped_bwd_dgrad": (c_int, [c_int64, c_int, c_int, c_int, P, P, P, P, P, P, P, P, P, P, P, P]),
    "lmoe_grouped_bwd_wgrad": (c_int, [c_int64, c_int, c_int, c_int, P, P, P, P, P, P, P, P, P]),
    "lmoe_grouped_rows_bf16": (c_int, [c_int64, c_int, c_int, c_int, P, P, c_int, P, P, P, P, P]),
    "lmoe_grouped_wgrad_bf16": (c_int, [c_int64, c_int, c_int, c_int, P, P, P, P, P, P]),
    "lmoe_gather_rows": (c_int, [P, P, c_int, c_int64, c_int, P, P, P]),
    "lmoe_combine_rows": (c_int, [P, P, P, c_int, c_int, c_int, P, c_int64, P]),
    "lmoe_combine_bwd_rows": (c_int, [P, P, P, P, c_int64, c_int, c_int, P, P, P, P]),
    "lmoe_invert_perm": (c_int, [P, c_int64, P, P]),
    "lmoe_ep_plan": (c_int, [P, c_int, c_int, c_int, P, P, P, P, P, P]),
    "lmoe_ep_tables": (c_int, [P, c_int, c_int, c_int, c_int64, P, P, P, P, P, P, P, P]),
    "lmoe_ep_zero_pads": (c_int, [P, c_int, P, P, P, c_int, c_int, c_int, P]),
    "lmoe_ep_dispatch": (c_int, [P, P, P, P, P, c_int64, c_int, c_int, c_int, c_int, c_int64, P, P, P]),
    "lmoe_ep_dispatch_bwd": (c_int, [P, P, P, P, P, P, P, c_int64, c_int, c_int, c_int, c_int, c_int64, P, P, P, P]),
    "lmoe_ep_return": (c_int, [P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int64, P, P]),
    "lmoe_combine_rows_add": (c_int, [P, P, P, P, c_int64, c_int, c_int, c_int, P, c_int64, P]),
    "lmoe_gemm_swiglu_bf16": (c_int, [c_int, c_int, c_int, P, c_int64, P, c_int64, P, c_int64, P, c_int64, P, P]),
    "lmoe_grouped_fwd_gather": (c_int, [c_int64, c_int, c_int, c_int, P, c_int64, P, c_int, c_int, c_int64, P, P, P, P, P,
                                         P, P, P, P]),
    "lmoe_grouped_bwd_wgrad_gather": (c_int, [c_int64, c_int, c_int, c_int, P, c_int64, P, c_int, c_int, c_int64, P, P, P,
                                               P, P, P, P, P]),
    "lmoe_epd_send": (c_int, [P, P, P, P, P, P, c_int64, c_int, c_int, c_int, c_int, c_int, c_int64, c_int64, P, P, P, P,
                               P, P]),
    "lmoe_epd_gather": (c_int, [P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int64, c_int64, P, P, P, P]),
    "lmoe_epd_reduce_return": (c_int, [P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int64, c_int64, P, P,
                                        P]),
    "lmoe_epd_sum": (c_int, [P, P, c_int64, c_int, c_int, c_int, c_int, c_int64, P, c_int64, P]),
    "lmoe_ep_flag_barrier": (c_int, [P, P, c_int, c_int, P, P]),
    "lmoe_fp8_quantize": (c_int, [P, c_int64, c_int, P, P, P, P, P]),
    "lmoe_gemm_fp8": (c_int, [c_int, c_int, c_int, P, c_int64, c_int, P, c_int64, c_int, P, P, P, c_int64, P, P]),
    "lmoe_grouped_gateup_fp8": (c_int, [c_int64, c_int, c_int, c_int, P, P, P, P, P, P, P, P, P, P]),
    "lmoe_grouped_rows_fp8": (c_int, [c_int64, c_int, c_int, c_int, P, P, c_int, P, P, P, P, P, P, P]),
    "lmoe_grouped_wgrad_fp8": (c_int, [c_int64, c_int, c_int, c_int, P, P, P, P, P, P, P, P]),
    "lmoe_rmsnorm_workspace_bytes": (c_size_t, [c_int]),
    "lmoe_rmsnorm_fwd": (c_int, [P, P, c_float, c_int64, c_int, P, P, P]),
    "lmoe_add_bf16": (c_int, [P, P, P, c_int64, P]),
    "lmoe_rmsnorm_bwd": (c_int, [P, P, P, P, P, c_int64, c_int, P, P, P, c_size_t, P]),
    "lmoe_router_bias_update": (c_int, [SP, P, c_float, P, P, P]),
    "lmoe_cast_f32_to_bf16": (c_int, [P, P, c_int64, P]),
    "lmoe_cast_bf16_to_f32": (c_int, [P, P, c_int64, P]),
}

_lib: Optional[ctypes.CDLL] = None


def load() -> ctypes.CDLL:
    """Loads the library (once).  torch is imported first so that the CUDA runtime it bundles is
    the one the library binds to."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise LmoeError(
            f"{LIB_PATH} is missing: build it with `python -m swamla_b200.build` "
            "(there is no CPU or PyTorch fallback for this path)")
    import torch  # noqa: F401  (loads libcudart)
    lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the export is missing
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def status_string(code: int) -> str:
    return load().lmoe_status_string(int(code)).decode()


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        raise LmoeError(f"{what or 'lmoe call'} failed with code {rc}: {status_string(rc)}")


def ptr(t) -> Optional[int]:
    """Device pointer of a torch tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def call(name: str, *args) -> None:
    check(getattr(load(), name)(*args), name)
