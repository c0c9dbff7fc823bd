"""ctypes binding of ``libmmoe_b200.so`` (declared in ``include/mmoe.h``).

The library is the product: there is no Python or CPU stand-in for any of its kernels.  If it is missing every operator
of the package raises :class:`RuntimeError` telling how to build it.  Status codes of the C ABI are mapped onto the
exception classes the reference raises for the same conditions (``backend/frontend.py:67-69,261-270,402-418``).
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

_LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_lib", "libmmoe_b200.so")

MMOE_OK = 0
MMOE_ERR_INVALID_ARGUMENT = 1
MMOE_ERR_UNSUPPORTED = 2
MMOE_ERR_CUDA = 3
MMOE_ERR_ARCH = 4
MMOE_ERR_NOT_PREPARED = 5
MMOE_ERR_DEVICE_TIMEOUT = 6

ENGINE_TENSOR_CORE = 0
ENGINE_SCALAR_VALIDATION = 1

#: every symbol ``include/mmoe.h`` declares
EXPORTED_SYMBOLS = (
    "mmoe_layout", "mmoe_block_m", "mmoe_prepare", "mmoe_stage_inputs", "mmoe_dispatch_count", "mmoe_dispatch_pack",
    "mmoe_dispatch_place", "mmoe_experts", "mmoe_combine", "mmoe_forward", "mmoe_read_status", "mmoe_status_string",
    "mmoe_last_error", "mmoe_abi_version", "mmoe_set_tuning", "mmoe_route_order_noalloc", "mmoe_ep_dispatch", "mmoe_ep_return",
    "mmoe_experts_ep_return", "mmoe_forward_ep", "mmoe_transform_weights",
    "mmoe_plan_shared", "mmoe_experts_select", "mmoe_route_stage_inputs", "mmoe_stage_inputs_nvfp4",
    "mmoe_combine_residual",
)


class MmoeGeometry(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in (
        "num_ranks", "rank", "num_experts", "num_topk", "hidden", "intermediate", "num_shared_experts",
        "num_max_tokens")]


_LAYOUT_FIELDS = (
    "total_bytes", "x", "x_sf", "topk_idx", "topk_weights", "shared_x_sf", "shared_sf_rows", "send_count",
    "send_offset", "route_pos", "sorted_route", "sort_scratch", "recv_count", "plan", "send_x", "send_sf", "send_w",
    "recv_x", "recv_sf", "recv_w", "pool_x", "pool_sf", "pool_w", "pool_dst", "act_x", "act_sf", "shared_act_x",
    "shared_act_sf", "ret", "ret_recv", "shared_out", "ep_sync", "status", "pool_rows", "pool_sf_rows", "max_routes", "max_tiles")


class MmoeLayout(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in _LAYOUT_FIELDS]


class MmoeWeights(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in (
        "w13", "w13_sf", "w2", "w2_sf", "shared_w13", "shared_w13_sf", "shared_w2", "shared_w2_sf")] + [
        ("w13_slice_stride", ctypes.c_int64), ("w2_slice_stride", ctypes.c_int64)]


class MmoeOptions(ctypes.Structure):
    _fields_ = [("activation_clamp", ctypes.c_float), ("fast_math", ctypes.c_int32), ("engine", ctypes.c_int32),
                ("timeout_ms", ctypes.c_int32), ("layer_mask", ctypes.c_int32), ("residual", ctypes.c_void_p)]


_lib: Optional[ctypes.CDLL] = None


def library_path() -> str:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    """Load the CUDA library (once).  Raises ``RuntimeError`` when it has not been built: there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise RuntimeError(
            f"{_LIB_PATH} is missing: build it with `python vllm_plugin_b200/csrc/build.py` (nvcc, sm_100a). "
            "The MegaMoE backend has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(_LIB_PATH)
    vp, i32 = ctypes.c_void_p, ctypes.c_int32
    geo_p = ctypes.POINTER(MmoeGeometry)
    lib.mmoe_layout.argtypes = [geo_p, ctypes.POINTER(MmoeLayout)]
    lib.mmoe_block_m.argtypes = [i32, i32, i32, i32]
    lib.mmoe_prepare.argtypes = [geo_p, ctypes.POINTER(i32), i32, ctypes.POINTER(i32), vp]
    lib.mmoe_stage_inputs.argtypes = [geo_p, vp, vp, vp, i32, vp, vp, i32, i32, vp]
    lib.mmoe_route_stage_inputs.argtypes = [geo_p, vp, vp, vp, i32, vp, vp, i32, vp, i32, i32, vp]
    lib.mmoe_stage_inputs_nvfp4.argtypes = [vp, ctypes.c_float, vp, vp, i32, i32, vp]
    lib.mmoe_dispatch_count.argtypes = [geo_p, vp, i32, vp]
    lib.mmoe_dispatch_pack.argtypes = [geo_p, vp, i32, vp]
    lib.mmoe_dispatch_place.argtypes = [geo_p, vp, i32, i32, vp, vp]
    lib.mmoe_experts.argtypes = [geo_p, vp, ctypes.POINTER(MmoeWeights), ctypes.POINTER(MmoeOptions), i32, i32, vp]
    lib.mmoe_combine.argtypes = [geo_p, vp, vp, i32, vp]
    lib.mmoe_combine_residual.argtypes = [geo_p, vp, vp, vp, i32, vp]
    lib.mmoe_forward.argtypes = [geo_p, vp, ctypes.POINTER(MmoeWeights), ctypes.POINTER(MmoeOptions), vp, i32, i32, vp, vp]
    lib.mmoe_read_status.argtypes = [geo_p, vp, ctypes.POINTER(i32), vp]
    lib.mmoe_status_string.argtypes = [i32]
    lib.mmoe_status_string.restype = ctypes.c_char_p
    lib.mmoe_last_error.argtypes = []
    lib.mmoe_last_error.restype = ctypes.c_char_p
    lib.mmoe_abi_version.argtypes = []
    lib.mmoe_set_tuning.argtypes = [i32, i32]
    lib.mmoe_ep_dispatch.argtypes = [geo_p, vp, ctypes.POINTER(vp), i32, ctypes.POINTER(MmoeOptions), vp]
    lib.mmoe_ep_return.argtypes = [geo_p, vp, ctypes.POINTER(vp), ctypes.POINTER(MmoeOptions), vp]
    lib.mmoe_forward_ep.argtypes = [geo_p, vp, ctypes.POINTER(vp), ctypes.POINTER(MmoeWeights), ctypes.POINTER(MmoeOptions),
                                    vp, i32, i32, vp, vp]
    lib.mmoe_plan_shared.argtypes = [geo_p, vp, i32, i32, vp]
    lib.mmoe_experts_select.argtypes = [geo_p, vp, ctypes.POINTER(MmoeWeights), ctypes.POINTER(MmoeOptions), i32, i32, i32, vp]
    lib.mmoe_transform_weights.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]
    lib.mmoe_experts_ep_return.argtypes = [geo_p, vp, ctypes.POINTER(vp), ctypes.POINTER(MmoeWeights),
                                           ctypes.POINTER(MmoeOptions), i32, i32, vp]
    lib.mmoe_route_order_noalloc.argtypes = [vp, i32, i32, i32, vp, vp, vp, vp, vp]
    for name in EXPORTED_SYMBOLS:
        fn = getattr(lib, name)
        if fn.restype is not ctypes.c_char_p:
            fn.restype = ctypes.c_int
    _lib = lib
    return lib


def check(code: int) -> None:
    """Raise the exception class the reference uses for the failed condition."""
    if code == MMOE_OK:
        return
    lib = load()
    detail = lib.mmoe_last_error().decode() or lib.mmoe_status_string(code).decode()
    if code == MMOE_ERR_INVALID_ARGUMENT:
        raise AssertionError(detail)
    if code == MMOE_ERR_UNSUPPORTED:
        raise NotImplementedError(detail)
    raise RuntimeError(f"{lib.mmoe_status_string(code).decode()}: {detail}")


def layout_of(geo: MmoeGeometry) -> MmoeLayout:
    lay = MmoeLayout()
    check(load().mmoe_layout(ctypes.byref(geo), ctypes.byref(lay)))
    return lay
