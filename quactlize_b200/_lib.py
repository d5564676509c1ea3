"""ctypes binding of libquactlize_b200.so (the C-ABI device library).  There is no fallback: if the library is missing
or a symbol does not resolve, importing an op raises."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# QUACTLIZE_B200_LIB selects another build of the same library (as QUACTLIZE_PPU_LIB does for the reference loader)
LIB_PATH = os.environ.get("QUACTLIZE_B200_LIB") or os.path.join(_HERE, "csrc", "libquactlize_b200.so")
_lib = None

P, I, I64 = C.c_void_p, C.c_int, C.c_int64


class ConfigV2(C.Structure):
    _fields_ = [("enable_cuda_kernel", C.c_bool), ("name", C.c_char_p), ("tile_m", C.c_int32), ("tile_n", C.c_int32),
                ("tile_k", C.c_int32), ("warp_m", C.c_int32), ("warp_n", C.c_int32), ("stages", C.c_int32)]


# name -> (restype, argtypes)
SIGNATURES = {
    "quactlize_ppu_vecdot": (I, [P, I64, P, P, I, I, I]),
    "quactlize_ppu_vecdot_dense": (I, [P, I64, P, P, I, I, I]),
    "quactlize_ppu_vecdot_dense_dev_v1": (I, [P, I64, P, P, I, I, I, P]),
    "quactlize_ppu_vecdot_moe": (I, [P, I64, P, P, P, I, I, I, I, I, I]),
    "quactlize_ppu_vecdot_moe_config_v1": (I, [P, I64, P, P, P, I, I, I, I, I, I, C.c_char_p]),
    "quactlize_ppu_vecdot_moe_config_valid_v1": (C.c_int32, [I, I, I, I, I, I, I, C.c_char_p]),
    "quactlize_ppu_list_valid_vecdot_moe_configs_v2": (C.c_int32, [P, C.c_int32, I, I, I, I, I, I, I]),
    "quactlize_ppu_dequantize": (I, [P, I64, P, I, I]),
    "quactlize_ppu_prepass": (I, [P, I64, P, P, I, P, P, I, I, I]),
    "quactlize_ppu_prepass_unit": (I, [P, P, P, I, I, I, I, I]),
    "quactlize_b200_vecdot_dev_v1": (I, [P, I64, P, P, I, I, I, P]),
    "quactlize_b200_vecdot_dense2_dev_v1": (I, [P, I, P, I, I64, P, P, P, I, I, P]),
    "quactlize_b200_vecdot_rows_dev_v1": (I, [P, I64, P, P, I, I, I, I, I, P]),
    "quactlize_b200_vecdot_moe_dev_v1": (I, [P, I64, P, P, P, I, I, I, I, I, I, P]),
    "quactlize_b200_dequantize_dev_v1": (I, [P, I64, P, I, I, P]),
    "quactlize_b200_prepass_unit_dev_v1": (I, [P, P, P, I, I, I, I, I, P]),
    "quactlize_ppu_gemv_lowbit": (I, [P, P, P, P, P, P, I, I, I, I, I, I, P, I]),
    "quactlize_ppu_gemv_lowbit_config_v1": (I, [P, P, P, P, P, P, I, I, I, I, I, C.c_char_p]),
    "quactlize_ppu_gemv_lowbit_config_valid_v1": (C.c_int32, [I, I, I, I, I, C.c_char_p]),
    "quactlize_ppu_gemv_lowbit_dev_v1": (I, [P, P, P, P, P, P, I, I, I, I, I, P, C.c_char_p]),
    "quactlize_ppu_bc_gemv": (I, [P, P, P, P, P, P, I, I, I, I, I, I]),
    "quactlize_ppu_bc_gemv_dev_v1": (I, [P, P, P, P, P, P, I, I, I, I, I, I, P]),
    "quactlize_b200_gemv_lowbit_moe_dev_v1": (I, [P, P, P, P, P, P, I, I, I, I, I, I, P, I, P]),
    "quactlize_b200_gemv_plane_dev_v1": (I, [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, P, I, P]),
    "quactlize_ppu_list_configs": (C.c_int32, [P]),
    "quactlize_ppu_list_grouped_configs": (C.c_int32, [P]),
    "quactlize_ppu_list_valid_dense_lowbit_configs_v2": (C.c_int32, [P, C.c_int32, I, I, I, I, I]),
    "quactlize_ppu_list_valid_dense_fully_quantized_configs_v2": (C.c_int32, [P, C.c_int32, I, I, I, I, I]),
    "quactlize_ppu_list_valid_grouped_fully_quantized_configs_v2": (C.c_int32, [P, C.c_int32, I, I, I, I, I, I, I]),
    "quactlize_ppu_dense_lowbit_config_valid_v1": (C.c_int32, [I, I, I, I, I, C.c_char_p]),
    "quactlize_ppu_dense_fully_quantized_config_valid_v1": (C.c_int32, [I, I, I, I, I, C.c_char_p]),
    "quactlize_ppu_grouped_lowbit_config_valid_v1": (C.c_int32, [I, I, I, I, I, I, I, C.c_char_p]),
    "quactlize_ppu_grouped_fully_quantized_config_valid_v1": (C.c_int32, [I, I, I, I, I, I, I, C.c_char_p]),
    "quactlize_ppu_dense_lowbit": (I, [P, P, P, P, P, P, I, I, I, I, I]),
    "quactlize_ppu_dense_lowbit_config_v1": (I, [P, P, P, P, P, P, I, I, I, I, I, C.c_char_p]),
    "quactlize_ppu_dense_fully_quantized": (I, [P, P, P, P, P, I, I, I, I]),
    "quactlize_ppu_dense_fully_quantized_config_v1": (I, [P, P, P, P, P, I, I, I, I, C.c_char_p]),
    "quactlize_ppu_dense_fully_quantized_workspace_bytes_v1": (I64, [I, I, I, I]),
    "quactlize_ppu_dense_fully_quantized_dev_v1": (I, [P, P, P, P, P, I, I, I, I, P, I64, P]),
    "quactlize_ppu_dense_fully_quantized_dev_v2": (I, [P, P, P, P, P, I, I, I, I, P, I64, P, C.c_char_p]),
    "quactlize_ppu_grouped_lowbit": (I, [P, P, P, P, P, P, I, I, I, I, I, I]),
    "quactlize_ppu_grouped_lowbit_config_v1": (I, [P, P, P, P, P, P, I, I, I, I, I, I, C.c_char_p]),
    "quactlize_ppu_grouped_lowbit_workspace_bytes_v1": (I64, [I, I, I, I, I, I]),
    "quactlize_ppu_grouped_lowbit_dev_v1": (I, [P, P, P, P, P, P, I, I, I, I, I, I, I, P, I64, P]),
    "quactlize_ppu_grouped_lowbit_dev_v2": (I, [P, P, P, P, P, P, I, I, I, I, I, I, I, P, I64, P, C.c_char_p]),
    "quactlize_ppu_grouped_fully_quantized": (I, [P, P, P, P, P, P, I, I, I, I, I]),
    "quactlize_ppu_grouped_fully_quantized_config_v1": (I, [P, P, P, P, P, P, I, I, I, I, I, C.c_char_p]),
    "quactlize_ppu_grouped_fully_quantized_workspace_bytes_v1": (I64, [I, I, I, I, I]),
    "quactlize_ppu_grouped_fully_quantized_dev_v1": (I, [P, P, P, P, P, P, I, I, I, I, I, I, P, I64, P]),
    "quactlize_ppu_grouped_fully_quantized_dev_v2": (I, [P, P, P, P, P, P, I, I, I, I, I, I, P, I64, P, C.c_char_p]),
    "quactlize_b200_gemm_plane_dev_v1": (I, [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, P]),
    "quactlize_b200_gemm_plane_dev_v2": (I, [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, P, P]),
    "quactlize_b200_peer_alloc": (I, [C.c_longlong, C.POINTER(C.c_void_p), C.c_char_p]),
    "quactlize_b200_peer_open": (I, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "quactlize_b200_peer_close": (I, [P]),
    "quactlize_b200_peer_free": (I, [P]),
    "quactlize_b200_ep_count_dev_v1": (I, [P, I, I, P, P]),
    "quactlize_b200_ep_plan_dev_v1": (I, [P, P, I, I, I, I, I, P, P, P, P, P, P]),
    "quactlize_b200_ep_dispatch_dev_v1": (I, [P, P, P, P, P, P, I, I, I, P]),
    "quactlize_b200_ep_return_addr_dev_v1": (I, [P, P, I, P, I, I, P, P]),
    "quactlize_b200_ep_combine_dev_v1": (I, [P, P, P, P, I, I, I, P]),
    "quactlize_b200_ep_sync_bytes": (I, [I, I]),
    "quactlize_b200_ep_sync_dev_v1": (I, [P, I, I, I, P, I, P]),
    "quactlize_b200_silu_mul_dev_v1": (I, [P, P, P, I, I, P]),
    "quactlize_b200_gemm_plane_splitk_workspace_bytes_v1": (I64, [I, I, I]),
    "quactlize_b200_gemm_plane_splitk_dev_v1": (I, [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, I, P, I64, P]),
    "quactlize_b200_dense_fully_quantized_static_v1": (I, [P, P, P, P, P, I, I, I, I, P]),
    "quactlize_ppu_units_bytes": (I64, [I, I, I]),
    "quactlize_ppu_prepare_units": (I, [P, P, I, I, I]),
    "quactlize_ppu_prepare_units_grouped": (I, [P, P, I, I, I, I]),
    "quactlize_ppu_prepare_fully_quantized_v1": (I, [P, P, P, P, I, I, I, I]),
    "quactlize_ppu_recover_fully_quantized_v1": (I, [P, P, P, P, I, I, I, I]),
    "quactlize_ppu_prepare_dense": (I, [P, P, P, P, I, I, I]),
    "quactlize_ppu_recover_dense": (I, [P, P, P, P, I, I, I]),
    "quactlize_ppu_prepare_dense_for_tile": (I, [P, P, P, P, I, I, I, I]),
    "quactlize_ppu_recover_dense_for_tile": (I, [P, P, P, P, I, I, I, I]),
    "quactlize_b200_prepare_gemv": (I, [P, P, P, P, P, I, I, I, I]),
    "quactlize_b200_pack_units": (I, [P, P, I, I, I, I]),
    "quactlize_b200_xplane_to_native": (I, [P, P, P, P, I, I, I]),
    "quactlize_b200_native_to_xplane": (I, [P, P, P, P, I, I, I]),
    "quactlize_b200_xplane_slot": (C.c_longlong, [I, I, I, I, I]),
    "quactlize_b200_rt_fail_next": (None, [I]),
    "quactlize_b200_rt_trim": (None, []),
    "quactlize_b200_rt_last_status": (I, []),
    "quactlize_b200_device_wait_status": (I, []),
    "quactlize_b200_debug_wait_probe": (I, [C.c_longlong, P]),
    "quactlize_b200_debug_gemm_swap_launches": (C.c_longlong, []),
    "quactlize_b200_unpack_dev_v1": (I, [P, I64, P, P, P, I, I, P]),
    "quactlize_b200_planes_dequantize_dev_v1": (I, [P, P, P, P, P, I, I, I, I, I, I, I, P]),
}


def lib():
    """The loaded library with typed entry points.  Raises ImportError when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is not built. Build it with:  python -m quactlize_b200.build")
        h = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(h, name)          # AttributeError if the library does not export what the header declares
            fn.restype, fn.argtypes = res, args
        _lib = h
    return _lib
