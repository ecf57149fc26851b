"""ctypes binding of libnf4b200.so (the C ABI declared in include/nf4_b200.h).

There is no fallback: if the shared library is missing the import of any compute
entry point fails with an explicit error telling how to build it.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libnf4b200.so")

OK = 0
LAYOUT_OUT_IN = 0
LAYOUT_IN_OUT = 1
DTYPE_BF16 = 0
DTYPE_F32 = 1


class Nf4Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"nf4 status {status}: {message}")
        self.status = status


class PeerOutputs(C.Structure):
    """``nf4_peer_outputs`` (include/nf4_b200.h)."""
    _fields_ = [("struct_bytes", C.c_uint32), ("world", C.c_int32), ("rank", C.c_int32),
                ("y_full", C.c_void_p * 8), ("ldy_full", C.c_uint64), ("arrivals", C.c_void_p * 8),
                ("signal", C.c_uint32), ("wait_expected", C.c_uint32), ("wait_arrivals", C.c_void_p)]


class LinearArgs(C.Structure):
    """Mirror of ``nf4_linear_args`` (include/nf4_b200.h)."""

    _fields_ = [
        ("struct_bytes", C.c_uint32),
        ("layout", C.c_int32),
        ("io_dtype", C.c_int32),
        ("y_f32", C.c_int32),
        ("rows", C.c_uint64),
        ("d_in", C.c_uint64),
        ("d_out", C.c_uint64),
        ("x", C.c_void_p),
        ("packed", C.c_void_p),
        ("absmax", C.c_void_p),
        ("scale_codes", C.c_void_p),
        ("scale_of_scales", C.c_void_p),
        ("bias", C.c_void_p),
        ("lora_a", C.c_void_p),
        ("lora_b", C.c_void_p),
        ("lora_rank", C.c_uint32),
        ("lora_scale", C.c_float),
        ("y", C.c_void_p),
        ("ldy", C.c_uint64),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_uint64),
    ]


_vp, _u64, _i32, _u32, _f32 = C.c_void_p, C.c_uint64, C.c_int32, C.c_uint32, C.c_float

# name -> (restype, argtypes)
SIGNATURES = {
    "nf4_version": (_i32, []),
    "nf4_last_error": (C.c_char_p, []),
    "nf4_kernel_launch_count": (_u64, []),
    "nf4_device_status": (_i32, [C.POINTER(_i32), C.POINTER(_i32), C.POINTER(_i32)]),
    "nf4_selftest_bounded_wait": (_i32, [_u64, C.POINTER(_u64)]),
    "nf4_selfcheck_code_selection": (_i32, [_u64, _u64, C.POINTER(_u64)]),
    "nf4_selfcheck_quantize_fast_path": (_i32, [_u64, _u64, _f32, C.POINTER(_u64)]),
    "nf4_quantize_transposed_workspace_bytes": (_u64, [_u64, _u64]),
    "nf4_quantize_transposed_dev": (_i32, [_vp, _i32, _u64, _u64, _vp, _vp, _vp, _u64, _vp]),
    "nf4_embedding_gather_dev": (_i32, [_vp, _vp, _vp, _vp, _u64, _u64, _vp, _u64, _vp, _i32, _vp]),
    "nf4_levels": (None, [_vp]),
    "nf4_estimated_resident_bytes": (_u64, [_u64, _i32]),
    "nf4_num_blocks": (_u64, [_u64]),
    "nf4_packed_bytes": (_u64, [_u64]),
    "nf4_quantize_dev": (_i32, [_vp, _u64, _vp, _vp, _vp]),
    "nf4_quantize_host": (_i32, [_vp, _u64, _vp, _vp]),
    "nf4_quantize_unpacked_dev": (_i32, [_vp, _u64, _vp, _vp, _vp]),
    "nf4_double_quantize_dev": (_i32, [_vp, _u64, _vp, _vp, _vp]),
    "nf4_double_quantize_host": (_i32, [_vp, _u64, _vp, _vp]),
    "nf4_dequantize_dev": (_i32, [_vp, _u64, _vp, _vp, _vp, _vp, _vp]),
    "nf4_dequantize_host": (_i32, [_vp, _u64, _vp, _vp, _vp, _vp]),
    "nf4_dequantize_unpacked_dev": (_i32, [_vp, _u64, _vp, _vp, _vp, _vp, _vp]),
    "nf4_quantize_dequantize_workspace_bytes": (_u64, [_u64]),
    "nf4_quantize_dequantize_dev": (_i32, [_vp, _u64, _i32, _vp, _vp, _u64, _vp]),
    "nf4_quantize_dequantize_host": (_i32, [_vp, _u64, _i32, _vp]),
    "nf4_linear_workspace_bytes": (_u64, [_u64, _u64, _u64, _u32]),
    "nf4_linear_forward_dev": (_i32, [C.POINTER(LinearArgs), _vp]),
    "nf4_lora_workspace_bytes": (_u64, [_u64, _u32]),
    "nf4_lora_forward_dev": (_i32, [_vp, _u64, _u64, _u64, _vp, _vp, _u32, _f32, _i32, _i32, _vp, _u64, _vp,
                                    _u64, _vp]),
    "nf4_lora_delta_weight_dev": (_i32, [_vp, _vp, _u64, _u64, _u32, _f32, _i32, _i32, _vp, _vp]),
    "nf4_qlora_merge_dev": (_i32, [_vp, _vp, _vp, _vp, _u64, _u64, _i32, _vp, _vp, _u32, _f32, _i32, _vp, _vp]),
    "nf4_qlora_backward_workspace_bytes": (_u64, [_u64, _u64, _u64, _u32]),
    "nf4_qlora_backward_dev": (_i32, [C.POINTER(LinearArgs), _vp, _vp, _vp, _vp, _vp]),
    "nf4_sharded_gather_bytes": (_u64, [_u64, _u64, _i32, _i32, _i32]),
    "nf4_sharded_linear_forward_dev": (_i32, [C.POINTER(LinearArgs), _vp, _i32, _i32, _vp, _u64, _vp, _u64, _vp]),
    "nf4_linear_noalloc_scratch_bytes": (_u64, []),
    "nf4_linear_forward_grouped_dev": (_i32, [C.POINTER(LinearArgs), _u32, _vp]),
    "nf4_reserve_sms": (_i32, [_i32]),
    "nf4_decode_share_plan": (_i32, [_u32, _u32, _u32, _u32, _u32, C.POINTER(_u32)]),
    "nf4_prefill_share_plan": (_i32, [_u64, _u64, _u64, _u32, C.POINTER(_u32), C.POINTER(_u32), _u32]),
    "nf4_linear_forward_scatter_dev": (_i32, [C.POINTER(LinearArgs), C.POINTER(PeerOutputs), _vp]),
    "nf4_peer_arrivals_wait_dev": (_i32, [_vp, _u32, _u32, _vp]),
    "nf4_peer_push_columns_dev": (_i32, [C.POINTER(PeerOutputs), _u64, _u64, _i32, _vp, _vp]),
    "nf4_linear_forward_noalloc_dev": (_i32, [C.POINTER(LinearArgs), _vp]),
    "nf4_weight_from_values_host": (_i32, [_vp, _u64, _u64, _i32, _i32, C.POINTER(_vp)]),
    "nf4_weight_from_packed_host": (_i32, [_vp, _vp, _vp, _f32, _u64, _u64, _i32,
                                           C.POINTER(_vp)]),
    "nf4_weight_free": (None, [_vp]),
    "nf4_weight_resident_bytes": (_u64, [_vp]),
    "nf4_weight_download_host": (_i32, [_vp, _vp, _vp, _vp, _vp]),
    "nf4_weight_dequantize_host": (_i32, [_vp, _vp]),
    "nf4_weight_attach_lora_host": (_i32, [_vp, _vp, _vp, _u32, _f32, _i32]),
    "nf4_weight_linear_forward_host": (_i32, [_vp, _vp, _u64, _i32, _vp, _vp, _vp, _u32, _f32,
                                              _vp]),
}

_lib = None


def load() -> C.CDLL:
    """Load libnf4b200.so; raise (never fall back) when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m unifur_b200.build` "
                "(nvcc, sm_100a).  This package has no CPU or PyTorch fallback.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error() -> str:
    return load().nf4_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    if status != OK:
        raise Nf4Error(status, last_error())


def launch_count() -> int:
    return int(load().nf4_kernel_launch_count())
