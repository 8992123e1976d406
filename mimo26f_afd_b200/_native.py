"""ctypes binding of ``libm26b_expert.so`` (declarations: ``include/m26b_expert.h``)."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libm26b_expert.so")

# Every symbol include/m26b_expert.h declares.
SYMBOLS = (
    "m26b_layer_new", "m26b_layer_new_tp", "m26b_layer_new_from_checkpoint", "m26b_layer_all_normal",
    "m26b_layer_i_local", "m26b_layer_free", "m26b_scratch_new", "m26b_scratch_free", "m26b_ffn", "m26b_ffn_dev",
    "m26b_scratch_status", "m26b_scratch_set_debug", "m26b_scratch_timings", "m26b_scratch_peek", "m26b_quantize_dev",
    "m26b_route_reduce_dev", "m26b_rank_sum_dev", "m26b_plan_static", "m26b_version",
    "m26b_exchange_new", "m26b_exchange_connect", "m26b_exchange_connect_local", "m26b_exchange_plane",
    "m26b_exchange_set_wait_ms", "m26b_exchange_publish_as", "m26b_exchange_sum_dev", "m26b_exchange_status",
    "m26b_exchange_free",
    "m26b_layer_new_from_checkpoint_ep", "m26b_ep_new", "m26b_ep_connect", "m26b_ep_connect_local", "m26b_ep_rows",
    "m26b_ep_set_wait_ms", "m26b_ep_publish_as", "m26b_ep_begin_dev", "m26b_ep_compute_dev", "m26b_ep_finish_dev",
    "m26b_ep_status", "m26b_ep_free", "m26b_produce_dev",
    "m26b_rank_sum_residual_dev", "m26b_exchange_sum_residual_dev", "m26b_scratch_set_route_output", "m26b_ep_set_route_output",
    "m26b_ffn_tp", "m26b_ffn_tp_dev", "m26b_ep_ffn", "m26b_layer_image", "m26b_layer_new_from_checkpoint_ep_replicated",
    "m26b_frame_request_bytes", "m26b_frame_return_bytes", "m26b_frame_crc32c", "m26b_frame_crc32c_table", "m26b_frame_encode_request",
    "m26b_serve_frame", "m26b_frame_parse_return", "m26b_frame_check_request",
)

_lib = None


def lib() -> C.CDLL:
    """Load the CUDA library. There is no fallback: a missing build is an error."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it first (python -c 'import __graft_entry__ as g; g.build()'). "
            "This package has no CPU or PyTorch fallback for the expert FFN."
        )
    L = C.CDLL(LIB_PATH)
    vp, u8p, i32p, f32p, u16p, u32p = C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p
    err = (C.c_char_p, C.c_size_t)
    L.m26b_layer_new.argtypes = [u8p, C.c_uint64, C.c_uint32, C.POINTER(vp), *err]
    L.m26b_layer_new_tp.argtypes = [u8p, C.c_uint64, C.c_uint32, C.c_uint32, C.POINTER(vp), *err]
    L.m26b_layer_new_from_checkpoint.argtypes = [u8p] * 6 + [C.c_uint32, C.c_uint32, C.POINTER(vp), *err]
    L.m26b_layer_all_normal.argtypes = [vp]
    L.m26b_layer_i_local.argtypes = [vp]
    L.m26b_layer_image.argtypes = [vp, C.c_int, C.POINTER(C.c_uint64)]
    L.m26b_layer_image.restype = C.c_void_p
    L.m26b_layer_free.argtypes = [vp]
    L.m26b_layer_free.restype = None
    L.m26b_scratch_new.argtypes = [C.POINTER(vp), *err]
    L.m26b_scratch_free.argtypes = [vp]
    L.m26b_scratch_free.restype = None
    L.m26b_ffn.argtypes = [vp, vp, u8p, C.c_size_t, u8p, C.c_size_t, i32p, f32p, C.c_uint32, u16p, f32p, *err]
    L.m26b_ffn_dev.argtypes = [vp, vp, vp, C.c_int, u8p, C.c_int, i32p, f32p, C.c_uint32, u16p, f32p, vp, *err]
    L.m26b_scratch_status.argtypes = [vp, vp, *err]
    L.m26b_scratch_set_debug.argtypes = [vp, C.c_uint32]
    L.m26b_ffn_tp_dev.argtypes = [vp, vp, vp, vp, C.c_int, u8p, C.c_int, i32p, f32p, C.c_uint32, f32p, f32p, vp, *err]
    L.m26b_ffn_tp.argtypes = [vp, vp, vp, u8p, C.c_size_t, u8p, C.c_size_t, i32p, f32p, C.c_uint32, f32p, f32p, *err]
    L.m26b_ep_ffn.argtypes = [vp, vp, vp, u8p, C.c_size_t, u8p, C.c_size_t, i32p, f32p, C.c_uint32, u16p, *err]
    L.m26b_scratch_set_route_output.argtypes = [vp, C.c_int]
    L.m26b_ep_set_route_output.argtypes = [vp, C.c_int]
    L.m26b_scratch_timings.argtypes = [vp, f32p, *err]
    L.m26b_scratch_peek.argtypes = [vp, C.c_int, vp, C.c_uint64, *err]
    L.m26b_quantize_dev.argtypes = [vp, C.c_int, C.c_uint64, C.c_int, u8p, u8p, u32p, vp, *err]
    L.m26b_route_reduce_dev.argtypes = [f32p, f32p, C.c_uint32, f32p, u16p, u32p, vp, *err]
    L.m26b_rank_sum_dev.argtypes = [C.POINTER(vp), C.c_int, C.c_uint64, f32p, vp, *err]
    L.m26b_plan_static.argtypes = [i32p, f32p, C.c_uint32, i32p, i32p, f32p, u32p, vp, *err]
    L.m26b_version.restype = C.c_char_p
    L.m26b_exchange_new.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.POINTER(vp), u8p, *err]
    L.m26b_exchange_connect.argtypes = [vp, u8p, *err]
    L.m26b_exchange_connect_local.argtypes = [vp, C.POINTER(vp), *err]
    L.m26b_exchange_plane.argtypes = [vp]
    L.m26b_exchange_plane.restype = C.c_void_p
    L.m26b_exchange_set_wait_ms.argtypes = [vp, C.c_uint32]
    L.m26b_exchange_publish_as.argtypes = [vp, C.c_uint32, vp, *err]
    L.m26b_exchange_sum_dev.argtypes = [vp, C.c_uint64, f32p, vp, *err]
    L.m26b_exchange_status.argtypes = [vp, vp, *err]
    L.m26b_exchange_free.argtypes = [vp]
    L.m26b_exchange_free.restype = None
    L.m26b_layer_new_from_checkpoint_ep.argtypes = [u8p] * 6 + [C.c_uint32, C.c_uint32, C.POINTER(vp), *err]
    L.m26b_layer_new_from_checkpoint_ep_replicated.argtypes = [u8p] * 12 + [i32p, C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(vp), *err]
    L.m26b_ep_new.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(vp), u8p, *err]
    L.m26b_ep_connect.argtypes = [vp, u8p, *err]
    L.m26b_ep_connect_local.argtypes = [vp, C.POINTER(vp), *err]
    L.m26b_ep_rows.argtypes = [vp, C.c_uint32]
    L.m26b_ep_set_wait_ms.argtypes = [vp, C.c_uint32]
    L.m26b_ep_publish_as.argtypes = [vp, C.c_uint32, C.c_uint32, vp, *err]
    L.m26b_ep_begin_dev.argtypes = [vp, vp, C.c_int, u8p, C.c_int, i32p, f32p, C.c_uint32, vp, *err]
    L.m26b_ep_compute_dev.argtypes = [vp, vp, vp, vp, *err]
    L.m26b_ep_finish_dev.argtypes = [vp, u16p, f32p, vp, *err]
    L.m26b_ep_status.argtypes = [vp, vp, *err]
    L.m26b_ep_free.argtypes = [vp]
    L.m26b_ep_free.restype = None
    L.m26b_rank_sum_residual_dev.argtypes = [C.POINTER(vp), C.c_int, C.c_uint64, f32p, f32p, vp, *err]
    L.m26b_exchange_sum_residual_dev.argtypes = [vp, C.c_uint64, f32p, f32p, vp, *err]
    L.m26b_frame_request_bytes.argtypes = [C.c_uint32]
    L.m26b_frame_request_bytes.restype = C.c_uint64
    L.m26b_frame_return_bytes.argtypes = [C.c_uint32]
    L.m26b_frame_return_bytes.restype = C.c_uint64
    L.m26b_frame_crc32c.argtypes = [u8p, C.c_uint64]
    L.m26b_frame_crc32c.restype = C.c_uint32
    L.m26b_frame_crc32c_table.argtypes = [u8p, C.c_uint64]
    L.m26b_frame_crc32c_table.restype = C.c_uint32
    L.m26b_frame_encode_request.argtypes = [u8p, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint64, C.c_uint64, u8p, C.c_size_t, u8p,
                                            C.c_size_t, i32p, f32p, C.c_uint32, C.c_int, C.POINTER(C.c_uint64), *err]
    L.m26b_serve_frame.argtypes = [vp, vp, u8p, C.c_uint64, u8p, C.c_uint64, C.POINTER(C.c_uint64), C.c_int, C.c_uint64, f32p, *err]
    L.m26b_frame_parse_return.argtypes = [u8p, C.c_uint64, C.c_int, C.POINTER(C.c_uint64), C.POINTER(C.c_uint32), C.POINTER(C.c_uint32),
                                          C.POINTER(C.c_uint32), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), *err]
    L.m26b_frame_check_request.argtypes = [u8p, C.c_uint64, C.c_int, C.POINTER(C.c_uint32), C.POINTER(C.c_uint64),
                                           C.POINTER(C.c_uint32), *err]
    L.m26b_produce_dev.argtypes = [f32p, f32p, C.c_uint32, i32p, f32p, vp, C.c_int, C.c_int, u8p, u8p, u32p, vp, *err]
    for name in SYMBOLS:
        if name not in ("m26b_layer_free", "m26b_scratch_free", "m26b_version", "m26b_exchange_plane", "m26b_exchange_free", "m26b_layer_image",
                        "m26b_ep_free", "m26b_frame_request_bytes", "m26b_frame_return_bytes", "m26b_frame_crc32c",
                        "m26b_frame_crc32c_table"):
            getattr(L, name).restype = C.c_int
    _lib = L
    return L
