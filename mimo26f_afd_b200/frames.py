"""DS41RTE3 v3 request / return frames over the C ABI: the data format either side of the expert FFN.

A request frame carries, for ``rows`` tokens, a 40-byte descriptor, eight 12-byte route entries and the 4,224-byte
quantised hidden row each (``crates/mimo26-wire/src/layout.rs``: 4,360 bytes per token); the return frame carries the
rank's 8,192-byte BF16 row per token. ``serve_frame`` is the expert daemon's per-request work
(``crates/mimo26-spark/src/serve.rs:206-246``): request frame in, sealed return frame out.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _native
from .expert import ExpertError, Layer, Scratch, _check

H, TOPK = 4096, 8
HEADER_LEN, REQUEST_ROW_BYTES, RETURN_ROW_BYTES = 128, 4360, 8192


def crc32c(data: bytes) -> int:
    buf = (C.c_uint8 * len(data)).from_buffer_copy(data) if data else None
    return int(_native.lib().m26b_frame_crc32c(C.addressof(buf) if buf is not None else None, len(data)))


def crc32c_table(data: bytes) -> int:
    """The table path only (the cross-check of the instruction path ``crc32c`` may take)."""
    buf = (C.c_uint8 * len(data)).from_buffer_copy(data) if data else None
    return int(_native.lib().m26b_frame_crc32c_table(C.addressof(buf) if buf is not None else None, len(data)))


def request_bytes(rows: int) -> int:
    return int(_native.lib().m26b_frame_request_bytes(rows))


def return_bytes(rows: int) -> int:
    return int(_native.lib().m26b_frame_return_bytes(rows))


def encode_request(payload: np.ndarray, scales: np.ndarray, ids: np.ndarray, weights: np.ndarray, *, request_id: int = 1,
                   layer_id: int = 0, executor_id: int = 0, seq: int = 0, seal: bool = True) -> bytes:
    """The coordinator's request frame for decode-kind rows (frame.rs:569-652 plus the hidden rows and the seal)."""
    payload = np.ascontiguousarray(payload, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    rows = ids.size // TOPK
    if rows == 0 or payload.size != rows * H or scales.size != rows * H // 32 or weights.size != rows * TOPK:
        raise ExpertError(1, "frame: extents do not match")
    out = np.empty(request_bytes(rows), np.uint8)
    n, err = C.c_uint64(), C.create_string_buffer(256)
    _check(_native.lib().m26b_frame_encode_request(out.ctypes.data, out.size, request_id, layer_id, executor_id, seq,
                                                   payload.ctypes.data, H, scales.ctypes.data, H // 32, ids.ctypes.data,
                                                   weights.ctypes.data, rows, 1 if seal else 0, C.byref(n), err, 256), err)
    return out[:n.value].tobytes()


def check_request(frame: bytes, check_crc: bool = True):
    """(rows, request_id, layer_id) of a request frame the daemon would accept; raises ``ExpertError`` (code 6) otherwise."""
    buf = np.frombuffer(frame, np.uint8)
    rows, rid, lid, err = C.c_uint32(), C.c_uint64(), C.c_uint32(), C.create_string_buffer(256)
    _check(_native.lib().m26b_frame_check_request(buf.ctypes.data, buf.size, 1 if check_crc else 0, C.byref(rows), C.byref(rid),
                                                  C.byref(lid), err, 256), err)
    return rows.value, rid.value, lid.value


def serve_frame(layer: Layer, scratch: Scratch, request: bytes, *, check_crc: bool = True, reply_seq: int = 0) -> bytes:
    buf = np.frombuffer(request, np.uint8)
    rows = (max(buf.size, HEADER_LEN) - HEADER_LEN) // REQUEST_ROW_BYTES + 1
    reply = np.empty(return_bytes(rows), np.uint8)
    n, err = C.c_uint64(), C.create_string_buffer(256)
    _check(_native.lib().m26b_serve_frame(layer._h, scratch._h, buf.ctypes.data, buf.size, reply.ctypes.data, reply.size,
                                          C.byref(n), 1 if check_crc else 0, reply_seq, None, err, 256), err)
    return reply[:n.value].tobytes()


def parse_return(frame: bytes, check_crc: bool = True):
    """(dict of header fields, BF16 rows as uint16 [rows, 4096]) of a return frame."""
    buf = np.frombuffer(frame, np.uint8)
    rid, lid, rows, status, seq, off = C.c_uint64(), C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint64(), C.c_uint64()
    err = C.create_string_buffer(256)
    _check(_native.lib().m26b_frame_parse_return(buf.ctypes.data, buf.size, 1 if check_crc else 0, C.byref(rid), C.byref(lid),
                                                 C.byref(rows), C.byref(status), C.byref(seq), C.byref(off), err, 256), err)
    body = np.frombuffer(frame, np.dtype("<u2"), count=rows.value * H, offset=off.value).reshape(rows.value, H)
    return dict(request_id=rid.value, layer_id=lid.value, rows=rows.value, status=status.value, seq=seq.value), body
