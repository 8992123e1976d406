"""Python binding of the CPU oracle (``oracle/oracle.c``) and, when present, of the reference's own
host-compiled units (``oracle/_ref/libm26ref.so``, built by ``make -C oracle ref`` from the reference tree).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline
legs as the checker. Nothing in the product package imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(_HERE, "liboracle.so")
REF_LIB = os.path.join(_HERE, "_ref", "libm26ref.so")
H, I, E, TOPK = 4096, 2048, 256, 8
_lib = None
_ref = None


def build(ref: bool = False) -> None:
    """Compile the oracle (and optionally the reference units) with the committed Makefile."""
    subprocess.run(["make", "-C", _HERE] + (["ref"] if ref else []), check=True, capture_output=True)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build()
        L = C.CDLL(LIB)
        p = C.c_void_p
        L.orc_e4m3_decode.argtypes = [C.c_uint8]
        L.orc_e4m3_decode.restype = C.c_float
        L.orc_quant_wire.argtypes = [p, C.c_uint64, p, p]
        L.orc_quant_wire.restype = None
        L.orc_quant_v1.argtypes = [p, C.c_uint64, p, p, p]
        L.orc_quant_v1.restype = C.c_uint64
        L.orc_dequant_v1.argtypes = [p, p, C.c_uint64, p]
        L.orc_mxfp4_unpack.argtypes = [p, p, C.c_uint64, C.c_uint64, p]
        L.orc_mxfp4_unpack.restype = None
        L.orc_plan.argtypes = [p, p, C.c_uint32, p, p, p, p, p]
        L.orc_activation.argtypes = [C.c_float, C.c_float]
        L.orc_activation.restype = C.c_float
        L.orc_expert_ffn.argtypes = [p, p, C.c_uint32, p, p, p, p, p, p, C.c_uint32, C.c_uint32, p, p, p, p, p, p]
        L.orc_bf16_rne.argtypes = [C.c_float]
        L.orc_bf16_rne.restype = C.c_uint16
        L.orc_route_reduce.argtypes = [p, p, C.c_uint32, p, p]
        L.orc_route_reduce_h.argtypes = [p, p, C.c_uint32, C.c_uint32, p, p]
        L.orc_rank_sum.argtypes = [p, C.c_uint32, C.c_uint64, p]
        L.orc_rank_sum.restype = None
        L.orc_router_from_logits.argtypes = [p, p, C.c_uint32, C.c_uint32, C.c_uint32, p, p]
        L.orc_router_from_logits.restype = None
        L.orc_ffn_layer.argtypes = [p] * 6 + [C.c_uint32, C.c_uint32, p, p, p, p, C.c_uint32, p, p, p, p, p, p]
        L.orc_cpu_path.argtypes = [p] * 10 + [C.c_uint32, C.c_uint32, C.c_uint32, p, p]
        L.orc_cpu_path.restype = C.c_uint32
        _lib = L
    return _lib


def ref_lib():
    """The reference's own quantiser / planner / reducer, or None when it was not built."""
    global _ref
    if _ref is None and os.path.exists(REF_LIB):
        R = C.CDLL(REF_LIB)
        p = C.c_void_p
        R.ref_quantize_host.argtypes = [p, C.c_uint64, p, p, p]
        R.ref_quantize_host.restype = C.c_uint32
        R.ref_plan_host.argtypes = [C.c_uint32, C.c_uint32, p, p, p, p, p, p, p, p, p]
        R.ref_plan_host.restype = C.c_uint32
        R.ref_reduce_host.argtypes = [C.c_uint32, p, p, p, p, p]
        R.ref_reduce_host.restype = C.c_uint32
        _ref = R
    return _ref


def _a(x, dtype):
    return np.ascontiguousarray(x, dtype=dtype)


def _p(a):
    return None if a is None else a.ctypes.data


def e4m3_table() -> np.ndarray:
    return np.array([lib().orc_e4m3_decode(c) for c in range(256)], dtype=np.float32)


def quant_wire(x):
    x = _a(x, np.float32)
    payload = np.empty(x.shape, np.uint8)
    scales = np.empty(x.shape[:-1] + (x.shape[-1] // 32,), np.uint8)
    lib().orc_quant_wire(_p(x), x.size, _p(payload), _p(scales))
    return payload, scales


def quant_v1(x):
    """Returns (payload, scales, block_faults); faulting blocks keep zero bytes."""
    x = _a(x, np.float32)
    payload = np.zeros(x.shape, np.uint8)
    scales = np.zeros(x.shape[:-1] + (x.shape[-1] // 32,), np.uint8)
    faults = np.zeros(x.size // 32, np.uint32)
    lib().orc_quant_v1(_p(x), x.size, _p(payload), _p(scales), _p(faults))
    return payload, scales, faults


def dequant_v1(payload, scales):
    payload, scales = _a(payload, np.uint8), _a(scales, np.uint8)
    out = np.empty(payload.shape, np.float32)
    if lib().orc_dequant_v1(_p(payload), _p(scales), payload.size, _p(out)):
        raise ValueError("quantizer-v1 decode fault (scale byte outside 105..247, NaN code or overflow)")
    return out


def mxfp4_unpack(packed, scales):
    packed, scales = _a(packed, np.uint8), _a(scales, np.uint8)
    rows, half = packed.shape
    out = np.empty((rows, half * 2), np.float32)
    lib().orc_mxfp4_unpack(_p(packed), _p(scales), rows, half * 2, _p(out))
    return out


def plan(ids, weights, resident=None):
    """Stable plan: returns (status, inverse, original_routes, grouped_weights, counts)."""
    ids, weights = _a(ids, np.int32).reshape(-1), _a(weights, np.float32).reshape(-1)
    rows = ids.size // TOPK
    resident = np.ones(E, np.uint8) if resident is None else _a(resident, np.uint8)
    inv, orig = np.full(ids.size, -1, np.int32), np.full(ids.size, -1, np.int32)
    gw, counts = np.zeros(ids.size, np.float32), np.zeros(E, np.uint32)
    st = lib().orc_plan(_p(ids), _p(weights), rows, _p(resident), _p(inv), _p(orig), _p(gw), _p(counts))
    return st, inv, orig, gw, counts


def activation(g, u):
    g, u = _a(g, np.float32), _a(u, np.float32)
    f = lib().orc_activation
    return np.array([f(float(a), float(b)) for a, b in zip(g.reshape(-1), u.reshape(-1))], np.float32).reshape(g.shape)


def expert_ffn(xq, xs, gate_w, gate_s, up_w, up_s, down_w, down_s, i0=0, il=I):
    """One expert on m rows for intermediate slice [i0, i0+il): dict of gate, up, h, mid_q, mid_s, y."""
    xq, xs = _a(xq, np.uint8), _a(xs, np.uint8)
    m = xq.shape[0]
    o = dict(gate=np.empty((m, il), np.float32), up=np.empty((m, il), np.float32), h=np.empty((m, il), np.float32),
             mid_q=np.empty((m, il), np.uint8), mid_s=np.empty((m, il // 32), np.uint8), y=np.empty((m, H), np.float32))
    ws = [_a(t, np.uint8) for t in (gate_w, gate_s, up_w, up_s, down_w, down_s)]
    rc = lib().orc_expert_ffn(_p(xq), _p(xs), m, *[_p(t) for t in ws], i0, il, _p(o["gate"]), _p(o["up"]), _p(o["h"]),
                              _p(o["mid_q"]), _p(o["mid_s"]), _p(o["y"]))
    o["rc"] = rc
    return o


def route_reduce(y, weights, hidden=H):
    """y [rows,8,hidden] unweighted, weights [rows,8] -> (status, partial f32, bf16)."""
    y, weights = _a(y, np.float32), _a(weights, np.float32)
    rows = weights.size // TOPK
    partial, bf16 = np.empty((rows, hidden), np.float32), np.empty((rows, hidden), np.uint16)
    rc = lib().orc_route_reduce_h(_p(y), _p(weights), rows, hidden, _p(partial), _p(bf16))
    return rc, partial, bf16


def rank_sum(planes):
    planes = _a(planes, np.uint16)
    g, n = planes.shape[0], planes[0].size
    out = np.empty(planes.shape[1:], np.float32)
    lib().orc_rank_sum(_p(planes), g, n, _p(out))
    return out


def router_from_logits(logits, bias, top_k=8):
    """crates/mimo26-coordinator/src/router.rs:42-80: (indices int32 [T, top_k], weights float32 [T, top_k])."""
    logits = _a(logits, np.float32)
    t, e = logits.shape
    b = None if bias is None else _a(bias, np.float32)
    idx = np.empty((t, top_k), np.int32)
    w = np.empty((t, top_k), np.float32)
    lib().orc_router_from_logits(_p(logits), None if b is None else _p(b), t, e, top_k, _p(idx), _p(w))
    return idx, w


def ffn_layer(tensors, xq, xs, ids, weights, tp_rank=0, tp_size=1, stages=False):
    """One rank's layer FFN. ``tensors``: dict of the six stacked checkpoint tensors (uint8).
    Returns dict(rc, y [routes,4096], partial, bf16 [, h, mid_q, mid_s in grouped order])."""
    xq, xs = _a(xq, np.uint8), _a(xs, np.uint8)
    ids, weights = _a(ids, np.int32).reshape(-1), _a(weights, np.float32).reshape(-1)
    rows = xq.shape[0]
    routes, il = rows * TOPK, I // tp_size
    o = dict(y=np.zeros((routes, H), np.float32), partial=np.empty((rows, H), np.float32),
             bf16=np.empty((rows, H), np.uint16))
    if stages:
        o.update(h=np.zeros((routes, il), np.float32), mid_q=np.zeros((routes, il), np.uint8),
                 mid_s=np.zeros((routes, il // 32), np.uint8))
    names = ("gate_w", "gate_s", "up_w", "up_s", "down_w", "down_s")
    ws = [_a(tensors[n], np.uint8) for n in names]
    o["rc"] = lib().orc_ffn_layer(*[_p(t) for t in ws], tp_rank, tp_size, _p(xq), _p(xs), _p(ids), _p(weights), rows,
                                  _p(o["y"]), _p(o["partial"]), _p(o["bf16"]), _p(o.get("h")), _p(o.get("mid_q")),
                                  _p(o.get("mid_s")))
    return o


def cpu_path(tensors, xq, xs, ids, weights, e_lo=0, e_hi=E):
    """The reference's CPU expert path (E-FP32 lattice) over experts [e_lo, e_hi): (routed rows, f32, bf16)."""
    xq, xs = _a(xq, np.uint8), _a(xs, np.uint8)
    ids, weights = _a(ids, np.int32).reshape(-1), _a(weights, np.float32).reshape(-1)
    rows = xq.shape[0]
    out, bf = np.empty((rows, H), np.float32), np.empty((rows, H), np.uint16)
    names = ("gate_w", "gate_s", "up_w", "up_s", "down_w", "down_s")
    ws = [_a(tensors[n], np.uint8) for n in names]
    done = lib().orc_cpu_path(*[_p(t) for t in ws], _p(xq), _p(xs), _p(ids), _p(weights), rows, e_lo, e_hi, _p(out), _p(bf))
    return done, out, bf
