"""Host-side mirror of the reference's expert-rank wrapper, over the C ABI.

Names, argument meaning and error behaviour follow ``crates/mimo26-spark/src/b1.rs``:
``Layer`` (b1.rs:57-92) owns one MoE layer's prepared weights, ``Scratch`` (b1.rs:94-120)
the per-request device buffers and stream, ``ffn`` / ``ffn_strided`` (b1.rs:131-176) run one
rank's expert FFN on host rows and return ``FfnStats`` (b1.rs:122-129). Failures raise
``ExpertError`` carrying the library's message, where the Rust returns ``Err(String)``.

Device-pointer entry points take anything with a ``data_ptr()`` (a torch CUDA tensor) or a
plain integer address; torch is only the allocator here.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _native

H = 4096
TOPK = 8


class ExpertError(RuntimeError):
    """A nonzero return of the C ABI: ``code`` 1 argument, 2 CUDA, 3 plan rejected, 4 numerical fault,
    5 a peer's plane did not arrive within the exchange's wait bound."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code
        self.message = message


def _check(rc: int, err) -> None:
    if rc != 0:
        raise ExpertError(rc, err.value.decode("utf-8", "replace"))


def _ptr(x) -> int:
    if x is None:
        return 0
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return int(x.data_ptr())
    if isinstance(x, np.ndarray):
        return int(x.ctypes.data)
    raise TypeError(f"cannot take an address of {type(x)!r}")


def version() -> str:
    return _native.lib().m26b_version().decode()


class Layer:
    """One MoE layer's prepared operand image on the current CUDA device (b1.rs:57-92)."""

    def __init__(self, handle: int):
        self._h = C.c_void_p(handle)

    @classmethod
    def new(cls, canonical_dev, nbytes: int, rank: int) -> "Layer":
        """From the reference's canonical-v2 TP4 rank image in device memory (b1.rs:72-84)."""
        out, err = C.c_void_p(), C.create_string_buffer(256)
        _check(_native.lib().m26b_layer_new(_ptr(canonical_dev), nbytes, rank, C.byref(out), err, 256), err)
        return cls(out.value)

    @classmethod
    def new_tp(cls, canonical_dev, nbytes: int, tp_rank: int, tp_size: int) -> "Layer":
        out, err = C.c_void_p(), C.create_string_buffer(256)
        _check(_native.lib().m26b_layer_new_tp(_ptr(canonical_dev), nbytes, tp_rank, tp_size, C.byref(out), err, 256), err)
        return cls(out.value)

    @classmethod
    def from_checkpoint(cls, gate_w, gate_s, up_w, up_s, down_w, down_s, tp_rank: int = 0, tp_size: int = 1) -> "Layer":
        """From the six checkpoint tensors stacked over the 256 experts, all on the device."""
        out, err = C.c_void_p(), C.create_string_buffer(256)
        _check(_native.lib().m26b_layer_new_from_checkpoint(
            _ptr(gate_w), _ptr(gate_s), _ptr(up_w), _ptr(up_s), _ptr(down_w), _ptr(down_s), tp_rank, tp_size,
            C.byref(out), err, 256), err)
        return cls(out.value)

    @classmethod
    def from_checkpoint_ep(cls, gate_w, gate_s, up_w, up_s, down_w, down_s, ep_rank: int, ep_size: int, replicas=None,
                           replica_ids=None) -> "Layer":
        """Expert-parallel rank: the six tensors stacked over this rank's 256 / ep_size experts only. ``replicas`` (the six
        tensors stacked over the experts ``replica_ids``, the same set on every rank) adds copies of popular experts: a
        route to one of them is served where its token lives."""
        out, err = C.c_void_p(), C.create_string_buffer(256)
        if replica_ids is not None and len(replica_ids):
            rid = np.ascontiguousarray(replica_ids, dtype=np.int32)
            _check(_native.lib().m26b_layer_new_from_checkpoint_ep_replicated(
                _ptr(gate_w), _ptr(gate_s), _ptr(up_w), _ptr(up_s), _ptr(down_w), _ptr(down_s), *[_ptr(t) for t in replicas],
                rid.ctypes.data, rid.size, ep_rank, ep_size, C.byref(out), err, 256), err)
            return cls(out.value)
        _check(_native.lib().m26b_layer_new_from_checkpoint_ep(
            _ptr(gate_w), _ptr(gate_s), _ptr(up_w), _ptr(up_s), _ptr(down_w), _ptr(down_s), ep_rank, ep_size,
            C.byref(out), err, 256), err)
        return cls(out.value)

    IMAGES = {"w13": 0, "s13": 1, "w2": 2, "s2": 3, "s13h": 4}

    def image(self, which: str):
        """(device address, bytes) of a prepared operand image: ``w13`` / ``s13`` / ``w2`` / ``s2`` / ``s13h`` (the gate/up
        scale blocks regrouped for half items) (read-only)."""
        n = C.c_uint64()
        p = _native.lib().m26b_layer_image(self._h, self.IMAGES[which], C.byref(n))
        if not p:
            raise ExpertError(1, "m26b layer image: bad handle")
        return int(p), int(n.value)

    def all_scales_normal(self) -> bool:
        return _native.lib().m26b_layer_all_normal(self._h) != 0

    @property
    def i_local(self) -> int:
        return _native.lib().m26b_layer_i_local(self._h)

    def close(self) -> None:
        if self._h:
            _native.lib().m26b_layer_free(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Scratch:
    """Per-request device scratch and stream (b1.rs:94-120)."""

    PEEK = {"meta": 0, "inverse": 1, "original_routes": 2, "grouped_weights": 3, "x_payload": 4, "x_scales": 5,
            "mid_payload": 6, "mid_f32": 7, "y": 8, "partial": 9, "mid_scales": 10}

    def __init__(self):
        out, err = C.c_void_p(), C.create_string_buffer(256)
        _check(_native.lib().m26b_scratch_new(C.byref(out), err, 256), err)
        self._h = out

    def set_debug(self, flags: int) -> None:
        _native.lib().m26b_scratch_set_debug(self._h, flags)

    def set_route_output(self, bf16: bool) -> None:
        """FC2 rows as BF16 instead of FP32 (the reference's opt-in ``MIMO26_B1_Y=bf16``, b1_serve.cu:400-406):
        half the FC2 write and combine read, not bit-identical to the FP32 mode."""
        if _native.lib().m26b_scratch_set_route_output(self._h, 1 if bf16 else 0):
            raise ExpertError(1, "m26b scratch: bad route-output type")

    def status(self, stream=None) -> None:
        """Wait for the last ``ffn_dev`` on this scratch and raise on a plan or numerical fault."""
        err = C.create_string_buffer(256)
        _check(_native.lib().m26b_scratch_status(self._h, _ptr(stream), err, 256), err)

    def timings(self) -> dict:
        """Per-kernel GPU milliseconds of the last pass (needs ``set_debug(2)`` before the pass)."""
        ms = (C.c_float * 6)()
        err = C.create_string_buffer(256)
        _check(_native.lib().m26b_scratch_timings(self._h, ms, err, 256), err)
        return dict(zip(("quantize", "plan", "permute", "fc1", "fc2", "combine"), [float(v) for v in ms]))

    def peek(self, what: str, dtype, shape) -> np.ndarray:
        """Copy a stage buffer of the last pass to the host (parity tests)."""
        out = np.empty(shape, dtype=dtype)
        err = C.create_string_buffer(256)
        _check(_native.lib().m26b_scratch_peek(self._h, self.PEEK[what], out.ctypes.data, out.nbytes, err, 256), err)
        return out

    def close(self) -> None:
        if self._h:
            _native.lib().m26b_scratch_free(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


@dataclass
class FfnStats:
    """Stage timings of one ``ffn`` call (b1.rs:122-129)."""
    upload_plan_ms: float
    gpu_ms: float
    tail_ms: float
    groups: int
    phase_ms: tuple  # FC1 (with plan, permute and the fused quantiser), 0, FC2, combine; zeros unless Scratch.set_debug(4)


def _ffn_raw(layer, scratch, payload_ptr, payload_pitch, scales_ptr, scales_pitch, ids, weights, rows, bf16_out):
    if rows == 0 or ids.size != rows * TOPK or weights.size != rows * TOPK or bf16_out.size != rows * H:
        raise ExpertError(1, f"b1 ffn: extents do not match {rows} rows")
    ms = (C.c_float * 8)()
    err = C.create_string_buffer(256)
    rc = _native.lib().m26b_ffn(layer._h, scratch._h, payload_ptr, payload_pitch, scales_ptr, scales_pitch,
                                ids.ctypes.data, weights.ctypes.data, rows, bf16_out.ctypes.data, ms, err, 256)
    _check(rc, err)
    return FfnStats(ms[0], ms[1], ms[2], int(ms[3]), (ms[4], ms[5], ms[6], ms[7]))


def ffn(layer: Layer, scratch: Scratch, payload: np.ndarray, scales: np.ndarray, ids: np.ndarray, weights: np.ndarray,
        rows: int, bf16_out: np.ndarray) -> FfnStats:
    """One rank's FFN for ``rows`` tokens on host arrays (b1.rs:131-152): ``payload`` [rows*4096] E4M3,
    ``scales`` [rows*128] UE8M0, ``ids`` / ``weights`` [rows*8] token-major top-8; writes BF16 [rows*4096]."""
    payload = np.ascontiguousarray(payload, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    if rows == 0 or payload.size != rows * H or scales.size != rows * H // 32:
        raise ExpertError(1, f"b1 ffn: extents do not match {rows} rows")
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    return _ffn_raw(layer, scratch, payload.ctypes.data, H, scales.ctypes.data, H // 32, ids, weights, rows, bf16_out)


def ffn_strided(layer: Layer, scratch: Scratch, hidden: np.ndarray, row_stride: int, ids: np.ndarray,
                weights: np.ndarray, rows: int, bf16_out: np.ndarray) -> FfnStats:
    """``ffn`` on the request frame's interleaved rows read in place (b1.rs:154-176): each row is
    4096 payload bytes followed by its 128 scale bytes, ``row_stride`` bytes apart."""
    hidden = np.ascontiguousarray(hidden, dtype=np.uint8)
    if rows == 0 or row_stride < H + H // 32 or hidden.size < (rows - 1) * row_stride + H + H // 32:
        raise ExpertError(1, f"b1 ffn: hidden rows do not match {rows} rows of {row_stride} B")
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    base = hidden.ctypes.data
    return _ffn_raw(layer, scratch, base, row_stride, base + H, row_stride, ids, weights, rows, bf16_out)


def ffn_tp(layer: Layer, scratch: Scratch, exchange: "Exchange", payload, scales, ids, weights, rows: int, sum_out=None) -> FfnStats:
    """``ffn`` for one rank of a tensor-parallel group: host rows in, the rank-ordered FP32 sum of every rank's plane out
    (``sum_out`` [rows*4096] float32 in host memory, or None on ranks that do not need it). Arguments are host arrays or
    addresses of (pinned) host buffers. Every rank of the group makes the call for every request."""
    ms = (C.c_float * 8)()
    err = C.create_string_buffer(256)
    rc = _native.lib().m26b_ffn_tp(layer._h, scratch._h, exchange._h, _ptr(payload), H, _ptr(scales), H // 32, _ptr(ids),
                                   _ptr(weights), rows, _ptr(sum_out), ms, err, 256)
    _check(rc, err)
    return FfnStats(ms[0], ms[1], ms[2], int(ms[3]), (ms[4], ms[5], ms[6], ms[7]))


X_BF16, X_F32, X_E4M3 = 0, 1, 2
CODEC_WIRE, CODEC_QUANT_V1 = 0, 1


def ffn_dev(layer: Layer, scratch: Scratch, x, ids, weights, rows: int, bf16_out, *, x_dtype: int = X_BF16,
            x_scales=None, codec: int = CODEC_WIRE, partial_out=None, stream=None) -> None:
    """Device-resident FFN: enqueue on ``stream`` and return; ``Scratch.status`` reports faults."""
    err = C.create_string_buffer(256)
    rc = _native.lib().m26b_ffn_dev(layer._h, scratch._h, _ptr(x), x_dtype, _ptr(x_scales), codec, _ptr(ids),
                                    _ptr(weights), rows, _ptr(bf16_out), _ptr(partial_out), _ptr(stream), err, 256)
    _check(rc, err)


def ffn_tp_dev(layer: Layer, scratch: Scratch, exchange: "Exchange", x, ids, weights, rows: int, sum_out, *,
               x_dtype: int = X_BF16, x_scales=None, codec: int = CODEC_WIRE, residual=None, stream=None) -> None:
    """``ffn_dev`` for a rank of a tensor-parallel group, with the combine and the plane exchange in one kernel: leaves
    the rank-ordered FP32 sum of every rank's BF16 plane (+ ``residual``) in ``sum_out`` [rows, 4096] on every rank.
    One step of ``exchange``; every rank makes the call. ``Scratch.status`` / ``Exchange.status`` report faults."""
    err = C.create_string_buffer(256)
    rc = _native.lib().m26b_ffn_tp_dev(layer._h, scratch._h, exchange._h, _ptr(x), x_dtype, _ptr(x_scales), codec, _ptr(ids),
                                       _ptr(weights), rows, _ptr(residual), _ptr(sum_out), _ptr(stream), err, 256)
    _check(rc, err)


def quantize_dev(x, x_dtype: int, n_elems: int, codec: int, payload, scales, fault, stream=None) -> None:
    err = C.create_string_buffer(256)
    _check(_native.lib().m26b_quantize_dev(_ptr(x), x_dtype, n_elems, codec, _ptr(payload), _ptr(scales), _ptr(fault),
                                           _ptr(stream), err, 256), err)


def produce_dev(logits, bias, rows: int, ids_out, weights_out, x=None, x_dtype: int = X_BF16, codec: int = CODEC_WIRE,
                payload=None, scales=None, fault=None, stream=None) -> None:
    """Router top-8 from FP32 logits [rows, 256] (router.rs:42-80) and, when ``x`` is given, the activation quantiser,
    in one launch. Outputs are what ``ffn_dev`` takes."""
    err = C.create_string_buffer(256)
    _check(_native.lib().m26b_produce_dev(_ptr(logits), _ptr(bias), rows, _ptr(ids_out), _ptr(weights_out), _ptr(x), x_dtype,
                                          codec, _ptr(payload), _ptr(scales), _ptr(fault), _ptr(stream), err, 256), err)


def route_reduce_dev(y, weights, rows: int, partial, bf16, fault, stream=None) -> None:
    err = C.create_string_buffer(256)
    _check(_native.lib().m26b_route_reduce_dev(_ptr(y), _ptr(weights), rows, _ptr(partial), _ptr(bf16), _ptr(fault),
                                               _ptr(stream), err, 256), err)


def rank_sum_dev(planes, n: int, out, stream=None, residual=None) -> None:
    """FP32 sum of BF16 planes in rank order; ``planes`` is a sequence of device buffers. With ``residual`` the
    coordinator's ``h += f`` is folded in: out = residual + sum (``residual`` may be ``out`` itself)."""
    arr = (C.c_void_p * len(planes))(*[_ptr(p) for p in planes])
    err = C.create_string_buffer(256)
    _check(_native.lib().m26b_rank_sum_residual_dev(arr, len(planes), n, _ptr(residual), _ptr(out), _ptr(stream), err, 256), err)


class Exchange:
    """This rank's window of the plane exchange between the GPUs of one box (one process per GPU).

    ``plane()`` is the device address the next step's BF16 plane goes to (pass it as ``bf16_out`` of ``ffn_dev``);
    ``sum(n, out_f32)`` enqueues the one kernel that publishes the plane, waits for the peers' and adds all planes in
    rank order, reading the peers' over NVLink. Stands where the reference has the RDMA return path and the
    coordinator's sum (crates/mimo26-wire/src/l4.rs:169-244, crates/mimo26-coordinator/kernels/glue.cu:202-213)."""

    HANDLE_BYTES = 64

    def __init__(self, plane_bytes: int, rank: int, world: int, export: bool = True):
        out, err = C.c_void_p(), C.create_string_buffer(256)
        self.handle = (C.c_uint8 * self.HANDLE_BYTES)() if export else None
        _check(_native.lib().m26b_exchange_new(plane_bytes, rank, world, C.byref(out),
                                               C.addressof(self.handle) if export else None, err, 256), err)
        self._h, self.rank, self.world, self.plane_bytes = out, rank, world, plane_bytes

    def handle_bytes(self) -> bytes:
        return bytes(self.handle)

    def connect(self, handles: bytes) -> None:
        """``handles``: every rank's ``handle_bytes()`` concatenated in rank order."""
        if len(handles) != self.world * self.HANDLE_BYTES:
            raise ExpertError(1, "m26b exchange connect: need one 64-byte handle per rank")
        buf = (C.c_uint8 * len(handles)).from_buffer_copy(handles)
        err = C.create_string_buffer(256)
        _check(_native.lib().m26b_exchange_connect(self._h, C.addressof(buf), err, 256), err)

    def connect_local(self, windows) -> None:
        arr = (C.c_void_p * self.world)(*[w._h.value for w in windows])
        err = C.create_string_buffer(256)
        _check(_native.lib().m26b_exchange_connect_local(self._h, arr, err, 256), err)

    def plane(self) -> int:
        return int(_native.lib().m26b_exchange_plane(self._h))

    def set_wait_ms(self, ms: int) -> None:
        _native.lib().m26b_exchange_set_wait_ms(self._h, ms)

    def publish_as(self, peer_rank: int, stream=None) -> None:
        err = C.create_string_buffer(256)
        _check(_native.lib().m26b_exchange_publish_as(self._h, peer_rank, _ptr(stream), err, 256), err)

    def sum(self, n_elems: int, out_f32, stream=None, residual=None) -> None:
        """out = rank-ordered sum of every rank's plane (+ ``residual``, which may be ``out_f32`` itself)."""
        err = C.create_string_buffer(256)
        _check(_native.lib().m26b_exchange_sum_residual_dev(self._h, n_elems, _ptr(residual), _ptr(out_f32), _ptr(stream), err, 256), err)

    def status(self, stream=None) -> None:
        err = C.create_string_buffer(256)
        _check(_native.lib().m26b_exchange_status(self._h, _ptr(stream), err, 256), err)

    def close(self) -> None:
        if self._h:
            _native.lib().m26b_exchange_free(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ExpertParallel:
    """This rank's side of expert parallelism inside one box (one process per GPU): experts are split over the ranks,
    tokens too; token rows are read from their owners and result rows written to them through peer mappings.
    ``step`` = ``begin`` + ``compute`` + ``finish``; every rank runs the three in the same order."""

    HANDLE_BYTES = 64

    def __init__(self, tokens: int, rank: int, world: int, export: bool = True):
        out, err = C.c_void_p(), C.create_string_buffer(256)
        self.handle = (C.c_uint8 * self.HANDLE_BYTES)() if export else None
        _check(_native.lib().m26b_ep_new(tokens, rank, world, C.byref(out), C.addressof(self.handle) if export else None,
                                         err, 256), err)
        self._h, self.rank, self.world, self.tokens = out, rank, world, tokens

    def handle_bytes(self) -> bytes:
        return bytes(self.handle)

    def rows(self, rank=None) -> int:
        return _native.lib().m26b_ep_rows(self._h, self.rank if rank is None else rank)

    def connect(self, handles: bytes) -> None:
        if len(handles) != self.world * self.HANDLE_BYTES:
            raise ExpertError(1, "m26b ep connect: need one 64-byte handle per rank")
        buf = (C.c_uint8 * len(handles)).from_buffer_copy(handles)
        err = C.create_string_buffer(256)
        _check(_native.lib().m26b_ep_connect(self._h, C.addressof(buf), err, 256), err)

    def connect_local(self, all_ranks) -> None:
        arr = (C.c_void_p * self.world)(*[w._h.value for w in all_ranks])
        err = C.create_string_buffer(256)
        _check(_native.lib().m26b_ep_connect_local(self._h, arr, err, 256), err)

    def set_wait_ms(self, ms: int) -> None:
        _native.lib().m26b_ep_set_wait_ms(self._h, ms)

    def set_route_output(self, bf16: bool) -> None:
        """Result rows cross NVLink and are combined as BF16 instead of FP32; every rank must use the same setting."""
        if _native.lib().m26b_ep_set_route_output(self._h, 1 if bf16 else 0):
            raise ExpertError(1, "m26b ep: bad route-output type")

    def publish_as(self, peer_rank: int, which: int, stream=None) -> None:
        err = C.create_string_buffer(256)
        _check(_native.lib().m26b_ep_publish_as(self._h, peer_rank, which, _ptr(stream), err, 256), err)

    def begin(self, x, ids, weights, rows: int, *, x_dtype: int = 0, x_scales=None, codec: int = 0, stream=None) -> None:
        err = C.create_string_buffer(256)
        _check(_native.lib().m26b_ep_begin_dev(self._h, _ptr(x), x_dtype, _ptr(x_scales), codec, _ptr(ids), _ptr(weights), rows,
                                               _ptr(stream), err, 256), err)

    def compute(self, layer: "Layer", scratch: "Scratch", stream=None) -> None:
        err = C.create_string_buffer(256)
        _check(_native.lib().m26b_ep_compute_dev(self._h, layer._h, scratch._h, _ptr(stream), err, 256), err)

    def finish(self, bf16_out, partial_out=None, stream=None) -> None:
        err = C.create_string_buffer(256)
        _check(_native.lib().m26b_ep_finish_dev(self._h, _ptr(bf16_out), _ptr(partial_out), _ptr(stream), err, 256), err)

    def step(self, layer, scratch, x, ids, weights, rows, bf16_out, *, partial_out=None, x_dtype=0, x_scales=None, codec=0,
             stream=None) -> None:
        self.begin(x, ids, weights, rows, x_dtype=x_dtype, x_scales=x_scales, codec=codec, stream=stream)
        self.compute(layer, scratch, stream=stream)
        self.finish(bf16_out, partial_out, stream=stream)

    def ffn_host(self, layer: "Layer", scratch: "Scratch", payload, scales, ids, weights, rows: int, bf16_out) -> None:
        """One step from host memory: this rank's quantised rows, ids and weights up, its BF16 rows back (synchronous)."""
        err = C.create_string_buffer(256)
        _check(_native.lib().m26b_ep_ffn(self._h, layer._h, scratch._h, _ptr(payload), H, _ptr(scales), H // 32, _ptr(ids),
                                         _ptr(weights), rows, _ptr(bf16_out), err, 256), err)

    def status(self, stream=None) -> None:
        err = C.create_string_buffer(256)
        _check(_native.lib().m26b_ep_status(self._h, _ptr(stream), err, 256), err)

    def close(self) -> None:
        if self._h:
            _native.lib().m26b_ep_free(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


PLAN_STATIC_MAX_ROWS = 4096


def plan_static(ids, weights, rows: int, inverse, original_routes, grouped_weights, meta, stream=None) -> None:
    """Stable route plan that allocates nothing: for callers that must not touch the device allocator while
    they run (all free memory already committed to weights, or no tolerance for cudaMalloc's device-wide stall).
    Device buffers in and out; at most ``PLAN_STATIC_MAX_ROWS`` rows. The planner's working memory is a fixed array
    inside the library shared by every call on the GPU, so calls that overlap on the device race."""
    err = C.create_string_buffer(256)
    _check(_native.lib().m26b_plan_static(_ptr(ids), _ptr(weights), rows, _ptr(inverse), _ptr(original_routes),
                                          _ptr(grouped_weights), _ptr(meta), _ptr(stream), err, 256), err)
