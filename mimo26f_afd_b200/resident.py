"""One expert rank's serving state: the verified slice files of its rank, layers prepared on first touch, and the
per-request function that turns a request frame into a return frame (an error-status frame when the request fails).

Mirrors the expert daemon of the reference: ``Resident`` (``crates/mimo26-spark/src/resident.rs``: manifest index,
grouped image of a layer read on demand, no host-side copy kept), ``ensure_b1_layer`` (``src/main.rs:126-146``: read,
upload, prepare, free the canonical device copy, warn on exceptional scales), the request loop
(``main.rs:348-460``) and ``error_return_for`` (``main.rs:104-122``: status Error, flags 0, zero rows, ids copied).
The transport is the caller's; this is the work between receiving a frame and sending one.
"""
from __future__ import annotations

import os
import struct
import sys
import time

import numpy as np

from . import staging


class Resident:
    """(layer, expert) -> slice file of one rank, from the manifest of a staged directory. ``verify=True`` runs the
    identity readback of that rank first and refuses to construct on any mismatch."""

    def __init__(self, directory: str, rank: int, verify: bool = True):
        self.dir, self.rank = directory, rank
        if verify:
            staging.readback(directory, rank)
        with open(os.path.join(directory, staging.MANIFEST_NAME)) as f:
            man = staging.parse_manifest(f.read())
        self.ranks = man["geometry"]["ep_ranks"]
        if not 0 <= rank < self.ranks:
            raise staging.StagingError(f"rank {rank} of {self.ranks}")
        self.files = {(s["layer"], s["expert"]): s["file"] for s in man["slices"] if s["rank"] == rank}
        self.slices = len(self.files)

    def slice(self, layer: int, expert: int) -> bytes:
        if (layer, expert) not in self.files:
            raise staging.StagingError(f"missing slice L{layer:02d}_E{expert:03d}")
        with open(os.path.join(self.dir, self.files[(layer, expert)]), "rb") as f:
            return f.read()

    def grouped_image(self, layer: int, experts: int = staging.EXPERTS_PER_LAYER) -> np.ndarray:
        """The layer's slices in expert-id order, back to back (the image ``Layer.new_tp`` takes)."""
        return np.frombuffer(b"".join(self.slice(layer, e) for e in range(experts)), np.uint8)


def _prepare_on_device(image: np.ndarray, rank: int, ranks: int):
    import torch

    from .expert import Layer

    dev = torch.from_numpy(image).cuda()                      # the canonical copy lives only until the layer is prepared
    layer = Layer.new_tp(dev, image.size, rank, ranks)
    del dev
    return layer


class ExpertRank:
    """Layers prepared on first touch and the per-request function. ``prepare(image, rank, ranks)`` and
    ``serve(layer, scratch, request, check_crc, reply_seq)`` are injectable so the bookkeeping runs without a GPU."""

    def __init__(self, resident: Resident, scratch=None, prepare=_prepare_on_device, serve=None, check_crc: bool = True,
                 log=sys.stderr):
        self.resident, self.scratch, self.prepare, self.check_crc, self.log = resident, scratch, prepare, check_crc, log
        if serve is None:
            from . import frames

            serve = lambda layer, scratch, request, check_crc, seq: frames.serve_frame(layer, scratch, request, check_crc=check_crc, reply_seq=seq)
        self.serve = serve
        self.layers, self.load_ms, self.seq = {}, {}, 0

    def ensure_layer(self, layer_id: int) -> float:
        """Milliseconds spent preparing ``layer_id`` (0.0 when it is already resident)."""
        if layer_id in self.layers:
            return 0.0
        t0 = time.perf_counter()
        image = self.resident.grouped_image(layer_id)
        layer = self.prepare(image, self.resident.rank, self.resident.ranks)
        if hasattr(layer, "all_scales_normal") and not layer.all_scales_normal() and self.log:
            print(f"L{layer_id}: exceptional weight scales present (byte 255 is served as 254)", file=self.log)
        self.layers[layer_id] = layer
        self.load_ms[layer_id] = (time.perf_counter() - t0) * 1e3
        return self.load_ms[layer_id]

    def handle(self, request: bytes) -> bytes:
        """Request frame -> return frame. A request that cannot be served (unknown layer, rejected plan, numerical
        fault) gets an error-status return carrying its ids; a frame that is not a valid request raises."""
        from . import frames
        from .expert import ExpertError

        rows, request_id, layer_id = frames.check_request(request, self.check_crc)
        self.seq += 1
        try:
            self.ensure_layer(layer_id)
            return self.serve(self.layers[layer_id], self.scratch, request, self.check_crc, self.seq)
        except (ExpertError, staging.StagingError) as e:
            if self.log:
                print(f"request {request_id} layer {layer_id}: {e}", file=self.log)
            return error_return(request, rows, self.seq, self.check_crc)


def error_return(request: bytes, rows: int, seq: int, seal: bool = True) -> bytes:
    """main.rs:104-122: the request's ids, status Error, flags 0, ``rows`` zero rows of 8,192 bytes."""
    from . import frames

    request_id, placement = struct.unpack_from("<QQ", request, 16)
    (layer_id,) = struct.unpack_from("<I", request, 32)
    executor_id, token_position = struct.unpack_from("<QQ", request, 96)
    h = bytearray(128)
    h[0:8] = b"DS41RTE3"
    struct.pack_into("<HHI", h, 8, 3, 2, 128)
    struct.pack_into("<QQIIIHH", h, 16, request_id, placement, layer_id, rows, 4096, 1, 1)
    struct.pack_into("<III", h, 48, 8, 0, 0)
    struct.pack_into("<QQQ", h, 60, rows * 8192, rows * 8192, 128 + rows * 8192)
    struct.pack_into("<III", h, 84, 0, 8192, 1)
    struct.pack_into("<QQQ", h, 96, executor_id, token_position, seq)
    frame = bytearray(bytes(h) + bytes(rows * 8192))
    if seal:
        struct.pack_into("<I", frame, 120, frames.crc32c(bytes(frame)))
    return bytes(frame)
