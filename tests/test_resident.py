"""The expert rank's serving state without a GPU: manifest index of a rank, grouped images read on demand, layers
prepared on first touch exactly once, error-status returns (crates/mimo26-spark/src/resident.rs, main.rs:104-146)."""
import os

import numpy as np
import pytest

from mimo26f_afd_b200 import frames, resident, staging
from test_staging import checkpoint, expert_tensors, write_safetensors  # noqa: F401  (fixture and helpers)


class FakeLayer:
    def __init__(self, image):
        self.image = image

    def all_scales_normal(self):
        return True


def test_resident_index_and_grouped_image(checkpoint, tmp_path):
    out = str(tmp_path / "s")
    staging.repack(checkpoint, out, ranks=4, layers=[1], experts=[0, 1, 2])
    r = resident.Resident(out, rank=2)
    assert r.ranks == 4 and r.slices == 3
    img = r.grouped_image(1, experts=3)
    assert img.size == 3 * 3342336
    assert img[:3342336].tobytes() == open(os.path.join(out, staging.slice_file_name(1, 0, 2)), "rb").read()
    with pytest.raises(staging.StagingError) as e:
        r.grouped_image(1)                                     # experts 3..255 were not staged
    assert "missing slice L01_E003" in str(e.value)
    blob = bytearray(open(os.path.join(out, staging.slice_file_name(1, 1, 2)), "rb").read()); blob[7] ^= 1
    open(os.path.join(out, staging.slice_file_name(1, 1, 2)), "wb").write(blob)
    with pytest.raises(staging.StagingError):
        resident.Resident(out, rank=2)                         # the boot readback refuses this rank
    assert resident.Resident(out, rank=3).slices == 3          # ... but not the others


def test_layers_are_prepared_once_and_failures_become_error_returns(checkpoint, tmp_path):
    import mimo26f_afd_b200 as M

    out = str(tmp_path / "s")
    staging.repack(checkpoint, out, ranks=4, layers=[1], experts=[0, 1, 2])
    r = resident.Resident(out, rank=0)
    r.grouped_image = lambda layer, experts=3, _g=r.grouped_image: _g(layer, 3)     # a three-expert "layer" for this test
    prepared, served = [], []

    def prepare(image, rank, ranks):
        prepared.append((image.size, rank, ranks))
        return FakeLayer(image)

    def serve(layer, scratch, request, check_crc, seq):
        served.append(seq)
        if len(served) == 2:
            raise M.ExpertError(3, "m26b plan: invalid routes (id/residency/weight/duplicate)")
        return b"reply"

    rank = resident.ExpertRank(r, prepare=prepare, serve=serve, log=None)
    rng = np.random.default_rng(0)
    rows = 2
    req = frames.encode_request(rng.integers(0, 255, (rows, 4096), dtype=np.uint8), np.full((rows, 128), 120, np.uint8),
                                np.tile(np.arange(8, dtype=np.int32), (rows, 1)), np.full((rows, 8), 0.125, np.float32),
                                request_id=41, layer_id=1, executor_id=6)
    assert rank.handle(req) == b"reply" and prepared == [(3 * 3342336, 0, 4)] and rank.load_ms[1] > 0
    reply = rank.handle(req)                                   # second call: the serve function fails
    assert len(prepared) == 1                                  # the layer was not prepared again
    with pytest.raises(M.ExpertError):
        frames.parse_return(reply[:-1])
    import struct

    assert len(reply) == 128 + rows * 8192 and not any(reply[128:])
    kind, = struct.unpack_from("<H", reply, 10)
    request_id, = struct.unpack_from("<Q", reply, 16)
    flags, stride, status = struct.unpack_from("<III", reply, 84)
    executor, _, seq = struct.unpack_from("<QQQ", reply, 96)
    assert (kind, request_id, flags, stride, status, executor, seq) == (2, 41, 0, 8192, 1, 6, 2)
    meta, body = frames.parse_return(reply)                    # an error return is still a well-formed, sealed frame
    assert meta["status"] == 1 and meta["rows"] == rows and not body.any()
    other = frames.encode_request(rng.integers(0, 255, (1, 4096), dtype=np.uint8), np.full((1, 128), 120, np.uint8),
                                  np.arange(8, dtype=np.int32)[None], np.full((1, 8), 0.125, np.float32), layer_id=9)
    reply = rank.handle(other)                                 # a layer that was never staged
    assert frames.parse_return(reply)[0]["status"] == 1 and len(prepared) == 1
    with pytest.raises(M.ExpertError):
        rank.handle(req[:-3])                                  # not a frame at all: that is the transport's problem
