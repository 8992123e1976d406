"""DS41RTE3 v3 frames: layout contracts, the checksum and the rejection rules, through the C ABI (no GPU needed).

Pins available in the reference tree: the RFC 3720 check value of CRC32C (crates/mimo26-wire/tests/wire_layout.rs:128-131),
the table-against-bitwise cross-check of the same file (300-321), the row contracts 4,360 / 8,192 bytes and the field
offsets of src/layout.rs, the dtype / kind / flag codes. The reference holds no stored encoded frame (its tests encode
with its own encoder), so the frame bytes are checked field by field against layout.rs here."""
import struct

import numpy as np
import pytest


def crc32c_bitwise(data: bytes) -> int:
    crc = 0xFFFFFFFF
    for b in data:
        crc ^= b
        for _ in range(8):
            crc = (crc >> 1) ^ 0x82F63B78 if crc & 1 else crc >> 1
    return crc ^ 0xFFFFFFFF


def make_request(rows=3, seed=1, **kw):
    from mimo26f_afd_b200 import frames

    rng = np.random.default_rng(seed)
    p = rng.integers(0, 256, (rows, 4096), dtype=np.uint8)
    s = rng.integers(105, 248, (rows, 128), dtype=np.uint8)
    ids = np.stack([rng.permutation(256)[:8] for _ in range(rows)]).astype(np.int32)
    w = rng.random((rows, 8), dtype=np.float32)
    return frames.encode_request(p, s, ids, w, **kw), (p, s, ids, w)


def test_crc32c_known_answers_and_bitwise_cross_check():
    from mimo26f_afd_b200 import frames

    assert frames.crc32c(b"123456789") == 0xE3069283            # RFC 3720 / iSCSI check value
    assert frames.crc32c(b"") == 0
    x, long = 0x12345678, bytearray()
    for _ in range(1024):                                       # the reference test's LCG byte string
        x = (x * 1664525 + 1013904223) & 0xFFFFFFFF
        long.append(x >> 24)
    for sample in (b"a", b"123456789", bytes(300), bytes(long), bytes(long[3:517])):
        assert frames.crc32c(sample) == crc32c_bitwise(sample) == frames.crc32c_table(sample)
    assert frames.crc32c(b"123456789") != 0xCBF43926            # that is CRC-32 (IEEE), the wrong family


def test_row_contracts_and_request_layout_field_by_field():
    from mimo26f_afd_b200 import frames

    assert frames.request_bytes(1) - 128 == 4360 and frames.return_bytes(1) - 128 == 8192
    rows = 3
    f, (p, s, ids, w) = make_request(rows, request_id=0x1122334455667788, layer_id=41, executor_id=7, seq=99)
    assert len(f) == 128 + rows * 4360
    assert f[0:8] == b"DS41RTE3"
    version, kind, header_len = struct.unpack_from("<HHI", f, 8)
    assert (version, kind, header_len) == (3, 1, 128)
    request_id, placement, layer, row_count, dim, dtype, source = struct.unpack_from("<QQIIIHH", f, 16)
    assert (request_id, placement, layer, row_count, dim, dtype, source) == (0x1122334455667788, 1, 41, rows, 4096, 7, 1)
    route_count, desc_bytes, route_bytes = struct.unpack_from("<III", f, 48)
    assert (route_count, desc_bytes, route_bytes) == (rows * 8, rows * 40, rows * 96)
    payload_bytes, logical, wire = struct.unpack_from("<QQQ", f, 60)
    assert (payload_bytes, logical, wire) == (rows * 4224, rows * 4360, len(f))
    flags, stride, status = struct.unpack_from("<III", f, 84)
    assert (flags, stride, status) == (0, 4224, 0)
    executor, position, seq, crc, reserved = struct.unpack_from("<QQQII", f, 96)
    assert (executor, position, seq, reserved) == (7, 0, 99, 0)
    zeroed = bytearray(f); zeroed[120:124] = b"\0\0\0\0"
    assert crc == crc32c_bitwise(bytes(zeroed))                 # checksum over the frame with its own field zero
    for t in range(rows):                                       # 40-byte descriptors
        row_id, sk, pad0, src_req, pos, r_off, r_cnt, pad1 = struct.unpack_from("<QHHQQIII", f, 128 + 40 * t)
        assert (row_id, sk, pad0, src_req, pos, r_off, r_cnt, pad1) == (t, 1, 0, 0x1122334455667788, t, 8 * t, 8, 0)
    base = 128 + 40 * rows
    for j in range(rows * 8):                                   # 12-byte route entries: row, expert, weight
        row_index, expert, weight = struct.unpack_from("<IIf", f, base + 12 * j)
        assert (row_index, expert) == (j // 8, ids.reshape(-1)[j]) and weight == w.reshape(-1)[j]
    base += 96 * rows
    body = np.frombuffer(f, np.uint8, offset=base).reshape(rows, 4224)
    assert np.array_equal(body[:, :4096], p) and np.array_equal(body[:, 4096:], s)
    assert frames.check_request(f) == (rows, 0x1122334455667788, 41)


def test_request_rejections_name_their_reason():
    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import frames

    f, _ = make_request(2)

    def rejected(frame, word, check_crc=True):
        with pytest.raises(M.ExpertError) as e:
            frames.check_request(bytes(frame), check_crc)
        assert e.value.code == 6 and word in e.value.message, e.value.message

    b = bytearray(f); b[0] = ord("X"); rejected(b, "magic")
    b = bytearray(f); b[8] = 2; rejected(b, "version")
    b = bytearray(f); b[10] = 9; rejected(b, "kind")
    rejected(f[:-1], "truncated")
    rejected(f + b"\0", "trailing")
    rejected(f[:100], "too short")
    b = bytearray(f); b[5000] ^= 0x10; rejected(b, "corrupt")       # one flipped payload bit
    b = bytearray(f); b[40] ^= 0x01; rejected(b, "corrupt")         # one flipped header bit: the header is covered too
    # with the checksum off (the reference's MIMO26_WIRE_NOCRC=1 mode) the structural rules still hold
    b = bytearray(f); struct.pack_into("<I", b, 88, 4228); rejected(b, "payload_bytes", check_crc=False)
    b = bytearray(f); struct.pack_into("<I", b, 40, 2048); rejected(b, "hidden_dim", check_crc=False)
    b = bytearray(f); struct.pack_into("<H", b, 44, 1); rejected(b, "dtype", check_crc=False)
    b = bytearray(f); struct.pack_into("<I", b, 128 + 32, 7); rejected(b, "routes, want 8", check_crc=False)
    b = bytearray(f); struct.pack_into("<I", b, 128 + 80, 1); rejected(b, "route row", check_crc=False)       # entry 0 names row 1
    b = bytearray(f); struct.pack_into("<I", b, 128 + 28, 12); rejected(b, "route range", check_crc=False)
    b = bytearray(f); struct.pack_into("<I", b, 36, 0); rejected(b, "row_count", check_crc=False)


def test_return_frame_rules():
    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import frames

    rows = 2
    body = np.arange(rows * 4096, dtype="<u2").tobytes()
    hdr = bytearray(128)
    hdr[0:8] = b"DS41RTE3"
    struct.pack_into("<HHI", hdr, 8, 3, 2, 128)
    struct.pack_into("<QQIIIHH", hdr, 16, 55, 1, 4, rows, 4096, 1, 1)
    struct.pack_into("<III", hdr, 48, 8, 0, 0)
    struct.pack_into("<QQQ", hdr, 60, rows * 8192, rows * 8192, 128 + rows * 8192)
    struct.pack_into("<III", hdr, 84, (1 << 9) | (1 << 16), 8192, 0)
    struct.pack_into("<QQQ", hdr, 96, 0, 0, 12)
    frame = bytearray(bytes(hdr) + body)
    struct.pack_into("<I", frame, 120, crc32c_bitwise(bytes(frame)))
    meta, got = frames.parse_return(bytes(frame))
    assert meta == dict(request_id=55, layer_id=4, rows=rows, status=0, seq=12)
    assert np.array_equal(got.reshape(-1), np.arange(rows * 4096, dtype=np.uint16))
    bad = bytearray(frame); struct.pack_into("<I", bad, 84, 1 << 9)     # not marked compact BF16: the per-route FP32 wall
    with pytest.raises(M.ExpertError) as e:
        frames.parse_return(bytes(bad), check_crc=False)
    assert e.value.code == 6 and "pre-summed" in e.value.message
    with pytest.raises(M.ExpertError):
        frames.parse_return(bytes(frame[:-2]))


@pytest.mark.gpu
def test_serve_frame_round_trip_equals_the_host_entry_point():
    import torch

    import mimo26f_afd_b200 as M
    import oracle
    from mimo26f_afd_b200 import frames, synth

    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    seed, tokens = synth.MASTER_SEED, 6
    wts = synth.layer_torch(seed, dev)
    layer = M.Layer.from_checkpoint(*[wts[n] for n in synth.TENSORS])
    del wts
    scratch = M.Scratch()
    x = synth.bf16_to_f32_np(synth.activations_bf16(seed, tokens))
    ids, w = synth.routing(seed, tokens, 0.0)
    xq, xs = oracle.quant_wire(x)
    want = np.zeros((tokens, 4096), np.uint16)
    M.ffn(layer, scratch, xq.reshape(-1), xs.reshape(-1), ids.reshape(-1), w.reshape(-1), tokens, want.reshape(-1))
    request = frames.encode_request(xq, xs, ids, w, request_id=900, layer_id=17, executor_id=3, seq=5)
    reply = frames.serve_frame(layer, scratch, request, reply_seq=6)
    assert len(reply) == 128 + tokens * 8192
    meta, rows = frames.parse_return(reply)
    assert meta == dict(request_id=900, layer_id=17, rows=tokens, status=0, seq=6)
    assert np.array_equal(rows, want)
    flags, stride = struct.unpack_from("<II", reply, 84)
    assert flags == (1 << 9) | (1 << 16) and stride == 8192
    zeroed = bytearray(reply); zeroed[120:124] = b"\0\0\0\0"
    assert struct.unpack_from("<I", reply, 120)[0] == crc32c_bitwise(bytes(zeroed))
    corrupt = bytearray(request); corrupt[3000] ^= 4
    with pytest.raises(M.ExpertError) as e:
        frames.serve_frame(layer, scratch, bytes(corrupt))
    assert e.value.code == 6
    dup = ids.copy(); dup[1, 3] = dup[1, 0]                     # the plan's own rejection comes through the frame path
    with pytest.raises(M.ExpertError) as e:
        frames.serve_frame(layer, scratch, frames.encode_request(xq, xs, dup, w))
    assert e.value.code == 3
    again = frames.serve_frame(layer, scratch, request, check_crc=False)
    assert struct.unpack_from("<I", again, 120)[0] == 0 and np.array_equal(frames.parse_return(again, check_crc=False)[1], want)
