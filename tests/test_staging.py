"""Offline staging with identity (CPU only): safetensors header reader, slice layout v2, manifest v2, boot readback.
Mirrors the reference's crates/mimo26-repack tests: layout offsets and totals (tests/layout.rs), reader refusals
(tests/safetensors_reader.rs), manifest strictness (tests/manifest.rs), determinism (tests/determinism.rs), identity
readback that reports every bad file and refuses v1 (tests/identity_readback.rs), TP4 slices against the rank geometry
(tests/tp4_identity.rs), SHA-256 known answers (tests/sha256_vectors.rs)."""
import json
import os
import struct

import numpy as np
import pytest

from mimo26f_afd_b200 import staging, synth

SEED = 0x26AFD


def write_safetensors(path, tensors, metadata=None):
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, arr in tensors.items():
        b = np.ascontiguousarray(arr, np.uint8).tobytes()
        header[name] = dict(dtype="U8", shape=list(arr.shape), data_offsets=[off, off + len(b)])
        blobs.append(b)
        off += len(b)
    text = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + b"".join(blobs))


def expert_tensors(layer, expert):
    names = {"gate_w": ("gate_proj", False), "gate_s": ("gate_proj", True), "up_w": ("up_proj", False), "up_s": ("up_proj", True),
             "down_w": ("down_proj", False), "down_s": ("down_proj", True)}
    return {staging.tensor_name(layer, expert, proj, scale): synth.expert_tensor_np(SEED + layer, key, expert)
            for key, (proj, scale) in names.items()}


@pytest.fixture()
def checkpoint(tmp_path):
    d = tmp_path / "ckpt"
    d.mkdir()
    tensors = {}
    for e in (0, 1, 2):
        tensors.update(expert_tensors(1, e))
    write_safetensors(d / "model_pp0_ep0_shard0.safetensors", tensors, metadata={"format": "pt"})
    return str(d)


def test_layout_offsets_and_totals():
    t = staging.layout_table(4)
    assert [(r["proj"], r["region"], r["off"], r["len"]) for r in t] == [
        ("gate_proj", "payload", 0, 1048576), ("gate_proj", "scales", 1048576, 65536), ("up_proj", "payload", 1114112, 1048576),
        ("up_proj", "scales", 2162688, 65536), ("down_proj", "payload", 2228224, 1048576), ("down_proj", "scales", 3276800, 65536)]
    assert staging.slice_bytes(4) == 3342336 and staging.EXPERT_BYTES == 13369344
    for g in (1, 2, 4, 8):
        assert staging.layout_table(g)[-1]["off"] + staging.layout_table(g)[-1]["len"] == staging.EXPERT_BYTES // g
    assert staging.slice_file_name(1, 0, 0) == "L01_E000_R0.slice"
    assert staging.tensor_name(3, 17, "down_proj", True) == "model.layers.3.mlp.experts.17.down_proj.weight_scale"


def test_sha256_known_answers():
    assert staging.sha256_hex(b"") == "e3b0c44298fc1c149afbf4c8996fb92427ae41e4649b934ca495991b7852b855"
    assert staging.sha256_hex(b"abc") == "ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad"


def test_slices_equal_the_rank_geometry_and_tile_the_expert(checkpoint, tmp_path):
    out = str(tmp_path / "slices")
    man = staging.repack(checkpoint, out, ranks=4, layers=[1], experts=[0, 1, 2])
    assert len(man["slices"]) == 12
    t = [synth.expert_tensor_np(SEED + 1, n, 2) for n in synth.TENSORS]
    gate_w, gate_s, up_w, up_s, down_w, down_s = t
    total = 0
    for r in range(4):
        image = np.fromfile(os.path.join(out, staging.slice_file_name(1, 2, r)), np.uint8)
        assert image.size == 3342336
        assert np.array_equal(image[:1048576].reshape(512, 2048), gate_w[512 * r:512 * (r + 1)])
        assert np.array_equal(image[1048576:1114112].reshape(512, 128), gate_s[512 * r:512 * (r + 1)])
        assert np.array_equal(image[1114112:2162688].reshape(512, 2048), up_w[512 * r:512 * (r + 1)])
        assert np.array_equal(image[2228224:3276800].reshape(4096, 256), down_w[:, 256 * r:256 * (r + 1)])
        assert np.array_equal(image[3276800:].reshape(4096, 16), down_s[:, 16 * r:16 * (r + 1)])
        total += image.size
    assert total == staging.EXPERT_BYTES                      # the four slices tile the expert: no padding, no tail
    # the same bytes the library's own test image builder makes for a rank
    tensors = {n: np.stack([synth.expert_tensor_np(SEED + 1, n, e) for e in (0, 1, 2)]) for n in synth.TENSORS}
    want = synth.canonical_rank_image_np(tensors, [0, 1, 2], 3, 4)
    got = np.concatenate([np.fromfile(os.path.join(out, staging.slice_file_name(1, e, 3)), np.uint8) for e in (0, 1, 2)])
    assert np.array_equal(got, want.reshape(-1)[:got.size]) or np.array_equal(got, want.reshape(-1))


def test_repack_is_deterministic_and_readback_matches(checkpoint, tmp_path):
    a, b = str(tmp_path / "a"), str(tmp_path / "b")
    staging.repack(checkpoint, a, ranks=2, layers=[1], experts=[0, 1])
    staging.repack(checkpoint, b, ranks=2, layers=[1], experts=[0, 1])
    for fn in sorted(os.listdir(a)):
        assert open(os.path.join(a, fn), "rb").read() == open(os.path.join(b, fn), "rb").read(), fn
    rep = staging.readback(a)
    assert len(rep) == 4 and all(s == "match" for s, _, _ in rep)
    assert len(staging.readback(a, rank=1)) == 2
    assert staging.main(["verify", a]) == 0


def test_readback_reports_every_bad_file_and_refuses(checkpoint, tmp_path):
    out = str(tmp_path / "s")
    staging.repack(checkpoint, out, ranks=4, layers=[1], experts=[0, 1])
    p0 = os.path.join(out, staging.slice_file_name(1, 0, 0))
    blob = bytearray(open(p0, "rb").read()); blob[12345] ^= 1
    open(p0, "wb").write(blob)                                                 # one flipped bit
    open(os.path.join(out, staging.slice_file_name(1, 0, 1)), "ab").write(b"\0")   # one byte too long
    os.remove(os.path.join(out, staging.slice_file_name(1, 1, 2)))                 # gone
    open(os.path.join(out, "L09_E000_R0.slice"), "wb").write(b"x")                 # not in the manifest
    with pytest.raises(staging.StagingError) as e:
        staging.readback(out)
    msg = str(e.value)
    for word in ("sha_mismatch L01_E000_R0", "size_mismatch L01_E000_R1", "missing L01_E001_R2", "unlisted L09_E000_R0"):
        assert word in msg, msg
    assert len(staging.readback(out, rank=3)) == 2            # the untouched rank still serves
    with pytest.raises(staging.StagingError):
        staging.load_rank_image(out, 1, 0)


def test_manifest_is_strict_and_version_1_is_refused(checkpoint, tmp_path):
    out = str(tmp_path / "s")
    staging.repack(checkpoint, out, ranks=4, layers=[1], experts=[0])
    text = open(os.path.join(out, staging.MANIFEST_NAME)).read()
    m = staging.parse_manifest(text)
    assert m["geometry"]["quarter_slice_bytes"] == 3342336 and staging.manifest_text(m) == text

    def refused(mutate, word):
        doc = json.loads(text)
        mutate(doc)
        with pytest.raises(staging.StagingError) as e:
            staging.parse_manifest(json.dumps(doc))
        assert word in str(e.value), str(e.value)

    refused(lambda d: d.update(version=1), "version 1")
    refused(lambda d: d.update(version=3), "version 3")
    refused(lambda d: d.update(format="other"), "format")
    refused(lambda d: d.update(extra=1), "top-level")
    refused(lambda d: d["geometry"].update(hidden=4097), "geometry")
    refused(lambda d: d["layout"][0].update(len=5), "layout")
    refused(lambda d: d["slices"][0].update(sha256="XYZ"), "sha256")
    refused(lambda d: d["slices"][0].update(bytes=7), "bytes")
    refused(lambda d: d["slices"][0].update(rank=2), "name does not match")
    refused(lambda d: d["slices"][0].pop("layer"), "slice entry fields")
    refused(lambda d: d["slices"].append(dict(d["slices"][0])), "listed twice")
    with pytest.raises(staging.StagingError):
        staging.parse_manifest(text.replace('"version": 2', '"version": 2, "version": 2'))     # duplicate key


def test_safetensors_reader_refusals(tmp_path):
    good = tmp_path / "g.safetensors"
    write_safetensors(good, {"a": np.arange(6, dtype=np.uint8).reshape(2, 3)})
    h = staging.SafetensorsHeader(str(good))
    assert np.array_equal(h.read_tensor("a"), np.arange(6, dtype=np.uint8).reshape(2, 3))
    with pytest.raises(staging.StagingError):
        h.read_tensor("b")
    raw = good.read_bytes()

    def refused(data, word):
        p = tmp_path / "bad.safetensors"
        p.write_bytes(data)
        with pytest.raises(staging.StagingError) as e:
            staging.SafetensorsHeader(str(p))
        assert word in str(e.value), str(e.value)

    refused(raw[:5], "shorter than")
    refused(struct.pack("<Q", 10 ** 9) + raw[8:], "does not fit")
    refused(struct.pack("<Q", 0) + raw[8:], "does not fit")
    refused(raw[:-1], "truncated")
    hdr_len = struct.unpack("<Q", raw[:8])[0]
    refused(raw[:8] + b"\xff" * hdr_len + raw[8 + hdr_len:], "UTF-8")
    text = json.dumps({"a": {"dtype": "U8", "shape": [6], "data_offsets": [0, 6], "extra": 1}}).encode()
    refused(struct.pack("<Q", len(text)) + text + bytes(6), "exactly dtype")
    text = b'{"a": {"dtype": "U8", "shape": [6], "data_offsets": [0, 6]}, "a": {"dtype": "U8", "shape": [6], "data_offsets": [0, 6]}}'
    refused(struct.pack("<Q", len(text)) + text + bytes(6), "duplicate")
    wrong = tmp_path / "f32.safetensors"
    text = json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}).encode()
    wrong.write_bytes(struct.pack("<Q", len(text)) + text + bytes(8))
    with pytest.raises(staging.StagingError):
        staging.SafetensorsHeader(str(wrong)).read_tensor("a")


def test_repack_names_what_is_missing(checkpoint, tmp_path):
    with pytest.raises(staging.StagingError) as e:
        staging.repack(checkpoint, str(tmp_path / "o"), ranks=4, layers=[1], experts=[0, 7])
    assert "missing tensor model.layers.1.mlp.experts.7.gate_proj.weight" in str(e.value)
    with pytest.raises(staging.StagingError):
        staging.build_slice({}, 4, 4)
