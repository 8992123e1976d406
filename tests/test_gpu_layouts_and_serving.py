"""GPU tests around the path's two ends: the weight repack as a byte permutation, staged slice files -> prepared layer ->
FFN, and the rank's serving state holding two real layers and answering request frames."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

H, I, TOPK = 4096, 2048, 8
SEED = 0x26AFD


class _DevView:
    """A device address as something torch can wrap (CUDA array interface)."""

    def __init__(self, ptr, n, typestr="|u1"):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 2}


def _image(layer, which, dev):
    import torch

    ptr, n = layer.image(which)
    return torch.as_tensor(_DevView(ptr, n), device=dev)


def _coded(n, k, bits, dev):
    """Byte k of a position code: ((index >> (bits * k)) & (2^bits - 1)) for index 0..n-1, as uint8 on the device."""
    import torch

    idx = torch.arange(n, dtype=torch.int64, device=dev)
    return ((idx >> (bits * k)) & ((1 << bits) - 1)).to(torch.uint8)


def _expected_maps(n_experts, il, dev):
    """Source position (index into the stacked source tensor of its projection) of every byte of the four operand images,
    from the documented layout, plus which projection a gate/up byte comes from (0 gate, 1 up)."""
    import torch

    ar = lambda n: torch.arange(n, dtype=torch.int64, device=dev)
    # w13 [E][il/128][256][2048]: r < 128 -> gate row 128 j + r, else up row 128 j + r - 128
    e, j, r, b = torch.meshgrid(ar(n_experts), ar(il // 128), ar(256), ar(H // 2), indexing="ij")
    w13_src = (e * il + j * 128 + (r % 128)) * (H // 2) + b
    w13_up = (r >= 128).to(torch.uint8)
    # s13 [E][il/128][32][2][512]: byte (r % 32) * 16 + (r / 32) * 4 + kb <- scales[row 128 j + r][4 c + kb]
    e, j, c, blk, o = torch.meshgrid(ar(n_experts), ar(il // 128), ar(H // 128), ar(2), ar(512), indexing="ij")
    rr, kb = (o >> 4) + 32 * ((o >> 2) & 3), o & 3
    s13_src = (e * il + j * 128 + rr) * (H // 32) + c * 4 + kb
    s13_up = blk.to(torch.uint8)
    # w2 [E][4096][il/2]: identity over the rank's K slice
    w2_src = ar(n_experts * H * (il // 2))
    # s2 [E][16][il/128][2][512]: block b covers rows 256 t + 128 b + r
    e, t, c, blk, o = torch.meshgrid(ar(n_experts), ar(H // 256), ar(il // 128), ar(2), ar(512), indexing="ij")
    rr, kb = (o >> 4) + 32 * ((o >> 2) & 3), o & 3
    s2_src = (e * H + t * 256 + blk * 128 + rr) * (il // 32) + c * 4 + kb
    return dict(w13=(w13_src.reshape(-1), w13_up.reshape(-1)), s13=(s13_src.reshape(-1), s13_up.reshape(-1)),
                w2=(w2_src, None), s2=(s2_src.reshape(-1), None))


def test_repack_is_a_byte_permutation():
    """Every source byte of the six checkpoint tensors lands exactly once in the prepared operand image, at the
    documented place, unchanged (the reference proves the same of its prepare step: kernels/b1/prepared.cuh:63-88 and
    tests/b1/host.cpp). The sources carry position codes: byte k of each position over four (payload, 8 bits each) or
    five (scales, 7 bits each, so that the reserved byte 255 does not occur) layers built from them; gate and up carry
    the same codes and are told apart by a fifth / sixth layer. 32 experts (one expert-parallel rank of eight)."""
    import torch

    import mimo26f_afd_b200 as M

    dev = torch.device("cuda:0")
    n_e = 32
    shapes = {"gate_w": (n_e, I, H // 2), "gate_s": (n_e, I, H // 32), "up_w": (n_e, I, H // 2), "up_s": (n_e, I, H // 32),
              "down_w": (n_e, H, I // 2), "down_s": (n_e, H, I // 32)}
    exp = _expected_maps(n_e, I, dev)
    got = {k: torch.zeros_like(v[0]) for k, v in exp.items()}
    names = ("gate_w", "gate_s", "up_w", "up_s", "down_w", "down_s")
    for k in range(5):
        src = {}
        for name in names:
            n = int(np.prod(shapes[name]))
            bits = 7 if name.endswith("_s") else 8
            src[name] = _coded(n, k, bits, dev).reshape(shapes[name]) if (bits == 7 or k < 4) else torch.zeros(shapes[name], dtype=torch.uint8, device=dev)
        layer = M.Layer.from_checkpoint_ep(*[src[n] for n in names], ep_rank=3, ep_size=8)
        for which in ("w13", "s13", "w2", "s2"):
            bits = 7 if which.startswith("s") else 8
            if bits == 7 or k < 4:
                got[which] |= _image(layer, which, dev).to(torch.int64) << (bits * k)
        layer.close()
        del src
    for which in ("w13", "s13", "w2", "s2"):
        want_src, _ = exp[which]
        assert torch.equal(got[which], want_src), which
    # a permutation: gate and up halves of w13 / s13 each cover their source exactly once, w2 / s2 theirs
    for which in ("w13", "s13"):
        want_src, up = exp[which]
        for half in (0, 1):
            idx = torch.sort(got[which][up == half]).values
            assert torch.equal(idx, torch.arange(idx.numel(), dtype=torch.int64, device=dev)), (which, half)
    for which in ("w2", "s2"):
        idx = torch.sort(got[which]).values
        assert torch.equal(idx, torch.arange(idx.numel(), dtype=torch.int64, device=dev)), which
    # gate and up are not swapped: gate = 0x11 everywhere, up = 0x22 everywhere
    src = {n: torch.full(shapes[n], 0x11 if n.startswith("gate") else 0x22 if n.startswith("up") else 0x33, dtype=torch.uint8, device=dev)
           for n in names}
    layer = M.Layer.from_checkpoint_ep(*[src[n] for n in names], ep_rank=0, ep_size=8)
    for which in ("w13", "s13"):
        img = _image(layer, which, dev)
        assert torch.equal(img == 0x22, exp[which][1].bool()) and torch.equal(img == 0x11, ~exp[which][1].bool()), which
    layer.close()
    # the only value the repack changes: reserved scale byte 255 is stored as 254 (crates/mimo26-expert/src/mxfp4.rs:24-29)
    for name in names:
        n = int(np.prod(shapes[name]))
        src[name] = (torch.arange(n, dtype=torch.int64, device=dev) % 256).to(torch.uint8).reshape(shapes[name])
    layer = M.Layer.from_checkpoint_ep(*[src[n] for n in names], ep_rank=0, ep_size=8)
    assert not layer.all_scales_normal()
    for which, g, u in (("w13", "gate_w", "up_w"), ("s13", "gate_s", "up_s"), ("w2", "down_w", None), ("s2", "down_s", None)):
        want_src, up = exp[which]
        want = src[g].reshape(-1)[want_src]
        if u is not None:
            want = torch.where(up.bool(), src[u].reshape(-1)[want_src], want)
        if which.startswith("s"):
            want = torch.where(want == 255, torch.full_like(want, 254), want)
        assert torch.equal(_image(layer, which, dev), want), which
    layer.close()


def test_repack_of_a_tensor_parallel_rank_from_the_canonical_image():
    """The same placement for a rank of eight built from the canonical rank image (256 experts, local width 256):
    position codes over the image, decoded from the prepared operand image and compared with the layout."""
    import torch

    import mimo26f_afd_b200 as M

    dev = torch.device("cuda:0")
    g, il = 8, I // 8
    gp, gs = il * (H // 2), il * (H // 32)
    dp, ds = H * (il // 2), H * (il // 32)
    image = 2 * (gp + gs) + dp + ds
    n = image * 256
    ar = lambda m: torch.arange(m, dtype=torch.int64, device=dev)
    got = {w: None for w in ("w13", "s13", "w2", "s2", "s13h")}
    for k in range(5):                                      # 7-bit codes: 35 bits cover the image, byte 255 never occurs
        src = _coded(n, k, 7, dev)
        layer = M.Layer.new_tp(src, n, 5, g)
        for which in got:
            v = _image(layer, which, dev).to(torch.int64) << (7 * k)
            got[which] = v if got[which] is None else got[which] | v
        layer.close()
        del src
    e, j, r, b = torch.meshgrid(ar(256), ar(il // 128), ar(256), ar(H // 2), indexing="ij")
    want = e * image + torch.where(r < 128, 0, gp + gs) + (j * 128 + r % 128) * (H // 2) + b
    assert torch.equal(got["w13"], want.reshape(-1))
    e, j, c, blk, o = torch.meshgrid(ar(256), ar(il // 128), ar(H // 128), ar(2), ar(512), indexing="ij")
    rr, kb = (o >> 4) + 32 * ((o >> 2) & 3), o & 3
    want = e * image + gp + blk * (gp + gs) + (j * 128 + rr) * (H // 32) + c * 4 + kb
    assert torch.equal(got["s13"], want.reshape(-1))
    # the regrouped scale image of half items: block (tile j, half h, chunk c) = 64 gate rows, then the 64 up rows of the
    # same features; a permutation of s13
    e, j, h, c, o = torch.meshgrid(ar(256), ar(il // 128), ar(2), ar(H // 128), ar(512), indexing="ij")
    grp, kb = (o >> 2) & 3, o & 3
    rr = 64 * h + 32 * (grp & 1) + (o >> 4)
    want = e * image + gp + (grp >> 1) * (gp + gs) + (j * 128 + rr) * (H // 32) + c * 4 + kb
    assert torch.equal(got["s13h"], want.reshape(-1))
    assert torch.equal(torch.sort(got["s13h"]).values, torch.sort(got["s13"]).values)
    e, h, b = torch.meshgrid(ar(256), ar(H), ar(il // 2), indexing="ij")
    assert torch.equal(got["w2"], (e * image + 2 * (gp + gs) + h * (il // 2) + b).reshape(-1))
    e, t, c, blk, o = torch.meshgrid(ar(256), ar(H // 256), ar(il // 128), ar(2), ar(512), indexing="ij")
    rr, kb = (o >> 4) + 32 * ((o >> 2) & 3), o & 3
    want = e * image + 2 * (gp + gs) + dp + (t * 256 + blk * 128 + rr) * (il // 32) + c * 4 + kb
    assert torch.equal(got["s2"], want.reshape(-1))


# ------------------------------------------------------------------------------------------ staged slices -> layer -> FFN
STAGED_EXPERTS = 16


def _write_checkpoint(path, layers):
    import json
    import struct

    from mimo26f_afd_b200 import staging, synth

    names = {"gate_w": ("gate_proj", False), "gate_s": ("gate_proj", True), "up_w": ("up_proj", False), "up_s": ("up_proj", True),
             "down_w": ("down_proj", False), "down_s": ("down_proj", True)}
    header, blobs, off = {"__metadata__": {"format": "pt"}}, [], 0
    for layer in layers:
        for e in range(STAGED_EXPERTS):
            for key, (proj, scale) in names.items():
                arr = synth.expert_tensor_np(SEED + layer, key, e)
                b = arr.tobytes()
                header[staging.tensor_name(layer, e, proj, scale)] = dict(dtype="U8", shape=list(arr.shape), data_offsets=[off, off + len(b)])
                blobs.append(b)
                off += len(b)
    text = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text)
        for b in blobs:
            f.write(b)


def _routes_among(tokens, n_experts, seed):
    """Top-8 routes over experts 0..n_experts-1 only (distinct per token), weights positive and summing to one."""
    rng = np.random.default_rng(seed)
    ids = np.stack([rng.permutation(n_experts)[:TOPK] for _ in range(tokens)]).astype(np.int32)
    w = rng.uniform(0.05, 1.0, (tokens, TOPK)).astype(np.float32)
    return ids, (w / w.sum(axis=1, keepdims=True, dtype=np.float32)).astype(np.float32)


def _layer_tensors(layer_id):
    from mimo26f_afd_b200 import synth

    return synth.layer_np(SEED + layer_id, range(STAGED_EXPERTS))


def test_staged_slices_to_layer_to_ffn(tmp_path, oracle_mod):
    """The reference's boot path (crates/mimo26-spark/src/boot.rs:34-46): repack a checkpoint into slice files and a
    manifest, verify them, build the rank's image from the files, prepare the layer from it, and serve. Ranks of four,
    sixteen experts staged (the others are zero slices no route points at); every rank's partial is compared with the
    oracle's slice of the same rank, and the rank-ordered sum of the four with the oracle's wire result."""
    import torch

    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import expert, staging, synth

    dev = torch.device("cuda:0")
    ckpt = tmp_path / "ckpt"
    ckpt.mkdir()
    _write_checkpoint(ckpt / "model_pp0_ep0_shard0.safetensors", [1])
    out = str(tmp_path / "slices")
    man = staging.repack(str(ckpt), out, ranks=4, layers=[1], experts=range(STAGED_EXPERTS))
    assert len(man["slices"]) == STAGED_EXPERTS * 4
    assert len(staging.readback(out)) == STAGED_EXPERTS * 4
    tokens = 24
    x_bits = synth.activations_bf16(SEED + 21, tokens)
    xq, xs = oracle_mod.quant_wire(synth.bf16_to_f32_np(x_bits))
    ids, w = _routes_among(tokens, STAGED_EXPERTS, 5)
    tensors = _layer_tensors(1)
    planes, ref_planes = [], []
    s = M.Scratch()
    for r in range(4):
        res = staging.readback(out, r)
        assert all(st == "match" for st, _, _ in res)
        image = np.zeros((256, staging.slice_bytes(4)), np.uint8)
        for e in range(STAGED_EXPERTS):
            with open(os.path.join(out, staging.slice_file_name(1, e, r)), "rb") as f:
                image[e] = np.frombuffer(f.read(), np.uint8)
        assert np.array_equal(image[:STAGED_EXPERTS], synth.canonical_rank_image_np(tensors, range(STAGED_EXPERTS), r, 4)[:STAGED_EXPERTS])
        img_d = torch.from_numpy(image.reshape(-1)).to(dev)
        L = M.Layer.new_tp(img_d, image.size, r, 4)
        del img_d
        bf = torch.empty((tokens, H), dtype=torch.int16, device=dev)
        part = torch.empty((tokens, H), dtype=torch.float32, device=dev)
        expert.ffn_dev(L, s, torch.from_numpy(xq).to(dev), torch.from_numpy(ids).to(dev), torch.from_numpy(w).to(dev), tokens, bf,
                       partial_out=part, x_dtype=expert.X_E4M3, x_scales=torch.from_numpy(xs).to(dev))
        s.status()
        ref = oracle_mod.ffn_layer(tensors, xq, xs, ids, w, tp_rank=r, tp_size=4)
        assert ref["rc"] == 0
        got = part.cpu().numpy()
        assert np.linalg.norm(got - ref["partial"]) / np.linalg.norm(ref["partial"]) <= 1e-3
        planes.append(bf.cpu().numpy().view(np.uint16))
        ref_planes.append(ref["bf16"])
        L.close()
    total = torch.empty((tokens, H), dtype=torch.float32, device=dev)
    expert.rank_sum_dev([torch.from_numpy(p.view(np.int16)).to(dev) for p in planes], tokens * H, total)
    torch.cuda.synchronize()
    want = oracle_mod.rank_sum(np.stack(ref_planes))
    assert np.linalg.norm(total.cpu().numpy() - want) / np.linalg.norm(want) <= 1e-3
    # a flipped byte in one slice file: the readback names the file and nothing is served from the directory
    victim = os.path.join(out, staging.slice_file_name(1, 3, 2))
    raw = bytearray(open(victim, "rb").read())
    raw[1000] ^= 0x40
    open(victim, "wb").write(bytes(raw))
    with pytest.raises(staging.StagingError) as e:
        staging.readback(out, 2)
    assert "sha_mismatch" in str(e.value) and "L01_E003_R2.slice" in str(e.value)


def test_rank_state_serves_two_layers_through_frames(tmp_path, oracle_mod):
    """The expert daemon's per-request work on a device (crates/mimo26-spark/src/main.rs:126-146, 348-460): slice files of
    two layers staged and verified, layers prepared on first touch and kept, request frames in, sealed return frames
    out; requests for both layers alternate, nothing is prepared twice, and each reply equals the oracle's rank partial
    to one BF16 ulp. A rejected plan comes back as an error-status frame and the rank keeps serving."""
    import torch

    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import frames, resident, staging, synth

    ckpt = tmp_path / "ckpt"
    ckpt.mkdir()
    _write_checkpoint(ckpt / "model_pp0_ep0_shard0.safetensors", [1, 2])
    out = str(tmp_path / "slices")
    staging.repack(str(ckpt), out, ranks=8, layers=[1, 2], experts=range(STAGED_EXPERTS))

    class SparseResident(resident.Resident):
        """Only sixteen experts per layer are staged here; the others are zero slices that no route points at."""

        def slice(self, layer, expert):
            if (layer, expert) in self.files:
                return super().slice(layer, expert)
            return bytes(staging.slice_bytes(self.ranks))

    rank = 6
    res = SparseResident(out, rank, verify=True)
    assert res.ranks == 8 and res.slices == 2 * STAGED_EXPERTS
    er = resident.ExpertRank(res, scratch=M.Scratch(), log=None)
    tokens = 12
    dec = lambda b: (b.astype(np.uint32) << 16).view(np.float32)
    served = []
    for i, layer_id in enumerate((1, 2, 1, 2, 2, 1)):
        x_bits = synth.activations_bf16(SEED + 30 + i, tokens)
        xq, xs = oracle_mod.quant_wire(synth.bf16_to_f32_np(x_bits))
        ids, w = _routes_among(tokens, STAGED_EXPERTS, 40 + i)
        req = frames.encode_request(xq, xs, ids, w, request_id=100 + i, layer_id=layer_id)
        reply = er.handle(req)
        meta, got = frames.parse_return(reply)
        assert (meta["request_id"], meta["layer_id"], meta["rows"], meta["status"], meta["seq"]) == (100 + i, layer_id, tokens, 0, i + 1)
        ref = oracle_mod.ffn_layer(_layer_tensors(layer_id), xq, xs, ids, w, tp_rank=rank, tp_size=8)
        assert ref["rc"] == 0
        # BF16 rows against the oracle's FP32 plane: half a BF16 ulp on top of the end-to-end bar; element-wise one BF16
        # ulp, except on the tokens where an intermediate crossed an E4M3 bin (counted in the single-rank tests)
        assert np.linalg.norm(dec(got) - ref["partial"]) / np.linalg.norm(ref["partial"]) <= 1e-3 + 2.0 ** -8
        close = np.abs(dec(got) - dec(ref["bf16"])) <= 2.0 ** -7 * np.abs(ref["partial"]) + 1e-4
        assert close.mean() >= 0.99, (i, close.mean())
        served.append(layer_id)
    assert sorted(er.layers) == [1, 2] and set(er.load_ms) == {1, 2}          # two layers resident, each prepared once
    assert er.ensure_layer(1) == 0.0 and er.ensure_layer(2) == 0.0
    # a request whose plan is rejected (an expert twice in a row): error-status return with the request's ids
    ids_bad = ids.copy()
    ids_bad[0, 1] = ids_bad[0, 0]
    reply = er.handle(frames.encode_request(xq, xs, ids_bad, w, request_id=900, layer_id=1))
    meta, body = frames.parse_return(reply)
    assert meta["request_id"] == 900 and meta["status"] == 1 and meta["rows"] == tokens and not body.any()
    reply = er.handle(frames.encode_request(xq, xs, ids, w, request_id=901, layer_id=2))
    assert frames.parse_return(reply)[0]["status"] == 0
    for layer in er.layers.values():
        layer.close()
