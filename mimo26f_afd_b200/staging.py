"""Offline staging with identity: checkpoint shards -> per-(layer, expert, rank) slice files + a sha256 manifest, and
the boot-time readback that refuses anything that does not match.

The step before the hot path: it makes the bytes a rank serves reproducible and auditable. Mirrors the reference's
repack tool (``crates/mimo26-repack``): the safetensors header reader (``src/safetensors.rs``), the pinned slice layout
v2 (``src/geom.rs:22-50``: gate payload, gate scales, up payload, up scales, down payload, down scales; gate/up rows
``[r I/G, (r+1) I/G)``, down K columns of the same range), the manifest v2 (``src/manifest.rs``) and the identity readback
(``src/identity.rs``: every file is checked and reported, any mismatch refuses to serve; a version-1 manifest is refused
because v1 slices were strided and byte lengths alone cannot tell them apart). The rank count is the reference's 4 by
default and may be 1, 2, 4 or 8 here (the library's ``m26b_layer_new_tp`` consumes such images).

    python -m mimo26f_afd_b200.staging repack CHECKPOINT_DIR OUT_DIR [--ranks 4] [--layers 1,2]
    python -m mimo26f_afd_b200.staging verify OUT_DIR

Host-side file work only: nothing here touches the GPU or the CUDA library.
"""
from __future__ import annotations

import hashlib
import json
import os
import re
import struct
import sys

import numpy as np

HIDDEN, INTERMEDIATE, EXPERTS_PER_LAYER, MOE_LAYERS, FIRST_MOE_LAYER = 4096, 2048, 256, 47, 1
EXPERT_BYTES = 13_369_344
FORMAT, VERSION = "mimo26-repack-manifest", 2
PROJS = ("gate_proj", "up_proj", "down_proj")
MANIFEST_NAME = "manifest.json"


class StagingError(RuntimeError):
    pass


# ------------------------------------------------------------------------------------------ geometry
def slice_bytes(ranks: int = 4) -> int:
    return EXPERT_BYTES // ranks


def layout_table(ranks: int = 4):
    """The pinned layout of one slice: (proj, region, offset, length) in file order (geom.rs:36-50 for 4 ranks)."""
    il = INTERMEDIATE // ranks
    rows = {"gate_proj": (il, HIDDEN), "up_proj": (il, HIDDEN), "down_proj": (HIDDEN, il)}
    out, off = [], 0
    for proj in PROJS:
        r, k = rows[proj]
        for region, n in (("payload", r * k // 2), ("scales", r * k // 32)):
            out.append(dict(proj=proj, region=region, off=off, len=n))
            off += n
    assert off == slice_bytes(ranks)
    return out


def tensor_name(layer: int, expert: int, proj: str, scale: bool) -> str:
    return f"model.layers.{layer}.mlp.experts.{expert}.{proj}.weight" + ("_scale" if scale else "")


def slice_file_name(layer: int, expert: int, rank: int) -> str:
    return f"L{layer:02d}_E{expert:03d}_R{rank}.slice"


def checkpoint_shapes():
    return {"gate_proj": ((INTERMEDIATE, HIDDEN // 2), (INTERMEDIATE, HIDDEN // 32)),
            "up_proj": ((INTERMEDIATE, HIDDEN // 2), (INTERMEDIATE, HIDDEN // 32)),
            "down_proj": ((HIDDEN, INTERMEDIATE // 2), (HIDDEN, INTERMEDIATE // 32))}


def build_slice(tensors: dict, rank: int, ranks: int = 4) -> bytes:
    """One expert's slice for ``rank``: ``tensors[proj] = (weight u8 [out, in/2], weight_scale u8 [out, in/32])``
    (repack.rs:135-163). Rows / K columns of a rank are contiguous, so K32 scale blocks never straddle ranks."""
    if ranks not in (1, 2, 4, 8) or not 0 <= rank < ranks:
        raise StagingError(f"rank {rank} / ranks {ranks}: ranks must be 1, 2, 4 or 8")
    il = INTERMEDIATE // ranks
    shapes = checkpoint_shapes()
    parts = []
    for proj in PROJS:
        w, s = (np.ascontiguousarray(a, dtype=np.uint8) for a in tensors[proj])
        if w.shape != shapes[proj][0] or s.shape != shapes[proj][1]:
            raise StagingError(f"{proj}: shapes {w.shape} / {s.shape}, want {shapes[proj][0]} / {shapes[proj][1]}")
        if proj == "down_proj":
            parts += [w[:, rank * il // 2:(rank + 1) * il // 2], s[:, rank * il // 32:(rank + 1) * il // 32]]
        else:
            parts += [w[rank * il:(rank + 1) * il], s[rank * il:(rank + 1) * il]]
    image = b"".join(np.ascontiguousarray(p).tobytes() for p in parts)
    assert len(image) == slice_bytes(ranks)
    return image


# ------------------------------------------------------------------------------------------ safetensors header
class SafetensorsHeader:
    """``<u64 LE header_len><JSON header><data>``; entries ``{"dtype", "shape", "data_offsets": [a, b]}`` relative to the
    data region (safetensors.rs:46-90). Read-only; every declared range must lie inside the file."""

    def __init__(self, path: str):
        self.path = path
        file_len = os.path.getsize(path)
        if file_len < 8:
            raise StagingError(f"{path}: file is {file_len} B, shorter than the 8-byte header length")
        with open(path, "rb") as f:
            (header_len,) = struct.unpack("<Q", f.read(8))
            if header_len == 0 or header_len > file_len - 8:
                raise StagingError(f"{path}: header length {header_len} does not fit in {file_len} B")
            raw = f.read(header_len)
        try:
            text = raw.decode("utf-8")
        except UnicodeDecodeError as e:
            raise StagingError(f"{path}: header is not UTF-8: {e}") from None
        try:
            doc = json.loads(text, object_pairs_hook=_no_duplicate_keys)
        except (ValueError, StagingError) as e:
            raise StagingError(f"{path}: {e}") from None
        if not isinstance(doc, dict):
            raise StagingError(f"{path}: header is not a JSON object")
        self.data_start, self.file_len, self.tensors = 8 + header_len, file_len, {}
        for name, ent in doc.items():
            if name == "__metadata__":
                continue
            if not isinstance(ent, dict) or set(ent) != {"dtype", "shape", "data_offsets"}:
                raise StagingError(f"{path}: tensor {name!r}: entry must have exactly dtype, shape, data_offsets")
            a, b = ent["data_offsets"]
            if not (isinstance(a, int) and isinstance(b, int) and 0 <= a <= b):
                raise StagingError(f"{path}: tensor {name!r}: bad data_offsets {ent['data_offsets']}")
            if self.data_start + b > file_len:
                raise StagingError(f"{path}:{name}: truncated: declared end {self.data_start + b}, file has {file_len} B")
            self.tensors[name] = dict(dtype=ent["dtype"], shape=[int(d) for d in ent["shape"]], data_offsets=(a, b))

    def read_tensor(self, name: str) -> np.ndarray:
        if name not in self.tensors:
            raise StagingError(f"missing tensor {name}")
        t = self.tensors[name]
        if t["dtype"] != "U8":
            raise StagingError(f"{name}: dtype {t['dtype']}, expert weights are U8")
        a, b = t["data_offsets"]
        if b - a != int(np.prod(t["shape"])):
            raise StagingError(f"{name}: {b - a} bytes for shape {t['shape']}")
        with open(self.path, "rb") as f:
            f.seek(self.data_start + a)
            return np.frombuffer(f.read(b - a), np.uint8).reshape(t["shape"])


def _no_duplicate_keys(pairs):
    out = {}
    for k, v in pairs:
        if k in out:
            raise StagingError(f"duplicate key {k!r}")
        out[k] = v
    return out


def index_checkpoint(checkpoint_dir: str):
    """tensor name -> (shard file, header) over every ``*.safetensors`` of a directory; a name in two shards is an error."""
    index = {}
    for fn in sorted(os.listdir(checkpoint_dir)):
        if not fn.endswith(".safetensors"):
            continue
        hdr = SafetensorsHeader(os.path.join(checkpoint_dir, fn))
        for name in hdr.tensors:
            if name in index:
                raise StagingError(f"tensor {name} appears in {index[name][0]} and {fn}")
            index[name] = (fn, hdr)
    return index


# ------------------------------------------------------------------------------------------ manifest
def sha256_hex(data: bytes) -> str:
    return hashlib.sha256(data).hexdigest()


def new_manifest(ranks: int = 4) -> dict:
    return dict(format=FORMAT, version=VERSION, generated_by="mimo26f-afd-b200 staging 1",
                geometry=dict(hidden=HIDDEN, intermediate=INTERMEDIATE, experts_per_layer=EXPERTS_PER_LAYER, moe_layers=MOE_LAYERS,
                              ep_ranks=ranks, expert_bytes=EXPERT_BYTES, quarter_slice_bytes=slice_bytes(ranks)),
                layout=layout_table(ranks), slices=[])


def manifest_text(m: dict) -> str:
    """Deterministic bytes: fixed key order, slices in file-name order, two-space indent, trailing newline."""
    m = dict(m, slices=sorted(m["slices"], key=lambda s: s["file"]))
    return json.dumps(m, indent=2) + "\n"


_SLICE_KEYS = ("file", "sha256", "bytes", "layer", "expert", "rank", "source")
_GEOMETRY_KEYS = ("hidden", "intermediate", "experts_per_layer", "moe_layers", "ep_ranks", "expert_bytes", "quarter_slice_bytes")


def parse_manifest(text: str) -> dict:
    """Strict: an unknown or missing field, a malformed sha, or a geometry / layout that disagrees with the compiled-in
    constants is an error, never a default (manifest.rs:1-8); version 1 is refused by name."""
    try:
        m = json.loads(text, object_pairs_hook=_no_duplicate_keys)
    except ValueError as e:
        raise StagingError(f"manifest: {e}") from None
    if not isinstance(m, dict) or tuple(m) != ("format", "version", "generated_by", "geometry", "layout", "slices"):
        raise StagingError("manifest: top-level fields must be format, version, generated_by, geometry, layout, slices")
    if m["format"] != FORMAT:
        raise StagingError(f"manifest: format {m['format']!r}, want {FORMAT!r}")
    if m["version"] == 1:
        raise StagingError("manifest: version 1 slices are strided-output artifacts; regenerate them, they cannot be relabelled")
    if m["version"] != VERSION:
        raise StagingError(f"manifest: version {m['version']}, want {VERSION}")
    g = m["geometry"]
    if not isinstance(g, dict) or tuple(g) != _GEOMETRY_KEYS:
        raise StagingError("manifest: geometry fields")
    ranks = g["ep_ranks"]
    if ranks not in (1, 2, 4, 8) or g != new_manifest(ranks)["geometry"]:
        raise StagingError("manifest: geometry disagrees with the compiled-in constants")
    if m["layout"] != layout_table(ranks):
        raise StagingError("manifest: layout table disagrees with the pinned slice layout")
    seen = set()
    for s in m["slices"]:
        if not isinstance(s, dict) or tuple(s) != _SLICE_KEYS:
            raise StagingError("manifest: slice entry fields")
        if not re.fullmatch(r"[0-9a-f]{64}", s["sha256"]):
            raise StagingError(f"manifest: {s['file']}: malformed sha256")
        if s["bytes"] != slice_bytes(ranks):
            raise StagingError(f"manifest: {s['file']}: {s['bytes']} bytes, want {slice_bytes(ranks)}")
        if s["file"] != slice_file_name(s["layer"], s["expert"], s["rank"]) or not 0 <= s["rank"] < ranks:
            raise StagingError(f"manifest: {s['file']}: name does not match layer / expert / rank")
        if s["file"] in seen:
            raise StagingError(f"manifest: {s['file']} listed twice")
        seen.add(s["file"])
        src = s["source"]
        if not isinstance(src, dict) or tuple(src) != ("shard", "tensors") or len(src["tensors"]) != 6:
            raise StagingError(f"manifest: {s['file']}: source must name a shard and six tensors")
        for t in src["tensors"]:
            if tuple(t) != ("name", "shape", "dtype") or t["dtype"] != "U8":
                raise StagingError(f"manifest: {s['file']}: source tensor fields")
    return m


# ------------------------------------------------------------------------------------------ repack and readback
def repack(checkpoint_dir: str, out_dir: str, ranks: int = 4, layers=None, experts=None) -> dict:
    """Write the slice files of the given layers (default: every MoE layer the checkpoint holds) and the manifest.
    Deterministic: the same checkpoint gives the same bytes, manifest included."""
    index = index_checkpoint(checkpoint_dir)
    if layers is None:
        layers = sorted({int(m.group(1)) for n in index if (m := re.match(r"model\.layers\.(\d+)\.mlp\.experts\.", n))})
    experts = range(EXPERTS_PER_LAYER) if experts is None else experts
    os.makedirs(out_dir, exist_ok=True)
    man = new_manifest(ranks)
    shapes = checkpoint_shapes()
    for layer in layers:
        for e in experts:
            tensors, src, shards = {}, [], set()
            for proj in PROJS:
                pair = []
                for scale in (False, True):
                    name = tensor_name(layer, e, proj, scale)
                    if name not in index:
                        raise StagingError(f"missing tensor {name}")
                    shard, hdr = index[name]
                    shards.add(shard)
                    arr = hdr.read_tensor(name)
                    if arr.shape != shapes[proj][1 if scale else 0]:
                        raise StagingError(f"{name}: shape {arr.shape}, want {shapes[proj][1 if scale else 0]}")
                    pair.append(arr)
                    src.append(dict(name=name, shape=list(arr.shape), dtype="U8"))
                tensors[proj] = tuple(pair)
            if len(shards) != 1:
                raise StagingError(f"layer {layer} expert {e}: tensors spread over shards {sorted(shards)}")
            for r in range(ranks):
                image = build_slice(tensors, r, ranks)
                fn = slice_file_name(layer, e, r)
                with open(os.path.join(out_dir, fn), "wb") as f:
                    f.write(image)
                man["slices"].append(dict(file=fn, sha256=sha256_hex(image), bytes=len(image), layer=layer, expert=e, rank=r,
                                          source=dict(shard=shards.copy().pop(), tensors=src)))
    with open(os.path.join(out_dir, MANIFEST_NAME), "w") as f:
        f.write(manifest_text(man))
    return man


def readback(out_dir: str, rank=None):
    """The boot check (identity.rs): every listed file (of ``rank``, or of all ranks) is read and compared; files in the
    directory that the manifest does not list are reported too. Returns the list of (status, file, detail); raises
    ``StagingError`` naming every bad file if any is not a match."""
    with open(os.path.join(out_dir, MANIFEST_NAME)) as f:
        man = parse_manifest(f.read())
    report, listed = [], set()
    for s in man["slices"]:
        if rank is not None and s["rank"] != rank:
            continue
        listed.add(s["file"])
        path = os.path.join(out_dir, s["file"])
        if not os.path.exists(path):
            report.append(("missing", s["file"], ""))
            continue
        size = os.path.getsize(path)
        if size != s["bytes"]:
            report.append(("size_mismatch", s["file"], f"want {s['bytes']}, got {size}"))
            continue
        with open(path, "rb") as f:
            got = sha256_hex(f.read())
        report.append(("match", s["file"], got) if got == s["sha256"] else ("sha_mismatch", s["file"], f"want {s['sha256']}, got {got}"))
    for fn in sorted(os.listdir(out_dir)):
        if fn.endswith(".slice") and fn not in listed and (rank is None or fn.endswith(f"_R{rank}.slice")):
            report.append(("unlisted", fn, ""))
    bad = [r for r in report if r[0] != "match"]
    if bad:
        raise StagingError("identity readback refuses to serve: " + "; ".join(f"{s} {f} {d}".strip() for s, f, d in bad))
    return report


def load_rank_image(out_dir: str, layer: int, rank: int) -> np.ndarray:
    """The 256 verified slices of (layer, rank) back to back: the canonical image ``Layer.new_tp`` takes (after a copy to
    the device). Refuses to return anything if the readback of that rank fails."""
    readback(out_dir, rank)
    parts = []
    for e in range(EXPERTS_PER_LAYER):
        with open(os.path.join(out_dir, slice_file_name(layer, e, rank)), "rb") as f:
            parts.append(f.read())
    return np.frombuffer(b"".join(parts), np.uint8)


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) >= 3 and argv[0] == "repack":
        ranks, layers = 4, None
        for i, a in enumerate(argv):
            if a == "--ranks":
                ranks = int(argv[i + 1])
            if a == "--layers":
                layers = [int(v) for v in argv[i + 1].split(",")]
        man = repack(argv[1], argv[2], ranks, layers)
        print(f"wrote {len(man['slices'])} slices of {slice_bytes(ranks)} B and {MANIFEST_NAME} to {argv[2]}")
        return 0
    if len(argv) == 2 and argv[0] == "verify":
        rep = readback(argv[1])
        print(f"{len(rep)} slices match their manifest")
        return 0
    print(__doc__)
    return 2


if __name__ == "__main__":
    sys.exit(main())
