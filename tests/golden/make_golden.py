"""Generate tests/golden/*.npz by RUNNING THE REFERENCE's own Python code.

Run in the development container, where the reference tree is mounted:

    python tests/golden/make_golden.py [REFERENCE_TREE]

Imports (never copies) from the reference tree:
  oracle/lattice/quant_v1.py                     codec of record e4m3fn-k32-v1
  crates/mimo26-repack/tests/lattice_oracle.py   E-W4A8-v1 FFN reference (expert, reduce_routes, activation)
  spike/mxfp4.py                                 MXFP4 decode reference
  spike/quant.py                                 E4M3 nearest encoder (ties to the larger magnitude), the
                                                 Python twin of crates/mimo26-load/src/e4m3.rs:50-81
and reads the reference's golden data files oracle/goldens/{e4m3_decode_table,mxfp4_golden}.json (values only).
(bench/fixtures/expert_nibble_fixture.json holds sampled outputs of real checkpoint blocks whose weight bytes
are not in the reference tree, so it cannot pin a decoder here and is not imported.)

The wire quantiser's scale rule exists only in Rust (crates/mimo26-coordinator/src/wire.rs:62-70); this script
evaluates that formula literally in float64 (ceil(log2(amax/448)) + 127, clamped to 0..254, 0 for a zero
block) and encodes payloads with the reference's spike/quant.py::encode_e4m3.

Seeded inputs come from mimo26f_afd_b200/synth.py (loaded by path; numpy only).
"""
import importlib.util
import json
import os
import sys

import numpy as np

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("M26B_REFERENCE_TREE", "")
if not REF:
    raise SystemExit("usage: make_golden.py REFERENCE_TREE   (or set M26B_REFERENCE_TREE)")
HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
# the reference's packages must win: keep this repository's root (which has its own `oracle/`) off sys.path
sys.path = [p for p in sys.path if os.path.abspath(p or ".") != REPO]
sys.path.insert(0, os.path.join(REF, "crates/mimo26-repack/tests"))
sys.path.insert(0, REF)


def load(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


synth = load("synth", os.path.join(REPO, "mimo26f_afd_b200/synth.py"))
import lattice_oracle as LO  # noqa: E402  (reference)
from oracle.lattice import quant_v1 as Q  # noqa: E402  (reference)
from spike import mxfp4 as MX  # noqa: E402  (reference)
from spike import quant as SQ  # noqa: E402  (reference)

rng = np.random.default_rng(0x26B1)


def quant_corpus():
    """FP32 inputs that stress the codec: code centres, tie neighbours, amax transitions, the 1e-4 floor,
    subnormals, signed zeros, wide magnitudes (after crates/mimo26-expert/tests/b1/quant_compare.py:23-60)."""
    blocks = []
    grid = Q.e4m3fn_decode(np.array([c for c in range(128) if c != 0x7F], np.uint8))
    for k in (-20, -13, -9, -1, 0, 3, 30):
        vals = np.ldexp(grid, k)
        mids = np.ldexp((grid[:-1] + grid[1:]) / 2, k)
        for arr in (vals, mids, np.nextafter(mids.astype(np.float32), np.float32(0)), np.nextafter(mids.astype(np.float32), np.float32(np.inf))):
            a = np.asarray(arr, np.float32)
            a = np.concatenate([a, np.zeros((-a.size) % 32, np.float32)])
            blk = a.reshape(-1, 32).copy()
            blk[:, 0] = np.float32(np.ldexp(448.0, k))  # pin the block maximum so the scale is k
            blocks.append(blk)
            blocks.append(-blk)
    for amax in (448.0, np.nextafter(np.float32(448.0), np.float32(1e9)), 447.99, 1e-4, np.nextafter(np.float32(1e-4), np.float32(0)),
                 np.nextafter(np.float32(1e-4), np.float32(1)), 1e-30, 1e-45, 3e38, 0.0, 1.75, 1.7500001, 3.5, 7.0):
        blk = (rng.uniform(-1, 1, (4, 32)) * float(amax)).astype(np.float32)
        blk[:, 5] = np.float32(amax)
        blocks.append(blk)
    z = np.zeros((2, 32), np.float32); z[1, ::2] = -0.0
    blocks.append(z)
    wide = (rng.normal(size=(1500, 32)) * np.exp(rng.uniform(-40, 40, (1500, 1)))).astype(np.float32)
    blocks.append(wide)
    bf = rng.normal(size=(1500, 32)).astype(np.float32)
    blocks.append(synth.bf16_to_f32_np(synth.bf16_rne_np(bf)))  # BF16-exact values: E4M3 ties are common
    return np.concatenate(blocks).astype(np.float32)


def wire_reference(x):
    """wire.rs:53-78 evaluated literally in float64 + the reference's Python encoder."""
    xb = x.reshape(-1, 32).astype(np.float64)
    amax = np.max(np.abs(np.nan_to_num(xb, nan=0.0)), axis=1)
    with np.errstate(divide="ignore"):
        e = np.ceil(np.log2(amax / 448.0)) + 127.0
    s = np.where(amax == 0.0, 0.0, np.clip(e, 0.0, 254.0)).astype(np.uint8)
    scaled = xb * np.ldexp(1.0, 127 - s.astype(np.int64))[:, None]
    return SQ.encode_e4m3(scaled).reshape(x.shape), s


def main():
    out = {}
    # --- reference golden data files (values only)
    e4 = json.load(open(os.path.join(REF, "oracle/goldens/e4m3_decode_table.json")))
    mxg = json.load(open(os.path.join(REF, "oracle/goldens/mxfp4_golden.json")))
    out["e4m3_table_keys"] = np.array(sorted(e4.keys()))
    json.dump({"e4m3_decode_table": e4, "mxfp4_golden": mxg}, open(os.path.join(HERE, "reference_goldens.json"), "w"))

    # --- quantiser v1 (codec of record)
    x = quant_corpus()
    p, s = Q.encode_blocks(x.reshape(-1, 32))
    out["qv1_x_bits"] = x.view(np.uint32)
    out["qv1_payload"] = p.reshape(-1)
    out["qv1_scales"] = s.reshape(-1)
    out["qv1_decoded_bits"] = Q.decode_blocks(p, s).reshape(-1).view(np.uint32)
    # --- wire quantiser on the finite part of the same corpus + BF16 N(0,1) rows
    wp, ws = wire_reference(x)
    out["wire_payload"] = wp.reshape(-1)
    out["wire_scales"] = ws
    # --- MXFP4 decode
    pk = rng.integers(0, 256, size=(64, 512), dtype=np.uint8)
    sc = np.resize(np.arange(256, dtype=np.uint8), (64, 32))
    out["mx_packed"], out["mx_scales"] = pk, sc
    out["mx_unpacked_bits"] = MX.unpack(pk, sc, naive=False).view(np.uint32)
    # --- activation
    g = np.concatenate([rng.normal(size=2000) * 4, [-100.0, -0.0, 0.0, 100.0, 88.0, -88.0, 1e-30, -1e-30]]).astype(np.float32)
    u = np.concatenate([rng.normal(size=2000), np.ones(8)]).astype(np.float32)
    out["act_g_bits"], out["act_u_bits"] = g.view(np.uint32), u.view(np.uint32)
    out["act_h_bits"] = LO.activation(g, u).view(np.uint32)
    # --- one expert at the real shape on seeded MXFP4 weights, 4 tokens (lattice_oracle.expert)
    seed, e = synth.MASTER_SEED, 7
    T = {n: synth.expert_tensor_np(seed, n, e) for n in synth.TENSORS}
    xa = synth.bf16_to_f32_np(synth.activations_bf16(seed, 4))
    xp, xs = Q.encode_blocks(xa)
    mats = [MX.unpack(T[a], T[b], naive=False).astype(np.float64) for a, b in (("gate_w", "gate_s"), ("up_w", "up_s"), ("down_w", "down_s"))]
    r = LO.expert(xp, xs, *mats)
    out["exp_seed"], out["exp_expert"] = np.array([seed]), np.array([e])
    out["exp_xp"], out["exp_xs"] = xp, xs
    for k in ("gate", "up", "h"):
        out["exp_" + k + "_bits"] = r[k].view(np.uint32)
    out["exp_mid_payload"], out["exp_mid_scales"] = r["mid_payload"], r["mid_scales"]
    out["exp_full_bits"] = LO.f32(r["full"]).view(np.uint32)
    out["exp_partial_bits"] = LO.f32(r["partial"]).view(np.uint32)
    # --- weight-once ordered reduce, per-rank BF16, rank-ordered sum (lattice_oracle.reduce_routes)
    part = rng.normal(size=(4, 6, 8, 64)) * np.exp(rng.uniform(-3, 3, (4, 6, 8, 1)))
    part[0, 0, :4, 0] = [1e8, -1e8, 1.0, 1.0]
    part[:, 1, 0, 1] = [2.0 ** 24, 1.0, -(2.0 ** 24), 1.0]
    wts = rng.uniform(0, 1, (6, 8)).astype(np.float32)
    wts[1, 0] = 1.0; wts[1, 1:] = 0.0
    rank, decoded, final = LO.reduce_routes(part, wts)
    out["red_partial_bits"] = LO.f32(part).view(np.uint32)
    out["red_weights_bits"] = wts.view(np.uint32)
    out["red_rank_bits"], out["red_decoded_bits"], out["red_final_bits"] = rank.view(np.uint32), decoded.view(np.uint32), final.view(np.uint32)
    np.savez_compressed(os.path.join(HERE, "reference_vectors.npz"), **out)
    print("wrote", os.path.join(HERE, "reference_vectors.npz"), {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
