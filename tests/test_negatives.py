"""Negatives: every rule of the path that a plausible implementation gets wrong has a naive variant here, and the
naive variant must FAIL against the reference-generated golden vectors. A golden comparison that a wrong rule also
passes pins nothing; these tests show that the pins of test_oracle_pins.py discriminate. The rules and their naive
variants are the ones the reference's own suites name (nibble order and reserved scale byte:
crates/mimo26-expert/src/lib.rs:59-122; weight-once, no fused multiply-add, no reassociation, BF16 round before the rank
sum, rank order: crates/mimo26-repack/tests/lattice_oracle.py mutations; quantiser ties and floor:
oracle/tests/test_lattice_quant_v1.py)."""
import numpy as np


def f32(bits):
    return np.ascontiguousarray(bits, dtype=np.uint32).view(np.float32)


def bf16_rne(x):
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


# ------------------------------------------------------------------------------------------ MXFP4 decode
def test_high_nibble_first_decode_fails_the_golden(oracle_mod, golden):
    packed, scales = golden["mx_packed"], golden["mx_scales"]
    good = oracle_mod.mxfp4_unpack(packed, scales)
    assert np.array_equal(good.view(np.uint32), golden["mx_unpacked_bits"])
    swapped = ((packed >> 4) | (packed << 4)).astype(np.uint8)            # naive: high nibble = even k
    bad = oracle_mod.mxfp4_unpack(swapped, scales)
    assert (bad.view(np.uint32) != golden["mx_unpacked_bits"]).mean() > 0.3


def test_reserved_scale_byte_is_clamped_not_infinite(oracle_mod):
    packed = np.full((1, 16), 0x22, np.uint8)                               # code 2 = 1.0 in both nibbles
    top = oracle_mod.mxfp4_unpack(packed, np.array([[255]], np.uint8))
    assert np.isfinite(top).all() and np.array_equal(top, oracle_mod.mxfp4_unpack(packed, np.array([[254]], np.uint8)))
    with np.errstate(over="ignore"):
        naive = np.ldexp(np.float64(1.0), 255 - 127).astype(np.float32)     # 2^128 does not exist in FP32
    assert np.isinf(naive)


# ------------------------------------------------------------------------------------------ quantisers
def _encode_e4m3_rne(v):
    """E4M3 (finite, saturating at 448) of float64 values, ties to even: the wrong rule for the wire codec."""
    a = np.minimum(np.abs(v), 448.0)
    e = np.floor(np.log2(np.maximum(a, 2.0 ** -9)))
    e = np.maximum(e, -6.0)
    q = 2.0 ** (e - 3)
    m = np.rint(a / q)                                                      # numpy rounds half to even
    a2 = np.minimum(m * q, 448.0)
    e2 = np.maximum(np.floor(np.log2(np.maximum(a2, 2.0 ** -9))), -6.0)
    sub = a2 < 2.0 ** -6
    mant = np.where(sub, a2 / 2.0 ** -9, (a2 / 2.0 ** e2 - 1.0) * 8.0)
    code = np.where(sub, mant, (e2 + 7) * 8 + mant).astype(np.uint8)
    return (code | np.where(np.signbit(v), 0x80, 0)).astype(np.uint8)


def test_wire_quantiser_with_ties_to_even_fails_the_golden(oracle_mod, golden):
    x = f32(golden["qv1_x_bits"])
    finite = np.isfinite(x).all(axis=1)
    p, s = oracle_mod.quant_wire(x[finite])
    want = golden["wire_payload"].reshape(-1, 32)[finite]
    assert np.array_equal(p, want) and np.array_equal(s.reshape(-1), golden["wire_scales"][finite])
    scale_inv = np.ldexp(1.0, 127 - s.astype(np.int64)).reshape(-1, 1)
    naive = _encode_e4m3_rne(x[finite].astype(np.float64) * scale_inv)
    live = s.reshape(-1) != 0
    assert (naive[live] != want[live]).any(), "the corpus holds exact ties: ties-to-even must differ somewhere"
    assert (naive[live] != want[live]).mean() < 0.05                        # and only there


def test_quant_v1_without_the_floor_fails_the_golden(oracle_mod, golden):
    x = f32(golden["qv1_x_bits"])
    finite = np.isfinite(x).all(axis=1)
    amax = np.abs(x[finite]).max(axis=1)
    tiny = amax < 1e-4
    assert tiny.any()
    scales = golden["qv1_scales"][finite]
    assert (scales[tiny] == 105).all()                                      # floor 1e-4 -> exponent -22
    with np.errstate(divide="ignore"):
        naive = np.where(amax > 0, np.ceil(np.log2(np.maximum(amax, 1e-300) / 448.0)) + 127, 0)
    assert (naive[tiny] != 105).any()


def test_quant_v1_clipping_instead_of_fault_is_not_the_codec(oracle_mod):
    x = np.zeros((1, 32), np.float32)
    x[0, 3] = np.inf
    p, s, fault = oracle_mod.quant_v1(x)
    assert fault[0] == 1                                                    # reported, not clipped to 448


# ------------------------------------------------------------------------------------------ combine and rank sum
def _reduce_variants(part, w):
    """part [T,8,H] f32, w [T,8] f32 -> dict of FP32 planes under the right rule and four wrong ones."""
    t, k, h = part.shape
    out = {}
    v = np.zeros((t, h), np.float32)
    for j in range(k):
        v = (v + (w[:, j, None] * part[:, j, :]).astype(np.float32)).astype(np.float32)
    out["right"] = v
    v = np.zeros((t, h), np.float64)
    acc = np.zeros((t, h), np.float32)
    for j in range(k):                                                      # fused multiply-add: one rounding
        acc = (acc.astype(np.float64) + w[:, j, None].astype(np.float64) * part[:, j, :].astype(np.float64)).astype(np.float32)
    out["fma"] = acc
    prod = (w[:, :, None] * part).astype(np.float32)
    out["pairwise"] = ((prod[:, 0] + prod[:, 1]) + (prod[:, 2] + prod[:, 3]) + ((prod[:, 4] + prod[:, 5]) + (prod[:, 6] + prod[:, 7]))).astype(np.float32)
    v = np.zeros((t, h), np.float32)
    for j in range(k):                                                      # weight applied twice
        v = (v + (w[:, j, None] * (w[:, j, None] * part[:, j, :]).astype(np.float32)).astype(np.float32)).astype(np.float32)
    out["weight_twice"] = v
    v = np.zeros((t, h), np.float32)
    for j in reversed(range(k)):                                            # slots in the other order
        v = (v + (w[:, j, None] * part[:, j, :]).astype(np.float32)).astype(np.float32)
    out["reversed"] = v
    return out


def test_combine_variants_fail_the_golden(oracle_mod, golden):
    part, w = f32(golden["red_partial_bits"]), f32(golden["red_weights_bits"])
    wrong = {k: 0 for k in ("fma", "pairwise", "weight_twice", "reversed")}
    for r in range(4):
        variants = _reduce_variants(part[r], w)
        assert np.array_equal(variants["right"].view(np.uint32), golden["red_rank_bits"][r])
        rc, partial, _ = oracle_mod.route_reduce(part[r], w, hidden=part.shape[-1])
        assert rc == 0 and np.array_equal(partial.view(np.uint32), golden["red_rank_bits"][r])
        for k in wrong:
            wrong[k] += int((variants[k].view(np.uint32) != golden["red_rank_bits"][r]).sum())
    assert all(n > 0 for n in wrong.values()), wrong


def test_rank_sum_variants_fail_the_golden(oracle_mod, golden):
    ranks = f32(golden["red_rank_bits"])                                    # [4, T, H] FP32 per-rank partials
    planes = np.stack([bf16_rne(ranks[r]).reshape(ranks[r].shape) for r in range(4)])
    assert np.array_equal(oracle_mod.rank_sum(planes.reshape(4, -1)).view(np.uint32), golden["red_final_bits"].reshape(-1))
    no_round = np.zeros_like(ranks[0])
    for r in range(4):                                                      # summing the FP32 partials without the BF16 wire round
        no_round = (no_round + ranks[r]).astype(np.float32)
    assert (no_round.view(np.uint32) != golden["red_final_bits"]).any()
    rev = oracle_mod.rank_sum(planes[::-1].reshape(4, -1).copy())
    order = np.array([[2.0 ** 24], [1.0], [-(2.0 ** 24)], [1.0]], np.float32)
    bits = (order.view(np.uint32) >> 16).astype(np.uint16)
    assert oracle_mod.rank_sum(bits)[0] != oracle_mod.rank_sum(bits[[0, 2, 1, 3]])[0]
    assert rev.shape == (ranks[0].size,)


# ------------------------------------------------------------------------------------------ activation and FFN stages
def test_naive_activations_fail_the_golden(oracle_mod, golden):
    g, u = f32(golden["act_g_bits"]), f32(golden["act_u_bits"])
    want = golden["act_h_bits"]
    assert np.array_equal(oracle_mod.activation(g, u).view(np.uint32), want)
    with np.errstate(over="ignore", invalid="ignore"):
        plain = ((g / (np.float32(1.0) + np.exp(-g, dtype=np.float32))).astype(np.float32) * u).astype(np.float32)
        clamped = (((np.clip(g, -60, 60) / (1.0 + np.exp(-np.clip(g, -60, 60).astype(np.float64)))).astype(np.float32)) * u).astype(np.float32)
    finite = np.isfinite(f32(want))
    assert (plain.view(np.uint32)[finite] != want[finite]).any()            # a positive exponential / FP32 divide differs in bits
    assert (clamped.view(np.uint32)[finite] != want[finite]).any()          # the coordinator's clamped FP64 form is another lattice


def test_ffn_stage_variants_fail_the_golden(oracle_mod, golden):
    from mimo26f_afd_b200 import synth

    seed, e = int(golden["exp_seed"][0]), int(golden["exp_expert"][0])
    t = [synth.expert_tensor_np(seed, n, e) for n in synth.TENSORS]
    full = oracle_mod.expert_ffn(golden["exp_xp"], golden["exp_xs"], *t)
    want = f32(golden["exp_full_bits"])
    assert np.array_equal(full["y"], want)
    tol = lambda got: (np.abs(got - want) <= 1e-5 + 1e-5 * np.abs(want)).all()
    # FC2 on the unquantised intermediate (dropping the FC1 -> FC2 quantiser) leaves the stage tolerance
    down = oracle_mod.mxfp4_unpack(t[4], t[5]).astype(np.float64)
    y_noq = (full["h"].astype(np.float64) @ down.T).astype(np.float32)
    assert not tol(y_noq)
    # rounding the intermediate to BF16 before the quantiser changes intermediate bytes
    h_bf = (bf16_rne(full["h"]).astype(np.uint32) << 16).view(np.float32).reshape(full["h"].shape)
    pq, ps, _ = oracle_mod.quant_v1(h_bf)
    assert (pq.reshape(full["mid_q"].shape) != golden["exp_mid_payload"]).any()
    # gate and up swapped (the prepared image of the reference stores up first): another function altogether
    swapped = oracle_mod.expert_ffn(golden["exp_xp"], golden["exp_xs"], t[2], t[3], t[0], t[1], t[4], t[5])
    assert not tol(swapped["y"])
