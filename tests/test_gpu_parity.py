"""Parity of the CUDA path against the CPU oracle, through the C ABI, on a B200.

Bars: quantised bytes, permutation indices, the ordered combine, BF16 rounding and the rank sum are compared
bit for bit; GEMM stages against the oracle's FP64-dot lattice within the reference's componentwise
tolerance 1e-5 + 1e-5 |want| (crates/mimo26-repack/tests/lattice_compare.py:12-13) and end to end within
relative L2 <= 1e-3 and max-abs <= 2e-2 on the FP32 pre-BF16 plane.

An E4M3 bin crossing (a last-bit difference of the FP32 intermediate that lands on the other side of a
quantiser rounding boundary) is legitimate and is counted, never hidden: the intermediate bytes must equal
the codec applied to the candidate's OWN FP32 intermediate exactly, FC2 is checked against the oracle run on
the candidate's own intermediate bytes, and the end-to-end max-abs bound is applied to rows without a crossing.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

H, I, TOPK = 4096, 2048, 8
SEED = 0x26AFD


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) / max(np.linalg.norm(b.astype(np.float64)), 1e-30))


@pytest.fixture(scope="module")
def dev():
    import torch

    assert torch.cuda.is_available(), "these tests need the GPU box"
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def weights(dev):
    from mimo26f_afd_b200 import synth

    return synth.layer_torch(SEED, dev)


@pytest.fixture(scope="module")
def layer(weights):
    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import synth

    return M.Layer.from_checkpoint(*[weights[n] for n in synth.TENSORS])


@pytest.fixture(scope="module")
def scratch():
    import mimo26f_afd_b200 as M

    s = M.Scratch()
    s.set_debug(1)
    return s


def to_dev(a, dev):
    import torch

    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).to(dev)
    return torch.from_numpy(a).to(dev)


def run_dev(layer, scratch, dev, x_bits, ids, w, codec=0, x_dtype=0, x_scales=None):
    import torch

    from mimo26f_afd_b200 import expert

    t = ids.shape[0]
    out = torch.empty((t, H), dtype=torch.int16, device=dev)
    part = torch.empty((t, H), dtype=torch.float32, device=dev)
    xs = None if x_scales is None else to_dev(x_scales, dev)
    xd, idd, wd = to_dev(x_bits, dev), to_dev(ids, dev), to_dev(w, dev)
    expert.ffn_dev(layer, scratch, xd, idd, wd, t, out, partial_out=part, codec=codec, x_dtype=x_dtype, x_scales=xs)
    scratch.status()
    return out.cpu().numpy().view(np.uint16), part.cpu().numpy()


# ------------------------------------------------------------------------------------------ quantisers
@pytest.mark.parametrize("codec", [0, 1])
def test_quantisers_bit_exact_on_reference_corpus(dev, golden, codec):
    import torch

    from mimo26f_afd_b200 import expert

    x = np.ascontiguousarray(golden["qv1_x_bits"]).view(np.float32).reshape(-1)
    xd = torch.from_numpy(x).to(dev)
    p = torch.zeros(x.size, dtype=torch.uint8, device=dev)
    s = torch.zeros(x.size // 32, dtype=torch.uint8, device=dev)
    f = torch.zeros(1, dtype=torch.int32, device=dev)
    expert.quantize_dev(xd, expert.X_F32, x.size, codec, p, s, f)
    torch.cuda.synchronize()
    assert int(f.item()) == 0
    want_p, want_s = (golden["wire_payload"], golden["wire_scales"]) if codec == 0 else (golden["qv1_payload"], golden["qv1_scales"])
    assert np.array_equal(s.cpu().numpy(), want_s)
    assert np.array_equal(p.cpu().numpy(), want_p)


@pytest.mark.parametrize("codec", [0, 1])
def test_quantisers_bf16_input_and_ragged_sizes(dev, oracle_mod, codec):
    import torch

    from mimo26f_afd_b200 import expert, synth

    for tokens in (1, 3, 16):
        bits = synth.activations_bf16(SEED + tokens, tokens)
        bits[0, :32] = 0                                   # a zero block
        bits[0, 32:64] = synth.bf16_rne_np(np.full(32, 1e-20, np.float32))
        x = synth.bf16_to_f32_np(bits)
        p = torch.zeros(bits.size, dtype=torch.uint8, device=dev)
        s = torch.zeros(bits.size // 32, dtype=torch.uint8, device=dev)
        f = torch.zeros(1, dtype=torch.int32, device=dev)
        expert.quantize_dev(to_dev(bits, dev), expert.X_BF16, bits.size, codec, p, s, f)
        torch.cuda.synchronize()
        if codec == 0:
            wp, ws = oracle_mod.quant_wire(x)
            assert ws.reshape(-1)[0] == 0
        else:
            wp, ws, _ = oracle_mod.quant_v1(x)
        assert np.array_equal(p.cpu().numpy(), wp.reshape(-1)) and np.array_equal(s.cpu().numpy(), ws.reshape(-1))


def test_wire_quantiser_wide_dynamic_range_and_ties(dev, oracle_mod):
    """The wire codec over the whole FP32 range: block maxima from 2^-140 to 2^120, elements down to 2^-60 of their
    block's maximum, exact ties and their neighbours at every grid point, signed zeros, infinities and NaN."""
    import torch

    from mimo26f_afd_b200 import expert

    rng = np.random.default_rng(17)
    n_blocks = 8192
    exp = rng.integers(-140, 121, size=(n_blocks, 1)).astype(np.float64)
    rel = rng.integers(-60, 1, size=(n_blocks, 32)).astype(np.float64)
    mant = 1.0 + rng.integers(0, 1 << 23, size=(n_blocks, 32)) / float(1 << 23)
    sign = np.where(rng.integers(0, 2, size=(n_blocks, 32)) == 1, -1.0, 1.0)
    with np.errstate(over="ignore", under="ignore"):
        x = (sign * mant * np.exp2(exp + rel)).astype(np.float32)
    # ties: (m + 1/2) quanta of the E4M3 grid, and one FP32 ulp either side, scaled into each block
    grid = np.array([(8 + m + 0.5) / 8.0 * 2.0 ** e for e in range(-6, 9) for m in range(8)] + [(m + 0.5) * 2.0 ** -9 for m in range(8)])
    for b in range(0, 2048):
        s = 2.0 ** int(exp[b, 0])
        t = np.float32(grid[b % grid.size] * s / 256.0)
        x[b, 1:4] = [np.nextafter(t, np.float32(0)), t, np.nextafter(t, np.float32(np.inf))]
        x[b, 0] = np.float32(256.0 * s / 256.0 * 1.75)
    x[4000, 5], x[4001, 6], x[4002, 7], x[4003, :] = np.inf, -np.inf, np.nan, 0.0
    x[4004, 3] = -0.0
    want_p, want_s = oracle_mod.quant_wire(x)
    xd = torch.from_numpy(x).to(dev)
    p = torch.empty(x.size, dtype=torch.uint8, device=dev)
    s_ = torch.empty(x.size // 32, dtype=torch.uint8, device=dev)
    fault = torch.zeros(1, dtype=torch.int32, device=dev)
    expert.quantize_dev(xd, expert.X_F32, x.size, expert.CODEC_WIRE, p, s_, fault)
    torch.cuda.synchronize()
    assert np.array_equal(s_.cpu().numpy(), want_s.reshape(-1))
    assert np.array_equal(p.cpu().numpy(), want_p.reshape(-1))


def test_producer_router_and_quantiser_in_one_launch(dev, oracle_mod):
    """Router top-8 from FP32 logits against the oracle (indices exact, weights within one FP32 ulp: the device's FP64
    exp is not correctly rounded) on the reference-generated fixture and on a larger seeded batch with ties; the
    quantiser half of the same launch writes the bytes the stand-alone quantiser writes."""
    import os

    import torch

    from mimo26f_afd_b200 import expert, synth

    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "router_vectors.npz"))
    cases = [(g["logits_bits"].view(np.float32), g["bias_bits"].view(np.float32), g["idx"], g["weight_bits"].view(np.float32))]
    rng = np.random.default_rng(23)
    big = (rng.standard_normal((1000, 256)) * 1.5).astype(np.float32)
    big[5] = 0.0                                              # a 256-way tie
    big[6, 10:20] = big[6, 30]                                # ties inside a row
    bias = (rng.standard_normal(256) * 0.05).astype(np.float32)
    cases.append((big, bias, *oracle_mod.router_from_logits(big, bias)))
    cases.append((big, None, *oracle_mod.router_from_logits(big, None)))
    for logits, b, want_idx, want_w in cases:
        t = logits.shape[0]
        x_bits = synth.activations_bf16(SEED + 11, t)
        ids = torch.empty((t, TOPK), dtype=torch.int32, device=dev)
        w = torch.empty((t, TOPK), dtype=torch.float32, device=dev)
        p = torch.empty((t, H), dtype=torch.uint8, device=dev)
        s_ = torch.empty((t, H // 32), dtype=torch.uint8, device=dev)
        fault = torch.zeros(1, dtype=torch.int32, device=dev)
        expert.produce_dev(to_dev(logits, dev), None if b is None else to_dev(b, dev), t, ids, w, x=to_dev(x_bits, dev),
                           payload=p, scales=s_, fault=fault)
        torch.cuda.synchronize()
        assert np.array_equal(ids.cpu().numpy(), want_idx)
        got_w = w.cpu().numpy()
        ulp = np.abs(got_w.view(np.int32).astype(np.int64) - np.ascontiguousarray(want_w).view(np.int32).astype(np.int64))
        assert ulp.max() <= 1, ulp.max()
        oq, os_ = oracle_mod.quant_wire(synth.bf16_to_f32_np(x_bits))
        assert np.array_equal(p.cpu().numpy(), oq) and np.array_equal(s_.cpu().numpy(), os_) and int(fault.item()) == 0
        # routing only
        ids2 = torch.empty_like(ids); w2 = torch.empty_like(w)
        expert.produce_dev(to_dev(logits, dev), None if b is None else to_dev(b, dev), t, ids2, w2)
        torch.cuda.synchronize()
        assert torch.equal(ids2, ids) and torch.equal(w2, w)


def test_quant_v1_faults_write_nothing(dev):
    import torch

    from mimo26f_afd_b200 import expert

    x = np.ones(96, np.float32)
    x[40] = np.inf
    p = torch.full((96,), 0xEE, dtype=torch.uint8, device=dev)
    s = torch.full((3,), 0xEE, dtype=torch.uint8, device=dev)
    f = torch.zeros(1, dtype=torch.int32, device=dev)
    expert.quantize_dev(torch.from_numpy(x).to(dev), expert.X_F32, 96, 1, p, s, f)
    torch.cuda.synchronize()
    assert int(f.item()) == 4
    assert (p.cpu().numpy()[32:64] == 0xEE).all() and s.cpu().numpy()[1] == 0xEE      # the faulting block is untouched
    assert (p.cpu().numpy()[:32] == 0x78).all() and s.cpu().numpy()[0] == 119          # 1.0 = 256 x 2^-8


# ------------------------------------------------------------------------------------------ combine, rank sum
def test_route_reduce_bit_exact_and_faults(dev, oracle_mod):
    import torch

    from mimo26f_afd_b200 import expert

    rng = np.random.default_rng(3)
    rows = 5
    y = (rng.normal(size=(rows, 8, H)) * 9).astype(np.float32)
    y[0, :4, 0] = [1e8, -1e8, 1.0, 1.0]                       # order matters
    y[1, :2, 1] = [1 - 2.0 ** -23, 1.0]
    w = rng.uniform(0, 1, (rows, 8)).astype(np.float32)
    w[1, 0] = 1 + 2.0 ** -23                                  # separate multiply and add, no FMA
    partial = torch.empty((rows, H), dtype=torch.float32, device=dev)
    bf = torch.empty((rows, H), dtype=torch.int16, device=dev)
    f = torch.zeros(1, dtype=torch.int32, device=dev)
    expert.route_reduce_dev(to_dev(y, dev), to_dev(w, dev), rows, partial, bf, f)
    torch.cuda.synchronize()
    rc, wp, wb = oracle_mod.route_reduce(y, w)
    assert rc == 0 and int(f.item()) == 0
    assert np.array_equal(partial.cpu().numpy().view(np.uint32), wp.view(np.uint32))
    assert np.array_equal(bf.cpu().numpy().view(np.uint16), wb)
    w[2, 5] = np.nan
    expert.route_reduce_dev(to_dev(y, dev), to_dev(w, dev), rows, partial, bf, f)
    torch.cuda.synchronize()
    assert int(f.item()) == 8


def test_rank_sum_order(dev, oracle_mod):
    import torch

    from mimo26f_afd_b200 import expert, synth

    rng = np.random.default_rng(4)
    n = 3 * H + 5
    planes = synth.bf16_rne_np((rng.normal(size=(8, n)) * 100).astype(np.float32))
    planes[:4, 0] = synth.bf16_rne_np(np.array([2.0 ** 24, 1.0, -(2.0 ** 24), 1.0], np.float32))
    for g in (1, 2, 4, 8):
        out = torch.empty(n, dtype=torch.float32, device=dev)
        expert.rank_sum_dev([to_dev(planes[r], dev) for r in range(g)], n, out)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy().view(np.uint32), oracle_mod.rank_sum(planes[:g]).view(np.uint32))
    # the coordinator's h += f folded in: identical to summing first and adding afterwards, also in place
    h = rng.standard_normal(n).astype(np.float32)
    want = (h + oracle_mod.rank_sum(planes[:4])).astype(np.float32)
    hd = to_dev(h, dev)
    out = torch.empty(n, dtype=torch.float32, device=dev)
    expert.rank_sum_dev([to_dev(planes[r], dev) for r in range(4)], n, out, residual=hd)
    expert.rank_sum_dev([to_dev(planes[r], dev) for r in range(4)], n, hd, residual=hd)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    assert np.array_equal(hd.cpu().numpy().view(np.uint32), want.view(np.uint32))
    out = torch.empty(n, dtype=torch.float32, device=dev)
    expert.rank_sum_dev([to_dev(planes[r], dev) for r in (0, 2, 1, 3)], n, out)
    torch.cuda.synchronize()
    assert out.cpu().numpy()[0] == 2.0                        # the swapped order gives the other answer


class _DevView:
    """A device address as something torch can wrap (CUDA array interface)."""

    def __init__(self, ptr, n, typestr):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 2}


def test_plane_exchange_two_windows_one_process(dev, oracle_mod):
    """The exchange kernel with both ranks' windows in this process: a rank's peer is published from the host, so no
    kernel waits for another kernel. Checks the rank-ordered sum, the alternating slots and the bounded wait."""
    import torch

    import mimo26f_afd_b200 as M

    n = 16 * H
    rng = np.random.default_rng(11)
    ex = [M.Exchange(n * 2, r, 2, export=False) for r in range(2)]
    for e in ex:
        e.connect_local(ex)
    out = [torch.empty(n, dtype=torch.float32, device=dev) for _ in range(2)]
    for step in range(3):
        planes = (rng.standard_normal((2, n)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
        planes[0, 0], planes[1, 0] = 0x4B80, 0x3F80           # 2^24 + 1: the order of the additions shows
        for r in range(2):
            torch.as_tensor(_DevView(ex[r].plane(), n, "<i2"), device=dev).copy_(to_dev(planes[r], dev))
        torch.cuda.synchronize()
        for r in range(2):
            ex[r].publish_as(1 - r)
            ex[r].sum(n, out[r])
            ex[r].status()
        want = oracle_mod.rank_sum(planes)
        for r in range(2):
            assert np.array_equal(out[r].cpu().numpy().view(np.uint32), want.view(np.uint32)), (step, r)
        if step == 1:                                           # the same step's planes again, with h += f folded in
            h = rng.standard_normal(n).astype(np.float32)
            for r in range(2):
                torch.as_tensor(_DevView(ex[r].plane(), n, "<i2"), device=dev).copy_(to_dev(planes[r], dev))
            torch.cuda.synchronize()
            for r in range(2):
                hd = to_dev(h, dev)
                ex[r].publish_as(1 - r)
                ex[r].sum(n, hd, residual=hd)
                ex[r].status()
                assert np.array_equal(hd.cpu().numpy().view(np.uint32), (h + want).astype(np.float32).view(np.uint32))
    # a peer that never publishes: the wait runs out, the status says so, and the window works again afterwards
    ex[0].set_wait_ms(20)
    ex[0].sum(n, out[0])
    with pytest.raises(M.ExpertError) as e:
        ex[0].status()
    assert e.value.code == 5 and "gave up waiting" in e.value.message
    ex[1].publish_as(0); ex[1].sum(n, out[1]); ex[1].status()   # rank 1 catches up with the step rank 0 lost
    ex[0].publish_as(1); ex[0].sum(n, out[0]); ex[0].status()
    with pytest.raises(M.ExpertError):
        ex[0].sum(n + 4, out[0])                                # not a multiple of 8 / larger than the plane
    for e_ in ex:
        e_.close()


@pytest.mark.parametrize("tokens,zipf,n_rep", [(3, 0.0, 0), (9, 0.0, 0), (96, 1.2, 0), (300, 0.0, 0), (96, 1.2, 6), (700, 1.0, 12)])
def test_expert_parallel_two_ranks_one_process_equals_single_gpu(layer, scratch, dev, tokens, zipf, n_rep):
    """Expert parallelism with both ranks in this process (each rank's rendezvous is marked reached from the host, so no
    kernel waits for another kernel): experts split 128 / 128, tokens split in two blocks, rows gathered from and
    results scattered to the owner's window. Output must equal the single-GPU layer's bit for bit. With n_rep > 0 both
    ranks also hold copies of the batch's n_rep busiest experts (routes to those are served where the token lives), and
    every route must still be served exactly once."""
    import torch

    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import synth

    x_bits = synth.activations_bf16(SEED + 3, tokens)
    ids, w = synth.routing(SEED + 3, tokens, zipf)
    bf_ref, part_ref = run_dev(layer, scratch, dev, x_bits, ids, w)
    layers, eps = [], []
    counts = np.bincount(ids.reshape(-1), minlength=256)
    hot = np.argsort(-counts, kind="stable")[:n_rep].astype(np.int32)
    reps = synth.layer_torch(SEED, dev, experts=hot) if n_rep else None
    for r in range(2):
        wt = synth.layer_torch(SEED, dev, n_experts=128, first_expert=128 * r)
        layers.append(M.Layer.from_checkpoint_ep(*[wt[n] for n in synth.TENSORS], ep_rank=r, ep_size=2,
                                                 replicas=[reps[n] for n in synth.TENSORS] if n_rep else None, replica_ids=hot))
        del wt
        eps.append(M.ExpertParallel(tokens, r, 2, export=False))
    for e in eps:
        e.connect_local(eps)
    s2 = M.Scratch()
    lo = [0, eps[0].rows(0), tokens]
    assert eps[0].rows(0) + eps[0].rows(1) == tokens and eps[1].rows() == tokens - lo[1]
    xd, idd, wd = to_dev(x_bits, dev), to_dev(ids, dev), to_dev(w, dev)
    outs = [torch.empty((lo[r + 1] - lo[r], H), dtype=torch.int16, device=dev) for r in range(2)]
    parts = [torch.empty((lo[r + 1] - lo[r], H), dtype=torch.float32, device=dev) for r in range(2)]
    for step in range(2):
        for r in range(2):
            eps[r].publish_as(1 - r, 0)
            eps[r].begin(xd[lo[r]:lo[r + 1]], idd[lo[r]:lo[r + 1]], wd[lo[r]:lo[r + 1]], lo[r + 1] - lo[r])
        for r in range(2):
            eps[r].publish_as(1 - r, 1)
            eps[r].compute(layers[r], s2)
            s2.status()
        for r in range(2):
            eps[r].finish(outs[r], parts[r])
            eps[r].status()
        torch.cuda.synchronize()
        for r in range(2):
            assert np.array_equal(outs[r].cpu().numpy().view(np.uint16), bf_ref[lo[r]:lo[r + 1]]), (step, r)
            assert np.array_equal(parts[r].cpu().numpy().view(np.uint32), part_ref[lo[r]:lo[r + 1]].view(np.uint32)), (step, r)
        if n_rep and step == 0:
            # the rank that ran last planned only the routes it serves: the replicated experts' routes of its own tokens
            # plus its own block's routes of all tokens
            inv = s2.peek("inverse", np.int32, (tokens * TOPK,))
            mine = np.isin(ids, hot) & (np.arange(tokens)[:, None] >= lo[1]) | (~np.isin(ids, hot) & (ids >= 128))
            assert np.array_equal(inv >= 0, mine.reshape(-1))
    # a rendezvous nobody else reaches: bounded wait, status 5, window usable afterwards
    eps[0].set_wait_ms(20)
    eps[0].begin(xd[lo[0]:lo[1]], idd[lo[0]:lo[1]], wd[lo[0]:lo[1]], lo[1])
    with pytest.raises(M.ExpertError) as e:
        eps[0].status()
    assert e.value.code == 5
    eps[1].publish_as(0, 0)                                  # rank 1 catches up with the step rank 0 lost
    eps[1].begin(xd[lo[1]:], idd[lo[1]:], wd[lo[1]:], tokens - lo[1])
    eps[1].status()
    # an expert id outside [0, 256) on any rank's tokens is still a plan rejection on every expert-parallel rank
    bad = to_dev(np.where(np.arange(tokens * TOPK).reshape(tokens, TOPK) == tokens * TOPK - 1, 300, ids).astype(np.int32), dev)
    for r in range(2):
        eps[r].publish_as(1 - r, 0)
        eps[r].begin(xd[lo[r]:lo[r + 1]], bad[lo[r]:lo[r + 1]], wd[lo[r]:lo[r + 1]], lo[r + 1] - lo[r])
    eps[0].publish_as(1, 1)
    eps[0].compute(layers[0], s2)
    with pytest.raises(M.ExpertError) as e:
        s2.status()
    assert e.value.code == 3
    with pytest.raises(M.ExpertError) as e:
        eps[0].compute(layers[1], s2)                       # the other rank's layer: refused before anything is launched
    assert e.value.code == 1
    for e_ in eps:
        e_.close()


# ------------------------------------------------------------------------------------------ the whole path
def fc2_bound(oracle_mod, tensors, ids, inverse, mid_q, mid_s, want_y, tp_rank=0, tp_size=1):
    """Componentwise bound for an FC2 output against the oracle's exactly-summed dot: the reference comparator's
    1e-5 + 1e-5 |want| (crates/mimo26-repack/tests/lattice_compare.py:12-13) plus the forward error of an FP32 running
    sum over the K = I_local / 32 block-scaled MMA steps. Every product is exact in FP32 range; the accumulator is rounded
    once per MMA step and its magnitude never exceeds S = sum_k |mid_k w_k|, so the error is at most
    (K / 32) * 2^-24 * S for round-to-nearest, twice that for a truncating adder: 2 * (K / 32) * 2^-24 * S is used.
    (The reference bounds its own wire sum the same way: 3 * 2^-24 * sum |decoded y_r|, lattice_compare.py:118-121.)
    mid_q / mid_s are in grouped order, want_y in original route order."""
    il = I // tp_size
    i0 = tp_rank * il
    # dequantise the intermediate: payload code x 2^(scale - 127)
    table = oracle_mod.e4m3_table()
    mid = np.abs(table[mid_q].astype(np.float64) * np.exp2(np.repeat(mid_s.astype(np.int32) - 127, 32, axis=1)))
    S = np.zeros(want_y.shape, np.float64)
    flat = ids.reshape(-1)
    for e in np.unique(flat):
        routes_e = np.nonzero(flat == e)[0]
        wd = np.abs(oracle_mod.mxfp4_unpack(tensors["down_w"][e], tensors["down_s"][e])[:, i0:i0 + il]).astype(np.float64)
        S[routes_e] = mid[inverse[routes_e]] @ wd.T
    steps = il // 32
    return 1e-5 + 1e-5 * np.abs(want_y) + 2.0 * steps * 2.0 ** -24 * S


def check_ffn(layer, scratch, dev, oracle_mod, tokens, zipf, codec, tp_rank=0, tp_size=1, seed=SEED):
    from mimo26f_afd_b200 import synth

    x_bits = synth.activations_bf16(seed, tokens)
    ids, w = synth.routing(seed, tokens, zipf)
    bf, partial = run_dev(layer, scratch, dev, x_bits, ids, w, codec=codec)
    routes, il = tokens * TOPK, I // tp_size
    x = synth.bf16_to_f32_np(x_bits)
    oxq, oxs = oracle_mod.quant_wire(x) if codec == 0 else oracle_mod.quant_v1(x)[:2]
    # (1) quantised activations and permutation indices: exact
    assert np.array_equal(scratch.peek("x_payload", np.uint8, (tokens, H)), oxq)
    assert np.array_equal(scratch.peek("x_scales", np.uint8, (tokens, H // 32)), oxs)
    st, oinv, oorig, ogw, counts = oracle_mod.plan(ids, w)
    assert st == 0
    assert np.array_equal(scratch.peek("inverse", np.int32, (routes,)), oinv)
    assert np.array_equal(scratch.peek("original_routes", np.int32, (routes,)), oorig)
    assert np.array_equal(scratch.peek("grouped_weights", np.float32, (routes,)).view(np.uint32), ogw.view(np.uint32))
    meta = scratch.peek("meta", np.uint32, (8,))
    assert meta[0] == 0 and meta[4] == (counts > 0).sum() and meta[5] == counts.max()
    # (2) FC1 + activation against the lattice oracle; intermediate bytes against the codec on the candidate's own FP32
    tensors = synth.layer_np(SEED, np.unique(ids))
    ref = oracle_mod.ffn_layer(tensors, oxq, oxs, ids, w, tp_rank=tp_rank, tp_size=tp_size, stages=True)
    assert ref["rc"] == 0
    h = scratch.peek("mid_f32", np.float32, (routes, il))
    assert (np.abs(h - ref["h"]) <= 1e-5 + 1e-5 * np.abs(ref["h"])).all()
    mid_q = scratch.peek("mid_payload", np.uint8, (routes, il))
    mid_s = scratch.peek("mid_scales", np.uint8, (routes, il // 32))
    p_own, s_own, f_own = oracle_mod.quant_v1(h)
    assert not f_own.any() and np.array_equal(mid_q, p_own) and np.array_equal(mid_s, s_own)
    assert np.array_equal(mid_s, ref["mid_s"]) or (mid_s != ref["mid_s"]).sum() <= 2
    crossed_rows = np.unique(np.nonzero(mid_q != ref["mid_q"])[0])          # grouped rows with an E4M3 bin crossing
    crossings = int((mid_q != ref["mid_q"]).sum())
    assert crossings <= max(4, mid_q.size // 50000), crossings
    # (3) FC2 against the oracle on the rows without a crossing, componentwise: the protocol's 1e-5 + 1e-5 |want| plus the
    # accumulation term of an FP32 running sum (see fc2_bound)
    y = scratch.peek("y", np.float32, (routes, H))
    clean = np.ones(routes, bool)
    clean[oorig[crossed_rows]] = False
    bound = fc2_bound(oracle_mod, tensors, ids, oinv, ref["mid_q"], ref["mid_s"], ref["y"], tp_rank, tp_size)
    excess = np.abs(y[clean] - ref["y"][clean]) - (1e-5 + 1e-5 * np.abs(ref["y"][clean]))
    assert (np.abs(y[clean] - ref["y"][clean]) <= bound[clean]).all(), float((excess / (bound[clean] - 1e-5 - 1e-5 * np.abs(ref["y"][clean]))).max())
    # (4) ordered combine and BF16: exact given the candidate's own y
    rc, p_own, b_own = oracle_mod.route_reduce(y, w)
    assert rc == 0
    assert np.array_equal(p_own.view(np.uint32), partial.view(np.uint32)) and np.array_equal(b_own, bf)
    # (5) end to end, on the FP32 pre-BF16 plane
    assert rel_l2(partial, ref["partial"]) <= 1e-3
    clean_tokens = np.ones(tokens, bool)
    clean_tokens[oorig[crossed_rows] // TOPK] = False
    assert np.abs(partial[clean_tokens] - ref["partial"][clean_tokens]).max() <= 2e-2
    flips = int((bf != ref["bf16"]).sum())
    dec = lambda b: (b.astype(np.uint32) << 16).view(np.float32)
    # a BF16 ulp is at most 2^-7 of the value: outputs agree with the oracle to one ulp (plus the FP32 tolerance near zero)
    assert (np.abs(dec(bf) - dec(ref["bf16"]))[clean_tokens] <= 2.0 ** -7 * np.abs(ref["partial"][clean_tokens]) + 1e-4).all()
    return dict(crossings=crossings, bf16_flips=flips, rel_l2=rel_l2(partial, ref["partial"]))


def test_ffn_decode_16_tokens_wire_codec(layer, scratch, dev, oracle_mod):
    """The decode batch: 16 tokens, uniform routing, 128 routes over about 102 experts."""
    r = check_ffn(layer, scratch, dev, oracle_mod, 16, 0.0, codec=0)
    print("decode16", r)


def test_ffn_decode_16_tokens_quant_v1_input(layer, scratch, dev, oracle_mod):
    r = check_ffn(layer, scratch, dev, oracle_mod, 16, 0.0, codec=1, seed=SEED + 1)
    print("decode16 v1", r)


def test_ffn_verify_round_128_tokens_zipf(layer, scratch, dev, oracle_mod):
    """The speculative verify round: 16 streams x 8 tokens, Zipf(1.2) expert popularity (one expert gets most rows)."""
    r = check_ffn(layer, scratch, dev, oracle_mod, 128, 1.2, codec=0)
    print("verify128", r)


@pytest.mark.parametrize("tokens", [1, 2, 33, 113])
def test_ffn_ragged_token_counts(layer, scratch, dev, oracle_mod, tokens):
    """1 and 2 tokens also run FC1 with half items (64 gate + 64 up rows per item): fewer than two rounds of full items."""
    check_ffn(layer, scratch, dev, oracle_mod, tokens, 0.7, codec=0, seed=SEED + tokens)


@pytest.mark.parametrize("tp_rank,tp_size,tokens", [(3, 8, 16), (1, 4, 9), (7, 8, 18)])
def test_ffn_tensor_parallel_rank_stages_with_half_items(weights, scratch, dev, oracle_mod, tp_rank, tp_size, tokens):
    """A rank of a tensor-parallel group on the decode batch, every stage against the oracle's slice: these sizes run FC1
    with half items (the up accumulators cross from their warps to the gate warps through shared memory)."""
    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import synth

    L = M.Layer.from_checkpoint(*[weights[n] for n in synth.TENSORS], tp_rank=tp_rank, tp_size=tp_size)
    try:
        check_ffn(L, scratch, dev, oracle_mod, tokens, 0.0, codec=0, tp_rank=tp_rank, tp_size=tp_size, seed=SEED + 31 * tokens)
    finally:
        L.close()


@pytest.mark.parametrize("tokens,cut,zipf", [(129, 1, 1.5), (130, 111, 0.5), (145, 61, 1.5), (513, 325, 0.0), (1025, 350, 1.5), (2469, 1206, 0.0)])
def test_bytes_do_not_depend_on_the_batch_cut(layer, scratch, dev, oracle_mod, tokens, cut, zipf):
    """A token's output bytes depend on its own row and routes only: the same tokens served as one batch or as two
    give identical FP32 planes and BF16 rows, although the two forms take different paths (fused or general prologue,
    one-CTA tiles of 16..128 rows or CTA-pair tiles of 256, different positions inside an expert's group). The sizes sit
    on the edges of those classes. Plan indices are checked against the oracle at each size."""
    from mimo26f_afd_b200 import synth

    x_bits = synth.activations_bf16(SEED + tokens, tokens)
    ids, w = synth.routing(SEED + tokens, tokens, zipf)
    bf, part = run_dev(layer, scratch, dev, x_bits, ids, w)
    st, oinv, _, _, _ = oracle_mod.plan(ids, w)
    assert st == 0 and np.array_equal(scratch.peek("inverse", np.int32, (tokens * TOPK,)), oinv)
    bf_a, part_a = run_dev(layer, scratch, dev, x_bits[:cut], ids[:cut], w[:cut])
    bf_b, part_b = run_dev(layer, scratch, dev, x_bits[cut:], ids[cut:], w[cut:])
    assert np.array_equal(np.concatenate([bf_a, bf_b]), bf)
    assert np.array_equal(np.concatenate([part_a, part_b]).view(np.uint32), part.view(np.uint32))


@pytest.mark.parametrize("tokens", [7, 32, 33, 128])
def test_small_request_prologue_input_forms_agree(layer, scratch, dev, oracle_mod, tokens):
    """Requests of at most 128 tokens quantise, plan and permute in one launch (256 threads per CTA up to 32 tokens,
    1024 above). BF16 and FP32 activations (both codecs)
    and caller-quantised E4M3 rows must give the same bytes at every stage, and the quant_v1 faults must surface."""
    from mimo26f_afd_b200 import synth
    import mimo26f_afd_b200 as M

    x_bits = synth.activations_bf16(SEED + 7, tokens)
    x = synth.bf16_to_f32_np(x_bits)
    ids, w = synth.routing(SEED + 7, tokens, 0.6)
    for codec in (0, 1):
        bf_a, part_a = run_dev(layer, scratch, dev, x_bits, ids, w, codec=codec, x_dtype=0)
        xq = scratch.peek("x_payload", np.uint8, (tokens, H))
        xs = scratch.peek("x_scales", np.uint8, (tokens, H // 32))
        oq, os_ = oracle_mod.quant_wire(x) if codec == 0 else oracle_mod.quant_v1(x)[:2]
        assert np.array_equal(xq, oq) and np.array_equal(xs, os_)
        bf_b, part_b = run_dev(layer, scratch, dev, x, ids, w, codec=codec, x_dtype=1)
        assert np.array_equal(bf_a, bf_b) and np.array_equal(part_a.view(np.uint32), part_b.view(np.uint32))
        bf_c, part_c = run_dev(layer, scratch, dev, xq, ids, w, x_dtype=2, x_scales=xs)
        assert np.array_equal(bf_a, bf_c) and np.array_equal(part_a.view(np.uint32), part_c.view(np.uint32))
    bad = x.copy(); bad[tokens - 1, 77] = np.inf
    with pytest.raises(M.ExpertError) as e:
        run_dev(layer, scratch, dev, bad, ids, w, codec=1, x_dtype=1)
    assert e.value.code == 4
    run_dev(layer, scratch, dev, x_bits, ids, w)              # usable afterwards


def test_wrong_nibble_order_is_visible_and_outputs_stay_inside_their_rows(layer, scratch, dev, oracle_mod):
    """Two negatives on the whole path. (1) Against an oracle fed nibble-swapped weights (high nibble = even k, the
    naive order) the result is nowhere near the tolerance, so the parity tests do see the nibble order. (2) Poisoned
    guard rows after both output planes are untouched."""
    import torch

    from mimo26f_afd_b200 import expert, synth

    tokens = 5
    x_bits = synth.activations_bf16(SEED + 9, tokens)
    ids, w = synth.routing(SEED + 9, tokens, 0.0)
    out = torch.full((tokens + 2, H), 0x7FC1, dtype=torch.int16, device=dev)
    part = torch.full((tokens + 2, H), float("nan"), dtype=torch.float32, device=dev)
    expert.ffn_dev(layer, scratch, to_dev(x_bits, dev), to_dev(ids, dev), to_dev(w, dev), tokens, out, partial_out=part)
    scratch.status()
    assert (out[tokens:].cpu().numpy() == 0x7FC1).all() and np.isnan(part[tokens:].cpu().numpy()).all()
    got = part[:tokens].cpu().numpy()
    assert np.isfinite(got).all()
    xq, xs = oracle_mod.quant_wire(synth.bf16_to_f32_np(x_bits))
    tensors = synth.layer_np(SEED, np.unique(ids))
    good = oracle_mod.ffn_layer(tensors, xq, xs, ids, w)
    assert rel_l2(got, good["partial"]) <= 1e-3
    swap = lambda a: ((a >> 4) | (a << 4)).astype(np.uint8)
    naive = {k: (swap(v) if k.endswith("_w") else v) for k, v in tensors.items()}     # payload tensors end in _w
    bad = oracle_mod.ffn_layer(naive, xq, xs, ids, w)
    assert bad["rc"] == 0 and rel_l2(got, bad["partial"]) > 0.5


def test_exchange_sum_is_rank_ordered_in_all_24_arrival_orders(dev, oracle_mod):
    """Four ranks' windows in this process; the planes are written and published in every one of the 24 orders (the
    reference's coordinator test walks the same 24 arrival orders, crates/mimo26-wire/tests/r8_rank_order.rs); the sum
    must be the rank-ordered one every time. The planes are chosen so that every other order of additions differs."""
    import itertools

    import torch

    import mimo26f_afd_b200 as M

    n = 4096
    vals = np.array([2.0 ** 24, 1.0, -(2.0 ** 24), 1.0], np.float32)       # rank order: ((2^24 + 1) - 2^24) + 1 = 1
    planes = np.repeat((vals.view(np.uint32) >> 16).astype(np.uint16)[:, None], n, axis=1)
    rng = np.random.default_rng(5)
    planes[:, 1:] = (rng.standard_normal((4, n - 1)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    want = oracle_mod.rank_sum(planes)
    assert want[0] == 1.0
    ex = [M.Exchange(n * 2, r, 4, export=False) for r in range(4)]
    for e in ex:
        e.connect_local(ex)
    out = torch.empty(n, dtype=torch.float32, device=dev)
    for order in itertools.permutations(range(4)):
        for r in order:
            torch.as_tensor(_DevView(ex[r].plane(), n, "<i2"), device=dev).copy_(to_dev(planes[r], dev))
            if r != 0:
                ex[0].publish_as(r)
        ex[0].sum(n, out)
        ex[0].status()
        assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32)), order
        for r in range(1, 4):                               # the other ranks take the same step (their sums are not read)
            for q in range(4):
                if q != r:
                    ex[r].publish_as(q)
            ex[r].sum(n, torch.empty(n, dtype=torch.float32, device=dev))
            ex[r].status()
    for e in ex:
        e.close()


def test_tp4_from_canonical_image_matches_reference_slices(weights, dev, oracle_mod):
    """m26b_layer_new on the reference's canonical-v2 TP4 rank images: each rank's partial equals the oracle's
    rank slice, and the rank-ordered sum of the four BF16 planes equals the oracle's wire result bit for bit
    once the planes themselves agree."""
    import torch

    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import expert, synth

    tokens = 8
    x_bits = synth.activations_bf16(SEED + 5, tokens)
    ids, w = synth.routing(SEED + 5, tokens, 0.0)
    experts = np.unique(ids)
    tensors = synth.layer_np(SEED, experts)
    x = synth.bf16_to_f32_np(x_bits)
    oxq, oxs = oracle_mod.quant_wire(x)
    planes, ref_planes = [], []
    s = M.Scratch()
    for r in range(4):
        image = synth.canonical_rank_image_np(tensors, experts, r, 4)
        img_d = torch.from_numpy(image).to(dev)
        L = M.Layer.new(img_d, image.size, r)
        assert L.i_local == 512 and not L.all_scales_normal()   # experts without routes are zero-filled here: scale byte 0
        del img_d                                            # the image may be freed after layer_new
        bf, partial = run_dev(L, s, dev, oxq, ids, w, x_dtype=expert.X_E4M3, x_scales=oxs)
        ref = oracle_mod.ffn_layer(tensors, oxq, oxs, ids, w, tp_rank=r, tp_size=4)
        assert rel_l2(partial, ref["partial"]) <= 1e-3
        dec = lambda b: (b.astype(np.uint32) << 16).view(np.float32)
        # one BF16 ulp except where an intermediate crossed an E4M3 bin (counted in the single-rank tests)
        assert (np.abs(dec(bf) - dec(ref["bf16"])) <= 2.0 ** -7 * np.abs(ref["partial"]) + 1e-4).mean() >= 0.999
        planes.append(bf)
        ref_planes.append(ref["bf16"])
        L.close()
    out = torch.empty((tokens, H), dtype=torch.float32, device=dev)
    expert.rank_sum_dev([to_dev(p, dev) for p in planes], tokens * H, out)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), oracle_mod.rank_sum(np.stack(planes)).view(np.uint32))
    assert rel_l2(out.cpu().numpy(), oracle_mod.rank_sum(np.stack(ref_planes))) <= 1e-3


def test_host_abi_ffn_and_strided_frame(layer, scratch, dev, oracle_mod):
    """The reference-compatible host entry point: separate arrays and the request frame's 4224-byte rows."""
    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import synth

    tokens = 16
    x = synth.bf16_to_f32_np(synth.activations_bf16(SEED, tokens))
    ids, w = synth.routing(SEED, tokens, 0.0)
    xq, xs = oracle_mod.quant_wire(x)
    bf_dev, _ = run_dev(layer, scratch, dev, synth.activations_bf16(SEED, tokens), ids, w)
    bf = np.zeros((tokens, H), np.uint16)
    stats = M.ffn(layer, scratch, xq.reshape(-1), xs.reshape(-1), ids.reshape(-1), w.reshape(-1), tokens, bf.reshape(-1))
    assert np.array_equal(bf, bf_dev)
    assert stats.gpu_ms > 0 and stats.groups > 0 and len(stats.phase_ms) == 4
    # the split of the GPU time into stages costs the overlap of the kernels: measured only when asked for
    assert stats.phase_ms == (0.0, 0.0, 0.0, 0.0)
    scratch.set_debug(1 | 4)
    staged = M.ffn(layer, scratch, xq.reshape(-1), xs.reshape(-1), ids.reshape(-1), w.reshape(-1), tokens, bf.reshape(-1))
    scratch.set_debug(1)
    assert np.array_equal(bf, bf_dev)
    assert staged.phase_ms[0] > 0 and staged.phase_ms[1] == 0 and staged.phase_ms[2] > 0 and staged.phase_ms[3] > 0
    assert abs(sum(staged.phase_ms) - staged.gpu_ms) <= 0.02 * staged.gpu_ms + 0.005
    frame = np.zeros((tokens, 4224), np.uint8)
    frame[:, :H] = xq
    frame[:, H:] = xs
    bf2 = np.zeros((tokens, H), np.uint16)
    M.ffn_strided(layer, scratch, frame.reshape(-1), 4224, ids.reshape(-1), w.reshape(-1), tokens, bf2.reshape(-1))
    assert np.array_equal(bf2, bf_dev)


def test_plan_rejections_and_input_faults(layer, scratch, dev, oracle_mod):
    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import synth

    tokens = 4
    x = synth.bf16_to_f32_np(synth.activations_bf16(SEED, tokens))
    ids, w = synth.routing(SEED, tokens, 0.0)
    xq, xs = oracle_mod.quant_wire(x)
    bf = np.zeros((tokens, H), np.uint16)

    def call(i=ids, ww=w, q=xq, s=xs):
        return M.ffn(layer, scratch, q.reshape(-1), s.reshape(-1), i.reshape(-1), ww.reshape(-1), tokens, bf.reshape(-1))

    call()
    for mutate in ("dup", "neg", "big", "nan_w", "neg_w"):
        i2, w2 = ids.copy(), w.copy()
        if mutate == "dup":
            i2[1, 5] = i2[1, 0]
        elif mutate == "neg":
            i2[2, 2] = -1
        elif mutate == "big":
            i2[0, 7] = 256
        elif mutate == "nan_w":
            w2[3, 3] = np.nan
        else:
            w2[0, 0] = -0.5
        with pytest.raises(M.ExpertError) as e:
            call(i2, w2)
        assert e.value.code == 3 and "invalid routes" in e.value.message, mutate
    s2 = xs.copy(); s2[1, 7] = 0                       # a scale byte outside 105..247 poisons the row
    with pytest.raises(M.ExpertError) as e:
        call(s=s2)
    assert e.value.code == 4 and "input fault" in e.value.message
    q2 = xq.copy(); q2[2, 100] = 0x7F                  # an E4M3 NaN code
    with pytest.raises(M.ExpertError) as e:
        call(q=q2)
    assert e.value.code == 4
    call()                                             # the handles stay usable after every rejection


def test_exceptional_weight_scales(dev, oracle_mod):
    """Scale bytes 0, 1 and 60 (tiny scales) against the oracle, and the reserved byte 255: the checkpoint
    contract decodes it as 254 = 2^127 (crates/mimo26-expert/src/mxfp4.rs:24-29) where the hardware would read
    NaN. The 255/254 blocks carry zero payload, so the result is finite exactly when 255 was stored as 254."""
    import torch

    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import expert, synth

    tokens = 2
    ids = np.array([[0, 1, 2, 3, 4, 5, 6, 7], [7, 6, 5, 4, 3, 2, 1, 0]], np.int32)
    w = np.full((2, 8), 0.125, np.float32)
    tensors = synth.layer_np(SEED + 9, range(8), scale_lo=120, scale_hi=122)
    tensors["gate_s"][0, :, 0] = 0
    tensors["up_s"][1, :, 5] = 1
    tensors["gate_s"][3, 17, :] = 60
    tensors["down_s"][2, :, 3] = 255
    tensors["down_w"][2][:, 3 * 16:4 * 16] = 0
    tensors["up_s"][4, :, 9] = 254
    tensors["up_w"][4][:, 9 * 16:10 * 16] = 0
    x = synth.bf16_to_f32_np(synth.activations_bf16(SEED, tokens))
    xq, xs, _ = oracle_mod.quant_v1(x)
    dt = {n: torch.from_numpy(tensors[n]).to(dev) for n in synth.TENSORS}
    L = M.Layer.from_checkpoint(*[dt[n] for n in synth.TENSORS])
    assert not L.all_scales_normal()
    s = M.Scratch()
    bf, partial = run_dev(L, s, dev, xq, ids, w, x_dtype=expert.X_E4M3, x_scales=xs)
    ref = oracle_mod.ffn_layer(tensors, xq, xs, ids, w)
    assert ref["rc"] == 0 and np.isfinite(partial).all()
    assert rel_l2(partial, ref["partial"]) <= 1e-3


# ------------------------------------------------------------------------------------------ full size, by properties
def test_prefill_8192_tokens_properties_and_sampled_oracle(layer, dev, oracle_mod):
    """The 8,192-token prefill segment at full size. The oracle cannot run 65,536 routes, so: (a) the output is row-local -
    permuting the tokens permutes the outputs bit for bit, and two half-size calls give the same bytes; (b)
    doubling the route weights doubles the FP32 plane exactly; (c) the routes of two experts are checked
    against the oracle."""
    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import synth

    tokens = 8192
    s = M.Scratch()
    s.set_debug(0)
    x_bits = synth.activations_bf16(SEED + 2, tokens)
    ids, w = synth.routing(SEED + 2, tokens, 0.0)
    bf, partial = run_dev(layer, s, dev, x_bits, ids, w)
    y = s.peek("y", np.float32, (tokens * TOPK, H))
    meta = s.peek("meta", np.uint32, (8,))
    assert meta[0] == 0 and meta[4] == 256
    perm = np.random.default_rng(1).permutation(tokens)
    bf_p, partial_p = run_dev(layer, s, dev, x_bits[perm], ids[perm], w[perm])
    assert np.array_equal(bf_p, bf[perm]) and np.array_equal(partial_p.view(np.uint32), partial[perm].view(np.uint32))
    half = tokens // 2
    bf_a, _ = run_dev(layer, s, dev, x_bits[:half], ids[:half], w[:half])
    bf_b, _ = run_dev(layer, s, dev, x_bits[half:], ids[half:], w[half:])
    assert np.array_equal(np.concatenate([bf_a, bf_b]), bf)
    _, partial2 = run_dev(layer, s, dev, x_bits, ids, (w * np.float32(2)).astype(np.float32))
    assert np.array_equal(partial2.view(np.uint32), (partial * np.float32(2)).view(np.uint32))
    # sampled oracle, stage by stage, over 18 experts (every 16th, the busiest and the least busy): for each, the first and
    # last routed row, the rows either side of every token-tile boundary (tiles of this expert are `width` rows: the
    # last row of one CTA-pair tile and the first of the next; the two CTAs of a pair hold the two halves of a tile's
    # rows and every row spans the weight rows of both), the tail tile's last row, and a few rows in between
    s.set_debug(1)
    bf_d, partial_d = run_dev(layer, s, dev, x_bits, ids, w)
    assert np.array_equal(bf_d, bf) and np.array_equal(partial_d.view(np.uint32), partial.view(np.uint32))   # the dump build computes the same bytes
    routes = tokens * TOPK
    inv = s.peek("inverse", np.int32, (routes,))
    h_all = s.peek("mid_f32", np.float32, (routes, I))
    mq_all = s.peek("mid_payload", np.uint8, (routes, I))
    y = s.peek("y", np.float32, (routes, H))
    st, oinv, oorig, _, counts = oracle_mod.plan(ids, w)
    assert st == 0 and np.array_equal(inv, oinv)
    x = synth.bf16_to_f32_np(x_bits)
    flat = ids.reshape(-1)
    chosen = sorted(set(list(range(3, 256, 16)) + [int(np.argmax(counts)), int(np.argmin(counts))]))
    assert len(chosen) >= 16
    rng = np.random.default_rng(8)
    crossings = checked = 0
    table = oracle_mod.e4m3_table()
    for e in chosen:
        r_e = np.nonzero(flat == e)[0]                      # this expert's routes in request order = grouped order (stable)
        c = r_e.size
        n_tiles = -(-c // 128)
        width = (-(-c // n_tiles) + 15) // 16 * 16
        pick = {0, c - 1}
        for t in range(1, n_tiles):
            pick.update({t * width - 1, t * width})
        pick.update({width // 2 - 1, width // 2})            # the two CTAs' halves of the first tile meet here
        pick.update(int(v) for v in rng.integers(0, c, 4))
        pick = np.array(sorted(v for v in pick if 0 <= v < c))
        rr = r_e[pick]
        assert np.array_equal(inv[rr], inv[r_e[0]] + pick)   # grouped rows of the expert are contiguous and in order
        xq, xs = oracle_mod.quant_wire(x[rr // TOPK])
        t6 = [synth.expert_tensor_np(SEED, n, e) for n in synth.TENSORS]
        ref = oracle_mod.expert_ffn(xq, xs, *t6)
        assert ref["rc"] == 0
        g = inv[rr]
        assert (np.abs(h_all[g] - ref["h"]) <= 1e-5 + 1e-5 * np.abs(ref["h"])).all(), e
        p_own, s_own, f_own = oracle_mod.quant_v1(h_all[g])
        assert not f_own.any() and np.array_equal(mq_all[g], p_own), e
        crossed = (mq_all[g] != ref["mid_q"]).any(axis=1)
        crossings += int((mq_all[g] != ref["mid_q"]).sum())
        mid = np.abs(table[ref["mid_q"]].astype(np.float64) * np.exp2(np.repeat(ref["mid_s"].astype(np.int32) - 127, 32, axis=1)))
        wd = np.abs(oracle_mod.mxfp4_unpack(t6[4], t6[5])).astype(np.float64)
        bound = 1e-5 + 1e-5 * np.abs(ref["y"]) + 2.0 * (I // 32) * 2.0 ** -24 * (mid @ wd.T)
        ok_rows = ~crossed
        assert (np.abs(y[rr][ok_rows] - ref["y"][ok_rows]) <= bound[ok_rows]).all(), e
        assert rel_l2(y[rr], ref["y"]) <= 1e-3
        checked += pick.size
    assert checked >= 16 * 8 and crossings <= max(4, checked * I // 50000), (checked, crossings)


def test_config4_65536_tokens_zipf_through_the_host_entry_point(layer, dev, oracle_mod):
    """The long-prefill batch (65,536 tokens, Zipf 1.0: one expert receives about 62,000 rows) on one GPU through
    m26b_ffn, which cuts it into passes of 16,384 tokens. Properties: the bytes do not depend on the cut (four
    quarter-size calls and a shifted cut give the same rows), and sampled tokens match the oracle end to end."""
    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import synth

    tokens = 65536
    s = M.Scratch()
    ids, w = synth.routing(SEED + 4, tokens, 1.0)
    counts = np.bincount(ids.reshape(-1), minlength=256)
    assert counts.max() > 40000 and (counts > 0).all()
    # sampled tokens: both sides of every pass boundary (passes of 16,384 tokens), both sides of the other cut below, the
    # ends, and a seeded scatter; 40 tokens, 320 routes
    sample = np.unique(np.concatenate([[0, 1, 9999, 10000, 16383, 16384, 32767, 32768, 40000, 49151, 49152, 65534, 65535],
                                       np.random.default_rng(5).integers(0, tokens, 27)]))
    # quantised rows: seeded bytes directly (valid E4M3 codes, scale bytes 118..125), the host entry point's own input form
    rng = np.random.default_rng(99)
    xq = rng.integers(0, 256, (tokens, H), dtype=np.uint8)
    xq[(xq & 0x7F) == 0x7F] ^= 1
    xs = rng.integers(118, 126, (tokens, H // 32), dtype=np.uint8)
    bf = np.empty((tokens, H), np.uint16)
    st = M.ffn(layer, s, xq.reshape(-1), xs.reshape(-1), ids.reshape(-1), w.reshape(-1), tokens, bf.reshape(-1))
    assert st.groups > 0
    # another cut: 10,000 tokens first, then the rest (passes start at other tokens)
    cut = 10000
    bf_a = np.empty((cut, H), np.uint16)
    bf_b = np.empty((tokens - cut, H), np.uint16)
    M.ffn(layer, s, xq[:cut].reshape(-1), xs[:cut].reshape(-1), ids[:cut].reshape(-1), w[:cut].reshape(-1), cut, bf_a.reshape(-1))
    M.ffn(layer, s, xq[cut:].reshape(-1), xs[cut:].reshape(-1), ids[cut:].reshape(-1), w[cut:].reshape(-1), tokens - cut, bf_b.reshape(-1))
    assert np.array_equal(bf[:cut], bf_a) and np.array_equal(bf[cut:], bf_b)
    # sampled tokens against the oracle (their experts' weights only)
    tensors = synth.layer_np(SEED, np.unique(ids[sample]))
    ref = oracle_mod.ffn_layer(tensors, xq[sample], xs[sample], ids[sample], w[sample])
    assert ref["rc"] == 0
    dec = lambda b: (b.astype(np.uint32) << 16).view(np.float32)
    got = dec(bf[sample])
    assert rel_l2(got, ref["partial"]) <= 1e-3 + 2.0 ** -8          # BF16 output against the FP32 plane: half a BF16 ulp on top
    # elementwise: one BF16 ulp, except where an E4M3 bin crossing of the intermediate moved an output (counted, rare)
    # (these seeded bytes give outputs of magnitude ~1000, so the absolute part of the bound scales with the row)
    rms = np.sqrt((ref["partial"].astype(np.float64) ** 2).mean(axis=1, keepdims=True))
    beyond = np.abs(got - dec(ref["bf16"])) > 2.0 ** -7 * np.abs(ref["partial"]) + 1e-3 * rms
    assert beyond.mean() < 2e-3, beyond.mean()


# ------------------------------------------------------------------------------------------ BF16 route outputs (opt-in)
@pytest.mark.parametrize("tokens,zipf", [(16, 0.0), (300, 1.0)])
def test_bf16_route_outputs_follow_the_reference_variant(layer, dev, oracle_mod, tokens, zipf):
    """The route-output option (the reference's MIMO26_B1_Y=bf16, crates/mimo26-spark/kernels/b1_serve.cu:98-143): FC2's rows
    are the FP32 rows rounded to BF16 (nearest even), bit for bit, and the combine is the same ordered multiply / add on
    the widened values. Both the single-CTA and the CTA-pair kernels. Not bit-identical to the FP32 mode; the deviation
    is printed and stays within the end-to-end bar."""
    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import synth

    x_bits = synth.activations_bf16(SEED + 60, tokens)
    ids, w = synth.routing(SEED + 60, tokens, zipf)
    s = M.Scratch()
    bf32, part32 = run_dev(layer, s, dev, x_bits, ids, w)
    y32 = s.peek("y", np.float32, (tokens * TOPK, H))
    s.set_route_output(True)
    bf16, part16 = run_dev(layer, s, dev, x_bits, ids, w)
    y16 = s.peek("y", np.uint16, (tokens * TOPK, H))
    assert np.array_equal(y16, synth.bf16_rne_np(y32))
    rc, p_want, b_want = oracle_mod.route_reduce(synth.bf16_to_f32_np(y16), w)
    assert rc == 0 and np.array_equal(part16.view(np.uint32), p_want.view(np.uint32)) and np.array_equal(bf16, b_want)
    dev_l2 = rel_l2(part16, part32)
    print("bf16 route outputs: rel L2 against the FP32 mode", dev_l2, "BF16 rows that differ", int((bf16 != bf32).any(axis=1).sum()))
    assert dev_l2 <= 1e-3 + 2.0 ** -8
    s.set_route_output(False)
    bf_again, _ = run_dev(layer, s, dev, x_bits, ids, w)
    assert np.array_equal(bf_again, bf32)


# ------------------------------------------------------------------------------------------ tensor-parallel host entry point
def test_ffn_tp_host_entry_point_one_rank_and_two_windows(weights, dev, oracle_mod):
    """m26b_ffn_tp / m26b_ffn_tp_dev through ctypes on one GPU. World 1: the sum of one plane equals the BF16 output
    widened (+ residual). World 2 with both windows in this process, no kernel ever waiting for another kernel: up to 512
    tokens (combine and exchange fused) rank 0's chunk flags are marked from the host, rank 1's call pushes its plane and
    flags into rank 0's window, and rank 0's call then finds them; above 512 tokens rank 1's plane is written first and
    its publication marked from the host. Rank 0's sum equals the oracle's rank-ordered sum of the two planes bit for
    bit, and the oracle's wire result within the end-to-end bar."""
    import torch

    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import expert, synth

    for tokens in (16, 200, 600):
        fused = tokens <= 512
        x_bits = synth.activations_bf16(SEED + 70, tokens)
        ids, w = synth.routing(SEED + 70, tokens, 0.0)
        xq, xs = oracle_mod.quant_wire(synth.bf16_to_f32_np(x_bits))
        xqd, xsd = to_dev(xq, dev), to_dev(xs, dev)
        idd, wd = to_dev(ids, dev), to_dev(w, dev)
        # world 1
        L = M.Layer.from_checkpoint(*[weights[n] for n in synth.TENSORS])
        s = M.Scratch()
        ex = M.Exchange(tokens * H * 2, 0, 1, export=False)
        total = np.empty((tokens, H), np.float32)
        st = M.ffn_tp(L, s, ex, xq, xs, ids, w, tokens, total)
        assert st.gpu_ms > 0 and st.groups > 0
        bf = np.empty((tokens, H), np.uint16)
        M.ffn(L, s, xq.reshape(-1), xs.reshape(-1), ids.reshape(-1), w.reshape(-1), tokens, bf.reshape(-1))
        assert np.array_equal(total.view(np.uint32), synth.bf16_to_f32_np(bf).view(np.uint32))
        M.ffn_tp(L, s, ex, xq, xs, ids, w, tokens, None)       # a rank that does not download
        # the device form, from BF16 activations, with the residual folded in
        res = torch.randn(tokens, H, device=dev)
        got = torch.empty(tokens, H, device=dev)
        expert.ffn_tp_dev(L, s, ex, to_dev(x_bits.view(np.int16), dev), idd, wd, tokens, got, residual=res)
        s.status(); ex.status()
        want = res.cpu().numpy() + synth.bf16_to_f32_np(bf)
        assert np.array_equal(got.cpu().numpy().view(np.uint32), want.astype(np.float32).view(np.uint32))
        ex.close(); L.close()
        # world 2, both windows here
        layers = [M.Layer.from_checkpoint(*[weights[n] for n in synth.TENSORS], tp_rank=r, tp_size=2) for r in range(2)]
        exs = [M.Exchange(tokens * H * 2, r, 2, export=False) for r in range(2)]
        for e in exs:
            e.connect_local(exs)
        s1 = M.Scratch()
        plane1_d = torch.empty(tokens * H, dtype=torch.int16, device=dev)
        expert.ffn_dev(layers[1], s1, xqd, idd, wd, tokens, plane1_d, x_dtype=expert.X_E4M3, x_scales=xsd)
        s1.status()
        plane1 = plane1_d.cpu().numpy().view(np.uint16).reshape(tokens, H)
        bf0 = np.empty((tokens, H), np.uint16)
        M.ffn(layers[0], s, xq.reshape(-1), xs.reshape(-1), ids.reshape(-1), w.reshape(-1), tokens, bf0.reshape(-1))
        want = oracle_mod.rank_sum(np.stack([bf0, plane1]))
        sum1 = torch.empty(tokens * H, dtype=torch.float32, device=dev)
        for step in range(3):                                   # both slots and a reuse
            if fused:
                exs[1].publish_as(0)
                expert.ffn_tp_dev(layers[1], s1, exs[1], xqd, idd, wd, tokens, sum1, x_dtype=expert.X_E4M3, x_scales=xsd)
                s1.status(); exs[1].status()
                torch.cuda.synchronize()
                M.ffn_tp(layers[0], s, exs[0], xq, xs, ids, w, tokens, total)
            else:
                expert.ffn_dev(layers[1], s1, xqd, idd, wd, tokens, exs[1].plane(), x_dtype=expert.X_E4M3, x_scales=xsd)
                s1.status()
                exs[0].publish_as(1)
                torch.cuda.synchronize()
                M.ffn_tp(layers[0], s, exs[0], xq, xs, ids, w, tokens, total)
                exs[1].publish_as(0)                            # rank 1 takes the same step (its sum is not read here)
                exs[1].sum(tokens * H, sum1)
                exs[1].status()
            assert np.array_equal(total.view(np.uint32), want.view(np.uint32)), (tokens, step)
        if fused:
            # rank 1 once more, now that rank 0's chunks of the last step are in its window: the same sum on both ranks
            # (the two slots alternate, so a step of rank 1 alone re-reads rank 0's chunks of two steps back: same data)
            exs[1].publish_as(0)
            expert.ffn_tp_dev(layers[1], s1, exs[1], xqd, idd, wd, tokens, sum1, x_dtype=expert.X_E4M3, x_scales=xsd)
            s1.status(); exs[1].status()
            assert np.array_equal(sum1.cpu().numpy().view(np.uint32).reshape(tokens, H), want.view(np.uint32))
        if fused and tokens == 16:
            # a peer that never delivers: rank 0's bounded wait runs out, the call's status names the late rank (code 5),
            # nothing hangs or faults and the handles stay usable
            exs[0].set_wait_ms(20)
            expert.ffn_tp_dev(layers[0], s, exs[0], xqd, idd, wd, tokens, sum1, x_dtype=expert.X_E4M3, x_scales=xsd)
            s.status(); exs[0].status()                         # rank 1 has already pushed this step (its extra one above)
            assert np.array_equal(sum1.cpu().numpy().view(np.uint32).reshape(tokens, H), want.view(np.uint32))
            expert.ffn_tp_dev(layers[0], s, exs[0], xqd, idd, wd, tokens, sum1, x_dtype=expert.X_E4M3, x_scales=xsd)
            s.status()
            with pytest.raises(M.ExpertError) as e:
                exs[0].status()
            assert e.value.code == 5 and "0x2" in str(e.value)
            exs[0].status()                                     # the error word was cleared
            bf_again = np.empty((tokens, H), np.uint16)
            M.ffn(layers[0], s, xq.reshape(-1), xs.reshape(-1), ids.reshape(-1), w.reshape(-1), tokens, bf_again.reshape(-1))
            assert np.array_equal(bf_again, bf0)
        if tokens <= 200:
            ref = [oracle_mod.ffn_layer(synth.layer_np(SEED, np.unique(ids)), xq, xs, ids, w, tp_rank=r, tp_size=2) for r in range(2)]
            wire = oracle_mod.rank_sum(np.stack([r["bf16"] for r in ref]))
            assert rel_l2(total, wire) <= 1e-3
        # a layer of another rank, or a request larger than the plane, is refused before anything runs
        with pytest.raises(M.ExpertError) as e:
            M.ffn_tp(layers[1], s, exs[0], xq, xs, ids, w, tokens, total)
        assert e.value.code == 1
        with pytest.raises(M.ExpertError) as e:
            expert.ffn_tp_dev(layers[1], s, exs[0], xqd, idd, wd, tokens, sum1, x_dtype=expert.X_E4M3, x_scales=xsd)
        assert e.value.code == 1
        for e_ in exs:
            e_.close()
        for l_ in layers:
            l_.close()
