"""world_size-2 run of the multi-rank exchange on CPU (gloo): each rank computes its tensor-parallel partial
with the oracle, the planes cross with the package's all-gather, and the rank-ordered FP32 sum (done by the
oracle here; by the library's kernel on GPUs) must equal the single-process reference on every rank."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from mimo26f_afd_b200 import synth, tp

    seed, tokens = 0x26AFD, 2
    ids = np.array([[3, 9, 3 + 8, 40, 41, 42, 43, 44], [9, 3, 50, 51, 52, 53, 54, 55]], np.int32)
    w = np.full((2, 8), 0.125, np.float32)
    experts = np.unique(ids)[:2]          # keep the CPU work small: only experts 3 and 9 carry weight
    w[~np.isin(ids, experts)] = 0.0
    x = synth.bf16_to_f32_np(synth.activations_bf16(seed, tokens))
    xq, xs = oracle.quant_wire(x)
    tensors = synth.layer_np(seed, np.unique(ids))
    i0, il = tp.tp_slice(rank, world)
    assert (i0, il) == (rank * 2048 // world, 2048 // world)
    mine = oracle.ffn_layer(tensors, xq, xs, ids, w, tp_rank=rank, tp_size=world)
    assert mine["rc"] == 0
    plane = torch.from_numpy(mine["bf16"].view(np.int16).copy())
    planes = tp.all_gather_planes(plane)
    got = oracle.rank_sum(np.stack([p.numpy().view(np.uint16) for p in planes]))
    # every rank holds every plane, in rank order
    want_planes = [oracle.ffn_layer(tensors, xq, xs, ids, w, tp_rank=r, tp_size=world)["bf16"] for r in range(world)]
    want = oracle.rank_sum(np.stack(want_planes))
    ok = all(np.array_equal(p.numpy().view(np.uint16), wp) for p, wp in zip(planes, want_planes))
    full = oracle.ffn_layer(tensors, xq, xs, ids, w)["partial"]
    rel = float(np.linalg.norm(got - full) / np.linalg.norm(full))
    lo, hi = tp.shard_tokens(10, rank, world)
    q.put((rank, ok and np.array_equal(got.view(np.uint32), want.view(np.uint32)), rel, (lo, hi)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_tp2_exchange_and_rank_ordered_sum():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0, "a rank failed or never finished"
    res = sorted(q.get(timeout=10) for _ in range(2))
    assert [r[1] for r in res] == [True, True]
    # per-rank BF16 rounding before the sum costs about 1e-3 relative L2 against the unrounded full-width result
    assert all(r[2] < 5e-3 for r in res)
    assert [r[3] for r in res] == [(0, 5), (5, 10)]


def test_tp_slice_rejects_bad_geometry():
    from mimo26f_afd_b200 import tp

    with pytest.raises(ValueError):
        tp.tp_slice(0, 3)
    with pytest.raises(ValueError):
        tp.tp_slice(4, 4)
    assert tp.tp_slice(3, 4) == (1536, 512)
    assert tp.shard_tokens(7, 2, 4) == (4, 6)


def test_serving_rank_with_replicated_experts():
    """Host form of the planner's rule for expert parallelism: routes to replicated experts stay with the token's owner,
    the others go to the expert's home rank; every route is served by exactly one rank, and replicating the busiest
    experts of a skewed batch evens the load out."""
    from mimo26f_afd_b200 import synth, tp

    ids, _ = synth.routing(0x26AFD, 4096, 1.0)
    for world in (2, 4, 8):
        home = tp.serving_rank(ids, world)
        assert np.array_equal(home, ids // (256 // world))
        hot = tp.busiest_experts(ids, 32)
        assert len(set(hot.tolist())) == 32
        counts = np.bincount(ids.reshape(-1), minlength=256)
        assert counts[hot].min() >= np.delete(counts, hot).max()
        serve = tp.serving_rank(ids, world, hot)
        lo_hi = [tp.shard_tokens(4096, r, world) for r in range(world)]
        for r, (lo, hi) in enumerate(lo_hi):
            mine = serve == r
            rep = np.isin(ids, hot)
            own_tok = np.zeros(4096, bool); own_tok[lo:hi] = True
            assert np.array_equal(mine, (rep & own_tok[:, None]) | (~rep & (ids // (256 // world) == r)))
        load0 = np.bincount(home.reshape(-1), minlength=world)
        load1 = np.bincount(serve.reshape(-1), minlength=world)
        assert load1.sum() == ids.size and load1.max() / load1.mean() < load0.max() / load0.mean()
        assert load1.max() / load1.mean() < 1.15
