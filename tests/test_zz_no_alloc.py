"""m26b_plan_static: the route planner for callers that cannot allocate device memory (everything already given to
resident weights, or no room for cudaMalloc's device-wide synchronisation on the serving path). Its scratch is a
fixed array inside the library, so this test checks what such a caller relies on: two calls in a row, the second
smaller than the first so stale scratch would show, each bit-identical to the plan the allocating entry point
(m26b_ffn_dev, read back with m26b_scratch_peek) computes for the same routes; and an over-size request is refused
with a message instead of overrunning the array. Collected last on purpose."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_plan_static_matches_allocating_planner_twice_in_a_row():
    import torch

    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import expert, synth

    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    seed = 0x26AFD
    weights = synth.layer_torch(seed, dev)
    layer = M.Layer.from_checkpoint(*[weights[n] for n in synth.TENSORS])
    del weights
    scratch = M.Scratch()
    for tokens, zipf in ((700, 1.2), (16, 0.0)):
        ids, w = synth.routing(seed + tokens, tokens, zipf)
        routes = tokens * 8
        idd, wd = torch.from_numpy(ids).to(dev), torch.from_numpy(w).to(dev)
        # reference result: the planner inside the allocating entry point
        x = torch.from_numpy(synth.activations_bf16(seed, tokens).view(np.int16)).to(dev)
        out = torch.empty((tokens, 4096), dtype=torch.int16, device=dev)
        expert.ffn_dev(layer, scratch, x, idd, wd, tokens, out)
        scratch.status()
        want_inv = scratch.peek("inverse", np.int32, (routes,))
        want_orig = scratch.peek("original_routes", np.int32, (routes,))
        want_gw = scratch.peek("grouped_weights", np.float32, (routes,))
        want_meta = scratch.peek("meta", np.uint32, (8,))
        # the allocation-free entry point, outputs pre-filled so an unwritten element shows
        inv = torch.full((routes,), -7, dtype=torch.int32, device=dev)
        orig = torch.full((routes,), -7, dtype=torch.int32, device=dev)
        gw = torch.full((routes,), -7.0, dtype=torch.float32, device=dev)
        meta = torch.full((8,), 77, dtype=torch.int32, device=dev)
        M.plan_static(idd, wd, tokens, inv, orig, gw, meta)
        torch.cuda.synchronize()
        assert np.array_equal(inv.cpu().numpy(), want_inv)
        assert np.array_equal(orig.cpu().numpy(), want_orig)
        assert np.array_equal(gw.cpu().numpy().view(np.uint32), want_gw.view(np.uint32))
        got_meta = meta.cpu().numpy().view(np.uint32)
        assert got_meta[0] == 0 and got_meta[4] == want_meta[4] and got_meta[5] == want_meta[5]
        assert np.array_equal(orig.cpu().numpy(), np.argsort(ids.reshape(-1), kind="stable"))
    # a rejected plan reports it and leaves the handles usable
    bad = ids.copy(); bad[3, 5] = bad[3, 0]
    M.plan_static(torch.from_numpy(bad).to(dev), wd, 16, inv, orig, gw, meta)
    torch.cuda.synchronize()
    assert meta.cpu().numpy().view(np.uint32)[0] == 1
    with pytest.raises(M.ExpertError) as e:
        M.plan_static(idd, wd, expert.PLAN_STATIC_MAX_ROWS + 1, inv, orig, gw, meta)
    assert e.value.code == 1 and "exceed the built-in scratch" in e.value.message
