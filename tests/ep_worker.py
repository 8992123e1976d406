"""One rank of the multi-GPU expert-parallel check (launched by test_tp_multi_gpu.py through torch.distributed.run).

Every rank holds its block of the experts and its block of the tokens, runs the expert-parallel step, and compares its
output rows with the single-GPU layer run on the same rank over the whole batch: they must be identical bit for bit."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch
    import torch.distributed as dist

    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import expert, synth, tp

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    seed, H = synth.MASTER_SEED, 4096
    w = synth.layer_torch(seed, dev)
    full = M.Layer.from_checkpoint(*[w[n] for n in synth.TENSORS])
    del w
    n_local = 256 // world
    w = synth.layer_torch(seed, dev, n_experts=n_local, first_expert=rank * n_local)
    mine = M.Layer.from_checkpoint_ep(*[w[n] for n in synth.TENSORS], ep_rank=rank, ep_size=world)
    del w
    scratch, scratch_full = M.Scratch(), M.Scratch()
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    plain = mine
    for tokens, zipf, n_rep in ((16, 0.0, 0), (1000, 1.0, 0), (20000, 0.0, 0), (3000, 1.0, 16)):
        if n_rep:
            # copies of the batch's busiest experts on every rank: their routes are served where the tokens live
            all_ids, _ = synth.routing(seed, tokens, zipf)
            hot = np.argsort(-np.bincount(all_ids.reshape(-1), minlength=256), kind="stable")[:n_rep].astype(np.int32)
            w = synth.layer_torch(seed, dev, n_experts=n_local, first_expert=rank * n_local)
            reps = synth.layer_torch(seed, dev, experts=hot)
            mine = M.Layer.from_checkpoint_ep(*[w[n] for n in synth.TENSORS], ep_rank=rank, ep_size=world,
                                              replicas=[reps[n] for n in synth.TENSORS], replica_ids=hot)
            del w, reps
        else:
            mine = plain
        ep = tp.make_expert_parallel(tokens)
        lo, hi = tp.shard_tokens(tokens, rank, world)
        x_bits = synth.activations_bf16(seed, tokens)
        ids, wts = synth.routing(seed, tokens, zipf)
        xd = torch.from_numpy(x_bits.view(np.int16)).to(dev)
        idd, wd = torch.from_numpy(ids).to(dev), torch.from_numpy(wts).to(dev)
        ref = torch.empty((tokens, H), dtype=torch.int16, device=dev)
        ref_part = torch.empty((tokens, H), dtype=torch.float32, device=dev)
        if tokens <= 16384:
            expert.ffn_dev(full, scratch_full, xd, idd, wd, tokens, ref, partial_out=ref_part, stream=stream.cuda_stream)
            scratch_full.status(stream.cuda_stream)
        else:   # larger than one pass of the device entry point: two halves (row-local math)
            h = tokens // 2
            for a, b in ((0, h), (h, tokens)):
                expert.ffn_dev(full, scratch_full, xd[a:b], idd[a:b], wd[a:b], b - a, ref[a:b], partial_out=ref_part[a:b],
                               stream=stream.cuda_stream)
                scratch_full.status(stream.cuda_stream)
        out = torch.empty((hi - lo, H), dtype=torch.int16, device=dev)
        part = torch.empty((hi - lo, H), dtype=torch.float32, device=dev)
        for step in range(2):
            ep.step(mine, scratch, xd[lo:hi], idd[lo:hi], wd[lo:hi], hi - lo, out, partial_out=part, stream=stream.cuda_stream)
            scratch.status(stream.cuda_stream)
            ep.status(stream.cuda_stream)
            torch.cuda.synchronize()
            assert torch.equal(out, ref[lo:hi]), (tokens, step, rank)
            assert torch.equal(part.view(torch.int32), ref_part[lo:hi].view(torch.int32)), (tokens, step, rank)
        dist.barrier()
        ep.close()
    if rank == 0:
        print("EP_WORKER_OK", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
