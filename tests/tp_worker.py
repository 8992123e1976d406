"""One rank of the multi-GPU tensor-parallel check (launched by test_tp_multi_gpu.py through torch.distributed.run).

Every rank builds its slice of the synthetic layer, runs the same batch, and the ranks' BF16 planes are summed three ways:
by the NVLink peer-memory exchange kernel (pull), by the combine kernel that pushes its chunks into the peers' windows and
adds what the peers pushed (one kernel), and by an NCCL all-gather followed by the rank-sum kernel. The three must agree
bit for bit, on every rank, and match the CPU oracle of the whole layer within the end-to-end tolerance."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch
    import torch.distributed as dist

    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import expert, synth, tp
    import oracle

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    seed, H = synth.MASTER_SEED, 4096
    w = synth.layer_torch(seed, dev)
    layer = M.Layer.from_checkpoint(*[w[n] for n in synth.TENSORS], tp_rank=rank, tp_size=world)
    del w
    scratch = M.Scratch()
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    for tokens in (16, 300):
        ex = tp.make_exchange(tokens)
        x_bits = synth.activations_bf16(seed, tokens)
        ids, wts = synth.routing(seed, tokens, 0.0)
        xd = torch.from_numpy(x_bits.view(np.int16)).to(dev)
        idd, wd = torch.from_numpy(ids).to(dev), torch.from_numpy(wts).to(dev)
        peer_sum = torch.empty((tokens, H), dtype=torch.float32, device=dev)
        nccl_sum = torch.empty((tokens, H), dtype=torch.float32, device=dev)
        plane = torch.empty((tokens, H), dtype=torch.int16, device=dev)
        for step in range(3):                                   # three steps: both slots and a reuse
            expert.ffn_dev(layer, scratch, xd, idd, wd, tokens, ex.plane(), stream=stream.cuda_stream)
            ex.sum(tokens * H, peer_sum, stream=stream.cuda_stream)
            scratch.status(stream.cuda_stream)
            ex.status(stream.cuda_stream)
            expert.ffn_dev(layer, scratch, xd, idd, wd, tokens, plane, stream=stream.cuda_stream)
            scratch.status(stream.cuda_stream)
            tp.tp_combine(plane, nccl_sum, stream=stream.cuda_stream)
            torch.cuda.synchronize()
            assert torch.equal(peer_sum.view(torch.int32), nccl_sum.view(torch.int32)), (tokens, step, rank)
        res = torch.randn((tokens, H), device=dev)
        for step in range(3):                                   # combine and exchange in one kernel, residual folded in
            peer_sum.zero_()
            expert.ffn_tp_dev(layer, scratch, ex, xd, idd, wd, tokens, peer_sum, residual=res if step == 2 else None,
                              stream=stream.cuda_stream)
            scratch.status(stream.cuda_stream)
            ex.status(stream.cuda_stream)
            torch.cuda.synchronize()
            want = nccl_sum + res if step == 2 else nccl_sum
            assert torch.equal(peer_sum.view(torch.int32), want.view(torch.int32)), ("fused", tokens, step, rank)
        expert.ffn_dev(layer, scratch, xd, idd, wd, tokens, ex.plane(), stream=stream.cuda_stream)   # and the pull form again
        ex.sum(tokens * H, peer_sum, stream=stream.cuda_stream)
        ex.status(stream.cuda_stream)
        torch.cuda.synchronize()
        assert torch.equal(peer_sum.view(torch.int32), nccl_sum.view(torch.int32)), ("pull after fused", tokens, rank)
        if tokens == 16:
            x = synth.bf16_to_f32_np(x_bits)
            xq, xs = oracle.quant_wire(x)
            ref = oracle.ffn_layer(synth.layer_np(seed, np.unique(ids)), xq, xs, ids, wts, stages=True)
            got = peer_sum.cpu().numpy()
            rel = np.linalg.norm(got - ref["partial"]) / np.linalg.norm(ref["partial"])
            # each rank rounds its partial plane to BF16 before the sum: 2^-9 relative per plane on top of the FP32 bar
            assert rel <= 1e-3 + world * 2.0 ** -9, rel
        dist.barrier()
        ex.close()
    if rank == 0:
        print("TP_WORKER_OK", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
