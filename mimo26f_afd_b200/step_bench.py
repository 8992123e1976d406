"""Replay step-histogram workloads through the expert FFN on one GPU and report the bandwidth verdict the reference
reports for them: distinct expert weight bytes of a step / the step's time (``harness/route_hist.py``,
``crates/mimo26-expert/tests/gpu/step_hist.h``; timing discipline of ``tests/b1_core/bench_connected.cuh:21-88``: warm-up
passes, 31 CUDA-event samples per step, the median, the L2 flushed before every sample).

    python -m mimo26f_afd_b200.step_bench --name C16-w8 [--file steps.json] [--steps 32]

Without ``--file`` the histograms come from seeded Zipf(1.2) routing at the workload's token count (the traced
workloads of the reference are not available here). Prints one JSON line.
"""
import argparse
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch

    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import expert, step_hist, synth

    ap = argparse.ArgumentParser()
    ap.add_argument("--name", default="C16-w8", choices=sorted(step_hist.WORKLOAD_TOKENS))
    ap.add_argument("--file", default=None)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--samples", type=int, default=31)
    args = ap.parse_args()
    if args.file:
        w = step_hist.load(args.file, args.name)
    else:
        w = step_hist.parse(step_hist.synthetic_workload(args.name, args.steps), args.name)
    steps = w["steps"][:args.steps]
    dev = torch.device("cuda:0")
    seed = synth.MASTER_SEED
    wts = synth.layer_torch(seed, dev)
    layer = M.Layer.from_checkpoint(*[wts[n] for n in synth.TENSORS])
    del wts
    scratch = M.Scratch()
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    tokens = step_hist.WORKLOAD_TOKENS[args.name]
    xd = torch.from_numpy(synth.activations_bf16(seed, tokens).view(np.int16)).to(dev)
    out = torch.empty((tokens, 4096), dtype=torch.int16, device=dev)
    per_step = []
    for i, step in enumerate(steps):
        ids, wt = step_hist.step_batch(step, step_hist.sample_seed(w["seed"], i, 0))
        idd, wd = torch.from_numpy(ids).to(dev), torch.from_numpy(wt).to(dev)
        for _ in range(3):
            expert.ffn_dev(layer, scratch, xd, idd, wd, tokens, out, stream=stream.cuda_stream)
        scratch.status(stream.cuda_stream)
        times = []
        for _ in range(args.samples):
            flush.fill_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            expert.ffn_dev(layer, scratch, xd, idd, wd, tokens, out, stream=stream.cuda_stream)
            b.record(stream)
            b.synchronize()
            times.append(a.elapsed_time(b))
        scratch.status(stream.cuda_stream)
        ms = float(np.median(times))
        per_step.append(dict(layer=step["layer"], experts=step["experts"], max_m=max(step["hist"]), us=ms * 1e3,
                             distinct_gbs=step["experts"] * 13369344 / (ms * 1e-3) / 1e9))
    us = np.array([s["us"] for s in per_step])
    gbs = np.array([s["distinct_gbs"] for s in per_step])
    print(json.dumps(dict(workload=args.name, tokens=tokens, steps=len(per_step), samples_per_step=args.samples,
                          source=args.file or "synthetic Zipf(1.2) histograms", us_per_step_median=float(np.median(us)),
                          us_per_step_max=float(us.max()), distinct_weight_gbs_median=float(np.median(gbs)),
                          distinct_weight_gbs_min=float(gbs.min()), tokens_per_s=float(tokens / (np.mean(us) * 1e-6)),
                          experts_per_step_mean=float(np.mean([s["experts"] for s in per_step])),
                          gpu=torch.cuda.get_device_name(0), version=M.version())), flush=True)


if __name__ == "__main__":
    main()
