#!/usr/bin/env python
"""Benchmark of the routed-expert FFN hot path (one MoE layer) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one pass of the hot path over one batch of seeded synthetic input: activation quantisation, route plan,
token permutation, grouped gate/up GEMM + SwiGLU + intermediate quantiser, grouped down GEMM, ordered top-8
combine. The headline workload (`value`) is BASELINE.json configs[1], the 16-token decode batch; the same JSON
line carries the 8,192-token prefill segment (configs[3]) under "prefill". Weights are resident in HBM, inputs are
resident in HBM for `value`, and on the host (pinned) for `e2e`, which goes through the reference-compatible
host entry point m26b_ffn with both copies inside the timed region.

The timed region is `steps` plain steps (one CUDA-event pair around each, nothing inside, so consecutive kernels
overlap their launch and set-up as they do in service). The same steps then run once more with an event between
every two kernels; those per-kernel durations feed `roofline` and `kernels_ms`, and that slower step time is
reported beside the plain one as `ms_per_step_with_kernel_events`.

With N > 1 ranks the layer is tensor-parallel over the intermediate dimension (the reference's own TP4 scheme,
generalised): every rank runs the whole batch on its 1/N slice of every expert and the BF16 partial planes are
exchanged with one NCCL all-gather and summed in rank order on every rank. Total work is fixed: "strong" scaling.

--impl reference times the reference's CPU expert path (the port in oracle/oracle.c of
crates/mimo26-spark/src/main.rs:75-95) on the host cores, on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H, I, E, TOPK = 4096, 2048, 256, 8
EXPERT_BYTES = 13369344                     # 3 x 2048 x 4096 x 17/32 (payload + scales)
FLOP_PER_TOKEN = 402653184                  # 3 GEMMs x 2 x 4096 x 2048 x top-8
MXF8F6F4_PEAK_TFLOPS = 4450.0               # measured on this pool: profiles/mxf8f6f4_mma_rate.md (burst, small codes)
MXF8F6F4_RANDOM_BURST_TFLOPS = 3694.0       # same probe on random operands, first 7 ms launch
MXF8F6F4_RANDOM_SUSTAINED_TFLOPS = 3193.0   # same, after three seconds (1.32 GHz under the 1000 W limit)
# dram__bytes_read.sum + dram__bytes_write.sum of one FC1 launch at N = 1, from the ncu captures summarised in
# profiles/gemm_mx_decode16.md and profiles/gemm_mx_prefill8k.md (the seeded workloads are the same every run)
FC1_TRAFFIC_BYTES = {"decode16": 915809536, "prefill8k": 2774330624}
WORKLOADS = {
    "decode16": dict(tokens=16, zipf=0.0, desc="16-token decode batch, uniform routing (BASELINE configs[1])"),
    "prefill8k": dict(tokens=8192, zipf=0.0, desc="8192-token prefill segment, uniform routing (BASELINE configs[3])"),
    "prefill64k": dict(tokens=65536, zipf=1.0, desc="65536-token batch, Zipf(1.0) expert popularity (BASELINE configs[4]; "
                                                     "expert-parallel only: --parallel ep with --gpus 2/4/8)"),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """SM clock and throttle reasons while the timed region runs: read through NVML every 2 ms (read-only queries), or,
    where NVML cannot be loaded, from `nvidia-smi -lms 200`."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index, self.nvml, self.stop = [], None, index, None, threading.Event()

    def _nvml_handle(self):
        import pynvml

        pynvml.nvmlInit()
        try:
            import torch

            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            handle = pynvml.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
        except Exception:
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
        return pynvml, handle

    def _poll(self):
        nv, h = self.nvml
        bits = (nv.nvmlClocksThrottleReasonHwSlowdown, nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                nv.nvmlClocksThrottleReasonSwThermalSlowdown, nv.nvmlClocksThrottleReasonSwPowerCap)
        top = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
        while not self.stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                why = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                self.rows.append([str(mhz), str(top), "0"] + ["Active" if why & b else "Not Active" for b in bits])
            except Exception:
                break
            self.stop.wait(0.002)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __enter__(self):
        try:
            self.nvml = self._nvml_handle()
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
            return self
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.nvml:
            self.stop.set()
            self.t.join(1.0)
        elif self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            self.proc.wait(5)

    def summary(self):
        ok = [r for r in self.rows if len(r) >= 7 and r[0].isdigit()]
        if not ok:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        reasons = [n for i, n in enumerate(self.NAMES) if any(r[3 + i].lower().startswith("active") for r in ok)]
        return dict(sm_mhz=float(np.median([int(r[0]) for r in ok])), sm_max_mhz=float(ok[0][1]), reasons=reasons,
                    samples=len(ok), source="nvml" if self.nvml else "nvidia-smi")


def cpu_reference_arm(args, rank):
    """The reference's CPU expert path on the host cores, bounded sample of the headline workload."""
    if rank != 0:
        return
    # the launcher for several ranks pins every process to one OpenMP thread; this arm runs on rank 0 alone and takes all cores
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    import oracle
    from mimo26f_afd_b200 import synth

    wl = WORKLOADS[args.workload]
    seed, tokens = synth.MASTER_SEED, wl["tokens"]
    ids, w = synth.routing(seed, tokens, wl["zipf"])
    x = synth.bf16_to_f32_np(synth.activations_bf16(seed, tokens))
    xq, xs = oracle.quant_wire(x)
    active = np.unique(ids)
    # sample: the first experts (by id) that together hold about `budget` routed rows; the 16-token batch runs whole
    budget_rows = tokens * TOPK if tokens <= 16 else 256
    take, rows = [], 0
    for e in active:
        take.append(int(e)); rows += int((ids == e).sum())
        if rows >= budget_rows:
            break
    e_lo, e_hi = take[0], take[-1] + 1
    tensors = synth.layer_np(seed, [e for e in active if e_lo <= e < e_hi])
    cores = os.cpu_count() or 1
    times, done = [], 0
    for it in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        done, _, _ = oracle.cpu_path(tensors, xq, xs, ids, w, e_lo, e_hi)
        if it >= args.warmup:
            times.append(time.perf_counter() - t0)
    step = float(np.mean(times))
    value = tokens * (done / (tokens * TOPK)) / step          # tokens/s if the whole batch ran at the sample's rate
    sample = f"experts {e_lo}..{e_hi - 1} of the batch: {done} of {tokens * TOPK} routed rows per step, extrapolated by rows"
    line = dict(impl="reference", metric="moe_expert_ffn_tokens_per_s_per_layer", value=value, unit="tokens/s",
                n_gpus=args.gpus, steps=args.steps, warmup=args.warmup, ms_per_step=step * 1e3, higher_is_better=True,
                scaling="strong", vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=args.workload, tokens=tokens, routing="uniform" if not wl["zipf"] else f"zipf{wl['zipf']}",
                            note="reference CPU expert path (E-FP32 lattice), port in oracle/oracle.c"),
                cpu_baseline=dict(value=value, unit="tokens/s", cores=cores, kind="port", sample=sample),
                e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


def run_workload(name, layer, scratch, dev, stream, args, rank, world, peaks):
    """Times `steps` passes (device-resident inputs) and `steps` end-to-end passes (host buffers)."""
    import torch
    import torch.distributed as dist

    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import expert, synth, tp

    wl = WORKLOADS[name]
    tokens, seed = wl["tokens"], synth.MASTER_SEED
    x_bits = synth.activations_bf16(seed, tokens)
    ids, w = synth.routing(seed, tokens, wl["zipf"])
    active = int(len(np.unique(ids)))
    xd = torch.from_numpy(x_bits.view(np.int16)).to(dev)
    idd, wd = torch.from_numpy(ids).to(dev), torch.from_numpy(w).to(dev)
    out = torch.empty((tokens, H), dtype=torch.int16, device=dev)
    total = torch.empty((tokens, H), dtype=torch.float32, device=dev) if world > 1 else None
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)       # > 126 MB L2

    # N > 1: the ranks' BF16 planes are summed by the NVLink peer-memory exchange kernel (--exchange peer, default) or by
    # an NCCL all-gather followed by the rank-sum kernel (--exchange nccl)
    ex = tp.make_exchange(tokens) if world > 1 and args.exchange == "peer" else None

    def step():
        if ex is not None:
            expert.ffn_dev(layer, scratch, xd, idd, wd, tokens, ex.plane(), stream=stream.cuda_stream)
            ex.sum(tokens * H, total, stream=stream.cuda_stream)
            return
        expert.ffn_dev(layer, scratch, xd, idd, wd, tokens, out, stream=stream.cuda_stream)
        if world > 1:
            tp.tp_combine(out, total, stream=stream.cuda_stream)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_steps(with_kernel_events):
        """`steps` iterations, each bracketed by CUDA events on the launching stream, L2 flushed before each."""
        scratch.set_debug(2 if with_kernel_events else 0)
        step()                                               # the first pass after a mode change is not timed
        scratch.status(stream.cuda_stream)
        sync_all()
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        per_kernel = []
        for a, b in pairs:
            flush.fill_(1)                                   # L2 flush between timed iterations (not timed)
            a.record(stream)
            step()
            b.record(stream)
            b.synchronize()
            if with_kernel_events:
                per_kernel.append(scratch.timings())
        sync_all()
        scratch.status(stream.cuda_stream)
        return pairs, per_kernel

    scratch.set_debug(0)
    for _ in range(args.warmup):
        step()
    scratch.status(stream.cuda_stream)
    sync_all()
    with ClockSampler(dev.index or 0) as clocks:
        # the timed region proper: no events inside a step, so the kernels of a step overlap as they do in service
        ev, _ = timed_steps(False)
        # the same steps again with an event between every two kernels: the per-kernel durations of the roofline
        ev_k, kern = timed_steps(True)
    scratch.set_debug(2)
    ms_instrumented = float(np.mean([a.elapsed_time(b) for a, b in ev_k]))
    ms = np.array([a.elapsed_time(b) for a, b in ev])
    t = torch.tensor([float(ms.sum())], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)             # max over ranks
    total_ms = float(t.item())
    value = tokens * args.steps / (total_ms * 1e-3)

    # end to end through the reference-compatible host entry point: pinned host buffers, copies inside the timed region
    xq = scratch.peek("x_payload", np.uint8, (tokens, H))
    xs = scratch.peek("x_scales", np.uint8, (tokens, H // 32))
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
    hq, hs, hi, hw = pin(xq), pin(xs), pin(ids), pin(w)
    hout = torch.empty((tokens, H), dtype=torch.int16).pin_memory()
    import ctypes as C
    from mimo26f_afd_b200 import _native
    err = C.create_string_buffer(256)

    if world > 1:
        # tensor-parallel ranks: quantised rows, ids and weights go up from pinned memory, the device entry point runs
        # the rank's slice, the planes are summed across ranks, and the FP32 result comes back to pinned memory
        dq, ds = torch.empty_like(hq, device=dev), torch.empty_like(hs, device=dev)
        di, dw = torch.empty_like(hi, device=dev), torch.empty_like(hw, device=dev)
        htotal = torch.empty((tokens, H), dtype=torch.float32).pin_memory()

    def e2e_step():
        if world == 1:
            rc = _native.lib().m26b_ffn(layer._h, scratch._h, hq.data_ptr(), H, hs.data_ptr(), H // 32, hi.data_ptr(),
                                        hw.data_ptr(), tokens, hout.data_ptr(), None, err, 256)
            if rc:
                raise M.ExpertError(rc, err.value.decode())
            return
        with torch.cuda.stream(stream):
            dq.copy_(hq, non_blocking=True); ds.copy_(hs, non_blocking=True)
            di.copy_(hi, non_blocking=True); dw.copy_(hw, non_blocking=True)
            dst = ex.plane() if ex is not None else out
            expert.ffn_dev(layer, scratch, dq, di, dw, tokens, dst, x_dtype=expert.X_E4M3, x_scales=ds, stream=stream.cuda_stream)
            if ex is not None:
                ex.sum(tokens * H, total, stream=stream.cuda_stream)
            else:
                tp.tp_combine(out, total, stream=stream.cuda_stream)
            htotal.copy_(total, non_blocking=True)
        scratch.status(stream.cuda_stream)

    for _ in range(max(args.warmup, 10) if tokens <= 128 else min(args.warmup, 3)):   # short calls: let clocks and the driver settle
        e2e_step()
    sync_all()
    with ClockSampler(dev.index or 0) as clocks_e2e:           # the end-to-end region is timed too: its samples join the record
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
    clocks.rows += clocks_e2e.rows
    t = torch.tensor([e2e_s], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = tokens * args.steps / float(t.item())
    h2d = tokens * (H + H // 32 + TOPK * 8)
    d2h = (tokens * H * 2 if world == 1 else tokens * H * 4) + 64
    if ex is not None:
        ex.status(stream.cuda_stream)
        sync_all()
        ex.close()

    # roofline of the dominant kernel (FC1): algorithmic work of that launch / its mean event-timed duration
    fc1_ms = float(np.mean([k["fc1"] for k in kern]))
    il = I // world
    routes = tokens * TOPK
    if name == "decode16":
        fc1_bytes = active * (2 * il * (H // 2) + 2 * il * (H // 32)) + routes * (H + H // 32) + routes * (il + il // 32)
        roof = dict(bound="hbm", achieved=fc1_bytes / (fc1_ms * 1e-3) / 1e9, peak=peaks["hbm_gbs"], unit="GB/s",
                    peak_source=f"{peaks['source']} copy bandwidth (MEASURED_PEAKS.json)", kernel="gemm_mx_kernel<FC1>",
                    algorithmic_bytes=fc1_bytes, traffic=FC1_TRAFFIC_BYTES[name] if world == 1 else None)
    else:
        fc1_flops = 2.0 * 2 * H * il * routes
        roof = dict(bound="tensor", achieved=fc1_flops / (fc1_ms * 1e-3) / 1e12, peak=MXF8F6F4_PEAK_TFLOPS, unit="TFLOP/s",
                    peak_source="measured tcgen05 kind::mxf8f6f4 dense rate on this pool (profiles/mxf8f6f4_mma_rate.md); "
                                f"MEASURED_PEAKS.json holds only bf16 = {peaks['bf16_tflops']} TF/s",
                    kernel="gemm_mx_pair_kernel<FC1>", algorithmic_flops=fc1_flops,
                    traffic=FC1_TRAFFIC_BYTES[name] if world == 1 else None)
        roof["frac_of_random_operand_burst"] = roof["achieved"] / MXF8F6F4_RANDOM_BURST_TFLOPS
        roof["frac_of_random_operand_sustained"] = roof["achieved"] / MXF8F6F4_RANDOM_SUSTAINED_TFLOPS
    roof["frac"] = roof["achieved"] / roof["peak"]
    roof["kernel_ms"] = fc1_ms
    whole = dict(hbm_gbs=(active * EXPERT_BYTES / world + tokens * H * 4 + routes * 8) / (total_ms / args.steps * 1e-3) / 1e9,
                 tflops=FLOP_PER_TOKEN * tokens / world / (total_ms / args.steps * 1e-3) / 1e12)
    launches = (4 if tokens <= 128 else 6 if routes <= 4096 else 8) + (1 if world > 1 else 0)
    return dict(workload=name, tokens=tokens, active_experts=active, value=value, ms_per_step=total_ms / args.steps,
                ms_per_step_with_kernel_events=ms_instrumented,
                e2e=dict(value=e2e_value, unit="tokens/s", h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h),
                roofline=roof, whole_step=whole, kernels_ms={k: float(np.mean([x[k] for x in kern])) for k in kern[0]},
                clocks=clocks.summary(), gpu_launches=launches * args.steps)


def cpu_baseline_for(name, steps_budget_s=20.0):
    """The oracle's port of the reference CPU path on this host, bounded sample (rank 0, N = 1 only)."""
    import oracle
    from mimo26f_afd_b200 import synth

    wl = WORKLOADS[name]
    tokens, seed = wl["tokens"], synth.MASTER_SEED
    ids, w = synth.routing(seed, tokens, wl["zipf"])
    sub = min(tokens, 16)                                   # the sample keeps whole tokens of the batch
    ids_s, w_s = ids[:sub], w[:sub]
    xq, xs = oracle.quant_wire(synth.bf16_to_f32_np(synth.activations_bf16(seed, tokens)[:sub]))
    active = np.unique(ids_s)
    take, rows = [], 0
    for e in active:                                        # 16 tokens = 128 routed rows: the decode batch runs whole
        take.append(int(e)); rows += int((ids_s == e).sum())
        if rows >= sub * TOPK:
            break
    tensors = synth.layer_np(seed, take)
    oracle.cpu_path(tensors, xq, xs, ids_s, w_s, take[0], take[-1] + 1)          # warm-up (page in the weights)
    reps, t0 = 0, time.perf_counter()
    while True:                                             # the 16-token batch takes a fraction of a second: repeat it for ~10 s
        done, _, _ = oracle.cpu_path(tensors, xq, xs, ids_s, w_s, take[0], take[-1] + 1)
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= 10.0 or reps >= 200:
            break
    value = reps * (done / TOPK) / dt
    return dict(value=value, unit="tokens/s", cores=os.cpu_count() or 1, kind="port",
                sample=f"{reps} x {done} routed rows ({done / TOPK:.2f} token-equivalents) of the first {sub} tokens, experts "
                       f"{take[0]}..{take[-1]}, {dt:.1f} s in all; reference CPU expert path (E-FP32), OpenMP over output rows")


def run_expert_parallel(name, dev, stream, args, rank, world):
    """Expert-parallel step (--parallel ep): rank r holds 256 / N experts and owns 1 / N of the tokens; rows are gathered
    from and results scattered to their owners over NVLink inside the permutation and FC2 kernels."""
    import torch
    import torch.distributed as dist

    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import expert, synth, tp

    wl = WORKLOADS[name]
    tokens, seed = wl["tokens"], synth.MASTER_SEED
    n_local = E // world
    wts = synth.layer_torch(seed, dev, n_experts=n_local, first_expert=rank * n_local)
    layer = M.Layer.from_checkpoint_ep(*[wts[n] for n in synth.TENSORS], ep_rank=rank, ep_size=world)
    del wts
    torch.cuda.empty_cache()
    scratch = M.Scratch()
    ep = tp.make_expert_parallel(tokens)
    lo, hi = tp.shard_tokens(tokens, rank, world)
    rows = hi - lo
    ids, w = synth.routing(seed, tokens, wl["zipf"])
    counts = np.bincount(ids.reshape(-1), minlength=E)
    per_rank = counts.reshape(world, n_local).sum(1)
    x_bits = synth.activations_bf16(seed, rows, first_token=lo)
    xd = torch.from_numpy(np.ascontiguousarray(x_bits).view(np.int16)).to(dev)
    idd, wd = torch.from_numpy(np.ascontiguousarray(ids[lo:hi])).to(dev), torch.from_numpy(np.ascontiguousarray(w[lo:hi])).to(dev)
    out = torch.empty((rows, H), dtype=torch.int16, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step():
        ep.step(layer, scratch, xd, idd, wd, rows, out, stream=stream.cuda_stream)

    def sync_all():
        dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    scratch.status(stream.cuda_stream); ep.status(stream.cuda_stream)
    sync_all()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    with ClockSampler(dev.index or 0) as clocks:
        for a, b in ev:
            flush.fill_(1)
            a.record(stream); step(); b.record(stream)
            b.synchronize()
        sync_all()
    scratch.status(stream.cuda_stream); ep.status(stream.cuda_stream)
    t = torch.tensor([float(sum(a.elapsed_time(b) for a, b in ev))], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    value = tokens * args.steps / (total_ms * 1e-3)

    # end to end: this rank's BF16 rows, ids and weights from pinned memory, its BF16 result rows back to pinned memory
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
    hx, hi_, hw = pin(x_bits.view(np.int16)), pin(ids[lo:hi]), pin(w[lo:hi])
    hout = torch.empty((rows, H), dtype=torch.int16).pin_memory()

    def e2e_step():
        with torch.cuda.stream(stream):
            xd.copy_(hx, non_blocking=True); idd.copy_(hi_, non_blocking=True); wd.copy_(hw, non_blocking=True)
            step()
            hout.copy_(out, non_blocking=True)
        scratch.status(stream.cuda_stream)

    for _ in range(2):
        e2e_step()
    sync_all()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    torch.cuda.synchronize()
    t = torch.tensor([time.perf_counter() - t0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = tokens * args.steps / float(t.item())
    ep.status(stream.cuda_stream)
    sync_all()
    ep.close()
    step_s = total_ms / args.steps * 1e-3
    # the busiest rank bounds the step: its share of the routed rows x FLOP per routed row
    busiest = float(per_rank.max()) * (FLOP_PER_TOKEN / TOPK)
    roof = dict(bound="tensor", kernel="whole expert-parallel step on the busiest rank (FC1 + FC2 + gather/scatter over NVLink)",
                achieved=busiest / step_s / 1e12, peak=MXF8F6F4_PEAK_TFLOPS, unit="TFLOP/s", traffic=None,
                algorithmic_flops=busiest, peak_source="measured tcgen05 kind::mxf8f6f4 dense rate (profiles/mxf8f6f4_mma_rate.md)")
    roof["frac"] = roof["achieved"] / roof["peak"]
    launches = 3 + 2 + 8 * ((tokens + 16383) // 16384) + 1
    return dict(workload=name, tokens=tokens, active_experts=int((counts > 0).sum()), value=value, ms_per_step=total_ms / args.steps,
                e2e=dict(value=e2e_value, unit="tokens/s", h2d_bytes_per_step=rows * (H * 2 + TOPK * 8) * world,
                         d2h_bytes_per_step=rows * H * 2 * world),
                roofline=roof, clocks=clocks.summary(), gpu_launches=launches * args.steps,
                whole_step=dict(tflops=FLOP_PER_TOKEN * tokens / step_s / 1e12, tflops_per_gpu=FLOP_PER_TOKEN * tokens / world / step_s / 1e12,
                                routed_rows_per_rank=[int(v) for v in per_rank],
                                imbalance=float(per_rank.max() / per_rank.mean()),
                                nvlink_bytes_in_busiest_rank=int(per_rank.max() * (world - 1) / world * (H + H // 32)),
                                nvlink_bytes_out_busiest_rank=int(per_rank.max() * (world - 1) / world * H * 4)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode16", choices=sorted(WORKLOADS))
    ap.add_argument("--no-prefill", action="store_true", help="skip the 8192-token prefill sub-result")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: how the ranks' planes are summed (NVLink peer-memory kernel, or NCCL all-gather + sum kernel)")
    ap.add_argument("--parallel", default="tp", choices=["tp", "ep"],
                    help="N > 1: tensor parallel over the intermediate dimension (default) or expert parallel")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        cpu_reference_arm(args, rank)
        return

    import torch
    import torch.distributed as dist

    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import synth

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: the product has no CPU path (use --impl reference for the CPU baseline)")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    peaks = measured_peaks()
    if args.parallel == "ep" or args.workload == "prefill64k":
        if world < 2:
            raise SystemExit("--parallel ep / prefill64k need --gpus 2, 4 or 8 (launch with torch.distributed.run)")
        stream = torch.cuda.Stream(device=dev)
        torch.cuda.set_stream(stream)
        r = run_expert_parallel(args.workload, dev, stream, args, rank, world)
        if rank == 0:
            line = dict(metric="moe_expert_ffn_tokens_per_s_per_layer", value=r["value"], unit="tokens/s", n_gpus=world,
                        steps=args.steps, warmup=args.warmup, ms_per_step=r["ms_per_step"], higher_is_better=True,
                        scaling="strong", vs_baseline=None, dtype="e4m3 x e2m1 (mxf8f6f4), f32 accumulate", data="synthetic",
                        config=dict(workload=args.workload, description=WORKLOADS[args.workload]["desc"], tokens=r["tokens"],
                                    top_k=TOPK, experts=E, hidden=H, intermediate=I, active_experts=r["active_experts"],
                                    parallelism=f"ep{world}", l2="flushed between timed iterations",
                                    input_codec="wire (FP8 E4M3 + UE8M0 K32)"),
                        e2e=r["e2e"], gpu_launches=r["gpu_launches"], clocks=r["clocks"], roofline=r["roofline"],
                        whole_step=r["whole_step"], cpu_baseline=None)
            print(json.dumps(line), flush=True)
        dist.barrier()
        dist.destroy_process_group()
        return
    weights = synth.layer_torch(synth.MASTER_SEED, dev)
    layer = M.Layer.from_checkpoint(*[weights[n] for n in synth.TENSORS], tp_rank=rank, tp_size=world)
    del weights
    torch.cuda.empty_cache()
    scratch = M.Scratch()
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)

    main_r = run_workload(args.workload, layer, scratch, dev, stream, args, rank, world, peaks)
    extra = None
    if not args.no_prefill and args.workload == "decode16":
        sub = argparse.Namespace(**vars(args))
        sub.steps, sub.warmup = max(3, min(args.steps, 10)), max(3, min(args.warmup, 5))
        extra = run_workload("prefill8k", layer, scratch, dev, stream, sub, rank, world, peaks)
        extra["parallelism"] = f"tp{world}" if world > 1 else "single"
    prefill_ep = None
    if extra is not None and world > 1:
        # Prefill under tensor parallelism repeats the per-token work on every rank and stops scaling at two GPUs; the
        # scheme for prefill on several GPUs is expert parallelism, so the same segment is also reported that way.
        layer.close()
        del layer
        torch.cuda.empty_cache()
        prefill_ep = run_expert_parallel("prefill8k", dev, stream, sub, rank, world)
        prefill_ep["parallelism"] = f"ep{world}"
    if rank == 0:
        cpu = cpu_baseline_for(args.workload) if world == 1 else None
        line = dict(metric="moe_expert_ffn_tokens_per_s_per_layer", value=main_r["value"], unit="tokens/s", n_gpus=world,
                    steps=args.steps, warmup=args.warmup, ms_per_step=main_r["ms_per_step"], higher_is_better=True,
                    scaling="strong" if world > 1 else "weak", vs_baseline=None, dtype="e4m3 x e2m1 (mxf8f6f4), f32 accumulate",
                    data="synthetic",
                    config=dict(workload=args.workload, description=WORKLOADS[args.workload]["desc"], tokens=main_r["tokens"],
                                top_k=TOPK, experts=E, hidden=H, intermediate=I, active_experts=main_r["active_experts"],
                                parallelism=f"tp{world}" if world > 1 else "single",
                                exchange=(args.exchange if world > 1 else None), l2="flushed between timed iterations",
                                input_codec="wire (FP8 E4M3 + UE8M0 K32)"),
                    e2e=main_r["e2e"], gpu_launches=main_r["gpu_launches"], clocks=main_r["clocks"], roofline=main_r["roofline"],
                    whole_step=main_r["whole_step"], kernels_ms=main_r["kernels_ms"],
                    ms_per_step_with_kernel_events=main_r["ms_per_step_with_kernel_events"], cpu_baseline=cpu)
        if extra:
            line["prefill"] = {k: extra[k] for k in ("workload", "tokens", "value", "ms_per_step", "ms_per_step_with_kernel_events", "e2e", "roofline", "whole_step",
                                                     "kernels_ms", "clocks")}
            line["prefill"]["unit"] = "tokens/s"
            line["prefill"]["parallelism"] = extra["parallelism"]
        if prefill_ep:
            line["prefill_expert_parallel"] = {k: prefill_ep[k] for k in ("workload", "tokens", "value", "ms_per_step", "e2e", "roofline",
                                                                           "whole_step", "clocks", "parallelism")}
            line["prefill_expert_parallel"]["unit"] = "tokens/s"
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
