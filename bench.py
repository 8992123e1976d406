#!/usr/bin/env python
"""Benchmark of the routed-expert FFN hot path (one MoE layer) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one pass of the hot path over one batch of seeded synthetic input: activation quantisation, route plan,
token permutation, grouped gate/up GEMM + SwiGLU + intermediate quantiser, grouped down GEMM, ordered top-8
combine (and, with N > 1 ranks, the exchange between the GPUs). The headline workload (`value`) is the 16-token
decode batch; the same JSON line carries the 128-token verify round, the 8,192-token prefill segment and, on several
GPUs, the 65,536-token batch, each under its own key. Weights are resident in HBM; inputs are resident in HBM for
`value` and in pinned host memory for `e2e`, which goes through the library's host entry points (m26b_ffn, m26b_ffn_tp,
m26b_ep_ffn) with both copies inside the timed region.

Timing discipline (after the reference's own bench, crates/mimo26-expert/tests/b1_core/bench_connected.cuh:21-88): warm-up,
then K samples (31 by default), each preceded by a barrier over the ranks, a device synchronisation and an L2 flush and
bracketed by CUDA events on the launching stream; a sample's time is the maximum over the ranks; the median is reported
with min / max / mean and the spread between ranks; correctness is checked before AND after the timed region, and an
identity record (GPU, SMs, commit, command, seed) goes with every line. No events sit inside a timed step (they would
break the overlap of consecutive kernels); per-kernel durations for the roofline come from a few extra instrumented steps.

With N > 1 ranks the layer is tensor-parallel over the intermediate dimension (the reference's own TP4 scheme,
generalised): every rank runs the whole batch on its 1/N slice of every expert and the BF16 partial planes are summed in
rank order by one kernel per rank that reads the peers' planes over NVLink (--exchange nccl: an NCCL all-gather followed
by the sum kernel). Prefill-sized batches are also run expert-parallel (rank r holds 256 / N experts and 1 / N of the
tokens). Total work is fixed as N grows: strong scaling. Before and after timing every rank checks that the peer
exchange and the NCCL path give identical bits, rank 0 checks the sum against the CPU oracle, and the expert-parallel
step is compared bit for bit with the single-GPU layer; a mismatch ends the run with a non-zero exit code.

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
MXF8F6F4_PEAK_TFLOPS = 4450.0               # tcgen05 kind::mxf8f6f4 dense rate measured on this pool (burst, operands of a few small codes)
MXF8F6F4_RANDOM_BURST_TFLOPS = 3694.0       # same instruction stream on random operands, first 7 ms launch
MXF8F6F4_RANDOM_SUSTAINED_TFLOPS = 3193.0   # same, after three seconds (1.32 GHz under the 1000 W limit)
WORKLOADS = {
    "decode16": dict(tokens=16, zipf=0.0, desc="16-token decode batch, uniform routing"),
    "verify128": dict(tokens=128, zipf=1.2, desc="speculative verify round: 16 streams x 8 tokens, Zipf(1.2) expert popularity"),
    "prefill8k": dict(tokens=8192, zipf=0.0, desc="8192-token prefill segment, uniform routing"),
    "prefill64k": dict(tokens=65536, zipf=1.0, desc="65536-token batch, Zipf(1.0) expert popularity"),
}


def workload_config(name):
    """The `config` of a JSON line: the workload only, identical for both arms of the benchmark."""
    wl = WORKLOADS[name]
    return dict(workload=name, description=wl["desc"], tokens=wl["tokens"], top_k=TOPK, experts=E, hidden=H, intermediate=I,
                routing="uniform" if not wl["zipf"] else f"zipf{wl['zipf']}", activations="bf16 N(0,1)",
                weights="MXFP4 (E2M1 + UE8M0 per 32), scale bytes 118..122", input_codec="wire (FP8 E4M3 + UE8M0 K32)")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def profiled_traffic():
    """DRAM bytes per launch of the dominant kernel from the committed ncu captures (profiles/traffic.json, written next
    to the summaries it comes from); {} when the file is absent."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        return json.load(open(path))
    except (OSError, ValueError):
        return {}


def identity(args, dev=None):
    rec = dict(command=" ".join([os.path.basename(sys.executable)] + sys.argv), seed=hex(0x26AFD), host_cores=os.cpu_count())
    try:
        rec["commit"] = subprocess.run(["git", "-C", ROOT, "rev-parse", "--short", "HEAD"], capture_output=True, text=True, timeout=5).stdout.strip() or None
    except Exception:
        rec["commit"] = None
    if dev is not None:
        import torch

        p = torch.cuda.get_device_properties(dev)
        rec.update(gpu=p.name, sms=p.multi_processor_count, arch=f"sm_{p.major}{p.minor}", hbm_gib=round(p.total_memory / 2 ** 30, 1),
                   torch=torch.__version__, cuda=torch.version.cuda)
    return rec


def stats(ms):
    a = np.asarray(ms, dtype=np.float64)
    return dict(median=float(np.median(a)), min=float(a.min()), max=float(a.max()), mean=float(a.mean()), samples=int(a.size))


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
    x = synth.bf16_to_f32_np(synth.activations_bf16(seed, min(tokens, 8192)))
    xq, xs = oracle.quant_wire(x)
    ids, w = ids[:xq.shape[0]], w[:xq.shape[0]]
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
    st = stats([t * 1e3 for t in times])
    step = st["median"] * 1e-3
    value = tokens * (done / (tokens * TOPK)) / step          # tokens/s if the whole batch ran at the sample's rate
    sample = f"experts {e_lo}..{e_hi - 1} of the batch: {done} of {tokens * TOPK} routed rows per step, extrapolated by rows"
    line = dict(impl="reference", metric="moe_expert_ffn_tokens_per_s_per_layer", value=value, unit="tokens/s",
                n_gpus=args.gpus, steps=args.steps, warmup=args.warmup, ms_per_step=step * 1e3, ms_per_step_stats=st,
                higher_is_better=True, scaling="strong", vs_baseline=None, dtype="f32", data="synthetic",
                config=workload_config(args.workload),
                note="reference CPU expert path (E-FP32 lattice, crates/mimo26-spark/src/main.rs:75-95), port in oracle/oracle.c, OpenMP over output rows",
                cpu_baseline=dict(value=value, unit="tokens/s", cores=cores, kind="port", sample=sample),
                e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0), identity=identity(args))
    print(json.dumps(line), flush=True)


class Ctx:
    """What every measurement needs: device, launching stream, ranks, the L2 flush buffer."""

    def __init__(self, args, dev, stream, rank, world):
        import torch

        self.args, self.dev, self.stream, self.rank, self.world = args, dev, stream, rank, world
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)       # > 126 MB L2
        self.peaks = measured_peaks()
        self.traffic = profiled_traffic()

    def barrier(self):
        import torch
        import torch.distributed as dist

        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def over_ranks(self, ms):
        """Per-sample maximum over the ranks of this rank's per-sample times, and the median spread between ranks."""
        import torch
        import torch.distributed as dist

        mine = torch.tensor(ms, dtype=torch.float64, device=self.dev)
        if self.world == 1:
            return [float(v) for v in ms], 0.0
        every = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(every, mine)
        m = torch.stack(every)
        return [float(v) for v in m.max(0).values.cpu()], float((m.max(0).values - m.min(0).values).median().item())

    def all_true(self, ok):
        import torch
        import torch.distributed as dist

        if self.world == 1:
            return bool(ok)
        t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=self.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    def timed_device(self, step, k, align=None):
        """k samples of step() on the launching stream: barrier + synchronise + L2 flush before each (not timed), CUDA
        events around it. `align` (several ranks): a device-side rendezvous of the ranks enqueued right before the first
        event, so that every rank's sample starts within a microsecond of the others', as consecutive steps of a serving
        loop do (each step ends in the exchange, which is such a rendezvous); without it the host barrier and the flush
        leave the ranks several microseconds apart, and that skew would be counted as step time of the earliest rank."""
        import torch

        ms = []
        for _ in range(k):
            self.barrier()
            self.flush.fill_(1)
            if align is not None:
                align()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(self.stream)
            step()
            b.record(self.stream)
            b.synchronize()
            ms.append(a.elapsed_time(b))
        return self.over_ranks(ms)

    def timed_host(self, call, k):
        """k samples of a synchronous host call (uploads and downloads inside), wall clock each. The calls follow one
        another as in a serving loop (with several ranks a barrier lines them up before each sample); no L2 flush: a
        step streams 1.4 to 3.4 GB of expert weights, an order of magnitude more than the L2 holds."""
        ms = []
        for _ in range(k):
            if self.world > 1:
                self.barrier()
            t0 = time.perf_counter()
            call()
            ms.append((time.perf_counter() - t0) * 1e3)
        return self.over_ranks(ms)


def make_inputs(ctx, name, lo=None, hi=None):
    """Seeded inputs of a workload: routes on the host and the device, BF16 activation rows [lo, hi) on the device. Batches
    above 8,192 tokens get their activations from the device-side generator (nothing on the host reads their values)."""
    import torch

    from mimo26f_afd_b200 import synth

    wl = WORKLOADS[name]
    tokens, seed = wl["tokens"], synth.MASTER_SEED
    lo, hi = (0, tokens) if lo is None else (lo, hi)
    ids, w = synth.routing(seed, tokens, wl["zipf"])
    if tokens > 8192:
        xd, x_bits = synth.activations_bf16_torch(seed, hi - lo, ctx.dev, first_token=lo), None
    else:
        x_bits = synth.activations_bf16(seed, hi - lo, first_token=lo)
        xd = torch.from_numpy(np.ascontiguousarray(x_bits).view(np.int16)).to(ctx.dev)
    idd = torch.from_numpy(np.ascontiguousarray(ids[lo:hi])).to(ctx.dev)
    wd = torch.from_numpy(np.ascontiguousarray(w[lo:hi])).to(ctx.dev)
    return dict(tokens=tokens, ids=ids, w=w, x_bits=x_bits, xd=xd, idd=idd, wd=wd, active=int(len(np.unique(ids))))


def quantised_on_device(ctx, xd, rows):
    """The library's own wire quantiser on device rows -> pinned host copies (what a coordinator would send)."""
    import torch

    from mimo26f_afd_b200 import expert

    q = torch.empty((rows, H), dtype=torch.uint8, device=ctx.dev)
    s = torch.empty((rows, H // 32), dtype=torch.uint8, device=ctx.dev)
    f = torch.zeros(1, dtype=torch.int32, device=ctx.dev)
    if rows:
        expert.quantize_dev(xd, expert.X_BF16, rows * H, expert.CODEC_WIRE, q, s, f, stream=ctx.stream.cuda_stream)
    torch.cuda.synchronize()
    return q.cpu().pin_memory(), s.cpu().pin_memory()


PASS_ROWS = 16384          # rows per call of the device entry point


def run_tp(ctx, name, layer, scratch, k, y16=False, with_e2e=True, with_kernels=True):
    """One workload on the (tensor-parallel) layer: device-resident timing, per-kernel durations, end to end."""
    import torch

    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import expert, tp

    args, world, dev, stream = ctx.args, ctx.world, ctx.dev, ctx.stream
    inp = make_inputs(ctx, name)
    tokens, ids, w = inp["tokens"], inp["ids"], inp["w"]
    xd, idd, wd = inp["xd"], inp["idd"], inp["wd"]
    out = torch.empty((tokens, H), dtype=torch.int16, device=dev)
    total = torch.empty((tokens, H), dtype=torch.float32, device=dev) if world > 1 else None
    ex = tp.make_exchange(tokens) if world > 1 and args.exchange in ("peer", "pull") else None
    scratch.set_route_output(y16)

    def step():
        if ex is not None and tokens <= PASS_ROWS and args.exchange == "peer":
            # combine and exchange in one kernel up to 512 tokens; the library falls back to combine + pull exchange above
            expert.ffn_tp_dev(layer, scratch, ex, xd, idd, wd, tokens, total, stream=stream.cuda_stream)
            return
        dst = ex.plane() if ex is not None else out.data_ptr()
        for r0 in range(0, tokens, PASS_ROWS):
            n = min(PASS_ROWS, tokens - r0)
            expert.ffn_dev(layer, scratch, xd[r0:r0 + n], idd[r0:r0 + n], wd[r0:r0 + n], n, dst + r0 * H * 2, stream=stream.cuda_stream)
        if ex is not None:
            ex.sum(tokens * H, total, stream=stream.cuda_stream)
        elif world > 1:
            tp.tp_combine(out, total, stream=stream.cuda_stream)

    def check():
        scratch.status(stream.cuda_stream)
        if ex is not None:
            ex.status(stream.cuda_stream)

    scratch.set_debug(0)
    for _ in range(args.warmup):
        step()
    check()
    # the exchange kernel on an (unread) plane is the ranks' device-side rendezvous before each sample
    align = (lambda: ex.sum(8, total, stream=stream.cuda_stream)) if ex is not None else None
    with ClockSampler(dev.index or 0) as clocks:
        ms, spread = ctx.timed_device(step, k, align)
    check()
    st = stats(ms)
    res = dict(workload=name, tokens=tokens, active_experts=inp["active"], parallelism=f"tp{world}" if world > 1 else "single",
               route_outputs="bf16" if y16 else "f32", value=tokens / (st["median"] * 1e-3), unit="tokens/s",
               ms_per_step=st["median"], ms_per_step_stats=st, rank_spread_ms=spread, clocks=clocks.summary())
    il, routes = I // (world * args.rank_slice), tokens * TOPK
    if with_kernels and tokens <= PASS_ROWS:
        # the same step with an event between every two kernels: per-kernel durations for the roofline
        scratch.set_debug(2)
        step(); check()
        kern = []
        for _ in range(5):
            ctx.barrier(); ctx.flush.fill_(1)
            step()
            kern.append(scratch.timings())
            check()
        scratch.set_debug(0)
        km = {key: float(np.median([x[key] for x in kern])) for key in kern[0]}
        res["kernels_ms"] = km
        fc1_ms, fc2_ms = km["fc1"], km["fc2"]
        if tokens <= 128:
            fc1_bytes = inp["active"] * (2 * il * (H // 2) + 2 * il * (H // 32)) + routes * (H + H // 32) + routes * (il + il // 32)
            roof = dict(bound="hbm", achieved=fc1_bytes / (fc1_ms * 1e-3) / 1e9, peak=ctx.peaks["hbm_gbs"], unit="GB/s",
                        peak_source=f"{ctx.peaks['source']} copy bandwidth", kernel="gemm_mx_kernel<FC1>", algorithmic_bytes=fc1_bytes)
        else:
            fc1_flops = 2.0 * 2 * H * il * routes
            roof = dict(bound="tensor", achieved=fc1_flops / (fc1_ms * 1e-3) / 1e12, peak=MXF8F6F4_PEAK_TFLOPS, unit="TFLOP/s",
                        peak_source="tcgen05 kind::mxf8f6f4 dense rate measured on this pool with the same instruction (burst, few small "
                                    f"codes); the measured bf16 cuBLAS figure is {ctx.peaks['bf16_tflops']} TF/s",
                        kernel="gemm_mx_pair_kernel<FC1>", algorithmic_flops=fc1_flops)
            roof["frac_of_random_operand_burst"] = roof["achieved"] / MXF8F6F4_RANDOM_BURST_TFLOPS
            roof["frac_of_random_operand_sustained"] = roof["achieved"] / MXF8F6F4_RANDOM_SUSTAINED_TFLOPS
            fc2_flops = 2.0 * H * il * routes
            roof["fc2"] = dict(kernel="gemm_mx_pair_kernel<FC2>", achieved=fc2_flops / (fc2_ms * 1e-3) / 1e12, kernel_ms=fc2_ms,
                               frac=fc2_flops / (fc2_ms * 1e-3) / 1e12 / MXF8F6F4_PEAK_TFLOPS)
        roof["frac"] = roof["achieved"] / roof["peak"]
        roof["kernel_ms"] = fc1_ms
        t = ctx.traffic.get(name) if world == 1 and not y16 else None
        roof["traffic"] = t.get("fc1_dram_bytes") if t else None
        if t:
            roof["traffic_source"] = t.get("source")
        res["roofline"] = roof
    step_s = st["median"] * 1e-3
    res["whole_step"] = dict(hbm_gbs=(inp["active"] * EXPERT_BYTES / world + tokens * H * 4 + routes * 8) / step_s / 1e9,
                             tflops=FLOP_PER_TOKEN * tokens / step_s / 1e12, tflops_per_gpu=FLOP_PER_TOKEN * tokens / world / step_s / 1e12)
    passes = (tokens + PASS_ROWS - 1) // PASS_ROWS
    per_pass = 4 if tokens <= 128 else 5 if routes <= 4096 else 7
    fused_exchange = ex is not None and tokens <= 512 and args.exchange == "peer"
    res["gpu_launches_per_step"] = passes * per_pass + (1 if world > 1 and not fused_exchange else 0)
    if world > 1:
        res["exchange"] = ("combine + push exchange in one kernel" if fused_exchange else
                           "pull exchange kernel" if ex is not None else "nccl all-gather + rank-sum kernel")

    if with_e2e and tokens <= PASS_ROWS:
        # end to end through the host entry points: pinned host buffers, copies inside the timed region
        hq, hs = quantised_on_device(ctx, xd, tokens)
        pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
        hi_, hw = pin(ids), pin(w)
        if world == 1:
            hout = torch.empty((tokens, H), dtype=torch.int16).pin_memory()
            call = lambda: M.ffn(layer, scratch, hq.numpy().reshape(-1), hs.numpy().reshape(-1), hi_.numpy().reshape(-1), hw.numpy().reshape(-1),
                                 tokens, hout.numpy().view(np.uint16).reshape(-1))
            d2h = tokens * H * 2 + 64
        else:
            ex2 = ex if ex is not None else tp.make_exchange(tokens)
            hsum = torch.empty((tokens, H), dtype=torch.float32).pin_memory() if ctx.rank == 0 else None
            call = lambda: M.ffn_tp(layer, scratch, ex2, hq.data_ptr(), hs.data_ptr(), hi_.data_ptr(), hw.data_ptr(), tokens,
                                    hsum.data_ptr() if hsum is not None else None)
            d2h = tokens * H * 4 + 64 * world
        for _ in range(max(args.warmup, 10) if tokens <= 128 else 3):      # short calls: let clocks and the driver settle
            call()
        with ClockSampler(dev.index or 0) as clocks_e2e:
            ms_e, spread_e = ctx.timed_host(call, k)
        se = stats(ms_e)
        res["e2e"] = dict(value=tokens / (se["median"] * 1e-3), unit="tokens/s", ms_per_step=se["median"], ms_per_step_stats=se,
                          rank_spread_ms=spread_e, h2d_bytes_per_step=world * tokens * (H + H // 32 + TOPK * 8), d2h_bytes_per_step=d2h,
                          entry_point="m26b_ffn" if world == 1 else "m26b_ffn_tp (every rank uploads the request; rank 0 downloads the FP32 sum)",
                          clocks=clocks_e2e.summary())
        if world > 1 and ex is None:
            ex2.close()
    if ex is not None:
        check()
        ctx.barrier()
        ex.close()
    scratch.set_route_output(False)
    return res


def run_ep(ctx, name, layer, scratch, k, y16=False, with_e2e=True, hot=None):
    """Expert-parallel step: rank r holds 256 / N experts and owns 1 / N of the tokens; rows are gathered from and results
    scattered to their owners over NVLink inside the permutation and FC2 kernels. `hot`: the experts every rank holds a
    copy of (their routes are served by the token's owner)."""
    import torch

    from mimo26f_afd_b200 import tp

    args, world, dev, stream = ctx.args, ctx.world, ctx.dev, ctx.stream
    wl = WORKLOADS[name]
    tokens = wl["tokens"]
    lo, hi = tp.shard_tokens(tokens, ctx.rank, world)
    rows = hi - lo
    inp = make_inputs(ctx, name, lo, hi)
    ids, w = inp["ids"], inp["w"]
    xd, idd, wd = inp["xd"], inp["idd"], inp["wd"]
    n_local = E // world
    counts = np.bincount(ids.reshape(-1), minlength=E)
    serving = tp.serving_rank(ids, world, hot)
    per_rank = np.bincount(serving.reshape(-1), minlength=world)
    owner = tp.serving_rank(ids, world, np.arange(E))          # with every expert replicated a route stays with its token's owner
    crossing = int((serving != owner).sum())                   # routed rows whose token lives on another rank
    ep = tp.make_expert_parallel(tokens)
    ep.set_route_output(y16)
    out = torch.empty((max(rows, 1), H), dtype=torch.int16, device=dev)

    def step():
        ep.step(layer, scratch, xd, idd, wd, rows, out, stream=stream.cuda_stream)

    def check():
        scratch.status(stream.cuda_stream)
        ep.status(stream.cuda_stream)

    for _ in range(args.warmup):
        step()
    check()
    with ClockSampler(dev.index or 0) as clocks:
        ms, spread = ctx.timed_device(step, k)
    check()
    st = stats(ms)
    step_s = st["median"] * 1e-3
    busiest = float(per_rank.max()) * (FLOP_PER_TOKEN / TOPK)       # the busiest rank bounds the step
    res = dict(workload=name, tokens=tokens, active_experts=int((counts > 0).sum()), parallelism=f"ep{world}",
               route_outputs="bf16" if y16 else "f32", value=tokens / step_s, unit="tokens/s", ms_per_step=st["median"],
               ms_per_step_stats=st, rank_spread_ms=spread, clocks=clocks.summary(),
               roofline=dict(bound="tensor" if tokens > 128 else "hbm", kernel="whole expert-parallel step on the busiest rank",
                             achieved=busiest / step_s / 1e12, peak=MXF8F6F4_PEAK_TFLOPS, unit="TFLOP/s", traffic=None,
                             frac=busiest / step_s / 1e12 / MXF8F6F4_PEAK_TFLOPS, algorithmic_flops=busiest),
               whole_step=dict(tflops=FLOP_PER_TOKEN * tokens / step_s / 1e12, tflops_per_gpu=FLOP_PER_TOKEN * tokens / world / step_s / 1e12,
                               routed_rows_per_rank=[int(v) for v in per_rank], imbalance=float(per_rank.max() / max(per_rank.mean(), 1e-9)),
                               imbalance_without_replicas=float(counts.reshape(world, n_local).sum(1).max() / max(counts.sum() / world, 1e-9)),
                               replicated_experts=0 if hot is None else int(len(hot)),
                               routed_rows_crossing_nvlink=crossing, nvlink_bytes_in=crossing * (H + H // 32),
                               nvlink_bytes_out=crossing * H * (2 if y16 else 4)),
               gpu_launches_per_step=3 + 2 + 6 * ((tokens + PASS_ROWS - 1) // PASS_ROWS) + 1)
    if with_e2e:
        hq, hs = quantised_on_device(ctx, xd, rows)
        pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
        hi_, hw = pin(ids[lo:hi]), pin(w[lo:hi])
        hout = torch.empty((max(rows, 1), H), dtype=torch.int16).pin_memory()
        call = lambda: ep.ffn_host(layer, scratch, hq.data_ptr(), hs.data_ptr(), hi_.data_ptr(), hw.data_ptr(), rows, hout.data_ptr())
        for _ in range(3):
            call()
        ms_e, spread_e = ctx.timed_host(call, k)
        se = stats(ms_e)
        res["e2e"] = dict(value=tokens / (se["median"] * 1e-3), unit="tokens/s", ms_per_step=se["median"], ms_per_step_stats=se,
                          rank_spread_ms=spread_e, h2d_bytes_per_step=tokens * (H + H // 32 + TOPK * 8), d2h_bytes_per_step=tokens * H * 2,
                          entry_point="m26b_ep_ffn (every rank uploads its token block and downloads its BF16 rows)")
    check()
    ctx.barrier()
    ep.close()
    return res


REPLICATED_EXPERTS = 32      # copies of the busiest experts on every expert-parallel rank when the routing is skewed


def build_ep_layer(ctx, name):
    """This rank's expert-parallel layer for a workload: its block of 256 / N experts and, when the workload's routing is
    skewed, copies of the batch's busiest experts (the same set on every rank: all ranks see the same seeded routing, as a
    serving system would share its popularity statistics)."""
    import torch

    import mimo26f_afd_b200 as M
    from mimo26f_afd_b200 import synth, tp

    wl = WORKLOADS[name]
    n_local = E // ctx.world
    hot = None
    if wl["zipf"]:
        ids, _ = synth.routing(synth.MASTER_SEED, wl["tokens"], wl["zipf"])
        hot = tp.busiest_experts(ids, REPLICATED_EXPERTS)
    wts = synth.layer_torch(synth.MASTER_SEED, ctx.dev, n_experts=n_local, first_expert=ctx.rank * n_local)
    reps = synth.layer_torch(synth.MASTER_SEED, ctx.dev, experts=hot) if hot is not None else None
    layer = M.Layer.from_checkpoint_ep(*[wts[n] for n in synth.TENSORS], ep_rank=ctx.rank, ep_size=ctx.world,
                                       replicas=[reps[n] for n in synth.TENSORS] if hot is not None else None, replica_ids=hot)
    del wts, reps
    torch.cuda.empty_cache()
    return layer, hot


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) / max(np.linalg.norm(b.astype(np.float64)), 1e-30))


def parity_tp(ctx, layer, scratch):
    """Correctness of the (tensor-parallel) layer on the 16-token batch: quantised bytes and plan indices exact against the
    CPU oracle; with several ranks the peer-memory exchange and the NCCL path must give identical bits on every rank and
    rank 0 compares the sum with the oracle's wire result (rel L2 <= 1e-3 + N 2^-9: every plane is rounded to BF16 first)."""
    import torch

    import oracle
    from mimo26f_afd_b200 import expert, synth, tp

    world, dev, stream = ctx.world, ctx.dev, ctx.stream
    out = dict(ok=True)
    for tokens, zipf in ((16, 0.0), (300, 1.2)):
        seed = synth.MASTER_SEED + 77
        x_bits = synth.activations_bf16(seed, tokens)
        ids, w = synth.routing(seed, tokens, zipf)
        xd = torch.from_numpy(x_bits.view(np.int16)).to(dev)
        idd, wd = torch.from_numpy(ids).to(dev), torch.from_numpy(w).to(dev)
        plane = torch.empty((tokens, H), dtype=torch.int16, device=dev)
        part = torch.empty((tokens, H), dtype=torch.float32, device=dev)
        expert.ffn_dev(layer, scratch, xd, idd, wd, tokens, plane, partial_out=part, stream=stream.cuda_stream)
        scratch.status(stream.cuda_stream)
        xq, xs = oracle.quant_wire(synth.bf16_to_f32_np(x_bits))
        st, oinv, _, _, _ = oracle.plan(ids, w)
        exact = (st == 0 and np.array_equal(scratch.peek("x_payload", np.uint8, (tokens, H)), xq)
                 and np.array_equal(scratch.peek("x_scales", np.uint8, (tokens, H // 32)), xs)
                 and np.array_equal(scratch.peek("inverse", np.int32, (tokens * TOPK,)), oinv))
        out[f"quantised_bytes_and_plan_exact_{tokens}"] = bool(exact)
        out["ok"] &= bool(exact)
        if world == 1:
            if tokens == 16:
                ref = oracle.ffn_layer(synth.layer_np(synth.MASTER_SEED, np.unique(ids)), xq, xs, ids, w)
                r = rel_l2(part.cpu().numpy(), ref["partial"])
                out["rel_l2_vs_oracle"] = r
                out["bf16_flips_vs_oracle"] = int((plane.cpu().numpy().view(np.uint16) != ref["bf16"]).sum())
                out["ok"] &= ref["rc"] == 0 and r <= 1e-3
            continue
        ex = tp.make_exchange(tokens)
        peer_sum = torch.empty((tokens, H), dtype=torch.float32, device=dev)
        nccl_sum = torch.empty((tokens, H), dtype=torch.float32, device=dev)
        same = True
        for _ in range(3):                                      # both slots and a reuse
            expert.ffn_dev(layer, scratch, xd, idd, wd, tokens, ex.plane(), stream=stream.cuda_stream)
            ex.sum(tokens * H, peer_sum, stream=stream.cuda_stream)
            scratch.status(stream.cuda_stream)
            ex.status(stream.cuda_stream)
            tp.tp_combine(plane, nccl_sum, stream=stream.cuda_stream)
            torch.cuda.synchronize()
            same &= bool(torch.equal(peer_sum.view(torch.int32), nccl_sum.view(torch.int32)))
        out[f"peer_exchange_equals_nccl_sum_{tokens}"] = ctx.all_true(same)
        out["ok"] &= out[f"peer_exchange_equals_nccl_sum_{tokens}"]
        same = True
        for _ in range(3):                                      # the same with combine and exchange in one kernel
            peer_sum.zero_()
            expert.ffn_tp_dev(layer, scratch, ex, xd, idd, wd, tokens, peer_sum, stream=stream.cuda_stream)
            scratch.status(stream.cuda_stream)
            ex.status(stream.cuda_stream)
            torch.cuda.synchronize()
            same &= bool(torch.equal(peer_sum.view(torch.int32), nccl_sum.view(torch.int32)))
        out[f"fused_combine_exchange_equals_nccl_sum_{tokens}"] = ctx.all_true(same)
        out["ok"] &= out[f"fused_combine_exchange_equals_nccl_sum_{tokens}"]
        if tokens == 16 and ctx.rank == 0:
            tensors = synth.layer_np(synth.MASTER_SEED, np.unique(ids))
            planes = [oracle.ffn_layer(tensors, xq, xs, ids, w, tp_rank=r, tp_size=world)["bf16"] for r in range(world)]
            wire = oracle.rank_sum(np.stack(planes))
            r = rel_l2(peer_sum.cpu().numpy(), wire)
            out["rel_l2_vs_oracle_wire_sum"] = r
            out["rel_l2_bound"] = 1e-3 + world * 2.0 ** -9
            out["ok"] &= r <= 1e-3 + world * 2.0 ** -9
        ctx.barrier()
        ex.close()
    out["ok"] = ctx.all_true(out["ok"])
    return out


def parity_ep(ctx, ep_layer, full_layer, scratch, scratch_full, tag=""):
    """The expert-parallel step against the single-GPU layer run on the same rank over the whole batch: bit for bit, FP32
    plane and BF16 rows (a GEMM row does not depend on how routes are tiled, nor on which rank serves it)."""
    import torch

    from mimo26f_afd_b200 import expert, synth, tp

    dev, stream, world = ctx.dev, ctx.stream, ctx.world
    out = dict(ok=True)
    for tokens, zipf in ((16, 0.0), (1000, 1.0)):
        seed = synth.MASTER_SEED + 78
        x_bits = synth.activations_bf16(seed, tokens)
        ids, w = synth.routing(seed, tokens, zipf)
        lo, hi = tp.shard_tokens(tokens, ctx.rank, world)
        xd = torch.from_numpy(x_bits.view(np.int16)).to(dev)
        idd, wd = torch.from_numpy(ids).to(dev), torch.from_numpy(w).to(dev)
        ref = torch.empty((tokens, H), dtype=torch.int16, device=dev)
        ref_part = torch.empty((tokens, H), dtype=torch.float32, device=dev)
        expert.ffn_dev(full_layer, scratch_full, xd, idd, wd, tokens, ref, partial_out=ref_part, stream=stream.cuda_stream)
        scratch_full.status(stream.cuda_stream)
        ep = tp.make_expert_parallel(tokens)
        got = torch.empty((max(hi - lo, 1), H), dtype=torch.int16, device=dev)
        part = torch.empty((max(hi - lo, 1), H), dtype=torch.float32, device=dev)
        same = True
        for _ in range(2):
            ep.step(ep_layer, scratch, xd[lo:hi], idd[lo:hi], wd[lo:hi], hi - lo, got, partial_out=part, stream=stream.cuda_stream)
            scratch.status(stream.cuda_stream)
            ep.status(stream.cuda_stream)
            torch.cuda.synchronize()
            same &= bool(torch.equal(got[:hi - lo], ref[lo:hi])) and bool(torch.equal(part[:hi - lo].view(torch.int32), ref_part[lo:hi].view(torch.int32)))
        out[f"expert_parallel{tag}_equals_single_gpu_{tokens}"] = ctx.all_true(same)
        out["ok"] &= out[f"expert_parallel{tag}_equals_single_gpu_{tokens}"]
        ctx.barrier()
        ep.close()
    return out


def cpu_baseline_for(name):
    """The oracle's port of the reference CPU path on this host, bounded sample (rank 0, N = 1 only)."""
    import oracle
    from mimo26f_afd_b200 import synth

    wl = WORKLOADS[name]
    tokens, seed = wl["tokens"], synth.MASTER_SEED
    ids, w = synth.routing(seed, tokens, wl["zipf"])
    sub = min(tokens, 16)                                   # the sample keeps whole tokens of the batch
    ids_s, w_s = ids[:sub], w[:sub]
    xq, xs = oracle.quant_wire(synth.bf16_to_f32_np(synth.activations_bf16(seed, sub)))
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


def fail(ctx, what, parity):
    if ctx.rank == 0:
        print(json.dumps(dict(error=f"parity check failed ({what})", parity=parity)), file=sys.stderr, flush=True)
    sys.exit(3)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=31)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode16", choices=["decode16", "verify128", "prefill8k"],
                    help="the headline workload of the JSON line (the others are reported under their own keys)")
    ap.add_argument("--no-extra", action="store_true", help="headline workload only: no sub-results, no CPU baseline")
    ap.add_argument("--rank-slice", type=int, default=1, choices=[1, 2, 4, 8],
                    help="with --gpus 1: run ONE rank's share of a G-way tensor-parallel step (rank 0's slice of every expert, no "
                         "exchange) on this GPU; for profiling a rank's kernels, not a benchmark result")
    ap.add_argument("--exchange", default="peer", choices=["peer", "pull", "nccl"],
                    help="N > 1: how the ranks' planes are summed: peer = NVLink peer memory, combine and exchange in one kernel up "
                         "to 512 tokens (the default); pull = combine kernel, then the exchange kernel that reads the peers' planes; "
                         "nccl = NCCL all-gather + sum kernel")
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
    k, k_big = args.steps, max(3, min(args.steps, 7))
    weights = synth.layer_torch(synth.MASTER_SEED, dev)
    if args.rank_slice > 1 and world > 1:
        raise SystemExit("--rank-slice is for --gpus 1")
    layer = M.Layer.from_checkpoint(*[weights[n] for n in synth.TENSORS], tp_rank=rank, tp_size=world * args.rank_slice)
    del weights
    torch.cuda.empty_cache()
    scratch = M.Scratch()
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    ctx = Ctx(args, dev, stream, rank, world)
    if args.rank_slice > 1:
        # one rank's kernels on one GPU: timings only (the parity block needs the whole layer, sub-results mean nothing here)
        r = run_tp(ctx, args.workload, layer, scratch, args.steps, with_e2e=False)
        print(json.dumps(dict(note=f"one rank's share of a {args.rank_slice}-way tensor-parallel step on one GPU, no exchange: not a benchmark result",
                              rank_slice=args.rank_slice, config=workload_config(args.workload), ms_per_step=r["ms_per_step"],
                              ms_per_step_stats=r["ms_per_step_stats"], kernels_ms=r.get("kernels_ms"), roofline=r.get("roofline"),
                              clocks=r["clocks"], identity=identity(args, dev))), flush=True)
        return

    parity = dict(checked=True, before=parity_tp(ctx, layer, scratch))
    if not parity["before"]["ok"]:
        fail(ctx, "before timing", parity)
    main_r = run_tp(ctx, args.workload, layer, scratch, k)
    extra = {}
    if not args.no_extra:
        for name, key in (("decode16", "decode16"), ("verify128", "verify128"), ("prefill8k", "prefill")):
            if name != args.workload:
                extra[key] = run_tp(ctx, name, layer, scratch, k)
        if world == 1:
            extra["prefill_bf16_route_outputs"] = run_tp(ctx, "prefill8k", layer, scratch, k, y16=True, with_e2e=False)
        else:
            extra["prefill64k_tp"] = run_tp(ctx, "prefill64k", layer, scratch, k_big, with_e2e=False, with_kernels=False)
    parity["after"] = parity_tp(ctx, layer, scratch)
    if not parity["after"]["ok"]:
        fail(ctx, "after timing", parity)
    if world > 1 and not args.no_extra:
        # Prefill under tensor parallelism repeats the per-token work on every rank; the scheme for prefill on several GPUs
        # is expert parallelism, so the same batches are also reported that way (and the decode batch, for comparison).
        layer.close()
        del layer
        torch.cuda.empty_cache()
        ep_layer, _ = build_ep_layer(ctx, "prefill8k")
        ep_layer_hot, hot = build_ep_layer(ctx, "prefill64k")
        weights = synth.layer_torch(synth.MASTER_SEED, dev)
        full_layer = M.Layer.from_checkpoint(*[weights[n] for n in synth.TENSORS])
        del weights
        torch.cuda.empty_cache()
        scratch_full = M.Scratch()

        def ep_parity(key):
            parity[key] = parity_ep(ctx, ep_layer, full_layer, scratch, scratch_full)
            parity[key].update({k2: v for k2, v in parity_ep(ctx, ep_layer_hot, full_layer, scratch, scratch_full, "_with_replicas").items() if k2 != "ok"})
            parity[key]["ok"] = all(v for k2, v in parity[key].items() if k2 != "ok")
            if not parity[key]["ok"]:
                fail(ctx, key, parity)

        ep_parity("expert_parallel_before")
        extra["prefill_expert_parallel"] = run_ep(ctx, "prefill8k", ep_layer, scratch, k)
        extra["prefill_expert_parallel_bf16_route_outputs"] = run_ep(ctx, "prefill8k", ep_layer, scratch, k, y16=True, with_e2e=False)
        extra["decode16_expert_parallel"] = run_ep(ctx, "decode16", ep_layer, scratch, k, with_e2e=False)
        extra["prefill64k_ep_no_replicas"] = run_ep(ctx, "prefill64k", ep_layer, scratch, k_big, with_e2e=False)
        extra["prefill64k_ep"] = run_ep(ctx, "prefill64k", ep_layer_hot, scratch, k_big, with_e2e=False, hot=hot)
        extra["prefill64k_ep_bf16_route_outputs"] = run_ep(ctx, "prefill64k", ep_layer_hot, scratch, k_big, y16=True, with_e2e=False, hot=hot)
        ep_parity("expert_parallel_after")
    if rank == 0:
        cpu = cpu_baseline_for(args.workload) if world == 1 and not args.no_extra else None
        line = dict(metric="moe_expert_ffn_tokens_per_s_per_layer", value=main_r["value"], unit="tokens/s", n_gpus=world,
                    steps=k, warmup=args.warmup, ms_per_step=main_r["ms_per_step"], ms_per_step_stats=main_r["ms_per_step_stats"],
                    rank_spread_ms=main_r["rank_spread_ms"], higher_is_better=True, scaling="strong", vs_baseline=None,
                    dtype="e4m3 x e2m1 (mxf8f6f4), f32 accumulate", data="synthetic", config=workload_config(args.workload),
                    parallelism=main_r["parallelism"], exchange=(args.exchange if world > 1 else None),
                    timing="value: per sample a barrier over the ranks, a device synchronise and an L2 flush (256 MB fill), with several "
                           "ranks a device-side rendezvous (one exchange kernel on an unread plane), then CUDA events "
                           "on the launching stream around the step, max over ranks, value = tokens / median sample; e2e: wall clock "
                           "around each synchronous host call, calls back to back (inputs larger than L2: 1.4-3.4 GB of weights per step)",
                    active_experts=main_r["active_experts"], e2e=main_r.get("e2e"), gpu_launches=main_r["gpu_launches_per_step"] * k,
                    clocks=main_r["clocks"], roofline=main_r.get("roofline"), whole_step=main_r["whole_step"],
                    kernels_ms=main_r.get("kernels_ms"), cpu_baseline=cpu, parity=parity, identity=identity(args, dev))
        line.update(extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
