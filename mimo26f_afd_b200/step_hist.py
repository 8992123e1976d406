"""Trace-driven step workloads: per-layer-step histograms of M (routed rows per active expert) turned back into token
batches that load the experts exactly that way.

The reference derives these histograms from routing traces of real prompts (``harness/route_hist.py``: workloads
``C1-w8`` = 8, ``C4-w8`` = 32, ``C16-w8`` = 128 tokens per step) and replays them against its kernels
(``crates/mimo26-expert/tests/gpu/step_hist.h``). A step is ``{"layer": L, "hist": {"M": count, ...}}``: ``count``
distinct experts receive ``M`` rows each. The file format and its checks follow ``step_hist.h:13-38``; the expert
assignment is the same seeded Fisher-Yates shuffle of the 256 ids over the same SplitMix64 stream (``step_hist.h:39-62``)
so a step touches the same experts here as there. What is new here is ``step_batch``: a top-8 routing table with
distinct experts per token that realises a histogram, so the whole path (plan included) runs on it unchanged.
"""
from __future__ import annotations

import json

import numpy as np

TOPK, EXPERTS = 8, 256
WORKLOAD_TOKENS = {"C1-w8": 8, "C4-w8": 32, "C16-w8": 128}
_MASK = (1 << 64) - 1


class StepHistError(ValueError):
    pass


def _random64(state: int):
    state = (state + 0x9E3779B97F4A7C15) & _MASK
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return state, z ^ (z >> 31)


def sample_seed(seed: int, step: int, sample: int) -> int:
    seed ^= ((step + 1) * 0xD1B54A32D192ED03) & _MASK
    seed ^= ((sample + 1) * 0x94D049BB133111EB) & _MASK
    return _random64(seed & _MASK)[1]


def parse(doc, name: str):
    """The steps of workload ``name`` from a parsed JSON document, with the reference's checks."""
    if name not in doc or not isinstance(doc[name], dict):
        raise StepHistError("workload must be an object")
    w = doc[name]
    if "steps" not in w:
        raise StepHistError("per-layer-step histograms required; aggregate hist cannot reconstruct simultaneous expert loads")
    steps = w["steps"]
    if not isinstance(steps, list) or not 1 <= len(steps) <= 100000:
        raise StepHistError("step count must be 1..100000")
    tokens = WORKLOAD_TOKENS.get(name, 0)
    out = []
    for raw in steps:
        layer = raw.get("layer")
        if not isinstance(layer, int) or not 1 <= layer <= 47:
            raise StepHistError("MoE layer must be 1..47")
        h = raw.get("hist")
        if not isinstance(h, dict) or not h:
            raise StepHistError("empty/non-object step histogram")
        hist, experts, routes = {}, 0, 0
        for key, count in h.items():
            if not key or key[0] == "0" or not key.isdigit():
                raise StepHistError("noncanonical M key")
            m = int(key)
            if not 1 <= m <= 128:
                raise StepHistError("M must be 1..128")
            if not isinstance(count, int) or not 1 <= count <= 256:
                raise StepHistError("active count must be 1..256")
            hist[m] = count
            experts += count
            routes += m * count
            if experts > 256:
                raise StepHistError("more than 256 distinct experts in one layer-step")
            if tokens and m > tokens:
                raise StepHistError("M exceeds workload token count")
        if tokens and routes != tokens * TOPK:
            raise StepHistError("route count differs from top8 workload contract")
        out.append(dict(layer=layer, hist=dict(sorted(hist.items())), experts=experts, routes=routes))
    return dict(name=name, seed=int(w.get("seed", 20260924)), steps=out)


def assign_experts(step, seed: int):
    """[(M, [expert ids])] in ascending M: the seeded shuffle of 0..255 dealt to the bins in order."""
    ids = list(range(EXPERTS))
    state = seed & _MASK
    for i in range(EXPERTS - 1, 0, -1):
        state, r = _random64(state)
        j = r % (i + 1)
        ids[i], ids[j] = ids[j], ids[i]
    out, used = [], 0
    for m, n in step["hist"].items():
        out.append((m, ids[used:used + n]))
        used += n
    return out


def step_batch(step, seed: int, tokens: int | None = None):
    """(ids int32 [T, 8], weights float32 [T, 8]) whose per-expert row counts are the step's histogram, with eight
    distinct experts per token. The routes, sorted by expert, are dealt to the tokens round-robin: an expert's M copies
    sit in M consecutive positions and M <= T, so no token receives an expert twice."""
    routes = step["routes"]
    if routes % TOPK:
        raise StepHistError("route count is not a multiple of 8")
    t = routes // TOPK if tokens is None else tokens
    if t * TOPK != routes:
        raise StepHistError("route count differs from top8 workload contract")
    flat = []
    for m, experts in assign_experts(step, seed):
        if m > t:
            raise StepHistError("M exceeds workload token count")
        for e in experts:
            flat += [e] * m
    ids = np.asarray(flat, np.int32).reshape(TOPK, t).T.copy()             # position p -> token p % T, slot p // T
    assert all(len(set(row)) == TOPK for row in ids.tolist())
    state = (seed ^ 0x5DEECE66D) & _MASK
    logits = np.empty((t, TOPK), np.float64)
    for i in range(t * TOPK):
        state, r = _random64(state)
        logits.flat[i] = (r >> 11) / float(1 << 53)
    w = np.exp(logits)
    return ids, (w / w.sum(axis=1, keepdims=True)).astype(np.float32)


def histogram_of(ids) -> dict:
    counts = np.bincount(np.asarray(ids).reshape(-1), minlength=EXPERTS)
    ms, ns = np.unique(counts[counts > 0], return_counts=True)
    return {int(m): int(n) for m, n in zip(ms, ns)}


def synthetic_workload(name: str, n_steps: int, seed: int = 20260924, zipf: float = 1.2):
    """A stand-in for a traced workload (the traces are not available): histograms of seeded Zipf-skewed top-8 routing at
    the workload's token count, in the file format above."""
    from . import synth

    tokens = WORKLOAD_TOKENS[name]
    steps = []
    for i in range(n_steps):
        ids, _ = synth.routing(seed + i, tokens, zipf)
        steps.append(dict(layer=1 + i % 47, hist={str(m): n for m, n in histogram_of(ids).items()}))
    return {name: dict(seed=seed, steps=steps)}


def load(path: str, name: str):
    with open(path) as f:
        return parse(json.load(f), name)
