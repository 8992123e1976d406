"""Seeded synthetic inputs for the routed-expert FFN: MXFP4 weights in the checkpoint layout,
BF16 activations and top-8 routing.

They stand in for the real checkpoint and routing traces, which this build never sees. The
generator is SplitMix64 used as a counter-based hash (``value_i = mix(base + (i+1) * GOLDEN)``),
the constants of the reference's trace generator (``crates/mimo26-expert/tests/gpu/step_hist.h:44-47``),
so any slice of any tensor can be produced independently and bit-identically by numpy on the
host (for the CPU oracle) and by torch on the device (for a whole 3.4 GB layer).

Weights (``crates/mimo26-expert/src/mxfp4.rs:13-19`` layout): payload bytes uniform over 0..255
(all 16 E2M1 codes, low nibble = even k), scale bytes uniform over ``scale_lo..scale_hi``
(default 118..122, exponents -9..-5; real checkpoints hold 118..125,
``crates/mimo26-expert/src/fixture.rs:28-36``).
"""
from __future__ import annotations

import numpy as np

GOLDEN = 0x9E3779B97F4A7C15
M1 = 0xBF58476D1CE4E5B9
M2 = 0x94D049BB133111EB
MASTER_SEED = 0x26AFD

H, I, E, TOPK = 4096, 2048, 256, 8
TENSORS = ("gate_w", "gate_s", "up_w", "up_s", "down_w", "down_s")
SHAPES = {"gate_w": (I, H // 2), "gate_s": (I, H // 32), "up_w": (I, H // 2), "up_s": (I, H // 32),
          "down_w": (H, I // 2), "down_s": (H, I // 32)}
_U64 = np.uint64


def _mix_np(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = (z ^ (z >> _U64(30))) * _U64(M1)
        z = (z ^ (z >> _U64(27))) * _U64(M2)
        return z ^ (z >> _U64(31))


def stream_base(seed: int, *ids: int) -> int:
    """Base state of the sub-stream named by ``ids`` (tensor index, expert, ...)."""
    z = seed & 0xFFFFFFFFFFFFFFFF
    for v in ids:
        z = int(_mix_np(np.array([(z + (v + 1) * GOLDEN) & 0xFFFFFFFFFFFFFFFF], dtype=_U64))[0])
    return z


def words_np(base: int, n: int, start: int = 0) -> np.ndarray:
    """Words ``start .. start+n`` of a stream, as uint64."""
    with np.errstate(over="ignore"):
        idx = np.arange(start + 1, start + n + 1, dtype=_U64)
        return _mix_np(_U64(base) + idx * _U64(GOLDEN))


def _scale_bytes_np(raw: np.ndarray, lo: int, hi: int) -> np.ndarray:
    return (lo + ((raw.astype(np.uint16) * (hi - lo + 1)) >> 8)).astype(np.uint8)


def expert_tensor_np(seed: int, name: str, expert: int, scale_lo: int = 118, scale_hi: int = 122) -> np.ndarray:
    """One expert's tensor ``name`` (uint8, checkpoint shape)."""
    shape = SHAPES[name]
    n = shape[0] * shape[1]
    raw = words_np(stream_base(seed, TENSORS.index(name), expert), n // 8).view(np.uint8)
    if name.endswith("_s"):
        raw = _scale_bytes_np(raw, scale_lo, scale_hi)
    return raw.reshape(shape)


def layer_np(seed: int, experts, scale_lo: int = 118, scale_hi: int = 122) -> dict:
    """Host copies of the six stacked tensors with only ``experts`` filled (others zero)."""
    out = {}
    for name in TENSORS:
        t = np.zeros((E,) + SHAPES[name], dtype=np.uint8)
        for e in experts:
            t[e] = expert_tensor_np(seed, name, int(e), scale_lo, scale_hi)
        out[name] = t
    return out


def layer_torch(seed: int, device, scale_lo: int = 118, scale_hi: int = 122, n_experts: int = E, first_expert: int = 0,
                experts=None) -> dict:
    """Experts ``first_expert .. first_expert + n_experts - 1`` (default all 256), or the experts listed in ``experts`` in
    that order, generated on ``device`` with torch integer ops; bit-identical to ``expert_tensor_np``. torch is the
    device allocator here, not a compute path."""
    import torch

    ids = [first_expert + e for e in range(n_experts)] if experts is None else [int(e) for e in experts]
    E = len(ids)  # noqa: N806 (shadows the module constant inside this function only)

    def s64(v: int) -> int:
        return v - (1 << 64) if v >= (1 << 63) else v

    def lsr(z, n):
        return (z >> n) & ((1 << (64 - n)) - 1)

    out = {}
    for ti, name in enumerate(TENSORS):
        shape = SHAPES[name]
        n_words = shape[0] * shape[1] // 8
        bases = torch.tensor([s64(stream_base(seed, ti, e)) for e in ids], dtype=torch.int64, device=device)
        res = torch.empty((E, n_words), dtype=torch.int64, device=device)
        idx = torch.arange(1, n_words + 1, dtype=torch.int64, device=device) * s64(GOLDEN)
        for e0 in range(0, E, 32):  # bound the temporaries
            z = bases[e0:e0 + 32, None] + idx[None, :]
            z = (z ^ lsr(z, 30)) * s64(M1)
            z = (z ^ lsr(z, 27)) * s64(M2)
            res[e0:e0 + 32] = z ^ lsr(z, 31)
        raw = res.view(torch.uint8).reshape((E,) + shape)
        if name.endswith("_s"):
            raw = (scale_lo + ((raw.to(torch.int32) * (scale_hi - scale_lo + 1)) >> 8)).to(torch.uint8)
        out[name] = raw.contiguous()
        del res
    return out


def bf16_rne_np(x: np.ndarray) -> np.ndarray:
    """float32 -> BF16 bits (uint16), round to nearest even."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_to_f32_np(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def normal_np(seed: int, stream: int, n: int, start: int = 0) -> np.ndarray:
    """Values ``start .. start + n`` of a stream of N(0,1) float32 (Box-Muller on the stream's words)."""
    w = words_np(stream_base(seed, 100 + stream), n, start)
    u1 = ((w >> _U64(40)).astype(np.float64) + 1.0) / 16777217.0
    u2 = ((w & _U64(0xFFFFFF)).astype(np.float64)) / 16777216.0
    return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32)


def activations_bf16(seed: int, tokens: int, first_token: int = 0) -> np.ndarray:
    """BF16 activations N(0,1) of tokens ``first_token .. first_token + tokens``, shape [tokens, 4096], as uint16 bit
    patterns. The values of a token do not depend on how the batch is cut."""
    return bf16_rne_np(normal_np(seed, 0, tokens * H, first_token * H)).reshape(tokens, H)


def activations_bf16_torch(seed: int, tokens: int, device, first_token: int = 0):
    """Device-side generator for batches too large to make on the host in reasonable time: BF16 N(0,1) bit patterns
    [tokens, 4096] as int16, a deterministic function of (seed, token, column) on the same counter stream as
    ``activations_bf16`` but with the Box-Muller step in FP32 on the device, so the two are NOT bit-identical. Used
    where no host-side oracle looks at the values (timing of the 65,536-token batch). torch is the allocator and the
    element-wise engine here, not a compute path of the library."""
    import torch

    def s64(v: int) -> int:
        return v - (1 << 64) if v >= (1 << 63) else v

    def lsr(z, n):
        return (z >> n) & ((1 << (64 - n)) - 1)

    base = s64(stream_base(seed, 100))
    out = torch.empty((tokens, H), dtype=torch.int16, device=device)
    step = 2048
    for t0 in range(0, tokens, step):
        n = min(step, tokens - t0)
        idx = torch.arange((first_token + t0) * H + 1, (first_token + t0 + n) * H + 1, dtype=torch.int64, device=device)
        z = base + idx * s64(GOLDEN)
        z = (z ^ lsr(z, 30)) * s64(M1)
        z = (z ^ lsr(z, 27)) * s64(M2)
        z = z ^ lsr(z, 31)
        u1 = (lsr(z, 40).to(torch.float32) + 1.0) / 16777217.0
        u2 = (z & 0xFFFFFF).to(torch.float32) / 16777216.0
        g = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(6.283185307179586 * u2)
        out[t0:t0 + n] = g.to(torch.bfloat16).view(torch.int16).reshape(n, H)
    return out


def routing(seed: int, tokens: int, zipf_s: float = 0.0):
    """Top-8 routing: FP32 logits N(0,1) (+ log popularity, Zipf exponent ``zipf_s`` over a seeded
    expert permutation), top-8 by value with ties to the lower id
    (``crates/mimo26-coordinator/src/router.rs:61-68``), weights = FP32 softmax of the selected logits.
    Returns (ids int32 [tokens,8], weights float32 [tokens,8])."""
    logits = normal_np(seed, 1, tokens * E).reshape(tokens, E)
    if zipf_s > 0.0:
        perm = np.argsort(words_np(stream_base(seed, 102), E), kind="stable")
        p = (np.arange(1, E + 1, dtype=np.float64) ** -zipf_s)
        p /= p.sum()
        logp = np.empty(E, dtype=np.float32)
        logp[perm] = np.log(p).astype(np.float32)
        logits = (logits + logp[None, :]).astype(np.float32)
    ids = np.argsort(-logits, axis=1, kind="stable")[:, :TOPK].astype(np.int32)
    sel = np.take_along_axis(logits, ids, axis=1).astype(np.float32)
    ex = np.exp(sel - sel.max(axis=1, keepdims=True)).astype(np.float32)
    w = (ex / ex.sum(axis=1, keepdims=True, dtype=np.float32)).astype(np.float32)
    return np.ascontiguousarray(ids), np.ascontiguousarray(w)


def canonical_rank_image_np(tensors: dict, experts, tp_rank: int, tp_size: int) -> np.ndarray:
    """The reference's canonical-v2 rank image (``crates/mimo26-repack/src/repack.rs:135-163`` build_slice,
    generalised from TP4): per expert gate payload | gate scales | up payload | up scales | down payload |
    down scales for rows/columns of this rank. Only ``experts`` are filled."""
    il = I // tp_size
    r0 = tp_rank * il
    image = 2 * (il * (H // 2) + il * (H // 32)) + H * (il // 2) + H * (il // 32)
    out = np.zeros((E, image), dtype=np.uint8)
    for e in experts:
        parts = [tensors["gate_w"][e, r0:r0 + il].reshape(-1), tensors["gate_s"][e, r0:r0 + il].reshape(-1),
                 tensors["up_w"][e, r0:r0 + il].reshape(-1), tensors["up_s"][e, r0:r0 + il].reshape(-1),
                 tensors["down_w"][e][:, r0 // 2:(r0 + il) // 2].reshape(-1),
                 tensors["down_s"][e][:, r0 // 32:(r0 + il) // 32].reshape(-1)]
        out[e] = np.concatenate(parts)
    return out
