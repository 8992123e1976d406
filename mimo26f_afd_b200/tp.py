"""Multi-GPU layouts of the expert FFN on one NVSwitch box: one process per GPU, torch.distributed for the plumbing.

The reference shards the expert intermediate dimension over four machines (TP4: rank r owns gate/up rows
[512 r, 512 (r+1)) and the matching down columns, ``crates/mimo26-repack/src/geom.rs:29-35``) and sums the four
BF16 partial planes on the coordinator in FP32, in rank order (``crates/mimo26-coordinator/kernels/glue.cu:202-213``,
``crates/mimo26-wire/src/l4.rs:169-244``). Here the ranks are G in {1, 2, 4, 8} GPUs: inputs are replicated and each
rank produces a full-width BF16 partial. For decode-sized steps ``expert.ffn_tp_dev`` runs the combine and the exchange as
one kernel (every rank stores its BF16 codes, tagged with the step number, into windows the peers have mapped, and adds
what the peers stored). Otherwise the planes stay where each rank's combine wrote them, in such a window, and one kernel
per rank adds them in rank order while reading the peers' planes over NVLink (``make_exchange`` / ``Exchange.sum``);
``tp_combine`` is the alternative that gathers the planes with one NCCL
all-gather and sums them with the library's kernel (also what runs on CPU tensors over gloo in the tests). Both keep
the reference's bit-exact rank-ordered sum (an NCCL ring reduce would round per hop, in ring order). ``make_expert_parallel``
connects the windows of the expert-parallel step (experts and tokens split over the ranks).
"""
from __future__ import annotations

H, I = 4096, 2048


def tp_slice(tp_rank: int, tp_size: int):
    """(first intermediate feature, local width) of a rank; every K32 / K128 block stays inside one rank."""
    if tp_size not in (1, 2, 4, 8) or not 0 <= tp_rank < tp_size:
        raise ValueError(f"tp_rank {tp_rank} / tp_size {tp_size}: tp_size must be 1, 2, 4 or 8")
    il = I // tp_size
    return tp_rank * il, il


def shard_tokens(tokens: int, rank: int, world: int):
    """Data-parallel split of a token batch: contiguous [lo, hi) for this rank (used when ranks serve
    independent requests; no collective on the data path)."""
    base, extra = divmod(tokens, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def serving_rank(ids, world: int, replicated=None):
    """Which expert-parallel rank serves each route of a batch: ``ids`` int [tokens, 8] -> int array [tokens, 8].
    A route to an expert in ``replicated`` (experts every rank holds a copy of) is served by the rank that owns the
    route's token (``shard_tokens``); every other route by the rank whose block of 256 / world experts holds the expert.
    The library's planner applies the same rule on the device; this host form is for load statistics (rows per rank,
    rows that cross NVLink) and for choosing which experts to replicate."""
    import numpy as np

    ids = np.asarray(ids)
    tokens = ids.shape[0]
    his = np.array([shard_tokens(tokens, r, world)[1] for r in range(world)])
    owner = np.searchsorted(his, np.arange(tokens), side="right")[:, None]
    home = ids // (256 // world)
    if replicated is None or len(replicated) == 0:
        return home
    return np.where(np.isin(ids, np.asarray(replicated)), owner, home)


def busiest_experts(ids, n: int):
    """The ``n`` experts with the most routes in ``ids`` (ties to the lower id): a replication set for ``serving_rank`` /
    ``Layer.from_checkpoint_ep(replica_ids=...)`` when the batch itself is the popularity statistic."""
    import numpy as np

    counts = np.bincount(np.asarray(ids).reshape(-1), minlength=256)
    return np.argsort(-counts, kind="stable")[:n].astype(np.int32)


def all_gather_planes(plane, group=None):
    """All-gather one BF16 partial plane [tokens, 4096] per rank; returns the list in rank order.
    Works on CUDA tensors (NCCL) and on CPU tensors (gloo), so the exchange can be tested without GPUs."""
    import torch.distributed as dist

    import torch

    world = dist.get_world_size(group)
    # exchanged as raw bytes: the planes are bit patterns, and not every backend moves 16-bit integer tensors
    raw = plane.contiguous().view(torch.uint8)
    out = [torch.empty_like(raw) for _ in range(world)]
    dist.all_gather(out, raw, group=group)
    return [o.view(plane.dtype).view(plane.shape) for o in out]


def make_exchange(tokens: int, group=None):
    """This rank's exchange window for planes of up to ``tokens`` rows, connected to every peer of ``group``:
    the 64-byte window handles travel through one host-side all-gather, after which the ranks read each other's
    planes directly over NVLink (``Exchange.sum``) with no library collective on the data path."""
    import torch.distributed as dist

    from . import expert

    rank, world = dist.get_rank(group), dist.get_world_size(group)
    ex = expert.Exchange(((tokens * H * 2 + 255) // 256) * 256, rank, world)
    handles = [None] * world
    dist.all_gather_object(handles, ex.handle_bytes(), group=group)
    ex.connect(b"".join(handles))
    dist.barrier(group)          # every window is mapped everywhere before the first publication
    return ex


def make_expert_parallel(tokens: int, group=None):
    """This rank's expert-parallel window for steps of ``tokens`` tokens (over all ranks), connected to every peer.
    Rank r owns tokens ``shard_tokens(tokens, r, world)`` and experts [r 256 / world, (r + 1) 256 / world)."""
    import torch.distributed as dist

    from . import expert

    rank, world = dist.get_rank(group), dist.get_world_size(group)
    ep = expert.ExpertParallel(tokens, rank, world)
    lo, hi = shard_tokens(tokens, rank, world)
    assert ep.rows() == hi - lo
    handles = [None] * world
    dist.all_gather_object(handles, ep.handle_bytes(), group=group)
    ep.connect(b"".join(handles))
    dist.barrier(group)
    return ep


def tp_combine(plane, out_f32, group=None, stream=None):
    """Rank-ordered FP32 sum of every rank's BF16 plane into ``out_f32`` (CUDA tensors)."""
    from . import expert

    planes = all_gather_planes(plane, group)
    if not plane.is_cuda:
        raise RuntimeError("tp_combine sums on the GPU; there is no CPU path (tests use the oracle for the sum)")
    expert.rank_sum_dev(planes, plane.numel(), out_f32, stream=stream)
    return planes
