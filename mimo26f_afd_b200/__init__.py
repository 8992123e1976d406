"""B200-native routed-expert FFN: the host-side mirror of the reference's expert-rank API.

The compute lives in ``libm26b_expert.so`` (hand-written CUDA for sm_100a behind a C ABI,
``include/m26b_expert.h``). This package binds it with ctypes and mirrors the reference's
Rust wrapper (``crates/mimo26-spark/src/b1.rs``): ``Layer``, ``Scratch``, ``ffn``,
``ffn_strided``, ``FfnStats``. There is no CPU path: importing the bindings without the
built library raises.
"""
from .expert import (  # noqa: F401
    Exchange,
    ExpertError,
    ExpertParallel,
    FfnStats,
    Layer,
    Scratch,
    ffn,
    ffn_dev,
    ffn_strided,
    ffn_tp,
    ffn_tp_dev,
    plan_static,
    produce_dev,
    quantize_dev,
    rank_sum_dev,
    route_reduce_dev,
    version,
)

HIDDEN = 4096
INTERMEDIATE = 2048
EXPERTS = 256
TOPK = 8
