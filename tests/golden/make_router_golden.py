"""Generate tests/golden/router_vectors.npz by RUNNING THE REFERENCE's router (oracle/mimo26/nn/layers.py::router,
the Python twin of crates/mimo26-coordinator/src/router.rs:42-80).

    python tests/golden/make_router_golden.py [REFERENCE_TREE]

The reference function takes activations and a router matrix; an identity matrix makes its FP32 logits equal the
activations bit for bit (each dot product has one nonzero term), so the stored logits are exactly what it scored.
Logits are seeded N(0, 2); the selection bias is N(0, 0.05) as FP32 (`e_score_correction_bias`). No exact ties occur in
this data (the tie rule, lower expert id first, exists only in the Rust and is tested separately)."""
import os
import sys

import numpy as np

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("M26B_REFERENCE_TREE", "")
if not REF:
    raise SystemExit("usage: make_router_golden.py REFERENCE_TREE   (or set M26B_REFERENCE_TREE)")
HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path = [p for p in sys.path if os.path.abspath(p or ".") != REPO]
sys.path.insert(0, REF)

from oracle.mimo26.nn.layers import router  # noqa: E402  (reference)


def main():
    rng = np.random.default_rng(0x26AFD)
    tokens, experts, top_k = 96, 256, 8
    logits = (rng.standard_normal((tokens, experts)) * 2.0).astype(np.float32)
    logits[0] *= 8.0           # saturated sigmoids
    logits[1] *= 0.01          # all scores near 1/2: selection decided by the bias
    bias = (rng.standard_normal(experts) * 0.05).astype(np.float32)
    idx, wts = router(logits, np.eye(experts, dtype=np.float32), top_k=top_k, bias=bias)
    idx0, wts0 = router(logits, np.eye(experts, dtype=np.float32), top_k=top_k, bias=None)
    np.savez_compressed(os.path.join(HERE, "router_vectors.npz"), logits_bits=logits.view(np.uint32), bias_bits=bias.view(np.uint32),
                        idx=idx.astype(np.int32), weight_bits=wts.view(np.uint32), idx_nobias=idx0.astype(np.int32),
                        weight_nobias_bits=wts0.view(np.uint32))
    print("router goldens:", idx.shape, wts.dtype)


if __name__ == "__main__":
    main()
