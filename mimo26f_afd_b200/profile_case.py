"""A small, self-ending run of the expert FFN for profilers: builds the seeded layer, then runs `iters` passes of
`tokens` tokens on one GPU.

    python -m mimo26f_afd_b200.profile_case TOKENS [ZIPF_S] [ITERS]

Used as the command under `ncu` (see profiles/): capture with `-k regex:gemm_mx -s <2*(ITERS-1)> -c 2` to take the
FC1 and FC2 launches of the last pass."""
import sys, numpy as np, torch
sys.path.insert(0, __import__('os').path.dirname(__import__('os').path.dirname(__import__('os').path.abspath(__file__))))
import mimo26f_afd_b200 as M
from mimo26f_afd_b200 import synth, expert
T = int(sys.argv[1]); zipf = float(sys.argv[2]) if len(sys.argv) > 2 else 0.0; iters = int(sys.argv[3]) if len(sys.argv) > 3 else 3
seed = synth.MASTER_SEED
dev = torch.device('cuda:0')
W = synth.layer_torch(seed, dev)
L = M.Layer.from_checkpoint(*[W[n] for n in synth.TENSORS])
del W; torch.cuda.empty_cache()
S = M.Scratch()
st = torch.cuda.Stream(); torch.cuda.set_stream(st)
x_bits = synth.activations_bf16(seed, T); ids, wts = synth.routing(seed, T, zipf)
xd = torch.from_numpy(x_bits.view(np.int16)).to(dev); idd = torch.from_numpy(ids).to(dev); wd = torch.from_numpy(wts).to(dev)
out = torch.empty((T, 4096), dtype=torch.int16, device=dev)
for _ in range(iters):
    expert.ffn_dev(L, S, xd, idd, wd, T, out, stream=st.cuda_stream)
    S.status(st.cuda_stream)
print('done', T, S.peek('meta', np.uint32, (8,)))
