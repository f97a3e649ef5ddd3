"""One launch (three, the first two as warm-up) of the tcgen05 prefill attention on random q/k/v of a 2,048-token
prompt with the 7B head shapes: the small workload on which this kernel is profiled.  Not a test."""
import sys, os
sys.path.insert(0, os.getcwd())
import torch
from types import SimpleNamespace
from cima_b200.kernels import Kernels
K = Kernels(verbose=False)
dev = "cuda"
nh, nkv, hd = 28, 4, 128
lens = [2048]
T = sum(lens)
qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=dev, dtype=torch.bfloat16)
out = torch.empty(T, nh * hd, device=dev, dtype=torch.bfloat16)
t32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
tiles = sorted(((i, r0) for i, n in enumerate(lens) for r0 in range(0, n, 128)), key=lambda x: -x[1])
b = SimpleNamespace(n_q_tiles_tc=len(tiles), q_tile_tc_seq=t32([x[0] for x in tiles]), q_tile_tc_row0=t32([x[1] for x in tiles]),
                    seq_first_row=t32([0, T]))
for _ in range(3):
    K.attention_prefill_tc(qkv, b, out, nh, nkv, hd, 0.088, 0)
torch.cuda.synchronize()
print("ok", K.device_errors())
