"""Writes tests/golden/topk_cuda_ties.npz: what torch.topk returns ON A CUDA DEVICE for inputs
full of ties.  Needs a GPU (the tie order of torch.topk differs between its CPU and CUDA
kernels, and the engine runs on CUDA).  Run on a B200 with torch 2.11:

    python tests/golden/make_topk_tie_fixture.py [out.npz]

Inputs are small integers (alphabet of 1, 3 or 12 values), so every dtype holds them exactly.
"""
import sys
from pathlib import Path

import numpy as np
import torch

out = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).resolve().parent / "topk_cuda_ties.npz"
res = {}
for dtype, dn in ((torch.bfloat16, "bf16"), (torch.float32, "f32"), (torch.float16, "f16")):
    for (E, K) in ((8, 2), (128, 8), (64, 4), (16, 4), (256, 8), (128, 1), (60, 4), (8, 8), (32, 32), (64, 6)):
        for T in (7, 300):
            for alphabet in (1, 3, 12):
                g = torch.Generator().manual_seed(1234 + E * 7 + K * 3 + T)
                v = torch.randint(0, alphabet, (T, E), generator=g).to(torch.float32)
                _, idx = torch.topk(v.to("cuda").to(dtype), K, dim=-1)
                tag = f"{dn}_E{E}_K{K}_T{T}_A{alphabet}"
                res[tag + "_in"] = v[:16].numpy().astype(np.int8)
                res[tag + "_idx"] = idx[:16].cpu().numpy().astype(np.int16)
np.savez_compressed(out, **res)
print("wrote", out, len(res) // 2, "cases")
