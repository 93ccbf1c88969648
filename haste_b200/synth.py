"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configurations.

The XMC datasets whose shapes these borrow are not reproduced: features are Gaussian (optionally L2-normalised
or rectified), weights uniform in +-1/sqrt(fan_in), index rows are distinct uniform draws sorted ascending, and
targets are multi-hot rows whose label ids follow a Zipf law over label rank.
"""
import math

import numpy as np
import torch

WORKLOADS = {
    # name: B, D, L, F, G, avg positives, zipf exponent, features, loss
    "c1": dict(B=64, D=768, L=30938, F=32, G=32, avg_pos=19.0, zipf=1.1, x="normal", loss="bce"),
    "c2": dict(B=512, D=768, L=131073, F=128, G=64, avg_pos=5.4, zipf=1.1, x="l2norm", loss="bce"),
    "c3": dict(B=512, D=768, L=670091, F=64, G=128, avg_pos=5.5, zipf=1.0, x="l2norm", loss="squared_hinge"),
    "c4": dict(B=256, D=4096, L=501070, F=128, G=64, avg_pos=4.8, zipf=1.1, x="relu", loss="bce"),
    "c5": dict(B=1024, D=768, L=2812281, F=64, G=128, avg_pos=36.0, zipf=1.2, x="l2norm", loss="bce"),
}


def make_layer(D, L, F, G, seed=42):
    """(loc int32 [NG,F], W bf16 [L,F], bias bf16 [L]) on the CPU."""
    gen = torch.Generator().manual_seed(seed)
    NG = (L + G - 1) // G
    keys = torch.rand(NG, D, generator=gen)
    loc = keys.topk(F, dim=1).indices.sort(dim=1).values.to(torch.int32)
    bound = 1.0 / math.sqrt(F)
    W = ((torch.rand(L, F, generator=gen) * 2 - 1) * bound).to(torch.bfloat16)
    bias = torch.zeros(L, dtype=torch.bfloat16)
    return loc, W, bias


def make_batch(B, D, L, avg_pos, zipf, x_kind, seed):
    """(X bf16 [B,D], targets int32 [nnz,2] of (row, label)) on the CPU."""
    gen = torch.Generator().manual_seed(seed)
    X = torch.randn(B, D, generator=gen)
    if x_kind == "l2norm":
        X = X / X.norm(dim=1, keepdim=True)
    elif x_kind == "relu":
        X = X.clamp(min=0)
    X = X.to(torch.bfloat16)
    rs = np.random.RandomState(seed)
    p = 1.0 / np.arange(1, L + 1, dtype=np.float64) ** zipf
    cdf = np.cumsum(p)
    cdf /= cdf[-1]
    npos = np.maximum(1, rs.poisson(avg_pos, size=B))
    rows, cols = [], []
    for b in range(B):
        want = int(npos[b])
        draw = np.minimum(np.searchsorted(cdf, rs.rand(want * 4 + 8)), L - 1)
        _, first = np.unique(draw, return_index=True)
        picked = np.sort(draw[np.sort(first)][:want])
        rows.append(np.full(len(picked), b, np.int32))
        cols.append(picked.astype(np.int32))
    tg = torch.from_numpy(np.stack([np.concatenate(rows), np.concatenate(cols)], 1).astype(np.int32))
    return X, tg
