"""CPU baseline of the FFI train step: the PyTorch gather/einsum restatement, fp32, all host threads.

TEST / BENCHMARK INFRASTRUCTURE ONLY (timed by the benchmark's CPU-baseline legs; never imported by the
shipped package).  Same math as oracle/ffi_oracle.py:train_step — forward (shared_ffi/ffi_forward_kernels.cu:
167-262), loss gradient (src/runner.py:469-478 for BCE; this project's squared hinge), backward-features
(shared_ffi/ffi_backward_features.cu:134-212), backward-weights with bf16 rounding
(shared_ffi/ffi_backward_weights.cu:166-258, 81-89) and SGD + weight decay + stochastic rounding
(shared_ffi/sr_triton.py:109-168) — but in fp32 with torch's threaded kernels instead of fp64 sums, because
this one is measured, not used as the checker.
"""
import numpy as np
import torch

from . import philox as px
from .ffi_oracle import LOSS_BCE, LOSS_SQHINGE, _bits_to_bf16


def cpu_train_step(loc, X, W, bias, targets, G, loss_kind, lr, wd, seed, step, grad_scale=1.0, row0=0,
                   groups_per_chunk=128):
    """One step on CPU tensors.  W (bf16 [L,F]) and bias (bf16 [L]) are updated IN PLACE; returns (dX fp32 [B,D],
    loss float).  Works chunk by chunk over the label groups so the [B, labels] temporaries stay small."""
    B, D = X.shape
    L, F = W.shape
    NG = loc.shape[0]
    Xf = X.float()
    dX = torch.zeros(B, D, dtype=torch.float32)
    loss = 0.0
    tr, tc = targets[:, 0].long(), targets[:, 1].long()
    order = torch.argsort(tc)
    tr, tc = tr[order], tc[order]
    lr32, wd32 = np.float32(lr), np.float32(wd)
    for g0 in range(0, NG, groups_per_chunk):
        g1 = min(NG, g0 + groups_per_chunk)
        l0, l1 = g0 * G, min(L, g1 * G)
        n = l1 - l0
        npad = (g1 - g0) * G
        idx = loc[g0:g1].long()
        Xg = Xf[:, idx]                                                   # [B, ng, F]
        Wc = torch.zeros(npad, F)
        Wc[:n] = W[l0:l1].float()
        Wc = Wc.view(g1 - g0, G, F)
        Z = torch.einsum('bgf,gnf->bgn', Xg, Wc).reshape(B, npad)
        if bias is not None:
            Z[:, :n] += bias[l0:l1].float()
        Z = Z.to(torch.bfloat16).float()
        lo, hi = torch.searchsorted(tc, torch.tensor([l0, l1]))
        Y = torch.zeros(B, npad)
        Y[tr[lo:hi], tc[lo:hi] - l0] = 1.0
        if loss_kind == LOSS_BCE:
            loss += float((Z[:, :n].clamp(min=0) - Z[:, :n] * Y[:, :n] + torch.log1p(torch.exp(-Z[:, :n].abs()))).sum())
            dY = torch.sigmoid(Z) - Y
        else:
            s = 2.0 * Y - 1.0
            m = (1.0 - s * Z).clamp(min=0)
            loss += float((m[:, :n] * m[:, :n]).sum())
            dY = -2.0 * s * m
        dY = (dY * grad_scale).to(torch.bfloat16).float()
        dY[:, n:] = 0
        dYg = dY.view(B, g1 - g0, G)
        dW = torch.einsum('bgn,bgf->gnf', dYg, Xg).reshape(npad, F)[:n].to(torch.bfloat16).float()
        dXg = torch.einsum('bgn,gnf->bgf', dYg, Wc)
        dX.scatter_add_(1, idx.reshape(1, -1).expand(B, -1), dXg.reshape(B, -1))
        # SGD + wd (fused multiply-add emulated by fp64 here: measured path, not the checker) + SR, packed stream
        w32 = W[l0:l1].float().numpy()
        g32 = dW.numpy()
        g2 = (wd32 * w32.astype(np.float64) + g32).astype(np.float32)
        wn = (w32.astype(np.float64) - np.float64(lr32) * g2).astype(np.float32)
        rows = np.arange(l0, l1, dtype=np.int64)[:, None] + row0
        r16 = px.rand16_packed(seed, step, rows, np.arange(F, dtype=np.int64)[None, :])
        W[l0:l1] = _bits_to_bf16(px.sr_bf16_bits(wn, r16))
        if bias is not None:
            db = dY[:, :n].sum(0).to(torch.bfloat16).float().numpy()
            b32 = bias[l0:l1].float().numpy()
            bn = (b32.astype(np.float64) - np.float64(lr32) * (wd32 * b32.astype(np.float64) + db).astype(np.float32)).astype(np.float32)
            rb = px.rand16_packed(int(seed) ^ 0x62696173, step, rows[:, 0], np.zeros(n, np.int64))
            bias[l0:l1] = _bits_to_bf16(px.sr_bf16_bits(bn, rb))
    return dX, loss * grad_scale
