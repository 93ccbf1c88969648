"""Generate golden vectors for forward / backward-features / backward-weights from the REFERENCE's own CUDA kernels.

Run once on a machine with a GPU, after ``python oracle/build_ref.py <reference checkout>`` has built the
reference's extension into oracle/_ref/ (its wmma kernels run as legacy code on sm_100):

    python tests/golden/make_golden_gpu.py <output dir>

and copy the ``ref_gemm_*.npz`` files it writes into tests/golden/.  Each file holds the inputs (bit patterns for
bf16 tensors) and what the reference's ``ffi_forward_cuda``, ``ffi_backward_features_cuda`` and
``ffi_backward_weights_cuda`` (shared_ffi/ffi_wrapper.cpp:28-44) returned for them.

The reference supports group sizes 16/32/64 only, and (G=64, F=128) needs more than the 48 KB of dynamic shared
memory its launches may use (ffi_forward_kernels.cu:676-697, ffi_backward_features.cu:559-616).  For those cases
and for G=128 the reference runs at ``ref_gsize`` = 32 on an index table whose rows are repeated G/32 times — the
same mathematical layer (every label still reads the index row of its group).
Only inputs are used that the reference's index arithmetic handles: contiguous tensors, valid indices, B*L < 2^31.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import build_ref, ffi_oracle as fo  # noqa: E402

CASES = [  # name, B, D, L, F, G, gsize the reference runs at
    ("g32_f32", 48, 96, 173, 32, 32, 32),
    ("g64_f64", 64, 128, 130, 64, 64, 64),
    ("g16_f16", 40, 64, 75, 16, 16, 16),
    ("g32_f128", 72, 200, 257, 128, 32, 32),
    ("g128_f64", 128, 256, 300, 64, 128, 32),
    ("g64_f128", 130, 192, 201, 128, 64, 32),
]


def bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def reference_outputs(ref, loc, X, W, bias, dY, G, gsize):
    """Run the three reference kernels.  All tensors on the GPU; returns (Z bf16 [B,L], dXt fp32 [D,B], dW bf16 [L,F])."""
    B, D = X.shape
    L, F = W.shape
    loc_ref = loc if gsize == G else loc.repeat_interleave(G // gsize, 0).contiguous()
    xt = X.t().contiguous()
    z = ref.ffi_forward_cuda(loc_ref, xt, W, bias, B, D, F, L, gsize)
    dxt = ref.ffi_backward_features_cuda(xt, W, loc_ref, dY, B, D, F, L, gsize)
    dw = ref.ffi_backward_weights_cuda(xt, W, loc_ref, dY, B, D, F, L, gsize)
    torch.cuda.synchronize()
    return z.contiguous(), dxt, dw


def main(out_dir):
    ref = build_ref.load()
    if ref is None:
        raise SystemExit("oracle/_ref is not built: run oracle/build_ref.py first")
    os.makedirs(out_dir, exist_ok=True)
    for name, B, D, L, F, G, gsize in CASES:
        assert B * L < 2 ** 31
        inp = fo.make_inputs(B, D, L, F, G, 3, 1.1, seed=1000 + L, x_kind="normal", bias_zero=False)
        gen = torch.Generator().manual_seed(L)
        dY = (torch.randn(B, L, generator=gen) * 0.5).to(torch.bfloat16)
        assert D >= F and tuple(inp["loc"].shape) == ((L + G - 1) // G, F), "index table must be [NG,F] (needs D >= F)"
        dev = {k: inp[k].cuda() for k in ("loc", "X", "W", "bias")}
        z, dxt, dw = reference_outputs(ref, dev["loc"], dev["X"], dev["W"], dev["bias"], dY.cuda(), G, gsize)
        # how the CPU restatement compares (informational; the tests assert it)
        z_o = fo.forward(inp["loc"], inp["X"], inp["W"], inp["bias"], G, round_bf16=True)
        dw_o = fo.backward_weights(inp["loc"], inp["X"], dY, G, L, round_bf16=True)
        dx_o = fo.backward_features(inp["loc"], inp["W"], dY, G, D)
        print(f"{name}: Z identical {float((bits(z) == bits(z_o)).mean()):.4f}  dW identical {float((bits(dw) == bits(dw_o)).mean()):.4f}  "
              f"dXt max err {float((dxt.cpu() - dx_o).abs().max()):.3e} of {float(dx_o.abs().max()):.3e}", flush=True)
        np.savez_compressed(os.path.join(out_dir, f"ref_gemm_{name}.npz"), B=B, D=D, L=L, F=F, G=G, ref_gsize=gsize,
                            loc=inp["loc"].numpy(), X=bits(inp["X"]), W=bits(inp["W"]), bias=bits(inp["bias"]), dY=bits(dY),
                            Z=bits(z), dXt=dxt.cpu().numpy(), dW=bits(dw))


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
