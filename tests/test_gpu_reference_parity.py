"""Parity of the tensor-core kernels with the REFERENCE's own CUDA kernels (forward, backward-features,
backward-weights), through the C ABI.

Two sources of reference results:
  * tests/golden/ref_gemm_*.npz — outputs of the reference's kernels, produced once on a B200 by
    tests/golden/make_golden_gpu.py; always checked.
  * the reference's extension itself, when oracle/_ref/ holds a build of it (oracle/build_ref.py); then the same
    seeded inputs go through both implementations on this GPU, at small ragged shapes, at the full size of the
    CPU-runnable benchmark configuration and at slices of the larger ones.  Skipped when the build is absent.

Tolerance (bf16 inputs, fp32 accumulation, the two implementations sum in different orders): rel 1e-2 plus abs 1e-3
of the tensor's magnitude.  Reference limits respected: group size 16/32/64 (G=128 and (64,128) run as G=32 on an
index table with repeated rows — the same layer), B*L < 2^31, valid indices, contiguous tensors.
"""
import glob
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import build_ref
from oracle import ffi_oracle as fo

REL, ABS = 1e-2, 1e-3
GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_gemm_*.npz")))


@pytest.fixture(scope="module")
def ffi():
    import haste_b200.ffi as ffi
    return ffi


@pytest.fixture(scope="module")
def ref():
    m = build_ref.load()
    if m is None:
        pytest.skip("the reference extension is not built under oracle/_ref")
    return m


def _close(got, want, what):
    got, want = got.float().cpu(), want.float().cpu()
    tol = ABS * max(1.0, float(want.abs().max())) + REL * want.abs()
    bad = (got - want).abs() > tol
    assert not bad.any(), f"{what}: {int(bad.sum())}/{bad.numel()} outside tolerance, max err {float((got - want).abs().max())}"


def _bf16(bits):
    return fo._bits_to_bf16(bits)


def test_golden_files_present():
    assert len(GOLDEN) >= 6, "reference-generated fixtures tests/golden/ref_gemm_*.npz are missing"


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[9:-4] for p in GOLDEN])
def test_kernels_match_reference_golden(ffi, path):
    d = np.load(path)
    G = int(d["G"])
    loc = torch.from_numpy(d["loc"]).cuda()
    X, W, bias, dY = (_bf16(d[k]).cuda() for k in ("X", "W", "bias", "dY"))
    xt = X.t().contiguous()
    _close(ffi.forward(loc, xt, W, bias, G), _bf16(d["Z"]), "forward")
    _close(ffi.backward_features(xt, W, loc, dY, G), torch.from_numpy(d["dXt"]), "backward-features")
    dw, _ = ffi.backward_weights(xt, W, loc, dY, G, want_dbias=True)
    _close(dw, _bf16(d["dW"]), "backward-weights")
    dxt2, dw2, _ = ffi.backward_both(xt, W, loc, dY, G)
    _close(dxt2, torch.from_numpy(d["dXt"]), "backward (both), dXt")
    _close(dw2, _bf16(d["dW"]), "backward (both), dW")


def _ref_run(ref, loc, xt, W, bias, dY, G):
    """The reference's three kernels on GPU tensors.  G outside its supported set, or (64,128), runs as G=32 with
    repeated index rows."""
    D, B = xt.shape
    L, F = W.shape
    assert B * L < 2 ** 31 and tuple(loc.shape) == ((L + G - 1) // G, F) and int(loc.max()) < D
    gs = G if (G in (16, 32, 64) and not (G == 64 and F == 128)) else 32
    loc_r = loc if gs == G else loc.repeat_interleave(G // gs, 0).contiguous()
    torch.cuda.synchronize()                # the reference launches on the legacy default stream
    if dY is None:
        z = ref.ffi_forward_cuda(loc_r, xt, W, bias, B, D, F, L, gs)
        torch.cuda.synchronize()
        return z
    dxt = ref.ffi_backward_features_cuda(xt, W, loc_r, dY, B, D, F, L, gs)
    dw = ref.ffi_backward_weights_cuda(xt, W, loc_r, dY, B, D, F, L, gs)
    torch.cuda.synchronize()
    return dxt, dw


LIVE = [  # B, D, L, F, G, x_kind
    (64, 768, 1000, 32, 32, "normal"),
    (130, 96, 300, 16, 16, "normal"),
    (200, 256, 1111, 64, 128, "normal"),
    (256, 512, 777, 128, 64, "normal"),
    (96, 200, 500, 48, 32, "normal"),
    (257, 128, 130, 96, 64, "normal"),
    (64, 768, 30938, 32, 32, "normal"),        # benchmark configuration 1 at full size
    (512, 768, 16385, 128, 64, "l2norm"),      # configuration 2, label slice with a ragged last group
    (512, 768, 20011, 64, 128, "l2norm"),      # configuration 3 (the headline shape), label slice
    (256, 4096, 12006, 128, 64, "relu"),       # configuration 4, label slice
    (1024, 768, 20009, 64, 128, "l2norm"),     # configuration 5, label slice
]


@pytest.mark.parametrize("case", LIVE, ids=[f"B{c[0]}_D{c[1]}_L{c[2]}_F{c[3]}_G{c[4]}" for c in LIVE])
def test_kernels_match_reference_live(ffi, ref, case):
    B, D, L, F, G, xk = case
    inp = fo.make_inputs(B, D, L, F, G, 3, 1.1, seed=L, x_kind=xk, bias_zero=False)
    loc, X, W, bias = (inp[k].cuda() for k in ("loc", "X", "W", "bias"))
    xt = X.t().contiguous()
    z_ref = _ref_run(ref, loc, xt, W, bias, None, G)
    z = ffi.forward(loc, xt, W, bias, G)
    _close(z, z_ref, "forward")
    # the gradient fed to both backwards: the BCE gradient of the reference's own logits, so that it has the value
    # distribution of training (most entries near sigmoid(z), a few near sigmoid(z) - 1)
    Y = torch.zeros(B, L, device="cuda")
    t = inp["targets"].cuda().long()
    Y[t[:, 0], t[:, 1]] = 1.0
    dY = (torch.sigmoid(z_ref.float()) - Y).to(torch.bfloat16).contiguous()
    dxt_ref, dw_ref = _ref_run(ref, loc, xt, W, bias, dY, G)
    _close(ffi.backward_features(xt, W, loc, dY, G), dxt_ref, "backward-features")
    dw, _ = ffi.backward_weights(xt, W, loc, dY, G, want_dbias=True)
    _close(dw, dw_ref, "backward-weights")
    dxt2, dw2, _ = ffi.backward_both(xt, W, loc, dY, G)
    _close(dxt2, dxt_ref, "backward (both), dXt")
    _close(dw2, dw_ref, "backward (both), dW")


@pytest.mark.parametrize("case", [(512, 768, 20011, "squared_hinge"), (1024, 768, 20009, "bce"), (200, 256, 1111, "bce")])
def test_fused_step_matches_reference_kernels(ffi, ref, case):
    """The fused tcgen05 step (G=128, F=64) against the reference's three kernels: the logits it formed against the
    reference forward; the weight / bias gradients it consumed and the dX it produced against the reference
    backwards fed with the loss gradient of the kernel's own logits (so the comparison isolates the products)."""
    import haste_b200._lib as lib
    B, D, L, loss = case
    F, G = 64, 128
    inp = fo.make_inputs(B, D, L, F, G, 6, 1.1, seed=L + 5, x_kind="l2norm", bias_zero=False)
    loc, X, W, bias, coo = (inp[k].cuda() for k in ("loc", "X", "W", "bias", "targets"))
    xt = X.t().contiguous()
    NG = (L + G - 1) // G
    ptr = torch.zeros(NG + 1, dtype=torch.int32, device="cuda")
    ent = torch.zeros(max(1, coo.shape[0]), dtype=torch.int32, device="cuda")
    ffi.targets_bucket(coo, 0, L, G, ptr, ent, torch.zeros(NG, dtype=torch.int32, device="cuda"))
    kind = lib.LOSS_SQHINGE if loss == "squared_hinge" else lib.LOSS_BCE
    w2, b2 = W.clone(), bias.clone()
    dxt = torch.empty(D, B, dtype=torch.float32, device="cuda")
    lbuf = torch.zeros(1, dtype=torch.float32, device="cuda")
    flags = ffi.make_flags(sr=True, contract=True, rng="packed", zero_dxt=True, loss=True)
    z, dw, db = ffi.train_step_dbg(loc, xt, w2, b2, ptr, ent, dxt, lbuf, G, 0, kind, 1.0, 0.05, 1e-4, 123, 0, flags)
    torch.cuda.synchronize()
    _close(z, _ref_run(ref, loc, xt, W, bias, None, G), "fused step logits")
    _, dY = fo.loss_and_grad(z.cpu(), inp["targets"], fo.LOSS_SQHINGE if loss == "squared_hinge" else fo.LOSS_BCE, 1.0)
    dxt_ref, dw_ref = _ref_run(ref, loc, xt, W, bias, dY.cuda().contiguous(), G)
    # BCE: the kernel's sigmoid is tanh.approx-based, its bf16 gradient may differ from the exact one by a step
    k = 2.0 if loss == "bce" else 1.0
    got, want = dw.float().cpu(), dw_ref.float().cpu()
    assert not ((got - want).abs() > k * (ABS * max(1.0, float(want.abs().max())) + REL * want.abs())).any(), "fused step dW"
    got, want = dxt.cpu(), dxt_ref.cpu()
    assert not ((got - want).abs() > k * (ABS * max(1.0, float(want.abs().max())) + REL * want.abs())).any(), "fused step dXt"
