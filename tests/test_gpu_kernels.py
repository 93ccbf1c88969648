"""GPU parity tests: every kernel is called through the C ABI (ctypes) and compared with the CPU oracle on
the same seeded inputs.  Integer / bit-pattern results must be identical; floating-point results use the
tolerances stated next to each check (logits and dX: rel 1e-2 / abs 1e-3 on bf16 inputs with fp32
accumulation)."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import ffi_oracle as fo
from oracle import philox as px

REL, ABS = 1e-2, 1e-3

SHAPES = [  # B, D, L, F, G
    (64, 768, 1000, 32, 32),
    (130, 96, 300, 16, 16),
    (200, 256, 1111, 64, 128),
    (256, 512, 777, 128, 64),
    (96, 200, 500, 48, 32),
    (33, 64, 40, 16, 128),
    (257, 128, 130, 96, 64),
]


@pytest.fixture(scope="module")
def hb():
    import haste_b200.ffi as ffi
    import haste_b200._lib as lib
    assert torch.cuda.is_available()
    return ffi, lib


def _inputs(B, D, L, F, G, seed=42, bias_zero=False, avg_pos=4):
    inp = fo.make_inputs(B, D, L, F, G, avg_pos, 1.1, seed=seed, x_kind="normal", bias_zero=bias_zero)
    dev = {k: v.cuda() for k, v in inp.items()}
    dev["Xt"] = dev["X"].t().contiguous()
    return inp, dev


def _bits(t):
    return fo._bf16_to_bits(t.detach().cpu())


def _ulp_bf16(x):
    x = np.abs(np.asarray(x, np.float32))
    e = np.floor(np.log2(np.maximum(x, 1e-30)))
    return np.exp2(e - 7).astype(np.float32)


def _assert_close(got, want, rel=REL, abs_=ABS, what=""):
    got, want = got.float().cpu(), want.float().cpu()
    err = (got - want).abs()
    tol = abs_ + rel * want.abs()
    bad = (err > tol)
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} outside tolerance, max err {float(err.max())}"


def _assert_bf16_ulp(got_bits, want_bits, max_ulp=2, max_frac=0.05, what="", extra_abs=0.0):
    """Bit patterns may differ in at most ``max_frac`` of the elements, and then by at most ``max_ulp`` bf16
    steps of the value plus ``extra_abs`` (array or scalar: the effect of a one-step difference in an input)."""
    g = px.bf16_bits_to_f32(got_bits).astype(np.float64)
    w = px.bf16_bits_to_f32(want_bits).astype(np.float64)
    neq = got_bits != want_bits
    frac = neq.mean()
    assert frac <= max_frac, f"{what}: {frac:.4f} of elements differ"
    if neq.any():
        tol = max_ulp * _ulp_bf16(w) + extra_abs
        over = (np.abs(g - w) - tol)[neq]
        assert over.max() <= 1e-12, f"{what}: a difference exceeds its tolerance by {over.max()}"


# ------------------------------------------------------------------------------------------------ GEMM phases
@pytest.mark.parametrize("shape", SHAPES)
def test_forward(hb, shape):
    ffi, _ = hb
    B, D, L, F, G = shape
    inp, dev = _inputs(*shape)
    z = ffi.forward(dev["loc"], dev["Xt"], dev["W"], dev["bias"], G)
    assert z.shape == (B, L)
    want = fo.forward(inp["loc"], inp["X"], inp["W"], inp["bias"], G, round_bf16=False)
    _assert_close(z, want, what="forward")
    # padding columns of the underlying buffer are exact zeros, as in the reference
    ldz = (L + 7) // 8 * 8
    if ldz > L:
        full = torch.as_strided(z, (B, ldz), (ldz, 1))
        assert (full[:, L:] == 0).all()
    z2 = ffi.forward(dev["loc"], dev["Xt"], dev["W"], None, G)
    _assert_close(z2, fo.forward(inp["loc"], inp["X"], inp["W"], None, G, round_bf16=False), what="forward nobias")


@pytest.mark.parametrize("shape", [(384, 512, 128 * 300 + 5, 64, 128), (264, 1024, 64 * 400 + 3, 128, 64)])
def test_forward_many_groups(hb, shape):
    """More label groups than SMs and several batch tiles per group, so that every ring of the persistent tcgen05
    forward wraps several times; ragged last group and ragged last batch tile; also into a column block of a
    wider buffer, where nothing outside the block may change."""
    ffi, _ = hb
    B, D, L, F, G = shape
    inp, dev = _inputs(*shape)
    want = fo.forward(inp["loc"], inp["X"], inp["W"], inp["bias"], G, round_bf16=False)
    z = ffi.forward(dev["loc"], dev["Xt"], dev["W"], dev["bias"], G)
    _assert_close(z, want, what="forward")
    ldz = (L + 7) // 8 * 8
    assert (torch.as_strided(z, (B, ldz), (ldz, 1))[:, L:] == 0).all()
    out = torch.full((B, (L + 31) // 8 * 8), 7.0, dtype=torch.bfloat16, device="cuda")     # row stride a multiple of 16 bytes
    ffi.forward_into(dev["loc"], dev["Xt"], dev["W"], dev["bias"], G, out, 16)
    assert torch.equal(out[:, 16:16 + L], z)
    assert (out[:, :16] == 7).all() and (out[:, 16 + L:] == 7).all()


@pytest.mark.parametrize("shape", [(384, 512, 128 * 300 + 5, 64, 128), (264, 1024, 64 * 400 + 3, 128, 64),
                                   (200, 256, 128 * 9 + 70, 64, 128), (136, 256, 64 * 11 + 6, 128, 64)])
def test_backward_one_pass_unaligned_rows(hb, shape):
    """The one-pass tcgen05 backward reads gradient rows at any 2-byte alignment: contiguous [B, L] with odd L (every
    row starts at a different offset inside a 16-byte granule), a column slice of a wider buffer that starts at an odd
    column, and aligned rows.  The memory right of every row's L columns holds NaN: nothing of it may leak into a
    result (the last group's tile covers columns beyond L)."""
    ffi, _ = hb
    B, D, L, F, G = shape
    inp, dev = _inputs(*shape)
    g = torch.Generator().manual_seed(5)
    dY = (torch.randn(B, L, generator=g) * 0.5).to(torch.bfloat16)
    want_x = fo.backward_features(inp["loc"], inp["W"], dY, G, D)
    want_w = fo.backward_weights(inp["loc"], inp["X"], dY, G, L, round_bf16=False)
    variants = {"contiguous": dY.cuda()}
    for name, (left, width) in {"odd column offset": (3, L + 3 + 6), "aligned rows": (8, (L + 8 + 15) // 8 * 8),
                                "even column offset": (2, L + 2 + 4)}.items():
        buf = torch.full((B, width), float("nan"), dtype=torch.bfloat16, device="cuda")
        buf[:, left:left + L] = dY.cuda()
        variants[name] = buf[:, left:left + L]
    results = {}
    for name, dy_dev in variants.items():
        dxt, dw, db = ffi.backward_both(dev["Xt"], dev["W"], dev["loc"], dy_dev, G)
        assert torch.isfinite(dxt).all() and torch.isfinite(dw.float()).all() and torch.isfinite(db.float()).all(), name
        _assert_close(dxt, want_x, rel=1e-2, abs_=1e-3 * max(1.0, float(want_x.abs().max())), what=f"dXt ({name})")
        _assert_close(dw, want_w, rel=1e-2, abs_=1e-3 * max(1.0, float(want_w.abs().max())), what=f"dW ({name})")
        _assert_close(db, dY.float().sum(0), rel=1e-2, abs_=2e-2, what=f"dbias ({name})")
        results[name] = (dw, db)
    # the weight and bias gradients do not depend on where the rows lie in memory (dxt is reduced with atomics)
    for name, (dw, db) in results.items():
        assert torch.equal(dw, results["contiguous"][0]) and torch.equal(db, results["contiguous"][1]), name


@pytest.mark.parametrize("shape", SHAPES)
def test_backward_features_and_weights(hb, shape):
    ffi, _ = hb
    B, D, L, F, G = shape
    inp, dev = _inputs(*shape)
    g = torch.Generator().manual_seed(1)
    dY = (torch.randn(B, L, generator=g) * 0.5).to(torch.bfloat16)
    for dy_dev in (dY.cuda(), torch.nn.functional.pad(dY, (0, 5)).cuda()[:, :L]):   # contiguous and padded rows
        dxt = ffi.backward_features(dev["Xt"], dev["W"], dev["loc"], dy_dev, G)
        want = fo.backward_features(inp["loc"], inp["W"], dY, G, D)
        _assert_close(dxt, want, rel=1e-2, abs_=1e-3 * max(1.0, float(want.abs().max())), what="bwd features")
        dw, db = ffi.backward_weights(dev["Xt"], dev["W"], dev["loc"], dy_dev, G, want_dbias=True)
        want_w = fo.backward_weights(inp["loc"], inp["X"], dY, G, L, round_bf16=False)
        _assert_close(dw, want_w, rel=1e-2, abs_=1e-3 * max(1.0, float(want_w.abs().max())), what="bwd weights")
        _assert_close(db, dY.float().sum(0), rel=1e-2, abs_=2e-2, what="bias grad")


# ------------------------------------------------------------------------------------------------ SR / SGD
def test_sr_round_golden(hb, golden_dir):
    ffi, _ = hb
    for seed in (123, 124, 2147483643):
        z = np.load(os.path.join(golden_dir, f"sr_round_seed{seed}.npz"))
        x = torch.from_numpy(z["x"]).cuda()
        out = torch.empty(x.shape, dtype=torch.bfloat16, device="cuda")
        ffi.sr_round(x, out, int(z["seed"]))
        assert np.array_equal(_bits(out), z["out"])


@pytest.mark.parametrize("name", ["wd", "mom", "rn", "mom_off"])
def test_sgd_update_golden(hb, golden_dir, name):
    """Bit-exact against the reference's Triton kernel (run in the interpreter, which keeps mul and add
    separate -> contract=False; its non-SR cast truncates, so 'rn' is checked against the oracle instead)."""
    ffi, _ = hb
    z = np.load(os.path.join(golden_dir, f"sgd_{name}.npz"))
    w = fo._bits_to_bf16(z["w"]).cuda()
    g = fo._bits_to_bf16(z["g"]).cuda()
    m = torch.from_numpy(z["m"].copy()).cuda()
    use_mom = bool(z["use_mom"]) and float(z["mu"]) != 0.0
    flags = ffi.make_flags(sr=bool(z["do_sr"]), contract=False, rng="reference")
    ffi.sgd_sr_update(w, g, m if use_mom else None, 0, float(z["lr"]), float(z["wd"]), float(z["mu"]) if use_mom else 0.0,
                      int(z["seed"]), 0, flags)
    if name == "rn":
        w32, _ = fo.sgd_math(fo._bits_to_bf16(z["w"]).float().numpy(), fo._bits_to_bf16(z["g"]).float().numpy(), None,
                             float(z["lr"]), float(z["wd"]), 0.0, False, False)
        assert np.array_equal(_bits(w), px.rn_bf16_bits(w32))
    else:
        assert np.array_equal(_bits(w), z["w_out"])
    assert np.array_equal(m.cpu().numpy(), z["m_out"])


@pytest.mark.parametrize("rng", ["reference", "packed"])
@pytest.mark.parametrize("contract", [True, False])
@pytest.mark.parametrize("shape", [(1000, 64), (333, 24), (77, 1), (50, 128)])
def test_sgd_update_oracle(hb, rng, contract, shape):
    ffi, _ = hb
    gen = torch.Generator().manual_seed(3)
    w = ((torch.rand(*shape, generator=gen) * 2 - 1) / 8).to(torch.bfloat16)
    g = (torch.randn(*shape, generator=gen) * 0.2).to(torch.bfloat16)
    m = torch.randn(*shape, generator=gen) * 0.1
    row0, seed, step = 5000, 777, 9
    for mu in (0.0, 0.9):
        r = fo.rand16_for(shape, seed, step, rng, row0)
        want_w, want_m = fo.sgd_update(w, g, m, 0.05, 1e-4, mu, True, True, r, contract=contract)
        wd_, md = w.clone().cuda(), m.clone().cuda()
        ffi.sgd_sr_update(wd_, g.cuda(), md if mu else None, row0, 0.05, 1e-4, mu, seed, step,
                          ffi.make_flags(sr=True, contract=contract, rng=rng))
        assert np.array_equal(_bits(wd_), fo._bf16_to_bits(want_w)), (rng, contract, mu)
        if mu:
            assert np.array_equal(md.cpu().numpy(), want_m.numpy())


def test_sr_unbiased_gpu(hb):
    """E[round(w)] = w within 3 sigma over 10^6 draws (both random streams), measured on the device."""
    ffi, _ = hb
    n, w0 = 1_000_000, 0.1234567
    for rng in ("reference", "packed"):
        g = torch.full((n // 64, 64), -w0, dtype=torch.float32, device="cuda").to(torch.bfloat16)
        # w_new32 = 0 - 0.777 * g: an fp32 value off the bf16 grid, rounded stochastically
        w = torch.zeros(n // 64, 64, dtype=torch.bfloat16, device="cuda")
        ffi.sgd_sr_update(w, g, None, 0, 0.777, 0.0, 0.0, 99, 3, ffi.make_flags(sr=True, contract=True, rng=rng))
        t32 = np.float32(-np.float32(0.777) * np.float32(float(g[0, 0].float())))
        vals = w.float().double().cpu().numpy().ravel()
        lo, hi = vals.min(), vals.max()
        assert lo < float(t32) < hi
        p = (float(t32) - lo) / (hi - lo)
        sigma = (hi - lo) * np.sqrt(p * (1 - p) / n)
        assert abs(vals.mean() - float(t32)) < 3 * sigma, rng


def test_dxt_to_dx_and_transpose(hb):
    ffi, _ = hb
    gen = torch.Generator().manual_seed(5)
    dxt = torch.randn(70, 45, generator=gen)
    dx = ffi.dxt_to_dx_sr(dxt.cuda(), 123)
    want = fo.stochastic_rounding(dxt.t().contiguous(), 123)
    assert np.array_equal(_bits(dx), fo._bf16_to_bits(want))
    x = torch.randn(45, 70, generator=gen).to(torch.bfloat16)
    assert torch.equal(ffi.transpose_bf16(x.cuda()).cpu(), x.t().contiguous())


# ------------------------------------------------------------------------------------------------ targets
def test_targets_bucket(hb):
    ffi, _ = hb
    B, L, G = 300, 5000, 64
    inp = fo.make_inputs(B, 64, L, 16, G, 12, 1.1, seed=9)
    coo = inp["targets"].cuda()
    for label0, Ls in ((0, L), (1024, 2000)):
        NG = (Ls + G - 1) // G
        ptr = torch.zeros(NG + 1, dtype=torch.int32, device="cuda")
        ent = torch.zeros(coo.shape[0], dtype=torch.int32, device="cuda")
        scratch = torch.zeros(NG, dtype=torch.int32, device="cuda")
        ffi.targets_bucket(coo, label0, Ls, G, ptr, ent, scratch)
        ptr_h, ent_h = ptr.cpu().numpy(), ent.cpu().numpy().view(np.uint32)
        t = inp["targets"].numpy()
        keep = (t[:, 1] >= label0) & (t[:, 1] < label0 + Ls)
        t = t[keep]
        assert ptr_h[0] == 0 and ptr_h[-1] == len(t)
        got = set()
        for g in range(NG):
            for e in ent_h[ptr_h[g]:ptr_h[g + 1]]:
                got.add((int(e >> 8), g * G + int(e & 0xFF) + label0))
        assert got == set((int(r), int(c)) for r, c in t)


# ------------------------------------------------------------------------------------------------ fused paths
@pytest.mark.parametrize("shape", [(64, 768, 1000, 32, 32), (200, 256, 1111, 64, 128), (256, 512, 777, 128, 64),
                                   (130, 96, 300, 16, 16)])
@pytest.mark.parametrize("rng", ["reference", "packed"])
def test_bww_sr_sgd_bit_exact(hb, shape, rng):
    """Fused backward-weights + update == (unfused backward-weights kernel -> oracle SGD/SR), bit for bit."""
    ffi, _ = hb
    B, D, L, F, G = shape
    inp, dev = _inputs(*shape)
    gen = torch.Generator().manual_seed(2)
    dY = (torch.randn(B, L, generator=gen) * 0.3).to(torch.bfloat16)
    dw, db = ffi.backward_weights(dev["Xt"], dev["W"], dev["loc"], dY.cuda(), G, want_dbias=True)
    label0, seed, step, lr, wd = 640, 123, 4, 0.05, 1e-4
    for mu in (0.0, 0.9):
        mom = torch.randn(L, F, generator=gen) * 0.01
        momb = torch.randn(L, generator=gen) * 0.01
        want_w, want_m = fo.sgd_update(inp["W"], dw.cpu(), mom, lr, wd, mu, True, True,
                                       fo.rand16_for((L, F), seed, step, rng, label0))
        want_b, want_mb = fo.sgd_update(inp["bias"], db.cpu(), momb, lr, wd, mu, True, True,
                                        fo.rand16_for((L, 1), seed, step, rng, label0, is_bias=True).reshape(L))
        w, b = dev["W"].clone(), dev["bias"].clone()
        md, mbd = mom.clone().cuda(), momb.clone().cuda()
        ffi.bww_sr_sgd(dev["Xt"], dev["loc"], dY.cuda(), w, b, md, mbd, G, label0, lr, wd, mu, seed, step,
                       ffi.make_flags(sr=True, contract=True, rng=rng))
        assert np.array_equal(_bits(w), fo._bf16_to_bits(want_w)), "weights"
        assert np.array_equal(_bits(b), fo._bf16_to_bits(want_b)), "bias"
        if mu:
            assert np.array_equal(md.cpu().numpy(), want_m.numpy())
            assert np.array_equal(mbd.cpu().numpy(), want_mb.numpy())


def _run_fused(ffi, lib, dev, shape, loss_kind, grad_scale, rng, label0=0, step=3, seed=123, lr=0.05, wd=1e-4, want_loss=True):
    B, D, L, F, G = shape
    NG = (L + G - 1) // G
    coo = dev["targets"].clone()
    coo[:, 1] += label0
    ptr = torch.zeros(NG + 1, dtype=torch.int32, device="cuda")
    ent = torch.zeros(max(1, coo.shape[0]), dtype=torch.int32, device="cuda")
    scratch = torch.zeros(NG, dtype=torch.int32, device="cuda")
    ffi.targets_bucket(coo, label0, L, G, ptr, ent, scratch)
    w, b = dev["W"].clone(), dev["bias"].clone()
    dxt = torch.full((D, B), 7.0, dtype=torch.float32, device="cuda")       # must be cleared by the flag
    loss = torch.zeros(1, dtype=torch.float32, device="cuda")
    ffi.train_step(dev["loc"], dev["Xt"], w, b, None, None, ptr, ent, dxt, loss, G, label0, loss_kind, grad_scale, lr, wd, 0.0,
                   seed, step, ffi.make_flags(sr=True, contract=True, rng=rng, zero_dxt=True, loss=want_loss))
    return w, b, dxt, loss


@pytest.mark.parametrize("shape", [(64, 768, 1000, 32, 32), (200, 256, 1111, 64, 128), (256, 512, 777, 128, 64),
                                   (130, 96, 300, 16, 16), (33, 64, 40, 16, 128)])
@pytest.mark.parametrize("loss_name", ["bce", "squared_hinge"])
def test_train_step_vs_oracle(hb, shape, loss_name):
    ffi, lib = hb
    B, D, L, F, G = shape
    kind = {"bce": lib.LOSS_BCE, "squared_hinge": lib.LOSS_SQHINGE}[loss_name]
    inp, dev = _inputs(*shape)
    scale = 1.0 if loss_name == "bce" else 0.25
    for rng in ("reference", "packed"):
        w, b, dxt, loss = _run_fused(ffi, lib, dev, shape, kind, scale, rng)
        ref = fo.train_step(inp["loc"], inp["X"], inp["W"], inp["bias"], inp["targets"], G, kind, 0.05, 1e-4, 123, step=3,
                            grad_scale=scale, rng_mode=rng)
        _assert_close(dxt, ref["dXt"], rel=1e-2, abs_=2e-3 * max(1.0, float(ref["dXt"].abs().max())), what="dXt")
        assert abs(float(loss) - ref["loss"]) <= 2e-3 * abs(ref["loss"]) + 1e-3, (float(loss), ref["loss"])
        # Not bit-exact by construction (the kernel's fp32 summation order differs from the oracle's fp64 sums, so a
        # logit can round to the neighbouring bf16 and move one dY entry by one bf16 step): a weight may move by
        # lr * (a few bf16 steps of dW + one bf16 step of dY times the largest |x|).  The bit-exact statement of
        # the fused step is test_train_step_hinge_bit_exact_chain.
        flip = 2.0 ** -7 * float(ref["dY"].float().abs().max()) * float(inp["X"].float().abs().max())
        gw = 0.05 * (4 * _ulp_bf16(ref["dW"].float().numpy()) + flip)
        gb = 0.05 * (4 * _ulp_bf16(ref["dbias"].float().numpy()) + 2.0 ** -7 * float(ref["dY"].float().abs().max()))
        _assert_bf16_ulp(_bits(w), fo._bf16_to_bits(ref["W_new"]), what="W", extra_abs=gw)
        _assert_bf16_ulp(_bits(b), fo._bf16_to_bits(ref["bias_new"]), max_ulp=2, max_frac=0.2, what="bias", extra_abs=gb)


@pytest.mark.parametrize("shape", [(200, 256, 1111, 32, 128), (256, 512, 777, 128, 64), (64, 768, 1000, 32, 32)])
def test_train_step_hinge_bit_exact_chain(hb, shape):
    """With the squared hinge (exact elementwise arithmetic) the warp-mma fused step must equal, bit for bit,
    forward kernel -> oracle loss gradient -> backward-weights kernel -> oracle SGD/SR (the unfused kernels share
    its accumulation order).  The tcgen05 fused step (G=128, F=64) has its own bit-exact chain in
    test_gpu_step_sm100.py."""
    ffi, lib = hb
    B, D, L, F, G = shape
    inp, dev = _inputs(*shape)
    scale, label0 = 0.5, 256
    z = ffi.forward(dev["loc"], dev["Xt"], dev["W"], dev["bias"], G)
    _, dY = fo.loss_and_grad(z.cpu(), inp["targets"], fo.LOSS_SQHINGE, scale)
    dw, db = ffi.backward_weights(dev["Xt"], dev["W"], dev["loc"], dY.cuda(), G, want_dbias=True)
    for rng in ("reference", "packed"):
        want_w, _ = fo.sgd_update(inp["W"], dw.cpu(), None, 0.05, 1e-4, 0.0, False, True,
                                  fo.rand16_for((L, F), 123, 3, rng, label0))
        want_b, _ = fo.sgd_update(inp["bias"], db.cpu(), None, 0.05, 1e-4, 0.0, False, True,
                                  fo.rand16_for((L, 1), 123, 3, rng, label0, is_bias=True).reshape(L))
        w, b, dxt, _ = _run_fused(ffi, lib, dev, shape, lib.LOSS_SQHINGE, scale, rng, label0=label0)
        assert np.array_equal(_bits(w), fo._bf16_to_bits(want_w))
        assert np.array_equal(_bits(b), fo._bf16_to_bits(want_b))
        dxt_unfused = ffi.backward_features(dev["Xt"], dev["W"], dev["loc"], dY.cuda(), G)
        _assert_close(dxt, dxt_unfused, rel=1e-4, abs_=1e-4 * max(1.0, float(dxt_unfused.abs().max())), what="dXt fused vs unfused")


def test_zero_lr_step_is_identity(hb):
    """lr = 0, wd = 0: stochastic rounding of an exact bf16 value never moves it."""
    ffi, lib = hb
    shape = (128, 256, 2000, 64, 128)
    inp, dev = _inputs(*shape)
    w, b, _, _ = _run_fused(ffi, lib, dev, shape, lib.LOSS_BCE, 1.0, "packed", lr=0.0, wd=0.0)
    assert torch.equal(w, dev["W"]) and torch.equal(b, dev["bias"])


# ------------------------------------------------------------------------------------------------ rewire
@pytest.mark.parametrize("cfg", [
    dict(D=96, L=150, F=32, G=32, mode="fraction", frac=0.25, thr=None, regrow="replace", init="zero", regroup=False),
    dict(D=300, L=200, F=48, G=64, mode="fraction", frac=0.15, thr=None, regrow="unused", init="zero", regroup=True),
    dict(D=96, L=70, F=16, G=16, mode="threshold", frac=None, thr=0.12, regrow="unused", init="random", regroup=True),
    dict(D=4096, L=1000, F=128, G=64, mode="fraction", frac=0.15, thr=None, regrow="unused", init="zero", regroup=True),
    dict(D=40, L=300, F=16, G=128, mode="fraction", frac=0.5, thr=None, regrow="unused", init="random", regroup=True),
])
def test_rewire_bit_exact(hb, cfg):
    ffi, _ = hb
    D, L, F, G = cfg["D"], cfg["L"], cfg["F"], cfg["G"]
    inp = fo.make_inputs(4, D, L, F, G, 1, 1.1, seed=13)
    NG = (L + G - 1) // G
    gen = torch.Generator().manual_seed(4)
    loc0 = torch.randint(0, D, (NG, F), generator=gen, dtype=torch.int32) if cfg["regrow"] == "replace" else inp["loc"]
    mom = torch.randn(L, F, generator=gen)
    seed, step, group0 = 31, 2, 7
    W1, loc1, mom1 = fo.rewire(inp["W"], loc0, G, D, cfg["mode"], cfg["frac"], cfg["thr"], init_mode=cfg["init"],
                               regrow=cfg["regrow"], regroup=cfg["regroup"], seed=seed, step=step, momentum=mom, group0=group0)
    w, loc, m = inp["W"].clone().cuda(), loc0.clone().cuda(), mom.clone().cuda()
    changed = torch.zeros(1, dtype=torch.int32, device="cuda")
    n_prune = int(F * cfg["frac"]) if cfg["mode"] == "fraction" else 0
    ffi.rewire(w, loc, m, D, G, group0, 1 if cfg["mode"] == "fraction" else 0, cfg["thr"] or 0.0, n_prune,
               0 if cfg["regrow"] == "replace" else 1, 0 if cfg["init"] == "zero" else 1, cfg["regroup"], seed, step, changed)
    assert np.array_equal(loc.cpu().numpy(), loc1.numpy()), "index table"
    assert np.array_equal(_bits(w), fo._bf16_to_bits(W1)), "weights"
    assert np.array_equal(m.cpu().numpy(), mom1.numpy()), "momentum"
    scores = fo.rewire_scores(inp["W"], G, NG)
    assert int(changed) == int(fo.prune_mask(scores, cfg["mode"], cfg["frac"], cfg["thr"]).sum())
    if cfg["regrow"] == "unused":
        rows = loc.cpu().numpy()
        assert all(len(set(r)) == F for r in rows), "an 'unused' regrow must leave rows duplicate-free"
    if cfg["regroup"]:
        assert (np.diff(loc.cpu().numpy(), axis=1) >= 0).all()


@pytest.mark.parametrize("cfg", [
    dict(D=96, L=150, F=32, G=32, score="mean", mode="fraction", frac=0.2, thr=None, regrow="replace", init="zero", regroup=False),
    dict(D=300, L=200, F=48, G=64, score="max", mode="fraction", frac=0.1, thr=None, regrow="unused", init="random", regroup=True),
    dict(D=96, L=70, F=16, G=16, score="max", mode="threshold", frac=None, thr=0.17, regrow="unused", init="zero", regroup=True),
    dict(D=768, L=128 * 300 + 11, F=64, G=128, score="max", mode="fraction", frac=0.15, thr=None, regrow="unused", init="zero", regroup=True),
    dict(D=768, L=128 * 300 + 11, F=64, G=128, score="mean", mode="fraction", frac=0.3, thr=None, regrow="replace", init="random", regroup=False),
])
def test_rewire_global_bit_exact(hb, cfg):
    """Layer-wide fraction pruning and max scores (the rule of the reference's GroupFixedFanInReal) against the
    oracle, bit for bit.  The max of bf16 magnitudes ties often, so the tie rule (lowest flat index) is exercised."""
    ffi, _ = hb
    D, L, F, G = cfg["D"], cfg["L"], cfg["F"], cfg["G"]
    inp = fo.make_inputs(4, D, L, F, G, 1, 1.1, seed=17)
    NG = (L + G - 1) // G
    gen = torch.Generator().manual_seed(4)
    loc0 = torch.randint(0, D, (NG, F), generator=gen, dtype=torch.int32) if cfg["regrow"] == "replace" else inp["loc"]
    mom = torch.randn(L, F, generator=gen)
    seed, step, group0 = 31, 2, 7
    W1, loc1, mom1 = fo.rewire(inp["W"], loc0, G, D, cfg["mode"], cfg["frac"], cfg["thr"], init_mode=cfg["init"],
                               regrow=cfg["regrow"], regroup=cfg["regroup"], seed=seed, step=step, momentum=mom, group0=group0,
                               score_mode=cfg["score"], prune_scope="global")
    w, loc, m = inp["W"].clone().cuda(), loc0.clone().cuda(), mom.clone().cuda()
    changed = torch.zeros(1, dtype=torch.int32, device="cuda")
    n_prune = int(NG * F * cfg["frac"]) if cfg["mode"] == "fraction" else 0
    ffi.rewire_ex(w, loc, m, D, G, group0, 0 if cfg["score"] == "mean" else 1, 2 if cfg["mode"] == "fraction" else 0, cfg["thr"] or 0.0,
                  n_prune, 0 if cfg["regrow"] == "replace" else 1, 0 if cfg["init"] == "zero" else 1, cfg["regroup"], seed, step, changed)
    scores = fo.rewire_scores(inp["W"], G, NG, cfg["score"])
    mask = fo.prune_mask(scores, cfg["mode"], cfg["frac"], cfg["thr"], "global")
    assert int(changed) == int(mask.sum())
    if cfg["mode"] == "fraction":
        assert int(mask.sum()) == n_prune
    assert np.array_equal(loc.cpu().numpy(), loc1.numpy()), "index table"
    assert np.array_equal(_bits(w), fo._bf16_to_bits(W1)), "weights"
    assert np.array_equal(m.cpu().numpy(), mom1.numpy()), "momentum"


@pytest.mark.parametrize("name", ["gfrac_mean", "gfrac_max", "thr_max"])
def test_rewire_global_reference_golden(hb, name):
    """The kernel against outputs of the reference's own GroupFixedFanInReal.rewire (run on CPU when the fixtures
    were made): which slots are pruned and which weight columns are zeroed.  The reference draws the new indices
    with torch.randint, so the index values themselves are compared only where nothing was pruned."""
    import os
    ffi, _ = hb
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", f"rewire_real_{name}.npz"))
    D, G, mode, score = int(z["D"]), int(z["G"]), str(z["mode"]), str(z["score"])
    W0 = torch.from_numpy(z["w0"].astype(np.int16)).view(torch.bfloat16)
    loc0 = torch.from_numpy(z["loc0"].copy())
    NG, F = loc0.shape
    w, loc = W0.clone().cuda(), loc0.clone().cuda()
    n_prune = int(NG * F * float(z["frac"])) if mode == "fraction" else 0
    ffi.rewire_ex(w, loc, None, D, G, 0, 0 if score == "mean" else 1, 2 if mode == "fraction" else 0, float(z["thr"]), n_prune,
                  0, 0, False, 3, 0, None)
    assert np.array_equal(_bits(w), z["w1"]), "zeroed weight columns"
    pruned = np.zeros((NG, F), bool)
    for g in range(NG):
        rows0, rows1 = z["w0"].reshape(-1, F)[g * G:(g + 1) * G], z["w1"].reshape(-1, F)[g * G:(g + 1) * G]
        pruned[g] = (rows1 == 0).all(axis=0) & ~(rows0 == 0).all(axis=0)
    assert np.array_equal(loc.cpu().numpy()[~pruned], z["loc1"][~pruned])
    assert pruned.sum() == len(z["injected"])


def test_regroup_preserves_output(hb):
    ffi, _ = hb
    B, D, L, F, G = 64, 256, 900, 64, 128
    inp, dev = _inputs(B, D, L, F, G)
    gen = torch.Generator().manual_seed(8)
    loc = torch.randint(0, D, ((L + G - 1) // G, F), generator=gen, dtype=torch.int32).cuda()   # unsorted rows
    z0 = ffi.forward(loc, dev["Xt"], dev["W"], dev["bias"], G)
    w = dev["W"].clone()
    ffi.rewire(w, loc, None, D, G, 0, 0, -1.0, 0, 0, 0, True, 0, 0, None)        # threshold -1: nothing pruned, regroup only
    z1 = ffi.forward(loc, dev["Xt"], w, dev["bias"], G)
    _assert_close(z1, z0, rel=1e-2, abs_=1e-3, what="regroup")
    assert (np.diff(loc.cpu().numpy(), axis=1) >= 0).all()


# ------------------------------------------------------------------------------------------------ errors
def test_error_convention(hb):
    ffi, lib = hb
    inp, dev = _inputs(16, 64, 100, 16, 32)
    with pytest.raises(RuntimeError, match="group size"):
        ffi.forward(dev["loc"], dev["Xt"], dev["W"], dev["bias"], 48)
    w24 = torch.zeros(100, 24, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="fan_in"):
        ffi.forward(dev["loc"], dev["Xt"], w24, None, 32)
    with pytest.raises(RuntimeError):
        ffi.forward(dev["loc"].cpu(), dev["Xt"], dev["W"], None, 32)
    bad = dev["loc"].clone()
    bad[0, 0] = 64
    with pytest.raises(RuntimeError, match="outside"):
        ffi.check_locations(bad, 64)
    ffi.check_locations(dev["loc"], 64)


@pytest.mark.parametrize("B,D", [(200, 96), (203, 90), (520, 776), (64, 128)])
def test_step_prepare(hb, B, D):
    """The one-launch preparation equals transpose + clears + haste_targets_bucket, on its 16-byte path (B and D
    multiples of 8; ragged 64 x 128 tiles) and on the element-wise one."""
    ffi, _ = hb
    L, G = 5000, 64
    inp = fo.make_inputs(B, D, L, 16, G, 12, 1.1, seed=9)
    x, coo = inp["X"].cuda(), inp["targets"].cuda()
    for label0, Ls in ((0, L), (1024, 2000)):
        NG = (Ls + G - 1) // G
        ptr0 = torch.zeros(NG + 1, dtype=torch.int32, device="cuda")
        ent0 = torch.zeros(coo.shape[0], dtype=torch.int32, device="cuda")
        ffi.targets_bucket(coo, label0, Ls, G, ptr0, ent0, torch.zeros(NG, dtype=torch.int32, device="cuda"))
        ptr1 = torch.full((NG + 1,), -1, dtype=torch.int32, device="cuda")
        ent1 = torch.full((coo.shape[0],), -1, dtype=torch.int32, device="cuda")
        xt = torch.empty(D, B, dtype=torch.bfloat16, device="cuda")
        dxt = torch.full((D, B), 5.0, device="cuda")
        loss = torch.full((1,), 3.0, device="cuda")
        ffi.step_prepare(x, xt, dxt, loss, coo, label0, Ls, G, ptr1, ent1)
        assert torch.equal(xt.cpu(), inp["X"].t().contiguous()) and float(loss) == 0.0 and not dxt.any()
        p0, p1 = ptr0.cpu().numpy(), ptr1.cpu().numpy()
        assert np.array_equal(p0, p1)
        e0, e1 = ent0.cpu().numpy(), ent1.cpu().numpy()
        for g in np.nonzero(np.diff(p0))[0]:
            assert sorted(e0[p0[g]:p0[g + 1]]) == sorted(e1[p1[g]:p1[g + 1]])


# ------------------------------------------------------------------------------------------------ inference top-k
@pytest.mark.parametrize("cfg", [
    dict(B=64, D=256, L=128 * 40 + 7, F=64, G=128, k=100, chunk=7),
    dict(B=33, D=96, L=1000, F=32, G=32, k=5, chunk=4),
    dict(B=16, D=128, L=300, F=16, G=64, k=128, chunk=2),
    dict(B=8, D=64, L=50, F=16, G=16, k=100, chunk=None),          # fewer labels than k: the tail stays (-inf, -1)
])
def test_topk_chunked_matches_full(hb, cfg):
    """Chunked forward + running top-k against torch.topk over the full logits of the same forward kernel.
    Values must match exactly; label ids must match wherever the value is unique in its row, and must point at a
    logit of that value everywhere (torch.topk leaves the order of equal values open; here it is by label id)."""
    ffi, _ = hb
    from haste_b200.infer import ffi_topk
    B, D, L, F, G, k = cfg["B"], cfg["D"], cfg["L"], cfg["F"], cfg["G"], cfg["k"]
    inp = fo.make_inputs(B, D, L, F, G, 2, 1.1, seed=29, x_kind="normal", bias_zero=False)
    dev = {n: v.cuda() for n, v in inp.items()}
    vals, idx = ffi_topk(dev["loc"], dev["W"], dev["bias"], dev["X"], k, G, groups_per_chunk=cfg["chunk"], label0=5)
    z = ffi.forward(dev["loc"], dev["X"].t().contiguous(), dev["W"], dev["bias"], G).float()
    kk = min(k, L)
    want_v, want_i = torch.topk(z, kk, dim=1)
    assert torch.equal(vals[:, :kk], want_v)
    if kk < k:
        assert torch.isinf(vals[:, kk:]).all() and (idx[:, kk:] == -1).all()
    got_i = idx[:, :kk].long() - 5
    assert (got_i >= 0).all() and (got_i < L).all()
    assert torch.equal(torch.gather(z, 1, got_i), want_v)                     # every id points at a logit of that value
    assert all(len(set(r.tolist())) == kk for r in got_i.cpu())               # no label twice
    # ties are ordered by label id
    same = vals[:, 1:kk] == vals[:, :kk - 1]
    assert (got_i[:, 1:][same] > got_i[:, :-1][same]).all()
    # where a value is unique in the row's top-k, the id is torch's id
    uniq = torch.ones_like(want_v, dtype=torch.bool)
    uniq[:, 1:] &= want_v[:, 1:] != want_v[:, :-1]
    uniq[:, :-1] &= want_v[:, :-1] != want_v[:, 1:]
    if kk == k:   # the last kept value may tie with one that was cut off
        uniq[:, -1] &= (z == want_v[:, -1:]).sum(1) == 1
    assert torch.equal(got_i[uniq], want_i[uniq])


@pytest.mark.parametrize("cfg", [
    dict(D=300, L=64 * 11 + 9, F=48, G=64, score="max", frac=0.1, regrow="unused", init="random", regroup=True, cuts=[3, 8]),
    dict(D=768, L=128 * 300 + 11, F=64, G=128, score="max", frac=0.15, regrow="unused", init="zero", regroup=True, cuts=[40, 41, 200]),
    dict(D=768, L=128 * 300 + 11, F=64, G=128, score="mean", frac=0.3, regrow="replace", init="random", regroup=False, cuts=[150]),
])
def test_rewire_layerwide_across_shards_bit_exact(hb, cfg):
    """The layer-wide fraction rule on a layer cut into label shards (haste_ffi_rewire_select_* + _prepared): the
    shards' histograms are summed between the phases and the tie counts gathered, exactly as ranks would exchange
    them; the result must equal the oracle's (and the single-shard kernel's) rewire of the whole layer, bit for bit —
    including which of the scores that tie at the threshold are pruned (max scores of bf16 magnitudes tie often)."""
    ffi, _ = hb
    from haste_b200.fused import layerwide_prune_count, tie_base_for_rank
    D, L, F, G = cfg["D"], cfg["L"], cfg["F"], cfg["G"]
    inp = fo.make_inputs(4, D, L, F, G, 1, 1.1, seed=23)
    NG = (L + G - 1) // G
    gen = torch.Generator().manual_seed(5)
    loc0 = torch.randint(0, D, (NG, F), generator=gen, dtype=torch.int32) if cfg["regrow"] == "replace" else inp["loc"]
    seed, step = 77, 4
    W1, loc1, _ = fo.rewire(inp["W"], loc0, G, D, "fraction", cfg["frac"], None, init_mode=cfg["init"], regrow=cfg["regrow"],
                            regroup=cfg["regroup"], seed=seed, step=step, group0=0, score_mode=cfg["score"], prune_scope="global")
    bounds = [0] + cfg["cuts"] + [NG]
    shards = []
    for g0, g1 in zip(bounds, bounds[1:]):
        l0, l1 = g0 * G, min(L, g1 * G)
        shards.append(dict(g0=g0, w=inp["W"][l0:l1].clone().cuda(), loc=loc0[g0:g1].clone().cuda()))
    k = layerwide_prune_count(NG, F, cfg["frac"])
    sels = [ffi.LayerwideSelect(s["w"], G, 0 if cfg["score"] == "mean" else 1) for s in shards]
    for s in sels:
        s.begin()
    total = sum(s.hist_hi.clone() for s in sels)
    for s in sels:
        s.hist_hi.copy_(total)
        s.refine(k)
    total = sum(s.hist_lo.clone() for s in sels)
    for s in sels:
        s.hist_lo.copy_(total)
        s.finish()
    ties = [int(s.ties.item()) for s in sels]
    n_changed = 0
    for r, (s, sh) in enumerate(zip(sels, shards)):
        changed = torch.zeros(1, dtype=torch.int32, device="cuda")
        s.apply(sh["loc"], None, D, sh["g0"], tie_base_for_rank(ties, r), 0 if cfg["regrow"] == "replace" else 1,
                0 if cfg["init"] == "zero" else 1, cfg["regroup"], seed, step, changed)
        n_changed += int(changed)
    assert n_changed == k
    assert np.array_equal(torch.cat([sh["loc"] for sh in shards]).cpu().numpy(), loc1.numpy()), "index table"
    assert np.array_equal(_bits(torch.cat([sh["w"] for sh in shards])), fo._bf16_to_bits(W1)), "weights"
