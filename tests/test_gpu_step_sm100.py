"""GPU parity tests of the tcgen05 fused train step (group size 128 / fan-in 64, and group size 64 / fan-in 128)
through the C ABI.

The kernel's debug outputs expose the bf16 logits and the bf16 gradients it consumed, which splits the check
into (a) tensor-core products against the oracle within the floating-point tolerance (rel 1e-2 / abs 1e-3 of
the magnitude) and (b) everything downstream of them — loss gradient (squared hinge is exact arithmetic),
SGD + weight decay + stochastic rounding — bit for bit."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import ffi_oracle as fo

F, G = 64, 128
SHAPES = [(200, 256, 1111), (512, 768, 5000), (128, 128, 384), (1024, 300, 2000), (8, 96, 100), (392, 768, 20000)]  # B, D, L
KINDS = [(128, 64), (64, 128)]          # (G, F) with a tcgen05 fused step
SHAPES_G64 = [(200, 256, 1111), (512, 768, 5000), (64, 128, 192), (1024, 300, 2000), (8, 160, 100), (256, 4096, 3018)]  # B, D, L


@pytest.fixture(scope="module")
def hb():
    import haste_b200.ffi as ffi
    import haste_b200._lib as lib
    return ffi, lib


def _bits(t):
    return fo._bf16_to_bits(t.detach().cpu())


def _close(got, want, rel, abs_, what):
    got, want = got.float().cpu(), want.float().cpu()
    bad = (got - want).abs() > abs_ + rel * want.abs()
    assert not bad.any(), f"{what}: {int(bad.sum())}/{bad.numel()} outside tolerance, max err {float((got - want).abs().max())}"


def _run(ffi, lib, inp, B, D, L, kind, scale, rng, label0=0, bias=True, step=3, seed=123, lr=0.05, wd=1e-4, G=G):
    dev = {k: v.cuda() for k, v in inp.items()}
    xt = dev["X"].t().contiguous()
    NG = (L + G - 1) // G
    coo = dev["targets"].clone()
    coo[:, 1] += label0
    ptr = torch.zeros(NG + 1, dtype=torch.int32, device="cuda")
    ent = torch.zeros(max(1, coo.shape[0]), dtype=torch.int32, device="cuda")
    scratch = torch.zeros(NG, dtype=torch.int32, device="cuda")
    ffi.targets_bucket(coo, label0, L, G, ptr, ent, scratch)
    w = dev["W"].clone()
    b = dev["bias"].clone() if bias else None
    dxt = torch.full((D, B), 3.0, dtype=torch.float32, device="cuda")
    loss = torch.zeros(1, dtype=torch.float32, device="cuda")
    flags = ffi.make_flags(sr=True, contract=True, rng=rng, zero_dxt=True, loss=True)
    z, dw, db = ffi.train_step_dbg(dev["loc"], xt, w, b, ptr, ent, dxt, loss, G, label0, kind, scale, lr, wd, seed, step, flags)
    torch.cuda.synchronize()
    return w, b, dxt, float(loss), z, dw, db


_CHAIN = [(128, 64, s) for s in SHAPES] + [(64, 128, s) for s in SHAPES_G64]


@pytest.mark.parametrize("case", _CHAIN, ids=[f"G{c[0]}F{c[1]}-B{c[2][0]}D{c[2][1]}L{c[2][2]}" for c in _CHAIN])
@pytest.mark.parametrize("rng", ["packed", "reference"])
def test_sm100_step_hinge_chain(hb, case, rng):
    ffi, lib = hb
    G, F, (B, D, L) = case
    inp = fo.make_inputs(B, D, L, F, G, 6, 1.1, seed=B + L, x_kind="normal", bias_zero=False)
    scale, label0 = 0.5, 384
    w, b, dxt, loss, z, dw, db = _run(ffi, lib, inp, B, D, L, lib.LOSS_SQHINGE, scale, rng, label0=label0, G=G)
    # (a) tensor-core products within tolerance
    z_ref = fo.forward(inp["loc"], inp["X"], inp["W"], inp["bias"], G, round_bf16=False)
    _close(z, z_ref, 1e-2, 1e-3 * max(1.0, float(z_ref.abs().max())), "logits")
    loss_ref, dY = fo.loss_and_grad(z.cpu(), inp["targets"], fo.LOSS_SQHINGE, scale)       # exact given the kernel's logits
    dw_ref = fo.backward_weights(inp["loc"], inp["X"], dY, G, L, round_bf16=False)
    _close(dw, dw_ref, 1e-2, 1e-3 * max(1.0, float(dw_ref.abs().max())), "dW")
    _close(db, dY.float().sum(0), 1e-2, 1e-3 * max(1.0, float(dY.float().sum(0).abs().max())), "dbias")
    dxt_ref = fo.backward_features(inp["loc"], inp["W"], dY, G, D)
    _close(dxt, dxt_ref, 1e-2, 1e-3 * max(1.0, float(dxt_ref.abs().max())), "dXt")
    assert abs(loss - loss_ref) <= 1e-3 * abs(loss_ref) + 1e-3
    # (b) the update, bit for bit, from the gradients the kernel consumed
    want_w, _ = fo.sgd_update(inp["W"], dw.cpu(), None, 0.05, 1e-4, 0.0, False, True, fo.rand16_for((L, F), 123, 3, rng, label0))
    want_b, _ = fo.sgd_update(inp["bias"], db.cpu(), None, 0.05, 1e-4, 0.0, False, True,
                              fo.rand16_for((L, 1), 123, 3, rng, label0, is_bias=True).reshape(L))
    assert np.array_equal(_bits(w), fo._bf16_to_bits(want_w)), "weights"
    assert np.array_equal(_bits(b), fo._bf16_to_bits(want_b)), "bias"


@pytest.mark.parametrize("kind", KINDS, ids=["G128F64", "G64F128"])
@pytest.mark.parametrize("shape", [(200, 256, 1111), (512, 768, 5000), (8, 160, 100)])
def test_sm100_step_bce_and_nobias(hb, shape, kind):
    ffi, lib = hb
    B, D, L = shape
    G, F = kind
    inp = fo.make_inputs(B, D, L, F, G, 12, 1.1, seed=7, x_kind="normal", bias_zero=False)
    for bias in (True, False):
        w, b, dxt, loss, z, dw, db = _run(ffi, lib, inp, B, D, L, lib.LOSS_BCE, 1.0, "packed", bias=bias, G=G)
        bias_t = inp["bias"] if bias else None
        z_ref = fo.forward(inp["loc"], inp["X"], inp["W"], bias_t, G, round_bf16=False)
        _close(z, z_ref, 1e-2, 1e-3 * max(1.0, float(z_ref.abs().max())), "logits")
        loss_ref, dY = fo.loss_and_grad(z.cpu(), inp["targets"], fo.LOSS_BCE, 1.0)
        assert abs(loss - loss_ref) <= 2e-3 * abs(loss_ref)
        dw_ref = fo.backward_weights(inp["loc"], inp["X"], dY, G, L, round_bf16=False)
        _close(dw, dw_ref, 2e-2, 2e-3 * max(1.0, float(dw_ref.abs().max())), "dW")      # sigmoid via tanh.approx: dY may differ by a bf16 step
        dxt_ref = fo.backward_features(inp["loc"], inp["W"], dY, G, D)
        _close(dxt, dxt_ref, 2e-2, 2e-3 * max(1.0, float(dxt_ref.abs().max())), "dXt")
        want_w, _ = fo.sgd_update(inp["W"], dw.cpu(), None, 0.05, 1e-4, 0.0, False, True, fo.rand16_for((L, F), 123, 3, "packed", 0))
        assert np.array_equal(_bits(w), fo._bf16_to_bits(want_w))


def test_sm100_step_repeatable_weights(hb):
    """Two runs on the same inputs give identical weights (the tensor-core products and the update are
    deterministic; only the dX atomics may reorder)."""
    ffi, lib = hb
    B, D, L = 512, 768, 9000
    inp = fo.make_inputs(B, D, L, F, G, 6, 1.0, seed=5, bias_zero=False)
    r1 = _run(ffi, lib, inp, B, D, L, lib.LOSS_SQHINGE, 1.0, "packed")
    r2 = _run(ffi, lib, inp, B, D, L, lib.LOSS_SQHINGE, 1.0, "packed")
    assert torch.equal(r1[0], r2[0]) and torch.equal(r1[1], r2[1])
    assert torch.allclose(r1[2], r2[2], rtol=1e-5, atol=1e-5 * float(r1[2].abs().max()))


@pytest.mark.parametrize("shape", SHAPES + [(512, 768, 670091 // 16)])
def test_sm100_forward(hb, shape):
    """tcgen05 forward (G=128, F=64) against the oracle, including the zero padding columns and the no-bias case."""
    ffi, _ = hb
    B, D, L = shape
    inp = fo.make_inputs(B, D, L, F, G, 2, 1.1, seed=L, x_kind="normal", bias_zero=False)
    dev = {k: v.cuda() for k, v in inp.items()}
    xt = dev["X"].t().contiguous()
    for bias in (dev["bias"], None):
        z = ffi.forward(dev["loc"], xt, dev["W"], bias, G)
        want = fo.forward(inp["loc"], inp["X"], inp["W"], inp["bias"] if bias is not None else None, G, round_bf16=False)
        _close(z, want, 1e-2, 1e-3 * max(1.0, float(want.abs().max())), "forward")
        ldz = (L + 7) // 8 * 8
        if ldz > L:
            assert (torch.as_strided(z, (B, ldz), (ldz, 1))[:, L:] == 0).all()


@pytest.mark.parametrize("shape", SHAPES + [(512, 768, 670091 // 16)])
def test_sm100_backward_both(hb, shape):
    """One-pass tcgen05 backward (G=128, F=64): dxt, dw and dbias against the oracle, for gradient rows that need
    padding (L % 8 != 0) and rows that are already aligned."""
    ffi, _ = hb
    B, D, L = shape
    inp = fo.make_inputs(B, D, L, F, G, 2, 1.1, seed=L + 1, x_kind="normal", bias_zero=False)
    dev = {k: v.cuda() for k, v in inp.items()}
    xt = dev["X"].t().contiguous()
    gen = torch.Generator().manual_seed(3)
    dY = (torch.randn(B, L, generator=gen) * 0.5).to(torch.bfloat16)
    ldp = (L + 7) // 8 * 8
    aligned = torch.zeros(B, ldp, dtype=torch.bfloat16, device="cuda")
    aligned[:, :L] = dY.cuda()
    want_x = fo.backward_features(inp["loc"], inp["W"], dY, G, D)
    want_w = fo.backward_weights(inp["loc"], inp["X"], dY, G, L, round_bf16=False)
    for dy_dev in (dY.cuda(), aligned[:, :L]):
        dxt, dw, db = ffi.backward_both(xt, dev["W"], dev["loc"], dy_dev, G)
        _close(dxt, want_x, 1e-2, 1e-3 * max(1.0, float(want_x.abs().max())), "dXt")
        _close(dw, want_w, 1e-2, 1e-3 * max(1.0, float(want_w.abs().max())), "dW")
        _close(db, dY.float().sum(0), 1e-2, 2e-2, "dbias")


@pytest.mark.parametrize("loss", ["squared_hinge", "bce"])
def test_sm100_step_rank_count_independent(hb, loss):
    """A layer split over ranks (contiguous group ranges) must give bit-identical weights and bias to the unsplit
    layer — random bits are drawn by global label, and the order in which a group's batch tiles enter its dW accumulator
    does not depend on where the group runs — and the same dX up to the fp32 summation order.  The ranks are run one
    after the other on this GPU; their dX are added on the host.  Splits: by estimated cost, and at explicit odd and
    even group boundaries (a rotation of the tile order by anything local — CTA index, shard-local group index —
    shows up as a few differing weights when a shard starts at a group index that is not a multiple of the tile count)."""
    from haste_b200.fused import FusedFFIShard, group_cost_from_targets, split_groups_by_cost
    B, D, L = 512, 256, 128 * 37 + 50                          # four batch tiles
    inp = fo.make_inputs(B, D, L, F, G, 6, 1.1, seed=11, bias_zero=False)
    X, coo = inp["X"].cuda(), inp["targets"].cuda()
    kw = dict(loss=loss, lr=0.05, weight_decay=1e-4, seed=123, rng="packed", grad_scale=0.5)

    def run(g0, g1):
        l0, l1 = min(L, g0 * G), min(L, g1 * G)
        sh = FusedFFIShard(inp["loc"][g0:g1].cuda().contiguous(), inp["W"][l0:l1].cuda().contiguous(),
                           inp["bias"][l0:l1].cuda().contiguous(), G, D, label0=l0, **kw)
        for _ in range(2):                                    # two steps: the second sees updated weights
            dxt, ls = sh.step(X, coo)
        torch.cuda.synchronize()
        return sh.w.clone(), sh.bias.clone(), dxt.clone(), float(ls)

    NG = (L + G - 1) // G
    w_all, b_all, dxt_all, loss_all = run(0, NG)
    cost = group_cost_from_targets(inp["targets"], L, G, B)
    for bounds in (split_groups_by_cost(cost, 3), [0, 9, NG], [0, 14, NG], [0, 5, 19, 20, NG], [0, 1, 2, NG]):
        assert bounds[0] == 0 and bounds[-1] == NG
        parts = [run(bounds[r], bounds[r + 1]) for r in range(len(bounds) - 1)]
        assert np.array_equal(_bits(torch.cat([p[0] for p in parts])), _bits(w_all)), bounds
        assert np.array_equal(_bits(torch.cat([p[1] for p in parts])), _bits(b_all)), bounds
        dxt_sum = sum(p[2] for p in parts)
        _close(dxt_sum, dxt_all, 1e-4, 1e-5 * float(dxt_all.abs().max()), "dX summed over ranks")
        assert abs(sum(p[3] for p in parts) - loss_all) <= 1e-4 * abs(loss_all) + 1e-6


@pytest.mark.parametrize("kind", KINDS, ids=["G128F64", "G64F128"])
def test_sm100_step_momentum(hb, kind):
    """Momentum (the reference's Amazon-3M run uses 0.9) inside the fused step: the debug step yields the gradients
    the update consumes (they do not depend on the optimizer), the production step then runs with preset momentum
    buffers; weights, bias and both buffers must equal the oracle's update of those gradients bit for bit."""
    ffi, lib = hb
    G, F = kind
    B, D, L = 256, 384, 1000
    lr, wd, mu, seed, step = 0.05, 1e-4, 0.9, 123, 5
    inp = fo.make_inputs(B, D, L, F, G, 6, 1.1, seed=21, x_kind="normal", bias_zero=False)
    _, _, _, _, _, dw, db = _run(ffi, lib, inp, B, D, L, lib.LOSS_BCE, 1.0, "packed", step=step, G=G)
    dev = {k: v.cuda() for k, v in inp.items()}
    xt = dev["X"].t().contiguous()
    NG = (L + G - 1) // G
    ptr = torch.zeros(NG + 1, dtype=torch.int32, device="cuda")
    ent = torch.zeros(max(1, dev["targets"].shape[0]), dtype=torch.int32, device="cuda")
    ffi.targets_bucket(dev["targets"], 0, L, G, ptr, ent, torch.zeros(NG, dtype=torch.int32, device="cuda"))
    gen = torch.Generator().manual_seed(3)
    mom_w0 = torch.randn(L, F, generator=gen) * 0.01
    mom_b0 = torch.randn(L, generator=gen) * 0.01
    w, b, mom_w, mom_b = dev["W"].clone(), dev["bias"].clone(), mom_w0.cuda(), mom_b0.cuda()
    dxt = torch.empty(D, B, dtype=torch.float32, device="cuda")
    flags = ffi.make_flags(sr=True, contract=True, rng="packed", zero_dxt=True, loss=False)
    ffi.train_step(dev["loc"], xt, w, b, mom_w, mom_b, ptr, ent, dxt, None, G, 0, lib.LOSS_BCE, 1.0, lr, wd, mu, seed, step, flags)
    torch.cuda.synchronize()
    want_w, want_mw = fo.sgd_update(inp["W"], dw.cpu(), mom_w0, lr, wd, mu, True, True, fo.rand16_for((L, F), seed, step, "packed", 0))
    want_b, want_mb = fo.sgd_update(inp["bias"], db.cpu(), mom_b0, lr, wd, mu, True, True,
                                    fo.rand16_for((L, 1), seed, step, "packed", 0, is_bias=True).reshape(L))
    assert np.array_equal(_bits(w), fo._bf16_to_bits(want_w)), "weights"
    assert np.array_equal(_bits(b), fo._bf16_to_bits(want_b)), "bias"
    assert torch.equal(mom_w.cpu(), want_mw), "weight momentum"
    assert torch.equal(mom_b.cpu(), want_mb), "bias momentum"


def test_sm100_step_wait_runs_out_and_recovers(hb):
    """The bounded-wait path: with a 1 ms wait limit and one barrier arrival withheld, the kernel returns by itself
    (no trap, no fault), the status poll reports HASTE_ERR_TIMEOUT exactly once, and the next step — TMEM was freed,
    the context is intact — runs normally and matches the oracle."""
    ffi, lib = hb
    B, D, L = 512, 256, 128 * 300
    inp = fo.make_inputs(B, D, L, F, G, 4, 1.1, seed=9, bias_zero=False)
    assert lib.lib.haste_poll_status() == lib.OK
    try:
        assert lib.lib.haste_debug_set_wait_limit(2_000_000) == lib.OK       # about 1 ms
        assert lib.lib.haste_debug_stall_next_step(1) == lib.OK
        _run(ffi, lib, inp, B, D, L, lib.LOSS_SQHINGE, 1.0, "packed")          # returns by itself; outputs invalid
    finally:
        lib.lib.haste_debug_set_wait_limit(4_000_000_000)
    assert lib.lib.haste_poll_status() == lib.ERR_TIMEOUT
    assert "wait id" in lib.last_error()
    assert lib.lib.haste_poll_status() == lib.OK                               # reported once
    w, b, dxt, loss, z, dw, db = _run(ffi, lib, inp, B, D, L, lib.LOSS_SQHINGE, 1.0, "packed")
    assert lib.lib.haste_poll_status() == lib.OK
    z_ref = fo.forward(inp["loc"], inp["X"], inp["W"], inp["bias"], G, round_bf16=False)
    _close(z, z_ref, 1e-2, 1e-3 * max(1.0, float(z_ref.abs().max())), "logits after recovery")
    want_w, _ = fo.sgd_update(inp["W"], dw.cpu(), None, 0.05, 1e-4, 0.0, False, True, fo.rand16_for((L, F), 123, 3, "packed", 0))
    assert np.array_equal(_bits(w), fo._bf16_to_bits(want_w))
