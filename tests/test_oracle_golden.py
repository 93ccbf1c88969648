"""Pin the CPU oracle against vectors produced by the reference's own code
(tests/golden/make_golden.py: Triton-interpreter runs of shared_ffi/sr_triton.py and a CPU run of
shared_ffi/rewire.py)."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import ffi_oracle as fo
from oracle import philox as px


def _bf16(bits):
    return fo._bits_to_bf16(np.asarray(bits, np.uint16))


def test_philox_known_answer():
    # Random123 known-answer vectors for philox4x32-10.
    out = px.philox4x32(0, 0, 0, 0, 0, 0)
    assert [int(v) for v in out] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    out = px.philox4x32(0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF)
    assert [int(v) for v in out] == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    out = px.philox4x32(0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344, 0xA4093822, 0x299F31D0)
    assert [int(v) for v in out] == [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]


def test_sr_round_matches_reference(golden_dir):
    files = sorted(glob.glob(os.path.join(golden_dir, "sr_round_seed*.npz")))
    assert len(files) == 3
    for f in files:
        z = np.load(f)
        got = fo.stochastic_rounding(torch.from_numpy(z["x"]), int(z["seed"]))
        assert np.array_equal(fo._bf16_to_bits(got), z["out"]), f


@pytest.mark.parametrize("name", ["wd", "mom", "rn", "mom_off"])
def test_sgd_update_matches_reference(golden_dir, name):
    z = np.load(os.path.join(golden_dir, f"sgd_{name}.npz"))
    w, g = _bf16(z["w"]), _bf16(z["g"])
    m = torch.from_numpy(z["m"].copy())
    r = fo.rand16_for(tuple(w.shape), int(z["seed"]), 0, "reference")
    # the interpreter evaluates mul and add separately -> contract=False
    w1, m1 = fo.sgd_update(w, g, m, float(z["lr"]), float(z["wd"]), float(z["mu"]), bool(z["use_mom"]),
                           bool(z["do_sr"]), r, contract=False)
    if name == "rn":
        # The Triton CPU interpreter truncates an fp32->bf16 ``.to()`` (compiled Triton rounds to
        # nearest even), so the non-SR golden pins the fp32 arithmetic through its high half only.
        w32, _ = fo.sgd_math(w.float().numpy(), g.float().numpy(), None, float(z["lr"]), float(z["wd"]),
                             0.0, False, False)
        assert np.array_equal((px.f32_bits(w32) >> 16).astype(np.uint16), z["w_out"])
        assert np.array_equal(fo._bf16_to_bits(w1), px.rn_bf16_bits(w32))
    else:
        assert np.array_equal(fo._bf16_to_bits(w1), z["w_out"])
    assert np.array_equal(m1.numpy(), z["m_out"])


@pytest.mark.parametrize("name", ["frac", "frac_g64", "thr"])
def test_rewire_matches_reference(golden_dir, name):
    z = np.load(os.path.join(golden_dir, f"rewire_ref_{name}.npz"))
    W0, loc0 = _bf16(z["w0"]), torch.from_numpy(z["loc0"].copy())
    mode = str(z["mode"])
    W1, loc1, _ = fo.rewire(W0, loc0, int(z["G"]), int(z["D"]), mode,
                            rewire_fraction=float(z["frac"]) if mode == "fraction" else None,
                            rewire_threshold=float(z["thr"]) if mode == "threshold" else None,
                            init_mode="zero", regroup=False, injected=z["injected"])
    assert np.array_equal(loc1.numpy(), z["loc1"])
    assert np.array_equal(fo._bf16_to_bits(W1), z["w1"])
    assert not np.array_equal(z["loc0"], z["loc1"])          # the case actually rewired something


@pytest.mark.parametrize("name", ["gfrac_mean", "gfrac_max", "thr_max"])
def test_rewire_global_matches_reference(golden_dir, name):
    """Global-fraction pruning and max scores against src/group_fanin_real.py:149-286 (run on CPU with injected
    indices).  torch.topk leaves the order of equal scores open, so the case must be tie-free at the selection
    boundary for the comparison to mean anything: that is asserted first."""
    z = np.load(os.path.join(golden_dir, f"rewire_real_{name}.npz"))
    W0, loc0 = _bf16(z["w0"]), torch.from_numpy(z["loc0"].copy())
    mode, score = str(z["mode"]), str(z["score"])
    NG, F = loc0.shape
    if mode == "fraction":
        sc = np.sort(fo.rewire_scores(W0, int(z["G"]), NG, score).reshape(-1))
        k = int(NG * F * float(z["frac"]))
        assert 0 < k < sc.size and sc[k - 1] < sc[k], "golden case has a tie at the selection boundary"
    W1, loc1, _ = fo.rewire(W0, loc0, int(z["G"]), int(z["D"]), mode,
                            rewire_fraction=float(z["frac"]) if mode == "fraction" else None,
                            rewire_threshold=float(z["thr"]) if mode == "threshold" else None,
                            init_mode="zero", regroup=False, injected=z["injected"], score_mode=score, prune_scope="global")
    assert np.array_equal(loc1.numpy(), z["loc1"])
    assert np.array_equal(fo._bf16_to_bits(W1), z["w1"])
    assert not np.array_equal(z["loc0"], z["loc1"])


def test_sr_unbiased():
    # E[round(w)] = w within 3 sigma over 1e6 draws, both random streams.
    w = np.float32(0.1234567)
    n = 1_000_000
    for mode in ("reference", "packed"):
        r = fo.rand16_for((n // 64, 64), 123, 7, mode)
        vals = px.bf16_bits_to_f32(px.sr_bf16_bits(np.full(r.shape, w, np.float32), r)).astype(np.float64)
        lo, hi = vals.min(), vals.max()
        p = (float(w) - lo) / (hi - lo)
        sigma = (hi - lo) * np.sqrt(p * (1 - p) / n)
        assert abs(vals.mean() - float(w)) < 3 * sigma, mode


def test_forward_backward_consistent_with_autograd():
    # the three GEMM restatements are mutually consistent: autograd of the forward formula
    torch.manual_seed(0)
    B, D, L, F, G = 8, 40, 50, 16, 16
    inp = fo.make_inputs(B, D, L, F, G, 3, 1.1, seed=3, x_kind="normal", bias_zero=False)
    X = inp["X"].float().requires_grad_(True)
    W = inp["W"].float().requires_grad_(True)
    NG = inp["loc"].shape[0]
    Wp = torch.zeros(NG * G, F); Wp[:L] = W
    Z = torch.einsum("bgf,gnf->bgn", X[:, inp["loc"].long()], Wp.view(NG, G, F)).reshape(B, -1)[:, :L]
    Z = Z + inp["bias"].float()
    dY = torch.randn(B, L).to(torch.bfloat16)
    Z.backward(dY.float())
    Zo = fo.forward(inp["loc"], inp["X"], inp["W"], inp["bias"], G, round_bf16=False)
    assert torch.allclose(Zo, Z.detach(), atol=1e-5)
    dXt = fo.backward_features(inp["loc"], inp["W"], dY, G, D)
    assert torch.allclose(dXt.t(), X.grad, atol=1e-4)
    dW = fo.backward_weights(inp["loc"], inp["X"], dY, G, L, round_bf16=False)
    assert torch.allclose(dW, W.grad, atol=1e-4)


_REF_GEMM = sorted(glob.glob(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_gemm_*.npz")))


def test_ref_gemm_goldens_present():
    assert len(_REF_GEMM) >= 6


@pytest.mark.parametrize("path", _REF_GEMM, ids=[os.path.basename(p)[9:-4] for p in _REF_GEMM])
def test_gemm_phases_match_reference_kernels(path):
    """forward / backward-features / backward-weights of the oracle against what the reference's own CUDA kernels
    returned for the same inputs (tests/golden/make_golden_gpu.py, run on a B200).  Both accumulate in fp32 and
    round once to bf16, in different summation orders: nearly every output is bit-identical, the rest differ by one
    bf16 step; the fp32 feature gradient (summed by atomics in the reference) agrees to fp32 rounding."""
    d = np.load(path)
    G, L, D = int(d["G"]), int(d["L"]), int(d["D"])
    loc = torch.from_numpy(d["loc"])
    X, W, bias, dY = (_bf16(d[k]) for k in ("X", "W", "bias", "dY"))

    def check_bf16(got, want_bits, what):
        gb = fo._bf16_to_bits(got)
        same = gb == want_bits
        assert same.mean() >= 0.995, f"{what}: only {same.mean():.4f} bit-identical"
        g, w = px.bf16_bits_to_f32(gb).astype(np.float64), px.bf16_bits_to_f32(want_bits).astype(np.float64)
        step = np.exp2(np.floor(np.log2(np.maximum(np.abs(w), 1e-30))) - 7)
        assert (np.abs(g - w) <= step + 1e-12)[~same].all(), f"{what}: a difference exceeds one bf16 step"

    check_bf16(fo.forward(loc, X, W, bias, G, round_bf16=True), d["Z"], "forward")
    check_bf16(fo.backward_weights(loc, X, dY, G, L, round_bf16=True), d["dW"], "backward-weights")
    dxt = fo.backward_features(loc, W, dY, G, D)
    want = torch.from_numpy(d["dXt"])
    assert torch.allclose(dxt, want, rtol=1e-5, atol=1e-5 * float(want.abs().max())), "backward-features"
