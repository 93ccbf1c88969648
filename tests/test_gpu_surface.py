"""GPU tests of the reference-facing Python surface (shared_ffi mirror): autograd op, optimizer, layer module,
fused shard.  Compared with the CPU oracle / plain PyTorch autograd on the same seeded inputs."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import ffi_oracle as fo


@pytest.fixture(scope="module")
def sf():
    import haste_b200
    return haste_b200.install_as_shared_ffi()


def _bits(t):
    return fo._bf16_to_bits(t.detach().cpu())


def test_install_alias(sf):
    import shared_ffi
    from shared_ffi.optim_sr import SRSgd
    from shared_ffi.sr_triton import sgd_update, stochastic_rounding
    from shared_ffi.ops import group_ffi_mul
    assert shared_ffi is sf and SRSgd is sf.SRSgd and callable(sgd_update) and callable(stochastic_rounding)


@pytest.mark.parametrize("shape", [(48, 96, 200, 32, 32), (3 * 20, 128, 333, 64, 64)])
def test_autograd_function(sf, shape):
    B, D, L, F, G = shape
    inp = fo.make_inputs(B, D, L, F, G, 3, 1.1, seed=21, x_kind="normal", bias_zero=False)
    X = inp["X"].cuda().requires_grad_(True)
    W = inp["W"].cuda().requires_grad_(True)
    bias = inp["bias"].cuda().requires_grad_(True)
    loc = inp["loc"].cuda()
    z = sf.ops.group_ffi_mul(X, W, loc, bias, G)
    assert z.shape == (B, L) and z.dtype == torch.bfloat16
    want = fo.forward(inp["loc"], inp["X"], inp["W"], inp["bias"], G, round_bf16=False)
    assert torch.allclose(z.float().cpu(), want, rtol=1e-2, atol=1e-3 * max(1.0, float(want.abs().max())))
    gen = torch.Generator().manual_seed(0)
    dY = (torch.randn(B, L, generator=gen) * 0.5).to(torch.bfloat16)
    z.backward(dY.cuda())
    dXt = fo.backward_features(inp["loc"], inp["W"], dY, G, D)
    # dX comes back in bf16 after stochastic rounding with the fixed seed 123 (bindings.py:44-50 of the reference):
    # compare with the oracle rounding of the oracle gradient within one bf16 step of its magnitude
    assert X.grad.dtype == torch.bfloat16 and X.grad.shape == (B, D)
    err = (X.grad.float().cpu() - dXt.t()).abs()
    assert float((err / (dXt.t().abs() * 2 ** -7 + 1e-3 * float(dXt.abs().max()))).max()) <= 2.0
    dW = fo.backward_weights(inp["loc"], inp["X"], dY, G, L, round_bf16=False)
    assert torch.allclose(W.grad.float().cpu(), dW, rtol=1e-2, atol=1e-3 * max(1.0, float(dW.abs().max())))
    assert torch.allclose(bias.grad.float().cpu(), dY.float().sum(0), rtol=1e-2, atol=2e-2)
    # 3-D input is flattened over its leading dimensions (ops.py:17-22 of the reference)
    z3 = sf.ops.group_ffi_mul(inp["X"].cuda().view(3, B // 3, D), W, loc, bias, G)
    assert z3.shape == (3, B // 3, L) and torch.equal(z3.reshape(B, L), z)


def test_srsgd_matches_oracle(sf):
    gen = torch.Generator().manual_seed(1)
    L, F = 300, 32
    for rng, mom in (("reference", 0.0), ("reference", 0.9), ("packed", 0.0)):
        w0 = ((torch.rand(L, F, generator=gen) * 2 - 1) / 6).to(torch.bfloat16)
        b0 = (torch.randn(L, generator=gen) * 0.1).to(torch.bfloat16)
        w = torch.nn.Parameter(w0.clone().cuda())
        b = torch.nn.Parameter(b0.clone().cuda())
        opt = sf.SRSgd([w, b], lr=0.05, weight_decay=1e-4, momentum=mom, seed=123, rng=rng)
        wo, bo = w0.clone(), b0.clone()
        mw, mb = torch.zeros(L, F), torch.zeros(L)
        for step in range(3):
            gw = (torch.randn(L, F, generator=gen) * 0.2).to(torch.bfloat16)
            gb = (torch.randn(L, generator=gen) * 0.2).to(torch.bfloat16)
            w.grad, b.grad = gw.cuda(), gb.cuda()
            opt.step()
            seed = 123 + step                      # the reference bumps the seed once per step
            rw = fo.rand16_for((L, F), seed, step, rng)
            rb = fo.rand16_for((L, 1), seed, step, rng, is_bias=True).reshape(L)
            wo, mw = fo.sgd_update(wo, gw, mw, 0.05, 1e-4, mom, True, True, rw)
            bo, mb = fo.sgd_update(bo, gb, mb, 0.05, 1e-4, mom, True, True, rb)
            assert np.array_equal(_bits(w.data), fo._bf16_to_bits(wo)), (rng, mom, step)
            assert np.array_equal(_bits(b.data), fo._bf16_to_bits(bo)), (rng, mom, step)
        assert opt.param_groups[0]["seed"] == 126
    # fp32 parameters take plain SGD
    p = torch.nn.Parameter(torch.ones(4, device="cuda"))
    opt = sf.SRSgd([p], lr=0.1, weight_decay=0.0)
    p.grad = torch.ones(4, device="cuda")
    opt.step()
    assert torch.allclose(p.data, torch.full((4,), 0.9, device="cuda"))


def test_layer_module_and_rewire(sf):
    torch.manual_seed(0)
    D, L, F, G = 128, 500, 32, 64
    layer = sf.GroupFixedFanIn(D, L, F, bias=True, device="cuda", dtype=torch.bfloat16, group_size=G, prune_mode="fraction",
                               rewire_fraction=0.25, init_mode="zero", regrow="unused", regroup=True, seed=5)
    assert layer.group_locations.shape == ((L + G - 1) // G, F) and layer.group_locations.dtype == torch.int32
    assert set(dict(layer.named_parameters())) == {"weights", "bias"} and "group_locations" in layer.state_dict()
    x = torch.randn(16, D, device="cuda", dtype=torch.bfloat16)
    y = layer(x)
    want = fo.forward(layer.group_locations.cpu(), x.cpu(), layer.weights.detach().cpu(), layer.bias.detach().cpu(), G, False)
    assert torch.allclose(y.float().cpu(), want, rtol=1e-2, atol=2e-3)
    W0, loc0 = layer.weights.detach().cpu().clone(), layer.group_locations.cpu().clone()
    n = layer.rewire()
    assert n == ((L + G - 1) // G) * int(F * 0.25)
    W1, loc1, _ = fo.rewire(W0, loc0, G, D, "fraction", 0.25, None, init_mode="zero", regrow="unused", regroup=True, seed=5, step=0)
    assert np.array_equal(layer.group_locations.cpu().numpy(), loc1.numpy())
    assert np.array_equal(_bits(layer.weights), fo._bf16_to_bits(W1))
    with pytest.raises(ValueError):
        sf.GroupFixedFanIn(D, L, F, prune_mode="fraction")
    with pytest.raises(AssertionError):
        sf.GroupFixedFanIn(D, L, F, rewire_threshold=0.1, group_size=48)


def test_fused_shard_matches_two_half_shards(sf):
    """Splitting the labels over two shards changes neither the updated weights (bit for bit: the random-bit
    counters are global) nor, up to summation order, the summed feature gradient."""
    from haste_b200.fused import FusedFFIShard, shard_labels
    B, D, L, F, G = 128, 256, 3000, 64, 128
    inp = fo.make_inputs(B, D, L, F, G, 6, 1.1, seed=77, bias_zero=False)
    x, tg = inp["X"].cuda(), inp["targets"].cuda()
    kw = dict(loss="squared_hinge", lr=0.05, weight_decay=1e-4, seed=123, rng="packed", grad_scale=0.5)
    full = FusedFFIShard(inp["loc"].cuda(), inp["W"].clone().cuda(), inp["bias"].clone().cuda(), G, D, **kw)
    dxt_full, loss_full = full.step(x, tg)
    dxt_full, loss_full = dxt_full.clone(), float(loss_full)
    dsum, lsum, ws = torch.zeros_like(dxt_full), 0.0, []
    for r in range(2):
        l0, l1, g0, g1 = shard_labels(L, G, 2, r)
        sh = FusedFFIShard(inp["loc"][g0:g1].cuda(), inp["W"][l0:l1].clone().cuda(), inp["bias"][l0:l1].clone().cuda(), G, D,
                           label0=l0, **kw)
        d, ls = sh.step(x, tg)
        dsum += d
        lsum += float(ls)
        ws.append(sh.w)
    assert torch.equal(torch.cat(ws), full.w)
    assert torch.allclose(dsum, dxt_full, rtol=1e-4, atol=1e-4 * float(dxt_full.abs().max()))
    assert abs(lsum - loss_full) <= 1e-4 * abs(loss_full)


def test_layer_real_global_rewire(sf):
    """``GroupFixedFanInReal`` (the class src/model.py builds): layer-wide fraction pruning with max scores."""
    D, L, F, G = 256, 128 * 9 + 5, 64, 128
    layer = sf.GroupFixedFanInReal(D, L, F, bias=True, device="cuda", dtype=torch.bfloat16, group_size=G, prune_mode="fraction",
                                   rewire_fraction=0.2, init_mode="zero", score_mode="max", regrow="replace", seed=9)
    W0, loc0 = layer.weights.detach().cpu().clone(), layer.group_locations.cpu().clone()
    n = layer.rewire()
    NG = loc0.shape[0]
    assert n == int(NG * F * 0.2)
    W1, loc1, _ = fo.rewire(W0, loc0, G, D, "fraction", 0.2, None, init_mode="zero", regrow="replace", regroup=False, seed=9, step=0,
                            score_mode="max", prune_scope="global")
    assert np.array_equal(layer.group_locations.cpu().numpy(), loc1.numpy())
    assert np.array_equal(fo._bf16_to_bits(layer.weights.detach().cpu()), fo._bf16_to_bits(W1))
    x = torch.randn(4, D, device="cuda", dtype=torch.bfloat16)
    assert layer(x).shape == (4, L)
