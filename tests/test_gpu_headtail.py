"""Head/tail glue (dense head + sparse tail in one logits matrix, no concatenation) against the reference's way of
computing it: two layers, ``torch.cat`` (src/model.py:245-248), autograd through both."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(64, 256, 40, 1000, 32, 32), (128, 768, 512, 128 * 9 + 5, 64, 128), (96, 300, 37, 64 * 7 + 3, 128, 64)])
def test_headtail_matches_concatenation(shape):
    from haste_b200.headtail import HeadTailFFI, penultimate_transposed
    from haste_b200.shared_ffi.ops import group_ffi_mul
    B, D, Lh, Lt, F, G = shape
    torch.manual_seed(B + Lt)
    m = HeadTailFFI(D, D, Lh, Lt, F, group_size=G, device="cuda", prune_mode="fraction", rewire_fraction=0.1, init_mode="zero")
    with torch.no_grad():
        m.tail_layer.bias.copy_(torch.randn(Lt, device="cuda") * 0.1)
    x = torch.randn(B, D, device="cuda").to(torch.bfloat16)
    gz = (torch.randn(B, Lh + Lt, device="cuda") * 0.1).to(torch.bfloat16)

    xa = x.clone().requires_grad_(True)
    za = m(xa)
    assert za.shape == (B, Lh + Lt)
    za.backward(gz)
    got = [za.detach(), xa.grad, m.head_layer.weight.grad.clone(), m.head_layer.bias.grad.clone(), m.tail_layer.weights.grad.clone(),
           m.tail_layer.bias.grad.clone()]
    m.zero_grad()

    xb = x.clone().requires_grad_(True)
    t = m.tail_layer
    zb = torch.cat((m.head_layer(xb), group_ffi_mul(xb, t.weights, t.group_locations, t.bias, gsize=G)), dim=1)
    zb.backward(gz)
    want = [zb.detach(), xb.grad, m.head_layer.weight.grad, m.head_layer.bias.grad, t.weights.grad, t.bias.grad]
    names = ["logits", "dX", "head dW", "head dbias", "tail dW", "tail dbias"]
    for g, w, n in zip(got, want, names):
        assert g.shape == w.shape, n
        if n in ("logits", "tail dW", "tail dbias"):
            assert torch.equal(g, w), n                          # same kernels, same inputs
        else:
            # dX sums the head's and the tail's parts in a different order; the head GEMMs run on differently strided views
            assert torch.allclose(g.float(), w.float(), rtol=2e-2, atol=2e-2 * float(w.float().abs().max())), n

    # the penultimate producer writes the transposed layout directly
    P = 128
    wp, bp = (torch.randn(P, D, device="cuda") * 0.05).to(torch.bfloat16), (torch.randn(P, device="cuda") * 0.05).to(torch.bfloat16)
    xt = penultimate_transposed(x, wp, bp, relu=True)
    ref = torch.relu(torch.nn.functional.linear(x, wp, bp)).t()
    assert xt.shape == (P, B) and xt.is_contiguous()
    assert torch.allclose(xt.float(), ref.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("loss", ["bce", "squared_hinge"])
@pytest.mark.parametrize("shape", [(128, 768, 96, 128 * 9 + 5, 64, 128), (72, 256, 40, 64 * 7 + 3, 128, 64)])
def test_fused_headtail_step_matches_concatenated_autograd(shape, loss):
    """``HeadTailFusedStep`` (fused FFI step for the tail, library GEMMs for the head, no [B,L] tensor) against the
    reference's formulation: concatenated logits, one loss over [B, L], autograd (src/model.py:245-248,
    src/runner.py:469-483).  Loss and the gradients with respect to both inputs within tolerance (bf16 logits, fp32
    sums in different orders); with lr = 0 and no weight decay the step leaves every parameter untouched; with lr > 0
    the tail's weights are bit-identical to a stand-alone fused step on the same shard."""
    from haste_b200 import ffi
    from haste_b200.fused import FusedFFIShard
    from haste_b200.headtail import HeadTailFusedStep
    from oracle import ffi_oracle as fo
    B, D, Lh, Lt, F, G = shape
    inp = fo.make_inputs(B, D, Lt, F, G, 3, 1.1, seed=B + Lt, x_kind="normal", bias_zero=False)
    dev = "cuda"
    g = torch.Generator().manual_seed(7)
    hw = (torch.randn(Lh, D, generator=g) * 0.02).to(torch.bfloat16).to(dev)
    hb = (torch.randn(Lh, generator=g) * 0.1).to(torch.bfloat16).to(dev)
    x = inp["X"].to(dev)
    # targets over the global label space: head labels 0..Lh-1, tail labels Lh..Lh+Lt-1
    tail_t = inp["targets"].clone()
    tail_t[:, 1] += Lh
    head_t = torch.stack([torch.randint(0, B, (4 * B,), generator=g), torch.randint(0, Lh, (4 * B,), generator=g)], 1).unique(dim=0).to(torch.int32)
    targets = torch.cat([head_t, tail_t]).to(dev).contiguous()
    gs = 0.25

    def make(lr, wd):
        sh = FusedFFIShard(inp["loc"].to(dev), inp["W"].to(dev).clone(), inp["bias"].to(dev).clone(), G, D, label0=Lh, loss=loss, lr=lr,
                           weight_decay=wd, seed=11, rng="packed", grad_scale=gs)
        return sh, HeadTailFusedStep(hw.clone(), hb.clone(), sh)

    # ---- gradients and loss, parameters frozen
    sh, ht = make(0.0, 0.0)
    d_head_x, dxt_tail, got_loss = ht.step(x, x, targets)
    assert torch.equal(ht.hw, hw) and torch.equal(ht.hb, hb) and torch.equal(sh.w, inp["W"].to(dev))
    xa = x.clone().float().requires_grad_(True)
    xt = x.t().contiguous()
    z_tail = ffi.forward(inp["loc"].to(dev), xt, inp["W"].to(dev), inp["bias"].to(dev), G).float()
    z = torch.cat((torch.nn.functional.linear(xa.to(torch.bfloat16), hw, hb).float(), z_tail), dim=1)
    y = torch.zeros(B, Lh + Lt, dtype=torch.bool, device=dev)
    y[targets[:, 0].long(), targets[:, 1].long()] = True
    zl = z.detach().clone().requires_grad_(True)
    if loss == "bce":
        want_loss = torch.nn.functional.binary_cross_entropy_with_logits(zl, y.float(), reduction="sum") * gs
    else:
        s = torch.where(y, 1.0, -1.0)
        want_loss = (torch.clamp_min(1.0 - s * zl, 0.0) ** 2).sum() * gs
    want_loss.backward()
    gz = zl.grad.to(torch.bfloat16)
    want_d_head_x = gz[:, :Lh].float() @ hw.float()
    want_dxt_tail = ffi.backward_features(xt, inp["W"].to(dev), inp["loc"].to(dev), gz[:, Lh:].contiguous(), G)
    want_loss = float(want_loss.detach())
    assert abs(float(got_loss) - want_loss) <= 2e-3 * abs(want_loss) + 1e-3
    for got, want, name in ((d_head_x, want_d_head_x, "d head x"), (dxt_tail, want_dxt_tail, "dX tail")):
        assert torch.allclose(got, want, rtol=2e-2, atol=2e-2 * float(want.abs().max())), name

    # ---- with an update: the tail equals the stand-alone fused step, the head's weights moved against its gradient
    sh1, ht1 = make(0.05, 1e-4)
    ht1.step(x, x, targets)
    sh2 = FusedFFIShard(inp["loc"].to(dev), inp["W"].to(dev).clone(), inp["bias"].to(dev).clone(), G, D, label0=Lh, loss=loss, lr=0.05,
                        weight_decay=1e-4, seed=11, rng="packed", grad_scale=gs)
    sh2.step(x, targets)
    assert torch.equal(sh1.w, sh2.w) and torch.equal(sh1.bias, sh2.bias)
    d_hw = gz[:, :Lh].float().t() @ x.float()
    moved = (ht1.hw.float() - hw.float())
    want_moved = -0.05 * (d_hw + 1e-4 * hw.float())
    # stochastic rounding is unbiased: the mean movement matches; element-wise within one bf16 step of the new weight
    # plus the bf16 rounding of the gradient the update consumed
    assert abs(float(moved.mean()) - float(want_moved.mean())) <= 0.05 * float(want_moved.abs().mean()) + 1e-6
    tol = float(ht1.hw.float().abs().max()) * 2 ** -7 + 0.05 * float(d_hw.abs().max()) * 2 ** -8 + 1e-6
    assert float((moved - want_moved).abs().max()) <= tol
