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
