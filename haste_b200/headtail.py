"""Head/tail output layer: a dense layer over the frequent ("head") labels next to the fixed-fan-in sparse layer over
the rest, producing ONE logits matrix [B, L_head + L_tail].

The reference computes the two parts separately and concatenates them (src/model.py:182-197 builds ``head_layer`` =
nn.Linear and ``tail_layer`` = GroupFixedFanInReal; :245-248 ``torch.cat((head_logits, tail_logits), dim=1)``), which
copies the [B, L_tail] tail logits once more, and autograd splits the gradient the same way on the way back.  Here the
sparse kernel writes its logits straight into the tail columns of the output buffer (``haste_ffi_forward_into``) and
the backward kernels read the tail columns of the incoming gradient in place (row stride = the full width), so no
[B, L_tail] copy exists in either direction.  The dense head is a plain library GEMM.

``penultimate_transposed`` is the producer on the other side of the path: the penultimate Linear (+ ReLU) of the
reference (src/model.py:157-161, 242-243) evaluated as W·Xᵀ, which yields the [D,B] layout the sparse kernels take
as input and saves the transpose pass.
"""
import torch

from . import ffi as _ffi
from .shared_ffi.rewire import GroupFixedFanInReal


class _HeadTailFunction(torch.autograd.Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, head_in, tail_in, head_w, head_b, tail_w, tail_loc, tail_b, gsize):
        B = tail_in.shape[0]
        Lh, Lt = head_w.shape[0], tail_w.shape[0]
        ld = (Lh + Lt + 7) // 8 * 8
        out = torch.empty(B, ld, dtype=torch.bfloat16, device=tail_in.device)
        tail_bf = tail_in if tail_in.dtype == torch.bfloat16 else tail_in.to(torch.bfloat16)
        xt = _ffi.transpose_bf16(tail_bf.contiguous())
        _ffi.forward_into(tail_loc, xt, tail_w, tail_b, int(gsize), out, Lh)          # tail columns, in place
        head_bf = head_in if head_in.dtype == torch.bfloat16 else head_in.to(torch.bfloat16)
        out[:, :Lh] = torch.nn.functional.linear(head_bf, head_w, head_b)             # [B, L_head]: the small part
        if ld > Lh + Lt:
            out[:, Lh + Lt:].zero_()
        ctx.save_for_backward(head_bf, xt, head_w, tail_w, tail_loc)
        ctx.gsize, ctx.Lh, ctx.Lt = int(gsize), Lh, Lt
        ctx.has_hb, ctx.has_tb = head_b is not None, tail_b is not None
        ctx.in_dtypes = (head_in.dtype, tail_in.dtype)
        return out.narrow(1, 0, Lh + Lt)

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, gz):
        head_bf, xt, head_w, tail_w, tail_loc = ctx.saved_tensors
        Lh, Lt = ctx.Lh, ctx.Lt
        if gz.dtype != torch.bfloat16:
            gz = gz.to(torch.bfloat16)
        if gz.stride(1) != 1:
            gz = gz.contiguous()
        g_head, g_tail = gz[:, :Lh], gz[:, Lh:Lh + Lt]                # views: the kernels take the row stride
        d_head_in = (g_head @ head_w).to(ctx.in_dtypes[0])
        d_head_w = g_head.t() @ head_bf
        d_head_b = g_head.sum(0) if ctx.has_hb else None
        dxt, d_tail_w, d_tail_b = _ffi.backward_both(xt, tail_w, tail_loc, g_tail, ctx.gsize, want_dbias=ctx.has_tb)
        d_tail_in = _ffi.dxt_to_dx_sr(dxt, 123)                       # as the reference's autograd op rounds dX (bindings.py:44-50)
        if ctx.in_dtypes[1] != torch.bfloat16:
            d_tail_in = d_tail_in.to(ctx.in_dtypes[1])
        return d_head_in, d_tail_in, d_head_w, d_head_b, d_tail_w, None, d_tail_b, None


class HeadTailFFI(torch.nn.Module):
    """``head_layer`` (dense, ``num_head`` labels) and ``tail_layer`` (``GroupFixedFanInReal``, ``num_tail`` labels) with
    the attribute names of the reference's model, evaluated into one logits matrix without a concatenation.
    ``forward(head_features, tail_features)``; pass the same tensor twice when both read the same features."""

    def __init__(self, head_in_features, tail_in_features, num_head, num_tail, fan_in, *, group_size=32, device=None, dtype=torch.bfloat16,
                 **tail_kwargs):
        super().__init__()
        self.head_layer = torch.nn.Linear(head_in_features, num_head, device=device, dtype=dtype)
        torch.nn.init.normal_(self.head_layer.weight, mean=0.0, std=0.02)            # src/model.py:185
        self.tail_layer = GroupFixedFanInReal(tail_in_features, num_tail, fan_in, bias=True, device=device, dtype=dtype,
                                              group_size=group_size, **tail_kwargs)

    def forward(self, head_features, tail_features=None):
        if tail_features is None:
            tail_features = head_features
        t = self.tail_layer
        return _HeadTailFunction.apply(head_features, tail_features, self.head_layer.weight, self.head_layer.bias, t.weights,
                                       t.group_locations, t.bias, t.group_size)

    def rewire(self):
        return self.tail_layer.rewire()


def penultimate_transposed(x, weight, bias=None, relu=True):
    """Penultimate layer evaluated directly into the transposed layout: returns act(W x^T + b) as bf16 [P, B], the
    ``xt`` the sparse kernels take (``ffi.forward`` / ``FusedFFIShard.step_xt``), instead of [B, P] followed by a
    transpose pass.  x [B, H], weight [P, H] (nn.Linear layout), bias [P] or None."""
    xt = weight.to(torch.bfloat16) @ x.to(torch.bfloat16).t()
    if bias is not None:
        xt = xt + bias.to(torch.bfloat16)[:, None]
    if relu:
        xt = torch.relu_(xt)
    return xt.contiguous()
