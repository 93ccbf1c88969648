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


class HeadTailFusedStep:
    """One training step of the head/tail output layer with no [B, L] tensor in either part and no autograd graph:
    the sparse tail runs the fused FFI step (forward, loss, both backward products and the SR-SGD update in one kernel,
    ``FusedFFIShard``), the dense head — ``num_head`` frequent labels, a [B, num_head] problem — runs as library GEMMs
    around an elementwise loss gradient, and its weights take the same SR-SGD update through ``haste_sgd_sr_update``.
    The loss is separable over labels (BCE with logits summed, or the squared hinge), so the two parts only share the
    COO target list — head labels are the global ids below ``num_head``, the shard is built with ``label0 = num_head``
    and drops them, as it drops the tail labels of other shards — and the scalar loss.

    Counterpart in the reference: ``head_layer`` / ``tail_layer`` evaluated separately, ``torch.cat`` of the logits, one
    loss over [B, L] and autograd back through the concatenation (src/model.py:182-197, 245-248; src/runner.py:469-483).
    """

    def __init__(self, head_weight, head_bias, tail_shard, *, momentum_head=None):
        if tail_shard.label0 != head_weight.shape[0]:
            raise ValueError("the tail shard's label0 must equal the number of head labels")
        self.hw, self.hb, self.tail = head_weight, head_bias, tail_shard
        self.num_head = head_weight.shape[0]
        self.mom_hw = momentum_head

    def _head_targets(self, targets, B):
        y = torch.zeros(B, self.num_head, dtype=torch.bool, device=targets.device)
        t = targets[targets[:, 1] < self.num_head].long()
        y[t[:, 0], t[:, 1]] = True
        return y

    @torch.no_grad()
    def step(self, head_x, tail_x, targets, want_loss=True):
        """``head_x`` [B, Dh], ``tail_x`` [B, D] (bf16), ``targets`` int32 [nnz, 2] (row, global label id).  Returns
        (d_head_x fp32 [B, Dh], dxt_tail fp32 [D, B], loss fp32 scalar tensor or None); weights, biases and momentum are
        updated in place."""
        sh = self.tail
        B = head_x.shape[0]
        seed, step_no = sh._keys()                     # this step's random-stream keys, shared by both parts
        # ---- tail: one preparation launch + the fused kernel
        dxt_tail, loss_tail = sh.step(tail_x, targets, want_loss=want_loss)
        # ---- head: logits rounded to bf16 as the reference's are, gradient in fp32, rounded to bf16 for the products
        z = torch.nn.functional.linear(head_x, self.hw, self.hb).float()
        y = self._head_targets(targets, B)
        gs = sh.grad_scale
        if sh.loss_kind == _lib_loss("bce"):
            g = (torch.sigmoid(z) - y.float()) * gs
            loss_head = (torch.nn.functional.softplus(z) - torch.where(y, z, torch.zeros_like(z))).sum() * gs if want_loss else None
        else:
            s = torch.where(y, 1.0, -1.0)
            m = torch.clamp_min(1.0 - s * z, 0.0)
            g = -2.0 * gs * s * m
            loss_head = (m * m).sum() * gs if want_loss else None
        g = g.to(torch.bfloat16)
        d_head_x = g.float() @ self.hw.float()
        d_hw = (g.float().t() @ head_x.float()).to(torch.bfloat16)
        flags = _ffi.make_flags(sr=sh.sr, contract=sh.contract, rng=sh.rng)
        # head rows are global labels 0 .. num_head-1: row0 = 0 keeps their random bits disjoint from the tail's
        _ffi.sgd_sr_update(self.hw, d_hw, self.mom_hw, 0, sh.lr, sh.wd, sh.mu if self.mom_hw is not None else 0.0, seed, step_no, flags)
        if self.hb is not None:
            d_hb = g.float().sum(0).to(torch.bfloat16)
            _ffi.sgd_sr_update(self.hb.view(-1, 1), d_hb.view(-1, 1), None, 0, sh.lr, sh.wd, 0.0, seed ^ 0x62696173, step_no, flags)
        loss = (loss_tail.reshape(()) + loss_head) if want_loss else None
        return d_head_x, dxt_tail, loss


def _lib_loss(name):
    from .fused import LOSSES
    return LOSSES[name]
