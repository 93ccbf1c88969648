"""Autograd op of the grouped fixed-fan-in product (mirrors shared_ffi/bindings.py:8-54)."""
from typing import Any, Optional

import torch

from .. import ffi as _ffi


class GroupFFIMulFunction(torch.autograd.Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx: Any, features: torch.Tensor, weights: torch.Tensor, group_locations: torch.Tensor,
                bias: Optional[torch.Tensor], gsize: int = 32) -> torch.Tensor:
        # The kernels compute in bf16 with fp32 accumulation; fp32 activations are cast at the boundary
        # (the reference's fp32 kernels silently compute in fp16, which is not imitated).
        ctx.in_dtype = features.dtype
        feats = features if features.dtype == torch.bfloat16 else features.to(torch.bfloat16)
        features_t = _ffi.transpose_bf16(feats.contiguous())
        ctx.save_for_backward(features_t, weights, group_locations)
        ctx.gsize = int(gsize)
        ctx.use_bias = bias is not None
        return _ffi.forward(group_locations, features_t, weights, bias, int(gsize))

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, grad_output):
        features_t, weights, group_locations = ctx.saved_tensors
        gsize = ctx.gsize
        if grad_output.dtype != torch.bfloat16:
            grad_output = grad_output.to(torch.bfloat16)
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        need_b = ctx.use_bias and ctx.needs_input_grad[3]
        input_gradient = weight_gradient = bias_gradient = None
        if need_x and need_w:
            # both gradients from one pass over grad_output
            dxt, weight_gradient, bias_gradient = _ffi.backward_both(features_t, weights, group_locations, grad_output, gsize,
                                                                     want_dbias=bool(need_b))
            input_gradient = _ffi.dxt_to_dx_sr(dxt, 123)
            if ctx.in_dtype != torch.bfloat16:
                input_gradient = input_gradient.to(ctx.in_dtype)
            return input_gradient, weight_gradient, None, bias_gradient, None
        if need_x:
            dxt = _ffi.backward_features(features_t, weights, group_locations, grad_output, gsize)
            # bindings.py:44-50 of the reference: transpose, then stochastic rounding with the fixed seed 123
            input_gradient = _ffi.dxt_to_dx_sr(dxt, 123)
            if ctx.in_dtype != torch.bfloat16:
                input_gradient = input_gradient.to(ctx.in_dtype)
        if need_w or need_b:
            weight_gradient, bias_gradient = _ffi.backward_weights(features_t, weights, group_locations, grad_output, gsize,
                                                                   want_dbias=True)
            if not need_b:
                bias_gradient = None
        return input_gradient, weight_gradient, None, bias_gradient, None
