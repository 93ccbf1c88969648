"""``group_ffi_mul`` (mirrors shared_ffi/ops.py:7-24): flattens leading dimensions, then the autograd op."""
from typing import Optional

import torch

from . import bindings as _bindings


def group_ffi_mul(features: torch.Tensor, weights: torch.Tensor, group_locations: torch.Tensor,
                  bias: Optional[torch.Tensor], gsize: int = 32):
    if features.ndim > 2:
        original_shape = features.shape[:-1]
        reshaped = features.reshape(-1, features.shape[-1])
        result = _bindings.GroupFFIMulFunction.apply(reshaped, weights, group_locations, bias, gsize)
        return result.reshape(original_shape + (weights.shape[0],))
    return _bindings.GroupFFIMulFunction.apply(features, weights, group_locations, bias, gsize)


__all__ = ["group_ffi_mul"]
