"""Drop-in mirror of the reference's ``shared_ffi`` package on the B200 kernels.

Same names, argument meaning and error behaviour as shared_ffi/__init__.py:3-33 of the reference:
``features`` is the TRANSPOSED feature matrix [D,B]; B, H(=D), FANIN and L are read from tensor sizes.
``_C`` stands in for the pybind11 module of ffi_wrapper.cpp:28-45.
"""
from types import SimpleNamespace

from .. import ffi as _ffi


def _ffi_forward_cuda(locations, features, weights, bias, B, H, FANIN, L, gsize=32):
    return _ffi.forward(locations, features, weights, bias, int(gsize))


def _ffi_backward_features_cuda(features, weights, locations, grad_outputs, B, H, FANIN, L, gsize=32):
    return _ffi.backward_features(features, weights, locations, grad_outputs, int(gsize))


def _ffi_backward_weights_cuda(features, weights, locations, grad_outputs, B, H, FANIN, L, gsize=32):
    return _ffi.backward_weights(features, weights, locations, grad_outputs, int(gsize))


_C = SimpleNamespace(ffi_forward_cuda=_ffi_forward_cuda,
                     ffi_backward_features_cuda=_ffi_backward_features_cuda,
                     ffi_backward_weights_cuda=_ffi_backward_weights_cuda)


def ffi_forward(locations, features, weights, bias=None, gsize=32):
    B, H = features.size(1), features.size(0)
    FANIN, L = weights.size(1), weights.size(0)
    return _C.ffi_forward_cuda(locations, features, weights, bias, int(B), int(H), int(FANIN), int(L), int(gsize))


def backward_features(features, weights, locations, grad_outputs, gsize=32):
    B, H = features.size(1), features.size(0)
    FANIN, L = weights.size(1), weights.size(0)
    return _C.ffi_backward_features_cuda(features, weights, locations, grad_outputs, int(B), int(H), int(FANIN), int(L), int(gsize))


def backward_weights(features, weights, locations, grad_outputs, gsize=32):
    B, H = features.size(1), features.size(0)
    FANIN, L = weights.size(1), weights.size(0)
    return _C.ffi_backward_weights_cuda(features, weights, locations, grad_outputs, int(B), int(H), int(FANIN), int(L), int(gsize))


from . import bindings, ops, sr_triton, optim_sr, rewire  # noqa: E402,F401
from .ops import group_ffi_mul  # noqa: E402,F401
from .optim_sr import SRSgd  # noqa: E402,F401
from .rewire import GroupFixedFanIn, GroupFixedFanInReal  # noqa: E402,F401
