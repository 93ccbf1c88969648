"""haste_b200 — B200 (sm_100a) kernels for the training hot path of HASTE's grouped fixed-fan-in sparse output
layer, behind the reference's Python surface.

    haste_b200.shared_ffi   drop-in mirror of the reference's ``shared_ffi`` package
    haste_b200.fused        fused train step and label sharding across GPUs
    haste_b200.ffi          tensor-level wrappers over the C ABI (include/haste_ffi.h)

Importing the compute modules requires the built ``libhaste_ffi.so``; there is no fallback path.
"""
import sys

__all__ = ["install_as_shared_ffi"]


def install_as_shared_ffi():
    """Register ``haste_b200.shared_ffi`` under the module name ``shared_ffi`` so code written against the
    reference (``import shared_ffi``, ``from shared_ffi.optim_sr import SRSgd``) runs unchanged."""
    from . import shared_ffi as pkg
    sys.modules["shared_ffi"] = pkg
    for sub in ("bindings", "ops", "sr_triton", "optim_sr", "rewire"):
        sys.modules[f"shared_ffi.{sub}"] = getattr(pkg, sub)
    return pkg
