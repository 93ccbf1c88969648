"""ctypes binding of libhaste_ffi.so (the C ABI declared in include/haste_ffi.h).

The library is the only compute path: if it is missing, importing this module raises — there is no
CPU or PyTorch fallback.  Build it with ``python -m haste_b200.build``.
"""
import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_longlong, c_uint32, c_uint64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libhaste_ffi.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} not found: the CUDA library has not been built. Run `python -m haste_b200.build` "
        "(needs nvcc; cross-compiles for sm_100a without a GPU). There is no fallback path.")

lib = ctypes.CDLL(LIB_PATH)

P, I64, F32, U64, U32, I32 = c_void_p, c_int64, c_float, c_uint64, c_uint32, c_int32

# name -> argtypes, in the order of include/haste_ffi.h
SIGNATURES = {
    "haste_ffi_forward": [P, P, P, P, P, I64, I64, I64, I64, I64, I64, P],
    "haste_ffi_forward_into": [P, P, P, P, P, I64, I64, I64, I64, I64, I64, I64, P],
    "haste_ffi_backward_features": [P, P, P, P, I64, I64, I64, I64, I64, I64, U32, P],
    "haste_ffi_backward_weights": [P, P, P, P, P, I64, I64, I64, I64, I64, I64, P],
    "haste_ffi_backward": [P, P, P, P, P, P, P, I64, I64, I64, I64, I64, I64, U32, P],
    "haste_pad_rows_bf16": [P, I64, P, I64, I64, I64, P],
    "haste_ffi_bww_sr_sgd": [P, P, P, P, P, P, P, I64, I64, I64, I64, I64, I64, I64, F32, F32, F32, U64, U32, U32, P],
    "haste_targets_bucket": [P, I64, I64, I64, I64, P, P, P, P],
    "haste_ffi_step_prepare": [P, P, P, P, P, I64, I64, I64, I64, P, P, I64, I64, P],
    "haste_targets_bucket_noalloc": [P, I64, I64, I64, I64, P, P, P],
    "haste_ffi_train_step": [P, P, P, P, P, P, P, P, P, P, I64, I64, I64, I64, I64, I64, I32, F32, F32, F32, F32, U64,
                             U32, U32, P],
    "haste_ffi_train_step_dbg": [P, P, P, P, P, P, P, P, P, P, I64, I64, I64, I64, I64, I64, I32, F32, F32, F32, F32, U64,
                                 U32, U32, P, I64, P, P, P],
    "haste_sr_round": [P, P, I64, U64, P],
    "haste_sgd_sr_update": [P, P, P, I64, I64, I64, F32, F32, F32, U64, U32, U32, P],
    "haste_dxt_to_dx_sr": [P, P, I64, I64, U64, P],
    "haste_transpose_bf16": [P, P, I64, I64, P],
    "haste_ffi_rewire": [P, P, P, I64, I64, I64, I64, I64, I32, F32, I32, I32, I32, I32, U64, U32, P, P],
    "haste_ffi_rewire_ex": [P, P, P, I64, I64, I64, I64, I64, I32, I32, F32, I64, I32, I32, I32, U64, U32, P, P, P],
    "haste_ffi_rewire_select_begin": [P, I64, I64, I64, I32, P, P],
    "haste_ffi_rewire_select_refine": [I64, I64, I64, I64, P, P],
    "haste_ffi_rewire_select_finish": [I64, I64, I64, P, P],
    "haste_ffi_rewire_prepared": [P, P, P, I64, I64, I64, I64, I64, I32, U32, I32, I32, I32, U64, U32, P, P, P],
    "haste_ffi_step": [P, P, I64, P, P, P, P, P, P, P, P, P, P, I64, I64, I64, I64, I64, I64, I32, F32, F32, F32, F32, U64, U32, U32, P],
    "haste_topk_update": [P, I64, I64, I64, I64, I32, P, P, P],
    "haste_ffi_topk": [P, P, P, P, P, I64, I64, I64, I64, I64, I64, I64, I32, I64, P, P, P],
    "haste_ffi_check_locations": [P, I64, I64, P],
    "haste_ffi_set_max_ctas": [I32],
    "haste_poll_status": [],
    "haste_debug_set_wait_limit": [c_longlong],
    "haste_debug_stall_next_step": [I32],
    "haste_debug_set_dependent_launch": [I32],
    "haste_probe_red_rate": [P, I64, I64, I32, I32, P],
    "haste_probe_gather_rate": [P, I64, I64, I32, I32, P],
    "haste_probe_umma_rate": [I32, I32, I32, I32, P, P],
}

for _name, _args in SIGNATURES.items():
    _fn = getattr(lib, _name)          # AttributeError here = the library does not export the symbol
    _fn.argtypes = _args
    _fn.restype = c_int
lib.haste_last_error_string.restype = c_char_p
lib.haste_last_error_string.argtypes = []
lib.haste_version.restype = c_int
lib.haste_version.argtypes = []

# status codes and flags (include/haste_ffi.h)
OK, ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_INDEX_RANGE, ERR_LAUNCH, ERR_TIMEOUT, ERR_TOO_LARGE = range(7)
LOSS_BCE, LOSS_SQHINGE = 0, 1
F_SR, F_CONTRACT, F_RNG_PACKED, F_ZERO_DXT, F_LOSS = 1, 2, 4, 8, 16


def last_error():
    return lib.haste_last_error_string().decode()


def check(status, what=""):
    """Raise RuntimeError (the reference's TORCH_CHECK convention) on a non-zero status."""
    if status != 0:
        raise RuntimeError(f"{what}: haste status {status}: {last_error()}")
