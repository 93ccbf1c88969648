"""``stochastic_rounding`` and ``sgd_update`` with the reference's signatures (shared_ffi/sr_triton.py:51-59,
172-213), running on the CUDA kernels — the module keeps its historical name so ``from shared_ffi.sr_triton
import sgd_update`` keeps working; no Triton is involved.

Random bits follow the reference's stream (Philox4x32-10 keyed by ``seed``, counter = flat element index),
so results are bit-identical to the reference's kernels for the same inputs.
"""
import torch

from .. import ffi as _ffi


def stochastic_rounding(x, output, seed):
    assert x.is_contiguous()
    assert output.is_contiguous()
    assert x.shape == output.shape
    assert x.dtype == torch.float32
    assert output.dtype != torch.float32
    if output.dtype != torch.bfloat16:
        raise RuntimeError("stochastic_rounding: only bfloat16 outputs are supported")
    _ffi.sr_round(x, output, int(seed))


def sgd_update(weights: torch.Tensor, gradient: torch.Tensor, momentum_buf: torch.Tensor, learning_rate: float,
               weight_decay: float, momentum: float, use_momentum: bool, stochastic_rounding: bool, seed: int,
               *, rng: str = "reference", step: int = 0, contract: bool = True, row0: int = 0):
    """Fused SGD + weight decay + optional momentum + stochastic rounding, in place on ``weights`` (bf16).

    Keyword-only extras (not in the reference): ``rng='packed'`` selects the cheaper random stream keyed by
    (seed, step); ``contract=False`` rounds multiply and add separately; ``row0`` is the global index of the
    first row when ``weights`` is a shard.
    """
    assert weights.is_contiguous(), "weights must be contiguous"
    assert gradient.is_contiguous(), "gradient must be contiguous"
    if weights.dtype != torch.bfloat16:
        raise RuntimeError("sgd_update: weights must be bfloat16")
    if gradient.dtype != torch.bfloat16:
        gradient = gradient.to(torch.bfloat16)
    use_mom = bool(use_momentum and momentum != 0.0)
    if use_mom:
        assert momentum_buf is not None and momentum_buf.is_contiguous(), "momentum_buf must be contiguous"
        assert weights.shape == gradient.shape == momentum_buf.shape
    flags = _ffi.make_flags(sr=bool(stochastic_rounding), contract=contract, rng=rng)
    _ffi.sgd_sr_update(weights, gradient, momentum_buf if use_mom else None, int(row0), float(learning_rate),
                       float(weight_decay), float(momentum) if use_mom else 0.0, int(seed), int(step), flags)
