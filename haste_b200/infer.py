"""Inference helpers for the FFI layer: per-row top-k labels without materialising the [B, L] logits.

The reference's evaluation computes all logits and calls ``torch.topk(logits, 100)`` (src/evaluate.py:151-156;
``topk(5)`` at :219).  At 670 K labels and a batch of 512 that matrix is 686 MB.  Here the label groups are
processed in chunks sized to stay in L2: the forward kernel writes one chunk of logits, ``haste_topk_update`` folds
it into the running top-k of every row, and the chunk buffer is reused.
"""
import torch

from . import ffi as _ffi


def ffi_topk(group_locations, weights, bias, features, k, group_size, *, groups_per_chunk=None, label0=0):
    """Top-k logits and label ids of every row of ``features`` [B, D] (bf16, CUDA) under the FFI layer
    (``group_locations`` int32 [NG, F], ``weights`` bf16 [L, F], ``bias`` bf16 [L] or None).

    Returns ``(values fp32 [B, k] descending, labels int32 [B, k])``; equal logits are ordered by label id, which
    makes the result unique (``torch.topk`` leaves that order open).  ``label0`` is added to the label ids (for a
    shard of a larger layer).  1 <= k <= 128.
    """
    if not 1 <= k <= 128:
        raise ValueError("k must be in [1, 128]")
    B, D = features.shape
    L, F = weights.shape
    G = int(group_size)
    NG = (L + G - 1) // G
    dev = features.device
    if groups_per_chunk is None:
        # about 64 MB of logits per chunk (well inside the 126 MB L2), in whole waves of one group per SM
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        per_group = B * G * 2
        groups_per_chunk = max(sms, (64 << 20) // per_group // sms * sms)
    xt = _ffi.transpose_bf16(features)
    vals = torch.full((B, k), float("-inf"), dtype=torch.float32, device=dev)
    idx = torch.full((B, k), -1, dtype=torch.int32, device=dev)
    # one library call walks the chunks (forward kernel, then the running top-k kernel, per chunk) on the current stream
    groups_per_chunk = min(int(groups_per_chunk), NG)
    zbuf = torch.empty(B, groups_per_chunk * G, dtype=torch.bfloat16, device=dev)
    _ffi.topk(group_locations, xt, weights, bias, zbuf, groups_per_chunk, k, G, label0, vals, idx)
    return vals, idx
