"""Tensor-level wrappers over the C ABI: extract pointers, sizes and the current stream, nothing else.

PyTorch is used for device memory and streams only.  Every function validates what the C side cannot
see (device, dtype, contiguity) and raises RuntimeError otherwise.
"""
import torch

from . import _lib
from ._lib import lib, check


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _req(t, name, dtype=None, contiguous=True):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (this library has no CPU path)")
    if dtype is not None and t.dtype != dtype:
        hint = (" (the kernels compute in bf16 with fp32 accumulation only: create the layer's parameters with "
                "dtype=torch.bfloat16 / run it under amp.dtype=bfloat16)") if dtype == torch.bfloat16 else ""
        raise RuntimeError(f"{name} must be {dtype}, got {t.dtype}{hint}")
    if contiguous and not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    return t


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def make_flags(sr=True, contract=True, rng="reference", zero_dxt=False, loss=False):
    if rng not in ("reference", "packed"):
        raise ValueError("rng must be 'reference' or 'packed'")
    return ((_lib.F_SR if sr else 0) | (_lib.F_CONTRACT if contract else 0) | (_lib.F_RNG_PACKED if rng == "packed" else 0)
            | (_lib.F_ZERO_DXT if zero_dxt else 0) | (_lib.F_LOSS if loss else 0))


def transpose_bf16(x):
    _req(x, "x", torch.bfloat16)
    B, D = x.shape
    xt = torch.empty(D, B, dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.haste_transpose_bf16(_ptr(x), _ptr(xt), B, D, _stream(x)), "transpose_bf16")
    return xt


def forward(loc, xt, w, bias, G):
    """z [B, L] (a view of a [B, ceil8(L)] buffer, like the reference's narrow())."""
    _req(loc, "locations", torch.int32); _req(xt, "features", torch.bfloat16); _req(w, "weights", torch.bfloat16)
    if bias is not None:
        _req(bias, "bias", torch.bfloat16)
    D, B = xt.shape
    L, F = w.shape
    ldz = (L + 7) // 8 * 8
    z = torch.empty(B, ldz, dtype=torch.bfloat16, device=xt.device)
    with torch.cuda.device(xt.device):
        check(lib.haste_ffi_forward(_ptr(loc), _ptr(xt), _ptr(w), _ptr(bias), _ptr(z), B, D, F, L, G, ldz, _stream(xt)),
              "ffi_forward")
    return z.narrow(1, 0, L)


def forward_into(loc, xt, w, bias, G, out, col0):
    """Write the logits into columns col0 .. col0+L-1 of ``out`` (bf16 [B, ld], row stride ld): no intermediate
    tensor, no concatenation.  Nothing outside that column block is written."""
    _req(loc, "locations", torch.int32); _req(xt, "features", torch.bfloat16); _req(w, "weights", torch.bfloat16)
    _req(out, "out", torch.bfloat16, contiguous=False)
    if bias is not None:
        _req(bias, "bias", torch.bfloat16)
    D, B = xt.shape
    L, F = w.shape
    if out.dim() != 2 or out.shape[0] != B or out.stride(1) != 1 or col0 < 0 or col0 + L > out.shape[1]:
        raise RuntimeError(f"out must be [B={B}, >= {col0 + L}] with unit column stride")
    with torch.cuda.device(xt.device):
        check(lib.haste_ffi_forward_into(_ptr(loc), _ptr(xt), _ptr(w), _ptr(bias), out.data_ptr() + 2 * col0, B, D, F, L, G,
                                         out.stride(0), L, _stream(xt)), "ffi_forward_into")
    return out


def _rows(dy, L):
    _req(dy, "grad_outputs", torch.bfloat16, contiguous=False)
    if dy.dim() != 2 or dy.shape[1] != L:
        raise RuntimeError(f"grad_outputs must be [B,{L}]")
    if dy.stride(1) != 1:
        dy = dy.contiguous()
    return dy, dy.stride(0)


def backward_features(xt, w, loc, dy, G):
    """dxt fp32 [D,B]."""
    _req(loc, "locations", torch.int32); _req(w, "weights", torch.bfloat16)
    D, B = xt.shape
    L, F = w.shape
    dy, ldy = _rows(dy, L)
    dxt = torch.empty(D, B, dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        check(lib.haste_ffi_backward_features(_ptr(w), _ptr(loc), _ptr(dy), _ptr(dxt), B, D, F, L, G, ldy, _lib.F_ZERO_DXT,
                                              _stream(w)), "ffi_backward_features")
    return dxt


def backward_weights(xt, w, loc, dy, G, want_dbias=False):
    """dw bf16 [L,F] (and dbias bf16 [L] when asked)."""
    _req(loc, "locations", torch.int32); _req(xt, "features", torch.bfloat16)
    D, B = xt.shape
    L, F = w.shape
    dy, ldy = _rows(dy, L)
    dw = torch.empty(L, F, dtype=torch.bfloat16, device=xt.device)
    db = torch.empty(L, dtype=torch.bfloat16, device=xt.device) if want_dbias else None
    with torch.cuda.device(xt.device):
        check(lib.haste_ffi_backward_weights(_ptr(xt), _ptr(loc), _ptr(dy), _ptr(dw), _ptr(db), B, D, F, L, G, ldy, _stream(xt)),
              "ffi_backward_weights")
    return (dw, db) if want_dbias else dw


def backward_both(xt, w, loc, dy, G, want_dbias=True):
    """(dxt fp32 [D,B], dw bf16 [L,F], dbias bf16 [L] or None) from one pass over dy where the shape allows."""
    _req(loc, "locations", torch.int32); _req(xt, "features", torch.bfloat16); _req(w, "weights", torch.bfloat16)
    D, B = xt.shape
    L, F = w.shape
    dy, ldy = _rows(dy, L)
    dev = xt.device
    with torch.cuda.device(dev):
        dxt = torch.empty(D, B, dtype=torch.float32, device=dev)
        dw = torch.empty(L, F, dtype=torch.bfloat16, device=dev)
        db = torch.empty(L, dtype=torch.bfloat16, device=dev) if want_dbias else None
        check(lib.haste_ffi_backward(_ptr(xt), _ptr(w), _ptr(loc), _ptr(dy), _ptr(dxt), _ptr(dw), _ptr(db), B, D, F, L, G, ldy,
                                     _lib.F_ZERO_DXT, _stream(xt)), "ffi_backward")
    return dxt, dw, db


def bww_sr_sgd(xt, loc, dy, w, bias, mom_w, mom_b, G, label0, lr, wd, mu, seed, step, flags):
    _req(loc, "locations", torch.int32); _req(xt, "features", torch.bfloat16); _req(w, "weights", torch.bfloat16)
    D, B = xt.shape
    L, F = w.shape
    dy, ldy = _rows(dy, L)
    with torch.cuda.device(xt.device):
        check(lib.haste_ffi_bww_sr_sgd(_ptr(xt), _ptr(loc), _ptr(dy), _ptr(w), _ptr(bias), _ptr(mom_w), _ptr(mom_b), B, D, F, L, G,
                                       ldy, label0, lr, wd, mu, seed, step, flags, _stream(xt)), "ffi_bww_sr_sgd")


def targets_bucket(coo, label0, L, G, tgt_ptr, tgt_ent, scratch):
    _req(coo, "targets", torch.int32)
    nnz = coo.shape[0]
    NG = (L + G - 1) // G
    if tgt_ptr.numel() < NG + 1 or scratch.numel() < NG or tgt_ent.numel() < nnz:
        raise RuntimeError("targets_bucket: output buffers too small")
    with torch.cuda.device(coo.device):
        check(lib.haste_targets_bucket(_ptr(coo), nnz, label0, L, G, _ptr(tgt_ptr), _ptr(tgt_ent), _ptr(scratch), _stream(coo)),
              "targets_bucket")


def step_prepare(x, xt, dxt, loss, coo, label0, L, G, tgt_ptr, tgt_ent):
    """One launch: xt <- x^T, dxt <- 0, loss <- 0, targets bucketed into (tgt_ptr, tgt_ent)."""
    _req(x, "x", torch.bfloat16); _req(xt, "xt", torch.bfloat16); _req(dxt, "dxt", torch.float32); _req(coo, "targets", torch.int32)
    B, D = x.shape
    nnz = coo.shape[0]
    if tgt_ent.numel() < nnz:
        raise RuntimeError("step_prepare: tgt_ent too small")
    with torch.cuda.device(x.device):
        check(lib.haste_ffi_step_prepare(_ptr(x), _ptr(xt), _ptr(dxt), _ptr(loss), _ptr(coo), nnz, label0, L, G, _ptr(tgt_ptr),
                                         _ptr(tgt_ent), B, D, _stream(x)), "ffi_step_prepare")


def step_prepare_on(stream_handle, x, xt, dxt, loss, coo, label0, L, G, tgt_ptr, tgt_ent):
    """``step_prepare`` on an explicit stream (a ``cudaStream_t`` as int) with the tensors' device current: the
    per-step path of the pipelined multi-GPU step, where dtype / contiguity are checked once by the caller."""
    B, D = x.shape
    check(lib.haste_ffi_step_prepare(x.data_ptr(), xt.data_ptr(), dxt.data_ptr(), loss.data_ptr(), coo.data_ptr(), coo.shape[0], label0, L, G,
                                     tgt_ptr.data_ptr(), tgt_ent.data_ptr(), B, D, stream_handle), "ffi_step_prepare")


def train_step_on(stream_handle, loc, xt, w, bias, mom_w, mom_b, tgt_ptr, tgt_ent, dxt, loss, G, label0, loss_kind, grad_scale, lr, wd, mu,
                  seed, step, flags):
    """``train_step`` on an explicit stream with the tensors' device current (see ``step_prepare_on``)."""
    D, B = xt.shape
    L, F = w.shape
    check(lib.haste_ffi_train_step(loc.data_ptr(), xt.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(mom_w), _ptr(mom_b), tgt_ptr.data_ptr(),
                                   tgt_ent.data_ptr(), dxt.data_ptr(), _ptr(loss), B, D, F, L, G, label0, loss_kind, grad_scale, lr, wd, mu,
                                   seed, step, flags, stream_handle), "ffi_train_step")


def train_step(loc, xt, w, bias, mom_w, mom_b, tgt_ptr, tgt_ent, dxt, loss, G, label0, loss_kind, grad_scale, lr, wd, mu,
               seed, step, flags):
    _req(loc, "locations", torch.int32); _req(xt, "features", torch.bfloat16); _req(w, "weights", torch.bfloat16)
    _req(dxt, "dxt", torch.float32)
    D, B = xt.shape
    L, F = w.shape
    with torch.cuda.device(xt.device):
        check(lib.haste_ffi_train_step(_ptr(loc), _ptr(xt), _ptr(w), _ptr(bias), _ptr(mom_w), _ptr(mom_b), _ptr(tgt_ptr),
                                       _ptr(tgt_ent), _ptr(dxt), _ptr(loss), B, D, F, L, G, label0, loss_kind, grad_scale, lr, wd,
                                       mu, seed, step, flags, _stream(xt)), "ffi_train_step")


def step(x, coo, loc, xt, w, bias, mom_w, mom_b, tgt_ptr, tgt_ent, dxt, loss, G, label0, loss_kind, grad_scale, lr, wd, mu, seed, step_no,
         flags):
    """Preparation + fused step in one library call (the per-step path of ``FusedFFIShard.step``: argument checks are
    the caller's, done once when the buffers are created)."""
    B, D = x.shape
    L, F = w.shape
    with torch.cuda.device(x.device):
        check(lib.haste_ffi_step(_ptr(x), _ptr(coo), coo.shape[0], _ptr(loc), _ptr(xt), _ptr(w), _ptr(bias), _ptr(mom_w), _ptr(mom_b),
                                 _ptr(tgt_ptr), _ptr(tgt_ent), _ptr(dxt), _ptr(loss), B, D, F, L, G, label0, loss_kind, grad_scale, lr, wd,
                                 mu, seed, step_no, flags, _stream(x)), "ffi_step")


def train_step_dbg(loc, xt, w, bias, tgt_ptr, tgt_ent, dxt, loss, G, label0, loss_kind, grad_scale, lr, wd, seed, step, flags):
    """The fused step with debug outputs: returns (z bf16 [B,L], dw bf16 [L,F], dbias bf16 [L])."""
    _req(loc, "locations", torch.int32); _req(xt, "features", torch.bfloat16); _req(w, "weights", torch.bfloat16)
    D, B = xt.shape
    L, F = w.shape
    z = torch.zeros(B, L, dtype=torch.bfloat16, device=xt.device)
    dw = torch.zeros(L, F, dtype=torch.bfloat16, device=xt.device)
    db = torch.zeros(L, dtype=torch.bfloat16, device=xt.device)
    with torch.cuda.device(xt.device):
        check(lib.haste_ffi_train_step_dbg(_ptr(loc), _ptr(xt), _ptr(w), _ptr(bias), None, None, _ptr(tgt_ptr), _ptr(tgt_ent),
                                           _ptr(dxt), _ptr(loss), B, D, F, L, G, label0, loss_kind, grad_scale, lr, wd, 0.0, seed,
                                           step, flags, _ptr(z), L, _ptr(dw), _ptr(db) if bias is not None else None, _stream(xt)),
              "ffi_train_step_dbg")
    return z, dw, db


def sr_round(x, out, seed):
    _req(x, "x", torch.float32); _req(out, "output", torch.bfloat16)
    with torch.cuda.device(x.device):
        check(lib.haste_sr_round(_ptr(x), _ptr(out), x.numel(), seed, _stream(x)), "sr_round")


def sgd_sr_update(w, grad, mom, row0, lr, wd, mu, seed, step, flags):
    _req(w, "weights", torch.bfloat16); _req(grad, "gradient", torch.bfloat16)
    rows = w.shape[0] if w.dim() >= 1 else 1
    cols = w.numel() // max(rows, 1) if w.dim() >= 2 else 1
    with torch.cuda.device(w.device):
        check(lib.haste_sgd_sr_update(_ptr(w), _ptr(grad), _ptr(mom), rows, cols, row0, lr, wd, mu, seed, step, flags, _stream(w)),
              "sgd_sr_update")


def dxt_to_dx_sr(dxt, seed=123):
    _req(dxt, "dxt", torch.float32)
    D, B = dxt.shape
    dx = torch.empty(B, D, dtype=torch.bfloat16, device=dxt.device)
    with torch.cuda.device(dxt.device):
        check(lib.haste_dxt_to_dx_sr(_ptr(dxt), _ptr(dx), B, D, seed, _stream(dxt)), "dxt_to_dx_sr")
    return dx


def rewire(w, loc, mom_w, D, G, group0, prune_mode, threshold, n_prune, regrow_mode, init_mode, regroup, seed, step, changed=None):
    _req(w, "weights", torch.bfloat16); _req(loc, "group_locations", torch.int32)
    L, F = w.shape
    with torch.cuda.device(w.device):
        check(lib.haste_ffi_rewire(_ptr(w), _ptr(loc), _ptr(mom_w), D, F, L, G, group0, prune_mode, float(threshold), int(n_prune),
                                   regrow_mode, init_mode, int(bool(regroup)), seed, step, _ptr(changed), _stream(w)), "ffi_rewire")


def rewire_scratch_words(NG, F):
    """32-bit words of device scratch for layer-wide fraction pruning (HASTE_REWIRE_SCRATCH_WORDS)."""
    return NG * F + NG + 2 + 2 * 65536 + 8


class LayerwideSelect:
    """The layer-wide fraction selection of one label shard, in phases (haste_ffi_rewire_select_*): between the phases
    the caller sums ``hist_hi`` / ``hist_lo`` over the shards and gathers ``ties``; ``apply`` then rewires the shard."""

    def __init__(self, w, G, score_mode):
        _req(w, "weights", torch.bfloat16)
        self.w, self.G, self.score_mode = w, int(G), int(score_mode)
        self.L, self.F = w.shape
        self.NG = (self.L + self.G - 1) // self.G
        self.scratch = torch.empty(rewire_scratch_words(self.NG, self.F), dtype=torch.int32, device=w.device)
        hi = self.NG * self.F + 2 + self.NG
        self.hist_hi = self.scratch[hi:hi + 65536]                 # views into the scratch: summed in place by the caller
        self.hist_lo = self.scratch[hi + 65536:hi + 2 * 65536]
        self.ties = self.scratch[hi + 2 * 65536 + 4:hi + 2 * 65536 + 5]

    def begin(self):
        with torch.cuda.device(self.w.device):
            check(lib.haste_ffi_rewire_select_begin(_ptr(self.w), self.F, self.L, self.G, self.score_mode, _ptr(self.scratch), _stream(self.w)),
                  "rewire_select_begin")

    def refine(self, k_layer):
        with torch.cuda.device(self.w.device):
            check(lib.haste_ffi_rewire_select_refine(self.F, self.L, self.G, int(k_layer), _ptr(self.scratch), _stream(self.w)), "rewire_select_refine")

    def finish(self):
        with torch.cuda.device(self.w.device):
            check(lib.haste_ffi_rewire_select_finish(self.F, self.L, self.G, _ptr(self.scratch), _stream(self.w)), "rewire_select_finish")

    def apply(self, loc, mom_w, D, group0, tie_base, regrow_mode, init_mode, regroup, seed, step, changed=None):
        _req(loc, "group_locations", torch.int32)
        with torch.cuda.device(self.w.device):
            check(lib.haste_ffi_rewire_prepared(_ptr(self.w), _ptr(loc), _ptr(mom_w), D, self.F, self.L, self.G, group0, self.score_mode,
                                                int(tie_base), regrow_mode, init_mode, int(bool(regroup)), seed, step, _ptr(self.scratch),
                                                _ptr(changed), _stream(self.w)), "rewire_prepared")


def rewire_ex(w, loc, mom_w, D, G, group0, score_mode, prune_mode, threshold, n_prune, regrow_mode, init_mode, regroup, seed, step,
              changed=None, scratch=None):
    """Rewire with 'mean'/'max' scores (0/1) and threshold / per-group fraction / layer-wide fraction pruning (0/1/2)."""
    _req(w, "weights", torch.bfloat16); _req(loc, "group_locations", torch.int32)
    L, F = w.shape
    NG = (L + G - 1) // G
    if prune_mode == 2 and scratch is None:
        scratch = torch.empty(rewire_scratch_words(NG, F), dtype=torch.int32, device=w.device)
    with torch.cuda.device(w.device):
        check(lib.haste_ffi_rewire_ex(_ptr(w), _ptr(loc), _ptr(mom_w), D, F, L, G, group0, score_mode, prune_mode, float(threshold), int(n_prune),
                                      regrow_mode, init_mode, int(bool(regroup)), seed, step, _ptr(scratch), _ptr(changed), _stream(w)),
              "ffi_rewire_ex")


def topk(loc, xt, w, bias, zbuf, groups_per_chunk, k, G, label0, vals, idx):
    """Chunked forward + running top-k of the whole layer in one library call (``zbuf``: bf16 [B, >= groups_per_chunk * G])."""
    _req(loc, "locations", torch.int32); _req(xt, "features", torch.bfloat16); _req(w, "weights", torch.bfloat16)
    _req(zbuf, "logit buffer", torch.bfloat16); _req(vals, "values", torch.float32); _req(idx, "labels", torch.int32)
    if bias is not None:
        _req(bias, "bias", torch.bfloat16)
    D, B = xt.shape
    L, F = w.shape
    with torch.cuda.device(xt.device):
        check(lib.haste_ffi_topk(_ptr(loc), _ptr(xt), _ptr(w), _ptr(bias), _ptr(zbuf), zbuf.stride(0), B, D, F, L, G, groups_per_chunk, k,
                                 label0, _ptr(vals), _ptr(idx), _stream(xt)), "ffi_topk")


def topk_update(z, C, col0, vals, idx):
    """Fold logits z[:, :C] (labels col0..col0+C-1) into the running top-k state (vals fp32 [B,k], idx int32 [B,k])."""
    _req(z, "logits", torch.bfloat16, contiguous=False); _req(vals, "vals", torch.float32); _req(idx, "idx", torch.int32)
    if z.dim() != 2 or z.stride(1) != 1:
        raise RuntimeError("logits must be [B, C] with unit column stride")
    B, k = vals.shape
    with torch.cuda.device(z.device):
        check(lib.haste_topk_update(_ptr(z), z.stride(0), B, C, col0, k, _ptr(vals), _ptr(idx), _stream(z)), "topk_update")


def check_locations(loc, D):
    _req(loc, "group_locations", torch.int32)
    with torch.cuda.device(loc.device):
        check(lib.haste_ffi_check_locations(_ptr(loc), loc.numel(), D, _stream(loc)), "check_locations")
