"""CPU oracle for the grouped fixed-fan-in (FFI) output layer (test infrastructure).

Notation: B batch, D input features, L labels, F fan-in, G group size,
NG = ceil(L/G).  ``loc`` int32 [NG,F]; ``X`` [B,D]; ``W`` bf16 [L,F];
``bias`` bf16 [L]; ``Z``/``dY`` [B,L].  All tensors are torch CPU tensors;
low-precision values are torch.bfloat16, arithmetic is fp32 (sums in fp64 where
the order of summation would otherwise matter for the comparison).

The math restated here, with the reference lines it follows:
  forward            shared_ffi/ffi_forward_kernels.cu:167-262 (+bias :85-93, zero pad :187-195)
  backward-features  shared_ffi/ffi_backward_features.cu:134-212
  backward-weights   shared_ffi/ffi_backward_weights.cu:166-258 (bf16 RN store :81-89)
  bias gradient      shared_ffi/bindings.py:39-42
  dX rounding        shared_ffi/bindings.py:44-50
  BCE loss           src/runner.py:469-478
  SGD + SR           shared_ffi/sr_triton.py:109-168, shared_ffi/optim_sr.py:53-62
  rewire             shared_ffi/rewire.py:143-239
"""
import math

import numpy as np
import torch

from . import philox as px

LOSS_BCE = 0
LOSS_SQHINGE = 1


# --------------------------------------------------------------------------- helpers
def _bf16_to_bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _bits_to_bf16(b):
    return torch.from_numpy(np.ascontiguousarray(b).view(np.int16).copy()).view(torch.bfloat16)


def _group_chunks(NG, per=256):
    for g0 in range(0, NG, per):
        yield g0, min(NG, g0 + per)


def _pad_rows(W, NG, G):
    """[L,F] -> [NG*G,F] float32 with zero rows past L (ffi_forward_kernels.cu:187-195)."""
    L, F = W.shape
    out = torch.zeros(NG * G, F, dtype=torch.float32)
    out[:L] = W.float()
    return out


# --------------------------------------------------------------------------- GEMM phases
def forward(loc, X, W, bias, G, round_bf16=True):
    """Z[b,l] = sum_k X[b, loc[l//G,k]] * W[l,k] (+ bias[l]); fp32 accumulate, RN to bf16."""
    B, D = X.shape
    L, F = W.shape
    NG = loc.shape[0]
    Xf = X.float()
    Wp = _pad_rows(W, NG, G).view(NG, G, F)
    Z = torch.empty(B, NG * G, dtype=torch.float32)
    for g0, g1 in _group_chunks(NG):
        Xg = Xf[:, loc[g0:g1].long()]                       # [B, ng, F]
        Z[:, g0 * G:g1 * G] = torch.einsum('bgf,gnf->bgn', Xg, Wp[g0:g1]).reshape(B, -1)
    Z = Z[:, :L]
    if bias is not None:
        Z = Z + bias.float()[None, :]
    return Z.to(torch.bfloat16) if round_bf16 else Z


def backward_features(loc, W, dY, G, D):
    """dXt[loc[g,k], b] += sum_{l in g} W[l,k] * dY[b,l]; returns fp32 [D,B] (the kernel's layout)."""
    B, L = dY.shape
    F = W.shape[1]
    NG = loc.shape[0]
    Wp = _pad_rows(W, NG, G).view(NG, G, F).double()
    dYp = torch.zeros(B, NG * G, dtype=torch.float64)
    dYp[:, :L] = dY.double()
    dYp = dYp.view(B, NG, G)
    dX = torch.zeros(B, D, dtype=torch.float64)
    for g0, g1 in _group_chunks(NG):
        dXg = torch.einsum('bgn,gnf->bgf', dYp[:, g0:g1], Wp[g0:g1])      # [B, ng, F]
        idx = loc[g0:g1].long().reshape(1, -1).expand(B, -1)
        dX.scatter_add_(1, idx, dXg.reshape(B, -1))
    return dX.t().contiguous().float()


def backward_weights(loc, X, dY, G, L, round_bf16=True):
    """dW[l,k] = sum_b dY[b,l] * X[b, loc[l//G,k]]; fp32 accumulate, RN to bf16."""
    B, D = X.shape
    NG, F = loc.shape
    Xf = X.double()
    dYp = torch.zeros(B, NG * G, dtype=torch.float64)
    dYp[:, :L] = dY.double()
    dYp = dYp.view(B, NG, G)
    dW = torch.empty(NG, G, F, dtype=torch.float64)
    for g0, g1 in _group_chunks(NG):
        Xg = Xf[:, loc[g0:g1].long()]
        dW[g0:g1] = torch.einsum('bgn,bgf->gnf', dYp[:, g0:g1], Xg)
    dW = dW.view(NG * G, F)[:L].float()
    return dW.to(torch.bfloat16) if round_bf16 else dW


def bias_grad(dY):
    """dbias = dY.sum(0) accumulated in fp32, rounded to the input dtype (bindings.py:39-42)."""
    return dY.float().sum(0).to(dY.dtype)


# --------------------------------------------------------------------------- losses
def dense_targets(targets, B, L):
    """COO [nnz,2] int32 (row, col) -> dense {0,1} fp32 [B,L] (src/data.py:38-44 builds the COO)."""
    Y = torch.zeros(B, L, dtype=torch.float32)
    if targets.numel():
        Y[targets[:, 0].long(), targets[:, 1].long()] = 1.0
    return Y


def loss_and_grad(Z, targets, loss_kind, grad_scale=1.0):
    """Loss value (fp64 python float) and dY = grad_scale * dLoss/dZ rounded to bf16.

    BCE with logits, sum reduction (src/runner.py:469-478): dY = sigmoid(z) - y.
    Squared hinge, targets +-1: loss = max(0, 1 - y z)^2, dY = -2 y max(0, 1 - y z).
    The squared hinge of the reference lives in a wheel that is not shipped
    (src/runner.py:18,483), so this definition is this project's own.
    """
    B, L = Z.shape
    z = Z.float()
    Y = dense_targets(targets, B, L)
    if loss_kind == LOSS_BCE:
        loss = (z.clamp(min=0).double().sum() - (z * Y).double().sum()
                + torch.log1p(torch.exp(-z.abs())).double().sum())
        g = torch.sigmoid(z) - Y
    elif loss_kind == LOSS_SQHINGE:
        s = 2.0 * Y - 1.0
        m = (1.0 - s * z).clamp(min=0)
        loss = (m * m).double().sum()
        g = -2.0 * s * m
    else:
        raise ValueError(loss_kind)
    return float(loss) * grad_scale, (g * grad_scale).to(torch.bfloat16)


# --------------------------------------------------------------------------- SR / SGD
def _fma32(a, b, c):
    """fp32 fused multiply-add: the product is exact in extended precision, rounded once."""
    r = (np.asarray(a, np.longdouble) * np.asarray(b, np.longdouble)) + np.asarray(c, np.longdouble)
    return r.astype(np.float32)


def sgd_math(w32, g32, m32, lr, wd, mu, use_mom, contract):
    """fp32 SGD arithmetic of sr_triton.py:140-158.  ``contract`` fuses mul+add the way the
    compiled Triton kernel does (fp fusion on); False keeps them separate (interpreter)."""
    lr32, wd32, mu32 = np.float32(lr), np.float32(wd), np.float32(mu)
    w32 = np.asarray(w32, np.float32)
    g32 = np.asarray(g32, np.float32)
    if contract:
        g2 = _fma32(wd32, w32, g32)
        if use_mom:
            m32 = _fma32(mu32, m32, g2)
            w_new = _fma32(-lr32, m32, w32)
        else:
            w_new = _fma32(-lr32, g2, w32)
    else:
        g2 = g32 + wd32 * w32
        if use_mom:
            m32 = mu32 * np.asarray(m32, np.float32) + g2
            w_new = w32 - lr32 * m32
        else:
            w_new = w32 - lr32 * g2
    return w_new.astype(np.float32), m32


def sgd_update(w, g, m, lr, wd, mu, use_mom, do_sr, r16, contract=True):
    """One fused SGD(+wd)(+momentum) step with stochastic (or RN) rounding to bf16.

    ``w``,``g`` bf16 torch tensors (any shape), ``m`` fp32 tensor or None, ``r16`` uint32 array
    of 16-bit random values with w's shape (ignored when ``do_sr`` is False).
    Returns (w_new bf16 tensor, m_new fp32 tensor or None).
    """
    use_mom = bool(use_mom and mu != 0.0)
    w32 = w.float().numpy()
    g32 = g.float().numpy()
    m32 = m.numpy().copy() if (m is not None and use_mom) else None
    w_new, m_new = sgd_math(w32, g32, m32, lr, wd, mu, use_mom, contract)
    if do_sr:
        bits = px.sr_bf16_bits(w_new, np.asarray(r16).reshape(w_new.shape))
    else:
        bits = px.rn_bf16_bits(w_new)
    out = _bits_to_bf16(bits.reshape(w32.shape))
    return out, (torch.from_numpy(np.asarray(m_new, np.float32)) if use_mom else m)


def stochastic_rounding(x32, seed):
    """sr_triton.stochastic_rounding: fp32 tensor -> bf16, reference stream over the flat index."""
    x = x32.contiguous().numpy()
    r = px.rand16_reference(seed, np.arange(x.size, dtype=np.int64)).reshape(x.shape)
    return _bits_to_bf16(px.sr_bf16_bits(x, r))


BIAS_KEY_XOR = 0x62696173   # packed stream: 1-D parameters use seed ^ this, so bias does not reuse column 0's bits


def rand16_for(shape, seed, step, mode, row0=0, is_bias=False):
    """Random 16-bit field for a [rows, cols] parameter.  mode 'reference': tl.randint stream over
    the flat index (row0 shifts to the global row); 'packed': one Philox call per 8 slots."""
    rows, cols = shape
    if mode != 'reference' and is_bias:
        seed = int(seed) ^ BIAS_KEY_XOR
    r = np.arange(rows, dtype=np.int64)[:, None] + row0
    c = np.arange(cols, dtype=np.int64)[None, :]
    if mode == 'reference':
        return px.rand16_reference(seed, r * cols + c)
    return px.rand16_packed(seed, step, r, c)


# --------------------------------------------------------------------------- whole step
def train_step(loc, X, W, bias, targets, G, loss_kind, lr, wd, seed, step=0, grad_scale=1.0,
               rng_mode='reference', contract=True, row0=0):
    """One fused training step of the layer, restated unfused:
    Z -> (loss, dY) -> dXt, dW(bf16), dbias(bf16) -> SGD+wd+SR on W and bias (momentum 0).

    ``row0``: global index of this shard's first label (label-sharded runs).
    Returns dict(Z, dY, loss, dXt, dW, W_new, bias_new).
    """
    B, D = X.shape
    L, F = W.shape
    Z = forward(loc, X, W, bias, G)
    loss, dY = loss_and_grad(Z, targets, loss_kind, grad_scale)
    dXt = backward_features(loc, W, dY, G, D)
    dW = backward_weights(loc, X, dY, G, L)
    r = rand16_for((L, F), seed, step, rng_mode, row0)
    W_new, _ = sgd_update(W, dW, None, lr, wd, 0.0, False, True, r, contract)
    out = dict(Z=Z, dY=dY, loss=loss, dXt=dXt, dW=dW, W_new=W_new, bias_new=None)
    if bias is not None:
        db = bias_grad(dY)
        rb = rand16_for((L, 1), seed, step, rng_mode, row0, is_bias=True).reshape(L)
        out['bias_new'], _ = sgd_update(bias, db, None, lr, wd, 0.0, False, True, rb, contract)
        out['dbias'] = db
    return out


# --------------------------------------------------------------------------- rewire
def rewire_scores(W, G, NG, score_mode='mean'):
    """'mean': score[g,k] = (sum over the group's real rows, in row order, of |w| in fp32) / row count
    (rewire.py:166-185; src/group_fanin_real.py:207-226).  Sequential fp32 accumulation so a kernel can
    reproduce it bit for bit.  'max': score[g,k] = max over the group's real rows of |w|
    (src/group_fanin_real.py:213-220)."""
    L, F = W.shape
    a = W.float().abs().numpy()
    scores = np.zeros((NG, F), np.float32)
    for g in range(NG):
        rows = a[g * G:min(L, (g + 1) * G)]
        if score_mode == 'max':
            scores[g] = rows.max(axis=0)
            continue
        acc = np.zeros(F, np.float32)
        for r in rows:
            acc = acc + r
        scores[g] = acc / np.float32(max(1, rows.shape[0]))
    return scores


def prune_mask(scores, prune_mode, rewire_fraction=None, rewire_threshold=None, prune_scope='group'):
    """rewire.py:187-204.  'fraction': the k = int(F*fraction) lowest scores per group, ties
    broken by lowest slot index (the reference leaves tie order to torch.topk).
    prune_scope 'global' (src/group_fanin_real.py:232-250): the k = int(NG*F*fraction) lowest scores of the
    whole layer, ties broken by lowest flat (group, slot) index."""
    NG, F = scores.shape
    if prune_mode == 'threshold':
        return scores < np.float32(rewire_threshold)
    if prune_scope == 'global':
        k = int(NG * F * rewire_fraction)
        mask = np.zeros(NG * F, bool)
        if k > 0:
            flat = scores.reshape(-1)
            order = np.lexsort((np.arange(NG * F), flat))                  # by score, then flat index
            mask[order[:k]] = True
        return mask.reshape(NG, F)
    k = int(F * rewire_fraction)
    mask = np.zeros((NG, F), bool)
    if k == 0:
        return mask
    order = np.lexsort((np.broadcast_to(np.arange(F), (NG, F)), scores), axis=1)  # by score, then slot
    np.put_along_axis(mask, order[:, :k], True, axis=1)
    return mask


def regrow_index(seed, step, g, slot, attempt, D):
    """Candidate input index for (group, slot, attempt): Philox4x32-10, key (seed, step),
    counter (g, slot, attempt, 0x5245), word 0 mapped to [0,D) by multiply-shift."""
    w0 = px.philox4x32(g, slot, attempt, 0x5245, seed, step)[0]
    return int((int(w0) * int(D)) >> 32)


def regrow_init_value(seed, step, l, k, F):
    """U(-1/sqrt(F), 1/sqrt(F)) for a re-grown weight, from Philox (counter (l,k,0,0x494E))."""
    w0 = px.philox4x32(l, k, 0, 0x494E, seed, step)[0]
    u = np.float32(int(w0) >> 8) * np.float32(1.0 / 16777216.0)           # [0,1)
    bound = np.float32(1.0 / math.sqrt(F))
    return np.float32(np.float32(2.0) * u - np.float32(1.0)) * bound


def rewire(W, loc, G, D, prune_mode, rewire_fraction=None, rewire_threshold=None,
           init_mode='zero', regrow='unused', regroup=True, seed=0, step=0,
           injected=None, momentum=None, group0=0, score_mode='mean', prune_scope='group'):
    """Prune + regrow (+ regroup).  Returns (W_new bf16, loc_new int32, momentum_new).

    regrow:
      'replace'  new index drawn uniformly with replacement (rewire.py:211-217 semantics;
                 duplicates inside a row are possible, as in the reference);
      'unused'   rejection-sample until the index is not already used by the row.
    ``injected``: optional 1-D int array consumed in row-major order of the prune mask in place
    of the Philox draws — how the reference (which uses torch.randint) is compared.
    regroup: sort each index row ascending (stable in slot order) and permute the group's weight
    (and momentum) columns with it; the layer's output is unchanged by this.
    Pruned columns are zeroed ('zero') or re-drawn from U(+-1/sqrt(F)) ('random').
    """
    L, F = W.shape
    NG = loc.shape[0]
    scores = rewire_scores(W, G, NG, score_mode)
    mask = prune_mask(scores, prune_mode, rewire_fraction, rewire_threshold, prune_scope)
    Wb = _bf16_to_bits(W).copy().reshape(L, F)
    locn = loc.numpy().astype(np.int32).copy()
    mom = momentum.numpy().copy() if momentum is not None else None
    inj = 0
    for g in range(NG):
        pr = np.nonzero(mask[g])[0]
        if pr.size == 0 and not regroup:
            continue
        used = set(int(v) for k, v in enumerate(locn[g]) if not mask[g, k])
        for k in pr:
            if injected is not None:
                v = int(injected[inj]); inj += 1
            elif regrow == 'replace':
                v = regrow_index(seed, step, group0 + g, int(k), 0, D)
            else:
                found = False
                for t in range(64):
                    v = regrow_index(seed, step, group0 + g, int(k), t, D)
                    if v not in used:
                        found = True
                        break
                while not found:                    # bounded fallback: next free index upward
                    v = (v + 1) % D
                    found = v not in used
                used.add(v)
            locn[g, k] = v
        l0, l1 = g * G, min(L, (g + 1) * G)
        for k in pr:
            if init_mode == 'zero':
                Wb[l0:l1, k] = 0
            else:
                vals = np.array([regrow_init_value(seed, step, group0 * G + l, int(k), F) for l in range(l0, l1)],
                                np.float32)
                Wb[l0:l1, k] = px.rn_bf16_bits(vals)
            if mom is not None:
                mom[l0:l1, k] = 0.0
        if regroup:
            order = np.argsort(locn[g].astype(np.int64) * 256 + np.arange(F), kind='stable')
            locn[g] = locn[g][order]
            Wb[l0:l1] = Wb[l0:l1][:, order]
            if mom is not None:
                mom[l0:l1] = mom[l0:l1][:, order]
    return (_bits_to_bf16(Wb), torch.from_numpy(locn),
            torch.from_numpy(mom) if mom is not None else None)


# --------------------------------------------------------------------------- synthetic inputs
def make_inputs(B, D, L, F, G, avg_pos, zipf_s, seed=42, x_kind='l2norm', bias_zero=True):
    """Seeded synthetic inputs with the shapes and value distributions the benchmark configs name
    (the XMC datasets those shapes come from are not reproduced).

    x_kind: 'normal' N(0,1); 'l2norm' N(0,1) rows scaled to unit length; 'relu' max(0,N(0,1)).
    loc: per group F distinct indices uniform in [0,D), sorted ascending.
    targets: COO (row, col), per row n ~ Poisson(avg_pos) clipped to >= 1, label ids without
    replacement from a Zipf(zipf_s) law over label rank.
    """
    gen = torch.Generator().manual_seed(seed)
    X = torch.randn(B, D, generator=gen)
    if x_kind == 'l2norm':
        X = X / X.norm(dim=1, keepdim=True)
    elif x_kind == 'relu':
        X = X.clamp(min=0)
    X = X.to(torch.bfloat16)
    bound = 1.0 / math.sqrt(F)
    W = ((torch.rand(L, F, generator=gen) * 2 - 1) * bound).to(torch.bfloat16)
    NG = (L + G - 1) // G
    rs = np.random.RandomState(seed)
    keys = rs.rand(NG, D).astype(np.float32)
    loc = np.sort(np.argsort(keys, axis=1, kind='stable')[:, :F], axis=1).astype(np.int32)
    bias = torch.zeros(L, dtype=torch.bfloat16)
    if not bias_zero:
        bias = (torch.randn(L, generator=gen) * 0.1).to(torch.bfloat16)
    p = 1.0 / np.arange(1, L + 1, dtype=np.float64) ** zipf_s
    cdf = np.cumsum(p / p.sum())
    rows, cols = [], []
    npos = np.maximum(1, rs.poisson(avg_pos, size=B))
    for b in range(B):
        want = int(npos[b])
        got = set()
        while len(got) < want:
            draw = np.searchsorted(cdf, rs.rand(want * 2))
            for c in draw:
                if len(got) < want:
                    got.add(int(min(c, L - 1)))
        for c in sorted(got):
            rows.append(b); cols.append(c)
    targets = torch.tensor(np.stack([rows, cols], 1), dtype=torch.int32)
    return dict(X=X, W=W, loc=torch.from_numpy(loc), bias=bias, targets=targets)
