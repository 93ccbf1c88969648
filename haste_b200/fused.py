"""Fused training step of the FFI layer, single shard and label-sharded across ranks.

``FusedFFIShard`` owns one contiguous range of label groups (weights, bias, index table, optional
momentum) and runs forward + loss gradient + both backwards + the SGD/stochastic-rounding update as one
kernel launch; neither logits nor their gradient are written to memory.

``ShardedFFILayer`` splits the groups of a layer contiguously over the ranks of a ``torch.distributed``
process group (features replicated, one process per GPU) and sums the per-rank feature gradients with a
single all-reduce — the only exchange step of the path.  Random-bit counters use global label indices, so
the updated weights do not depend on the number of ranks.
"""
import torch

from . import _lib
from . import ffi as _ffi

LOSSES = {"bce": _lib.LOSS_BCE, "squared_hinge": _lib.LOSS_SQHINGE}


def shard_groups(num_groups, world_size, rank):
    """Contiguous, near-equal split of ``num_groups`` label groups: returns [g0, g1) of ``rank``."""
    base, rem = divmod(num_groups, world_size)
    g0 = rank * base + min(rank, rem)
    return g0, g0 + base + (1 if rank < rem else 0)


def split_groups_by_cost(cost, world_size):
    """Contiguous split of label groups into ``world_size`` ranges of near-equal total ``cost``.

    ``cost``: one non-negative number per group (sequence or 1-D tensor).  Returns ``world_size + 1`` boundaries
    ``b`` with ``b[0] = 0``, ``b[-1] = len(cost)``, non-decreasing; rank ``r`` owns groups ``[b[r], b[r+1])``.
    Boundary ``r`` is placed where the running sum first reaches ``r / world_size`` of the total, so every range
    is within one group's cost of its fair share.  With uniform cost this is the split of ``shard_groups``
    up to where the remainder goes.
    """
    c = torch.as_tensor(cost, dtype=torch.float64).flatten().clamp_min(0)
    n = c.numel()
    if world_size <= 1 or n == 0:
        return [0] + [n] * max(world_size, 1)
    total = float(c.sum())
    if total <= 0:
        return [shard_groups(n, world_size, r)[0] for r in range(world_size)] + [n]
    csum = torch.cumsum(c, 0)
    bounds = [0]
    for r in range(1, world_size):
        k = int(torch.searchsorted(csum, torch.tensor(total * r / world_size, dtype=torch.float64)).item())
        # the group that crosses the mark goes to whichever side leaves the smaller excess
        if k < n and float(csum[k]) - total * r / world_size <= total * r / world_size - (float(csum[k - 1]) if k > 0 else 0.0):
            k += 1
        bounds.append(min(max(k, bounds[-1]), n))
    bounds.append(n)
    return bounds


def group_cost_from_targets(targets, L, G, B, general_chunk_cost=4.0, bitmap_cost=1.5):
    """Relative cost of each label group in the fused step, estimated from one batch's COO targets [nnz,2].

    A group costs its batch tiles; a 32-row x 16-label chunk that holds a positive takes the general branch of the
    loss epilogue (about ``general_chunk_cost`` more than a chunk without), and a group with more than 8 entries
    builds a shared-memory bitmap per tile (``bitmap_cost`` of a group).  Label frequencies are long-tailed, so a
    split by group count leaves the rank that owns the head labels well behind the others.  The two weights are fitted
    to per-rank kernel times on eight B200s: with 1.5 / 0.5 the rank holding the head groups ran 9 % (2.8M labels, BCE)
    and 5 % (670K labels, squared hinge) longer than the others, which corresponds to 2.3-2.9 times the modelled extra.
    """
    NG = (L + G - 1) // G
    t = torch.as_tensor(targets).to(torch.int64).cpu()
    cost = torch.ones(NG, dtype=torch.float64)
    if t.numel() == 0:
        return cost
    row, lab = t[:, 0], t[:, 1]
    keep = (lab >= 0) & (lab < L)
    row, lab = row[keep], lab[keep]
    grp = lab // G
    chunks_per_group = max(1, ((B + 31) // 32) * (G // 16))
    chunk_id = grp * chunks_per_group + (row // 32) * (G // 16) + (lab % G) // 16
    hit = torch.bincount(torch.unique(chunk_id) // chunks_per_group, minlength=NG).to(torch.float64)
    n_ent = torch.bincount(grp, minlength=NG)
    cost += general_chunk_cost * hit / chunks_per_group + bitmap_cost * (n_ent > 8).to(torch.float64)
    return cost


def shard_labels(L, G, world_size, rank):
    """Label range [l0, l1) and group range [g0, g1) owned by ``rank`` (whole groups only; the ragged last
    group goes to the last non-empty shard)."""
    NG = (L + G - 1) // G
    g0, g1 = shard_groups(NG, world_size, rank)
    return min(L, g0 * G), min(L, g1 * G), g0, g1


class FusedFFIShard:
    def __init__(self, group_locations, weights, bias, group_size, in_features, *, label0=0, loss="bce", lr=0.05,
                 weight_decay=0.0, momentum=0.0, seed=123, rng="packed", contract=True, grad_scale=1.0,
                 stochastic_rounding=True, max_nnz=1 << 16):
        if loss not in LOSSES:
            raise ValueError(f"loss must be one of {sorted(LOSSES)}")
        dev = weights.device
        self.loc, self.w, self.bias = group_locations, weights, bias
        self.G, self.D, self.label0 = int(group_size), int(in_features), int(label0)
        self.L, self.F = weights.shape
        self.NG = (self.L + self.G - 1) // self.G
        self.loss_kind, self.grad_scale = LOSSES[loss], float(grad_scale)
        self.lr, self.wd, self.mu, self.seed = float(lr), float(weight_decay), float(momentum), int(seed)
        self.rng, self.contract, self.sr = rng, bool(contract), bool(stochastic_rounding)
        self.steps = 0
        self.mom_w = torch.zeros_like(weights, dtype=torch.float32) if self.mu != 0.0 else None
        self.mom_b = torch.zeros_like(bias, dtype=torch.float32) if (self.mu != 0.0 and bias is not None) else None
        self.tgt_ptr = torch.zeros(self.NG + 1, dtype=torch.int32, device=dev)
        self.tgt_ent = torch.zeros(max_nnz, dtype=torch.int32, device=dev)
        self.scratch = torch.zeros(self.NG, dtype=torch.int32, device=dev)
        self.loss_buf = torch.zeros(1, dtype=torch.float32, device=dev)
        self._dxt = None
        self._xt = None

    def _keys(self):
        # reference stream: the optimizer's seed advances by one per step (optim_sr.py:59-62);
        # packed stream: key (seed, step)
        if self.rng == "reference":
            return self.seed + self.steps, 0
        return self.seed, self.steps

    def bucket_targets(self, targets):
        """``targets``: int32 [nnz,2] (row, GLOBAL label id) on the device.  Entries outside this shard are dropped."""
        if targets.shape[0] > self.tgt_ent.numel():
            self.tgt_ent = torch.zeros(int(targets.shape[0] * 1.5) + 1, dtype=torch.int32, device=targets.device)
        _ffi.targets_bucket(targets, self.label0, self.L, self.G, self.tgt_ptr, self.tgt_ent, self.scratch)

    def step_xt(self, xt, targets, dxt=None, want_loss=True):
        """One step given the transposed features [D,B] (bf16).  Returns (dxt fp32 [D,B], loss fp32 [1] or None)."""
        D, B = xt.shape
        if dxt is None:
            if self._dxt is None or self._dxt.shape != (D, B):
                self._dxt = torch.empty(D, B, dtype=torch.float32, device=xt.device)
            dxt = self._dxt
        self.bucket_targets(targets)
        if want_loss:
            self.loss_buf.zero_()
        seed, step = self._keys()
        flags = _ffi.make_flags(sr=self.sr, contract=self.contract, rng=self.rng, zero_dxt=True, loss=want_loss)
        _ffi.train_step(self.loc, xt, self.w, self.bias, self.mom_w, self.mom_b, self.tgt_ptr, self.tgt_ent, dxt,
                        self.loss_buf if want_loss else None, self.G, self.label0, self.loss_kind, self.grad_scale, self.lr,
                        self.wd, self.mu, seed, step, flags)
        self.steps += 1
        return dxt, (self.loss_buf if want_loss else None)

    def step(self, x, targets, want_loss=True):
        """One step given features [B,D] (bf16, device): one preparation launch (transpose, clears, target
        bucketing) and one fused-step launch."""
        B, D = x.shape
        if self.NG * 4 > 200 * 1024:                       # too many groups for the single-block bucketing
            return self.step_xt(_ffi.transpose_bf16(x), targets, want_loss=want_loss)
        if self._dxt is None or self._dxt.shape != (D, B):
            self._dxt = torch.empty(D, B, dtype=torch.float32, device=x.device)
            self._xt = torch.empty(D, B, dtype=torch.bfloat16, device=x.device)
        if targets.shape[0] > self.tgt_ent.numel():
            self.tgt_ent = torch.zeros(int(targets.shape[0] * 1.5) + 1, dtype=torch.int32, device=targets.device)
        if not (x.is_cuda and targets.is_cuda) or x.dtype != torch.bfloat16 or targets.dtype != torch.int32 or not x.is_contiguous() \
                or not targets.is_contiguous():
            raise RuntimeError("FusedFFIShard.step: features must be a contiguous CUDA bf16 [B,D] tensor, targets a contiguous CUDA int32 [nnz,2] tensor")
        seed, step = self._keys()
        flags = _ffi.make_flags(sr=self.sr, contract=self.contract, rng=self.rng, zero_dxt=False, loss=want_loss)
        # the loss word is cleared by the preparation launch either way; it is only accumulated when asked for
        _ffi.step(x, targets, self.loc, self._xt, self.w, self.bias, self.mom_w, self.mom_b, self.tgt_ptr, self.tgt_ent, self._dxt,
                  self.loss_buf, self.G, self.label0, self.loss_kind, self.grad_scale, self.lr, self.wd, self.mu, seed, step, flags)
        self.steps += 1
        return self._dxt, (self.loss_buf if want_loss else None)


class ShardedFFILayer:
    """Label-sharded layer: this rank's ``FusedFFIShard`` plus the dX all-reduce.

    ``full_*`` tensors describe the whole layer (on any device); each rank copies its slice to ``device``.
    ``group_cost`` (optional, one number per label group, identical on every rank) replaces the split by group
    count with a contiguous split of equal estimated cost; ``group_cost_from_targets`` derives it from a batch.

    Two ways to step:
      ``step(x, targets)``            kernel, then the all-reduce; returns the summed dX of this step.
      ``step_pipelined(x, targets, next_batch)``
                                      three streams: the fused kernel of this step (on ``reserve_sms`` fewer CTAs than
                                      the GPU has SMs) runs beside the all-reduce of the PREVIOUS step's dX and the
                                      preparation (transpose, clears, target bucketing) of the NEXT batch.  Returns the
                                      previous step's summed dX (None on the first call; valid until the next call,
                                      which reuses its buffer); ``flush()`` returns the last one.  Everything enqueued
                                      by a call has finished when the caller's stream passes the end of the call, so
                                      per-call device timing sees all of it.
    """

    def __init__(self, full_locations, full_weights, full_bias, group_size, in_features, device, *, process_group=None,
                 rank=None, world_size=None, group_cost=None, reserve_sms=None, **shard_kwargs):
        import torch.distributed as dist
        self.dist = dist
        self.pg = process_group
        if rank is None:
            rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        if world_size is None:
            world_size = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.rank, self.world = rank, world_size
        L = full_weights.shape[0]
        if group_cost is None:
            l0, l1, g0, g1 = shard_labels(L, group_size, world_size, rank)
        else:
            # contiguous ranges of near-equal estimated cost (every rank must pass the same costs)
            bounds = split_groups_by_cost(group_cost, world_size)
            g0, g1 = bounds[rank], bounds[rank + 1]
            l0, l1 = min(L, g0 * group_size), min(L, g1 * group_size)
        self.l0, self.l1, self.g0, self.g1 = l0, l1, g0, g1
        self.shard = FusedFFIShard(full_locations[g0:g1].to(device).contiguous(), full_weights[l0:l1].to(device).contiguous(),
                                   None if full_bias is None else full_bias[l0:l1].to(device).contiguous(), group_size,
                                   in_features, label0=l0, **shard_kwargs)
        on_gpu = torch.device(device).type == "cuda"
        self.comm_stream = torch.cuda.Stream(device=device) if (world_size > 1 and on_gpu) else None
        self.prep_stream = torch.cuda.Stream(device=device) if on_gpu else None
        # SMs the pipelined step leaves to the side streams; None = chosen at the first pipelined step (_choose_reserve)
        self.reserve_sms = None if reserve_sms is None else int(reserve_sms)
        self.comm_pg = process_group          # replaced by a communicator of the layer's own at the first pipelined step
        self._comm_ready = False
        self._on_gpu = on_gpu
        self._slots = None          # pipelined path: three sets of per-batch buffers (being reduced / computed / prepared)
        self._cur = 0               # slot of the batch the next step_pipelined call computes on
        self._staged = False        # slot _cur already holds a prepared batch
        self._pending = None        # slot whose dX still has to be all-reduced

    def step(self, x, targets, want_loss=True):
        """Returns (dxt summed over all ranks, this rank's loss part): kernel, then the all-reduce, on the caller's
        stream."""
        dxt, loss = self.shard.step(x, targets, want_loss=want_loss)
        allreduce_sum(dxt, self.pg, None, self.world)
        return dxt, loss

    # ------------------------------------------------------------------ pipelined path
    def _choose_reserve(self, B):
        """SMs left free for the collective and the preparation kernel.  The all-reduce of the 4*D*B bytes of dX gets
        slower with fewer CTAs and with more ranks (four B200s, 1.5 MB: 45 us with NCCL's default, 55 us with 16 CTAs, 82
        us with 8), the fused kernel gets slower with fewer SMs, and a kernel much longer than the collective loses more
        from missing SMs than it can win from the overlap.  Measured at 670K labels (per-step time, 8 / 12 / 16 SMs
        reserved): four ranks 88 / 85 / 87 us, eight ranks 90 / 70 / 60 us; at 2.8M labels four ranks 630 / - / 654 us, eight
        ranks 347 / - / 353 us."""
        sh = self.shard
        est_kernel_ms = 6.0 * B * sh.L * sh.F / 500e12 * 1e3        # the fused kernel sustains about 500 TFLOP/s
        if est_kernel_ms > 0.2 or self.world <= 2:
            return 8
        return 12 if self.world <= 4 else 16

    def _make_comm(self):
        """The pipelined step's all-reduce runs beside the persistent fused kernel, which holds every SM but
        ``reserve_sms``.  A collective that asks for more CTAs than that gets some of them only after the fused kernel's
        CTAs retire, or takes SMs from them (a fused-kernel CTA needs a whole SM's shared memory): either way the step
        becomes kernel + collective instead of their maximum.  So the dX all-reduce gets its own communicator, capped at
        ``reserve_sms`` CTAs that are launched singly, not as clusters of four (a cluster needs four free SMs of one GPC
        at the same moment).  Measured on four B200s at 670K labels: kernel alone on 132 CTAs 100 us, all-reduce of the
        1.5 MB dX alone 45 us; together 122 us with the default communicator, 105 us with this one.  Collective call:
        every rank reaches its first pipelined step at the same point of its program."""
        dist = self.dist
        self._comm_ready = True
        if not (self.world > 1 and self._on_gpu and dist.is_initialized() and dist.get_backend(self.pg) == "nccl"):
            return
        try:
            opts = dist.ProcessGroupNCCL.Options()
            opts.config.max_ctas = max(1, self.reserve_sms)
            opts.config.min_ctas = 1
            opts.config.cga_cluster_size = 1
            self.comm_pg = dist.new_group(ranks=dist.get_process_group_ranks(self.pg if self.pg is not None else dist.group.WORLD),
                                          backend="nccl", pg_options=opts)
        except (AttributeError, TypeError, RuntimeError):     # a torch without these options: the caller's group as it is
            self.comm_pg = self.pg

    def setup_pipeline(self, B):
        """Chooses ``reserve_sms`` (unless given) and creates the all-reduce communicator for batches of ``B`` rows; called
        by the first ``step_pipelined`` when the caller has not done it (a collective call: same point on every rank)."""
        if self.reserve_sms is None:
            self.reserve_sms = self._choose_reserve(B)
        if not self._comm_ready:
            self._make_comm()

    def _make_slots(self, B, D, nnz, dev):
        sh = self.shard
        self._slots = [dict(xt=torch.empty(D, B, dtype=torch.bfloat16, device=dev), dxt=torch.empty(D, B, dtype=torch.float32, device=dev),
                            ptr=torch.zeros(sh.NG + 1, dtype=torch.int32, device=dev), ent=torch.zeros(max(1, int(nnz * 1.5)), dtype=torch.int32, device=dev),
                            loss=torch.zeros(1, dtype=torch.float32, device=dev), prepared=torch.cuda.Event(), begun=torch.cuda.Event(),
                            reduced=torch.cuda.Event()) for _ in range(3)]

    def _prepare(self, slot, x, targets, stream):
        sh, b = self.shard, self._slots[slot]
        if targets.shape[0] > b["ent"].numel():
            b["ent"] = torch.zeros(int(targets.shape[0] * 1.5) + 1, dtype=torch.int32, device=targets.device)
        if x.dtype is not torch.bfloat16 or targets.dtype is not torch.int32 or not x.is_contiguous() or not targets.is_contiguous() \
                or not x.is_cuda or not targets.is_cuda:
            raise RuntimeError("step_pipelined: features must be a contiguous CUDA bf16 [B,D] tensor, targets a contiguous CUDA int32 [nnz,2] tensor")
        _ffi.step_prepare_on(stream.cuda_stream, x, b["xt"], b["dxt"], b["loss"], targets, sh.label0, sh.L, sh.G, b["ptr"], b["ent"])
        b["prepared"].record(stream)

    def step_pipelined(self, x, targets, next_batch=None, want_loss=True):
        """One step of the three-stream pipeline (see the class docstring).  ``next_batch``: (x, targets) of the
        following step, already on the device, or None.  Returns (previous step's summed dxt or None, this step's loss
        part as a device scalar)."""
        sh = self.shard
        dev = x.device
        if dev.index is not None and torch.cuda.current_device() != dev.index:
            with torch.cuda.device(dev):              # the library calls below take the current device
                return self.step_pipelined(x, targets, next_batch, want_loss)
        cur = torch.cuda.current_stream(dev)
        B, D = x.shape
        if self._slots is None or self._slots[0]["xt"].shape != (D, B):
            self._make_slots(B, D, max(targets.shape[0], 1 if next_batch is None else next_batch[1].shape[0]), dev)
            if self.world > 1:      # leave SMs free for the collective and the preparation kernels of the other streams
                self.setup_pipeline(B)
                _lib.check(_lib.lib.haste_ffi_set_max_ctas(max(1, _sm_count(dev) - self.reserve_sms)), "set_max_ctas")
        s = self._cur
        nxt = (s + 1) % 3           # the previous step's slot is (s + 2) % 3: three distinct buffers are live per call
        b = self._slots[s]
        if not self._staged:
            self._prepare(s, x, targets, cur)                 # first step: nothing was staged before
        prev = self._pending
        begun = b["begun"]
        begun.record(cur)                                     # the side streams start here: not before this call began
        # (1) this step's kernel goes to the GPU first, so that its CTAs are placed before those of the side streams
        cur.wait_event(b["prepared"])
        seed, step = sh._keys()
        flags = _ffi.make_flags(sr=sh.sr, contract=sh.contract, rng=sh.rng, zero_dxt=False, loss=want_loss)
        _ffi.train_step_on(cur.cuda_stream, sh.loc, b["xt"], sh.w, sh.bias, sh.mom_w, sh.mom_b, b["ptr"], b["ent"], b["dxt"],
                           b["loss"] if want_loss else None, sh.G, sh.label0, sh.loss_kind, sh.grad_scale, sh.lr, sh.wd, sh.mu, seed, step, flags)
        sh.steps += 1
        # (2) the previous step's all-reduce, beside this step's kernel (after the kernel that made its input)
        if prev is not None and self.world > 1:
            pb = self._slots[prev]
            self.comm_stream.wait_event(begun)
            with torch.cuda.stream(self.comm_stream):
                self.dist.all_reduce(pb["dxt"], op=self.dist.ReduceOp.SUM, group=self.comm_pg)
                pb["reduced"].record(self.comm_stream)
        # (3) the next batch's preparation, beside this step's kernel
        if next_batch is not None:
            self.prep_stream.wait_event(begun)
            self._prepare(nxt, next_batch[0], next_batch[1], self.prep_stream)
        # everything this call enqueued is done when the caller's stream gets past this point
        if prev is not None and self.world > 1:
            cur.wait_event(self._slots[prev]["reduced"])
        if next_batch is not None:
            cur.wait_event(self._slots[nxt]["prepared"])
        out = self._slots[prev]["dxt"] if prev is not None else None
        self._pending, self._cur, self._staged = s, nxt, next_batch is not None
        return out, (b["loss"] if want_loss else None)

    def close(self):
        """Releases the layer's own communicator (NCCL slows down when many communicators are alive in one process:
        measured with six).  Every rank calls it at the same point."""
        if self._comm_ready and self.comm_pg is not None and self.comm_pg is not self.pg:
            self.dist.destroy_process_group(self.comm_pg)
        self.comm_pg, self._comm_ready = self.pg, False

    def flush(self):
        """All-reduce the last step's dX (on the caller's stream) and return it."""
        if self._pending is None:
            return None
        dxt = self._slots[self._pending]["dxt"]
        allreduce_sum(dxt, self.pg, None, self.world)
        self._pending = None
        return dxt


def layerwide_prune_count(total_groups, fan_in, fraction):
    """Number of (group, slot) pairs the layer-wide fraction rule prunes: int(NG * F * fraction) over the WHOLE layer
    (src/group_fanin_real.py:232-250), whatever the sharding."""
    return int(int(total_groups) * int(fan_in) * float(fraction))


def tie_base_for_rank(ties_per_rank, rank):
    """Scores equal to the selection threshold are pruned in flat (group, slot) order of the whole layer; ranks hold
    contiguous label ranges in rank order, so a rank's ties come after those of all lower ranks."""
    return int(sum(int(t) for t in ties_per_rank[:rank]))


def rewire_layerwide_sharded(shard, fraction, total_groups, rank, world_size, process_group=None, *, score_mode="mean", regrow="replace",
                             init_mode="zero", regroup=False, seed=0, step=0):
    """Layer-wide fraction rewire of a label-sharded layer: every rank calls this with its ``FusedFFIShard``; the
    prune set is the one a single device holding the whole layer would choose.  Two all-reduces of a 65,536-bin
    histogram and one all-gather of a counter are the only exchanges.  Returns the number of pairs pruned on this rank."""
    import torch.distributed as dist
    k = layerwide_prune_count(total_groups, shard.F, fraction)
    if k == 0:
        return 0
    sel = _ffi.LayerwideSelect(shard.w, shard.G, {"mean": 0, "max": 1}[score_mode])
    multi = world_size > 1
    sel.begin()
    if multi:
        dist.all_reduce(sel.hist_hi, op=dist.ReduceOp.SUM, group=process_group)
    sel.refine(k)
    if multi:
        dist.all_reduce(sel.hist_lo, op=dist.ReduceOp.SUM, group=process_group)
    sel.finish()
    ties = [sel.ties.clone() for _ in range(world_size)]
    if multi:
        dist.all_gather(ties, sel.ties.clone(), group=process_group)
    else:
        ties = [sel.ties]
    base = tie_base_for_rank([int(t.item()) for t in ties], rank)
    changed = torch.zeros(1, dtype=torch.int32, device=shard.w.device)
    sel.apply(shard.loc, shard.mom_w, shard.D, shard.label0 // shard.G, base, {"replace": 0, "unused": 1}[regrow],
              {"zero": 0, "random": 1}[init_mode], regroup, seed, step, changed)
    return int(changed.item())


def _sm_count(device):
    return torch.cuda.get_device_properties(device).multi_processor_count


def allreduce_sum(t, process_group=None, comm_stream=None, world_size=None):
    """Sum ``t`` over the ranks in place (NCCL for CUDA tensors, any backend for CPU tensors).  With ``comm_stream`` the
    collective runs there, after the work already on the current stream, and the current stream waits for it."""
    import torch.distributed as dist
    if world_size is None:
        world_size = dist.get_world_size(process_group) if dist.is_initialized() else 1
    if world_size <= 1:
        return t
    if comm_stream is not None:
        comm_stream.wait_stream(torch.cuda.current_stream(t.device))
        with torch.cuda.stream(comm_stream):
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=process_group)
        torch.cuda.current_stream(t.device).wait_stream(comm_stream)
    else:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=process_group)
    return t
