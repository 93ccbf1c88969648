"""CPU-side tests: the C-ABI library loads and exports every declared symbol, the host-side sharding logic,
and a 2-rank gloo run of the label-sharded step (the oracle stands in for the kernels on CPU)."""
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built_lib():
    path = os.path.join(ROOT, "haste_b200", "libhaste_ffi.so")
    if not os.path.exists(path):
        from haste_b200 import build
        build.build()
    return path


def test_library_exports_every_declared_symbol(built_lib):
    import ctypes
    header = open(os.path.join(ROOT, "include", "haste_ffi.h")).read()
    declared = set(re.findall(r"\b(haste_[a-z0-9_]+)\s*\(", header))
    declared.discard("haste_stream_t")
    assert len(declared) >= 12
    lib = ctypes.CDLL(built_lib)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/haste_ffi.h but not exported"
    from haste_b200 import _lib
    assert set(_lib.SIGNATURES) | {"haste_last_error_string", "haste_version"} == declared
    assert _lib.lib.haste_version() >= 100


def test_argument_validation_without_gpu(built_lib):
    # status codes and messages of the C ABI for calls that are rejected before any CUDA work
    from haste_b200 import _lib
    rc = _lib.lib.haste_ffi_forward(None, None, None, None, None, 1, 1, 16, 1, 32, 8, None)
    assert rc == _lib.ERR_BAD_ARG and "NULL" in _lib.last_error()
    import ctypes
    buf = ctypes.create_string_buffer(64)
    addr = ctypes.addressof(buf)
    addr += (-addr) % 16
    rc = _lib.lib.haste_ffi_forward(addr, addr, addr, None, addr, 4, 8, 16, 10, 48, 16, None)
    assert rc == _lib.ERR_UNSUPPORTED and "group size" in _lib.last_error()
    rc = _lib.lib.haste_ffi_forward(addr, addr, addr, None, addr, 4, 8, 24, 10, 32, 16, None)
    assert rc == _lib.ERR_UNSUPPORTED and "fan_in" in _lib.last_error()
    rc = _lib.lib.haste_ffi_forward(addr, addr, addr, None, addr, 4, 8, 16, 10, 32, 8, None)
    assert rc == _lib.ERR_BAD_ARG and "ldz" in _lib.last_error()
    with pytest.raises(RuntimeError):
        _lib.check(rc, "forward")


def test_product_does_not_import_oracle():
    for dirpath, _, files in os.walk(os.path.join(ROOT, "haste_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", src, re.M), f"{f} imports the oracle"


def test_shard_partition():
    from haste_b200.fused import shard_groups, shard_labels
    for NG in (1, 7, 8, 5236, 21971):
        for R in (1, 2, 4, 8):
            ranges = [shard_groups(NG, R, r) for r in range(R)]
            assert ranges[0][0] == 0 and ranges[-1][1] == NG
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [b - a for a, b in ranges]
            assert max(sizes) - min(sizes) <= 1
    L, G = 670091, 128
    parts = [shard_labels(L, G, 8, r) for r in range(8)]
    assert parts[0][0] == 0 and parts[-1][1] == L and all(p[0] % G == 0 for p in parts)


def test_split_groups_by_cost():
    """Cost-weighted contiguous split: a partition, monotone, each range within one group's cost of its share."""
    import torch
    from haste_b200.fused import split_groups_by_cost, group_cost_from_targets
    assert split_groups_by_cost([1] * 10, 1) == [0, 10]
    assert split_groups_by_cost([0, 0, 0], 2)[0] == 0 and split_groups_by_cost([0, 0, 0], 2)[-1] == 3
    gen = torch.Generator().manual_seed(5)
    for n, R in ((1, 4), (7, 2), (100, 8), (5236, 8)):
        cost = torch.rand(n, generator=gen, dtype=torch.float64) + 0.1
        cost[0] = 25.0                                    # a heavy head group
        b = split_groups_by_cost(cost, R)
        assert len(b) == R + 1 and b[0] == 0 and b[-1] == n and all(x <= y for x, y in zip(b, b[1:]))
        share = float(cost.sum()) / R
        for r in range(R):
            tot = float(cost[b[r]:b[r + 1]].sum())
            assert tot <= share + float(cost.max()) + 1e-9
    # the estimate itself: a group full of positives costs more than an empty one, which costs exactly 1
    L, G, B = 1000, 128, 256
    rows = torch.arange(B).repeat_interleave(4)
    labs = torch.arange(4).repeat(B)                      # every row has labels 0..3: all in group 0
    cost = group_cost_from_targets(torch.stack([rows, labs], 1).to(torch.int32), L, G, B)
    assert cost.shape == (8,) and cost[0] > 1.0 and torch.all(cost[1:] == 1.0)
    assert torch.all(group_cost_from_targets(torch.zeros(0, 2, dtype=torch.int32), L, G, B) == 1.0)


def test_checkpoint_interop(tmp_path):
    """Reference-style state dict -> shards (count split and cost split) -> merged state dict is the identity;
    group-row inflation follows src/runner.py:324-334; the optimizer state keeps its rounding seed."""
    import torch
    from haste_b200 import checkpoint as ck
    from haste_b200.fused import FusedFFIShard
    gen = torch.Generator().manual_seed(2)
    D, L, F, G = 64, 128 * 5 + 17, 64, 128
    NG = (L + G - 1) // G
    sd = {"encoder.x": torch.zeros(3),
          "tail_layer.weights": torch.randn(L, F, generator=gen).to(torch.bfloat16),
          "tail_layer.bias": torch.randn(L, generator=gen).to(torch.bfloat16),
          "tail_layer.group_locations": torch.randint(0, D, (NG, F), generator=gen, dtype=torch.int32)}
    path = tmp_path / "ckpt.pt"
    torch.save({"state_dict": sd, "epoch": 3}, path)
    sd2 = torch.load(path)["state_dict"]
    inflated = ck.inflate_group_locations(sd2["tail_layer.group_locations"], L, G)
    assert inflated.shape == (L, F)
    for l in (0, G - 1, G, L - 1):
        assert torch.equal(inflated[l], sd["tail_layer.group_locations"][l // G])
    cost = torch.ones(NG, dtype=torch.float64)
    cost[0] = 3.0
    for gc in (None, cost):
        world = 3
        shards = [ck.shard_from_state_dict(sd2, "tail_layer.", G, D, r, world, "cpu", group_cost=gc, loss="bce", momentum=0.9, seed=77)
                  for r in range(world)]
        assert sum(s.L for s in shards) == L and shards[0].label0 == 0
        for i, s in enumerate(shards):
            s.steps = 5 + i
            s.mom_w.fill_(0.25)
        states = [ck.shard_state(s) for s in reversed(shards)]                 # any order
        merged = ck.merge_shard_states(states, prefix="tail_layer.")
        for k in ("weights", "bias", "group_locations"):
            assert torch.equal(merged["tail_layer." + k], sd["tail_layer." + k]), k
        # a fresh shard of the same range resumes with the same random-stream position and momentum
        fresh = ck.shard_from_state_dict(sd2, "tail_layer.", G, D, 1, world, "cpu", group_cost=gc, loss="bce", momentum=0.9, seed=1)
        fresh.w.zero_()
        ck.load_shard_state(fresh, [st for st in states if st["label0"] == fresh.label0][0])
        assert fresh.steps == 6 and fresh.seed == 77 and torch.equal(fresh.w, shards[1].w) and float(fresh.mom_w[0, 0]) == 0.25
        assert fresh._keys() == shards[1]._keys()
    with pytest.raises(ValueError):
        ck.merge_shard_states(states[:-1])                                     # the first shard is missing
    # SRSgd keeps seed and step counter in its param group, so optimizer.state_dict() round-trips them
    from haste_b200.shared_ffi.optim_sr import SRSgd
    p = torch.nn.Parameter(torch.zeros(4, 16, dtype=torch.bfloat16))
    opt = SRSgd([p], lr=0.1, seed=123, rng="packed")
    opt.param_groups[0]["seed"] += 7
    opt.param_groups[0]["step_count"] = 7
    opt2 = SRSgd([p], lr=0.1, seed=0)
    opt2.load_state_dict(opt.state_dict())
    assert opt2.param_groups[0]["seed"] == 130 and opt2.param_groups[0]["step_count"] == 7 and opt2.param_groups[0]["rng"] == "packed"


_WORKER = r"""
import os, sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from oracle import ffi_oracle as fo
from haste_b200.fused import shard_labels, allreduce_sum
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:" + sys.argv[2], rank=int(sys.argv[3]), world_size=2)
rank = dist.get_rank()
B, D, L, F, G = 32, 64, 700, 16, 32
inp = fo.make_inputs(B, D, L, F, G, 5, 1.1, seed=3, bias_zero=False)
l0, l1, g0, g1 = shard_labels(L, G, 2, rank)
tg = inp["targets"]
keep = (tg[:, 1] >= l0) & (tg[:, 1] < l1)
tl = tg[keep].clone(); tl[:, 1] -= l0
out = fo.train_step(inp["loc"][g0:g1], inp["X"], inp["W"][l0:l1], inp["bias"][l0:l1], tl, G, fo.LOSS_BCE, 0.05, 1e-4, 123,
                    step=2, rng_mode="packed", row0=l0)
dxt = out["dXt"].clone()
allreduce_sum(dxt)                        # the path's only exchange step
full = fo.train_step(inp["loc"], inp["X"], inp["W"], inp["bias"], tg, G, fo.LOSS_BCE, 0.05, 1e-4, 123, step=2, rng_mode="packed")
assert torch.allclose(dxt, full["dXt"], atol=1e-5), "summed dX differs from the unsharded step"
assert torch.equal(out["W_new"], full["W_new"][l0:l1]), "sharded weights differ"
assert torch.equal(out["bias_new"], full["bias_new"][l0:l1])
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
"""


def test_two_rank_gloo_sharded_step(tmp_path, built_lib):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    port = str(29500 + os.getpid() % 2000)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, port, str(r)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
             for r in range(2)]
    for p in procs:
        out, _ = p.communicate(timeout=300)
        assert p.returncode == 0, out.decode()


def test_srsgd_loads_reference_optimizer_state(built_lib):
    """A state dict with the key set the reference's SRSgd writes (shared_ffi/optim_sr.py:25-44: six group keys and a
    momentum_buf per parameter) loads, and the optimizer steps afterwards (the keys this class adds come back with
    their reference-compatible defaults)."""
    from haste_b200.shared_ffi.optim_sr import SRSgd
    p = torch.nn.Parameter(torch.ones(4, 3))
    opt = SRSgd([p], lr=0.1, weight_decay=0.0, momentum=0.9, seed=123)
    ref_state = {
        "state": {0: {"momentum_buf": torch.full((4, 3), 2.0)}},
        "param_groups": [{"lr": 0.5, "weight_decay": 0.0, "momentum": 0.9, "use_momentum": True,
                          "stochastic_rounding": True, "seed": 130, "params": [0]}],
    }
    opt.load_state_dict(ref_state)
    g = opt.param_groups[0]
    assert g["seed"] == 130 and g["rng"] == "reference" and g["contract"] is True and g["step_count"] == 0
    p.grad = torch.ones(4, 3)
    opt.step()                                    # fp32 parameter: the Python path, runs without a GPU
    # momentum 0.9 * 2 + 1 = 2.8; p = 1 - 0.5 * 2.8
    assert torch.allclose(p.data, torch.full((4, 3), 1.0 - 0.5 * 2.8))
    assert opt.param_groups[0]["seed"] == 131 and opt.param_groups[0]["step_count"] == 1


_LW_WORKER = r"""
import os, sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from oracle import ffi_oracle as fo
from haste_b200.fused import layerwide_prune_count, tie_base_for_rank
rank, world = int(sys.argv[2]), 2
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:" + sys.argv[3], rank=rank, world_size=world)
D, L, F, G, frac = 96, 64 * 9 + 5, 32, 64, 0.2
inp = fo.make_inputs(2, D, L, F, G, 1, 1.1, seed=3)
NG = (L + G - 1) // G
g0, g1 = (0, 4) if rank == 0 else (4, NG)
scores = fo.rewire_scores(inp["W"], G, NG, "max")                 # whole layer (for the check) ...
mine = scores[g0:g1].reshape(-1)                                   # ... and this rank's shard
bits = mine.view(np.uint32)
k = layerwide_prune_count(NG, F, frac)
# the three phases of the device selection, restated with numpy, with the same exchanges between them
hist_hi = torch.from_numpy(np.bincount(bits >> 16, minlength=65536).astype(np.int64)); dist.all_reduce(hist_hi)
c = np.cumsum(hist_hi.numpy()); hi = int(np.searchsorted(c, k)); k_in = k - (int(c[hi - 1]) if hi else 0)
inbin = bits[(bits >> 16) == hi]
hist_lo = torch.from_numpy(np.bincount(inbin & 0xFFFF, minlength=65536).astype(np.int64)); dist.all_reduce(hist_lo)
c = np.cumsum(hist_lo.numpy()); lo = int(np.searchsorted(c, k_in)); take = k_in - (int(c[lo - 1]) if lo else 0)
T = (hi << 16) | lo
ties = torch.tensor([int((bits == T).sum())]); allt = [torch.zeros_like(ties) for _ in range(world)]; dist.all_gather(allt, ties)
base = tie_base_for_rank([int(t) for t in allt], rank)
rank_among_ties = base + np.cumsum(bits == T) - 1
mask = (bits < T) | ((bits == T) & (rank_among_ties < take))
want = fo.prune_mask(scores, "fraction", frac, None, "global")[g0:g1].reshape(-1)
assert np.array_equal(mask, want), "prune set differs from the single-device rule"
tot = torch.tensor([int(mask.sum())]); dist.all_reduce(tot)
assert int(tot) == k
dist.destroy_process_group()
print("ok")
"""


def test_two_rank_gloo_layerwide_selection(tmp_path):
    """Host logic of the cross-rank layer-wide rewire selection (count, exchanges, tie order) on two gloo ranks: the
    union of the ranks' prune sets is the single-device rule's prune set."""
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "lw_worker.py"
    script.write_text(_LW_WORKER)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, str(r), str(port)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0 and "ok" in o, o


def test_pipeline_reserve_choice(built_lib):
    """SMs the pipelined multi-GPU step leaves to the collective: 8 for two ranks, 12 for up to four, 16 beyond, and 8
    whenever the fused kernel is long against the all-reduce (the rule's figures are measured, see the docstring)."""
    from haste_b200.fused import ShardedFFILayer

    class _Shard:                      # the rule only looks at the shard's label count and fan-in
        def __init__(self, L, F):
            self.L, self.F = L, F

    def choice(world, B, L_total, F):
        layer = ShardedFFILayer.__new__(ShardedFFILayer)
        layer.world, layer.shard = world, _Shard(L_total // world, F)
        return layer._choose_reserve(B)

    assert [choice(n, 512, 670091, 64) for n in (2, 4, 8)] == [8, 12, 16]           # 670K labels, B=512
    assert [choice(n, 1024, 2812281, 64) for n in (2, 4, 8)] == [8, 8, 8]           # 2.8M labels, B=1024: long kernels
    assert choice(16, 512, 670091, 64) == 16
