"""Checkpoint interop on a device: a file in the layout the reference's ``save_checkpoint`` writes
(src/runner.py:304-320: ``config``, ``state_dict``, ``label_map``, ``optimizer``, ``epoch``) is loaded into two CUDA
shards, the shards step, their states are merged back into the reference's state-dict entries, and the result equals
what a single shard over the whole layer produces (weights and bias bit for bit, dX up to the fp32 summation order).
Also: the layer module's rewiring stream position survives a state-dict round trip, and a state dict without it (as
the reference writes) still loads."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import ffi_oracle as fo


def test_reference_checkpoint_into_two_cuda_shards(tmp_path):
    from haste_b200 import checkpoint as ck
    from haste_b200.fused import FusedFFIShard
    B, D, F, G = 256, 256, 64, 128
    L = G * 21 + 77
    inp = fo.make_inputs(B, D, L, F, G, 6, 1.1, seed=31, bias_zero=False)
    sd = {"encoder.transformer.embeddings.word_embeddings.weight": torch.zeros(4, 8),
          "encoder.transformer.pooler.dense.bias": torch.zeros(8),                       # a bias that is not the layer's
          "tail_layer.weights": inp["W"], "tail_layer.bias": inp["bias"], "tail_layer.group_locations": inp["loc"]}
    path = tmp_path / "checkpoint.pt"
    torch.save({"config": {"model": {"ffi": {"fan_in": F, "group_size": G}}}, "state_dict": sd, "label_map": np.arange(L),
                "optimizer": {"state": {}, "param_groups": []}, "epoch": 7}, path)
    ckpt = torch.load(path, weights_only=False)
    assert set(ckpt) == {"config", "state_dict", "label_map", "optimizer", "epoch"}
    kw = dict(loss="bce", lr=0.05, weight_decay=1e-4, seed=123, rng="packed")
    X, coo = inp["X"].cuda(), inp["targets"].cuda()
    shards = [ck.shard_from_state_dict(ckpt["state_dict"], "tail_layer.", G, D, r, 2, "cuda", **kw) for r in range(2)]
    assert shards[0].label0 == 0 and shards[0].L + shards[1].L == L and shards[1].label0 == shards[0].L
    dx = None
    for _ in range(2):
        parts = [s.step(X, coo)[0].clone() for s in shards]
        dx = parts[0] + parts[1]
    whole = FusedFFIShard(inp["loc"].cuda(), inp["W"].clone().cuda(), inp["bias"].clone().cuda(), G, D, **kw)
    for _ in range(2):
        dx_whole = whole.step(X, coo)[0]
    torch.cuda.synchronize()
    merged = ck.merge_shard_states([ck.shard_state(s) for s in shards], prefix="tail_layer.")
    assert torch.equal(merged["tail_layer.weights"].view(torch.int16), whole.w.cpu().view(torch.int16))
    assert torch.equal(merged["tail_layer.bias"].view(torch.int16), whole.bias.cpu().view(torch.int16))
    assert torch.equal(merged["tail_layer.group_locations"], inp["loc"])
    assert torch.allclose(dx, dx_whole, rtol=1e-4, atol=1e-5 * float(dx_whole.abs().max()))
    # a saved shard resumes at the same position of the random stream
    st = ck.shard_state(shards[1])
    assert st["steps"] == 2 and st["seed"] == 123
    fresh = ck.shard_from_state_dict(ckpt["state_dict"], "tail_layer.", G, D, 1, 2, "cuda", **kw)
    ck.load_shard_state(fresh, st)
    a, b = shards[1].step(X, coo)[0].clone(), fresh.step(X, coo)[0].clone()
    torch.cuda.synchronize()
    assert torch.equal(fresh.w, shards[1].w) and torch.allclose(a, b, rtol=1e-4, atol=1e-5 * float(a.abs().max()))


def test_layer_state_dict_keeps_rewire_stream_position():
    from haste_b200.shared_ffi.rewire import GroupFixedFanIn
    kw = dict(group_size=32, prune_mode="fraction", rewire_fraction=0.25, init_mode="zero", regrow="unused", regroup=True)
    a = GroupFixedFanIn(128, 200, 32, device="cuda", dtype=torch.bfloat16, **kw)
    b = GroupFixedFanIn(192, 200, 32, device="cuda", dtype=torch.bfloat16, **kw)
    assert a.seed != b.seed                                   # default seeds differ between differently shaped layers
    a.rewire()
    sd = a.state_dict()
    assert sd["_extra_state"]["rewire_calls"] == 1
    c = GroupFixedFanIn(128, 200, 32, device="cuda", dtype=torch.bfloat16, **kw)
    c.load_state_dict(sd)
    assert c._rewire_calls == 1 and c.seed == a.seed
    a.rewire()
    c.rewire()
    assert torch.equal(a.group_locations, c.group_locations) and torch.equal(a.weights, c.weights)
    # a state dict as the reference writes it (no stream position) loads without complaint
    ref_sd = {k: v for k, v in sd.items() if k != "_extra_state"}
    d = GroupFixedFanIn(128, 200, 32, device="cuda", dtype=torch.bfloat16, **kw)
    d.load_state_dict(ref_sd)
    assert d._rewire_calls == 0
