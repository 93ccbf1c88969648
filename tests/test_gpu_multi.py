"""Two ranks on two GPUs (skipped when fewer are visible): the label-sharded, pipelined step against the same layer
on one GPU.  Updated weights and bias must be bit-identical (random bits are drawn by global label, the products are
deterministic), the summed feature gradient equal up to the fp32 summation order (rel 1e-4)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from oracle import ffi_oracle as fo
    from haste_b200.fused import FusedFFIShard, ShardedFFILayer, group_cost_from_targets
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    B, D, F, G = 256, 256, 64, 128
    L = G * 37 + 50
    inp = fo.make_inputs(B, D, L, F, G, 6, 1.1, seed=11, bias_zero=False)
    batches = [(inp["X"].to(dev), inp["targets"].to(dev))]
    inp2 = fo.make_inputs(B, D, L, F, G, 6, 1.1, seed=12, bias_zero=False)
    batches.append((inp2["X"].to(dev), inp2["targets"].to(dev)))
    kw = dict(loss="bce", lr=0.05, weight_decay=1e-4, seed=123, rng="packed", grad_scale=1.0)
    cost = group_cost_from_targets(inp["targets"], L, G, B)
    layer = ShardedFFILayer(inp["loc"], inp["W"], inp["bias"], G, D, dev, rank=rank, world_size=world, group_cost=cost, reserve_sms=8, **kw)
    outs = []
    n_steps = 4
    for i in range(n_steps):
        nxt = batches[(i + 1) % 2] if i + 1 < n_steps else None
        prev, _ = layer.step_pipelined(*batches[i % 2], next_batch=nxt)
        if prev is not None:
            outs.append(prev.clone())
    outs.append(layer.flush().clone())
    torch.cuda.synchronize(dev)
    assert len(outs) == n_steps
    # gather the shards on rank 0
    ws = [None] * world
    dist.all_gather_object(ws, (layer.l0, layer.shard.w.cpu(), layer.shard.bias.cpu()))
    if rank == 0:
        from haste_b200 import _lib
        _lib.check(_lib.lib.haste_ffi_set_max_ctas(0), "set_max_ctas")
        one = FusedFFIShard(inp["loc"].to(dev), inp["W"].clone().to(dev), inp["bias"].clone().to(dev), G, D, **kw)
        ref_dx = []
        for i in range(n_steps):
            dxt, _ = one.step(*batches[i % 2])
            ref_dx.append(dxt.clone())
        torch.cuda.synchronize(dev)
        ws.sort(key=lambda t: t[0])
        w_all = torch.cat([t[1] for t in ws])
        b_all = torch.cat([t[2] for t in ws])
        ok_w = torch.equal(w_all.view(torch.int16), one.w.cpu().view(torch.int16))
        ok_b = torch.equal(b_all.view(torch.int16), one.bias.cpu().view(torch.int16))
        errs = [float((a - b).abs().max() / (b.abs().max() + 1e-30)) for a, b in zip(outs, ref_dx)]
        np.save(os.path.join(out_dir, "result.npy"), np.array([float(ok_w), float(ok_b)] + errs))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_match_one(tmp_path):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    res = np.load(os.path.join(str(tmp_path), "result.npy"))
    assert res[0] == 1.0, "weights differ between the 2-rank and the 1-rank run"
    assert res[1] == 1.0, "bias differs between the 2-rank and the 1-rank run"
    assert (res[2:] <= 1e-4).all(), f"summed dX differs: relative errors {res[2:]}"
