#!/usr/bin/env python
"""Benchmark of the FFI train step (forward + loss gradient + backward-features + backward-weights + SGD/SR).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3] [--impl ours|reference]

For N > 1 launch one rank per GPU:
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

A "step" is one pass of the fused train step over one synthetic batch.  Rank 0 prints ONE JSON line.
  value     whole-job samples/s with the batch already resident in HBM, device-timed (CUDA events per step,
            L2 flushed between steps, max over ranks)
  e2e       same metric through the public API from pinned HOST buffers: host->device copy of the batch and
            device->host read of the loss inside the timed region
  roofline  the fused train-step kernel alone: 6*B*L*F flops / its CUDA-event duration, against the measured
            dense bf16 peak
  cpu_baseline  the CPU restatement (oracle/cpu_step.py) timed on this box's host cores on a bounded sample
Labels are sharded contiguously by group over the ranks (strong scaling: the layer is fixed, each rank owns
1/N of it), features are replicated, and the per-rank feature gradients are summed by one NCCL all-reduce.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch

METRIC = "FFI train-step samples/s @670K labels fan_in=64 B=512; % tensor/HBM roofline"
LR, WD, SEED = 0.05, 1e-4, 123
N_BATCHES = 4
# dram bytes (read+write) of one fused-step launch from an ncu capture; filled per workload when a capture exists
# (see profiles/); None = not captured yet.
NCU_TRAFFIC_BYTES = {"c3": 126.7e6}   # ncu capture of one launch at C3: dram read 90.9 MB + write 35.8 MB


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(bf16_tflops=p["bf16_tflops"], hbm_gbs=p["hbm_gbs"], source="measured")
    return dict(bf16_tflops=1590.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None

    def __enter__(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[])
        try:
            rows = [l.strip().split(",") for l in open(self.path) if l.strip()]
            sm = [float(r[0]) for r in rows]
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = float(rows[0][1])
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            out["reasons"] = [n for i, n in enumerate(names) if any("Active" in r[2 + i] and "Not" not in r[2 + i] for r in rows)]
            out["samples"] = len(rows)
        except Exception:
            pass
        return out


def build_problem(wl, rank, world, device):
    from haste_b200 import synth
    from haste_b200.fused import ShardedFFILayer, group_cost_from_targets
    c = synth.WORKLOADS[wl]
    loc, W, bias = synth.make_layer(c["D"], c["L"], c["F"], c["G"], seed=42)
    # the reference takes the squared hinge as a mean over [B,L] (src/runner.py:483); BCE as a sum (:469-478)
    grad_scale = 1.0 / (c["B"] * c["L"]) if c["loss"] == "squared_hinge" else 1.0
    batches = [synth.make_batch(c["B"], c["D"], c["L"], c["avg_pos"], c["zipf"], c["x"], seed=1000 + i) for i in range(N_BATCHES)]
    # label frequencies are long-tailed: ranks get contiguous group ranges of equal estimated cost, not equal count
    cost = group_cost_from_targets(batches[0][1], c["L"], c["G"], c["B"]) if world > 1 else None
    layer = ShardedFFILayer(loc, W, bias, c["G"], c["D"], device, rank=rank, world_size=world, group_cost=cost, loss=c["loss"], lr=LR,
                            weight_decay=WD, seed=SEED, rng="packed", grad_scale=grad_scale)
    return c, layer, batches, (loc, W, bias, grad_scale)


def run_ours(args):
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    from haste_b200 import ffi as hffi
    c, layer, batches, full = build_problem(args.workload, rank, world, device)
    shard = layer.shard
    B, D = c["B"], c["D"]
    dev_batches = [(x.to(device), t.to(device)) for x, t in batches]
    host_batches = [(x.pin_memory(), t.pin_memory()) for x, t in batches]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)          # > 126 MB of L2
    stream = torch.cuda.current_stream(device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    # ---------------- device-resident steps: per-step CUDA events, L2 flushed in between
    def device_step(i):
        x, t = dev_batches[i % N_BATCHES]
        return layer.step(x, t, want_loss=True)

    for i in range(args.warmup):
        flush.zero_()
        device_step(i)
    barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    with ClockSampler(local) as clocks:
        t_wall0 = time.perf_counter()
        for i in range(args.steps):
            flush.zero_()
            ev[i][0].record(stream)
            device_step(i)
            ev[i][1].record(stream)
        barrier()
        t_wall = time.perf_counter() - t_wall0
    step_ms = [a.elapsed_time(b) for a, b in ev]
    total_ms = torch.tensor([sum(step_ms)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(total_ms) / args.steps

    # ---------------- the fused kernel alone (roofline): events around the single launch, L2 flushed
    xt = hffi.transpose_bf16(dev_batches[0][0])
    shard.bucket_targets(dev_batches[0][1])
    kern_ms = []
    for i in range(3 + min(args.steps, 20)):
        flush.zero_()
        seed, stp = shard._keys()
        flags = hffi.make_flags(sr=True, contract=True, rng=shard.rng, zero_dxt=False, loss=True)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        shard._dxt.zero_()
        a.record(stream)
        hffi.train_step(shard.loc, xt, shard.w, shard.bias, None, None, shard.tgt_ptr, shard.tgt_ent, shard._dxt, shard.loss_buf,
                        shard.G, shard.label0, shard.loss_kind, shard.grad_scale, LR, WD, 0.0, seed, stp, flags)
        b.record(stream)
        torch.cuda.synchronize(device)
        if i >= 3:
            kern_ms.append(a.elapsed_time(b))
    kern = torch.tensor([statistics.mean(kern_ms)], dtype=torch.float64, device=device)
    kern_ranks = [float(kern)]
    if world > 1:
        gathered = [torch.zeros_like(kern) for _ in range(world)]
        dist.all_gather(gathered, kern)
        kern_ranks = [float(g) for g in gathered]
        dist.all_reduce(kern, op=dist.ReduceOp.MAX)
    kern_ms_avg = float(kern)

    # ---------------- end to end from pinned host buffers (H2D of the batch, D2H of the loss, every step)
    # Two device-side input slots: the copy of batch i+1 is enqueued on a copy stream while step i runs, as a
    # training loop's prefetcher would; every copy and every loss read-back still happens inside the timed region.
    max_nnz = max(t.shape[0] for _, t in batches)
    xbuf = [torch.empty(B, D, dtype=torch.bfloat16, device=device) for _ in range(2)]
    tbuf = [torch.empty(max_nnz, 2, dtype=torch.int32, device=device) for _ in range(2)]
    loss_host = torch.empty(1, dtype=torch.float32).pin_memory()
    copy_stream = torch.cuda.Stream(device=device)
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def enqueue_copy(i):
        s_ = i & 1
        xh, th = host_batches[i % N_BATCHES]
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[s_])          # the step that last read this slot has finished
            xbuf[s_].copy_(xh, non_blocking=True)
            tbuf[s_][: th.shape[0]].copy_(th, non_blocking=True)
            copied[s_].record(copy_stream)

    def e2e_step(i):
        s_ = i & 1
        nnz = host_batches[i % N_BATCHES][1].shape[0]
        stream.wait_event(copied[s_])
        _, loss = layer.step(xbuf[s_], tbuf[s_][:nnz], want_loss=True)
        consumed[s_].record(stream)
        loss_host.copy_(loss, non_blocking=True)
        enqueue_copy(i + 1)                               # overlaps this step's kernels
        stream.synchronize()
        copy_stream.synchronize()                         # the prefetch finishes inside this step's timed region
        return float(loss_host)

    for s_ in range(2):
        consumed[s_].record(stream)
    enqueue_copy(0)
    for i in range(args.warmup):
        e2e_step(i)
    barrier()
    e2e_s = 0.0
    for i in range(args.warmup, args.warmup + args.steps):
        flush.zero_()
        barrier()
        t0 = time.perf_counter()
        e2e_step(i)
        e2e_s += time.perf_counter() - t0
    e2e_t = torch.tensor([e2e_s], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e_t) * 1e3 / args.steps
    h2d = B * D * 2 + int(statistics.mean(t.shape[0] for _, t in batches)) * 8

    if rank == 0:
        peaks = measured_peaks()
        flops = 6.0 * B * c["L"] * c["F"]                       # whole layer, all ranks
        flops_rank = flops * (shard.L / c["L"])
        achieved = flops_rank / (kern_ms_avg * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": B / (ms_per_step * 1e-3), "unit": "samples/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.workload}: B={B} D={D} L={c['L']} fan_in={c['F']} G={c['G']} loss={c['loss']} "
                                   f"SR-SGD lr={LR} wd={WD} momentum=0 rng=packed",
                       "parallelism": f"labels sharded over {world} rank(s), features replicated, dX all-reduce",
                       "l2": "flushed between steps (256 MiB write) outside the timed regions; value: per-step CUDA events, e2e: per-step wall clock",
                       "layer_tflops": flops / (ms_per_step * 1e-3) / 1e12},
            "e2e": {"value": B / (e2e_ms * 1e-3), "unit": "samples/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_ms},
            "gpu_launches": 2 * args.steps,
            "clocks": clocks.summary(),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16_tflops"], "traffic": NCU_TRAFFIC_BYTES.get(args.workload) if world == 1 else None,
                         "kernel": "fused train step", "kernel_ms": kern_ms_avg, "kernel_ms_ranks": [round(k, 4) for k in kern_ranks], "peak_source": peaks["source"] + " burst bf16"},
            "wall_s_timed_region": t_wall,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args.workload, full, batches, budget_s=20.0)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def cpu_baseline(wl, full, batches, budget_s=20.0, steps=3):
    """Times oracle/cpu_step.py (kind "port": the reference has no CPU implementation) on a bounded sample:
    a leading fraction of the label groups, full batch, all host threads; scaled to the whole layer."""
    from haste_b200 import synth
    from oracle import cpu_step, ffi_oracle
    c = synth.WORKLOADS[wl]
    loc, W, bias, grad_scale = full
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    G, L = c["G"], c["L"]
    NG = (L + G - 1) // G
    frac_den = 16
    ng = max(1, NG // frac_den)
    kind = ffi_oracle.LOSS_SQHINGE if c["loss"] == "squared_hinge" else ffi_oracle.LOSS_BCE
    Ls = min(L, ng * G)
    Ws, bs, locs = W[:Ls].clone(), bias[:Ls].clone(), loc[:ng].clone()
    times = []
    t_start = time.perf_counter()
    for i in range(steps + 1):
        X, tg = batches[i % len(batches)]
        keep = tg[:, 1] < Ls
        t0 = time.perf_counter()
        cpu_step.cpu_train_step(locs, X, Ws, bs, tg[keep], G, kind, LR, WD, SEED, i, grad_scale=grad_scale)
        dt = time.perf_counter() - t0
        if i > 0:
            times.append(dt)
        if time.perf_counter() - t_start > budget_s and times:
            break
    t_step = statistics.median(times) * (NG / ng)
    return {"value": c["B"] / t_step, "unit": "samples/s", "cores": cores, "kind": "port",
            "sample": f"first {ng} of {NG} label groups ({Ls} labels), full batch, {len(times)} timed steps, scaled x{NG / ng:.2f}",
            "ms_per_step_scaled": t_step * 1e3}


def run_reference(args):
    """Reference arm.  The reference ships no CPU implementation of this path and its CUDA extension is not part
    of this repository, so this arm times the CPU restatement (oracle/cpu_step.py) with every host thread on a
    bounded sample of the same workload."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    from haste_b200 import synth
    c = synth.WORKLOADS[args.workload]
    loc, W, bias = synth.make_layer(c["D"], c["L"], c["F"], c["G"], seed=42)
    grad_scale = 1.0 / (c["B"] * c["L"]) if c["loss"] == "squared_hinge" else 1.0
    batches = [synth.make_batch(c["B"], c["D"], c["L"], c["avg_pos"], c["zipf"], c["x"], seed=1000 + i) for i in range(2)]
    cb = cpu_baseline(args.workload, (loc, W, bias, grad_scale), batches, budget_s=60.0, steps=max(1, min(args.steps, 5)))
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "samples/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["ms_per_step_scaled"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: B={c['B']} D={c['D']} L={c['L']} fan_in={c['F']} G={c['G']} loss={c['loss']} "
                                   f"SR-SGD lr={LR} wd={WD} momentum=0 rng=packed"},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_aux(args):
    """Device times of the other kernels of the path on the chosen workload (one GPU), each against the roofline
    that bounds it: the unfused forward / backward kernels and the streaming kernels are HBM-bound, so the figure
    is algorithmic bytes / time against the measured copy bandwidth.  Prints one JSON line per kernel."""
    from haste_b200 import synth, ffi as hffi
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    c = synth.WORKLOADS[args.workload]
    B, D, L, F, G = c["B"], c["D"], c["L"], c["F"], c["G"]
    loc, W, bias = synth.make_layer(D, L, F, G, seed=42)
    X, _ = synth.make_batch(B, D, L, c["avg_pos"], c["zipf"], c["x"], seed=1000)
    loc, W, bias, X = loc.to(dev), W.to(dev), bias.to(dev), X.to(dev)
    xt = hffi.transpose_bf16(X)
    NG = (L + G - 1) // G
    peaks = measured_peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timeit(fn, n=10):
        ts = []
        for i in range(n + 3):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
            if i >= 3:
                ts.append(a.elapsed_time(b))
        return statistics.mean(ts)

    z = hffi.forward(loc, xt, W, bias, G)
    dy = torch.randn(B, L, device=dev).to(torch.bfloat16)
    g = torch.randn(L, F, device=dev).to(torch.bfloat16)
    mom = torch.zeros(L, F, device=dev)
    w2 = W.clone()
    rw_scratch = torch.empty(hffi.rewire_scratch_words(NG, F), dtype=torch.int32, device=dev)
    fill_buf = torch.empty(768 << 20, dtype=torch.uint8, device=dev)
    from haste_b200.infer import ffi_topk
    x_bd = xt.t().contiguous()
    rows = [
        # what a write-only stream reaches on this GPU (a library fill): the yardstick for the forward, which writes [B,L]
        ("device fill 768 MiB (write-only yardstick, torch fill kernel)", lambda: fill_buf.zero_(), 768 << 20),
        ("ffi_forward (unfused, writes Z)", lambda: hffi.forward(loc, xt, W, bias, G), 2 * B * L + 2 * L * F + 4 * NG * F),
        ("ffi_backward_features (unfused, reads dY)", lambda: hffi.backward_features(xt, W, loc, dy, G), 2 * B * L + 2 * L * F + 4 * NG * F),
        ("ffi_backward_weights (unfused, reads dY, writes dW)", lambda: hffi.backward_weights(xt, W, loc, dy, G), 2 * B * L + 2 * L * F + 4 * NG * F),
        ("ffi_backward (both gradients, one pass over dY incl. row padding)", lambda: hffi.backward_both(xt, W, loc, dy, G), 2 * B * L + 2 * L * F + 2 * L * F + 4 * NG * F),
        ("ffi_bww_sr_sgd (backward-weights + SGD/SR, no dW)", lambda: hffi.bww_sr_sgd(xt, loc, dy, w2, None, None, None, G, 0, LR, WD, 0.0, SEED, 1, hffi.make_flags(rng="packed")), 2 * B * L + 4 * L * F + 4 * NG * F),
        ("sgd_sr_update packed stream", lambda: hffi.sgd_sr_update(w2, g, None, 0, LR, WD, 0.0, SEED, 1, hffi.make_flags(rng="packed")), 6 * L * F),
        ("sgd_sr_update reference stream", lambda: hffi.sgd_sr_update(w2, g, None, 0, LR, WD, 0.0, SEED, 1, hffi.make_flags(rng="reference")), 6 * L * F),
        ("sgd_sr_update packed + momentum", lambda: hffi.sgd_sr_update(w2, g, mom, 0, LR, WD, 0.9, SEED, 1, hffi.make_flags(rng="packed")), 14 * L * F),
        # inference top-100 (what the reference's evaluation does with torch.topk over the full logits): chunked forward +
        # running top-k, [B,L] never written; bytes = the layer read once + the result
        ("ffi_topk k=100 (chunked forward + running top-k, no [B,L] in HBM)", lambda: ffi_topk(loc, W, bias, x_bd, 100, G), 2 * L * F + 4 * NG * F + 8 * B * 100),
        ("forward + torch.topk k=100 (library top-k over the full [B,L] logits)", lambda: torch.topk(hffi.forward(loc, xt, W, bias, G), 100, dim=1), 4 * B * L + 2 * L * F + 4 * NG * F),
        ("rewire fraction 0.15, unused regrow, zero init, regroup", lambda: hffi.rewire(w2, loc, None, D, G, 0, 1, 0.0, int(F * 0.15), 1, 0, True, SEED, 1, None), 4 * L * F + 8 * NG * F),
        # layer-wide fraction with max scores (the reference model's layer class): the weights are read twice
        # (scores pass + rewire pass) and written once, the scores are written and read twice by the select block
        ("rewire layer-wide fraction 0.15, max score, unused regrow, zero init, regroup",
         lambda: hffi.rewire_ex(w2, loc, None, D, G, 0, 1, 2, 0.0, int(NG * F * 0.15), 1, 0, True, SEED, 1, None, rw_scratch), 6 * L * F + 8 * NG * F + 12 * NG * F),
    ]
    for name, fn, nbytes in rows:
        ms = timeit(fn)
        gbs = nbytes / (ms * 1e-3) / 1e9
        print(json.dumps({"kernel": name, "workload": args.workload, "ms": ms, "algorithmic_bytes": nbytes, "GB/s": gbs,
                          "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "bound": "hbm"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c3")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--aux", action="store_true", help="time the unfused and streaming kernels instead of the train step")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.aux:
        run_aux(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
