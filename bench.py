#!/usr/bin/env python
"""Benchmark of the FFI train step (forward + loss gradient + backward-features + backward-weights + SGD/SR).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3] [--impl ours|reference]

For N > 1 launch one rank per GPU:
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

A "step" is one pass of the fused train step over one synthetic batch.  Rank 0 prints ONE JSON line.
  value     whole-job samples/s with the batch already resident in HBM, device-timed: one CUDA-event pair per step on
            the launching stream, L2 flushed between steps outside the pairs; the per-step times are reduced with
            MAX over the ranks, ms_per_step is their median (the mean is reported beside it)
  e2e       same metric through the public API from pinned HOST buffers: host->device copy of the batch and
            device->host read of the loss inside the timed region
  roofline  the fused train-step kernel alone: 6*B*L*F flops / its CUDA-event duration, against the measured
            dense bf16 peak
  cpu_baseline  the CPU restatement (oracle/cpu_step.py) timed on this box's host cores on a bounded sample
Labels are sharded contiguously by group over the ranks (strong scaling: the layer is fixed, each rank owns
1/N of it), features are replicated, and the per-rank feature gradients are summed by one NCCL all-reduce.  At N > 1
the step is pipelined over three streams (ShardedFFILayer.step_pipelined): the all-reduce of step i-1 and the
preparation of batch i+1 run beside the fused kernel of step i, which leaves a few SMs free for them; everything a
step enqueues finishes inside that step's event pair, and the last all-reduce inside the last one.

--impl reference: the reference's own CUDA kernels (compiled from its sources into oracle/_ref, legacy wmma code on
this GPU) driven as its autograd function and training loop drive them, PyTorch ops for what the reference does in
PyTorch; falls back to the CPU restatement when that build or a GPU is absent.
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


def ncu_traffic_bytes(workload):
    """dram read+write bytes of one fused-step launch, from the ncu capture recorded in profiles/ncu_traffic.json
    (None when no capture of this workload is on record)."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    try:
        rec = json.load(open(path)).get(workload)
        return None if rec is None else float(rec["dram_bytes_read"]) + float(rec["dram_bytes_write"])
    except Exception:
        return None


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(bf16_tflops=p["bf16_tflops"], hbm_gbs=p["hbm_gbs"], source="measured")
    return dict(bf16_tflops=1590.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons while the timed region runs: NVML from a thread of this process (a first
    sample at once, then one every 10 ms, so that a region of a few milliseconds is still covered); nvidia-smi as a
    child process when the NVML module is missing.  Read-only queries."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None
        self.rows, self.thread, self.stop, self.max_mhz, self.nv, self.handle = [], None, False, None, None, None
        try:                                   # library start-up costs milliseconds: here, not inside a timed region
            import pynvml as nv
            nv.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(self.index).uuid)
                h = nv.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
            except Exception:
                h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            nv.nvmlDeviceGetCurrentClocksEventReasons(h)
            self.nv, self.handle = nv, h
        except Exception:
            self.nv = None

    def _nvml_loop(self, nv, h):
        while True:
            try:
                self.rows.append((nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM), nv.nvmlDeviceGetCurrentClocksEventReasons(h)))
            except Exception:
                pass
            if self.stop:
                return
            time.sleep(0.01)

    def __enter__(self):
        if self.nv is not None:
            import threading
            self.thread = threading.Thread(target=self._nvml_loop, args=(self.nv, self.handle), daemon=True)
            self.thread.start()
            return self
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.thread is not None:
            self.stop = True
            self.thread.join(timeout=2)
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
            if self.thread is not None:
                nv = self.nv
                bits = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                        "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
                out["sm_mhz"] = float(statistics.median(r[0] for r in self.rows))
                out["sm_max_mhz"] = self.max_mhz
                out["reasons"] = [n for n, b in bits.items() if any(r[1] & b for r in self.rows)]
                out["samples"] = len(self.rows)
                out["source"] = "nvml"
                return out
            rows = [l.strip().split(",") for l in open(self.path) if l.strip()]
            sm = [float(r[0]) for r in rows]
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = float(rows[0][1])
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            out["reasons"] = [n for i, n in enumerate(names) if any("Active" in r[2 + i] and "Not" not in r[2 + i] for r in rows)]
            out["samples"] = len(rows)
            out["source"] = "nvidia-smi"
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


def _time_steps(layer, dev_batches, steps, warmup, world, device, flush, dist, clocks_index=None):
    """Device-timed steps of the given layer: returns (per-step ms as MAX over ranks, wall seconds, clock summary)."""
    stream = torch.cuda.current_stream(device)
    pipelined = world > 1

    def one(i, last=False):
        x, t = dev_batches[i % N_BATCHES]
        if pipelined:
            layer.step_pipelined(x, t, next_batch=None if last else dev_batches[(i + 1) % N_BATCHES], want_loss=True)
            if last:
                layer.flush()            # the last all-reduce belongs to the last timed step
        else:
            layer.step(x, t, want_loss=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    sampler = ClockSampler(clocks_index) if clocks_index is not None else None
    if world > 1:
        # the first collectives of a communicator set up channels and buffers: keep that out of every timed step (the
        # layer reduces dX on a communicator of its own, its flush() on the default one)
        layer.setup_pipeline(dev_batches[0][0].shape[0])
        warm = torch.zeros_like(dev_batches[0][0], dtype=torch.float32)
        for _ in range(25):
            dist.all_reduce(warm, group=layer.comm_pg)
            dist.all_reduce(warm)
        barrier()
    for i in range(warmup):
        flush.zero_()
        one(i)
    if sampler:
        sampler.__enter__()          # the sampling thread starts while the warm-up drains, not inside the first timed step
    barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    t_wall0 = time.perf_counter()
    for i in range(steps):
        flush.zero_()
        ev[i][0].record(stream)
        one(warmup + i, last=(i == steps - 1))
        ev[i][1].record(stream)
    barrier()
    t_wall = time.perf_counter() - t_wall0
    if sampler:
        sampler.__exit__()
    ms = torch.tensor([a.elapsed_time(b) for a, b in ev], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.tolist(), t_wall, (sampler.summary() if sampler else None)


def _time_kernel(shard, x, t, device, flush, n, dist, world):
    """The fused kernel alone: events around the single launch, inputs prepared through the unfused entry points, L2
    flushed.  Returns (MAX over ranks of the mean ms, per-rank means)."""
    from haste_b200 import ffi as hffi
    stream = torch.cuda.current_stream(device)
    xt = hffi.transpose_bf16(x)
    shard.bucket_targets(t)
    dxt = torch.zeros(xt.shape, dtype=torch.float32, device=device)
    kern_ms = []
    for i in range(3 + n):
        flush.zero_()
        seed, stp = shard._keys()
        flags = hffi.make_flags(sr=True, contract=True, rng=shard.rng, zero_dxt=False, loss=True)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dxt.zero_()
        a.record(stream)
        hffi.train_step(shard.loc, xt, shard.w, shard.bias, None, None, shard.tgt_ptr, shard.tgt_ent, dxt, shard.loss_buf,
                        shard.G, shard.label0, shard.loss_kind, shard.grad_scale, LR, WD, 0.0, seed, stp, flags)
        b.record(stream)
        torch.cuda.synchronize(device)
        if i >= 3:
            kern_ms.append(a.elapsed_time(b))
    kern = torch.tensor([statistics.mean(kern_ms)], dtype=torch.float64, device=device)
    ranks = [float(kern)]
    if world > 1:
        gathered = [torch.zeros_like(kern) for _ in range(world)]
        dist.all_gather(gathered, kern)
        ranks = [float(g) for g in gathered]
        dist.all_reduce(kern, op=dist.ReduceOp.MAX)
    return float(kern), ranks


def _check_ranks_agree(layer, x, t, device, dist, world):
    """What the N ranks computed, checked outside every timed region: each rank's partial dX (its label shard) is
    summarised by two checksums (plain sum, and sum weighted by a fixed pattern), the checksums are all-gathered,
    and their sum must equal the checksums of the all-reduced dX on every rank.  Returns "ok" or raises."""
    dxt, _ = layer.shard.step(x, t, want_loss=False)
    torch.cuda.synchronize(device)
    pat = torch.linspace(0.5, 1.5, dxt.numel(), dtype=torch.float64, device=device).view_as(dxt)
    part = torch.stack([dxt.double().sum(), (dxt.double() * pat).sum(), dxt.double().abs().sum()])
    red = dxt.clone()
    dist.all_reduce(red, op=dist.ReduceOp.SUM)
    full = torch.stack([red.double().sum(), (red.double() * pat).sum()])
    parts = [torch.zeros_like(part) for _ in range(world)]
    dist.all_gather(parts, part)
    want = sum(p[:2] for p in parts)
    scale = sum(float(p[2]) for p in parts) + 1e-30
    err = float((full - want).abs().max()) / scale
    if not err <= 1e-5:
        raise RuntimeError(f"rank results disagree: reduced dX checksum differs from the sum of the partial checksums by {err:.3e} (relative)")
    # every rank holds the same reduced tensor
    same = torch.stack([red.double().sum(), (red.double() * pat).sum()])
    lo, hi = same.clone(), same.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    if not torch.equal(lo, hi):
        raise RuntimeError("the all-reduced dX differs between ranks")
    return "ok"


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
    step_ms, t_wall, clocks = _time_steps(layer, dev_batches, args.steps, args.warmup, world, device, flush, dist,
                                          clocks_index=local if rank == 0 else None)    # rank 0's GPU is sampled
    ms_per_step = statistics.median(step_ms)
    ms_mean = statistics.mean(step_ms)

    # ---------------- the fused kernel alone (roofline)
    kern_ms_avg, kern_ranks = _time_kernel(shard, dev_batches[0][0], dev_batches[0][1], device, flush, min(args.steps, 20), dist, world)

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
        if world > 1:
            # the previous step's all-reduce runs beside this step's kernel; this batch is prepared on this stream
            _, loss = layer.step_pipelined(xbuf[s_], tbuf[s_][:nnz], next_batch=None, want_loss=True)
        else:
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
    e2e_times = []
    for i in range(args.warmup, args.warmup + args.steps):
        flush.zero_()
        barrier()                                         # ranks start each step together; outside the timed region
        t0 = time.perf_counter()
        e2e_step(i)
        e2e_times.append(time.perf_counter() - t0)
    if world > 1:
        layer.flush()
    e2e_t = torch.tensor(e2e_times, dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_ms = statistics.median(e2e_t.tolist()) * 1e3
    h2d = B * D * 2 + int(statistics.mean(t.shape[0] for _, t in batches)) * 8

    # ---------------- N > 1: what the ranks computed, and the 2.8M-label workload in the same process
    parity_n, c5 = None, None
    if world > 1:
        parity_n = _check_ranks_agree(layer, dev_batches[0][0], dev_batches[0][1], device, dist, world)
        if args.workload == "c3" and not args.no_c5:
            c5 = _c5_lines(args, rank, world, device, flush, dist)

    if rank == 0:
        peaks = measured_peaks()
        flops = 6.0 * B * c["L"] * c["F"]                       # whole layer, all ranks
        flops_rank = flops * (shard.L / c["L"])
        achieved = flops_rank / (kern_ms_avg * 1e-3) / 1e12
        launches_per_step = 2 if world == 1 else 2            # preparation launch + fused kernel (the collective is NCCL's)
        line = {
            "metric": METRIC, "value": B / (ms_per_step * 1e-3), "unit": "samples/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "ms_per_step_mean": ms_mean, "ms_per_step_max": max(step_ms), "slowest_step": step_ms.index(max(step_ms)),
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": _workload_string(args.workload, c) + " rng=packed",
                       "parallelism": (f"labels sharded over {world} rank(s), features replicated, dX all-reduce"
                                       + ("" if world == 1 else f"; pipelined: all-reduce of step i-1 and preparation of batch i+1 run beside the kernel of "
                                          f"step i ({layer.reserve_sms} SMs left free), all of it inside step i's timed region, the last all-reduce inside the last step")),
                       "l2": "flushed between steps (256 MiB write) outside the timed regions; value: median of per-step CUDA-event times (MAX over ranks), e2e: median per-step wall clock",
                       "layer_tflops": flops / (ms_per_step * 1e-3) / 1e12},
            "e2e": {"value": B / (e2e_ms * 1e-3), "unit": "samples/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_ms},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16_tflops"], "traffic": ncu_traffic_bytes(args.workload) if world == 1 else None,
                         "kernel": "fused train step", "kernel_ms": kern_ms_avg, "kernel_ms_ranks": [round(k, 4) for k in kern_ranks], "peak_source": peaks["source"] + " burst bf16"},
            "wall_s_timed_region": t_wall,
        }
        if parity_n is not None:
            line["parity_n"] = parity_n
        if c5 is not None:
            line["c5"] = c5
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args.workload, full, batches, budget_s=20.0)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _c5_lines(args, rank, world, device, flush, dist):
    """The 2.8M-label workload (B=1024, BCE) on the same ranks, and on rank 0 alone for the ratio: the scale-out
    target is stated on this workload.  Fewer steps than the main line (a step is ten times longer)."""
    steps, warmup = max(5, min(args.steps, 30)), 3
    c, layer, batches, _ = build_problem("c5", rank, world, device)
    dev_batches = [(x.to(device), t.to(device)) for x, t in batches]
    ms, _, _ = _time_steps(layer, dev_batches, steps, warmup, world, device, flush, dist)
    kern, kern_ranks = _time_kernel(layer.shard, dev_batches[0][0], dev_batches[0][1], device, flush, 5, dist, world)
    parity = _check_ranks_agree(layer, dev_batches[0][0], dev_batches[0][1], device, dist, world)
    layer.close()
    del layer
    torch.cuda.empty_cache()
    out = {"value": c["B"] / (statistics.median(ms) * 1e-3), "unit": "samples/s", "ms_per_step": statistics.median(ms), "steps": steps,
           "kernel_ms_ranks": [round(k, 4) for k in kern_ranks], "parity_n": parity,
           "workload": f"c5: B={c['B']} D={c['D']} L={c['L']} fan_in={c['F']} G={c['G']} loss={c['loss']}"}
    # one GPU, same process: rank 0 holds the whole layer and uses every SM, the other ranks wait
    n1 = torch.zeros(2, dtype=torch.float64, device=device)
    if rank == 0:
        from haste_b200 import _lib
        _lib.check(_lib.lib.haste_ffi_set_max_ctas(0), "set_max_ctas")
        _, layer1, _, _ = build_problem("c5", 0, 1, device)
        ms1, _, _ = _time_steps(layer1, dev_batches, max(5, steps // 3), 3, 1, device, flush, dist)
        n1[0] = statistics.median(ms1)
        n1[1], _ = _time_kernel(layer1.shard, dev_batches[0][0], dev_batches[0][1], device, flush, 5, None, 1)
        del layer1
        torch.cuda.empty_cache()
    dist.all_reduce(n1, op=dist.ReduceOp.MAX)
    out["n1_ms_per_step"] = float(n1[0])
    out["vs_n1"] = float(n1[0]) / out["ms_per_step"]
    # the whole layer's fused kernel on one GPU against the measured bf16 burst peak (same definition as `roofline`)
    out["n1_kernel_ms"] = float(n1[1])
    out["n1_roofline_frac"] = 6.0 * c["B"] * c["L"] * c["F"] / (float(n1[1]) * 1e-3) / 1e12 / measured_peaks()["bf16_tflops"]
    return out


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
            "ms_per_step_scaled": t_step * 1e3, "timed_steps": len(times)}


def _workload_string(wl, c):
    return (f"{wl}: B={c['B']} D={c['D']} L={c['L']} fan_in={c['F']} G={c['G']} loss={c['loss']} "
            f"SR-SGD lr={LR} wd={WD} momentum=0")


def reference_gpu_step_fn(ref, c, loc, W, bias, device):
    """The reference's training step for this layer, driven the way its own code drives it: its CUDA kernels through
    an autograd function that restates shared_ffi/bindings.py:12-54 (transpose, forward kernel; backward: bias
    gradient by a column sum, backward-features kernel + transpose, backward-weights kernel), the loss written with
    PyTorch ops as src/runner.py:469-483 does, and PyTorch ops where the reference calls its Triton kernels, which
    cannot run unmodified on this Triton version (shared_ffi/sr_triton.py:13): the stochastic rounding of dX becomes
    a cast, the fused SGD + stochastic-rounding update one in-place elementwise pass with the same memory traffic
    (weights read and written, gradient read).  Shapes outside the reference's launch limits (group size 128, and
    (64,128) whose launch exceeds 48 KB of shared memory) run at group size 32 on an index table with repeated rows."""
    G, F, L, B, D = c["G"], c["F"], c["L"], c["B"], c["D"]
    gs = G if (G in (16, 32, 64) and not (G == 64 and F == 128)) else 32
    loc_r = (loc if gs == G else loc.repeat_interleave(G // gs, 0)).contiguous().to(device)
    Wp = torch.nn.Parameter(W.to(device))
    bp = torch.nn.Parameter(bias.to(device))

    class RefFFI(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x, w, b):
            xt = x.t().contiguous()
            ctx.save_for_backward(xt, w)
            return ref.ffi_forward_cuda(loc_r, xt, w, b, B, D, F, L, gs)

        @staticmethod
        def backward(ctx, gz):
            xt, w = ctx.saved_tensors
            gz = gz.contiguous()
            gb = gz.sum(0)
            gx = ref.ffi_backward_features_cuda(xt, w, loc_r, gz, B, D, F, L, gs).t().contiguous().to(torch.bfloat16)
            gw = ref.ffi_backward_weights_cuda(xt, w, loc_r, gz, B, D, F, L, gs)
            return gx, gw, gb

    def loss_fn(z, tg):
        rows, cols = tg[:, 0].long(), tg[:, 1].long()
        if c["loss"] == "bce":
            loss = z.clamp(min=0.0).sum(dtype=torch.float32)
            loss = loss - z[rows, cols].sum(dtype=torch.float32)
            return loss + (1 + (-torch.abs(z)).exp()).log().sum(dtype=torch.float32)
        zf = z.float()                      # squared hinge, mean over [B,L]: negatives everywhere, positives corrected
        t = (1.0 + zf).clamp(min=0.0)
        zp = zf[rows, cols]
        tot = (t * t).sum() + ((1.0 - zp).clamp(min=0.0) ** 2 - (1.0 + zp).clamp(min=0.0) ** 2).sum()
        return tot / (B * L)

    def step(x, tg):
        x = x.detach().requires_grad_(True)
        z = RefFFI.apply(x, Wp, bp)
        loss = loss_fn(z, tg)
        loss.backward()
        with torch.no_grad():
            Wp.add_(Wp.grad, alpha=-LR)
            bp.add_(bp.grad, alpha=-LR)
        Wp.grad = None
        bp.grad = None
        return x.grad, loss

    return step


def run_reference(args):
    """Reference arm (rank 0 only): the reference's CUDA kernels from oracle/_ref on this GPU when that build and a GPU
    are present, else the CPU restatement (oracle/cpu_step.py) with every host thread on a bounded sample."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    from haste_b200 import synth
    from oracle import build_ref
    c = synth.WORKLOADS[args.workload]
    loc, W, bias = synth.make_layer(c["D"], c["L"], c["F"], c["G"], seed=42)
    grad_scale = 1.0 / (c["B"] * c["L"]) if c["loss"] == "squared_hinge" else 1.0
    batches = [synth.make_batch(c["B"], c["D"], c["L"], c["avg_pos"], c["zipf"], c["x"], seed=1000 + i) for i in range(N_BATCHES)]
    config = {"workload": _workload_string(args.workload, c) + " rng=packed",
              "parallelism": "one GPU (rank 0 alone runs the reference arm)",
              "l2": "flushed between steps (256 MiB write) outside the timed regions"}
    ref = build_ref.load() if torch.cuda.is_available() else None
    if ref is not None and c["B"] * c["L"] >= 2 ** 31:
        ref = None                                   # the reference indexes [B,L] with 32-bit ints
    if ref is None:
        steps = max(1, min(args.steps, 5))
        cb = cpu_baseline(args.workload, (loc, W, bias, grad_scale), batches, budget_s=60.0, steps=steps)
        config["note"] = "CPU restatement on a bounded sample; ms_per_step is extrapolated to the whole layer (see cpu_baseline.sample)"
        line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "samples/s", "n_gpus": args.gpus,
                "steps": cb["timed_steps"], "warmup": 1, "ms_per_step": cb["ms_per_step_scaled"], "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config, "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    step = reference_gpu_step_fn(ref, c, loc, W, bias, device)
    host = [(x.pin_memory(), t.pin_memory()) for x, t in batches]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    B, D = c["B"], c["D"]
    h2d = B * D * 2 + int(statistics.mean(t.shape[0] for _, t in batches)) * 8

    def one(i):
        xh, th = host[i % N_BATCHES]
        x, t = xh.to(device, non_blocking=True), th.to(device, non_blocking=True)
        _, loss = step(x, t)
        return float(loss)                           # the reference's loop reads the loss back every step

    with ClockSampler(0) as clocks:
        for i in range(args.warmup):
            one(i)
        torch.cuda.synchronize(device)
        times = []
        for i in range(args.steps):
            flush.zero_()
            torch.cuda.synchronize(device)
            t0 = time.perf_counter()
            one(args.warmup + i)
            torch.cuda.synchronize(device)
            times.append(time.perf_counter() - t0)
    ms = statistics.median(times) * 1e3
    value = B / (ms * 1e-3)
    config["note"] = ("the reference's three CUDA kernels (legacy wmma code on this GPU) + PyTorch ops for loss, bias gradient and the "
                      "optimizer pass; host->device copy of the batch and read-back of the loss inside the timed region")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": config, "clocks": clocks.summary(),
            "cpu_baseline": {"value": value, "unit": "samples/s", "cores": 1, "kind": "reference",
                             "sample": f"whole workload, {args.steps} timed steps on GPU 0 (the reference has no CPU implementation; one host thread drives its CUDA kernels)"},
            "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4}}
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
        ("ffi_backward (both gradients, one pass over a contiguous [B,L] dY)", lambda: hffi.backward_both(xt, W, loc, dy, G), 2 * B * L + 2 * L * F + 2 * L * F + 4 * NG * F),
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
    rows += probe_rows(c, xt, dev, peaks, timeit)
    for name, fn, nbytes in rows:
        if nbytes is None:                                   # a probe that prints its own line
            fn()
            continue
        ms = timeit(fn)
        gbs = nbytes / (ms * 1e-3) / 1e9
        print(json.dumps({"kernel": name, "workload": args.workload, "ms": ms, "algorithmic_bytes": nbytes, "GB/s": gbs,
                          "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "bound": "hbm"}), flush=True)


def probe_rows(c, xt, dev, peaks, timeit):
    """Rate probes of the fused step's three resources at the workload's sizes (haste_probe_* entry points): the dX
    scatter as reduce-adds into dxt, the X gather (TMA gather4 against cp.async), and the tcgen05.mma issue rate."""
    from haste_b200 import _lib
    lib, check = _lib.lib, _lib.check
    B, D = c["B"], c["D"]
    if B % 128 != 0 or D < 128:
        return []
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    st = lambda: torch.cuda.current_stream(dev).cuda_stream
    dxt = torch.zeros(D, B, dtype=torch.float32, device=dev)
    tiles = 140                                              # 148 SMs x 140 tiles x 32 KB = 679 MB: one C3 step's scatter
    rows = []

    def emit(name, ms, unit_bytes, extra):
        gbs = unit_bytes / (ms * 1e-3) / 1e9
        print(json.dumps(dict(kernel=name, workload="probe", ms=ms, algorithmic_bytes=unit_bytes, **{"GB/s": gbs}, **extra)), flush=True)

    for mode, what in ((0, "scalar red, 128 B per warp instruction (the step's pattern)"), (1, "red.v4 along one row, 512 B per warp instruction"),
                       (2, "red.v4 across 32 rows, 16 B each (a transposed accumulator's pattern)")):
        def run(mode=mode, what=what):
            ms = timeit(lambda: check(lib.haste_probe_red_rate(dxt.data_ptr(), D, B, mode, tiles, st()), "probe"))
            emit(f"probe: dX scatter alone, {what}", ms, sms * tiles * 32768, {"bound": "l2 reduce-add"})
        rows.append((what, run, None))
    for mode, what in ((0, "TMA tile::gather4, 1 issuing warp"), (12, "TMA tile::gather4, 2 issuing warps"), (14, "TMA tile::gather4, 4 issuing warps"),
                       (1, "cp.async, 1 warp"), (2, "cp.async, 2 warps"), (4, "cp.async, 4 warps")):
        def run(mode=mode, what=what):
            ms = timeit(lambda: check(lib.haste_probe_gather_rate(xt.data_ptr(), D, B, mode, tiles, st()), "probe"))
            cyc = ms * 1e-3 * 1.965e9 / tiles
            emit(f"probe: X gather alone (64 rows x 256 B per tile), {what}", ms, sms * tiles * 16384,
                 {"bound": "l2 -> smem", "cycles_per_tile_at_1965MHz": cyc})
        rows.append((what, run, None))
    cyc = torch.zeros(2, dtype=torch.int64, device=dev)
    for N, amn, bmn, what in ((128, 1, 0, "forward: A MN-major, B K-major, N=128"), (64, 0, 1, "backward-features: A K-major, B MN-major, N=64"),
                              (80, 1, 0, "backward-weights: A MN-major, B K-major, N=80"), (144, 1, 0, "backward-weights at F=128: N=144")):
        def run(N=N, amn=amn, bmn=bmn, what=what):
            check(lib.haste_probe_umma_rate(N, amn, bmn, 64, cyc.data_ptr(), st()), "probe")
            torch.cuda.synchronize()
            n = 64 * 8
            print(json.dumps(dict(kernel=f"probe: tcgen05.mma M=128 K=16, {what}", workload="probe", issue_cycles_per_mma=float(cyc[0]) / n,
                                  complete_cycles_per_mma=float(cyc[1]) / n, ideal_cycles_per_mma=128.0 * N * 16 / 4096.0)), flush=True)
        rows.append((what, run, None))
    return rows


def run_comm_probe(args):
    """N > 1 (under torchrun): what the pipelined step's time is made of on the chosen workload.  Per-measurement CUDA
    events after a barrier + synchronise, MAX over ranks of the median of 30: the fused kernel alone at several CTA
    counts, the all-reduce of dX alone with the default communicator and with CTA-capped ones, the two side by side,
    and the per-step time of the real pipelined loop against the number of reserved SMs.  One JSON line per figure."""
    import torch.distributed as dist
    from haste_b200 import _lib, ffi as hffi, synth
    from haste_b200.fused import ShardedFFILayer
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    if world < 2:
        raise SystemExit("--comm-probe needs N > 1 ranks (launch under torch.distributed.run)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    c = synth.WORKLOADS[args.workload]
    B, D, L, F, G = c["B"], c["D"], c["L"], c["F"], c["G"]
    loc, W, bias = synth.make_layer(D, L, F, G, seed=42)
    grad_scale = 1.0 / (B * L) if c["loss"] == "squared_hinge" else 1.0
    batches = [synth.make_batch(B, D, L, c["avg_pos"], c["zipf"], c["x"], seed=1000 + i) for i in range(N_BATCHES)]
    dev_batches = [(x.to(device), t.to(device)) for x, t in batches]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    cur, side = torch.cuda.current_stream(device), torch.cuda.Stream(device=device)
    kw = dict(rank=rank, world_size=world, loss=c["loss"], lr=LR, weight_decay=WD, seed=SEED, rng="packed", grad_scale=grad_scale)

    def emit(what, us):
        if rank == 0:
            print(json.dumps({"probe": what, "workload": args.workload, "n_gpus": world, "us": round(us, 1)}), flush=True)

    def capped(n, cga=1):
        o = dist.ProcessGroupNCCL.Options()
        o.config.max_ctas, o.config.min_ctas, o.config.cga_cluster_size = n, 1, cga
        return dist.new_group(backend="nccl", pg_options=o)

    def timed(fn, n=30):
        ts = []
        for i in range(n + 5):
            flush.zero_()
            dist.barrier()
            torch.cuda.synchronize(device)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(cur); fn(); b.record(cur)
            torch.cuda.synchronize(device)
            if i >= 5:
                ts.append(a.elapsed_time(b))
        v = torch.tensor([statistics.median(ts)], device=device)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        return float(v) * 1e3

    layer = ShardedFFILayer(loc, W, bias, G, D, device, **kw)
    sh = layer.shard
    xt = hffi.transpose_bf16(dev_batches[0][0])
    sh.bucket_targets(dev_batches[0][1])
    dxt, buf = torch.zeros(D, B, device=device), torch.zeros(D, B, device=device)

    def kern():
        seed, stp = sh._keys()
        hffi.train_step(sh.loc, xt, sh.w, sh.bias, None, None, sh.tgt_ptr, sh.tgt_ent, dxt, sh.loss_buf, sh.G, sh.label0, sh.loss_kind,
                        sh.grad_scale, LR, WD, 0.0, seed, stp, hffi.make_flags(sr=True, contract=True, rng="packed", zero_dxt=False, loss=True))

    def both(pg):
        ev = torch.cuda.Event()
        ev.record(cur)
        kern()
        side.wait_event(ev)
        with torch.cuda.stream(side):
            dist.all_reduce(buf, group=pg)
            done = torch.cuda.Event()
            done.record(side)
        cur.wait_event(done)

    sms = torch.cuda.get_device_properties(device).multi_processor_count
    groups = {"default communicator": None, "at most 8 CTAs, launched singly": capped(8), "at most 16 CTAs, launched singly": capped(16),
              "at most 32 CTAs, launched singly": capped(32)}
    for free in (0, 8, 16):
        _lib.check(_lib.lib.haste_ffi_set_max_ctas(sms - free if free else 0), "set_max_ctas")
        emit(f"fused kernel alone, {free} SMs left free", timed(kern))
    for name, pg in groups.items():
        for _ in range(10):
            dist.all_reduce(buf, group=pg)
        emit(f"all-reduce of dX alone, {name}", timed(lambda: dist.all_reduce(buf, group=pg)))
    for free in (8, 16):
        _lib.check(_lib.lib.haste_ffi_set_max_ctas(sms - free), "set_max_ctas")
        for name, pg in groups.items():
            emit(f"kernel ({free} SMs left free) beside the all-reduce, {name}", timed(lambda: both(pg)))
    del layer
    for pg in groups.values():                        # communicators hold channels and buffers: one capped one at a time
        if pg is not None:
            dist.destroy_process_group(pg)
    for reserve, own in ((8, False), (8, True), (12, True), (16, True), (24, True)):
        layer = ShardedFFILayer(loc, W, bias, G, D, device, reserve_sms=reserve, **kw)
        if not own:
            layer._comm_ready = True                  # keep the caller's (default) communicator for the dX all-reduce
        ms, _, _ = _time_steps(layer, dev_batches, 60, 10, world, device, flush, dist)
        emit(f"pipelined step, {reserve} SMs reserved, " + ("capped communicator" if own else "default communicator"), statistics.median(ms) * 1e3)
        layer.close()
        del layer
        torch.cuda.empty_cache()
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c3")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-c5", action="store_true", help="N > 1: skip the extra 2.8M-label measurement")
    ap.add_argument("--aux", action="store_true", help="time the unfused and streaming kernels instead of the train step")
    ap.add_argument("--comm-probe", action="store_true", help="N > 1: kernel, all-reduce and their overlap against CTA caps and reserved SMs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.comm_probe:
        run_comm_probe(args)
    elif args.aux:
        run_aux(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
