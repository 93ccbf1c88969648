"""Generate the golden vectors under tests/golden/ from the REFERENCE's own code.

Run once, in a container that has the reference checkout (path given as argv[1]) and Triton:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference

What runs:
* shared_ffi/sr_triton.py (stochastic_rounding, sgd_update) in Triton's CPU interpreter.  The
  installed Triton rejects the literal ``& -65536`` on an unsigned value (sr_triton.py:13), so a
  scratch copy in a temp dir gets that one token rewritten as ``& 0xFFFF0000`` (same bits); the
  reference tree itself is never modified and no reference source is stored in this repository.
* src/group_fanin_real.py's GroupFixedFanInReal.rewire (global-fraction pruning, mean / max scores) likewise
* shared_ffi/rewire.py's GroupFixedFanIn.rewire on CPU tensors, with ``shared_ffi._C`` stubbed
  (the CUDA extension is not needed for rewire) and ``torch.randint`` replaced by a recorded
  index stream so the draw is reproducible without torch's generator.

Outputs: small .npz files holding inputs and the reference's outputs.
"""
import os
import sys
import tempfile
import types
import importlib.util

os.environ.setdefault("TRITON_INTERPRET", "1")
import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def load_patched_sr(ref):
    src = open(os.path.join(ref, "shared_ffi", "sr_triton.py")).read()
    src = src.replace("out & -65536", "out & 0xFFFF0000").replace("out & -1048576", "out & 0xFFF00000")
    tmp = tempfile.mkdtemp(prefix="sr_ref_")
    path = os.path.join(tmp, "sr_triton_scratch.py")
    with open(path, "w") as f:
        f.write(src)
    spec = importlib.util.spec_from_file_location("sr_triton_scratch", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def gen_sr(ref):
    sr = load_patched_sr(ref)
    g = torch.Generator().manual_seed(7)
    n = 3000
    # --- plain stochastic rounding, including exact-bf16 values, negatives, tiny and large values
    x = torch.randn(n, generator=g) * torch.logspace(-6, 4, n)
    x[:8] = torch.tensor([0.0, -0.0, 1.0, -1.0, 0.5, 3.140625, 1e-30, -65280.0])
    for seed in (123, 124, 2**31 - 5):
        out = torch.empty(n, dtype=torch.bfloat16)
        sr.stochastic_rounding(x, out, seed)
        np.savez(os.path.join(HERE, f"sr_round_seed{seed}.npz"), x=x.numpy(), seed=seed, out=bf16_bits(out))
    # --- fused SGD update: wd only, momentum, RN cast
    F = 24
    w = ((torch.rand(125, F, generator=g) * 2 - 1) / 8).to(torch.bfloat16)
    grad = (torch.randn(125, F, generator=g) * 0.3).to(torch.bfloat16)
    m0 = torch.randn(125, F, generator=g) * 0.1
    cases = [("wd", 0.05, 1e-4, 0.0, False, True, 123), ("mom", 0.05, 1e-4, 0.9, True, True, 124),
             ("rn", 0.01, 0.0, 0.0, False, False, 125), ("mom_off", 0.1, 1e-3, 0.9, False, True, 126)]
    for name, lr, wd, mu, use_mom, do_sr, seed in cases:
        wc, mc = w.clone(), m0.clone()
        sr.sgd_update(wc, grad, mc, lr, wd, mu, use_mom, do_sr, seed)
        np.savez(os.path.join(HERE, f"sgd_{name}.npz"), w=bf16_bits(w), g=bf16_bits(grad), m=m0.numpy(),
                 lr=lr, wd=wd, mu=mu, use_mom=use_mom, do_sr=do_sr, seed=seed,
                 w_out=bf16_bits(wc), m_out=mc.numpy())


def gen_rewire(ref):
    # import the reference package's rewire.py without its CUDA extension
    pkg = types.ModuleType("shared_ffi")
    pkg.__path__ = [os.path.join(ref, "shared_ffi")]
    pkg._C = types.ModuleType("shared_ffi._C")
    sys.modules["shared_ffi"] = pkg
    sys.modules["shared_ffi._C"] = pkg._C
    fake_sr = types.ModuleType("shared_ffi.sr_triton")
    fake_sr.stochastic_rounding = None
    sys.modules["shared_ffi.sr_triton"] = fake_sr
    spec = importlib.util.spec_from_file_location("shared_ffi.rewire", os.path.join(ref, "shared_ffi", "rewire.py"))
    rw = importlib.util.module_from_spec(spec)
    sys.modules["shared_ffi.rewire"] = rw
    spec.loader.exec_module(rw)

    real_randint = torch.randint
    for name, (D, L, F, G, mode, frac, thr) in {
        "frac": (96, 150, 32, 32, "fraction", 0.25, None),
        "frac_g64": (300, 200, 48, 64, "fraction", 0.15, None),
        "thr": (96, 70, 16, 16, "threshold", None, 0.12),
    }.items():
        torch.manual_seed(11)
        layer = rw.GroupFixedFanIn(D, L, F, bias=True, dtype=torch.bfloat16, group_size=G, prune_mode=mode,
                                   rewire_fraction=frac, rewire_threshold=thr, init_mode="zero")
        w0 = layer.weights.detach().clone()
        loc0 = layer.group_locations.clone()
        rs = np.random.RandomState(5)
        stream = rs.randint(0, D, size=loc0.numel()).astype(np.int32)
        used = {}

        def fake_randint(*a, **k):
            size = k.get("size", a[-1] if a else None)
            n = int(size[0])
            used["n"] = n
            return torch.from_numpy(stream[:n].copy()).to(k.get("dtype", torch.int64))

        torch.randint = fake_randint
        try:
            layer.rewire()
        finally:
            torch.randint = real_randint
        np.savez(os.path.join(HERE, f"rewire_ref_{name}.npz"), D=D, L=L, F=F, G=G, mode=mode,
                 frac=-1.0 if frac is None else frac, thr=-1.0 if thr is None else thr,
                 w0=bf16_bits(w0), loc0=loc0.numpy(), injected=stream[:used.get("n", 0)],
                 w1=bf16_bits(layer.weights.detach()), loc1=layer.group_locations.numpy())


def gen_rewire_real(ref):
    """src/group_fanin_real.py's GroupFixedFanInReal.rewire on CPU tensors (global-fraction pruning, mean / max
    scores), with ``shared_ffi`` stubbed (rewire needs no kernel) and ``torch.randint`` replaced by a recorded
    stream.  Inputs are checked to be tie-free at the selection boundary, where torch.topk's order is unspecified."""
    pkg = types.ModuleType("shared_ffi")
    pkg.ops = types.ModuleType("shared_ffi.ops")
    sys.modules["shared_ffi"] = pkg
    sys.modules["shared_ffi.ops"] = pkg.ops
    spec = importlib.util.spec_from_file_location("ref_group_fanin_real", os.path.join(ref, "src", "group_fanin_real.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    real_randint = torch.randint
    for name, (D, L, F, G, mode, frac, thr, score) in {
        "gfrac_mean": (96, 150, 32, 32, "fraction", 0.2, None, "mean"),
        "gfrac_max": (300, 200, 48, 64, "fraction", 0.1, None, "max"),
        "thr_max": (96, 70, 16, 16, "threshold", None, 0.17, "max"),
    }.items():
        torch.manual_seed(13)
        layer = mod.GroupFixedFanInReal(D, L, F, bias=True, dtype=torch.bfloat16, group_size=G, prune_mode=mode,
                                        rewire_fraction=frac, rewire_threshold=thr, init_mode="zero", score_mode=score)
        w0 = layer.weights.detach().clone()
        loc0 = layer.group_locations.clone()
        rs = np.random.RandomState(6)
        stream = rs.randint(0, D, size=loc0.numel()).astype(np.int32)
        used = {}

        def fake_randint(*a, **k):
            size = k.get("size", a[-1] if a else None)
            n = int(size[0])
            used["n"] = n
            return torch.from_numpy(stream[:n].copy()).to(k.get("dtype", torch.int64))

        torch.randint = fake_randint
        try:
            layer.rewire()
        finally:
            torch.randint = real_randint
        np.savez(os.path.join(HERE, f"rewire_real_{name}.npz"), D=D, L=L, F=F, G=G, mode=mode, score=score,
                 frac=-1.0 if frac is None else frac, thr=-1.0 if thr is None else thr,
                 w0=bf16_bits(w0), loc0=loc0.numpy(), injected=stream[:used.get("n", 0)],
                 w1=bf16_bits(layer.weights.detach()), loc1=layer.group_locations.numpy())


if __name__ == "__main__":
    ref = sys.argv[1]
    gen_sr(ref)
    gen_rewire(ref)
    gen_rewire_real(ref)
    print("golden vectors written to", HERE)
