"""CPU restatement of the reference's fixed-fan-in (FFI) output-layer math.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory: it is the checker the GPU kernels are compared against (tests,
the smoke check, and the CPU-baseline leg of the benchmark).  Every function
cites the reference file:line whose behaviour it restates.

Pinning status
--------------
* Philox / stochastic rounding / fused SGD update: PINNED.  The reference's
  Triton kernels (shared_ffi/sr_triton.py) were executed in the Triton CPU
  interpreter and their outputs are committed as golden vectors
  (tests/golden/sr_*.npz, generator tests/golden/make_golden.py).
* rewire (reference mode): PINNED against shared_ffi/rewire.py run on CPU with
  an injected index stream (tests/golden/rewire_ref_*.npz).
* forward / backward-features / backward-weights: the reference kernels are
  CUDA-only and cannot execute without a GPU; the restatement follows the
  kernels' arithmetic line by line but has no reference-produced vectors:
  "parity unpinned" for these three until the reference is run on a GPU.
* squared-hinge loss: the reference's implementation lives in a wheel that is
  not shipped with it; "parity unpinned".
"""
