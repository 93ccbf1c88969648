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
* forward / backward-features / backward-weights: PINNED.  The reference's own
  CUDA kernels (built from its sources by oracle/build_ref.py into oracle/_ref,
  where they run as legacy wmma code on a B200) produced
  tests/golden/ref_gemm_*.npz (generator tests/golden/make_golden_gpu.py); the
  restatement reproduces them: bf16 outputs bit-identical in >= 99.5 % of the
  entries and one bf16 step apart in the rest, the fp32 feature gradient to
  fp32 rounding (tests/test_oracle_golden.py).  On a GPU the same kernels are
  also run live beside the product's (tests/test_gpu_reference_parity.py).
* squared-hinge loss: the reference's implementation lives in a wheel that is
  not shipped with it; "parity unpinned".
"""
