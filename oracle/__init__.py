"""CPU oracle for the displaced-patch-parallel SDXL UNet hot path.

TEST INFRASTRUCTURE ONLY.  Everything in this package is a CPU restatement
(PyTorch fp32/fp64 on host tensors, numpy for the integer bookkeeping) of what
the reference implementation (sekstini/basedxl) computes on this path.  It is
the checker for the CUDA kernels: only the test-suite, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import it.
The shipped package never imports it and has no CPU fallback.

Parity pinning: the reference ships no golden vectors for this path (its only
test compares the matmul wrapper against ``torch.matmul`` with a loose
tolerance).  The functions here are therefore pinned against outputs of the
reference's own modules, executed unmodified on CPU / gloo ranks by
``tests/golden/make_golden.py``; the resulting fixtures live in
``tests/golden/*.npz`` and ``tests/test_oracle_golden.py`` checks every oracle
function against them.  The UNet *graph* (owned by the third-party package
``diffusers``, which is not available) has no pin: UNet-level parity is
"unpinned" with respect to diffusers and is anchored on the shared host graph
instead.

Nothing here needs compiling: the reference is pure Python, so the oracle is
too.
"""
