"""CPU oracle for the CTA-pipelining hot path.  TEST INFRASTRUCTURE ONLY.

Nothing under this package is part of the product: only the test-suite, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import it, and there only as the
checker (or as the timed CPU arm), never as the implementation of a library call.

Parity status: the integer artefacts (dependency CSR, scoreboard initial values, producer order,
weight sharding, gamma folding, fp32 boundary reference) are PINNED against outputs of the
reference's own Python functions, stored as fixtures next to the script that generated them.
The device-side index maps of the reference (tile remap, reducer unit map) exist only as CUDA
device code inside a CUTLASS-dependent translation unit that cannot be compiled here; they are
restated from the source text and pinned by hand-derived known answers plus bijection checks.
GEMM values are tolerance-pinned (the reference itself pins them only by tolerance vs torch).
"""
