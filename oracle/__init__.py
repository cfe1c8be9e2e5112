"""CPU oracle for the decode-layer hot path (test infrastructure, not product code).

A parameterised PyTorch restatement of the reference's math for the four ops of one
decoder-layer decode step: the skinny BF16 projection, paged FP8 gated attention,
the NVFP4 routed experts, and the whole layer.  Each function cites the reference
file:line it follows.  The reference hard-codes its shapes as module constants; the
functions here take every shape from their arguments so the same code checks both the
reference's native shapes and the benchmark shapes (head_dim 128, hidden 4096, 128 experts).

Only the tests, the smoke check and the CPU-baseline leg of the benchmark import this
package.  The CUDA path never does: it fails loudly when the extension is missing.

Parity status: pinned.  tests/golden/ holds outputs of the reference's own
`ref_kernel` functions (imported and run on CPU by tests/golden/make_golden.py);
tests/test_oracle_golden.py demands that this package reproduces them.

Deliberate deviations from the reference, both confined to input generation / casting:
  * `quant_e4m3` clamps to +-448 before the cast (torch's cast gives NaN above ~464,
    every kernel in the reference saturates: cvt.rn.satfinite).
  * inputs are drawn with a CPU torch.Generator so CPU oracle and GPU kernel see the same bits.
"""
