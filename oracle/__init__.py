"""CPU oracle — TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this.  It is used by tests/, by
__graft_entry__.smoke() as the checker, and by bench.py's CPU-baseline and
reference arms.  Two parts:

* numpy_oracle: the expected-value expressions the reference's own execution
  tests compare against (one function per kernel family, each citing the test);
* ssa_interp: a NumPy interpreter of printed typed-SSA text that follows the
  reference code generator's per-opcode semantics, so any kernel can be checked
  program by program.

Parity status: pinned.  The printed SSA this oracle consumes is compared
verbatim with the reference's own output (tests/golden/corpus_golden.json), and
the interpreter is checked against the known-answer vectors of the reference's
tests (softmax large-value rows, extremum NaN/signed-zero table, loop closed
forms, exact integer matmuls).  tl.dot / bf16 are absent from the reference:
that part is pinned only by the fp64 product.
"""
